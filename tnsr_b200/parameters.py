"""Named f32 parameters and tnsr's portable tensor archive.

Mirrors ``parameters::NamedParameters`` (src/parameters.rs:10-210,
docs/parameter-archive.md): a directory with ``manifest.json`` {version 1, dtype
"f32-le", data_file (a bare filename), config, tensors[{name, shape, offset,
count, group}]} and one raw little-endian f32 blob.  Tensor ranges are contiguous
from offset 0 and cover the blob exactly, names are unique, values are finite;
saving writes ``*.tmp`` files and renames them into place.  Entries are kept in
name order, as the reference's ``BTreeMap`` does, so a saved archive is
byte-compatible with what the Rust side writes.

``gpt_to_named`` / ``gpt_from_named`` map a ``Gpt`` to names of the form
``token_embedding``, ``blocks.3.attention.query_weight`` ... so weights can be
exchanged with a tnsr process without a Rust toolchain on this side.
"""
from __future__ import annotations

import json
import os
from collections import OrderedDict
from typing import Dict, Iterable, Tuple

import numpy as np

from .nn import Gpt, GptConfig, Parameter, TnsrError


class NamedParameters:
    def __init__(self):
        self._entries: Dict[str, Tuple[Parameter, str]] = {}

    def insert(self, name: str, values, shape, group: str) -> None:
        shape = [int(s) for s in shape]
        values = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        if not name or name in self._entries:
            raise TnsrError(f"empty or duplicate parameter name: {name}")
        if values.size != int(np.prod(shape, dtype=np.int64)):
            raise TnsrError(f"{name}: parameter length disagrees with shape")
        if not np.all(np.isfinite(values)):
            raise TnsrError(f"{name}: nonfinite parameter value")
        if not group:
            raise TnsrError(f"{name}: parameter group is empty")
        self._entries[name] = (Parameter(values, shape), group)

    def get(self, name: str, shape) -> Parameter:
        if name not in self._entries:
            raise TnsrError(f"missing parameter {name}")
        parameter = self._entries[name][0]
        if list(parameter.shape) != [int(s) for s in shape]:
            raise TnsrError(f"{name}: expected shape {list(shape)}, got {list(parameter.shape)}")
        return parameter

    def iter(self) -> Iterable[Tuple[str, Parameter, str]]:
        for name in sorted(self._entries):
            parameter, group = self._entries[name]
            yield name, parameter, group

    def validate_names(self, expected) -> None:
        actual, expected = set(self._entries), set(expected)
        if actual != expected:
            raise TnsrError(f"parameter keys mismatch; missing: {sorted(expected - actual)}; "
                            f"unexpected: {sorted(actual - expected)}")

    @classmethod
    def load(cls, directory: str):
        try:
            with open(os.path.join(directory, "manifest.json"), "rb") as f:
                manifest = json.loads(f.read())
        except OSError as e:
            raise TnsrError(f"read parameter manifest: {e}")
        except ValueError as e:
            raise TnsrError(f"parse parameter manifest: {e}")
        allowed = {"version", "dtype", "data_file", "config", "tensors"}
        if not isinstance(manifest, dict) or set(manifest) != allowed:
            raise TnsrError("parse parameter manifest: unknown or missing field")
        if manifest["version"] != 1 or manifest["dtype"] != "f32-le":
            raise TnsrError("unsupported parameter archive version/dtype")
        data_file = manifest["data_file"]
        if not isinstance(data_file, str) or data_file in ("", ".", "..") or os.path.basename(data_file) != data_file \
                or "/" in data_file or "\\" in data_file:
            raise TnsrError("archive data_file must be a filename")
        try:
            with open(os.path.join(directory, data_file), "rb") as f:
                blob = f.read()
        except OSError as e:
            raise TnsrError(f"read parameter data: {e}")
        if len(blob) % 4 != 0:
            raise TnsrError("truncated f32 parameter data")
        data = np.frombuffer(blob, dtype="<f4")
        parameters = cls()
        cursor = 0
        for tensor in manifest["tensors"]:
            if not isinstance(tensor, dict) or set(tensor) != {"name", "shape", "offset", "count", "group"}:
                raise TnsrError("parse parameter manifest: unknown or missing tensor field")
            name = tensor["name"]
            if tensor["offset"] != cursor:
                raise TnsrError(f"{name}: noncontiguous or overlapping parameter offset")
            count = 1
            for dim in tensor["shape"]:
                count *= int(dim)
                if count >= 1 << 64:
                    raise TnsrError("parameter shape overflows usize")
            if tensor["count"] != count:
                raise TnsrError(f"{name}: invalid parameter count")
            end = cursor + count
            if end > data.size:
                raise TnsrError(f"{name}: parameter data out of bounds")
            parameters.insert(name, data[cursor:end].astype(np.float32), tensor["shape"], tensor["group"])
            cursor = end
        if cursor != data.size:
            raise TnsrError("unreferenced trailing parameter data")
        return parameters, manifest["config"]

    def save(self, directory: str, config) -> None:
        os.makedirs(directory, exist_ok=True)
        tensors, offset = [], 0
        tmp = os.path.join(directory, "weights.f32.tmp")
        with open(tmp, "wb") as f:
            for name, parameter, group in self.iter():
                values = parameter.values()
                if not np.all(np.isfinite(values)):
                    raise TnsrError(f"{name}: refusing to save nonfinite parameters")
                f.write(values.astype("<f4").tobytes())
                tensors.append(OrderedDict(name=name, shape=list(parameter.shape), offset=offset, count=int(values.size),
                                           group=group))
                offset += int(values.size)
        os.replace(tmp, os.path.join(directory, "weights.f32"))
        manifest = OrderedDict(version=1, dtype="f32-le", data_file="weights.f32", config=config, tensors=tensors)
        tmp = os.path.join(directory, "manifest.json.tmp")
        with open(tmp, "w") as f:
            json.dump(manifest, f, indent=2)
        os.replace(tmp, os.path.join(directory, "manifest.json"))


_ATTENTION = ["query_weight", "query_bias", "key_weight", "key_bias", "value_weight", "value_bias", "output_weight",
              "output_bias"]
_BLOCK = ["attention_norm_weight", "attention_norm_bias", "feed_forward_norm_weight", "feed_forward_norm_bias"]
_FFN = {"swiglu": ["feed_forward_gate_weight", "feed_forward_gate_bias", "feed_forward_up_weight", "feed_forward_up_bias",
                   "feed_forward_down_weight", "feed_forward_down_bias"],
        "other": ["feed_forward_input_weight", "feed_forward_input_bias", "feed_forward_output_weight",
                  "feed_forward_output_bias"]}


def _named_fields(model: Gpt):
    yield "token_embedding", model.token_embedding
    yield "position_embedding", model.position_embedding
    yield "final_norm_weight", model.final_norm_weight
    yield "final_norm_bias", model.final_norm_bias
    for i, block in enumerate(model.blocks):
        for field in _ATTENTION:
            yield f"blocks.{i}.attention.{field}", getattr(block.attention, field)
        for field in _BLOCK + _FFN["swiglu" if block.activation == "swiglu" else "other"]:
            yield f"blocks.{i}.{field}", getattr(block, field)


def gpt_config_dict(config: GptConfig) -> dict:
    return dict(vocab_size=config.vocab_size, max_sequence_length=config.max_sequence_length, embed_dim=config.embed_dim,
                num_heads=config.num_heads, feed_forward_dim=config.feed_forward_dim, num_layers=config.num_layers,
                layer_norm_epsilon=config.layer_norm_epsilon, activation=config.activation, weight_dtype=config.weight_dtype)


def gpt_to_named(model: Gpt, group: str = "gpt") -> NamedParameters:
    named = NamedParameters()
    for name, parameter in _named_fields(model):
        named.insert(name, parameter.values(), parameter.shape, group)
    return named


def gpt_from_named(named: NamedParameters, config) -> Gpt:
    if isinstance(config, dict):
        config = GptConfig(**config)
    model = Gpt(config)
    fields = list(_named_fields(model))
    named.validate_names(name for name, _ in fields)
    for name, parameter in fields:
        parameter.set_values(named.get(name, parameter.shape).values())
    return model


def save_gpt(model: Gpt, directory: str) -> None:
    gpt_to_named(model).save(directory, gpt_config_dict(model.config()))


def load_gpt(directory: str) -> Gpt:
    named, config = NamedParameters.load(directory)
    return gpt_from_named(named, config)


# ---- serialised decoder state -------------------------------------------------------------------
# tnsr lists "serialized decoder state" as outside its decoder API (docs/kv-cache.md:94-95).  Here a session's
# state -- the live rows of its 2 * layers K/V tensors and its length -- travels in the same archive format as
# parameters: tensors `cache.<layer>.key` / `cache.<layer>.value` of shape [batch, length, embed_dim] (only the live
# prefix; rows past `length` are zero in a session by construction, src/nn/kv_cache.rs:238-257), group
# "decoder_state", and a config object that pins the shape the state belongs to.

def decoder_state_config(decoder) -> dict:
    c = decoder._model.config()
    return dict(kind="gpt_decoder_state", batch=decoder.batch_size(), capacity=decoder.capacity(), length=decoder.len(),
                num_layers=c.num_layers, embed_dim=c.embed_dim, num_heads=c.num_heads,
                attention_precision=decoder._options.attention_precision.value, weight_dtype=c.weight_dtype)


def save_decoder_state(decoder, directory: str) -> None:
    """Writes the K/V rows [0, len) of every layer and the length of `decoder` (a ``GptDecoder``) to `directory`."""
    if decoder._failed:
        raise TnsrError("decoder execution failed; reset the cache before reuse")
    config = decoder_state_config(decoder)
    named = NamedParameters()
    length = decoder.len()
    if length:
        for layer in range(config["num_layers"]):
            for which, name in enumerate(("key", "value")):
                rows = decoder._backend.read_cache(2 * layer + which)[:, :length, :]
                named.insert(f"cache.{layer:04d}.{name}", rows, rows.shape, "decoder_state")
    named.save(directory, config)


def load_decoder_state(decoder, directory: str) -> None:
    """Restores a state written by ``save_decoder_state`` into `decoder`, which must have the same batch, layer count,
    width and precision and enough capacity; its previous contents are discarded.  The weights are the caller's
    business, exactly as with a live session: a state only continues correctly under the weights that produced it."""
    named, config = NamedParameters.load(directory)
    if not isinstance(config, dict) or config.get("kind") != "gpt_decoder_state":
        raise TnsrError("archive does not hold a decoder state")
    mine = decoder_state_config(decoder)
    for key in ("batch", "num_layers", "embed_dim", "num_heads", "attention_precision", "weight_dtype"):
        if config.get(key) != mine[key]:
            raise TnsrError(f"decoder state mismatch: {key} is {config.get(key)!r}, this decoder has {mine[key]!r}")
    length = config.get("length")
    if not isinstance(length, int) or length < 0 or length > decoder.capacity():
        raise TnsrError("decoder context capacity exceeded")
    names = {f"cache.{layer:04d}.{name}" for layer in range(mine["num_layers"]) for name in ("key", "value")} if length else set()
    named.validate_names(names)
    decoder.reset()
    shape = [mine["batch"], length, mine["embed_dim"]]
    decoder._failed = True
    for layer in range(mine["num_layers"]) if length else ():
        for which, name in enumerate(("key", "value")):
            rows = named.get(f"cache.{layer:04d}.{name}", shape).values().reshape(shape)
            full = np.zeros((mine["batch"], decoder.capacity(), mine["embed_dim"]), dtype=np.float32)
            full[:, :length, :] = rows
            decoder._backend.write_cache(2 * layer + which, full)
    decoder._length = length
    decoder._revisions = [p.revision() for p in decoder._parameters]
    decoder._failed = False
