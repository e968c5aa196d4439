"""The token encoder of tnsr's forty_five example on the B200 operator set.

``Model::encode`` (examples/forty_five/mod.rs:329-407) is a bidirectional pre-norm transformer over short token rows:
token + token-type + position embeddings under an input mask, then per layer LayerNorm -> fused QKV projection ->
attention with an additive key mask (padding) -> output projection + residual -> LayerNorm -> SwiGLU feed-forward
(hidden = ceil(8 d / 3)) + residual, and a final LayerNorm.  Here every step is a call into ``libtnsr_b200.so``:
``tnsr_b200_encoder_embed``, ``tnsr_b200_layernorm`` (strict), ``tnsr_b200_gemm_f32_strict``,
``tnsr_b200_encoder_attention``, ``tnsr_b200_add_f32``, ``tnsr_b200_swiglu_f32`` -- f32, in the reference's CPU operation
order.  Weights come from the reference's own archive format (``NamedParameters``); torch only owns the device memory.

The policy / value heads of the example (pooling, trunks, card heads: mod.rs:408-574) are not part of this module.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _native
from .nn import TnsrError
from .parameters import NamedParameters

F32_MIN = np.float32(-3.4028234663852886e38)


@dataclass
class FortyFiveConfig:
    token_dim: int
    token_heads: int
    token_layers: int
    token_max_tokens: int
    token_vocab_size: int
    token_type_vocab_size: int
    phase_embed_dim: int
    num_phases: int
    use_phase_heads: bool
    use_card_conditioned_actions: bool
    use_separate_critic: bool
    use_privileged_critic: bool
    use_rope: bool
    use_swiglu: bool

    def validate(self):
        """``Model::validate`` (mod.rs:53-90), the part that concerns the encoder."""
        if not (self.use_swiglu and not self.use_rope and not self.use_privileged_critic):
            raise TnsrError("this port supports learned-position SwiGLU encoders and legal-information critics")
        if not (2 <= self.token_dim <= 4096 and self.token_heads > 0 and self.token_dim % self.token_heads == 0):
            raise TnsrError("invalid model width/heads")
        if not (0 < self.token_layers <= 128 and 0 < self.token_max_tokens <= 8192):
            raise TnsrError("invalid model layers/sequence")
        if self.use_card_conditioned_actions and not (self.use_phase_heads and self.token_max_tokens >= 15):
            raise TnsrError("card heads require phase heads and 15 token positions")
        if not (0 < self.token_vocab_size <= 1 << 24 and 0 < self.token_type_vocab_size <= 1 << 24):
            raise TnsrError("invalid embedding vocabulary")


def observation_inputs(config: FortyFiveConfig, token_ids, token_type_ids):
    """``Observations::inputs`` (mod.rs:645-698): ids, type ids, the input mask (1 where id != 0), the additive key
    mask (0 for live tokens -- and for position 0 of an all-padding row -- else f32::MIN) and the pooling mask."""
    ids = np.asarray(token_ids, dtype=np.int64)
    kinds = np.asarray(token_type_ids, dtype=np.int64)
    s = config.token_max_tokens
    if ids.ndim != 2 or ids.shape[0] == 0 or kinds.shape != ids.shape:
        raise TnsrError("observation batch sizes disagree or are empty")
    if ids.shape[1] != s:
        raise TnsrError(f"observation token width must be {s}")
    if ids.min() < 0 or ids.max() >= config.token_vocab_size or kinds.min() < 0 or kinds.max() >= config.token_type_vocab_size:
        raise TnsrError("token or type ID out of range")
    live = ids != 0
    first = np.zeros_like(live)
    first[:, 0] = True
    safe = live | (~live.any(axis=1, keepdims=True) & first)
    return (ids.astype(np.uint32), kinds.astype(np.uint32), live.astype(np.float32),
            np.where(safe, np.float32(0.0), F32_MIN).astype(np.float32),
            np.where(safe, np.float32(0.0), np.float32(-np.inf)).astype(np.float32))


class FortyFiveEncoder:
    def __init__(self, named: NamedParameters, config, prefix: str = "token_encoder", device: int = 0):
        import torch
        self.config = config if isinstance(config, FortyFiveConfig) else FortyFiveConfig(**config)
        self.config.validate()
        self.prefix = prefix
        self.torch = torch
        self.device = torch.device("cuda", device)
        c = self.config
        d, s = c.token_dim, c.token_max_tokens
        self.hidden = -(-8 * d // 3)
        self._w = {}

        def put(name, shape):
            values = named.get(f"{prefix}.{name}", list(shape)).values().reshape(shape)
            self._w[name] = torch.from_numpy(np.ascontiguousarray(values, dtype=np.float32)).to(self.device)

        put("token_embedding.weight", (c.token_vocab_size, d))
        put("token_type_embedding.weight", (c.token_type_vocab_size, d))
        put("position_embedding.weight", (s, d))
        for i in range(c.token_layers):
            p = f"encoder.layers.{i}"
            for norm in ("attn_norm", "ffn_norm"):
                put(f"{p}.{norm}.weight", (d,))
                put(f"{p}.{norm}.bias", (d,))
            for name, n_in, n_out in (("attention.qkv_proj", d, 3 * d), ("attention.out_proj", d, d),
                                      ("feed_forward.gate_proj", d, self.hidden), ("feed_forward.up_proj", d, self.hidden),
                                      ("feed_forward.down_proj", self.hidden, d)):
                put(f"{p}.{name}.weight", (n_out, n_in))        # [output, input]: the transposed operand of the GEMM
                put(f"{p}.{name}.bias", (n_out,))
        put("output_norm.weight", (d,))
        put("output_norm.bias", (d,))
        positions = np.arange(s, dtype=np.uint32)
        if c.use_card_conditioned_actions:
            positions[10:15] = 10                               # the five hand slots share one position (mod.rs:338-341)
        self._positions = torch.from_numpy(positions.view(np.int32)).to(self.device)
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)

    @classmethod
    def load(cls, directory: str, prefix: str = "token_encoder", device: int = 0) -> "FortyFiveEncoder":
        named, config = NamedParameters.load(directory)
        return cls(named, config, prefix, device)

    # -- plumbing --------------------------------------------------------------------------------
    def _call(self, name, *args):
        code = getattr(_native.lib(), name)(*args)
        if code != 0:
            raise TnsrError(f"{name}: {_native.last_error(None)}")

    @staticmethod
    def _p(t):
        return C.c_void_p(t.data_ptr())

    def _linear(self, x, name, rows, n_in, n_out, stream):
        out = self.torch.empty((rows, n_out), dtype=self.torch.float32, device=self.device)
        self._call("tnsr_b200_gemm_f32_strict", self._p(x), self._p(self._w[name + ".weight"]), self._p(self._w[name + ".bias"]),
                   self._p(out), rows, n_in, n_out, 1, stream)
        return out

    def _norm(self, x, name, rows, width, stream):
        out = self.torch.empty((rows, width), dtype=self.torch.float32, device=self.device)
        self._call("tnsr_b200_layernorm", self._p(x), self._p(self._w[name + ".weight"]), self._p(self._w[name + ".bias"]),
                   self._p(out), rows, width, 1e-5, 0, 1, stream)
        return out

    # -- Model::encode ---------------------------------------------------------------------------
    def encode(self, token_ids, token_type_ids) -> np.ndarray:
        """Encoded tokens ``[batch, token_max_tokens, token_dim]`` (after the output LayerNorm)."""
        torch, c = self.torch, self.config
        ids, kinds, initial, key_mask, _ = observation_inputs(c, token_ids, token_type_ids)
        batch, s, d, heads = ids.shape[0], c.token_max_tokens, c.token_dim, c.token_heads
        rows = batch * s
        with torch.cuda.device(self.device):
            stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            to_dev = lambda a, view=None: torch.from_numpy(np.ascontiguousarray(a).view(view) if view else np.ascontiguousarray(a)).to(self.device)
            d_ids, d_kinds = to_dev(ids, np.int32), to_dev(kinds, np.int32)
            d_initial, d_key = to_dev(initial), to_dev(key_mask)
            x = torch.empty((rows, d), dtype=torch.float32, device=self.device)
            self._status.zero_()
            self._call("tnsr_b200_encoder_embed", self._p(self._w["token_embedding.weight"]),
                       self._p(self._w["token_type_embedding.weight"]), self._p(self._w["position_embedding.weight"]),
                       self._p(d_ids), self._p(d_kinds), self._p(self._positions), self._p(d_initial), self._p(x), rows, s,
                       c.token_vocab_size, c.token_type_vocab_size, d, self._p(self._status), stream)
            for i in range(c.token_layers):
                p = f"encoder.layers.{i}"
                qkv = self._linear(self._norm(x, p + ".attn_norm", rows, d, stream), p + ".attention.qkv_proj", rows, d, 3 * d, stream)
                context = torch.empty((rows, d), dtype=torch.float32, device=self.device)
                base = qkv.data_ptr()
                self._call("tnsr_b200_encoder_attention", C.c_void_p(base), C.c_void_p(base + 4 * d), C.c_void_p(base + 8 * d),
                           3 * d, self._p(d_key), self._p(context), batch, s, heads, d // heads, stream)
                update = self._linear(context, p + ".attention.out_proj", rows, d, d, stream)
                self._call("tnsr_b200_add_f32", self._p(x), self._p(update), self._p(x), rows * d, stream)
                normalized = self._norm(x, p + ".ffn_norm", rows, d, stream)
                gate = self._linear(normalized, p + ".feed_forward.gate_proj", rows, d, self.hidden, stream)
                up = self._linear(normalized, p + ".feed_forward.up_proj", rows, d, self.hidden, stream)
                self._call("tnsr_b200_swiglu_f32", self._p(gate), self._p(up), self._p(gate), rows * self.hidden, stream)
                update = self._linear(gate, p + ".feed_forward.down_proj", rows, self.hidden, d, stream)
                self._call("tnsr_b200_add_f32", self._p(x), self._p(update), self._p(x), rows * d, stream)
            out = self._norm(x, "output_norm", rows, d, stream)
            torch.cuda.synchronize()
            if int(self._status.item()) != 0:
                raise TnsrError("token or type ID out of range")
            return out.cpu().numpy().reshape(batch, s, d)
