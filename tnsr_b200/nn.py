"""Host-side mirror of tnsr's cached-GPT API on top of the B200 library.

Names, argument meaning, guard order and error messages follow the reference:
``Backend`` (src/runtime.rs:15-25), ``GptConfig`` / ``Gpt`` (src/nn.rs:543-622),
``Gpt::decoder*`` / ``generate_cached`` (src/nn/kv_cache.rs:89-157),
``GptDecoder`` (src/nn/kv_cache.rs:160-389) and ``Parameter`` revisions
(src/tensor/storage.rs:17-117).  The reference is Rust; this module is the
Python statement of the same wrapper so the parity tests read like
tests/kv_cache.rs.  There is no CPU executor here: ``Backend.Cpu`` is refused.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

MAX_EXACT_F32_INTEGER = 1 << 24
USIZE_MAX = (1 << 64) - 1
ISIZE_MAX = (1 << 63) - 1


class TnsrError(RuntimeError):
    """The ``anyhow::Error`` of the reference: carries only a message."""


class Backend(enum.Enum):
    Cpu = "cpu"
    Cuda = "cuda"
    Ptx = "ptx"  # alias of Cuda, as in the reference


class GptAttentionPrecision(enum.Enum):
    F32 = "f32"
    Bf16 = "bf16"


class GptPrefillMode(enum.Enum):
    Auto = "auto"
    Scalar = "scalar"


@dataclass(frozen=True)
class GptDecoderOptions:
    attention_precision: GptAttentionPrecision = GptAttentionPrecision.F32
    prefill: GptPrefillMode = GptPrefillMode.Auto


class Parameter:
    """Shared, versioned f32 tensor: host writes bump ``revision``."""

    def __init__(self, values, shape):
        values = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        assert values.size == int(np.prod(shape, dtype=np.int64)), "parameter shape mismatch"
        self._values = values.copy()
        self._shape = tuple(int(s) for s in shape)
        self._revision = 0

    @property
    def shape(self):
        return self._shape

    def values(self) -> np.ndarray:
        return self._values.copy()

    def set_values(self, values) -> None:
        values = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        if values.size != self._values.size:
            raise TnsrError("parameter length changed")
        self._values = values.copy()
        self._revision = (self._revision + 1) & USIZE_MAX

    def revision(self) -> int:
        return self._revision

    def _view(self) -> np.ndarray:
        return self._values


def xavier_values(rows: int, columns: int, seed: int) -> np.ndarray:
    """``xavier_parameter`` (src/nn.rs:303-316): 64-bit LCG
    ``state = state * 6364136223846793005 + 1``; the top 24 bits give a unit in
    [0, 1); value = (unit * 2 - 1) * sqrt(6 / (rows + columns)), all in f32.
    The recurrence is unrolled in closed form so it vectorises:
    ``state_i = a^i * seed + (1 + a + ... + a^(i-1))`` modulo 2^64."""
    n = rows * columns
    a = np.uint64(6364136223846793005)
    with np.errstate(over="ignore"):
        powers = np.cumprod(np.full(n, a, dtype=np.uint64))              # a^1 .. a^n
        geometric = np.concatenate(([np.uint64(1)], np.cumsum(powers[:-1], dtype=np.uint64) + np.uint64(1)))
        state = powers * np.uint64(seed) + geometric
    unit = (state >> np.uint64(40)).astype(np.float32) / np.float32(1 << 24)
    limit = np.sqrt(np.float32(6.0) / np.float32(rows + columns), dtype=np.float32)
    return ((unit * np.float32(2.0) - np.float32(1.0)) * limit).astype(np.float32)


def xavier_parameter(rows: int, columns: int, seed: int) -> Parameter:
    return Parameter(xavier_values(rows, columns, seed), (rows, columns))


@dataclass
class GptConfig:
    vocab_size: int
    max_sequence_length: int
    embed_dim: int
    num_heads: int
    feed_forward_dim: int
    num_layers: int
    layer_norm_epsilon: float
    # Extensions beyond the reference's seven fields.  "relu" is nn::Gpt's own
    # block; "gelu" and "swiglu" use nn::gelu / nn::silu.  weight_dtype "bf16"
    # selects the tensor-core path (bf16 operands, f32 accumulation).
    activation: str = "relu"
    weight_dtype: str = "f32"


class MultiHeadAttention:
    def __init__(self, embed_dim: int, num_heads: int, seed_offset: int = 0):
        assert embed_dim > 0, "attention embed_dim must be non-zero"
        assert num_heads > 0, "attention num_heads must be non-zero"
        assert embed_dim % num_heads == 0, "attention embed_dim must be divisible by num_heads"
        zeros = lambda: Parameter(np.zeros(embed_dim, np.float32), (embed_dim,))
        self.query_weight = xavier_parameter(embed_dim, embed_dim, seed_offset + 1)
        self.query_bias = zeros()
        self.key_weight = xavier_parameter(embed_dim, embed_dim, seed_offset + 2)
        self.key_bias = zeros()
        self.value_weight = xavier_parameter(embed_dim, embed_dim, seed_offset + 3)
        self.value_bias = zeros()
        self.output_weight = xavier_parameter(embed_dim, embed_dim, seed_offset + 4)
        self.output_bias = zeros()


class TransformerBlock:
    """Pre-norm block (src/nn.rs:442-501).  With ``activation == "swiglu"`` the
    two-matrix FFN is replaced by gate/up/down (seeds +5, +6, +7)."""

    def __init__(self, embed_dim, num_heads, feed_forward_dim, epsilon, seed_offset=0, activation="relu"):
        assert feed_forward_dim > 0, "transformer feed_forward_dim must be non-zero"
        assert epsilon > 0.0 and np.isfinite(epsilon), "transformer epsilon must be finite and positive"
        d, f = embed_dim, feed_forward_dim
        ones = lambda n: Parameter(np.ones(n, np.float32), (n,))
        zeros = lambda n: Parameter(np.zeros(n, np.float32), (n,))
        self.attention = MultiHeadAttention(d, num_heads, seed_offset)
        self.attention_norm_weight, self.attention_norm_bias = ones(d), zeros(d)
        self.feed_forward_norm_weight, self.feed_forward_norm_bias = ones(d), zeros(d)
        self.activation = activation
        if activation == "swiglu":
            self.feed_forward_gate_weight = xavier_parameter(d, f, seed_offset + 5)
            self.feed_forward_gate_bias = zeros(f)
            self.feed_forward_up_weight = xavier_parameter(d, f, seed_offset + 6)
            self.feed_forward_up_bias = zeros(f)
            self.feed_forward_down_weight = xavier_parameter(f, d, seed_offset + 7)
            self.feed_forward_down_bias = zeros(d)
        else:
            self.feed_forward_input_weight = xavier_parameter(d, f, seed_offset + 5)
            self.feed_forward_input_bias = zeros(f)
            self.feed_forward_output_weight = xavier_parameter(f, d, seed_offset + 6)
            self.feed_forward_output_bias = zeros(d)
        self.epsilon = epsilon


class Gpt:
    """Decoder-only transformer with learned positions and a tied LM head."""

    def __init__(self, config: GptConfig):
        c = config
        assert c.vocab_size > 0, "GPT vocabulary must be non-empty"
        assert c.vocab_size - 1 <= MAX_EXACT_F32_INTEGER, \
            "GPT vocabulary indices must be exactly representable as f32"
        assert c.max_sequence_length > 0, "GPT maximum sequence length must be non-zero"
        assert c.max_sequence_length - 1 <= MAX_EXACT_F32_INTEGER, \
            "GPT position indices must be exactly representable as f32"
        assert c.embed_dim > 0, "GPT embedding width must be non-zero"
        assert c.num_layers > 0, "GPT must contain at least one layer"
        assert c.feed_forward_dim > 0, "GPT feed-forward width must be non-zero"
        assert c.num_heads > 0 and c.embed_dim % c.num_heads == 0, \
            "GPT embedding width must be divisible by a non-zero head count"
        assert np.isfinite(c.layer_norm_epsilon) and c.layer_norm_epsilon > 0.0, \
            "GPT layer norm epsilon must be finite and positive"
        assert c.activation in ("relu", "gelu", "swiglu")
        assert c.weight_dtype in ("f32", "bf16")
        self._config = c
        self.token_embedding = xavier_parameter(c.vocab_size, c.embed_dim, 101)
        self.position_embedding = xavier_parameter(c.max_sequence_length, c.embed_dim, 102)
        self.blocks = [
            TransformerBlock(c.embed_dim, c.num_heads, c.feed_forward_dim, c.layer_norm_epsilon,
                             1000 + layer * 100, c.activation)
            for layer in range(c.num_layers)
        ]
        self.final_norm_weight = Parameter(np.ones(c.embed_dim, np.float32), (c.embed_dim,))
        self.final_norm_bias = Parameter(np.zeros(c.embed_dim, np.float32), (c.embed_dim,))

    @classmethod
    def new(cls, config: GptConfig) -> "Gpt":
        return cls(config)

    def config(self) -> GptConfig:
        return self._config

    # -- sessions (src/nn/kv_cache.rs:89-115) --------------------------------
    def decoder(self, backend, batch_size: int) -> "GptDecoder":
        return self.decoder_with_capacity(backend, batch_size, self._config.max_sequence_length)

    def decoder_with_capacity(self, backend, batch_size: int, capacity: int) -> "GptDecoder":
        return self.decoder_with_options(backend, batch_size, capacity, GptDecoderOptions())

    def decoder_with_options(self, backend, batch_size: int, capacity: int,
                             options: GptDecoderOptions, **extra) -> "GptDecoder":
        return GptDecoder(self, backend, batch_size, capacity, options, **extra)

    # -- full-context paths (src/nn.rs:629-715) -------------------------------
    def forward(self, backend, token_ids) -> np.ndarray:
        """``Gpt::forward`` evaluated on the backend: logits ``[batch, sequence, vocabulary]``
        of a whole ``[batch, sequence]`` id block (a fresh session decoding one chunk is the same graph:
        src/nn/kv_cache/graph.rs with past = 0)."""
        ids = np.asarray(token_ids)
        if ids.ndim != 2:
            raise TnsrError("GPT token IDs must have shape [batch, sequence]")
        batch, sequence = ids.shape
        if batch == 0:
            raise TnsrError("GPT batch size must be non-zero")
        if sequence == 0:
            raise TnsrError("GPT sequence length must be non-zero")
        if sequence > self._config.max_sequence_length:
            raise TnsrError(f"GPT sequence length {sequence} exceeds configured maximum "
                            f"{self._config.max_sequence_length}")
        decoder = self.decoder_with_capacity(backend, batch, sequence)
        logits = decoder.decode([int(t) for t in ids.reshape(-1)])
        return logits.reshape(batch, sequence, self._config.vocab_size)

    def generate(self, backend, prompt: Sequence[int], max_new_tokens: int) -> List[int]:
        """``Gpt::generate``: greedy, re-running the whole retained context for every new token."""
        if len(prompt) == 0:
            raise TnsrError("GPT generation prompt must be non-empty")
        if not all(0 <= t < self._config.vocab_size for t in prompt):
            raise TnsrError("GPT generation prompt contains an out-of-range token")
        tokens = [int(t) for t in prompt]
        context = self._config.max_sequence_length
        decoder = None
        for _ in range(max_new_tokens):
            window = tokens[max(0, len(tokens) - context):]
            if decoder is None:
                decoder = self.decoder(backend, 1)
            decoder.reset()
            logits = decoder.decode(window)
            tokens.append(argmax_last(logits[logits.size - self._config.vocab_size:]))
        return tokens

    # -- greedy generation (src/nn/kv_cache.rs:121-157) ----------------------
    def generate_cached(self, backend, prompt: Sequence[int], max_new_tokens: int) -> List[int]:
        if len(prompt) == 0:
            raise TnsrError("GPT generation prompt must be non-empty")
        if not all(0 <= t < self._config.vocab_size for t in prompt):
            raise TnsrError("GPT generation prompt contains an out-of-range token")
        tokens = [int(t) for t in prompt]
        if max_new_tokens == 0:
            return tokens
        decoder = self.decoder(backend, 1)
        vocab = self._config.vocab_size
        for _ in range(max_new_tokens):
            if decoder.is_empty() or decoder.len() == decoder.capacity():
                decoder.reset()
                start = max(0, len(tokens) - decoder.capacity())
                logits = decoder.decode(tokens[start:])
            else:
                logits = decoder.decode(tokens[-1:])
            tokens.append(argmax_last(logits[logits.size - vocab:]))
        return tokens


def argmax_last(row: np.ndarray) -> int:
    """``max_by(total_cmp)``: last index of the maximum under IEEE totalOrder."""
    bits = np.ascontiguousarray(row, dtype=np.float32).view(np.int32).astype(np.int64)
    keys = bits ^ ((bits >> 31) & 0x7FFFFFFF)
    return int(keys.size - 1 - np.argmax(keys[::-1]))


def model_parameters(model: Gpt) -> List[Parameter]:
    """Canonical order (src/nn/kv_cache.rs:392-421)."""
    result = [model.token_embedding, model.position_embedding, model.final_norm_weight,
              model.final_norm_bias]
    for b in model.blocks:
        a = b.attention
        result += [a.query_weight, a.query_bias, a.key_weight, a.key_bias, a.value_weight,
                   a.value_bias, a.output_weight, a.output_bias, b.attention_norm_weight,
                   b.attention_norm_bias, b.feed_forward_norm_weight, b.feed_forward_norm_bias]
        if b.activation == "swiglu":
            result += [b.feed_forward_gate_weight, b.feed_forward_gate_bias,
                       b.feed_forward_up_weight, b.feed_forward_up_bias,
                       b.feed_forward_down_weight, b.feed_forward_down_bias]
        else:
            result += [b.feed_forward_input_weight, b.feed_forward_input_bias,
                       b.feed_forward_output_weight, b.feed_forward_output_bias]
    return result


class GptDecoder:
    """An inference session bound to one model, batch size and context capacity.

    ``decode`` takes row-major ``[batch, new_tokens]`` ids and returns logits for
    those positions only; all rows advance together; overflow is an error, not an
    eviction.  ``backend_impl`` lets a test drive the same wrapper with another
    backend object (``refresh(index, values)``, ``reset()``,
    ``decode(tokens[batch, chunk], position) -> flat f32 logits``).
    """

    def __init__(self, model: Gpt, backend, batch: int, capacity: int,
                 options: GptDecoderOptions = GptDecoderOptions(), backend_impl=None, device: int = 0):
        config = model.config()
        if not batch > 0:
            raise TnsrError("decoder batch size must be non-zero")
        if not (0 < capacity <= config.max_sequence_length):
            raise TnsrError("decoder capacity must fit the model context")
        elements = batch * capacity * config.embed_dim
        if elements > USIZE_MAX:
            raise TnsrError("decoder cache size overflow")
        if elements * 4 > USIZE_MAX:
            raise TnsrError("decoder cache byte size overflow")
        if elements * 4 > ISIZE_MAX:
            raise TnsrError("decoder cache exceeds allocation limits")
        if elements * 4 * config.num_layers * 2 > USIZE_MAX:
            raise TnsrError("decoder total cache size overflow")
        self._model = model
        self._parameters = model_parameters(model)
        self._revisions = [p.revision() for p in self._parameters]
        self._uploaded: List[Optional[int]] = [None] * len(self._parameters)
        self._batch, self._capacity, self._length = batch, capacity, 0
        self._failed = False
        self._options = options
        if backend_impl is not None:
            self._backend = backend_impl
        elif backend in (Backend.Cuda, Backend.Ptx):
            from .session import B200Session
            self._backend = B200Session(config, batch, capacity, options, device=device)
        elif backend == Backend.Cpu:
            raise TnsrError("this library has no CPU executor; use Backend.Cuda")
        else:
            raise TnsrError(f"unknown backend {backend!r}")
        self._refresh()

    # CudaDecoder::refresh (src/nn/kv_cache/cuda.rs:125-141): upload only the
    # tensors whose revision differs from the one last uploaded.
    def _refresh(self):
        for i, p in enumerate(self._parameters):
            rev = p.revision()
            if self._uploaded[i] != rev:
                self._backend.refresh(i, p._view())
                self._uploaded[i] = rev

    def len(self) -> int:
        return self._length

    def __len__(self) -> int:
        return self._length

    def is_empty(self) -> bool:
        return self._length == 0

    def capacity(self) -> int:
        return self._capacity

    def batch_size(self) -> int:
        return self._batch

    def reset(self) -> None:
        self._failed = True
        self._length = 0
        self._backend.reset()
        self._failed = False

    def save_state(self, directory: str) -> None:
        """K/V rows and length into a tensor archive (see ``parameters.save_decoder_state``)."""
        from .parameters import save_decoder_state
        save_decoder_state(self, directory)

    def load_state(self, directory: str) -> None:
        from .parameters import load_decoder_state
        load_decoder_state(self, directory)

    def decode(self, tokens: Sequence[int]) -> np.ndarray:
        if self._failed:
            raise TnsrError("decoder execution failed; reset the cache before reuse")
        n = len(tokens)
        if n == 0 or n % self._batch != 0:
            raise TnsrError("tokens must be a nonempty rectangular [batch, sequence] chunk")
        chunk = n // self._batch
        if chunk > self._capacity - self._length:
            raise TnsrError("decoder context capacity exceeded")
        vocab = self._model.config().vocab_size
        if not all(0 <= int(t) < vocab for t in tokens):
            raise TnsrError("decoder token is outside the vocabulary")
        revisions = [p.revision() for p in self._parameters]
        if not (self.is_empty() or revisions == self._revisions):
            raise TnsrError("model weights changed; reset the decoder cache")
        ids = np.asarray(tokens, dtype=np.uint32).reshape(self._batch, chunk)
        self._failed = True
        self._refresh()
        logits = self._backend.decode(ids, self._length)
        if [p.revision() for p in self._parameters] != revisions:
            raise TnsrError("model weights changed during decoding; reset the cache")
        self._revisions = revisions
        self._length += chunk
        self._failed = False
        return logits
