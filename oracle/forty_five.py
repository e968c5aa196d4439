"""CPU restatement of tnsr's forty_five actor/critic model (examples/forty_five/mod.rs), f32.

TEST INFRASTRUCTURE ONLY, like the rest of ``oracle/``.  It follows the example's graph function by function --
``Observations::inputs`` (mod.rs:645-698), ``Model::encode`` (:329-407, the token transformer this repository runs on
the GPU), ``pool`` (:408-427), ``forward`` (:458-521) and ``card_heads`` (:522-574) -- on numpy f32 arrays, using the
checker's own primitives for LayerNorm, SiLU, GELU and softmax.  It is pinned to the reference's fixture
``examples/forty_five/fixtures/tiny/reference.json`` (inputs, logits [2, 46] and values [2]; tolerance 2e-5 as in
examples/forty_five/tests.rs:38-44): tests/test_forty_five_host.py.
"""
import numpy as np

from . import oracle

F32_MIN = np.float32(-3.4028234663852886e38)


class Model:
    def __init__(self, named, config):
        """`named`: a ``tnsr_b200.parameters.NamedParameters`` (or anything with ``get(name, shape).values()``)."""
        self.c = dict(config)
        c = self.c
        if not (c["use_swiglu"] and not c["use_rope"] and not c["use_privileged_critic"]):
            raise ValueError("this port supports learned-position SwiGLU encoders and legal-information critics")
        self.named = named

    def p(self, name, shape):
        return self.named.get(name, list(shape)).values().reshape(shape).astype(np.float32)

    # -- Observations::inputs ------------------------------------------------------------------
    def inputs(self, token_ids, token_type_ids):
        ids = np.asarray(token_ids, dtype=np.int64)
        kinds = np.asarray(token_type_ids, dtype=np.int64)
        nonzero = ids != 0
        any_row = nonzero.any(axis=1, keepdims=True)
        first = np.zeros_like(nonzero)
        first[:, 0] = True
        safe = nonzero | (~any_row & first)
        initial = nonzero.astype(np.float32)
        key = np.where(safe, np.float32(0.0), F32_MIN).astype(np.float32)
        pool = np.where(safe, np.float32(0.0), np.float32(-np.inf)).astype(np.float32)
        return ids, kinds, initial, key, pool

    # -- helpers ---------------------------------------------------------------------------------
    def linear(self, prefix, x, n_in, n_out):
        w = self.p(prefix + ".weight", (n_out, n_in))
        b = self.p(prefix + ".bias", (n_out,))
        flat = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, n_in)
        return oracle.linear(flat, np.ascontiguousarray(w.T), b).reshape(x.shape[:-1] + (n_out,))

    def norm(self, prefix, x, width):
        return oracle.layer_norm(np.ascontiguousarray(x, dtype=np.float32), self.p(prefix + ".weight", (width,)),
                                 self.p(prefix + ".bias", (width,)), 1e-5)

    # -- Model::encode ---------------------------------------------------------------------------
    def encode(self, prefix, token_ids, token_type_ids):
        c = self.c
        d, s, heads = c["token_dim"], c["token_max_tokens"], c["token_heads"]
        head = d // heads
        hidden = -(-8 * d // 3)
        ids, kinds, initial, key_mask, _ = self.inputs(token_ids, token_type_ids)
        batch = ids.shape[0]
        positions = np.arange(s)
        if c["use_card_conditioned_actions"]:
            positions[10:15] = 10
        x = (self.p(prefix + ".token_embedding.weight", (c["token_vocab_size"], d))[ids]
             + self.p(prefix + ".token_type_embedding.weight", (c["token_type_vocab_size"], d))[kinds]
             + self.p(prefix + ".position_embedding.weight", (s, d))[positions][None])
        x = np.where(initial[..., None] != 0, x, np.float32(0.0)).astype(np.float32)
        scale = np.float32(1.0) / np.sqrt(np.float32(head))
        for i in range(c["token_layers"]):
            p = f"{prefix}.encoder.layers.{i}"
            qkv = self.linear(p + ".attention.qkv_proj", self.norm(p + ".attn_norm", x, d), d, 3 * d)
            split = lambda start: qkv[..., start:start + d].reshape(batch, s, heads, head).transpose(0, 2, 1, 3)
            q, k, v = split(0), split(d), split(2 * d)
            scores = oracle.matmul(np.ascontiguousarray(q), np.ascontiguousarray(k.transpose(0, 1, 3, 2))) * scale \
                + key_mask[:, None, None, :]
            weights = oracle.softmax(scores.astype(np.float32))
            context = oracle.matmul(weights, np.ascontiguousarray(v)).transpose(0, 2, 1, 3).reshape(batch, s, d)
            x = x + self.linear(p + ".attention.out_proj", context, d, d)
            normalized = self.norm(p + ".ffn_norm", x, d)
            gate = oracle.silu(self.linear(p + ".feed_forward.gate_proj", normalized, d, hidden))
            up = self.linear(p + ".feed_forward.up_proj", normalized, d, hidden)
            x = x + self.linear(p + ".feed_forward.down_proj", gate * up, hidden, d)
        return self.norm(prefix + ".output_norm", x, d)

    # -- pool / heads ------------------------------------------------------------------------------
    def pool(self, prefix, encoded, query, query_width, pool_mask):
        d = self.c["token_dim"]
        batch = encoded.shape[0]
        query = self.linear(prefix + ".query_proj", self.norm(prefix + ".query_norm", query, query_width), query_width, d)
        keys = self.linear(prefix + ".key_proj", encoded, d, d)
        values = self.linear(prefix + ".value_proj", encoded, d, d)
        scores = (query.reshape(batch, 1, d) * keys).sum(axis=2, dtype=np.float32) \
            * (np.float32(1.0) / np.sqrt(np.float32(d))) + pool_mask
        weights = oracle.softmax(scores.astype(np.float32))[..., None]
        return (weights * values).sum(axis=1, dtype=np.float32)

    def card_heads(self, policy, encoded):
        d = self.c["token_dim"]
        batch = encoded.shape[0]
        hand = np.ascontiguousarray(encoded[:, 10:15])
        query = self.linear("card_action_heads.play_query", policy, d, d).reshape(batch, 1, d)
        keys = self.linear("card_action_heads.play_keys", hand, d, d)
        bias = self.linear("card_action_heads.play_bias", hand, d, 1).reshape(batch, 5)
        play = (query * keys).sum(axis=2, dtype=np.float32) * (np.float32(1.0) / np.sqrt(np.float32(d))) + bias
        cards = self.linear("card_action_heads.discard_cards", hand, d, d)
        subsets = np.arange(32)
        membership = ((subsets[:, None] >> np.arange(5)[None]) & 1).astype(np.float32)
        counts = membership.sum(axis=1).astype(np.int64)
        scales = np.sqrt(np.maximum(counts, 1).astype(np.float32))
        subset = np.einsum("sk,bkd->bsd", membership, cards).astype(np.float32) / scales[None, :, None]
        count_embeddings = self.p("card_action_heads.discard_count_embedding.weight", (6, d))[counts]
        features = np.concatenate([subset, np.broadcast_to(count_embeddings[None], (batch, 32, d)),
                                   np.broadcast_to(policy.reshape(batch, 1, d), (batch, 32, d))], axis=2)
        features = self.norm("card_action_heads.discard_trunk.0", features, 3 * d)
        features = oracle.gelu(self.linear("card_action_heads.discard_trunk.1", features, 3 * d, d))
        discard = self.linear("card_action_heads.discard_trunk.3", features, d, 1).reshape(batch, 32)
        return discard, play

    # -- Model::forward ------------------------------------------------------------------------------
    def forward(self, token_ids, token_type_ids, phase_ids):
        c = self.c
        d, phase = c["token_dim"], c["phase_embed_dim"]
        *_, pool_mask = self.inputs(token_ids, token_type_ids)
        encoded = self.encode("token_encoder", token_ids, token_type_ids)
        cls = encoded[:, 0]
        phase_embedding = self.p("phase_embedding.weight", (c["num_phases"], phase))[np.asarray(phase_ids, dtype=np.int64)]
        pooled = self.pool("policy_pool", encoded, np.concatenate([cls, phase_embedding], axis=1), d + phase, pool_mask)
        features = self.norm("policy_trunk.0", np.concatenate([cls, pooled, phase_embedding], axis=1), 2 * d + phase)
        features = oracle.gelu(self.linear("policy_trunk.1", features, 2 * d + phase, d))
        policy = self.norm("policy_trunk.3", features, d)
        if c["use_phase_heads"]:
            if c["use_card_conditioned_actions"]:
                discard, play = self.card_heads(policy, encoded)
            else:
                discard, play = self.linear("discard_head", policy, d, 32), self.linear("play_head", policy, d, 5)
            logits = np.concatenate([self.linear("bid_head", policy, d, 5), self.linear("suit_head", policy, d, 4),
                                     discard, play], axis=1)
        else:
            logits = self.linear("policy_head", policy, d, 46)
        value_encoded = self.encode("critic_encoder", token_ids, token_type_ids) if c["use_separate_critic"] else encoded
        value_cls = value_encoded[:, 0]
        batch = value_cls.shape[0]
        query = np.broadcast_to(self.p("value_pool.query", (d,))[None], (batch, d))
        pooled = self.pool("value_pool.pool", value_encoded, query, d, pool_mask)
        features = self.norm("value_trunk.0", np.concatenate([value_cls, pooled], axis=1), 2 * d)
        features = oracle.gelu(self.linear("value_trunk.1", features, 2 * d, d))
        features = oracle.gelu(self.linear("value_trunk.3", features, d, d // 2))
        return logits.astype(np.float32), self.linear("value_trunk.5", features, d // 2, 1).reshape(batch)
