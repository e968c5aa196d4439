"""The forty_five token encoder (tnsr examples/forty_five/mod.rs:329-407) on the B200 operator set against the CPU
restatement, which tests/test_forty_five_host.py pins to the reference's own fixture."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import forty_five as cpu  # noqa: E402
from tnsr_b200.forty_five import FortyFiveEncoder, observation_inputs  # noqa: E402
from tnsr_b200.nn import TnsrError  # noqa: E402
from tnsr_b200.parameters import NamedParameters  # noqa: E402

FIXTURES = os.path.join(os.path.dirname(__file__), "golden", "forty_five")


@pytest.mark.parametrize("variant,prefix", [("tiny", "token_encoder"), ("tiny-separate", "token_encoder"),
                                            ("tiny-separate", "critic_encoder")])
def test_encoder_matches_the_checker_on_the_reference_archives(variant, prefix):
    named, config = NamedParameters.load(os.path.join(FIXTURES, variant))
    ids = [[1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 0], [0] * 16, [5, 0, 0, 9, 0, 0, 0, 0, 0, 0, 63, 62, 0, 1, 2, 3]]
    kinds = [[0, 1, 2, 3, 4, 5, 0, 1, 2, 3, 4, 5, 0, 1, 2, 0], [0] * 16, [1, 0, 0, 2, 0, 0, 0, 0, 0, 0, 5, 4, 0, 3, 2, 1]]
    want = cpu.Model(named, config).encode(prefix, ids, kinds)
    got = FortyFiveEncoder(named, config, prefix).encode(ids, kinds)
    assert got.shape == want.shape == (3, 16, 8)
    assert np.max(np.abs(got - want)) <= 2e-6


def test_encoder_at_a_wider_shape_with_padding_and_shared_hand_positions():
    config = dict(token_dim=96, token_heads=4, token_layers=3, token_max_tokens=40, token_vocab_size=70,
                  token_type_vocab_size=6, phase_embed_dim=4, num_phases=6, use_phase_heads=True,
                  use_card_conditioned_actions=True, use_separate_critic=False, use_privileged_critic=False, use_rope=False,
                  use_swiglu=True)
    d, s, hidden = 96, 40, 256
    rng = np.random.default_rng(71)
    named = NamedParameters()

    def add(name, shape, scale):
        named.insert("token_encoder." + name, (rng.standard_normal(shape) * scale).astype(np.float32), list(shape), "policy")

    add("token_embedding.weight", (70, d), 0.5)
    add("token_type_embedding.weight", (6, d), 0.5)
    add("position_embedding.weight", (s, d), 0.5)
    for i in range(3):
        p = f"encoder.layers.{i}"
        for norm in ("attn_norm", "ffn_norm"):
            named.insert(f"token_encoder.{p}.{norm}.weight", (1 + 0.1 * rng.standard_normal(d)).astype(np.float32), [d], "policy")
            add(f"{p}.{norm}.bias", (d,), 0.1)
        for name, n_in, n_out in (("attention.qkv_proj", d, 3 * d), ("attention.out_proj", d, d), ("feed_forward.gate_proj", d, hidden),
                                  ("feed_forward.up_proj", d, hidden), ("feed_forward.down_proj", hidden, d)):
            add(f"{p}.{name}.weight", (n_out, n_in), 0.08)
            add(f"{p}.{name}.bias", (n_out,), 0.05)
    named.insert("token_encoder.output_norm.weight", np.ones(d, np.float32), [d], "policy")
    add("output_norm.bias", (d,), 0.1)
    ids = rng.integers(0, 70, size=(5, s))
    ids[0, 25:] = 0                      # trailing padding
    ids[1, :] = 0                        # an all-padding row keeps position 0 as its only key
    ids[2, ::3] = 0                      # holes
    kinds = rng.integers(0, 6, size=(5, s))
    want = cpu.Model(named, config).encode("token_encoder", ids, kinds)
    encoder = FortyFiveEncoder(named, config)
    got = encoder.encode(ids, kinds)
    assert np.all(np.isfinite(got))
    assert np.max(np.abs(got - want)) <= 1e-5 * max(1.0, float(np.max(np.abs(want))))
    # padding never influences live rows: changing the type id of a padded slot changes nothing
    kinds2 = kinds.copy()
    kinds2[0, 30] = (kinds2[0, 30] + 1) % 6
    assert np.array_equal(encoder.encode(ids, kinds2), got)
    with pytest.raises(TnsrError):
        encoder.encode(ids[:, :39], kinds[:, :39])
    bad = ids.copy()
    bad[3, 3] = 70
    with pytest.raises(TnsrError):
        encoder.encode(bad, kinds)
    _, _, initial, key_mask, pool_mask = observation_inputs(encoder.config, ids, kinds)
    assert initial[1].sum() == 0 and key_mask[1, 0] == 0 and np.all(key_mask[1, 1:] < -1e38) and np.isneginf(pool_mask[1, 1])
