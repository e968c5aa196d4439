"""Regenerates the committed fixtures in this folder.

Run from the repository root in a checkout that has the tnsr sources mounted:

    python tests/golden/make_golden.py /path/to/tnsr

It reads the known-answer vectors that tnsr's own tests hold for the cached-GPT
path and writes them as JSON.  Nothing here executes reference code (it is Rust
and there is no toolchain for it); the vectors are the literals of
  src/nn/activations/tests.rs:8-167   19 input bit patterns and the sigmoid /
                                      silu / gelu outputs PyTorch 2.11 gave
  tests/indexed_ops.rs:25-36          embedding gather
  tests/transformer.rs:86-103         batched matmul
  src/graph/mixed.rs:126-135          bf16 narrowing
It also copies the reference's own data fixtures of the forty_five example (examples/forty_five/fixtures/{tiny,
tiny-separate}: the parameter archive `manifest.json` + `weights.f32`, and `reference.json`, the inputs and expected
outputs its tests check the encoder against) into forty_five/ byte for byte.
The second half derives fixtures from this repository's own CPU checker
(oracle/), so the GPU tests can run where neither tnsr nor the generator is
present: greedy token ids and logits of configuration 0.
"""
import json
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def activation_vectors(ref):
    text = open(os.path.join(ref, "src/nn/activations/tests.rs")).read()
    body = text[text.index("fn check("):text.index("let x = Parameter::new(data.clone()")]
    groups = re.findall(r"vec!\[((?:\s*f32::from_bits\(0x[0-9a-f]{8}\),?\s*)+)\]", body)
    vecs = [[int(h, 16) for h in re.findall(r"0x([0-9a-f]{8})", g)] for g in groups]
    assert len(vecs) == 7 and all(len(v) == 19 for v in vecs), [len(v) for v in vecs]
    names = re.findall(r'"(sigmoid|silu|gelu)",', body)
    assert names == ["sigmoid", "silu", "gelu"]
    out = {"source": "src/nn/activations/tests.rs:8-167", "tolerance": 2e-6, "input_bits": vecs[0]}
    for i, name in enumerate(names):
        out[name] = {"value_bits": vecs[1 + 2 * i], "gradient_bits": vecs[2 + 2 * i]}
    return out


def literal_vectors():
    return {
        "embedding": {
            "source": "tests/indexed_ops.rs:25-36",
            "weight": [1, 2, 3, 4, 5, 6, 7, 8], "weight_shape": [4, 2],
            "indices": [2, 0, 3, 1], "expected": [5, 6, 1, 2, 7, 8, 3, 4],
        },
        "embedding_invalid": {
            "source": "tests/indexed_ops.rs:98-118",
            "cases": [["nan", "finite"], ["inf", "finite"], [-1.0, "non-negative"], [1.5, "integer"],
                      [3.4028234663852886e38, "usize"], [3.0, "out of range"]],
        },
        "batched_matmul": {
            "source": "tests/transformer.rs:86-103",
            "left": [1, 2, 3, 4, 5, 6, -1, 0, 1, 2, -2, 1], "left_shape": [2, 2, 3],
            "right": [1, 0, 0, 1, 1, 1, 2, -1, 1, 3, -2, 2], "right_shape": [2, 3, 2],
            "expected": [4, 5, 10, 11, -4, 3, 0, -6],
        },
        "bf16_narrowing": {
            "source": "src/graph/mixed.rs:126-135",
            "input": [1 + 1 / 256, -1 - 1 / 256, 1e-43], "expected": [1.0, -1.0, 0.0],
        },
        "linear": {
            "source": "src/nn.rs unit tests (linear with and without bias)",
        },
    }


def config0(activation):
    """Configuration 0: vocab 96, d 128, 4 layers, 4 heads, FFN 512, context 128,
    matrices N(0, 0.02) from seed 0, biases 0, LayerNorm weight 1 / bias 0,
    prompt of 16 ids uniform in [0, 96) from seed 1, 64 greedy steps."""
    from oracle import oracle
    from tests.workloads import config0_model, config0_prompt
    cfg, arrays = config0_model(activation)
    model = oracle.OracleModel(cfg.vocab_size, cfg.max_sequence_length, cfg.embed_dim, cfg.num_heads,
                               cfg.feed_forward_dim, cfg.num_layers, cfg.layer_norm_epsilon, activation)
    model.set_params(arrays)
    prompt = config0_prompt()
    tokens = model.generate_cached(prompt, 64)
    assert tokens == model.generate(prompt, 64)
    logits = model.forward(np.asarray(tokens[:-1], dtype=np.uint32)[None, :])[0]
    top2 = np.sort(logits[15:], axis=1)[:, -2:]
    return {
        "prompt": [int(t) for t in prompt],
        "tokens": [int(t) for t in tokens],
        "min_top1_top2_margin": float((top2[:, 1] - top2[:, 0]).min()),
        "last_logits_bits": [int(x) for x in logits[-1].view(np.uint32)],
        "prefill_last_logits_bits": [int(x) for x in logits[15].view(np.uint32)],
    }


def copy_forty_five_fixtures(ref):
    import shutil
    for variant in ("tiny", "tiny-separate"):
        src = os.path.join(ref, "examples/forty_five/fixtures", variant)
        dst = os.path.join(HERE, "forty_five", variant)
        os.makedirs(dst, exist_ok=True)
        for name in ("manifest.json", "weights.f32", "reference.json"):
            if os.path.exists(os.path.join(src, name)):
                shutil.copyfile(os.path.join(src, name), os.path.join(dst, name))


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of tninesling/tnsr>")
    ref = sys.argv[1]
    copy_forty_five_fixtures(ref)
    data = literal_vectors()
    data["activations"] = activation_vectors(ref)
    with open(os.path.join(HERE, "reference_vectors.json"), "w") as f:
        json.dump(data, f, indent=1)
    cfg0 = {"relu": config0("relu"), "gelu": config0("gelu")}
    with open(os.path.join(HERE, "config0_greedy.json"), "w") as f:
        json.dump(cfg0, f, indent=1)
    print("wrote reference_vectors.json, config0_greedy.json")


if __name__ == "__main__":
    main()
