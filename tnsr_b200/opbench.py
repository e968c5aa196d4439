"""Operator-level measurements of the kernels behind the C ABI.

    python -m tnsr_b200.opbench gemm        # configuration 1: square sweep + skinny decode shapes
    python -m tnsr_b200.opbench skinny_gemm # only the skinny decode shapes of configuration 1 (M = 1, 8, 64; bf16 out)
    python -m tnsr_b200.opbench serving_gemms  # configuration 4's projection shapes at prefill and decode size
    python -m tnsr_b200.opbench mlp         # configuration 2: fused SwiGLU MLP 4096 x 2048 -> 5632 -> 2048
    python -m tnsr_b200.opbench attention   # configuration 3: 64 sessions x 16 heads x 64, ragged lengths <= 4096
    python -m tnsr_b200.opbench serving_attention  # configuration 4's decode attention: 256 x 12 x 64, 641 live keys
    python -m tnsr_b200.opbench elementwise # LayerNorm, SwiGLU, embedding, greedy pick
    python -m tnsr_b200.opbench prefill_attention  # configuration 4's prefill attention on both engines
    python -m tnsr_b200.opbench all

Every line is one JSON object: algorithmic flops / bytes, CUDA-event time (median of `--samples`
after 3 warm-up launches), achieved TFLOP/s or GB/s and the fraction of the measured peak
(MEASURED_PEAKS.json when present, else 6650 GB/s / 1590 TFLOP/s).  Between timed launches the
operands rotate through enough distinct copies to exceed the 126 MB L2 (or, where one operand set
is larger than L2 anyway, stay put).  torch only owns device memory and events here.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

import numpy as np
import torch

from . import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
L2_BYTES = 126 << 20


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def lib():
    return _native.lib()


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ok(code):
    if code != 0:
        raise RuntimeError(f"{_native.STATUS.get(code, code)}: {_native.last_error(None)}")


def timed(launch, sets, samples):
    """Median milliseconds of launch(i) over `samples` launches, rotating i over `sets` operand copies."""
    for i in range(3):
        launch(i % sets)
    torch.cuda.synchronize()
    times = []
    for i in range(samples):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        launch((i + 3) % sets)
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    return float(np.median(times)), times


def timed_graph(launch, sets, samples, reps=None):
    """Per-launch milliseconds of a SHORT kernel: `reps` launches, rotating over the operand copies, are captured into
    one CUDA graph and the replay is timed -- a single launch between two events would mostly measure the host (tensor-map
    encoding, the ctypes call, the launch itself), not the GPU.  Includes the ~1.2 us a dependent graph node costs."""
    reps = reps or max(sets, 16)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(3):
            launch(i % sets)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(reps):
                launch(i % sets)
        times = []
        for i in range(samples + 2):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            e1.synchronize()
            if i >= 2:
                times.append(e0.elapsed_time(e1) / reps)
    torch.cuda.synchronize()
    return float(np.median(times)), times


def copies_for(bytes_per_set):
    return max(1, min(64, -(-2 * L2_BYTES // max(bytes_per_set, 1))))


RESULTS = []      # every emitted record, for callers that import the bench functions
QUIET = False     # True: collect only


def emit(**kw):
    RESULTS.append(kw)
    if not QUIET:
        print(json.dumps(kw), flush=True)


def bench_gemm(samples, shapes=None, outs=("bf16", "f32")):
    hbm, tf, kind = peaks()
    if shapes is None:
        shapes = [(n, n, n) for n in (1024, 2048, 4096, 8192)] + [(m, 4096, 4096) for m in (1, 8, 64)]
    g = torch.Generator(device="cuda").manual_seed(2)
    for m, n, k in shapes:
        for out_dtype, name in ((1, "bf16"), (0, "f32")):
            if name not in outs:
                continue
            osz = 2 if out_dtype else 4
            per_set = 2 * (m * k + n * k) + osz * m * n
            sets = copies_for(per_set)
            a = [(torch.rand((m, k), device="cuda", generator=g) * 2 - 1).to(torch.bfloat16) for _ in range(sets)]
            b = [(torch.rand((n, k), device="cuda", generator=g) * 2 - 1).to(torch.bfloat16) for _ in range(sets)]
            o = [torch.empty((m, n), device="cuda", dtype=torch.bfloat16 if out_dtype else torch.float32) for _ in range(sets)]

            ws = torch.zeros(lib().tnsr_b200_gemm_workspace(), dtype=torch.uint8, device="cuda") if m <= 64 else None

            def launch(i):
                if ws is None:
                    ok(lib().tnsr_b200_gemm_bf16(ptr(a[i]), ptr(b[i]), None, None, ptr(o[i]), m, n, k, -1, out_dtype, stream()))
                else:   # few rows: lend split-K scratch, as a decoder session does
                    ok(lib().tnsr_b200_gemm_bf16_ws(ptr(a[i]), ptr(b[i]), None, None, ptr(o[i]), m, n, k, -1, out_dtype,
                                                    ptr(ws), ws.numel(), stream()))

            ms, _ = timed_graph(launch, sets, samples) if m <= 64 else timed(launch, sets, samples)
            ref = (a[0].float() @ b[0].float().T)
            launch(0)
            torch.cuda.synchronize()
            err = float((o[0].float() - ref).abs().max() / ref.abs().max())
            flops, nbytes = 2.0 * m * n * k, float(per_set)
            skinny = m <= 64
            emit(op="gemm_bf16", m=m, n=n, k=k, out=name, ms=ms, tflops=flops / ms / 1e9, frac_tensor=flops / ms / 1e9 / tf,
                 gbs=nbytes / ms / 1e6, frac_hbm=nbytes / ms / 1e6 / hbm, bound="hbm" if skinny else "tensor",
                 rel_err_vs_torch=err, operand_sets=sets, peaks=kind)
            del a, b, o


def bench_serving_gemms(samples):
    """The four projection shapes of configuration 4 at prefill (131 072 rows) and decode (256 rows) size."""
    hbm, tf, kind = peaks()
    g = torch.Generator(device="cuda").manual_seed(5)
    for rows in (131072, 256):
        for name, n, k, out_dtype, resid in (("qkv", 2304, 768, 1, False), ("attn_out", 768, 768, 0, True),
                                             ("gate_up", 4096, 768, 1, False), ("ffn_down", 768, 2048, 0, True)):
            osz = 2 if out_dtype else 4
            per_set = 2 * (rows * k + n * k) + osz * rows * n * (2 if resid else 1)
            sets = copies_for(per_set) if rows <= 1024 else 1    # small operands would otherwise sit in L2 between launches
            a = [(torch.randn((rows, k), device="cuda", generator=g)).to(torch.bfloat16) for _ in range(sets)]
            b = [(torch.randn((n, k), device="cuda", generator=g) * 0.02).to(torch.bfloat16) for _ in range(sets)]
            r = [torch.randn((rows, n), device="cuda", generator=g) if resid else None for _ in range(sets)]
            o = [torch.empty((rows, n), device="cuda", dtype=torch.bfloat16 if out_dtype else torch.float32) for _ in range(sets)]

            def launch(i):
                ok(lib().tnsr_b200_gemm_bf16(ptr(a[i]), ptr(b[i]), None, ptr(r[i]), ptr(o[i]), rows, n, k, -1, out_dtype, stream()))

            # decode-size launches are a few microseconds: time them inside a graph, as the decoder runs them
            ms, _ = timed_graph(launch, sets, samples) if rows <= 1024 else timed(launch, 1, samples)
            flops = 2.0 * rows * n * k
            emit(op="serving_gemm", which=name, rows=rows, n=n, k=k, out="bf16" if out_dtype else "f32+residual", ms=ms,
                 tflops=flops / ms / 1e9, frac_tensor=flops / ms / 1e9 / tf, operand_sets=sets,
                 timing="graph of back-to-back launches over rotating operand sets" if rows <= 1024 else "one launch between events",
                 peaks=kind)
            del a, b, r, o


def bench_mlp(samples):
    hbm, tf, kind = peaks()
    rows, d, f = 4096, 2048, 5632
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((rows, d), device="cuda", generator=g).to(torch.bfloat16)
    wg = (torch.randn((d, f), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    wu = (torch.randn((d, f), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    wd = (torch.randn((f, d), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    packed = torch.empty((2 * f, d), device="cuda", dtype=torch.bfloat16)
    ok(lib().tnsr_b200_pack_gate_up(ptr(wg), ptr(wu), None, None, ptr(packed), None, d, f, stream()))
    wdt = torch.empty((d, f), device="cuda", dtype=torch.bfloat16)
    ok(lib().tnsr_b200_transpose_bf16(ptr(wd), ptr(wdt), f, d, stream()))
    hidden = torch.empty((rows, f), device="cuda", dtype=torch.bfloat16)
    out = torch.empty((rows, d), device="cuda", dtype=torch.bfloat16)

    def launch(_):
        ok(lib().tnsr_b200_swiglu_mlp(ptr(x), ptr(packed), None, ptr(wdt), None, ptr(hidden), ptr(out), rows, d, f, stream()))

    ms, _ = timed(launch, 1, samples)
    ref = (torch.nn.functional.silu(x.float() @ wg.float()) * (x.float() @ wu.float())).to(torch.bfloat16).float() @ wd.float()
    err = float((out.float() - ref).abs().max() / ref.abs().max())
    flops = 3 * 2.0 * rows * d * f
    emit(op="swiglu_mlp", rows=rows, d=d, f=f, ms=ms, tflops=flops / ms / 1e9, frac_tensor=flops / ms / 1e9 / tf,
         rel_err_vs_torch=err, note="two launches: gate/up GEMM with SwiGLU epilogue, down GEMM; operands (170 MB) exceed L2",
         peaks=kind)


def bench_attention(samples, serving=False):
    """Configuration 3 (ragged lengths), or with serving=True the decode attention of configuration 4:
    256 sessions x 12 heads x 64 at 641 live keys (the mean over the 256 benchmark steps)."""
    hbm, _, kind = peaks()
    if serving:
        batch, heads, hd, capacity = 256, 12, 64, 769
        lengths = np.full(batch, 641, dtype=np.uint32)
    else:
        batch, heads, hd, capacity = 64, 16, 64, 4096
        lengths = np.random.default_rng(4).integers(1, capacity + 1, size=batch).astype(np.uint32)
    d = heads * hd
    g = torch.Generator(device="cuda").manual_seed(4)
    q = torch.randn((batch, d), device="cuda", generator=g).to(torch.bfloat16)
    kc = torch.randn((batch, capacity, d), device="cuda", generator=g).to(torch.bfloat16)
    vc = torch.randn((batch, capacity, d), device="cuda", generator=g).to(torch.bfloat16)
    ln = torch.from_numpy(lengths.view(np.int32)).cuda()
    out = torch.empty((batch, d), device="cuda", dtype=torch.bfloat16)
    ws_bytes = lib().tnsr_b200_decode_attention_workspace(batch, capacity, heads, hd)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")

    def launch(_):
        ok(lib().tnsr_b200_decode_attention(ptr(q), ptr(kc), ptr(vc), ptr(ln), ptr(out), ptr(ws), ws_bytes, batch, capacity,
                                            heads, hd, stream()))

    # plan + scan are a few launches of ~100 us in total: time a graph of 8 calls so that the host side (three ctypes
    # calls per launch) does not count; the live K/V rows (>= 505 MB) exceed L2 by themselves
    ms, _ = timed_graph(launch, 1, samples, reps=8)
    nbytes = float(lengths.astype(np.int64).sum()) * 4 * d + batch * 4 * d
    emit(op="decode_attention", batch=batch, heads=heads, head_dim=hd, capacity=capacity, live_keys=int(lengths.sum()),
         ms=ms, gbs=nbytes / ms / 1e6, frac_hbm=nbytes / ms / 1e6 / hbm, algorithmic_bytes=nbytes,
         note="plan + scan kernels per call (status-word memset included); live K/V (%.0f MB) exceeds L2" % (nbytes / 1e6),
         peaks=kind)


def bench_prefill_attention(samples, sessions=64):
    """Prefill attention of configuration 4 (512 new queries at position 0, 12 heads x 64, capacity 768) on both
    engines: tcgen05 (engine 0) and warp-level mma.sync (engine 1).  Causal FLOPs: 4 * hd per (query, visible key)."""
    _, tf, kind = peaks()
    heads, hd, chunk, position, capacity = 12, 64, 512, 0, 768
    d = heads * hd
    g = torch.Generator(device="cuda").manual_seed(6)
    q = torch.randn((sessions, chunk, d), device="cuda", generator=g).to(torch.bfloat16)
    kc = torch.randn((sessions, capacity, d), device="cuda", generator=g).to(torch.bfloat16)
    vc = torch.randn((sessions, capacity, d), device="cuda", generator=g).to(torch.bfloat16)
    out = torch.empty((sessions, chunk, d), device="cuda", dtype=torch.bfloat16)
    pairs = sessions * heads * sum(position + t + 1 for t in range(chunk))
    flops = 4.0 * hd * pairs
    results = {}
    for engine, name in ((0, "tcgen05"), (1, "mma.sync")):
        ok(lib().tnsr_b200_set_gemm_engine(engine))
        try:
            ms, _ = timed(lambda _: ok(lib().tnsr_b200_prefill_attention(ptr(q), ptr(kc), ptr(vc), ptr(out), sessions, chunk,
                                                                         position, capacity, heads, hd, stream())), 1, samples)
        finally:
            lib().tnsr_b200_set_gemm_engine(0)
        results[name] = out.float().clone()
        emit(op="prefill_attention", engine=name, sessions=sessions, chunk=chunk, position=position, heads=heads, head_dim=hd,
             ms=ms, causal_tflops=flops / ms / 1e9, frac_tensor=flops / ms / 1e9 / tf, peaks=kind)
    emit(op="prefill_attention", max_abs_difference_between_engines=float((results["tcgen05"] - results["mma.sync"]).abs().max()))


def bench_elementwise(samples):
    hbm, _, kind = peaks()
    rows, d = 131072, 768
    x = torch.randn((rows, d), device="cuda")
    w, b = torch.ones(d, device="cuda"), torch.zeros(d, device="cuda")
    y = torch.empty((rows, d), device="cuda", dtype=torch.bfloat16)
    ms, _ = timed(lambda _: ok(lib().tnsr_b200_layernorm(ptr(x), ptr(w), ptr(b), ptr(y), rows, d, 1e-5, 1, 0, stream())), 1, samples)
    nbytes = rows * d * 6.0
    emit(op="layernorm_f32_to_bf16", rows=rows, width=d, ms=ms, gbs=nbytes / ms / 1e6, frac_hbm=nbytes / ms / 1e6 / hbm, peaks=kind)
    n = 4096 * 5632 * 8
    gate = torch.randn(n, device="cuda").to(torch.bfloat16)
    up = torch.randn(n, device="cuda").to(torch.bfloat16)
    o = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms, _ = timed(lambda _: ok(lib().tnsr_b200_swiglu(ptr(gate), ptr(up), ptr(o), n, stream())), 1, samples)
    emit(op="swiglu_elementwise", elems=n, ms=ms, gbs=6.0 * n / ms / 1e6, frac_hbm=6.0 * n / ms / 1e6 / hbm, peaks=kind)
    rows, vocab = 4096, 32000
    logits = torch.randn((rows, vocab), device="cuda")
    ids = torch.empty(rows, device="cuda", dtype=torch.int32)
    ms, _ = timed(lambda _: ok(lib().tnsr_b200_argmax(ptr(logits), ptr(ids), rows, vocab, stream())), 1, samples)
    nbytes = rows * vocab * 4.0
    emit(op="argmax", rows=rows, vocab=vocab, ms=ms, gbs=nbytes / ms / 1e6, frac_hbm=nbytes / ms / 1e6 / hbm, peaks=kind)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "skinny_gemm", "serving_gemms", "mlp", "attention", "serving_attention", "elementwise", "prefill_attention", "all"])
    ap.add_argument("--samples", type=int, default=20)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        sys.exit("opbench needs a CUDA device")
    todo = (["gemm", "serving_gemms", "mlp", "attention", "serving_attention", "elementwise", "prefill_attention"]
            if args.what == "all" else [args.what])
    for name in todo:
        {"gemm": bench_gemm, "skinny_gemm": lambda n: bench_gemm(n, shapes=[(m, 4096, 4096) for m in (1, 8, 64)], outs=("bf16",)),
         "serving_gemms": bench_serving_gemms, "mlp": bench_mlp, "attention": bench_attention,
         "serving_attention": lambda n: bench_attention(n, serving=True),
         "elementwise": bench_elementwise, "prefill_attention": bench_prefill_attention}[name](args.samples)


if __name__ == "__main__":
    main()
