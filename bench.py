"""Benchmark of the cached-GPT decode hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K --warmup W   # CPU arm

Workload ("c4"): the serving configuration -- 12 layers, d_model 768, 12 heads x
64, SwiGLU 2048, vocab 32000, bf16 weights N(0, 0.02) seed 5; 256 independent
sessions, each a 512-token prefill of uniform random ids followed by greedy
decode steps.  Sessions are independent, so N GPUs hold disjoint shards and no
collective runs on the data path.  With the default `--scaling strong` the
configuration's 256 sessions are divided 256/N per GPU, as the configuration
words it (`weak_scaling` in the same line is the side measurement with all 256
sessions on every GPU; `--scaling weak` makes that the headline instead).  A
benchmark "step" is one decode step: one new token for every session of the
rank.  The timed region is K steps starting at position 512 (the default K =
256 is the configuration's decode length) with token ids living on the device,
timed with CUDA events on the session's stream; it is repeated `--repeats`
times from the same state, each repeat taken as the max over ranks, and
`value` is total tokens/s at the median repeat (all samples are in `timing`).
`e2e` repeats the K steps through the host API (`tnsr_b200_decoder_decode`):
ids go up from host memory and greedy ids come back every step.  At N = 1 the
line also carries `ops`: GEMM TFLOP/s, SwiGLU-MLP TFLOP/s and KV-attention GB/s
of the operator configurations.

`--workload c0|c1|c2|c3` measures the smaller configurations on one GPU (the f32
4-layer model end to end, the GEMM sweep, the SwiGLU MLP, ragged decode attention),
each with the CPU restatement timed beside it on a stated sample.

The CPU arm times this repository's restatement of the reference's CPU executor
(oracle/) on the host cores: the reference is Rust and cannot be built here.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOTAL_SESSIONS = 256
PREFILL = 512
DECODE_STEPS = 256
FALLBACK_HBM_GBS = 6650.0

# Per-launch DRAM traffic of decode_attention_kernel relative to its algorithmic
# bytes, from one ncu capture of the kernel at 256 sessions x 641 live keys (the mean
# length of the timed steps): dram__bytes_read.sum + dram__bytes_write.sum = 509.48 MB
# for 504.89 MB of live K/V rows and q/out.  Traffic grows in proportion to the live
# keys, so the ratio is applied to every step.
NCU_TRAFFIC_RATIO = 1.009


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=DECODE_STEPS)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--sessions", type=int, default=TOTAL_SESSIONS,
                    help="sessions in total (strong scaling) or per GPU (weak scaling)")
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="strong (the configuration's wording): --sessions are divided over the GPUs, 256/N each; "
                         "weak: every GPU holds --sessions sessions")
    ap.add_argument("--repeats", type=int, default=10, help="timed passes of K steps; value is their median")
    ap.add_argument("--no-weak", action="store_true", help="N > 1, strong scaling: skip the weak-scaling side measurement")
    ap.add_argument("--no-ops", action="store_true", help="N = 1: skip the operator configurations (c1-c3 headline values)")
    ap.add_argument("--prefill", type=int, default=PREFILL)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--workload", default="c4", choices=["c4", "c0", "c1", "c2", "c3"],
                    help="c4 (default): the serving decode benchmark; c0: the 4-layer d128 f32 model, 16-token prompt + 64 "
                         "greedy steps; c1: GEMM sweep; c2: SwiGLU MLP; c3: ragged decode attention -- each with the CPU "
                         "restatement timed beside it (1 GPU)")
    ap.add_argument("--samples", type=int, default=20, help="timed launches per case of the operator workloads")
    ap.add_argument("--step-parts", type=int, default=0, help="session configuration: parts a single-token step is divided into (0 = automatic)")
    ap.add_argument("--small-batch-mode", type=int, default=0, help="session configuration: 1 = operator-by-operator step also at <= 64 sessions")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def serving_config(args):
    from tnsr_b200.nn import GptConfig
    return GptConfig(vocab_size=args.vocab, max_sequence_length=2048, embed_dim=768, num_heads=12,
                     feed_forward_dim=2048, num_layers=args.layers, layer_norm_epsilon=1e-5,
                     activation="swiglu", weight_dtype="bf16")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            data = json.load(f)
        return float(data["hbm_gbs"]), "measured", data
    return FALLBACK_HBM_GBS, "fallback", {}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# CPU arm: the checker's decode step on the host cores
# ---------------------------------------------------------------------------
def cpu_decode_rate(args, steps, warmup, threads=None, budget_s=None):
    """tokens/s of the CPU restatement on `threads` host threads (one session per
    thread per step, all advancing together as the reference's batch does).
    The sessions start at position `prefill` on zeroed K/V rows: the arithmetic
    cost of a decode step does not depend on the cached values."""
    from oracle import oracle
    from tnsr_b200.synthetic import normal_model_arrays
    cfg = serving_config(args)
    threads = threads or oracle.max_threads()
    oracle.set_threads(threads)
    sessions = threads
    arrays = normal_model_arrays(cfg, seed=5, std=0.02)
    model = oracle.OracleModel(cfg.vocab_size, cfg.max_sequence_length, cfg.embed_dim, cfg.num_heads,
                               cfg.feed_forward_dim, cfg.num_layers, cfg.layer_norm_epsilon, "swiglu")
    model.set_params(arrays)
    del arrays
    capacity = min(cfg.max_sequence_length, args.prefill + steps + warmup + 1)
    dec = oracle.lib().oracle_decoder_create(model.handle, sessions, capacity)
    oracle.lib().oracle_decoder_set_len(dec, args.prefill)
    rng = np.random.default_rng(7)
    ids = rng.integers(0, cfg.vocab_size, size=sessions).astype(np.uint32)
    logits = np.empty((sessions, cfg.vocab_size), dtype=np.float32)
    pl = logits.ctypes.data_as(C.POINTER(C.c_float))

    def one_step():
        nonlocal ids
        rc = oracle.lib().oracle_decoder_decode(dec, ids.ctypes.data_as(C.POINTER(C.c_uint32)), 1, pl)
        assert rc == 0, rc
        ids = np.asarray([oracle.argmax_last(logits[s]) for s in range(sessions)], dtype=np.uint32)

    for _ in range(warmup):
        one_step()
    done = 0
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    elapsed = time.perf_counter() - t0
    oracle.lib().oracle_decoder_destroy(dec)
    oracle.set_threads(1)
    return {"tokens_per_s": sessions * done / elapsed, "threads": threads, "sessions": sessions, "steps": done,
            "elapsed_s": elapsed, "ms_per_step": elapsed / done * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = cpu_decode_rate(args, args.steps, args.warmup)
    sample = (f"{r['sessions']} sessions (one per host thread) x {r['steps']} decode steps from position {args.prefill}; "
              "CPU restatement of tnsr's SimpleExecutor path (oracle/), f32")
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": r["tokens_per_s"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": r["steps"], "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, args.gpus),
        "cpu_baseline": {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["threads"], "kind": "port",
                         "sample": sample},
        "e2e": {"value": r["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def sessions_per_gpu(args, n_gpus):
    """Per-rank session counts: the whole batch everywhere (weak) or contiguous shards of it (strong)."""
    from tnsr_b200.sharding import shard_sessions
    if args.scaling == "weak":
        return [args.sessions] * n_gpus
    return [shard_sessions(args.sessions, n_gpus, r)[1] for r in range(n_gpus)]


def workload_config(args, n_gpus):
    shards = sessions_per_gpu(args, n_gpus)
    per_gpu = shards[0] if len(set(shards)) == 1 else shards
    return {
        "workload": "c4: GPT 12x768 (12 heads x 64, SwiGLU 2048, vocab 32000, ctx 2048), "
                    f"{sum(shards)} sessions ({per_gpu} per GPU) x ({args.prefill}-token prefill + greedy decode), "
                    "1 token/session/step",
        "sessions_total": sum(shards), "sessions_per_gpu": per_gpu, "prefill": args.prefill,
        "layers": args.layers, "vocab": args.vocab,
        "parallelism": f"independent sessions on {n_gpus} GPU(s), {args.scaling} scaling, no collective",
        "l2": "inputs larger than L2: each step streams the live K/V rows (GBs) and 222 MB of weights",
    }


# ---------------------------------------------------------------------------
# the smaller configurations: this library on one GPU, the CPU restatement beside it
# ---------------------------------------------------------------------------
def _timed_cpu(fn, repeats=1):
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
    return best


def _op_line(args, metric, unit, value, ms, dtype, workload, roofline, cpu_baseline, cases, launches, clocks):
    return {"metric": metric, "value": value, "unit": unit, "n_gpus": 1, "steps": args.samples, "warmup": 3,
            "ms_per_step": ms, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": dtype,
            "data": "synthetic", "config": {"workload": workload, "l2": "operands rotate through copies larger than L2 "
                                            "or exceed it by themselves"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": None, "gpu_launches": launches, "clocks": clocks,
            "cases": cases}


def run_ops(args):
    """Configurations 0-3 on one GPU.  The GPU side is tnsr_b200.opbench (operator calls through the C ABI, CUDA events)
    or, for c0, the session API; the CPU side is the restatement in oracle/ on a stated sample."""
    import torch
    from tnsr_b200 import _native, opbench
    from oracle import oracle
    torch.cuda.set_device(0)
    opbench.QUIET = True
    hbm, tf, kind = opbench.peaks()
    lib = _native.lib()
    threads = oracle.max_threads()
    oracle.set_threads(threads)
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = lib.tnsr_b200_kernel_launches()
    rng = np.random.default_rng(2)
    if args.workload == "c0":
        from oracle.oracle import OracleBackend
        from tnsr_b200.nn import GptDecoder
        from tnsr_b200.synthetic import config0_model, config0_prompt, set_model_arrays
        from tnsr_b200 import Backend, Gpt
        from tnsr_b200.nn import argmax_last
        cfg, arrays = config0_model("relu")
        model = Gpt(cfg)
        set_model_arrays(model, arrays)
        prompt = [int(t) for t in config0_prompt()]

        def greedy(decoder):
            """reset, 16-token prefill, 64 cached greedy steps: (ids, prefill seconds, decode seconds)"""
            decoder.reset()
            t0 = time.perf_counter()
            logits = decoder.decode(prompt)
            t1 = time.perf_counter()
            ids = []
            for _ in range(64):
                ids.append(argmax_last(logits[logits.size - cfg.vocab_size:]))
                logits = decoder.decode([ids[-1]])
            return ids, t1 - t0, time.perf_counter() - t1

        gpu_dec = model.decoder(Backend.Cuda, 1)
        greedy(gpu_dec)                                           # first use: allocations, graph capture
        runs = [greedy(gpu_dec) for _ in range(max(5, args.samples // 2))]
        got = runs[-1][0]
        gpu_prefill_s, gpu_s = float(np.median([r[1] for r in runs])), float(np.median([r[2] for r in runs]))
        cpu_dec = GptDecoder(model, None, 1, cfg.max_sequence_length,
                             backend_impl=OracleBackend(cfg, 1, cfg.max_sequence_length, attention_bf16=False))
        greedy(cpu_dec)
        cpu_runs = [greedy(cpu_dec) for _ in range(3)]
        want = cpu_runs[-1][0]
        cpu_prefill_s, cpu_s = float(np.median([r[1] for r in cpu_runs])), float(np.median([r[2] for r in cpu_runs]))
        same = want == got
        weight_bytes = 4.0 * sum(int(np.asarray(a).size) for a in arrays)
        value = 64 / gpu_s
        roof = {"bound": "hbm", "achieved": weight_bytes * 64 / gpu_s / 1e9, "peak": hbm, "unit": "GB/s",
                "frac": weight_bytes * 64 / gpu_s / 1e9 / hbm, "traffic": None,
                "note": "latency-bound: 3.3 MB of f32 weights per step, kernels that keep the reference's operation order, "
                        "one host round trip per token (logits returned every step as the reference's decode does)"}
        cpu = {"value": 64 / cpu_s, "unit": "tokens/s", "cores": 1, "kind": "port",
               "sample": "the whole configuration: 16-token prefill (%.2f ms) + 64 cached greedy steps, batch 1, one thread, "
                         "same GptDecoder wrapper over the CPU restatement" % (cpu_prefill_s * 1e3)}
        line = _op_line(args, "decode_tokens_per_s", "tokens/s", value, gpu_s * 1e3 / 64, "f32",
                        "c0: GPT 4x128 (4 heads x 32, ReLU FFN 512, vocab 96, ctx 128), f32, batch 1, 16-token prompt then 64 cached "
                        "greedy steps through GptDecoder.decode (steps timed; prefill reported in cases)", roof, cpu,
                        [{"greedy_ids_equal_to_cpu": same, "us_per_token_gpu": gpu_s * 1e6 / 64, "us_per_token_cpu": cpu_s * 1e6 / 64,
                          "prefill_ms_gpu": gpu_prefill_s * 1e3, "prefill_ms_cpu": cpu_prefill_s * 1e3}],
                        0, None)
        line["e2e"] = {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4 * cfg.vocab_size}
    elif args.workload == "c1":
        opbench.bench_gemm(args.samples)
        cases = list(opbench.RESULTS)
        top = max((c for c in cases if c["m"] == 8192 and c["out"] == "bf16"), key=lambda c: c["tflops"])
        a = (rng.random((1024, 1024), dtype=np.float32) * 2 - 1)
        b = (rng.random((1024, 1024), dtype=np.float32) * 2 - 1)
        cpu_s = _timed_cpu(lambda: oracle.matmul_bf16(a, b))
        w = (rng.random((4096, 4096), dtype=np.float32) * 2 - 1)
        skinny = {}
        for m in (1, 8, 64):
            x = (rng.random((m, 4096), dtype=np.float32) * 2 - 1)
            skinny[m] = _timed_cpu(lambda: oracle.matmul_bf16(x, w))
        roof = {"bound": "tensor", "achieved": top["tflops"], "peak": tf, "unit": "TFLOP/s", "frac": top["tflops"] / tf,
                "traffic": None, "kernel": "gemm_tc_kernel<256,0>, 8192^3, bf16 out"}
        cpu = {"value": 2.0 * 1024 ** 3 / cpu_s / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": "1024^3 in %.2f s; skinny M=1/8/64 x 4096 x 4096 in %.3f / %.3f / %.3f s (reference operation order, "
                         "bf16-rounded operands, f32 accumulation); 8192^3 would take about %.0f s" %
                         (cpu_s, skinny[1], skinny[8], skinny[64], cpu_s * 512)}
        line = _op_line(args, "gemm_tflops", "TFLOP/s", top["tflops"], top["ms"], "bf16",
                        "c1: bf16 GEMM sweep M=N=K in {1024,2048,4096,8192} + skinny M in {1,8,64} x 4096 x 4096, bf16 and f32 out; "
                        "value = 8192^3 with bf16 output", roof, cpu, cases, 0, None)
    elif args.workload == "c2":
        opbench.bench_mlp(args.samples)
        r = opbench.RESULTS[-1]
        rows, d, f = 16, 2048, 5632
        x = rng.standard_normal((rows, d)).astype(np.float32)
        wg = (rng.standard_normal((d, f)) * 0.02).astype(np.float32)
        wu = (rng.standard_normal((d, f)) * 0.02).astype(np.float32)
        wd = (rng.standard_normal((f, d)) * 0.02).astype(np.float32)
        zf, zd = np.zeros(f, np.float32), np.zeros(d, np.float32)
        cpu_s = _timed_cpu(lambda: oracle.swiglu_mlp(x, wg, zf, wu, zf, wd, zd))
        roof = {"bound": "tensor", "achieved": r["tflops"], "peak": tf, "unit": "TFLOP/s", "frac": r["tflops"] / tf,
                "traffic": None, "kernel": "gemm_tc_kernel (gate/up + SwiGLU epilogue, then down)"}
        cpu = {"value": 3 * 2.0 * rows * d * f / cpu_s / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": "%d of the 4096 rows in %.2f s (f32, reference operation order); the whole block would take about %.0f s"
                         % (rows, cpu_s, cpu_s * 4096 / rows)}
        line = _op_line(args, "swiglu_mlp_tflops", "TFLOP/s", r["tflops"], r["ms"], "bf16",
                        "c2: fused SwiGLU MLP, x [4096, 2048] -> 5632 -> 2048, bf16", roof, cpu, [r], 0, None)
    else:
        opbench.bench_attention(args.samples)
        r = opbench.RESULTS[-1]
        batch, heads, hd, capacity = 16, 16, 64, 4096
        d = heads * hd
        lengths = np.random.default_rng(4).integers(1, capacity + 1, size=64).astype(np.uint32)[:batch]
        q = oracle.bf16_round_np(rng.standard_normal((batch, d)).astype(np.float32))
        kc = oracle.bf16_round_np(rng.standard_normal((batch, capacity, d)).astype(np.float32))
        vc = oracle.bf16_round_np(rng.standard_normal((batch, capacity, d)).astype(np.float32))
        cpu_s = _timed_cpu(lambda: oracle.decode_attention(q, kc, vc, lengths, heads))
        cpu_bytes = float(lengths.astype(np.int64).sum()) * 4 * d
        roof = {"bound": "hbm", "achieved": r["gbs"], "peak": hbm, "unit": "GB/s", "frac": r["gbs"] / hbm,
                "traffic": r["algorithmic_bytes"] * NCU_TRAFFIC_RATIO, "kernel": "da_plan_kernel + decode_attention_kernel<64,1> per call"}
        cpu = {"value": cpu_bytes / cpu_s / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": "the first 16 of the 64 sessions (%.0f MB of bf16 K/V, counted as on the GPU) in %.3f s" % (cpu_bytes / 1e6, cpu_s)}
        line = _op_line(args, "kv_attention_gbs", "GB/s", r["gbs"], r["ms"], "bf16",
                        "c3: decode attention, 64 sessions x 16 heads x 64, bf16 cache of capacity 4096, live lengths uniform [1, 4096] "
                        "(seed 4)", roof, cpu, [r], 0, None)
    line["gpu_launches"] = int(lib.tnsr_b200_kernel_launches() - launches0)
    line["clocks"] = sampler.stop()
    line["roofline"]["peak_source"] = kind
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# this library
# ---------------------------------------------------------------------------
def _percentile(xs, q):
    return float(np.percentile(np.asarray(xs, dtype=np.float64), q))


def measure_decode(args, cfg, sessions, rank, local_rank, world, barrier, reduce_max, full):
    """Prefill `sessions` sessions on this rank, then time K greedy steps from position `prefill`, `--repeats` times
    (every repeat starts over from the same position and ids).  Returns the per-repeat milliseconds (max over ranks)
    and, when `full`, the attention-kernel profile and the end-to-end loop as well."""
    import torch
    from tnsr_b200 import _native
    from tnsr_b200.session import B200Session
    from tnsr_b200.synthetic import normal_model_arrays

    K, W = args.steps, args.warmup
    capacity = min(cfg.max_sequence_length, args.prefill + max(K, W) + 1)
    # positions of the decode steps: prefill, prefill + 1, ...; a run longer than the context allows starts over at
    # `prefill` (the cache rows are overwritten), so any K can be timed
    span = capacity - args.prefill
    if span < 1:
        raise SystemExit("--prefill leaves no room for decode steps in the model context")

    def position_of(step):
        return args.prefill + step % span
    lib = _native.lib()
    arrays = normal_model_arrays(cfg, seed=5, std=0.02)
    sess = B200Session(cfg, sessions, capacity, device=local_rank, logits_mode="none", step_parts=args.step_parts,
                       small_batch_mode=args.small_batch_mode)
    for i, a in enumerate(arrays):
        sess.refresh(i, a)
    del arrays
    stream = torch.cuda.ExternalStream(sess.stream(), device=torch.device("cuda", local_rank))
    rng = np.random.default_rng(1000 + rank)
    prompt = rng.integers(0, cfg.vocab_size, size=(sessions, args.prefill)).astype(np.uint32)

    # ---- prefill (untimed for the metric; reported on the side) ----
    def prefill():
        sess.reset()
        d_prompt = torch.from_numpy(prompt.view(np.int32)).cuda()
        first = torch.empty(sessions, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        sess.decode_device(d_prompt.data_ptr(), args.prefill, 0, first.data_ptr())
        e1.record(stream)
        sess.synchronize()
        return first, e0.elapsed_time(e1)

    first, _ = prefill()              # warm-up pass (allocations, first-use costs)
    first, prefill_ms = prefill()
    first_host = first.cpu().numpy().astype(np.uint32)

    def fresh_ids():
        cur = first.clone()
        torch.cuda.synchronize()  # the copy ran on torch's stream; the session has its own
        return cur

    def device_loop(n, cur):
        """n greedy steps from position `prefill`; ids stay in `cur` on the device."""
        for step in range(n):
            sess.decode_device(cur.data_ptr(), 1, position_of(step), cur.data_ptr())
        return cur

    def timed_pass():
        cur = fresh_ids()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        last = device_loop(K, cur)
        e1.record(stream)
        sess.synchronize()
        return e0.elapsed_time(e1), last

    # ---- warm-up: W steps, then whole untimed passes until two in a row agree to 2 % (clocks, caches, graph) ----
    device_loop(W, fresh_ids())
    sess.synchronize()
    warm_passes, prev = 0, None
    t_warm = time.perf_counter()
    while warm_passes < 12 and time.perf_counter() - t_warm < 5.0:
        ms, _ = timed_pass()
        warm_passes += 1
        if prev is not None and abs(ms - prev) <= 0.02 * prev:
            break
        prev = ms

    # ---- the timed region: `repeats` passes of exactly K steps, each between barriers ----
    sampler = ClockSampler(local_rank)
    sampler.start()
    samples, launches = [], 0
    last = None
    for _ in range(args.repeats):
        barrier()
        launches0 = lib.tnsr_b200_kernel_launches()
        ms, last = timed_pass()
        launches = lib.tnsr_b200_kernel_launches() - launches0
        barrier()
        samples.append(ms)
    clocks = sampler.stop()
    samples = [reduce_max(x) for x in samples]
    tokens_after_timed = last.cpu().numpy().astype(np.uint32)
    out = {"sessions": sessions, "samples_ms": samples, "prefill_ms": reduce_max(prefill_ms), "launches": int(launches),
           "clocks": clocks, "warm_passes": warm_passes, "position_of": position_of}
    if not full:
        sess.close()
        return out

    # ---- instrumented replay of the same K steps: device time of the attention kernel ----
    sess.profile_attention(True)
    sess.attention_profile()
    device_loop(K, fresh_ids())
    out["attn_ms"], out["attn_launches"] = sess.attention_profile()
    sess.profile_attention(False)

    # ---- end to end through the host API ----
    if not args.no_e2e:
        cur = first_host.copy()
        for step in range(min(W, K)):
            _, cur = sess.decode_full(cur.reshape(sessions, 1), position_of(step))
        e2e_samples = []
        for _ in range(max(1, min(3, args.repeats))):
            cur = first_host.copy()
            barrier()
            t0 = time.perf_counter()
            for step in range(K):
                _, cur = sess.decode_full(cur.reshape(sessions, 1), position_of(step))
            torch.cuda.synchronize()
            e2e_samples.append(time.perf_counter() - t0)
            barrier()
        out["e2e_samples_s"] = [reduce_max(x) for x in e2e_samples]
        out["e2e_same_tokens"] = bool(np.array_equal(cur, tokens_after_timed))
    sess.close()
    return out


def operator_summary(samples):
    """Headline values of the operator configurations (GEMM TFLOP/s, SwiGLU MLP TFLOP/s, KV-attention GB/s), measured
    through the C ABI by tnsr_b200.opbench on the current device."""
    from tnsr_b200 import opbench
    opbench.QUIET = True
    del opbench.RESULTS[:]
    opbench.bench_gemm(samples, shapes=[(8192, 8192, 8192), (1, 4096, 4096), (8, 4096, 4096), (64, 4096, 4096)],
                       outs=("bf16",))
    opbench.bench_mlp(samples)
    opbench.bench_attention(samples)
    ops = {}
    for r in opbench.RESULTS:
        if r["op"] == "gemm_bf16":
            key = "c1_gemm_%dx%dx%d" % (r["m"], r["n"], r["k"])
            if r["bound"] == "tensor":
                ops[key] = {"tflops": r["tflops"], "frac_tensor": r["frac_tensor"], "ms": r["ms"]}
            else:
                ops[key] = {"us": r["ms"] * 1e3, "gbs": r["gbs"], "frac_hbm": r["frac_hbm"]}
        elif r["op"] == "swiglu_mlp":
            ops["c2_swiglu_mlp_4096x2048x5632"] = {"tflops": r["tflops"], "frac_tensor": r["frac_tensor"], "ms": r["ms"]}
        elif r["op"] == "decode_attention":
            ops["c3_decode_attention_64x16x64_ragged"] = {"gbs": r["gbs"], "frac_hbm": r["frac_hbm"], "ms": r["ms"]}
    ops["peaks"] = opbench.RESULTS[-1]["peaks"] if opbench.RESULTS else None
    return ops


def run_b200(args):
    import torch
    import torch.distributed as dist
    from tnsr_b200.sharding import shard_sessions

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(x):
        if world == 1:
            return float(x)
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_sum(x):
        if world == 1:
            return float(x)
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    cfg = serving_config(args)
    K, W = args.steps, args.warmup
    if args.scaling == "strong":
        _, sessions = shard_sessions(args.sessions, world, rank)   # contiguous blocks, sizes differ by at most one
        if sessions == 0:
            raise SystemExit("more GPUs than sessions")
    else:
        sessions = args.sessions
    main = measure_decode(args, cfg, sessions, rank, local_rank, world, barrier, reduce_max, full=True)
    total_sessions = int(reduce_sum(sessions))
    total_launches = int(reduce_sum(main["launches"]))
    weak = None
    if world > 1 and args.scaling == "strong" and not args.no_weak:
        # the same job with the configuration's whole batch on every GPU: the per-GPU step of the 1-GPU run
        weak = measure_decode(args, cfg, args.sessions, rank, local_rank, world, barrier, reduce_max, full=False)

    if rank == 0:
        d, layers, f = cfg.embed_dim, cfg.num_layers, cfg.feed_forward_dim
        peak, peak_kind, peaks = measured_peaks()
        position_of = main["position_of"]
        elapsed_ms = float(np.median(main["samples_ms"]))
        # algorithmic bytes of one attention launch at decode step t: every session's live K and V rows
        # (prefill + t + 1 keys x d x 2 B x 2 tensors) plus q and out rows
        live = float(np.mean([position_of(t) + 1 for t in range(K)]))     # keys a step at position p attends: p + 1
        bytes_per_launch = sessions * (live * d * 2 * 2 + 2 * d * 2)
        attn_ms, attn_launches = main["attn_ms"], main["attn_launches"]
        attn_avg_ms = attn_ms / max(attn_launches, 1)
        achieved = bytes_per_launch / (attn_avg_ms * 1e-3) / 1e9 if attn_launches else None
        peak_source = f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6650 GB/s"
        roofline = {
            "kernel": "decode_attention_kernel<64,1> (split-KV live-prefix scan)", "bound": "hbm",
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak if achieved else None,
            "peak_source": peak_source,
            "traffic": bytes_per_launch * NCU_TRAFFIC_RATIO if NCU_TRAFFIC_RATIO else None,
            "algorithmic_bytes_per_launch": bytes_per_launch, "avg_launch_ms": attn_avg_ms, "launches": attn_launches,
            "share_of_step": attn_ms / elapsed_ms if attn_launches else None,
            "how": "CUDA events around every launch of the kernel on the session's stream, in a replay of the same K steps",
        }
        # the whole step against the same roofline: live K/V of every layer plus every weight matrix once
        weight_bytes = 2.0 * (layers * (4 * d * d + 3 * d * f) + d * cfg.vocab_size)
        step_bytes = layers * bytes_per_launch + weight_bytes
        step_gbs = step_bytes / (elapsed_ms / K * 1e-3) / 1e9
        roofline_step = {"bound": "hbm", "achieved": step_gbs, "peak": peak, "unit": "GB/s", "frac": step_gbs / peak,
                         "peak_source": peak_source, "algorithmic_bytes_per_step": step_bytes,
                         "what": "rank 0's step: live K/V rows of all layers + every bf16 weight matrix once, over ms_per_step"}
        value = total_sessions * K / (elapsed_ms * 1e-3)
        flops_per_token = 2.0 * (layers * (4 * d * d + 3 * d * f)) + 2.0 * d * cfg.vocab_size
        prefill_tokens = total_sessions * args.prefill
        prefill_ms = main["prefill_ms"]
        line = {
            "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": elapsed_ms / K, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(args, world),
            "timing": {"repeats": len(main["samples_ms"]), "value_is": "median over repeats of K steps (max over ranks per repeat)",
                       "samples_ms_per_step": [x / K for x in main["samples_ms"]],
                       "p10_ms_per_step": _percentile(main["samples_ms"], 10) / K,
                       "p90_ms_per_step": _percentile(main["samples_ms"], 90) / K,
                       "untimed_warm_passes": main["warm_passes"]},
            "roofline": roofline, "roofline_step": roofline_step,
            "gpu_launches": total_launches,
            "clocks": main["clocks"],
            "prefill": {"tokens_per_s": prefill_tokens / (prefill_ms * 1e-3), "ms": prefill_ms,
                        "gemm_tflops": sessions * args.prefill * (flops_per_token - 2.0 * d * cfg.vocab_size) / (prefill_ms * 1e-3) / 1e12,
                        "note": "whole prefill step incl. attention and LayerNorm; rank 0's GEMM flops / max-over-ranks time"},
        }
        if "e2e_samples_s" in main:
            e2e_s = float(np.median(main["e2e_samples_s"]))
            line["e2e"] = {"value": total_sessions * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 4 * sessions,
                           "d2h_bytes_per_step": 4 * sessions + 4, "ms_per_step": e2e_s / K * 1e3,
                           "samples_ms_per_step": [x / K * 1e3 for x in main["e2e_samples_s"]],
                           "api": "tnsr_b200_decoder_decode, logits_mode NONE: ids up, greedy ids down, every step",
                           "same_tokens_as_device_loop": main["e2e_same_tokens"]}
        if weak:
            wms = float(np.median(weak["samples_ms"]))
            line["weak_scaling"] = {"sessions_per_gpu": args.sessions, "value": args.sessions * world * K / (wms * 1e-3),
                                    "unit": "tokens/s", "ms_per_step": wms / K,
                                    "note": "side measurement: the configuration's whole batch on every GPU"}
        if world == 1 and not args.no_ops:
            line["ops"] = operator_summary(args.samples)
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_decode_rate(args, steps=64, warmup=1, budget_s=20.0)
            line["cpu_baseline"] = {
                "value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["threads"], "kind": "port",
                "sample": f"{r['sessions']} sessions x {r['steps']} decode steps from position {args.prefill} "
                          f"({r['elapsed_s']:.1f} s); CPU restatement of tnsr's SimpleExecutor (oracle/), f32",
            }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload != "c4":
        if int(os.environ.get("RANK", "0")) == 0:
            run_ops(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
