"""CPU restatement of the library's next-token sampling rule (``tnsr_b200_sample_top_k``).

TEST INFRASTRUCTURE ONLY, like the rest of ``oracle/``.  The reference has no sampler (its decode loop is greedy,
src/nn/kv_cache.rs:121-157), so there is no reference vector to pin this to: *parity unpinned* against tnsr; what pins
it instead are (a) Philox4x32-10's published known-answer vectors (Salmon et al., "Parallel random numbers: as easy
as 1, 2, 3", SC'11; the same three vectors ship with Random123's kat_vectors), checked in tests/test_sampler_host.py,
and (b) the rule's own special case top_k = 1 == the reference's greedy pick ``max_by(total_cmp)``.

Rule (every arithmetic step is one rounded f32 operation unless stated):
  1. candidates = the top_k entries under (totalOrder key, index), largest first;
  2. in increasing index order: t = (l - l_max) / T;  w = f32(exp(f64(t)));  Z = ((w0 + w1) + ...);
  3. u = (x >> 8) * 2**-24, x = first word of Philox4x32-10(counter = (step, 0, session, 0), key = (seed lo, seed hi));
  4. pick = first candidate whose running sum exceeds u * Z, else the last candidate.
"""
import math

import numpy as np

M0, M1 = 0xD2511F53, 0xCD9E8D57
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = 0xFFFFFFFF


def philox4x32_10(counter, key):
    """Philox4x32 with ten rounds: counter and result are 4 words, key 2 words."""
    c = [int(x) & MASK for x in counter]
    k0, k1 = int(key[0]) & MASK, int(key[1]) & MASK
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k0) & MASK, p1 & MASK, ((p0 >> 32) ^ c[3] ^ k1) & MASK, p0 & MASK]
        k0, k1 = (k0 + W0) & MASK, (k1 + W1) & MASK
    return c


def uniform(seed, step, session):
    x = philox4x32_10((step, 0, session, 0), (seed & MASK, (seed >> 32) & MASK))[0]
    return np.float32(x >> 8) * np.float32(2.0 ** -24)


def total_order_keys(row):
    bits = np.ascontiguousarray(row, dtype=np.float32).view(np.int32).astype(np.int64)
    return bits ^ ((bits >> 31) & 0x7FFFFFFF)


def sample_row(row, temperature, top_k, seed, step, session):
    row = np.ascontiguousarray(row, dtype=np.float32)
    keys = total_order_keys(row)
    k = min(int(top_k), row.size)
    order = np.lexsort((np.arange(row.size), keys))[::-1][:k]      # by key, then index, largest first
    chosen = np.sort(order)
    best = row[order[0]]
    T = np.float32(temperature)
    weights, z = [], np.float32(0.0)
    for i in chosen:
        with np.errstate(invalid="ignore", over="ignore"):
            t = np.float32(np.float32(row[i] - best) / T)
        w = np.float32(math.exp(float(t))) if np.isfinite(t) else (np.float32(0.0) if t < 0 else np.float32(np.nan))
        weights.append(w)
        z = np.float32(z + w)
    target = np.float32(uniform(seed, step, session) * z)
    running = np.float32(0.0)
    for i, w in zip(chosen, weights):
        running = np.float32(running + w)
        if running > target:
            return int(i)
    return int(chosen[-1])


def sample(logits, temperature, top_k, seed, step, first_session=0):
    """ids[r] for logits [rows, vocab]; row r is session first_session + r; `step` is an int or one int per row."""
    logits = np.asarray(logits, dtype=np.float32)
    steps = np.broadcast_to(np.asarray(step, dtype=np.int64), (logits.shape[0],))
    return np.asarray([sample_row(logits[r], temperature, top_k, seed, int(steps[r]), first_session + r)
                       for r in range(logits.shape[0])], dtype=np.uint32)
