// Device-side sampling of the next token from a row of logits: temperature and top-k, one seeded
// counter-based random number per (session, position).
//
// No reference counterpart: tnsr's decoder loop is greedy only (src/nn/kv_cache.rs:121-157).  The rule is chosen so
// that it contains the reference's pick as a special case -- candidates are ordered like `max_by(total_cmp)`, ties
// towards the larger index, so top_k = 1 returns exactly the greedy id -- and so that a CPU restatement can follow
// it bit for bit:
//   1. candidates = the top_k entries of the row under (IEEE totalOrder key, index), largest first;
//   2. walk them in increasing index order: t_j = (l_j - l_max) / T in f32, w_j = (float)exp((double)t_j),
//      Z = ((w_0 + w_1) + ...) in f32;
//   3. u = (x >> 8) * 2^-24 with x the first word of Philox4x32-10 on counter (step, 0, session, 0) and key
//      (seed low, seed high), where step is the position the new token will take; target = u * Z;
//   4. the pick is the first candidate (index order) whose running sum exceeds the target, else the last one.
// Selection is a radix select over the sign-folded keys (four 8-bit passes over the row, which stays in L2),
// followed by an order-preserving compaction; the arithmetic of steps 2-4 runs over at most 256 candidates.
#include "common.cuh"

namespace tb {

constexpr uint32_t SAMPLE_MAX_K = 256;
constexpr uint32_t SAMPLE_THREADS = 256;

__device__ __forceinline__ uint32_t ordered_key(float x) { return (uint32_t)total_order_key(x) ^ 0x80000000u; }

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
}
// First output word of Philox4x32 with ten rounds.
__device__ __forceinline__ uint32_t philox_first(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
    uint32_t c[4] = {c0, c1, c2, c3};
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return c[0];
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_top_k_kernel(const float* __restrict__ logits, uint32_t vocab, uint32_t row_stride, float temperature, uint32_t top_k,
                    uint32_t seed_lo, uint32_t seed_hi, const uint32_t* __restrict__ d_step, uint32_t step_stride,
                    uint32_t step_add, uint32_t first_session, uint32_t* __restrict__ out) {
    __shared__ uint32_t hist[256];
    __shared__ uint32_t s_prefix, s_remaining, s_eq_total;
    __shared__ uint32_t warp_take[SAMPLE_THREADS / 32], warp_eq[SAMPLE_THREADS / 32];
    __shared__ uint32_t s_take_base, s_eq_base;
    __shared__ uint32_t cand_idx[SAMPLE_MAX_K];
    __shared__ float cand_val[SAMPLE_MAX_K];
    pdl_wait();
    pdl_trigger();
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = logits + (size_t)blockIdx.x * row_stride;
    const uint32_t k = top_k < vocab ? top_k : vocab;

    // ---- the k-th largest key: four 8-bit radix passes from the top byte ----
    if (tid == 0) { s_prefix = 0; s_remaining = k; }
    uint32_t mask = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        for (uint32_t i = tid; i < vocab; i += SAMPLE_THREADS) {
            const uint32_t uk = ordered_key(__ldg(row + i));
            if ((uk & mask) == prefix) atomicAdd(&hist[(uk >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t remaining = s_remaining, above = 0;
            int b = 255;
            for (; b > 0; --b) {
                if (above + hist[b] >= remaining) break;
                above += hist[b];
            }
            s_remaining = remaining - above;        // how many to take from bin b
            s_prefix = prefix | ((uint32_t)b << shift);
            s_eq_total = hist[b];
        }
        mask |= 255u << shift;
        __syncthreads();
    }
    const uint32_t threshold = s_prefix;                        // key of the k-th largest entry
    const uint32_t skip_eq = s_eq_total - s_remaining;          // ties go to the larger index: skip the first ones

    // ---- candidates in increasing index order ----
    if (tid == 0) { s_take_base = 0; s_eq_base = 0; }
    __syncthreads();
    for (uint32_t base = 0; base < vocab; base += SAMPLE_THREADS) {
        const uint32_t i = base + tid;
        float v = 0.0f;
        uint32_t uk = 0;
        const bool in = i < vocab;
        if (in) { v = __ldg(row + i); uk = ordered_key(v); }
        const bool eq = in && uk == threshold;
        const uint32_t eq_ballot = __ballot_sync(0xffffffffu, eq);
        if (lane == 0) warp_eq[warp] = __popc(eq_ballot);
        __syncthreads();
        uint32_t eq_before = s_eq_base + __popc(eq_ballot & ((1u << lane) - 1u));
        for (uint32_t w = 0; w < warp; ++w) eq_before += warp_eq[w];
        const bool take = in && (uk > threshold || (eq && eq_before >= skip_eq));
        const uint32_t take_ballot = __ballot_sync(0xffffffffu, take);
        if (lane == 0) warp_take[warp] = __popc(take_ballot);
        __syncthreads();
        uint32_t pos = s_take_base + __popc(take_ballot & ((1u << lane) - 1u));
        for (uint32_t w = 0; w < warp; ++w) pos += warp_take[w];
        if (take && pos < SAMPLE_MAX_K) { cand_idx[pos] = i; cand_val[pos] = v; }
        __syncthreads();
        if (tid == 0) {
            uint32_t t = 0, e = 0;
            for (uint32_t w = 0; w < SAMPLE_THREADS / 32; ++w) { t += warp_take[w]; e += warp_eq[w]; }
            s_take_base += t;
            s_eq_base += e;
        }
        __syncthreads();
    }

    // ---- the draw ----
    if (tid == 0) {
        const uint32_t n = s_take_base < SAMPLE_MAX_K ? s_take_base : SAMPLE_MAX_K;   // == k
        float best = cand_val[0];
        int best_key = total_order_key(best);
        for (uint32_t j = 1; j < n; ++j) {
            const int key = total_order_key(cand_val[j]);
            if (key >= best_key) { best_key = key; best = cand_val[j]; }
        }
        float z = 0.0f;
        for (uint32_t j = 0; j < n; ++j) {
            const float t = __fdiv_rn(__fsub_rn(cand_val[j], best), temperature);
            const float w = (float)exp((double)t);
            cand_val[j] = w;
            z = __fadd_rn(z, w);
        }
        const uint32_t step = (d_step ? d_step[(size_t)blockIdx.x * step_stride] : 0u) + step_add;
        const uint32_t x = philox_first(step, 0u, first_session + blockIdx.x, 0u, seed_lo, seed_hi);
        const float u = (float)(x >> 8) * (1.0f / 16777216.0f);
        const float target = __fmul_rn(u, z);
        float running = 0.0f;
        uint32_t pick = cand_idx[n - 1];
        for (uint32_t j = 0; j < n; ++j) {
            running = __fadd_rn(running, cand_val[j]);
            if (running > target) { pick = cand_idx[j]; break; }
        }
        out[blockIdx.x] = pick;
    }
}

int launch_sample_top_k(const float* logits, uint32_t* out, uint32_t rows, uint32_t vocab, uint32_t row_stride,
                        float temperature, uint32_t top_k, uint64_t seed, const uint32_t* d_step, uint32_t step_stride,
                        uint32_t step_add, uint32_t first_session, cudaStream_t stream) {
    if (rows == 0) return TNSR_B200_OK;
    if (!(temperature > 0.0f) || !std::isfinite(temperature) || top_k == 0 || top_k > SAMPLE_MAX_K || vocab == 0) {
        set_thread_error("sampling needs a finite temperature > 0 and 1 <= top_k <= 256");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    launch_kernel(sample_top_k_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, vocab, row_stride, temperature, top_k,
                  (uint32_t)(seed & 0xffffffffu), (uint32_t)(seed >> 32), d_step, step_stride, step_add, first_session, out);
    count_launch();
    return check_launch("sample_top_k");
}

}  // namespace tb
