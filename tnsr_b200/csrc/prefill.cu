// Tiled causal prefill attention over a bf16 K/V cache: `chunk` new queries per
// session attend keys 0 .. position + t (their own rows are already in the
// cache).  One CTA = 64 queries of one (session, head); keys stream through a
// double-buffered shared-memory tile (cp.async, 16 bytes per request) and both
// products run on the warp-level tensor cores (mma.sync m16n8k16, bf16 operands,
// f32 accumulators) with the softmax statistics kept in registers.  This plays
// the part of the reference's `decoder_prefill_bf16` (src/nn/kv_cache/prefill.rs:
// 170-607: 16/32 queries x 32-key steps on 16x16x16 wmma, key partitions merged
// afterwards); here one CTA walks all keys of its query block, so no merge pass.
// Large chunks at a host-known position go to the tcgen05 kernel (prefill_tc.cu);
// this one serves device-resident positions, short chunks and the CUDA-core-only
// engine setting.
#include "common.cuh"

namespace tb {

constexpr int PF_BQ = 64, PF_BK = 64, PF_HD = 64, PF_THREADS = 128;

__device__ __forceinline__ uint32_t pf_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pf_cp_async16(void* dst, const void* src, bool pred) {
    const uint32_t bytes = pred ? 16u : 0u;  // zero-fill when the row is out of range
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(pf_smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pf_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void pf_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float pf_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 64-dim rows are 128 bytes = 8 chunks of 16 bytes; chunk c of row r sits at c ^ (r & 7).
__device__ __forceinline__ uint32_t pf_off(uint32_t row, uint32_t dim) {
    return row * 128u + ((((dim >> 3) ^ row) & 7u) << 4) + ((dim & 7u) << 1);
}

__global__ void __launch_bounds__(PF_THREADS)
prefill_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                         bf16* __restrict__ out, uint32_t chunk, uint32_t position,
                         const uint32_t* __restrict__ d_position, uint32_t capacity, uint32_t heads, float scale_log2) {
    __shared__ __align__(128) uint8_t qs[PF_BQ * 128];
    __shared__ __align__(128) uint8_t ks[2][PF_BK * 128];
    __shared__ __align__(128) uint8_t vs[2][PF_BK * 128];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t g = lane >> 2, t4 = lane & 3;
    const uint32_t q0 = blockIdx.x * PF_BQ, h = blockIdx.y, s = blockIdx.z;
    const uint32_t d = heads * PF_HD;
    const uint32_t past = d_position ? *d_position : position;
    uint32_t last_q = min(q0 + PF_BQ, chunk) - 1;
    uint32_t total = past + last_q + 1;  // keys visible to the last query of this block
    if (total > capacity) total = capacity;
    const uint32_t n_tiles = (total + PF_BK - 1) / PF_BK;

    const bf16* qg = q + ((size_t)s * chunk) * d + (size_t)h * PF_HD;
    const bf16* kg = kc + ((size_t)s * capacity) * d + (size_t)h * PF_HD;
    const bf16* vg = vc + ((size_t)s * capacity) * d + (size_t)h * PF_HD;

    // 64 rows x 8 chunks = 512 requests per tile, 4 per thread
    auto load_kv = [&](uint32_t tile, uint32_t buf) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t e = tid + i * PF_THREADS, row = e >> 3, ch = e & 7;
            const uint32_t key = tile * PF_BK + row;
            const bool ok = key < total;
            const size_t goff = (size_t)(ok ? key : 0) * d + ch * 8;
            pf_cp_async16(ks[buf] + pf_off(row, ch * 8), kg + goff, ok);
            pf_cp_async16(vs[buf] + pf_off(row, ch * 8), vg + goff, ok);
        }
    };
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t e = tid + i * PF_THREADS, row = e >> 3, ch = e & 7;
        const bool ok = q0 + row < chunk;
        pf_cp_async16(qs + pf_off(row, ch * 8), qg + (size_t)(ok ? q0 + row : 0) * d + ch * 8, ok);
    }
    load_kv(0, 0);
    pf_commit();

    uint32_t qa[4][4];  // A fragments of this warp's 16 query rows, 4 k-steps
    float o[8][4];      // 16 x 64 output accumulators
#pragma unroll
    for (int i = 0; i < 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    const uint32_t qrow0 = q0 + warp * 16 + g, qrow1 = qrow0 + 8;   // query indices of this thread's two rows
    const uint32_t lim0 = past + qrow0, lim1 = past + qrow1;         // last visible key of each

    for (uint32_t tile = 0; tile < n_tiles; ++tile) {
        const uint32_t buf = tile & 1;
        if (tile + 1 < n_tiles) load_kv(tile + 1, buf ^ 1);
        pf_commit();
        pf_wait<1>();
        __syncthreads();
        if (tile == 0) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint32_t row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dim = kk * 16 + (lane >> 4) * 8;
                ldsm_x4(pf_smem_u32(qs + pf_off(row, dim)), qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
            }
        }
        // S = Q K^T : 16 x 64 per warp
        float sc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) { sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.0f; }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {  // pairs of 8-key tiles
                const uint32_t key = np * 16 + (lane & 7) + (lane >> 4) * 8, dim = kk * 16 + ((lane >> 3) & 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4(pf_smem_u32(ks[buf] + pf_off(key, dim)), b0, b1, b2, b3);
                mma_bf16(sc[2 * np], qa[kk], b0, b1);
                mma_bf16(sc[2 * np + 1], qa[kk], b2, b3);
            }
        }
        // scale, mask, running max
        const uint32_t kbase = tile * PF_BK;
        const bool need_mask = kbase + PF_BK - 1 > past + q0 + warp * 16;  // some key may be hidden from this warp's first row
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = sc[i][e] * scale_log2;
                if (need_mask) {
                    const uint32_t key = kbase + i * 8 + t4 * 2 + (e & 1);
                    const uint32_t lim = (e < 2) ? lim0 : lim1;
                    if (key > lim || key >= total) v = -INFINITY;
                }
                sc[i][e] = v;
            }
            mx0 = fmaxf(mx0, fmaxf(sc[i][0], sc[i][1]));
            mx1 = fmaxf(mx1, fmaxf(sc[i][2], sc[i][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float ms0 = (mx0 == -INFINITY) ? 0.0f : mx0, ms1 = (mx1 == -INFINITY) ? 0.0f : mx1;
        const float c0 = pf_ex2(m0 - ms0), c1 = pf_ex2(m1 - ms1);
        m0 = mx0;
        m1 = mx1;
        float rs0 = 0.0f, rs1 = 0.0f;
        uint32_t pa[4][4];  // P as A fragments: k-step kk covers keys 16kk .. 16kk+15
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float p0 = pf_ex2(sc[i][0] - ms0), p1 = pf_ex2(sc[i][1] - ms0);
            const float p2 = pf_ex2(sc[i][2] - ms1), p3 = pf_ex2(sc[i][3] - ms1);
            rs0 += p0 + p1;
            rs1 += p2 + p3;
            pa[i >> 1][(i & 1) * 2] = pack_bf16x2(p0, p1);
            pa[i >> 1][(i & 1) * 2 + 1] = pack_bf16x2(p2, p3);
        }
        l0 = l0 * c0 + rs0;
        l1 = l1 * c1 + rs1;
#pragma unroll
        for (int i = 0; i < 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {  // pairs of 8-dim tiles
                const uint32_t key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dim = np * 16 + (lane >> 4) * 8;
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(pf_smem_u32(vs[buf] + pf_off(key, dim)), b0, b1, b2, b3);
                mma_bf16(o[2 * np], pa[kk], b0, b1);
                mma_bf16(o[2 * np + 1], pa[kk], b2, b3);
            }
        }
        __syncthreads();
    }
    pf_wait<0>();
    // row sums live spread over the 4 lanes of a quad
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
    bf16* og = out + ((size_t)s * chunk) * d + (size_t)h * PF_HD;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t col = i * 8 + t4 * 2;
        if (qrow0 < chunk) *reinterpret_cast<uint32_t*>(og + (size_t)qrow0 * d + col) = pack_bf16x2(o[i][0] * i0, o[i][1] * i0);
        if (qrow1 < chunk) *reinterpret_cast<uint32_t*>(og + (size_t)qrow1 * d + col) = pack_bf16x2(o[i][2] * i1, o[i][3] * i1);
    }
}

bool prefill_attention_supported(uint32_t head_dim) { return head_dim == PF_HD; }

int launch_prefill_attention(const bf16* q, const bf16* k_cache, const bf16* v_cache, bf16* out,
                             uint32_t sessions, uint32_t chunk, uint32_t position,
                             const uint32_t* d_position, uint32_t capacity, uint32_t heads,
                             uint32_t head_dim, int* d_status, cudaStream_t stream) {
    if (sessions == 0 || chunk == 0) return TNSR_B200_OK;
    if (head_dim != PF_HD) {
        set_thread_error("prefill attention: head_dim must be 64");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    if (heads > 65535u || sessions > 65535u) return TNSR_B200_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
         reinterpret_cast<uintptr_t>(out)) % 16) {
        set_thread_error("prefill attention: pointers must be 16-byte aligned");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    if (prefill_attention_tc_eligible(sessions, chunk, position, d_position, capacity, heads, head_dim))
        return launch_prefill_attention_tc(q, k_cache, v_cache, out, sessions, chunk, position, capacity, heads, d_status, stream);
    const float scale_log2 = (1.0f / sqrtf((float)head_dim)) * 1.4426950408889634f;
    dim3 grid(ceil_div(chunk, PF_BQ), heads, sessions);
    prefill_attention_kernel<<<grid, PF_THREADS, 0, stream>>>(q, k_cache, v_cache, out, chunk, position, d_position,
                                                              capacity, heads, scale_log2);
    count_launch();
    return check_launch("prefill_attention");
}

}  // namespace tb
