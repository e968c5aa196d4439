// bf16 GEMM for at most 16 activation rows against a large weight matrix: out[m, n] = a[m, :] . bt[n, :].
//
// With so few rows the product is one pass over the weights: 2 * n * k bytes against 2 * m * n * k flops, i.e. HBM-bound
// by two orders of magnitude.  The kernel is therefore built around the weight stream and nothing else:
//  * a CTA owns 16 consecutive weight rows at a time (one column tile of the output) and walks all of K for them, so every
//    output element is produced by exactly one CTA -- no split-K, no partial tiles in L2, no hand-over between CTAs, no
//    scratch, and a summation order that depends on nothing but the shape;
//  * the activation rows (<= 16 x k bf16) are loaded once per CTA and stay in shared memory;
//  * the weight rows flow through a ring of 512-wide chunks filled by 16-byte cp.async copies whose addresses are
//    per-thread constants plus a running offset (the first version recomputed row and column of every copy: with eight
//    warps per SM that arithmetic, not memory, set the pace -- 4.8 M instructions for a 33.5 MB operand); the ring is
//    requested in full at the very start (before anything else), so after one memory latency the whole GPU has ~20 MB in
//    flight -- for a 4096 x 4096 matrix that is most of the operand.  (Bulk copies of one 1 KB row segment each were
//    slower still, 19.5 against 14.8 us: the copy engine's per-request cost dominates at that size, and a 16-row tile
//    has no larger contiguous piece.)
//  * products run on warp-level mma.sync.m16n8k16 (weight rows = M side, 8 activation rows = N side); the eight warps
//    take alternate k-steps of a chunk and their partial tiles are added in warp order at the end of a column tile.
// It replaces, for m <= 16, the tcgen05 few-row engine with split-K (gemm_skinny.cu), whose hand-over of partial tiles
// through L2 cost more than the products (reference policy for such shapes: src/tile/matmul_schedule.rs:487-646,
// src/graph/split_k.rs).
#include "common.cuh"

namespace tb {

namespace {

constexpr int GS_THREADS = 256;
constexpr int GS_KCH = 512;
constexpr int GS_PITCH = GS_KCH + 8;          // 1040 bytes per row: conflict-free ldmatrix
constexpr int GS_ROWS = 16;                   // weight rows per column tile
constexpr size_t GS_SMEM_LIMIT = 220 * 1024;

struct GsParams {
    const bf16* a;        // [m, k]
    const bf16* w;        // [n, k]
    void* out;
    uint32_t ldc, m, n, k;
    const float* bias;
    const float* residual;
    uint32_t ldr;
    int activation, out_dtype;
    uint32_t stages;
};

__device__ __forceinline__ uint32_t gs_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gs_cp16(void* dst, const void* src, bool valid) {
    const uint32_t n = valid ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(gs_smem(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void gs_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void gs_wait_pending(uint32_t n) {
    switch (n) {
        case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
        case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
        case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
        case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
    }
}
__device__ __forceinline__ void gs_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(gs_smem(p)));
}
__device__ __forceinline__ void gs_ldmatrix_x2(uint32_t (&r)[2], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(gs_smem(p)));
}
__device__ __forceinline__ void gs_mma(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// MT: activation rows padded to 8 or 16.
template <int MT>
__global__ void __launch_bounds__(GS_THREADS, 1)
gemm_stream_kernel(GsParams P) {
    constexpr int NT = MT / 8;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t apitch = P.k + 8;                                           // activation row pitch in elements
    bf16* abuf = reinterpret_cast<bf16*>(smem);                                // [MT][k + 8]
    bf16* ring = abuf + (size_t)MT * apitch;                                   // [stages][16][PITCH]
    float* red = reinterpret_cast<float*>(ring + (size_t)P.stages * GS_ROWS * GS_PITCH);   // [8 warps][16 * MT]

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t tiles = (P.n + GS_ROWS - 1) / GS_ROWS;
    const uint32_t chunks = (P.k + GS_KCH - 1) / GS_KCH;
    const uint32_t my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t total = my_tiles * chunks;                                  // ring slots this CTA consumes

    // Slot s = chunk (s % chunks) of this CTA's (s / chunks)-th column tile; one cp.async group per slot.  (Starting
    // every tile's walk over K at a different chunk, so that the CTAs do not all read the same column range at the same
    // moment, was measured and is slower: 15.5 against 14.2 us.)
    auto chunk_of = [&](uint32_t s) { return s % chunks; };
    // A thread always copies the same four (row, column) pieces of a chunk: rows r0, r0 + 4, r0 + 8, r0 + 12 at column kk.
    const uint32_t r0 = threadIdx.x >> 6, kk = (threadIdx.x & 63) * 8;
    const uint32_t dst_off = r0 * GS_PITCH + kk;
    auto issue = [&](uint32_t s) {
        if (s < total) {
            const uint32_t n0 = (blockIdx.x + (s / chunks) * gridDim.x) * GS_ROWS, k0 = chunk_of(s) * GS_KCH;
            bf16* dst = ring + (size_t)(s % P.stages) * GS_ROWS * GS_PITCH + dst_off;
            const bool col_ok = k0 + kk < P.k;
            const bf16* src = P.w + (size_t)(n0 + r0) * P.k + k0 + kk;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bool valid = col_ok && n0 + r0 + 4 * j < P.n;
                gs_cp16(dst + (size_t)j * 4 * GS_PITCH, valid ? src + (size_t)j * 4 * P.k : P.w, valid);
            }
        }
        gs_commit();        // a group per slot, also when it is empty: the wait counts stay uniform
    };
    // The weights do not depend on the previous kernel: request the whole ring before waiting for it.
    for (uint32_t s = 0; s + 1 < P.stages; ++s) issue(s);
    pdl_wait();
    pdl_trigger();
    {
        // activation rows: thread t copies pieces t, t + 256, ... of the [m, k] block; rows past m are zero-filled
        const uint32_t per_row = P.k / 8;
        for (uint32_t i = threadIdx.x; i < (uint32_t)MT * per_row; i += GS_THREADS) {
            const uint32_t r = i / per_row, c = (i % per_row) * 8;
            gs_cp16(abuf + (size_t)r * apitch + c, P.a + (r < P.m ? (size_t)r * P.k + c : 0), r < P.m);
        }
        gs_commit();
    }
    // groups so far, in order: slots 0 .. stages-2, then the activation rows

    float acc[NT][4];
    for (uint32_t s = 0; s < total; ++s) {
        const uint32_t step = s % chunks, ch = chunk_of(s);
        if (step == 0) {
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[j][e] = 0.0f;
        }
        issue(s + P.stages - 1);      // into the buffer slot s - 1 used: everyone left it at the barrier below
        // Slot s must have landed; the stages - 1 slots requested after it may still be on their way.  The first time the
        // activation rows must be there too, and their group sits behind the initial ring: only the newest group may pend.
        gs_wait_pending(s == 0 ? 1u : P.stages - 1);
        __syncthreads();
        const bf16* wt = ring + (size_t)(s % P.stages) * GS_ROWS * GS_PITCH;
        const uint32_t ksteps = min((uint32_t)GS_KCH, P.k - ch * GS_KCH) / 16;
        for (uint32_t ks = warp; ks < ksteps; ks += GS_THREADS / 32) {
            uint32_t a[4];
            gs_ldmatrix_x4(a, wt + (size_t)(lane & 15) * GS_PITCH + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                uint32_t b[2];
                gs_ldmatrix_x2(b, abuf + (size_t)(j * 8 + (lane & 7)) * apitch + ch * GS_KCH + ks * 16 + ((lane >> 3) & 1) * 8);
                gs_mma(acc[j], a, b);
            }
        }
        __syncthreads();            // the slot's buffer may be refilled by the next issue
        if (step + 1 == chunks) {
            // end of a column tile: add the eight warps' partial tiles in warp order, then the epilogue
            const uint32_t row = lane >> 2, col = (lane & 3) * 2;
            float* mine = red + (size_t)warp * GS_ROWS * MT;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint32_t m = j * 8 + col;
                mine[row * MT + m] = acc[j][0];
                mine[row * MT + m + 1] = acc[j][1];
                mine[(row + 8) * MT + m] = acc[j][2];
                mine[(row + 8) * MT + m + 1] = acc[j][3];
            }
            __syncthreads();
            const uint32_t n0 = (blockIdx.x + (s / chunks) * gridDim.x) * GS_ROWS;
            for (uint32_t o = threadIdx.x; o < (uint32_t)GS_ROWS * MT; o += GS_THREADS) {
                const uint32_t c = o % GS_ROWS, m = o / GS_ROWS;
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < GS_THREADS / 32; ++w) v += red[(size_t)w * GS_ROWS * MT + c * MT + m];
                const uint32_t colg = n0 + c;
                if (m < P.m && colg < P.n) {
                    if (P.bias) v += __ldg(P.bias + colg);
                    v = apply_activation(v, P.activation);
                    if (P.out_dtype == TNSR_B200_BF16) {
                        reinterpret_cast<bf16*>(P.out)[(size_t)m * P.ldc + colg] = __float2bfloat16_rn(v);
                    } else {
                        if (P.residual) v += P.residual[(size_t)m * P.ldr + colg];
                        reinterpret_cast<float*>(P.out)[(size_t)m * P.ldc + colg] = v;
                    }
                }
            }
            __syncthreads();
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
}

int gs_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

template <int MT>
int gs_launch(GsParams P, cudaStream_t stream) {
    const size_t fixed = (size_t)MT * (P.k + 8) * 2 + (size_t)(GS_THREADS / 32) * GS_ROWS * MT * 4;
    const size_t stage = (size_t)GS_ROWS * GS_PITCH * 2;
    uint32_t stages = (uint32_t)std::min<size_t>(8, (GS_SMEM_LIMIT - fixed) / stage);
    P.stages = stages;
    const size_t smem = fixed + stages * stage;
    static size_t configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || configured[dev] < smem) {
        if (cudaFuncSetAttribute(gemm_stream_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return check_launch("gemm_stream attribute");
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    const uint32_t tiles = ceil_div(P.n, (uint32_t)GS_ROWS);
    const uint32_t grid = std::min(tiles, (uint32_t)gs_sm_count());
    launch_kernel(gemm_stream_kernel<MT>, dim3(grid), dim3(GS_THREADS), smem, stream, P);
    count_launch();
    return check_launch("gemm_stream");
}

}  // namespace

bool gemm_stream_eligible(const bf16* a, const bf16* bt, uint32_t m, uint32_t n, uint32_t k, const GemmEpilogue& ep) {
    if (m < 1 || m > 16 || n < 16 || k % 16 != 0 || k < 16) return false;
    if (ep.rows_per_session != 0 || ep.round_bf16) return false;
    if (reinterpret_cast<uintptr_t>(a) % 16 != 0 || reinterpret_cast<uintptr_t>(bt) % 16 != 0) return false;
    const uint32_t mt = m <= 8 ? 8 : 16;
    const size_t fixed = (size_t)mt * (k + 8) * 2 + (size_t)(GS_THREADS / 32) * GS_ROWS * mt * 4;
    return fixed + 3 * (size_t)GS_ROWS * GS_PITCH * 2 <= GS_SMEM_LIMIT;     // the activation rows and a ring of at least 3
}

int launch_gemm_stream(const bf16* a, const bf16* bt, void* out, uint32_t ldc, uint32_t m, uint32_t n, uint32_t k,
                       const GemmEpilogue& ep, int* d_status, cudaStream_t stream) {
    (void)d_status;      // nothing in this kernel waits on another agent: there is no time-out to report
    GsParams P = {};
    P.a = a; P.w = bt; P.out = out; P.ldc = ldc; P.m = m; P.n = n; P.k = k;
    P.bias = ep.bias; P.residual = ep.residual; P.ldr = ep.ldr; P.activation = ep.activation; P.out_dtype = ep.out_dtype;
    return m <= 8 ? gs_launch<8>(P, stream) : gs_launch<16>(P, stream);
}

}  // namespace tb
