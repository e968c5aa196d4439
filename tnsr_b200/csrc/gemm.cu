// bf16 GEMM with f32 accumulation: out = epilogue(a[m,k] . bt[n,k]^T).
//
// Two engines share one epilogue:
//  * gemm_tc_kernel   -- the Blackwell path: TMA (cp.async.bulk.tensor, 128-byte
//    swizzle, one copy per CTA, no cluster forms) feeds a shared-memory ring,
//    one thread issues tcgen05.mma (M=128, N=BN, K=16 per instruction) into
//    double-buffered TMEM accumulators, eight epilogue warps drain them with
//    tcgen05.ld, transpose each 32x32 block through shared memory and write
//    coalesced rows while the next tile's main loop runs.  Persistent over tiles.
//  * gemm_simple_kernel -- CUDA-core kernel for shapes TMA cannot address
//    (k not a multiple of 8, unaligned pointers) and as the cross-check of the
//    tensor-core engine.
//
// This replaces the reference's tiled matmul path (wmma/mma.sync 64x64x32 tiles
// with cp.async double buffering and fused epilogues: src/tile/matmul_schedule.rs:
// 487-646, src/ptx/graph/matmul.rs:4-129, src/tile/graph.rs:712-1107).
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "tc_common.cuh"

namespace tb {

int g_gemm_engine = 0;
thread_local uint32_t t_lose_gemm_stage = 0;
struct EpiParams {
    GemmEpilogue ep;
    GemmQkvTargets qkv;
    void* out;
    uint32_t ldc;
    uint32_t m, n;  // n = columns of the accumulator (packed width for SWIGLU)
};

// ---- epilogue: scalar forms ---------------------------------------------------
__device__ __forceinline__ size_t map_out_row(const GemmEpilogue& ep, uint32_t row) {
    if (!ep.rows_per_session) return row;
    uint32_t off = ep.d_row_offset ? *ep.d_row_offset : ep.row_offset;
    return (size_t)(row / ep.rows_per_session) * ep.out_session_rows + off + row % ep.rows_per_session;
}

__device__ __forceinline__ void store_plain(const EpiParams& P, uint32_t row, uint32_t col, float acc) {
    float v = acc;
    if (P.ep.bias) v += P.ep.bias[col];
    v = apply_activation(v, P.ep.activation);
    size_t orow = map_out_row(P.ep, row);
    if (P.ep.out_dtype == TNSR_B200_BF16) {
        reinterpret_cast<bf16*>(P.out)[orow * P.ldc + col] = __float2bfloat16_rn(v);
    } else {
        if (P.ep.residual) v += P.ep.residual[(size_t)row * P.ep.ldr + col];
        reinterpret_cast<float*>(P.out)[orow * P.ldc + col] = v;
    }
}

__device__ __forceinline__ void store_qkv(const EpiParams& P, uint32_t row, uint32_t col, float acc) {
    float v = acc;
    if (P.ep.bias) v += P.ep.bias[col];
    const uint32_t d = P.qkv.d, which = col / d, c = col % d;
    if (which == 0) {
        P.qkv.q[(size_t)row * d + c] = __float2bfloat16_rn(v);
    } else {
        const uint32_t session = row / P.qkv.chunk;
        uint32_t pos = P.qkv.d_position ? P.qkv.d_position[session * P.qkv.position_stride] : P.qkv.position;
        size_t crow = kv_row(P.qkv.paging, session, pos + row % P.qkv.chunk, P.qkv.capacity);
        (which == 1 ? P.qkv.k_cache : P.qkv.v_cache)[crow * d + c] = __float2bfloat16_rn(v);
    }
}

// g, u: accumulators of packed columns pc and pc + 16; output column oc.
__device__ __forceinline__ void store_swiglu(const EpiParams& P, uint32_t row, uint32_t pc, uint32_t oc,
                                             float g, float u) {
    if (P.ep.bias) {
        g += P.ep.bias[pc];
        u += P.ep.bias[pc + 16];
    }
    reinterpret_cast<bf16*>(P.out)[(size_t)row * P.ldc + oc] = __float2bfloat16_rn(fast_silu(g) * u);
}

// ===========================================================================
// CUDA-core engine: 64x64 tile, 16x16 threads, 4x4 outputs per thread.
// ===========================================================================
constexpr int SB = 64, SK = 16;

template <int MODE>
__global__ void __launch_bounds__(256)
gemm_simple_kernel(const bf16* __restrict__ a, uint32_t lda, const bf16* __restrict__ bt, EpiParams P, uint32_t k) {
    __shared__ float as[SK][SB + 4];
    __shared__ float bs[SK][SB + 4];
    __shared__ float cs[SB][SB + 1];
    pdl_wait();
    pdl_trigger();
    const uint32_t tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const uint32_t m0 = blockIdx.y * SB, n0 = blockIdx.x * SB;
    float acc[4][4] = {};
    for (uint32_t k0 = 0; k0 < k; k0 += SK) {
        // 64 rows x 16 k per operand = 1024 elements, 4 per thread
        {
            uint32_t r = tid / 4, kk = (tid % 4) * 4;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t gk = k0 + kk + i;
                float va = 0.0f, vb = 0.0f;
                if (gk < k) {
                    if (m0 + r < P.m) va = __bfloat162float(a[(size_t)(m0 + r) * lda + gk]);
                    if (n0 + r < P.n) vb = __bfloat162float(bt[(size_t)(n0 + r) * k + gk]);
                }
                as[kk + i][r] = va;
                bs[kk + i][r] = vb;
            }
        }
        __syncthreads();
#pragma unroll
        for (int p = 0; p < SK; ++p) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = as[p][ty * 4 + i]; bv[i] = bs[p][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) cs[ty * 4 + i][tx * 4 + j] = acc[i][j];
    __syncthreads();
    if (MODE == GEMM_ARGMAX) {
        // one candidate per (row, 64-column tile): thread r scans its row of the tile in column order
        if (tid < SB && m0 + tid < P.m) {
            int best = 0;
            uint32_t best_i = 0;
            bool have = false;
            for (uint32_t c = 0; c < SB && n0 + c < P.n; ++c) {
                const int key = total_order_key(cs[tid][c]);
                if (!have || key >= best) { best = key; best_i = n0 + c; have = true; }
            }
            reinterpret_cast<uint2*>(P.out)[(size_t)(m0 + tid) * P.ldc + blockIdx.x] = make_uint2((uint32_t)best, best_i);
        }
    } else if (MODE == GEMM_SWIGLU) {
        // 64 packed columns = 2 blocks of (16 gate, 16 up) -> 32 output columns
        for (uint32_t e = tid; e < SB * 32; e += 256) {
            uint32_t r = e / 32, oc_local = e % 32;
            uint32_t pc_local = (oc_local / 16) * 32 + oc_local % 16;
            uint32_t row = m0 + r, pc = n0 + pc_local, oc = n0 / 2 + oc_local;
            if (row < P.m && pc + 16 < P.n)
                store_swiglu(P, row, pc, oc, cs[r][pc_local], cs[r][pc_local + 16]);
        }
    } else {
        for (uint32_t e = tid; e < SB * SB; e += 256) {
            uint32_t r = e / SB, c = e % SB, row = m0 + r, col = n0 + c;
            if (row < P.m && col < P.n) {
                if (MODE == GEMM_QKV) store_qkv(P, row, col, cs[r][c]);
                else store_plain(P, row, col, cs[r][c]);
            }
        }
    }
}

static int launch_simple(const bf16* a, uint32_t lda, const bf16* bt, const EpiParams& P, uint32_t k, GemmMode mode,
                         cudaStream_t stream) {
    dim3 grid(ceil_div(P.n, SB), ceil_div(P.m, SB));
    if (grid.y > 65535u) {
        set_thread_error("gemm: too many rows for the CUDA-core engine");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    switch (mode) {
        case GEMM_PLAIN: launch_kernel(gemm_simple_kernel<GEMM_PLAIN>, grid, dim3(256), 0, stream, a, lda, bt, P, k); break;
        case GEMM_QKV: launch_kernel(gemm_simple_kernel<GEMM_QKV>, grid, dim3(256), 0, stream, a, lda, bt, P, k); break;
        case GEMM_SWIGLU: launch_kernel(gemm_simple_kernel<GEMM_SWIGLU>, grid, dim3(256), 0, stream, a, lda, bt, P, k); break;
        case GEMM_ARGMAX: launch_kernel(gemm_simple_kernel<GEMM_ARGMAX>, grid, dim3(256), 0, stream, a, lda, bt, P, k); break;
    }
    count_launch();
    return check_launch("gemm_simple");
}

// ===========================================================================
// tcgen05 engine
// ===========================================================================
constexpr int BM = 128;           // rows per tile = TMEM lanes
constexpr int BK = 64;            // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;        // K per tcgen05.mma for 16-bit operands
// Epilogue warps per CTA (template parameter EPI): 8 = two per TMEM lane quarter, 16 = four per quarter; the warps of a
// quarter take 32-column chunks in turn.  Warp 0: TMA, warp 1: MMA + TMEM owner, warps 2 .. EPI + 1: epilogue.
constexpr uint32_t TC_STAGE_TILE_BYTES = 32 * 32 * 4;  // per-warp transpose buffer: 32 rows x 32 f32 columns

template <int BN, int EPI>
struct TcShape {
    static constexpr int THREADS = 64 + 32 * EPI;
    // 4 stages of 48 KB at BN 256 with 8 epilogue warps; 3 with 16 (their transpose buffers take 64 KB).
    // EPI 4 is the lean form of the narrow tiles (few rows, one tile per CTA: the decode step): half the shared memory
    // (about 115 KB) and at most 112 registers x 192 threads, so that a CTA of it fits on an SM beside a CTA of the lean
    // decode-attention kernel that works on the other half of the batch.
    static constexpr int STAGES = BN >= 256 ? (EPI > 8 ? 3 : 4) : (BN >= 128 ? 6 : (EPI == 4 ? (BN >= 64 ? 4 : 5) : 8));
    static constexpr uint32_t A_BYTES = BM * BK * 2;
    static constexpr uint32_t B_BYTES = BN * BK * 2;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;  // two accumulators; power of two
    static constexpr uint32_t SMEM_BYTES =
        STAGES * STAGE_BYTES + 1024 /* alignment slack */ + EPI * TC_STAGE_TILE_BYTES + 256 /* barriers */;
};

// Instruction descriptor, kind::f16: f32 accumulator (bit 4), bf16 A (bit 7)
// and B (bit 10), both K-major (bits 15, 16 clear), N/8 at bit 17, M/16 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc_bf16(uint32_t bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

struct TcParams {
    EpiParams epi;
    uint32_t k;
    uint32_t tiles_m, tiles_n;
    int* d_status;
    // 1: f32 output accumulated in place on the residual (out == residual): the epilogue hands each 32 x 32 block of
    // act(acc + bias) to a TMA reduce-add on `map_out` instead of reading, adding and storing the rows itself
    // 2: split-K: tile t is the k-block range (t % split_k) of output tile t / split_k, and its blocks are STORED into
    // the partial-sum buffer behind `map_out` at row (t % split_k) * split_rows + row (the first range adds the bias)
    uint32_t tma_reduce;
    uint32_t split_k, split_rows;
    // 1: bf16 destinations are written with bulk tensor stores of 32-row blocks (map_out; map_k / map_v for the caches
    // of the QKV routing) instead of per-lane stores
    uint32_t tma_store;
    uint64_t wait_limit_ns;   // bound of every mbarrier wait (tnsr_b200_set_wait_limit_ns)
    // Test hook (0 = off): the producer of CTA 0 leaves out the copies of k-block `lose_kb - 1` of its first tile, so
    // the MMA warp's wait for that stage runs out and the kernel leaves through its abort path.
    uint32_t lose_kb;
};

// Grouped tile order: 8 row-tiles share each column-tile before moving on, so a
// wave of CTAs re-reads few distinct operand tiles from L2.
__device__ __forceinline__ void tile_coords(uint32_t tile, uint32_t tiles_m, uint32_t tiles_n, uint32_t& tm, uint32_t& tn) {
    constexpr uint32_t GROUP = 8;
    const uint32_t per_group = GROUP * tiles_n;
    const uint32_t group = tile / per_group, first = group * GROUP;
    const uint32_t size = min(tiles_m - first, GROUP);
    const uint32_t in_group = tile % per_group;
    tm = first + in_group % size;
    tn = in_group / size;
}

// ---- epilogue of one 32-row x 32-column accumulator block, one warp ------------------
// tcgen05.ld hands every lane one ROW of the block (32 columns in registers).  Writing global
// memory that way would touch 32 different cache lines per store instruction, so the block is
// first transposed through a 4 KB shared-memory buffer private to the warp: lanes write their
// row (16-byte stores, XOR-swizzled in units of 4 columns so neither phase has bank conflicts),
// then lanes become COLUMNS and every global access is one contiguous segment per row.
__device__ __forceinline__ uint32_t stage_index(uint32_t r, uint32_t c) {
    return r * 32u + ((((c >> 2) ^ r) & 7u) << 2) + (c & 3u);
}

__device__ __forceinline__ float4 stage_load4(const float* stage, uint32_t r, uint32_t c4) {
    return *reinterpret_cast<const float4*>(stage + stage_index(r, c4));
}
__device__ __forceinline__ float4 act4(float4 v, int act) {
    if (act == ACT_NONE) return v;
    return make_float4(apply_activation(v.x, act), apply_activation(v.y, act), apply_activation(v.z, act), apply_activation(v.w, act));
}

// True when the f32 epilogue of this block takes its 16-byte path (whole block inside the matrix, aligned
// pointers and leading dimensions).
__device__ __forceinline__ bool f32_vector_path(const EpiParams& P, uint32_t col0) {
    const float* res = P.ep.residual;
    return col0 + 32 <= P.n && (reinterpret_cast<uintptr_t>(P.ep.bias) & 15) == 0 && P.ldc % 4 == 0 &&
           (reinterpret_cast<uintptr_t>(P.out) & 15) == 0 &&
           (!res || (P.ep.ldr % 4 == 0 && (reinterpret_cast<uintptr_t>(res) & 15) == 0));
}

// Residual values of this lane for the 16-byte f32 path: rows (it * 4 + lane / 8), columns 4 * (lane % 8) .. + 3.
__device__ __forceinline__ void load_residual_block(const EpiParams& P, uint32_t row0, uint32_t col0, uint32_t lane, float4* r4) {
    const float* res = P.ep.residual;
    const uint32_t c4 = 4 * (lane & 7), rsub = lane >> 3;
    const uint32_t rows = row0 < P.m ? min(32u, P.m - row0) : 0u;
#pragma unroll
    for (uint32_t it = 0; it < 8; ++it) {
        const uint32_t rr = it * 4 + rsub;
        r4[it] = (res && rr < rows) ? *reinterpret_cast<const float4*>(res + (size_t)(row0 + rr) * P.ep.ldr + col0 + c4)
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// In-place residual update through TMA: the lane's accumulator row (+ bias, activation) goes into the warp's 4 KB
// buffer in the 128-byte-swizzled layout of a 32-row x 32-column f32 box, and one bulk tensor reduce-add folds the
// box into the residual stream in global memory.  The warp neither reads the residual nor issues stores; rows and
// columns outside the matrix are clipped by the tensor map.  One add per element, so the result is the same
// residual + value an explicit read-add-store gives.
__device__ __forceinline__ void epilogue_block_reduce(const EpiParams& P, const CUtensorMap* map_out, float* stage,
                                                      uint32_t row0, uint32_t col0, const float* acc, uint32_t lane,
                                                      bool store = false, bool with_bias = true, uint32_t row_out = 0) {
    // the previous box of this warp must have been read out of the buffer
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncwarp();
    float4* row = reinterpret_cast<float4*>(stage) + lane * 8;
    const bool bias_vec = with_bias && P.ep.bias && (reinterpret_cast<uintptr_t>(P.ep.bias) & 15) == 0 && col0 + 32 <= P.n;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (bias_vec) {
            b = __ldg(reinterpret_cast<const float4*>(P.ep.bias + col0 + 4 * g));
        } else if (with_bias && P.ep.bias) {
            const uint32_t c = col0 + 4 * g;
            b = make_float4(c < P.n ? P.ep.bias[c] : 0.f, c + 1 < P.n ? P.ep.bias[c + 1] : 0.f,
                            c + 2 < P.n ? P.ep.bias[c + 2] : 0.f, c + 3 < P.n ? P.ep.bias[c + 3] : 0.f);
        }
        const float4 v = act4(make_float4(acc[4 * g] + b.x, acc[4 * g + 1] + b.y, acc[4 * g + 2] + b.z, acc[4 * g + 3] + b.w),
                              P.ep.activation);
        row[(g ^ lane) & 7] = v;     // 16-byte chunk g of row r sits at g ^ (r & 7)
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
        if (store)   // split-K: a partial sum of its own, added to the residual later in a fixed order
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                         ::"l"(map_out), "r"((int32_t)col0), "r"((int32_t)row_out), "r"(smem_u32(stage)) : "memory");
        else
            asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                         ::"l"(map_out), "r"((int32_t)col0), "r"((int32_t)row0), "r"(smem_u32(stage)) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
}

// bf16 destinations through TMA: bias / activation / SwiGLU and the conversion happen on the accumulator row the lane
// already holds; the 32-row block of bf16 goes into the warp's buffer in the swizzled layout of the store box (64-byte
// rows, or 32-byte rows after SwiGLU) and one bulk tensor store writes it: no read-back pass, no per-lane stores.
// The QKV routing stores a block either into q or, as rows pos + t of one session, into the K or V cache (blocks of
// 32 rows never straddle sessions: the host checks chunk % 32 == 0).
template <int MODE>
__device__ __forceinline__ void epilogue_block_store(const EpiParams& P, const CUtensorMap* map_out, const CUtensorMap* map_k,
                                                     const CUtensorMap* map_v, float* stage, uint32_t row0, uint32_t col0,
                                                     const float* acc, uint32_t lane, uint32_t parity, uint32_t qkv_pos) {
    // the 4 KB buffer holds two blocks; the store of the block before last must have been read out of its half
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    __syncwarp();
    stage += (parity & 1u) * 512;   // floats: 2 KB halves
    float b[32];
    if (P.ep.bias && (reinterpret_cast<uintptr_t>(P.ep.bias) & 15) == 0 && col0 + 32 <= P.n) {
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(P.ep.bias + col0 + 4 * g));
            b[4 * g] = t.x; b[4 * g + 1] = t.y; b[4 * g + 2] = t.z; b[4 * g + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) b[i] = (P.ep.bias && col0 + i < P.n) ? P.ep.bias[col0 + i] : 0.0f;
    }
    uint4* st = reinterpret_cast<uint4*>(stage);
    const uint32_t sm = smem_u32(stage);
    if (MODE == GEMM_SWIGLU) {
        uint32_t p[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            p[j] = pack_bf16x2(fast_silu(acc[2 * j] + b[2 * j]) * (acc[16 + 2 * j] + b[16 + 2 * j]),
                               fast_silu(acc[2 * j + 1] + b[2 * j + 1]) * (acc[17 + 2 * j] + b[17 + 2 * j]));
        // 32-byte rows, 32-byte swizzle: 16-byte chunk c of row r at c ^ ((r >> 2) & 1)
        st[lane * 2 + (0 ^ ((lane >> 2) & 1))] = make_uint4(p[0], p[1], p[2], p[3]);
        st[lane * 2 + (1 ^ ((lane >> 2) & 1))] = make_uint4(p[4], p[5], p[6], p[7]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                         ::"l"(map_out), "r"((int32_t)(col0 / 2)), "r"((int32_t)row0), "r"(sm) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        return;
    }
    const int act = MODE == GEMM_QKV ? ACT_NONE : P.ep.activation;
    uint32_t p[16];
#pragma unroll
    for (int j = 0; j < 16; ++j)
        p[j] = pack_bf16x2(apply_activation(acc[2 * j] + b[2 * j], act), apply_activation(acc[2 * j + 1] + b[2 * j + 1], act));
    // 64-byte rows, 64-byte swizzle: 16-byte chunk c of row r at c ^ ((r >> 1) & 3)
#pragma unroll
    for (uint32_t c = 0; c < 4; ++c)
        st[lane * 4 + (c ^ ((lane >> 1) & 3))] = make_uint4(p[4 * c], p[4 * c + 1], p[4 * c + 2], p[4 * c + 3]);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
        if (MODE == GEMM_QKV && col0 >= P.qkv.d) {
            const uint32_t which = col0 / P.qkv.d, c = col0 % P.qkv.d;
            const uint32_t pos = qkv_pos;   // read once per warp, not once per block: a dependent global load on the store's path
            const uint32_t session = row0 / P.qkv.chunk, t0 = row0 % P.qkv.chunk;
            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                         ::"l"(which == 1 ? map_k : map_v), "r"((int32_t)c), "r"((int32_t)(pos + t0)), "r"((int32_t)session), "r"(sm)
                         : "memory");
        } else {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                         ::"l"(map_out), "r"((int32_t)col0), "r"((int32_t)row0), "r"(sm) : "memory");
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
}

// `pre` (optional): residual values already fetched with load_residual_block for this very block.
template <int MODE>
__device__ __forceinline__ void epilogue_block(const EpiParams& P, float* stage, uint32_t row0, uint32_t col0,
                                               const float* acc, uint32_t lane, const float4* pre = nullptr) {
    if (row0 >= P.m || col0 >= P.n) return;  // warp-uniform
#pragma unroll
    for (int g = 0; g < 8; ++g)
        *reinterpret_cast<float4*>(stage + stage_index(lane, 4 * g)) = make_float4(acc[4 * g], acc[4 * g + 1], acc[4 * g + 2], acc[4 * g + 3]);
    __syncwarp();
    const uint32_t rows = min(32u, P.m - row0);
    // the vector paths need the whole 32-column block inside the matrix and a 16-byte aligned bias (if any)
    const bool full_cols = col0 + 32 <= P.n && (reinterpret_cast<uintptr_t>(P.ep.bias) & 15) == 0;
    if (MODE == GEMM_SWIGLU) {
        // columns [0,16) are gate, [16,32) the matching up columns.  A lane makes 4 outputs of one row:
        // 4 lanes per row, 8 rows per step.
        const uint32_t j = lane & 3, rsub = lane >> 2;
        bf16* out = reinterpret_cast<bf16*>(P.out);
        if (full_cols && P.ldc % 4 == 0 && (reinterpret_cast<uintptr_t>(out) & 7) == 0) {
            float4 bg = make_float4(0.f, 0.f, 0.f, 0.f), bu = bg;
            if (P.ep.bias) {
                bg = __ldg(reinterpret_cast<const float4*>(P.ep.bias + col0 + 4 * j));
                bu = __ldg(reinterpret_cast<const float4*>(P.ep.bias + col0 + 16 + 4 * j));
            }
            const uint32_t ocol = col0 / 2 + 4 * j;
#pragma unroll
            for (uint32_t it = 0; it < 4; ++it) {
                const uint32_t rr = it * 8 + rsub;
                if (rr < rows) {
                    const float4 g = stage_load4(stage, rr, 4 * j), u = stage_load4(stage, rr, 16 + 4 * j);
                    const uint2 o = make_uint2(pack_bf16x2(fast_silu(g.x + bg.x) * (u.x + bu.x), fast_silu(g.y + bg.y) * (u.y + bu.y)),
                                               pack_bf16x2(fast_silu(g.z + bg.z) * (u.z + bu.z), fast_silu(g.w + bg.w) * (u.w + bu.w)));
                    *reinterpret_cast<uint2*>(out + (size_t)(row0 + rr) * P.ldc + ocol) = o;
                }
            }
        } else {
            const uint32_t oc = lane & 15, half = lane >> 4;
            for (uint32_t rr = half; rr < rows; rr += 2)
                if (col0 + 16 + oc < P.n)
                    store_swiglu(P, row0 + rr, col0 + oc, col0 / 2 + oc, stage[stage_index(rr, oc)], stage[stage_index(rr, 16 + oc)]);
        }
    } else if (MODE == GEMM_QKV || P.ep.out_dtype == TNSR_B200_BF16) {
        // bf16 destinations: a lane converts 8 columns of one row (one 16-byte store): 4 lanes per row, 8 rows per step
        const uint32_t cg = lane & 3, rsub = lane >> 2, c8 = 8 * cg;
        bool fast = full_cols;
        bf16* base = reinterpret_cast<bf16*>(P.out);
        uint32_t ld = P.ldc, cbase = col0;
        uint32_t which = 0, pos = 0;
        if (MODE == GEMM_QKV) {
            const uint32_t d = P.qkv.d;
            fast = fast && d % 32 == 0;
            which = col0 / d;
            cbase = col0 % d;
            ld = d;
            base = which == 0 ? P.qkv.q : (which == 1 ? P.qkv.k_cache : P.qkv.v_cache);
            pos = (P.qkv.d_position && !P.qkv.position_stride) ? *P.qkv.d_position : P.qkv.position;
        }
        fast = fast && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0;
        if (fast) {
            float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
            if (P.ep.bias) {
                b0 = __ldg(reinterpret_cast<const float4*>(P.ep.bias + col0 + c8));
                b1 = __ldg(reinterpret_cast<const float4*>(P.ep.bias + col0 + c8 + 4));
            }
            const int act = MODE == GEMM_QKV ? ACT_NONE : P.ep.activation;
#pragma unroll
            for (uint32_t it = 0; it < 4; ++it) {
                const uint32_t rr = it * 8 + rsub;
                if (rr < rows) {
                    float4 v0 = stage_load4(stage, rr, c8), v1 = stage_load4(stage, rr, c8 + 4);
                    v0 = act4(make_float4(v0.x + b0.x, v0.y + b0.y, v0.z + b0.z, v0.w + b0.w), act);
                    v1 = act4(make_float4(v1.x + b1.x, v1.y + b1.y, v1.z + b1.z, v1.w + b1.w), act);
                    const uint32_t row = row0 + rr;
                    size_t orow;
                    if (MODE == GEMM_QKV) {
                        const uint32_t session = row / P.qkv.chunk;
                        const uint32_t p = P.qkv.position_stride ? P.qkv.d_position[session] : pos;   // ragged: one position per session
                        orow = which == 0 ? row : kv_row(P.qkv.paging, session, p + row % P.qkv.chunk, P.qkv.capacity);
                    }
                    else orow = map_out_row(P.ep, row);
                    *reinterpret_cast<uint4*>(base + orow * ld + cbase + c8) =
                        make_uint4(pack_bf16x2(v0.x, v0.y), pack_bf16x2(v0.z, v0.w), pack_bf16x2(v1.x, v1.y), pack_bf16x2(v1.z, v1.w));
                }
            }
        } else {
            for (uint32_t rr = 0; rr < rows; ++rr) {
                if (col0 + lane >= P.n) continue;
                if (MODE == GEMM_QKV) store_qkv(P, row0 + rr, col0 + lane, stage[stage_index(rr, lane)]);
                else store_plain(P, row0 + rr, col0 + lane, stage[stage_index(rr, lane)]);
            }
        }
    } else {
        // f32 output (+ optional residual): a lane owns 4 columns of one row (16 bytes): 8 lanes per row, 4 rows per step.
        // The residual may be the output buffer itself (the residual stream is updated in place), so all residual
        // rows are fetched before the first store.
        float* out = reinterpret_cast<float*>(P.out);
        const float* res = P.ep.residual;
        const uint32_t c4 = 4 * (lane & 7), rsub = lane >> 3;
        if (f32_vector_path(P, col0)) {
            float4 r4[8];
            if (pre) {
#pragma unroll
                for (uint32_t it = 0; it < 8; ++it) r4[it] = pre[it];
            } else {
                load_residual_block(P, row0, col0, lane, r4);
            }
            float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (P.ep.bias) bv = __ldg(reinterpret_cast<const float4*>(P.ep.bias + col0 + c4));
#pragma unroll
            for (uint32_t it = 0; it < 8; ++it) {
                const uint32_t rr = it * 4 + rsub;
                if (rr < rows) {
                    float4 v = stage_load4(stage, rr, c4);
                    v = act4(make_float4(v.x + bv.x, v.y + bv.y, v.z + bv.z, v.w + bv.w), P.ep.activation);
                    v = make_float4(v.x + r4[it].x, v.y + r4[it].y, v.z + r4[it].z, v.w + r4[it].w);
                    *reinterpret_cast<float4*>(out + map_out_row(P.ep, row0 + rr) * P.ldc + col0 + c4) = v;
                }
            }
        } else {
            const uint32_t col = col0 + lane;
            const bool col_ok = col < P.n;
            float rv[32];
#pragma unroll
            for (int rr = 0; rr < 32; ++rr)
                rv[rr] = (res && col_ok && (uint32_t)rr < rows) ? res[(size_t)(row0 + rr) * P.ep.ldr + col] : 0.0f;
            const float bv = (P.ep.bias && col_ok) ? __ldg(P.ep.bias + col) : 0.0f;
#pragma unroll
            for (int rr = 0; rr < 32; ++rr)
                if (col_ok && (uint32_t)rr < rows)
                    out[map_out_row(P.ep, row0 + rr) * P.ldc + col] = apply_activation(stage[stage_index(rr, lane)] + bv, P.ep.activation) + rv[rr];
        }
    }
    __syncwarp();  // the buffer is reused by the next block
}

template <int BN, int MODE, int EPI>
__global__ void __launch_bounds__(64 + 32 * EPI, EPI == 4 ? 3 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, TcParams prm) {
    using S = TcShape<BN, EPI>;
    constexpr int PER_QUARTER = EPI / 4;             // epilogue warps per TMEM lane quarter
    constexpr uint32_t CHUNK_STRIDE = 32 * PER_QUARTER;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte-swizzled tiles want a 1024-byte aligned base
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    float* stage_tiles = reinterpret_cast<float*>(smem + S::STAGES * S::STAGE_BYTES);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::STAGES * S::STAGE_BYTES + EPI * TC_STAGE_TILE_BYTES);
    uint64_t* empty_bar = full_bar + S::STAGES;
    uint64_t* acc_full = empty_bar + S::STAGES;   // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t split = (MODE == GEMM_PLAIN && prm.tma_reduce == 2) ? prm.split_k : 1u;
    const uint32_t num_tiles = prm.tiles_m * prm.tiles_n * split;
    const uint32_t num_kb = (prm.k + BK - 1) / BK;
    const uint32_t kb_per = (num_kb + split - 1) / split;    // the host picks split so that no range is empty

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(acc_full + s, 1); mbar_init(acc_empty + s, EPI); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // everything above touches only this CTA's shared memory; from here on the previous kernel must be done
    pdl_wait();
    pdl_trigger();
    if (warp == 1) {
        tmem_alloc(tmem_slot, S::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                uint32_t tm, tn;
                tile_coords(split == 1 ? tile : tile / split, prm.tiles_m, prm.tiles_n, tm, tn);
                const uint32_t kb0 = split == 1 ? 0u : (tile % split) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
                for (uint32_t kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, prm.wait_limit_ns)) { ok = false; break; }
                    uint8_t* sa = smem + stage * S::STAGE_BYTES;
                    const bool lost = prm.lose_kb && blockIdx.x == 0 && tile == blockIdx.x && kb + 1 == prm.lose_kb;
                    if (!lost) {   // a lost stage is never filled: its full barrier stays where it is
                        mbar_expect_tx(full_bar + stage, S::STAGE_BYTES);
                        tma_load_2d(sa, &map_a, (int32_t)(kb * BK), (int32_t)(tm * BM), full_bar + stage);
                        tma_load_2d(sa + S::A_BYTES, &map_b, (int32_t)(kb * BK), (int32_t)(tn * BN), full_bar + stage);
                    }
                    if (++stage == S::STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_bf16(BN);
            uint32_t stage = 0, phase = 0, it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
                const uint32_t ab = it & 1, aphase = (it >> 1) & 1;
                if (!mbar_wait(acc_empty + ab, aphase ^ 1, abort_flag, prm.wait_limit_ns)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + ab * BN;
                const uint32_t kb0 = split == 1 ? 0u : (tile % split) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
                for (uint32_t kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(full_bar + stage, phase, abort_flag, prm.wait_limit_ns)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
                    const uint64_t adesc = make_kmajor_sw128_desc(sa);
                    const uint64_t bdesc = make_kmajor_sw128_desc(sa + S::A_BYTES);
#pragma unroll
                    for (uint32_t kk = 0; kk < BK / UMMA_K; ++kk) {
                        // advancing K by 16 elements = 32 bytes inside the swizzle row: +2 in the address field
                        umma_bf16(d_tmem, adesc + kk * 2, bdesc + kk * 2, idesc, ((kb - kb0) | kk) != 0);
                    }
                    umma_commit(empty_bar + stage);  // stage reusable once these MMAs have read it
                    if (++stage == S::STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(acc_full + ab);
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        // TMEM lane quarter = warp % 4 (a warp may only read its own quarter); the warps of a quarter take the
        // 32-column chunks in turn (`half` = this warp's place among them).
        const uint32_t quarter = warp & 3, half = (warp - 2) >> 2;
        float* stage = stage_tiles + (warp - 2) * (TC_STAGE_TILE_BYTES / 4);
        uint32_t it = 0, store_parity = 0;
        const uint32_t qkv_pos = (MODE == GEMM_QKV && prm.tma_store)
                                     ? (prm.epi.qkv.d_position ? *prm.epi.qkv.d_position : prm.epi.qkv.position) : 0u;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
            const uint32_t ab = it & 1, aphase = (it >> 1) & 1;
            uint32_t tm, tn;
            tile_coords(split == 1 ? tile : tile / split, prm.tiles_m, prm.tiles_n, tm, tn);
            const uint32_t ks = split == 1 ? 0u : tile % split;
            const uint32_t row0 = tm * BM + quarter * 32;
            // f32 output with a residual: fetch this warp's first block of residual rows while the tile is still
            // being accumulated (the rows are final: only this warp rewrites them, after this read)
            float4 res_pre[8];
            bool have_pre = false;
            const bool reduce = MODE == GEMM_PLAIN && prm.tma_reduce;
            if (!reduce && MODE == GEMM_PLAIN && prm.epi.ep.out_dtype == TNSR_B200_F32 && prm.epi.ep.residual && half * 32 < (uint32_t)BN) {
                const uint32_t col0 = tn * BN + half * 32;
                if (row0 < prm.epi.m && col0 < prm.epi.n && f32_vector_path(prm.epi, col0)) {
                    load_residual_block(prm.epi, row0, col0, lane, res_pre);
                    have_pre = true;
                }
            }
            // what the epilogue reads besides the accumulator (the tile's bias columns, the step's position) is asked into
            // L1 while the tile is still being accumulated: a first-touch load after the wait is a whole L2 round trip
            // on the critical path of a one-tile launch (with many tiles per CTA the loads hit anyway: not done there)
            if (MODE != GEMM_ARGMAX && num_tiles <= gridDim.x) {
                const float* bias0 = prm.epi.ep.bias ? prm.epi.ep.bias + (size_t)tn * BN : nullptr;
                if (bias0 && lane * 32 < (uint32_t)BN && tn * BN + lane * 32 < prm.epi.n)
                    asm volatile("prefetch.global.L1 [%0];" ::"l"(bias0 + lane * 32));
                if (MODE == GEMM_QKV && lane == 31 && prm.epi.qkv.d_position)
                    asm volatile("prefetch.global.L1 [%0];" ::"l"(prm.epi.qkv.d_position));
            }
            if (!mbar_wait(acc_full + ab, aphase, abort_flag, prm.wait_limit_ns)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + ab * BN;
            if (MODE == GEMM_ARGMAX) {
                // no matrix leaves the kernel: every lane scans its own row; the first warp of the quarter does all chunks
                if (half == 0) {
                    int best = 0;
                    uint32_t best_i = 0;
                    bool have = false;
#pragma unroll 1
                    for (uint32_t c = 0; c < BN; c += 32) {
                        float acc[32];
                        tmem_ld32(taddr + c, acc);
                        tmem_ld_wait();
                        const uint32_t col0 = tn * BN + c;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int key = total_order_key(acc[i]);
                            if (col0 + i < prm.epi.n && (!have || key >= best)) { best = key; best_i = col0 + i; have = true; }
                        }
                    }
                    if (row0 + lane < prm.epi.m)
                        reinterpret_cast<uint2*>(prm.epi.out)[(size_t)(row0 + lane) * prm.epi.ldc + tn] = make_uint2((uint32_t)best, best_i);
                }
            } else {
#pragma unroll 1
                for (uint32_t c = half * 32; c < BN; c += CHUNK_STRIDE) {
                    float acc[32];
                    tmem_ld32(taddr + c, acc);
                    tmem_ld_wait();
                    const uint32_t col0 = tn * BN + c;
                    if (reduce) {
                        if (row0 < prm.epi.m && col0 < prm.epi.n)
                            epilogue_block_reduce(prm.epi, &map_out, stage, row0, col0, acc, lane, prm.tma_reduce == 2, ks == 0,
                                                  ks * prm.split_rows + row0);
                    } else if (prm.tma_store) {
                        if (row0 < prm.epi.m && col0 < prm.epi.n)
                            epilogue_block_store<MODE>(prm.epi, &map_out, &map_k, &map_v, stage, row0, col0, acc, lane, store_parity++, qkv_pos);
                    } else {
                        epilogue_block<MODE>(prm.epi, stage, row0, col0, acc, lane, (have_pre && c == half * 32) ? res_pre : nullptr);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + ab);
        }
        // bulk reduce operations of this warp must be complete before the CTA gives up its shared memory
        if (((MODE == GEMM_PLAIN && prm.tma_reduce) || prm.tma_store) && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // give copies that are still in flight time to land before the CTA's shared memory is released
        const uint64_t start = global_timer_ns();
        while (global_timer_ns() - start < 200000ull) __nanosleep(1000);
        if (threadIdx.x == 0 && prm.d_status) atomicCAS(prm.d_status, DEV_OK, DEV_TIMEOUT);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, S::TMEM_COLS);
    }
}

// ---- host: tensor maps ---------------------------------------------------------

// [rows, cols] bf16 row-major with `ld` elements between rows; box = 64 columns x box_rows rows.
static bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

template <int BN, int MODE, int EPI>
static int launch_tc_e(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap* mo, const TcParams& prm, cudaStream_t stream) {
    using S = TcShape<BN, EPI>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM_BYTES) != cudaSuccess)
            return check_launch("gemm_tc attribute");
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    uint32_t tiles = prm.tiles_m * prm.tiles_n * (prm.tma_reduce == 2 ? prm.split_k : 1u);
    uint32_t grid = tiles < (uint32_t)sm_count() ? tiles : (uint32_t)sm_count();
    launch_kernel(gemm_tc_kernel<BN, MODE, EPI>, dim3(grid), dim3(S::THREADS), S::SMEM_BYTES, stream, ma, mb, mo[0], mo[1], mo[2], prm);
    count_launch();
    return check_launch("gemm_tc");
}

// Wide tiles with a bf16 epilogue (QKV routing, SwiGLU) and a short K: the main loop of a K = 768 tile is shorter than
// 8 warps need to drain the previous accumulator, so these run 16 epilogue warps (and 3 ring stages instead of 4, which
// is why longer K keeps 8: there the deeper ring is worth more).
template <int BN, int MODE>
static int launch_tc_t(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap* mo, const TcParams& prm, cudaStream_t stream) {
    if (BN == 256 && (MODE == GEMM_QKV || MODE == GEMM_SWIGLU) && prm.k <= 1024)
        return launch_tc_e<BN, MODE, (BN == 256 && (MODE == GEMM_QKV || MODE == GEMM_SWIGLU)) ? 16 : 8>(ma, mb, mo, prm, stream);
    // narrow tiles: one epilogue warp per TMEM lane quarter is all a 32- or 64-column tile can use
    if (BN <= 64 && MODE != GEMM_ARGMAX) return launch_tc_e<BN, MODE, BN <= 64 ? 4 : 8>(ma, mb, mo, prm, stream);
    return launch_tc_e<BN, MODE, 8>(ma, mb, mo, prm, stream);
}

template <int BN>
static int launch_tc_mode(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap* mo, const TcParams& prm, GemmMode mode, cudaStream_t stream) {
    switch (mode) {
        case GEMM_PLAIN: return launch_tc_t<BN, GEMM_PLAIN>(ma, mb, mo, prm, stream);
        case GEMM_QKV: return launch_tc_t<BN, GEMM_QKV>(ma, mb, mo, prm, stream);
        case GEMM_SWIGLU: return launch_tc_t<BN, GEMM_SWIGLU>(ma, mb, mo, prm, stream);
        case GEMM_ARGMAX: return launch_tc_t<BN, GEMM_ARGMAX>(ma, mb, mo, prm, stream);
    }
    return TNSR_B200_ERR_INVALID_ARGUMENT;
}

static bool tc_eligible(const bf16* a, uint32_t lda, const bf16* bt, uint32_t k) {
    return k % 8 == 0 && lda % 8 == 0 && (reinterpret_cast<uintptr_t>(a) % 16 == 0) &&
           (reinterpret_cast<uintptr_t>(bt) % 16 == 0) && encode_fn() != nullptr;
}

// Shared body of the public launchers.  `tiles_n_out` (optional) receives the number of column
// tiles the chosen engine used, which GEMM_ARGMAX callers need to read the candidates back.
static int launch_gemm_impl(const bf16* a, const bf16* bt, void* out, uint32_t ldc, uint32_t m, uint32_t n, uint32_t k,
                            GemmMode mode, const GemmEpilogue& ep, const GemmQkvTargets* qkv, int* d_status,
                            uint32_t* tiles_n_out, cudaStream_t stream) {
    if (m == 0 || n == 0) return TNSR_B200_OK;
    if (k == 0) return TNSR_B200_ERR_INVALID_ARGUMENT;
    if (mode == GEMM_QKV && (!qkv || qkv->d == 0 || n != 3 * qkv->d || qkv->chunk == 0)) return TNSR_B200_ERR_INVALID_ARGUMENT;
    if (mode == GEMM_SWIGLU && n % 32 != 0) {
        set_thread_error("gemm: packed SwiGLU width must be a multiple of 32");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    if (ep.residual && ep.out_dtype != TNSR_B200_F32) return TNSR_B200_ERR_INVALID_ARGUMENT;
    EpiParams P;
    P.ep = ep;
    if (qkv) P.qkv = *qkv;
    P.out = out;
    P.ldc = ldc;
    P.m = m;
    P.n = n;
    const uint32_t lda = k;
    const bool can_tc = tc_eligible(a, lda, bt, k);
    auto simple = [&]() {
        if (mode == GEMM_ARGMAX) P.ldc = ceil_div(n, SB);
        if (tiles_n_out) *tiles_n_out = ceil_div(n, SB);
        return launch_simple(a, lda, bt, P, k, mode, stream);
    };
    if (g_gemm_engine == 1 || !can_tc) {
        if (ep.split_k > 1) {
            set_thread_error("gemm: split-K needs the tcgen05 engine");
            return TNSR_B200_ERR_INVALID_ARGUMENT;
        }
        if (g_gemm_engine == 2) {
            set_thread_error("gemm: shape or alignment outside the tcgen05 engine (k % 8, 16-byte pointers)");
            return TNSR_B200_ERR_UNSUPPORTED;
        }
        return simple();
    }
    const bool split_req = ep.split_k > 1;
    if (split_req) {
        // the caller planned with gemm_split_k(): anything that engine cannot honour is an error, not a silent fallback,
        // because the caller will add the partial sums it expects to find
        const bool form = mode == GEMM_PLAIN && ep.out_dtype == TNSR_B200_F32 && ep.residual && ep.residual == out && ep.ldr == ldc &&
                          ep.rows_per_session == 0 && !ep.round_bf16 && ep.activation == ACT_NONE && ldc % 4 == 0 && ep.split_partials &&
                          reinterpret_cast<uintptr_t>(ep.split_partials) % 16 == 0 && ep.split_rows % 32 == 0 && ep.split_rows >= m &&
                          ep.split_k == gemm_split_k(a, bt, m, n, k);
        if (!form) {
            set_thread_error("gemm: split-K asked for a form or a count the engine does not split");
            return TNSR_B200_ERR_INVALID_ARGUMENT;
        }
    }
    // A handful of rows against a large weight matrix: stream the weights with the operands swapped (gemm_skinny.cu)
    // when that engine can fill the GPU, i.e. with split-K scratch lent by the caller or with at least half as many
    // 128-column tiles as SMs.  Measured inside a CUDA graph, 4096 x 4096 weights: 14.8 / 16.3 us at 1 / 8 rows against
    // 28 us for the engine below; at 64 rows (33.6 against 21.5 us) and for the small matrices of a decode step (the
    // split-K hand-over through L2 costs more than it saves) the engine below is the faster one.
    // Engine 3 (tests) takes it for every eligible shape up to 64 rows.
    // Up to 16 rows against at least 4 M weight elements: one pass over the weights with no split-K (gemm_stream.cu).
    // Engine 4 (tests) takes it for every eligible shape.
    if (!split_req && mode == GEMM_PLAIN && m <= 16 && (g_gemm_engine == 0 || g_gemm_engine == 4) && gemm_stream_eligible(a, bt, m, n, k, ep) &&
        ((uint64_t)n * k >= (4ull << 20) || g_gemm_engine == 4))
        return launch_gemm_stream(a, bt, out, ldc, m, n, k, ep, d_status, stream);
    if (!split_req && mode == GEMM_PLAIN && m <= 64 && g_gemm_engine != 1 && gemm_skinny_eligible(a, bt, m, n, k, ep)) {
        const bool pays = m <= 16 && (uint64_t)n * k >= (4ull << 20) &&
                          ((ep.skinny_ws && ep.skinny_ws_bytes >= gemm_skinny_workspace_bytes()) ||
                           2 * ceil_div(n, 128u) >= (uint32_t)sm_count());
        if (pays || g_gemm_engine == 3)
            return launch_gemm_skinny(a, bt, out, ldc, m, n, k, ep, ep.skinny_ws, ep.skinny_ws_bytes, d_status, stream);
    }
    // tile width: the widest that still gives every SM a tile (32 at the narrowest)
    const uint32_t tiles_m = ceil_div(m, BM);
    uint32_t bn = 256;
    while (bn > 64 && (uint64_t)tiles_m * ceil_div(n, bn) < (uint64_t)sm_count()) bn >>= 1;
    if (bn == 64 && 2ull * tiles_m * ceil_div(n, 64) <= (uint64_t)sm_count()) bn = 32;  // very few tiles: halve once more
    if (split_req) bn = 32;   // many small tiles: every CTA takes in as little of both operands as possible
    TcParams prm;
    prm.k = k;
    prm.tiles_m = tiles_m;
    prm.tiles_n = ceil_div(n, bn);
    prm.split_k = 1;
    prm.split_rows = 0;
    prm.d_status = d_status;
    prm.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
    prm.lose_kb = t_lose_gemm_stage;   // one-shot test hook, see TcParams
    t_lose_gemm_stage = 0;
    CUtensorMap ma, mb;
    if (!make_map(&ma, a, m, k, lda, BM) || !make_map(&mb, bt, n, k, k, bn)) {
        if (g_gemm_engine == 2) {
            set_thread_error("gemm: tensor map encoding failed");
            return TNSR_B200_ERR_CUDA;
        }
        return simple();
    }
    if (mode == GEMM_ARGMAX) P.ldc = prm.tiles_n;
    if (tiles_n_out) *tiles_n_out = prm.tiles_n;
    // f32 result accumulated in place on the residual stream: let TMA do the read-add-write (see epilogue_block_reduce)
    CUtensorMap mo[3] = {ma, ma, ma};   // output map, K-cache map, V-cache map; placeholders when unused
    prm.tma_reduce = 0;
    prm.tma_store = 0;
    if (split_req) {
        EncodeTiledFn fn = encode_fn();
        cuuint64_t dims[2] = {n, (cuuint64_t)(ep.split_k - 1) * ep.split_rows + (uint64_t)ceil_div(m, 32u) * 32};
        cuuint64_t strides[1] = {(cuuint64_t)ldc * 4};
        cuuint32_t box[2] = {32, 32};
        cuuint32_t estr[2] = {1, 1};
        if (!fn || fn(&mo[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ep.split_partials, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            set_thread_error("gemm: tensor map encoding failed");
            return TNSR_B200_ERR_CUDA;
        }
        prm.tma_reduce = 2;
        prm.split_k = ep.split_k;
        prm.split_rows = ep.split_rows;
    } else if (mode == GEMM_PLAIN && ep.out_dtype == TNSR_B200_F32 && ep.residual && ep.residual == out && ep.ldr == ldc &&
        ep.rows_per_session == 0 && !ep.round_bf16 && ldc % 4 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
        EncodeTiledFn fn = encode_fn();
        cuuint64_t dims[2] = {n, m};
        cuuint64_t strides[1] = {(cuuint64_t)ldc * 4};
        cuuint32_t box[2] = {32, 32};
        cuuint32_t estr[2] = {1, 1};
        if (fn && fn(&mo[0], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
            prm.tma_reduce = 1;
        else
            mo[0] = ma;
    }
    // bf16 destinations: bulk tensor stores of 32-row blocks (see epilogue_block_store).  Measured: it pays where the
    // epilogue is the bottleneck and sixteen warps share the work -- the QKV and SwiGLU epilogues of wide tiles with a
    // short K (prefill 26.4 -> 25.8 ms) -- and costs 10 % on the plain bf16 epilogue with eight warps, which keeps
    // per-lane stores.
    if ((mode == GEMM_QKV || mode == GEMM_SWIGLU) && bn == 256 && k <= 1024 && ep.rows_per_session == 0 &&
        !ep.round_bf16) {
        EncodeTiledFn fn = encode_fn();
        auto bf16_map = [&](CUtensorMap* map, void* base, uint64_t cols, uint64_t rows, uint64_t ld, uint32_t box_cols,
                            CUtensorMapSwizzle swz) {
            if (!fn || !base || reinterpret_cast<uintptr_t>(base) % 16 != 0 || ld % 8 != 0) return false;
            cuuint64_t dims[2] = {cols, rows};
            cuuint64_t strides[1] = {ld * 2};
            cuuint32_t box[2] = {box_cols, 32};
            cuuint32_t estr[2] = {1, 1};
            return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      swz, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
        };
        bool okm = false;
        if (mode == GEMM_PLAIN) {
            okm = bf16_map(&mo[0], out, n, m, ldc, 32, CU_TENSOR_MAP_SWIZZLE_64B);
        } else if (mode == GEMM_SWIGLU) {
            okm = bf16_map(&mo[0], out, n / 2, m, ldc, 16, CU_TENSOR_MAP_SWIZZLE_32B);
        } else if (qkv && qkv->chunk % 32 == 0 && qkv->d % 32 == 0 && qkv->position_stride == 0 && m % qkv->chunk == 0 &&
                   !qkv->paging.table) {
            okm = bf16_map(&mo[0], qkv->q, qkv->d, m, qkv->d, 32, CU_TENSOR_MAP_SWIZZLE_64B);
            for (int which = 1; okm && which <= 2; ++which) {
                void* base = which == 1 ? (void*)qkv->k_cache : (void*)qkv->v_cache;
                if (!base || reinterpret_cast<uintptr_t>(base) % 16 != 0) { okm = false; break; }
                cuuint64_t dims[3] = {qkv->d, qkv->capacity, m / qkv->chunk};
                cuuint64_t strides[2] = {(cuuint64_t)qkv->d * 2, (cuuint64_t)qkv->capacity * qkv->d * 2};
                cuuint32_t box[3] = {32, 32, 1};
                cuuint32_t estr[3] = {1, 1, 1};
                okm = fn(&mo[which], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
            }
        }
        if (okm) prm.tma_store = 1;
        else mo[0] = mo[1] = mo[2] = ma;
    }
    prm.epi = P;
    switch (bn) {
        case 256: return launch_tc_mode<256>(ma, mb, mo, prm, mode, stream);
        case 128: return launch_tc_mode<128>(ma, mb, mo, prm, mode, stream);
        case 64: return launch_tc_mode<64>(ma, mb, mo, prm, mode, stream);
        default: return launch_tc_mode<32>(ma, mb, mo, prm, mode, stream);
    }
}

// Few rows against a narrow weight matrix (the attention-output and FFN-down projections of a decode step: 24 column
// tiles at d 768) leave most SMs without a tile while each of the others takes in its whole K extent at one SM's rate;
// dividing K puts the same bytes through four times as many SMs.
uint32_t gemm_split_k(const bf16* a, const bf16* bt, uint32_t m, uint32_t n, uint32_t k) {
    if (g_gemm_engine == 1 || !tc_eligible(a, k, bt, k)) return 0;
    if (m == 0 || m > 256 || k % BK != 0) return 0;
    if (m <= 64 && (uint64_t)n * k >= (4ull << 20)) return 0;   // the few-row engines take these shapes
    const uint32_t num_kb = k / BK, tiles_n = ceil_div(n, 32u);
    for (uint32_t s = 4; s >= 2; --s)
        if (num_kb % s == 0 && num_kb / s >= 2 && tiles_n * s <= (uint32_t)sm_count()) return s;
    return 0;
}

int launch_gemm_bf16(const bf16* a, const bf16* bt, void* out, uint32_t ldc, uint32_t m, uint32_t n,
                     uint32_t k, GemmMode mode, const GemmEpilogue& ep, const GemmQkvTargets* qkv,
                     int* d_status, cudaStream_t stream) {
    if (mode == GEMM_ARGMAX) return TNSR_B200_ERR_INVALID_ARGUMENT;  // use launch_lm_head_argmax
    return launch_gemm_impl(a, bt, out, ldc, m, n, k, mode, ep, qkv, d_status, nullptr, stream);
}

// ---- greedy ids from the LM head without materialising logits --------------------
// One warp per row folds the per-tile candidates; ties between tiles go to the larger index,
// which is the later tile, so the result is the last index of the row maximum.
__global__ void __launch_bounds__(128)
argmax_finish_kernel(const uint2* __restrict__ cand, uint32_t* __restrict__ ids, uint32_t rows, uint32_t tiles) {
    pdl_wait();
    pdl_trigger();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    int best = 0;
    uint32_t best_i = 0;
    bool have = false;
    for (uint32_t t = lane; t < tiles; t += 32) {
        const uint2 c = cand[(size_t)row * tiles + t];
        const int key = (int)c.x;
        if (!have || key > best || (key == best && c.y > best_i)) { best = key; best_i = c.y; have = true; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const int ok = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        const int oh = __shfl_xor_sync(0xffffffffu, (int)have, o);
        if (oh && (!have || ok > best || (ok == best && oi > best_i))) { best = ok; best_i = oi; have = true; }
    }
    if (lane == 0) ids[row] = best_i;
}

uint64_t lm_head_argmax_scratch_bytes(uint32_t rows, uint32_t n) { return (uint64_t)rows * ceil_div(n, 32) * sizeof(uint2); }

int launch_lm_head_argmax(const bf16* a, const bf16* bt, uint32_t m, uint32_t n, uint32_t k, void* candidates,
                          uint32_t* ids, int* d_status, cudaStream_t stream) {
    if (m == 0) return TNSR_B200_OK;
    if (n == 0 || !candidates || !ids) return TNSR_B200_ERR_INVALID_ARGUMENT;
    GemmEpilogue ep;
    uint32_t tiles = 0;
    int rc = launch_gemm_impl(a, bt, candidates, 0, m, n, k, GEMM_ARGMAX, ep, nullptr, d_status, &tiles, stream);
    if (rc) return rc;
    launch_kernel(argmax_finish_kernel, dim3(ceil_div(m, 4)), dim3(128), 0, stream, reinterpret_cast<const uint2*>(candidates), ids, m, tiles);
    count_launch();
    return check_launch("argmax_finish");
}

}  // namespace tb
