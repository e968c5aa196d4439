// bf16 GEMM for few rows (m <= 64: decode steps of small batches, the "skinny"
// shapes of the GEMM sweep): out[m, n] = act(a[m, k] . bt[n, k]^T + bias) (+ residual).
//
// With so few rows the job is to stream the weights once at HBM speed, so the
// operands swap places: 128 WEIGHT rows are the M side of tcgen05.mma (one TMEM lane
// per output column) and the activation rows, padded to 16 / 32 / 64, are its N side.
// The 16 KB weight tile of every k-block is then all payload (in the row-major
// arrangement a 128-row activation tile would be mostly padding), and the epilogue
// thread that owns TMEM lane l holds output column n0 + l for every row, so for a
// fixed row consecutive lanes write consecutive addresses.
//
// n / 128 tiles are too few CTAs to pull the whole HBM bandwidth, so when the caller
// lends scratch the K range of a tile is divided over `splits` CTAs (tiles x splits
// <= SMs).  Every split stores its f32 partial tile; the last one to arrive (a counter
// per tile and lane quarter) adds the partials in split order -- a fixed order, so the
// result does not depend on timing -- applies the epilogue and leaves the counter at
// zero for the next launch.
//
//   warp 0   TMA: weight tile [128 x 64] + activation tile [MP x 64] per k-block, 8 stages
//   warp 1   tcgen05.mma M128 x N(MP) x K16, accumulator in TMEM
//   warps 2-5 epilogue, one per TMEM lane quarter
//
// All waits are bounded (tc_common.cuh).
#include <algorithm>

#include "tc_common.cuh"

namespace tb {

constexpr int SK_ROWS = 128;     // weight rows per tile
constexpr int SK_BK = 64;
constexpr int SK_STAGES = 8;
constexpr int SK_THREADS = 192;
constexpr uint32_t SK_W_BYTES = SK_ROWS * SK_BK * 2;
constexpr uint32_t SK_MAX_SPLITS = 16;
constexpr uint32_t SK_COUNTER_BYTES = 8192;   // 4 counters per tile: up to 512 tiles with split-K

template <int MP>
struct SkShape {
    static constexpr uint32_t A_BYTES = MP * SK_BK * 2;
    static constexpr uint32_t STAGE_BYTES = SK_W_BYTES + A_BYTES;
    static constexpr uint32_t SMEM_BYTES = SK_STAGES * STAGE_BYTES + 1024 + 256;
    static constexpr uint32_t TMEM_COLS = MP < 32 ? 32 : MP;
    static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MP >> 3) << 17) | ((uint32_t)(SK_ROWS >> 4) << 24);
};

struct SkParams {
    const float* bias;
    const float* residual;
    uint32_t ldr;
    int activation, out_dtype;
    void* out;
    uint32_t ldc, m, n, k;
    uint32_t splits;
    const bf16* w;         // the weights again as a plain pointer, for the L2 prefetch
    float* partials;       // [tile][split][MP][128]
    uint32_t* counters;    // [tile][4]
    int* d_status;
    uint64_t wait_limit_ns;
};

__device__ __forceinline__ void sk_store(const SkParams& P, uint32_t row, uint32_t col, float acc) {
    float v = acc;
    if (P.bias) v += __ldg(P.bias + col);
    v = apply_activation(v, P.activation);
    if (P.out_dtype == TNSR_B200_BF16) {
        reinterpret_cast<bf16*>(P.out)[(size_t)row * P.ldc + col] = __float2bfloat16_rn(v);
    } else {
        if (P.residual) v += P.residual[(size_t)row * P.ldr + col];
        reinterpret_cast<float*>(P.out)[(size_t)row * P.ldc + col] = v;
    }
}

template <int MP>
__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, SkParams prm) {
    using S = SkShape<MP>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + SK_STAGES * S::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + SK_STAGES;
    uint64_t* acc_full = empty_bar + SK_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tile = blockIdx.x / prm.splits, split = blockIdx.x % prm.splits;
    const uint32_t num_kb = (prm.k + SK_BK - 1) / SK_BK;
    const uint32_t kb_begin = split * num_kb / prm.splits, kb_end = (split + 1) * num_kb / prm.splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SK_STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, 1); }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
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
        // A tiled copy touches 128 bytes of each of 128 weight rows, i.e. 128 DRAM pages per k-block and, over all CTAs,
        // far more open pages than HBM has banks.  So every lane first asks L2 to fetch its share of this CTA's weight
        // rows as long contiguous runs (the CTA's whole K range of a row at once); the tiled copies then find them in L2.
        {
            const uint32_t e0 = kb_begin * SK_BK, e1 = min(kb_end * SK_BK, prm.k);
            for (uint32_t r = lane; r < SK_ROWS; r += 32) {
                const uint32_t row = tile * SK_ROWS + r;
                if (row >= prm.n || e1 <= e0) continue;
                const char* p = reinterpret_cast<const char*>(prm.w + (size_t)row * prm.k + e0);
                uint32_t bytes = (e1 - e0) * 2;      // k % 8 == 0: a multiple of 16
                while (bytes) {
                    const uint32_t piece = bytes < 4096u ? bytes : 4096u;
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(piece) : "memory");
                    p += piece;
                    bytes -= piece;
                }
            }
        }
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            for (uint32_t kb = kb_begin; kb < kb_end; ++kb) {
                if (!mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, prm.wait_limit_ns)) break;
                uint8_t* sw = smem + stage * S::STAGE_BYTES;
                mbar_expect_tx(full_bar + stage, S::STAGE_BYTES);
                tma_load_2d(sw, &map_w, (int32_t)(kb * SK_BK), (int32_t)(tile * SK_ROWS), full_bar + stage);
                tma_load_2d(sw + SK_W_BYTES, &map_a, (int32_t)(kb * SK_BK), 0, full_bar + stage);
                if (++stage == SK_STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t kb = kb_begin; kb < kb_end; ++kb) {
                if (!mbar_wait(full_bar + stage, phase, abort_flag, prm.wait_limit_ns)) { ok = false; break; }
                tc_fence_after();
                const uint32_t sw = smem_u32(smem + stage * S::STAGE_BYTES);
                const uint64_t wdesc = make_kmajor_sw128_desc(sw);
                const uint64_t adesc = make_kmajor_sw128_desc(sw + SK_W_BYTES);
#pragma unroll
                for (uint32_t kk = 0; kk < SK_BK / 16; ++kk)
                    umma_bf16(tmem_base, wdesc + kk * 2, adesc + kk * 2, S::IDESC, ((kb - kb_begin) | kk) != 0);
                umma_commit(empty_bar + stage);
                if (++stage == SK_STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok) umma_commit(acc_full);
        }
    } else {
        // ---------------- epilogue: lane = output column, registers = rows ----------------
        const uint32_t quarter = warp & 3;
        const uint32_t col = tile * SK_ROWS + quarter * 32 + lane;
        if (kb_end > kb_begin ? mbar_wait(acc_full, 0, abort_flag, prm.wait_limit_ns) : true) {
            tc_fence_after();
            constexpr int LOADS = MP <= 32 ? 1 : MP / 32;
            float acc[LOADS * 32];
            if (kb_end > kb_begin) {
#pragma unroll
                for (int i = 0; i < LOADS; ++i) tmem_ld32(tmem_base + ((quarter * 32u) << 16) + i * 32, acc + i * 32);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < LOADS * 32; ++i) acc[i] = 0.0f;
            }
            const uint32_t rows = prm.m;   // <= MP
            if (prm.splits == 1) {
                if (col < prm.n) {
#pragma unroll
                    for (int j = 0; j < MP; ++j)
                        if ((uint32_t)j < rows) sk_store(prm, j, col, acc[j]);
                }
            } else {
                float* slots = prm.partials + (size_t)tile * prm.splits * MP * SK_ROWS + quarter * 32 + lane;
                const size_t slot_stride = (size_t)MP * SK_ROWS;
                float* mine = slots + split * slot_stride;
#pragma unroll
                for (int j = 0; j < MP; ++j)
                    if ((uint32_t)j < rows) __stcg(mine + j * SK_ROWS, acc[j]);
                __threadfence();
                __syncwarp();
                uint32_t* counter = prm.counters + tile * 4 + quarter;
                uint32_t arrived = 0;
                if (lane == 0) arrived = atomicAdd(counter, 1u);
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (arrived == prm.splits - 1) {
                    __threadfence();
                    if (col < prm.n) {
                        // split by split, all rows of a split in flight at once; per element the additions run in
                        // split order whoever arrived last
#pragma unroll
                        for (int j = 0; j < MP; ++j) acc[j] = (uint32_t)j < rows ? __ldcg(slots + j * SK_ROWS) : 0.0f;
                        for (uint32_t s = 1; s < prm.splits; ++s) {
                            float v[MP];
#pragma unroll
                            for (int j = 0; j < MP; ++j) v[j] = (uint32_t)j < rows ? __ldcg(slots + s * slot_stride + j * SK_ROWS) : 0.0f;
#pragma unroll
                            for (int j = 0; j < MP; ++j) acc[j] += v[j];
                        }
#pragma unroll
                        for (int j = 0; j < MP; ++j)
                            if ((uint32_t)j < rows) sk_store(prm, j, col, acc[j]);
                    }
                    if (lane == 0) *counter = 0;   // ready for the next launch
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
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

static bool sk_make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)SK_BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int sk_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// Scratch that serves every skinny GEMM: counters, then at most one [64 x 128] f32 partial tile per SM.
uint64_t gemm_skinny_workspace_bytes() { return SK_COUNTER_BYTES + (uint64_t)sk_sm_count() * 64 * SK_ROWS * 4; }

bool gemm_skinny_eligible(const bf16* a, const bf16* bt, uint32_t m, uint32_t n, uint32_t k, const GemmEpilogue& ep) {
    (void)n;
    return m >= 1 && m <= 64 && k % 8 == 0 && k >= 8 && ep.rows_per_session == 0 && !ep.round_bf16 &&
           reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(bt) % 16 == 0 && encode_fn() != nullptr;
}

template <int MP>
static int sk_launch(const CUtensorMap& mw, const CUtensorMap& ma, const SkParams& prm, uint32_t grid, cudaStream_t stream) {
    using S = SkShape<MP>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        if (cudaFuncSetAttribute(gemm_skinny_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM_BYTES) != cudaSuccess)
            return check_launch("gemm_skinny attribute");
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    launch_kernel(gemm_skinny_kernel<MP>, dim3(grid), dim3(SK_THREADS), (size_t)S::SMEM_BYTES, stream, mw, ma, prm);
    count_launch();
    return check_launch("gemm_skinny");
}

// `scratch` (optional, gemm_skinny_workspace_bytes(), zeroed once, 16-byte aligned) enables split-K.
int launch_gemm_skinny(const bf16* a, const bf16* bt, void* out, uint32_t ldc, uint32_t m, uint32_t n, uint32_t k,
                       const GemmEpilogue& ep, void* scratch, uint64_t scratch_bytes, int* d_status, cudaStream_t stream) {
    const uint32_t mp = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
    const uint32_t tiles = ceil_div(n, (uint32_t)SK_ROWS), num_kb = ceil_div(k, (uint32_t)SK_BK);
    SkParams prm;
    prm.bias = ep.bias;
    prm.residual = ep.residual;
    prm.ldr = ep.ldr;
    prm.activation = ep.activation;
    prm.out_dtype = ep.out_dtype;
    prm.out = out;
    prm.ldc = ldc;
    prm.m = m; prm.n = n; prm.k = k;
    prm.w = bt;
    prm.splits = 1;
    prm.partials = nullptr;
    prm.counters = nullptr;
    prm.d_status = d_status;
    prm.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
    if (scratch && reinterpret_cast<uintptr_t>(scratch) % 16 == 0 && scratch_bytes >= gemm_skinny_workspace_bytes() &&
        tiles < (uint32_t)sk_sm_count() && (uint64_t)tiles * 16 <= SK_COUNTER_BYTES) {
        uint32_t splits = std::min(std::min((uint32_t)sk_sm_count() / tiles, num_kb / 2), SK_MAX_SPLITS);
        if (splits > 1) {
            prm.splits = splits;
            prm.counters = reinterpret_cast<uint32_t*>(scratch);
            prm.partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + SK_COUNTER_BYTES);
        }
    }
    CUtensorMap mw, ma;
    if (!sk_make_map(&mw, bt, n, k, k, SK_ROWS) || !sk_make_map(&ma, a, m, k, k, mp)) {
        set_thread_error("skinny gemm: tensor map encoding failed");
        return TNSR_B200_ERR_CUDA;
    }
    const uint32_t grid = tiles * prm.splits;
    switch (mp) {
        case 16: return sk_launch<16>(mw, ma, prm, grid, stream);
        case 32: return sk_launch<32>(mw, ma, prm, grid, stream);
        default: return sk_launch<64>(mw, ma, prm, grid, stream);
    }
}

}  // namespace tb
