// Causal prefill attention on the 5th-generation tensor cores (tcgen05), head
// width 64, bf16 cache.  The job is the reference's `decoder_prefill_bf16`
// (src/nn/kv_cache/prefill.rs:170-607): `chunk` new queries per session attend
// keys 0 .. position + t of the cache that already holds their own rows.
//
// A work item = 128 queries of one (session, head); the accumulator row of a query
// is one TMEM lane.  Keys arrive in blocks of 128.  The CTAs are persistent: two per
// SM (about 100 KB of shared memory and 256 TMEM columns each, so one CTA's loads,
// softmax and hand-overs overlap the other's) walk the item list, longest items
// first, with TMEM and barriers set up once.
//
//   warp 0      TMA: per item the Q tile, then K and V blocks into a two-stage ring
//               (3-D tensor maps {width, live rows, sessions}: rows past
//               position + chunk read as zeros, so stale cache rows never meet
//               the arithmetic).
//   warp 1      one thread issues the MMAs: S_j = Q K_j^T (M128 N128 K64) into the
//               TMEM score buffer, O_j = P_j V_j (M128 N64 K128) into the TMEM
//               output buffer.  V is consumed where TMA put it, as an MN-major
//               operand -- no transpose pass.
//   warps 2-9   softmax, two threads per query row (a warp may only read its own
//               quarter of the TMEM lanes; the two warps of a quarter take 64 score
//               columns and 32 output columns each).  Per block: row maximum of the
//               own half, exchanged with the partner through shared memory; fold
//               O_{j-1} into the running output (rescaled by exp2(m_old - m_new));
//               exponentials as bf16 into the P tile in the K-major swizzled layout
//               the MMA reads.  Keys 0-63 of P_j go where K_j was (dead once S_j is
//               complete, not reloaded before P_j V_j is), keys 64-127 to a tile of
//               their own.
//
// Hand-overs (single-buffered, phase parity = running block count & 1; q_full / q_empty count items: the Q tile
// may be reloaded once the item's last S product is complete):
//   s_full   S_j complete                      MMA commit  -> softmax
//   pair     both halves of a row wrote their maximum      softmax <-> softmax (per lane quarter)
//   p_full   P_j written, S_j no longer needed softmax     -> MMA (issues S_{j+1}, then P_j V_j)
//   o_full   O_j complete, P_j no longer read  MMA commit  -> softmax (fold; then block j+1 may overwrite the
//                                                             upper P tile; the next P V overwrites O only after
//                                                             the following p_full, i.e. after the fold)
//
// Every wait is bounded; a wait that gives up raises the CTA's abort flag, the
// roles fall through to the common teardown and the status word is set.
#include <algorithm>

#include "tc_common.cuh"

namespace tb {

constexpr int PT_BQ = 128, PT_BK = 128, PT_HD = 64;
constexpr int PT_KV_STAGES = 2;
constexpr int PT_THREADS = 320;
constexpr uint32_t PT_TILE_BYTES = 128 * 128;         // 128 rows of 64 bf16
constexpr uint32_t PT_KV_BYTES = 2 * PT_TILE_BYTES;   // K block + V block
constexpr uint32_t PT_XM_BYTES = 2 * 2 * 128 * 4;     // row maxima: [block parity][half][row]
constexpr uint32_t PT_SMEM_BYTES = 1024 + PT_TILE_BYTES + PT_KV_STAGES * PT_KV_BYTES + PT_TILE_BYTES + PT_XM_BYTES + 256;
constexpr uint32_t PT_TMEM_COLS = 256;                // scores 128, outputs 64 (power of two)
constexpr uint32_t PT_O_COL = 128;

// kind::f16 instruction descriptors: f32 accumulator, bf16 operands, M = 128.
constexpr uint32_t PT_IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
// B operand (V) MN-major: bit 16
constexpr uint32_t PT_IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((64u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ float pt_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float pt_max4(const float* v) { return fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3])); }

struct PtParams {
    bf16* out;
    uint32_t chunk, position, heads, q_tiles, sessions;
    float scale_log2;
    int* d_status;
    uint64_t wait_limit_ns;
};

__global__ void __launch_bounds__(PT_THREADS, 2)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, PtParams prm) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint8_t* q_tile = smem;
    uint8_t* kv_ring = smem + PT_TILE_BYTES;
    uint8_t* p_upper = kv_ring + PT_KV_STAGES * PT_KV_BYTES;     // keys 64-127 of P
    float* xm = reinterpret_cast<float*>(p_upper + PT_TILE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_upper + PT_TILE_BYTES + PT_XM_BYTES);
    uint64_t* q_full = bars;                       // [1]
    uint64_t* kv_full = q_full + 1;                // [PT_KV_STAGES]
    uint64_t* kv_empty = kv_full + PT_KV_STAGES;   // [PT_KV_STAGES]
    uint64_t* s_full = kv_empty + PT_KV_STAGES;    // [1]
    uint64_t* p_full = s_full + 1;                 // [1]
    uint64_t* o_full = p_full + 1;                 // [1]
    uint64_t* pair = o_full + 1;                   // [4], one per lane quarter
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pair + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint64_t* q_empty = reinterpret_cast<uint64_t*>(tmem_slot + 2);   // [1]

    // Work items = (query tile, head, session), the longest query tiles (most key blocks) first; CTA c takes items
    // c, c + grid, c + 2 grid, ...  Every role walks the same list with the same counters, so the barrier phases
    // (a running count of key blocks for the K/V ring, S, P and O; a running count of items for Q) stay in step.
    const uint32_t per_tile = prm.heads * prm.sessions;
    const uint32_t total_items = prm.q_tiles * per_tile;
    auto item_coords = [&](uint32_t item, uint32_t& q0, uint32_t& h, uint32_t& s, uint32_t& n_blocks) {
        const uint32_t q_tile_index = prm.q_tiles - 1 - item / per_tile, rem = item % per_tile;
        q0 = q_tile_index * PT_BQ;
        h = rem % prm.heads;
        s = rem / prm.heads;
        const uint32_t last_q = min(q0 + PT_BQ, prm.chunk) - 1;
        const uint32_t total = prm.position + last_q + 1;          // keys visible to the tile's last query
        n_blocks = (total + PT_BK - 1) / PT_BK;
    };

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (int i = 0; i < PT_KV_STAGES; ++i) { mbar_init(kv_full + i, 1); mbar_init(kv_empty + i, 1); }
        mbar_init(s_full, 1);
        mbar_init(p_full, 8);
        mbar_init(o_full, 1);
        for (int i = 0; i < 4; ++i) mbar_init(pair + i, 2);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_wait();
    pdl_trigger();
    if (warp == 1) {
        tmem_alloc(tmem_slot, PT_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t g = 0, it = 0;     // key blocks and items so far
            bool ok = true;
            for (uint32_t item = blockIdx.x; ok && item < total_items; item += gridDim.x, ++it) {
                uint32_t q0, h, s, n_blocks;
                item_coords(item, q0, h, s, n_blocks);
                // the Q tile is free once every S product of the previous item has been computed
                if (it > 0 && !mbar_wait(q_empty, (it - 1) & 1, abort_flag, prm.wait_limit_ns)) break;
                mbar_expect_tx(q_full, PT_TILE_BYTES);
                tma_load_3d(q_tile, &map_q, (int32_t)(h * PT_HD), (int32_t)q0, (int32_t)s, q_full);
                for (uint32_t j = 0; j < n_blocks; ++j, ++g) {
                    const uint32_t stage = g % PT_KV_STAGES;
                    if (!mbar_wait(kv_empty + stage, ((g / PT_KV_STAGES) & 1) ^ 1, abort_flag, prm.wait_limit_ns)) { ok = false; break; }
                    uint8_t* dst = kv_ring + stage * PT_KV_BYTES;
                    mbar_expect_tx(kv_full + stage, PT_KV_BYTES);
                    tma_load_3d(dst, &map_k, (int32_t)(h * PT_HD), (int32_t)(j * PT_BK), (int32_t)s, kv_full + stage);
                    tma_load_3d(dst + PT_TILE_BYTES, &map_v, (int32_t)(h * PT_HD), (int32_t)(j * PT_BK), (int32_t)s, kv_full + stage);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint64_t qdesc = make_kmajor_sw128_desc(smem_u32(q_tile));
            // S = Q K^T for the block in ring slot `stage`: four K steps of 16 dims, +32 bytes inside the swizzle row each
            auto issue_s = [&](uint32_t stage) {
                const uint64_t kdesc = make_kmajor_sw128_desc(smem_u32(kv_ring + stage * PT_KV_BYTES));
#pragma unroll
                for (uint32_t kk = 0; kk < PT_HD / 16; ++kk) umma_bf16(tmem_base, qdesc + kk * 2, kdesc + kk * 2, PT_IDESC_S, kk != 0);
                umma_commit(s_full);
            };
            uint32_t g = 0, it = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; ok && item < total_items; item += gridDim.x, ++it) {
                uint32_t q0, h, s, n_blocks;
                item_coords(item, q0, h, s, n_blocks);
                if (!mbar_wait(q_full, it & 1, abort_flag, prm.wait_limit_ns)) break;
                if (!mbar_wait(kv_full + g % PT_KV_STAGES, (g / PT_KV_STAGES) & 1, abort_flag, prm.wait_limit_ns)) break;
                // the score buffer is free: its last reader signalled p_full of the previous block, which was waited for below
                tc_fence_after();
                issue_s(g % PT_KV_STAGES);
                if (n_blocks == 1) umma_commit(q_empty);
                for (uint32_t j = 0; j < n_blocks; ++j) {
                    const uint32_t b = g + j, stage = b % PT_KV_STAGES;
                    // P_j is in place and the softmax warps are done with S_j
                    if (!mbar_wait(p_full, b & 1, abort_flag, prm.wait_limit_ns)) { ok = false; break; }
                    if (j + 1 < n_blocks) {
                        const uint32_t next = (b + 1) % PT_KV_STAGES;
                        if (!mbar_wait(kv_full + next, ((b + 1) / PT_KV_STAGES) & 1, abort_flag, prm.wait_limit_ns)) { ok = false; break; }
                        tc_fence_after();
                        issue_s(next);
                        if (j + 2 == n_blocks) umma_commit(q_empty);   // that was the item's last S product
                    }
                    tc_fence_after();
                    // O_j = P_j V_j : eight K steps of 16 keys.  P: K-major, keys 0-63 in the K slot of this stage, keys
                    // 64-127 in the upper tile; V: MN-major, 16 keys = two 8-key groups 1024 bytes apart, so each step
                    // starts 2048 bytes further on.
                    const uint32_t p_lower = smem_u32(kv_ring + stage * PT_KV_BYTES);
                    const uint32_t v_addr = p_lower + PT_TILE_BYTES;
#pragma unroll
                    for (uint32_t kk = 0; kk < PT_BK / 16; ++kk) {
                        const uint64_t pdesc = make_kmajor_sw128_desc(kk < 4 ? p_lower : smem_u32(p_upper)) + (kk & 3) * 2;
                        const uint64_t vdesc = make_mnmajor_sw128_desc(v_addr + kk * 2048, PT_TILE_BYTES, 1024);
                        umma_bf16(tmem_base + PT_O_COL, pdesc, vdesc, PT_IDESC_O, kk != 0);
                    }
                    umma_commit(o_full);
                    umma_commit(kv_empty + stage);   // both products of this ring stage are done
                }
                g += n_blocks;
            }
        }
    } else {
        // ---------------- softmax warps: two threads per query row ----------------
        const uint32_t quarter = warp & 3, half = (warp - 2) >> 2;
        const uint32_t row = quarter * 32 + lane;
        const uint32_t lane_taddr = tmem_base + ((quarter * 32u) << 16);
        const float sl2 = prm.scale_log2;
        uint32_t pair_uses = 0, g = 0;
        bool ok = true;
        // Both threads of a row publish a value and read the partner's.
        auto exchange = [&](float mine, float& other) -> bool {
            float* slot = xm + (pair_uses & 1) * 256;
            slot[half * 128 + row] = mine;
            __syncwarp();
            if (lane == 0) mbar_arrive(pair + quarter);
            if (!mbar_wait(pair + quarter, pair_uses & 1, abort_flag, prm.wait_limit_ns)) return false;
            other = slot[(half ^ 1) * 128 + row];
            ++pair_uses;
            return true;
        };
        for (uint32_t item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
            uint32_t q0, h, s, n_blocks;
            item_coords(item, q0, h, s, n_blocks);
            const uint32_t q_idx = min(q0 + row, prm.chunk - 1);
            const uint32_t limit = prm.position + q_idx;             // last visible key of this row
            float acc[32];                                           // output columns [32 half, 32 half + 32)
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
            float m = -INFINITY, l = 0.0f, corr_pending = 0.0f;      // l: sum over this thread's key columns only
            // acc = acc * corr + O_b  (this thread's 32 outputs of block b, b counted over all items)
            auto fold = [&](uint32_t b, float corr) -> bool {
                if (!mbar_wait(o_full, b & 1, abort_flag, prm.wait_limit_ns)) return false;
                tc_fence_after();
                float v[32];
                tmem_ld32(lane_taddr + PT_O_COL + half * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] = fmaf(acc[i], corr, v[i]);
                return true;
            };

            for (uint32_t j = 0; j < n_blocks; ++j) {
                const uint32_t b = g + j;
                if (!mbar_wait(s_full, b & 1, abort_flag, prm.wait_limit_ns)) { ok = false; break; }
                tc_fence_after();
                const uint32_t taddr = lane_taddr + half * 64;
                const uint32_t kbase = j * PT_BK + half * 64;           // first key of this thread's columns
                const bool need_mask = kbase + 63 > limit;
                // pass 1: maximum of the raw scores of the own 64 columns (four independent chains)
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    float v[32];
                    tmem_ld32(taddr + c * 32, v);
                    tmem_ld_wait();
                    if (need_mask) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) if (kbase + c * 32 + i > limit) v[i] = -INFINITY;
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], v[i]);
                }
                float mx = pt_max4(mx4), other;
                if (!exchange(mx, other)) { ok = false; break; }
                mx = fmaxf(m, fmaxf(mx, other));
                const float ms = (mx == -INFINITY) ? 0.0f : mx;
                const float corr = pt_ex2((m - ms) * sl2);      // 0 for the first block
                m = mx;
                const float neg = -ms * sl2;
                // the previous block's output; once it is complete the upper P tile may be overwritten
                if (j > 0 && !fold(b - 1, corr_pending)) { ok = false; break; }
                corr_pending = corr;
                // pass 2: p = exp2(s * scale - m * scale) as bf16 into this thread's 128-byte row of the P tile
                // (16-byte chunk c of row r at c ^ (r & 7))
                uint8_t* p_row = (half ? p_upper : kv_ring + (b % PT_KV_STAGES) * PT_KV_BYTES) + row * 128u;
                float rs4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    float v[32];
                    tmem_ld32(taddr + c * 32, v);
                    tmem_ld_wait();
                    if (need_mask) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) if (kbase + c * 32 + i > limit) v[i] = -INFINITY;
                    }
                    uint32_t packed[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float p0 = pt_ex2(fmaf(v[2 * i], sl2, neg)), p1 = pt_ex2(fmaf(v[2 * i + 1], sl2, neg));
                        rs4[i & 3] += p0 + p1;
                        packed[i] = pack_bf16x2(p0, p1);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t chunk16 = (uint32_t)(c * 4 + i);
                        *reinterpret_cast<uint4*>(p_row + (((chunk16 ^ row) & 7u) << 4)) =
                            make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
                    }
                }
                l = l * corr + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
                // scores consumed: the buffer may take the next S; P written: visible to the tensor core, then signal
                tc_fence_before();
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full);
            }
            if (!ok) break;
            ok = fold(g + n_blocks - 1, corr_pending);
            float l_other = 0.0f;
            if (ok) ok = exchange(l, l_other);
            if (ok && q0 + row < prm.chunk) {
                const float inv = 1.0f / (l + l_other);
                bf16* og = prm.out + ((size_t)s * prm.chunk + q0 + row) * ((size_t)prm.heads * PT_HD) + (size_t)h * PT_HD + half * 32;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 w;
                    w.x = pack_bf16x2(acc[8 * i] * inv, acc[8 * i + 1] * inv);
                    w.y = pack_bf16x2(acc[8 * i + 2] * inv, acc[8 * i + 3] * inv);
                    w.z = pack_bf16x2(acc[8 * i + 4] * inv, acc[8 * i + 5] * inv);
                    w.w = pack_bf16x2(acc[8 * i + 6] * inv, acc[8 * i + 7] * inv);
                    *reinterpret_cast<uint4*>(og + 8 * i) = w;
                }
            }
            g += n_blocks;
        }
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
        tmem_dealloc(tmem_base, PT_TMEM_COLS);
    }
}

// {width, rows, sessions} bf16, `row_stride` elements between rows of one session, `session_rows`
// rows between sessions; box = 64 columns x 128 rows x 1 session.
static bool make_map3(CUtensorMap* map, const void* base, uint64_t width, uint64_t rows, uint64_t sessions,
                      uint64_t session_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {width, rows, sessions};
    cuuint64_t strides[2] = {width * 2, session_rows * width * 2};
    cuuint32_t box[3] = {(cuuint32_t)PT_HD, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool prefill_attention_tc_eligible(uint32_t sessions, uint32_t chunk, uint32_t position, const uint32_t* d_position,
                                   uint32_t capacity, uint32_t heads, uint32_t head_dim) {
    // the live row count goes into the tensor maps, so the position must be known on the host
    if (d_position != nullptr || head_dim != PT_HD) return false;
    if (g_gemm_engine == 1) return false;
    if ((uint64_t)position + chunk > capacity) return false;
    if (heads > 65535u || sessions > 65535u || chunk < 32) return false;
    return encode_fn() != nullptr;
}

int launch_prefill_attention_tc(const bf16* q, const bf16* k_cache, const bf16* v_cache, bf16* out, uint32_t sessions,
                                uint32_t chunk, uint32_t position, uint32_t capacity, uint32_t heads, int* d_status,
                                cudaStream_t stream) {
    const uint64_t width = (uint64_t)heads * PT_HD;
    CUtensorMap mq, mk, mv;
    if (!make_map3(&mq, q, width, chunk, sessions, chunk) ||
        !make_map3(&mk, k_cache, width, (uint64_t)position + chunk, sessions, capacity) ||
        !make_map3(&mv, v_cache, width, (uint64_t)position + chunk, sessions, capacity)) {
        set_thread_error("prefill attention: tensor map encoding failed");
        return TNSR_B200_ERR_CUDA;
    }
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        if (cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PT_SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 (int)cudaSharedmemCarveoutMaxShared) != cudaSuccess)
            return check_launch("prefill_attention_tc attribute");
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    PtParams prm;
    prm.out = out;
    prm.chunk = chunk;
    prm.position = position;
    prm.heads = heads;
    prm.q_tiles = ceil_div(chunk, (uint32_t)PT_BQ);
    prm.scale_log2 = (1.0f / sqrtf((float)PT_HD)) * 1.4426950408889634f;
    prm.d_status = d_status;
    prm.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
    prm.sessions = sessions;
    // persistent: two CTAs per SM walk the list of (query tile, head, session) items
    int dev_sms = 0;
    cudaDeviceGetAttribute(&dev_sms, cudaDevAttrMultiProcessorCount, dev);
    if (dev_sms <= 0) dev_sms = 148;
    const uint64_t items = (uint64_t)prm.q_tiles * heads * sessions;
    dim3 grid((unsigned)std::min<uint64_t>(items, 2ull * dev_sms));
    launch_kernel(prefill_attention_tc_kernel, grid, dim3(PT_THREADS), (size_t)PT_SMEM_BYTES, stream, mq, mk, mv, prm);
    count_launch();
    return check_launch("prefill_attention_tc");
}

}  // namespace tb
