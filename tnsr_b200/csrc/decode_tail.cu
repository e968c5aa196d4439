// One kernel for everything between two attention scans of a single-token step at small batch (<= 32 sessions):
// output projection + residual, LayerNorm, gate/up projection + SwiGLU, down projection + residual, the next layer's
// LayerNorm and its QKV projection with the K/V cache write.
//
// Why: at a few dozen sessions these seven operators carry almost no work, and as seven launches their cost is seven
// dependent latency chains (launch, prologue, first operand fetch, epilogue, drain: about 6 us each, measured).  The
// reference has the same structure and the same cost, one launch per stage (src/nn/kv_cache/cuda.rs:193-200).  Here
// they are four phases of one persistent grid, separated by grid-wide barriers; weight tiles for the next phase are
// already in flight while a CTA waits at the barrier (weights never depend on activations); the two LayerNorms are
// recomputed by every CTA from the f32 residual rows (a few dozen rows: cheaper than two more barriers).
//
// What a launch costs is neither HBM bandwidth nor the barriers themselves (all 148 CTAs copy the same 96 KB out of L2
// in 0.9 us, a grid barrier takes 1.1 us, both measured) but what each SM does alone, timed per phase with %globaltimer:
//   * dependent instruction chains, with one CTA per SM and little to switch to while a load, a shuffle or an MMA is in
//     flight: hence 16 warps, a LayerNorm row per 16 or 32 threads with all of its loads issued at once, the k-steps of
//     a chunk dealt over 8 or 16 groups of warps, and every global value an epilogue needs (bias, residual, position)
//     requested before the MMA loop rather than after it;
//   * shared-memory bandwidth in the MMA loop: a warp loads a weight fragment once and uses it for two session tiles
//     (one fragment load per MMA kept the loop at 0.7 us per 512-wide chunk);
//   * a few KB that every warp of every CTA wants at the same moment (LayerNorm scale and shift) sit in one or two L2
//     slices: fetched per warp they cost 4 us per LayerNorm, staged once per CTA into shared memory nothing measurable;
//   * an SM takes in about 64 bytes per clock from L2: the down projection's 131 KB of activations per CTA are 1.1 us
//     whatever the copy instruction (bulk copies of one row each were slower than 16-byte cp.async here).
//
// Shape of the work: with so few rows the projections are weight streaming, not tensor-core throughput.  A CTA owns 16
// output columns (32 packed gate/up columns) of a projection: its weight rows are read exactly once by the grid, the
// activation rows (<= 32) are re-read by every CTA from L2.  The products run on warp-level mma.sync.m16n8k16 (bf16 in,
// f32 out) with the weight rows as the M side and 8 sessions as the N side -- tcgen05's 64/128-row M side would leave a
// CTA either most of a projection or most of the MMA empty at this size.  K is walked in chunks of 512 through a ring of
// cp.async stages (four of 16 weight rows or two of 32, three of activation rows): for widths up to 2048 every weight
// chunk of a CTA's next tile is requested between arriving at the barrier and waiting on it.  Inside a chunk the k-steps alternate between
// the k-groups of warps, whose partial sums are added in a fixed order, so results do not depend on the number of
// sessions or on timing.
//
// Cross-CTA data (residual rows, attention output, the SwiGLU hidden rows) is read with L2-only loads (ld.global.cg,
// cp.async.cg): another CTA wrote it during this launch.  Every barrier wait is bounded; on expiry the kernel records
// DEV_TIMEOUT and all CTAs leave.
#include "common.cuh"

namespace tb {

namespace {

constexpr int DT_THREADS = 512;
constexpr int DT_WARPS = DT_THREADS / 32;
constexpr int DT_KCH = 512;                     // K elements per pipeline chunk
constexpr int DT_PITCH = DT_KCH + 8;            // shared-memory row pitch in elements: 1040 bytes, conflict-free ldmatrix
constexpr int DT_W_ROWS = 64;                   // weight rows in the ring: 4 stages of 16 or 2 stages of 32
constexpr int DT_A_STAGES = 3;                  // activation stages of MT rows each
constexpr int DT_RED_PITCH = 33;                // floats per session row of a k-group's partial sums: conflict-free both ways
constexpr int DT_MAX_D = 1024;                  // widest model: a LayerNorm row is held in the registers of its threads

enum : uint32_t { DT_PHASE_O = 1, DT_PHASE_GU = 2, DT_PHASE_DOWN = 4, DT_PHASE_QKV = 8 };

struct DtBarrier {
    uint32_t arrived;   // monotonically increasing within a launch
    uint32_t left;      // CTAs that have passed the last barrier; the last one clears both words
};

struct DtParams {
    uint32_t phases;
    uint32_t rows;                 // sessions in this launch (<= MT)
    uint32_t d, f;                 // model width, FFN width
    float eps;
    // residual stream and activations of the range
    float* h;                      // [rows, d] f32
    const bf16* att;               // [rows, d] attention output (phase O)
    bf16* ff;                      // [rows, f] SwiGLU hidden rows (written by GU, read by DOWN)
    bf16* q;                       // [rows, d] queries of the next layer (phase QKV)
    // this layer
    const bf16* wo; const float* bo;
    const float* ln2w; const float* ln2b;
    const bf16* wgu; const float* bgu;          // packed [2f, d]: 16 gate rows, 16 up rows, ...
    const bf16* wdown; const float* bdown;
    // next layer (phase QKV)
    const float* ln1w; const float* ln1b;
    const bf16* wqkv; const float* bqkv;        // [3d, d]
    bf16* k_cache; bf16* v_cache;
    uint32_t capacity;
    const uint32_t* d_position; uint32_t position; uint32_t position_stride;
    uint32_t first_session;        // session index of row 0 (contiguous caches are passed already offset: 0)
    KvPaging paging;
    DtBarrier* barrier;
    int* d_status;
    uint64_t wait_limit_ns;
};

__device__ __forceinline__ uint32_t dt_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void dt_cp16(void* dst, const void* src, bool valid) {
    const uint32_t n = valid ? 16u : 0u;        // src-size 0: the 16 bytes are zero-filled and nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dt_smem(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void dt_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void dt_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void dt_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(dt_smem(p)));
}
__device__ __forceinline__ void dt_mma(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ uint64_t dt_timer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Grid-wide barrier number `index` (0, 1, ...) of this launch, in two halves so that work which does not depend on the
// other CTAs (requests for the next phase's weights) sits between arriving and waiting.
__device__ __forceinline__ void dt_grid_arrive(const DtParams& P) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();                                   // this CTA's writes before its arrival
        atomicAdd(&P.barrier->arrived, 1u);
    }
}
// Returns false if the wait ran out.
__device__ __forceinline__ bool dt_grid_wait(const DtParams& P, uint32_t index, int* s_abort) {
    if (threadIdx.x == 0) {
        const uint32_t target = (index + 1) * gridDim.x;
        const uint64_t start = dt_timer();
        uint32_t seen;
        for (uint32_t it = 0;; ++it) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(&P.barrier->arrived) : "memory");
            if (seen >= target) break;
            if ((it & 15u) == 15u) {
                if (dt_timer() - start > P.wait_limit_ns || (P.d_status && *reinterpret_cast<volatile int*>(P.d_status) == DEV_TIMEOUT)) {
                    *s_abort = 1;
                    if (P.d_status) atomicCAS(P.d_status, DEV_OK, DEV_TIMEOUT);
                    break;
                }
            }
            __nanosleep(32);
        }
    }
    __syncthreads();
    return *reinterpret_cast<volatile int*>(s_abort) == 0;
}

// What a projection phase multiplies and where its results go.
struct DtGemm {
    const bf16* w;        // [n, k] K-major weights
    uint32_t n, k;
    uint32_t cols;        // columns per tile: 16, or 32 for the packed gate/up matrix
    const bf16* act;      // streamed activation rows [rows, k] (global), or nullptr: the rows are resident in `nbuf`
};

// Copies chunk `chunk` of the tile's weight rows (and, if streamed, of the activation rows) into a ring stage.
__device__ __forceinline__ void dt_issue_w(const DtGemm& g, uint32_t n0, uint32_t chunk, bf16* wstage) {
    const uint32_t k0 = chunk * DT_KCH;
    const uint32_t kk = (threadIdx.x & 63u) * 8;                       // 64 pieces of 16 bytes per row
#pragma unroll 1
    for (uint32_t r = threadIdx.x >> 6; r < g.cols; r += DT_THREADS / 64) {
        const bool valid = n0 + r < g.n && k0 + kk < g.k;
        dt_cp16(wstage + (size_t)r * DT_PITCH + kk, g.w + (valid ? (size_t)(n0 + r) * g.k + k0 + kk : 0), valid);
    }
}
__device__ __forceinline__ void dt_issue_a(const DtGemm& g, uint32_t rows, uint32_t mt, uint32_t chunk, bf16* astage) {
    if (!g.act) return;
    const uint32_t k0 = chunk * DT_KCH;
    const uint32_t kk = (threadIdx.x & 63u) * 8;
#pragma unroll 1
    for (uint32_t r = threadIdx.x >> 6; r < mt; r += DT_THREADS / 64) {
        const bool valid = r < rows && k0 + kk < g.k;
        dt_cp16(astage + (size_t)r * DT_PITCH + kk, g.act + (valid ? (size_t)r * g.k + k0 + kk : 0), valid);
    }
}
__device__ __forceinline__ uint32_t dt_stages(const DtGemm& g) {
    const uint32_t ws = DT_W_ROWS / g.cols;
    return g.act ? min(ws, (uint32_t)DT_A_STAGES) : ws;
}
__device__ __forceinline__ void dt_wait_pending(uint32_t n) {
    if (n == 0) dt_wait<0>();
    else if (n == 1) dt_wait<1>();
    else if (n == 2) dt_wait<2>();
    else dt_wait<3>();
}

// LayerNorm of the residual rows into `nbuf` ([MT][d + 8] bf16): two passes over registers, rsqrt of the biased variance,
// as layernorm_warp_kernel does.  Scale and shift come from shared memory: a few KB that every warp of every CTA wants
// at the same moment sit in one or two L2 slices, and fetched per warp they cost 4 us.  Warp w owns rows w and (MT 32)
// w + 16, lane l the float4s l, l + 32, ... of both: all loads of a thread are in flight together, the two rows' sums are
// independent butterfly reductions, and each scale / shift value read from shared memory serves both rows (with a row per
// 16 lanes the output pass ran at the shared-memory load rate: 24 16-byte loads per thread).  Rows past `rows` become zeros.
template <int MT>
__device__ __forceinline__ void dt_layernorm(const DtParams& P, const float* lnbuf, bf16* nbuf) {
    constexpr int RPW = MT / DT_WARPS;                     // rows per warp: 1 or 2
    constexpr int NV = DT_MAX_D / 128;                     // float4 per lane and row
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t d = P.d, nvec = d >> 2;
    float4 v[RPW][NV];
#pragma unroll
    for (int j = 0; j < RPW; ++j) {
        const uint32_t r = warp + j * DT_WARPS;
        const float4* xr = reinterpret_cast<const float4*>(P.h + (size_t)r * d);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const uint32_t c = lane + i * 32;
            v[j][i] = (r < P.rows && c < nvec) ? __ldcg(xr + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
    float inv[RPW];
#pragma unroll
    for (int j = 0; j < RPW; ++j) {
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) sum += (v[j][i].x + v[j][i].y) + (v[j][i].z + v[j][i].w);
#pragma unroll
        for (uint32_t o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float mean = sum / (float)d;
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (lane + i * 32 < nvec) {
                v[j][i].x -= mean; v[j][i].y -= mean; v[j][i].z -= mean; v[j][i].w -= mean;
                sq += (v[j][i].x * v[j][i].x + v[j][i].y * v[j][i].y) + (v[j][i].z * v[j][i].z + v[j][i].w * v[j][i].w);
            }
        }
#pragma unroll
        for (uint32_t o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        inv[j] = rsqrtf(sq / (float)d + P.eps);
    }
    const float4* wr = reinterpret_cast<const float4*>(lnbuf);               // scale, then shift: copies in shared memory
    const float4* br = reinterpret_cast<const float4*>(lnbuf + DT_MAX_D);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const uint32_t c = lane + i * 32;
        if (c < nvec) {
            const float4 ww = wr[c], bb = br[c];
#pragma unroll
            for (int j = 0; j < RPW; ++j) {
                const uint32_t r = warp + j * DT_WARPS;
                uint2* out = reinterpret_cast<uint2*>(nbuf + (size_t)r * (d + 8));
                out[c] = r < P.rows ? make_uint2(pack_bf16x2(v[j][i].x * inv[j] * ww.x + bb.x, v[j][i].y * inv[j] * ww.y + bb.y),
                                                 pack_bf16x2(v[j][i].z * inv[j] * ww.z + bb.z, v[j][i].w * inv[j] * ww.w + bb.w))
                                    : make_uint2(0u, 0u);
            }
        }
    }
}

// Requests a LayerNorm's scale and shift into `lnbuf` ([2][DT_MAX_D] f32) as one cp.async group.  They are weights: the
// request can go out before the barrier that the rows wait for.
__device__ __forceinline__ void dt_issue_ln(const float* w, const float* b, uint32_t d, float* lnbuf) {
    const uint32_t nvec = d >> 2;
    for (uint32_t i = threadIdx.x; i < 2 * nvec; i += DT_THREADS) {
        const bool shift = i >= nvec;
        const uint32_t c = shift ? i - nvec : i;
        dt_cp16(lnbuf + (shift ? DT_MAX_D : 0) + c * 4, (shift ? b : w) + c * 4, true);
    }
    dt_commit();
}

// Requests the first weight chunks of tile `n0` (as many as the ring holds), one cp.async group each; returns how many.
__device__ __forceinline__ uint32_t dt_prefetch_w(const DtGemm& g, uint32_t n0, bf16* wbuf) {
    const uint32_t chunks = (g.k + DT_KCH - 1) / DT_KCH;
    const uint32_t pre = min(dt_stages(g), chunks);
#pragma unroll 1
    for (uint32_t c = 0; c < pre; ++c) {
        dt_issue_w(g, n0, c, wbuf + (size_t)c * g.cols * DT_PITCH);
        dt_commit();
    }
    return pre;
}

// One tile of a projection: the products of the tile's columns c with all MT session rows, left in `red` as one partial
// sum per k-group: red[kg * MT * 33 + m * 33 + c] (f32).  The first `w_issued` weight chunks are already in flight
// (dt_prefetch_w).
//
// A warp takes two session tiles (16 sessions) and the k-steps kp, kp + KG, ... of every chunk, kp being its k-group:
// every weight fragment it loads from shared memory feeds two MMAs (four for the packed gate/up tile), which is what
// keeps the loop under the shared-memory bandwidth that one fragment load per MMA would need.
template <int MT>
__device__ __forceinline__ void dt_gemm_tile(const DtGemm& g, uint32_t rows, uint32_t n0, bf16* wbuf, bf16* abuf, const bf16* nbuf,
                                             uint32_t npitch, float* red, uint32_t w_issued) {
    constexpr uint32_t NP = MT / 16;                // pairs of session tiles: 1 or 2
    constexpr uint32_t KG = DT_WARPS / NP;          // k-groups: 16 or 8
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t kp = warp / NP, np = warp % NP;
    const uint32_t chunks = (g.k + DT_KCH - 1) / DT_KCH;
    const bool two = g.cols == 32;                  // a second 16-row weight tile (packed gate/up)
    const uint32_t S = dt_stages(g);
    const size_t wstage = (size_t)g.cols * DT_PITCH, astage = (size_t)MT * DT_PITCH;
    float acc[2][2][4];                             // [weight tile][session tile of the pair][fragment]
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[a][t][e] = 0.0f;

    // one cp.async group per chunk: its weights (unless already requested) and its activation rows (unless resident)
    const uint32_t pre = min(S, chunks);
#pragma unroll 1
    for (uint32_t c = 0; c < pre; ++c) {
        if (c >= w_issued) dt_issue_w(g, n0, c, wbuf + c * wstage);
        dt_issue_a(g, rows, MT, c, abuf + c * astage);
        dt_commit();
    }
#pragma unroll 1
    for (uint32_t ch = 0; ch < chunks; ++ch) {
        const uint32_t st = ch % S;
        dt_wait_pending(min(chunks - 1 - ch, S - 1));     // groups requested after this chunk's may still be in flight
        __syncthreads();
        const bf16* wt = wbuf + st * wstage;
        const bf16* at = g.act ? abuf + st * astage : nbuf + (size_t)ch * DT_KCH;
        const uint32_t apitch = g.act ? (uint32_t)DT_PITCH : npitch;
        const uint32_t ksteps = min((uint32_t)DT_KCH, g.k - ch * DT_KCH) / 16;
        const bf16* wp = wt + (size_t)(lane & 15) * DT_PITCH + (lane >> 4) * 8;
        // sessions np * 16 + [0, 16): matrices (rows 0-7, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 0-7), (rows 8-15, k 8-15)
        const bf16* ap = at + (size_t)(np * 16 + (lane >> 4) * 8 + (lane & 7)) * apitch + ((lane >> 3) & 1) * 8;
#pragma unroll 2
        for (uint32_t ks = kp; ks < ksteps; ks += KG) {
            uint32_t a0[4], a1[4], b[4];
            dt_ldmatrix_x4(a0, wp + ks * 16);
            dt_ldmatrix_x4(b, ap + ks * 16);
            if (two) dt_ldmatrix_x4(a1, wp + (size_t)16 * DT_PITCH + ks * 16);
            const uint32_t bl[2] = {b[0], b[1]}, bh[2] = {b[2], b[3]};
            dt_mma(acc[0][0], a0, bl);
            dt_mma(acc[0][1], a0, bh);
            if (two) {
                dt_mma(acc[1][0], a1, bl);
                dt_mma(acc[1][1], a1, bh);
            }
        }
        if (ch + S < chunks) {
            __syncthreads();        // every warp is done with this stage: refill it
            dt_issue_w(g, n0, ch + S, wbuf + st * wstage);
            dt_issue_a(g, rows, MT, ch + S, abuf + st * astage);
            dt_commit();
        }
    }
    // this k-group's partial sums: red[kp][m * 33 + c]
    const uint32_t row = lane >> 2;
    float* mine = red + (size_t)kp * MT * DT_RED_PITCH;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        if (t == 1 && !two) break;
        const uint32_t c = t * 16 + row;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t m = np * 16 + j * 8 + (lane & 3) * 2;
            mine[m * DT_RED_PITCH + c] = acc[t][j][0];
            mine[(m + 1) * DT_RED_PITCH + c] = acc[t][j][1];
            mine[m * DT_RED_PITCH + c + 8] = acc[t][j][2];
            mine[(m + 1) * DT_RED_PITCH + c + 8] = acc[t][j][3];
        }
    }
    __syncthreads();
}

// Sum over the k-groups of one output, in a fixed order.
template <int MT>
__device__ __forceinline__ float dt_reduced(const float* red, uint32_t idx) {
    constexpr uint32_t KG = DT_WARPS / (MT / 16);
    constexpr uint32_t STRIDE = MT * DT_RED_PITCH;
    float s[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        s[q] = 0.0f;
#pragma unroll
        for (uint32_t i = 0; i < KG / 4; ++i) s[q] += red[idx + (q * (KG / 4) + i) * STRIDE];
    }
    return (s[0] + s[1]) + (s[2] + s[3]);
}

// The projection of phase `ph` (0: attention output, 1: gate/up, 2: down, 3: next layer's QKV).
__device__ __forceinline__ DtGemm dt_phase_gemm(const DtParams& P, uint32_t ph) {
    DtGemm g;
    g.w = ph == 0 ? P.wo : ph == 1 ? P.wgu : ph == 2 ? P.wdown : P.wqkv;
    g.n = ph == 1 ? 2 * P.f : ph == 3 ? 3 * P.d : P.d;
    g.k = ph == 2 ? P.f : P.d;
    g.cols = ph == 1 ? 32u : 16u;
    g.act = ph == 0 ? P.att : ph == 2 ? P.ff : nullptr;
    return g;
}

template <int MT>
__global__ void __launch_bounds__(DT_THREADS, 1)
decode_tail_kernel(DtParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t KG = DT_WARPS / (MT / 16);
    bf16* wbuf = reinterpret_cast<bf16*>(smem);                                   // [DT_W_ROWS][PITCH]
    bf16* abuf = wbuf + (size_t)DT_W_ROWS * DT_PITCH;                             // [DT_A_STAGES][MT][PITCH], or the LayerNorm rows
    constexpr size_t act_elems = (size_t)DT_A_STAGES * MT * DT_PITCH;
    static_assert((size_t)MT * (DT_MAX_D + 8) <= act_elems, "LayerNorm rows must fit the activation ring");
    static_assert(16 * MT <= DT_THREADS, "one output per thread in the epilogue");
    float* red = reinterpret_cast<float*>(abuf + act_elems);                      // [KG][MT][33]
    float* lnbuf = red + (size_t)KG * MT * DT_RED_PITCH;                           // [2][DT_MAX_D]
    int* s_abort = reinterpret_cast<int*>(lnbuf + 2 * DT_MAX_D);
    if (threadIdx.x == 0) *s_abort = 0;
    // the next kernel of the stream may take each SM as this CTA leaves it, instead of after the grid has drained (it
    // cannot start earlier: this CTA's shared memory leaves it no room, and it waits for this grid in its pdl_wait)
    pdl_trigger();
    __syncthreads();

    const uint32_t d = P.d, f = P.f, rows = P.rows;
    const uint32_t npitch = d + 8;
    uint32_t barriers = 0, w0 = 0;
    bool ok = true, ln_ready = false;
    // the output of a tile this thread finishes: column c of the tile, session m
    const uint32_t c = threadIdx.x % 16, m = threadIdx.x / 16;

#pragma unroll 1
    for (uint32_t ph = 0; ph < 4 && ok; ++ph) {
        if (!((P.phases >> ph) & 1u)) continue;
        const DtGemm g = dt_phase_gemm(P, ph);
        const float* bias = ph == 0 ? P.bo : ph == 1 ? P.bgu : ph == 2 ? P.bdown : P.bqkv;
        if (ph & 1u) {
            // gate/up and QKV read the LayerNorm of the residual rows, which lives where the streamed activation
            // chunks of the other two phases do
            if (!ln_ready) dt_issue_ln(ph == 1 ? P.ln2w : P.ln1w, ph == 1 ? P.ln2b : P.ln1b, d, lnbuf);
            dt_wait_pending(w0);                 // the parameters' group is older than the w0 weight groups
            __syncthreads();
            ln_ready = false;
            dt_layernorm<MT>(P, lnbuf, abuf);
            __syncthreads();
        }
#pragma unroll 1
        for (uint32_t n0 = blockIdx.x * g.cols; n0 < g.n; n0 += gridDim.x * g.cols) {
            // what the epilogue will need from global memory, requested before the products
            const uint32_t col = n0 + c;
            const bool mine = m < rows && (ph == 1 || col < g.n);
            float b0 = 0.0f, b1 = 0.0f, hold = 0.0f;
            uint32_t pos = 0;
            if (mine) {
                b0 = __ldg(bias + col);
                if (ph == 1) b1 = __ldg(bias + col + 16);
                if (ph == 0 || ph == 2) hold = __ldcg(P.h + (size_t)m * d + col);
                if (ph == 3) pos = P.d_position ? P.d_position[(size_t)m * P.position_stride] : P.position;
            }
            dt_gemm_tile<MT>(g, rows, n0, wbuf, abuf, abuf, npitch, red, w0);
            w0 = 0;
            if (mine) {
                const float v = dt_reduced<MT>(red, m * DT_RED_PITCH + c) + b0;
                if (ph == 1) {
                    // packed columns [0, 16) are gate, [16, 32) the matching up columns -> 16 outputs
                    const float up = dt_reduced<MT>(red, m * DT_RED_PITCH + 16 + c) + b1;
                    P.ff[(size_t)m * f + n0 / 2 + c] = __float2bfloat16_rn(fast_silu(v) * up);
                } else if (ph != 3) {
                    P.h[(size_t)m * d + col] = hold + v;                   // h += projection + bias
                } else {
                    const bf16 vb = __float2bfloat16_rn(v);
                    const uint32_t which = col / d, cc = col - which * d;
                    if (which == 0) {
                        P.q[(size_t)m * d + cc] = vb;
                    } else {
                        const size_t crow = kv_row(P.paging, P.first_session + m, pos, P.capacity);
                        (which == 1 ? P.k_cache : P.v_cache)[crow * d + cc] = vb;
                    }
                }
            }
            __syncthreads();
        }
        // the next phase of this launch, if any: its weights and LayerNorm parameters do not depend on what the other
        // CTAs are still writing, so they are requested before the barrier
        uint32_t nx = ph + 1;
        while (nx < 4 && !((P.phases >> nx) & 1u)) ++nx;
        if (nx < 4) {
            dt_grid_arrive(P);
            const DtGemm gn = dt_phase_gemm(P, nx);
            if (nx & 1u) {
                dt_issue_ln(nx == 1 ? P.ln2w : P.ln1w, nx == 1 ? P.ln2b : P.ln1b, d, lnbuf);
                ln_ready = true;
            }
            const uint32_t n0 = blockIdx.x * gn.cols;
            if (n0 < gn.n) w0 = dt_prefetch_w(gn, n0, wbuf);
            ok = dt_grid_wait(P, barriers++, s_abort);
        }
    }
    // ---------------- leave: the last CTA out re-arms the barrier words for the next launch ----------------
    asm volatile("cp.async.wait_all;" ::: "memory");   // also copies issued for a phase that an abort skipped
    __syncthreads();
    if (threadIdx.x == 0 && barriers > 0) {
        __threadfence();
        if (atomicAdd(&P.barrier->left, 1u) == gridDim.x - 1) {
            P.barrier->arrived = 0;
            P.barrier->left = 0;
            __threadfence();
        }
    }
}

template <int MT>
size_t dt_smem_bytes() {
    return (size_t)DT_W_ROWS * DT_PITCH * 2 + (size_t)DT_A_STAGES * MT * DT_PITCH * 2 +
           (size_t)(DT_WARPS / (MT / 16)) * MT * DT_RED_PITCH * 4 + 2 * DT_MAX_D * 4 + 16;
}

int dt_sm_count() {
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
int dt_launch(const DtParams& P, cudaStream_t stream) {
    const size_t smem = dt_smem_bytes<MT>();
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        if (cudaFuncSetAttribute(decode_tail_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return check_launch("decode_tail attribute");
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    // one CTA per SM, all resident at once: the kernel's barriers need every CTA to be running
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)dt_sm_count());
    cfg.blockDim = dim3(DT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, decode_tail_kernel<MT>, P);
    count_launch();
    return check_launch("decode_tail");
}

}  // namespace

uint64_t decode_tail_workspace_bytes() { return 256; }

bool decode_tail_supported(uint32_t rows, uint32_t d, uint32_t f) {
    return rows >= 1 && rows <= 32 && d % 16 == 0 && d <= DT_MAX_D && f % 16 == 0 && f >= 16;
}

int launch_decode_tail(const DecodeTailArgs& a, cudaStream_t stream) {
    if (!decode_tail_supported(a.rows, a.d, a.f) || !a.workspace) {
        set_thread_error("decode tail: shape outside the fused kernel");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    DtParams P = {};
    P.phases = (a.run_o ? DT_PHASE_O : 0u) | (a.run_ffn ? (DT_PHASE_GU | DT_PHASE_DOWN) : 0u) | (a.run_qkv ? DT_PHASE_QKV : 0u);
    if (!P.phases) return TNSR_B200_OK;
    P.rows = a.rows; P.d = a.d; P.f = a.f; P.eps = a.eps;
    P.h = a.h; P.att = a.att; P.ff = a.ff; P.q = a.q;
    P.wo = a.wo; P.bo = a.bo; P.ln2w = a.ln2w; P.ln2b = a.ln2b; P.wgu = a.wgu; P.bgu = a.bgu; P.wdown = a.wdown; P.bdown = a.bdown;
    P.ln1w = a.ln1w; P.ln1b = a.ln1b; P.wqkv = a.wqkv; P.bqkv = a.bqkv;
    P.k_cache = a.k_cache; P.v_cache = a.v_cache; P.capacity = a.capacity;
    P.d_position = a.d_position; P.position = a.position; P.position_stride = a.position_stride;
    P.first_session = a.first_session;
    if (a.paging) P.paging = *a.paging;
    P.barrier = reinterpret_cast<DtBarrier*>(a.workspace);
    P.d_status = a.d_status;
    P.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
    if (a.rows <= 16) return dt_launch<16>(P, stream);
    return dt_launch<32>(P, stream);
}

}  // namespace tb
