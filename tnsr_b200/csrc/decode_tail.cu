// One kernel for everything between two attention scans of a single-token step at small batch (<= 64 sessions):
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
// Shape of the work: with so few rows the projections are weight streaming, not tensor-core throughput.  A CTA owns 16
// output columns (32 packed gate/up columns) of a projection: its weight rows are read exactly once by the grid, the
// activation rows (<= 64) are re-read by every CTA from L2.  The products run on warp-level mma.sync.m16n8k16 (bf16 in,
// f32 out) with the weight rows as the M side and 8 sessions as the N side -- tcgen05's 64/128-row M side would leave a
// CTA either most of a projection or most of the MMA empty at this size.  K is walked in chunks of 512 through a
// double-buffered cp.async pipeline; inside a chunk the k-steps alternate between two groups of warps whose partial
// sums are added in a fixed order, so results do not depend on the number of sessions or on timing.
//
// Cross-CTA data (residual rows, attention output, the SwiGLU hidden rows) is read with L2-only loads (ld.global.cg,
// cp.async.cg): another CTA wrote it during this launch.  Every barrier wait is bounded; on expiry the kernel records
// DEV_TIMEOUT and all CTAs leave.
#include "common.cuh"

namespace tb {

namespace {

constexpr int DT_THREADS = 256;
constexpr int DT_KCH = 512;                     // K elements per pipeline chunk
constexpr int DT_PITCH = DT_KCH + 8;            // shared-memory row pitch in elements: 1040 bytes, conflict-free ldmatrix
constexpr int DT_MAX_COLS = 32;                 // packed gate/up tile; plain projections use 16
constexpr int DT_MAX_D = 1024;                  // LayerNorm rows stay in registers up to this width

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
__device__ __forceinline__ void dt_ldmatrix_x2(uint32_t (&r)[2], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(dt_smem(p)));
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

// Grid-wide barrier number `index` (0, 1, ...) of this launch.  Returns false if the wait ran out.
__device__ __forceinline__ bool dt_grid_barrier(const DtParams& P, uint32_t index, int* s_abort) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();                                   // this CTA's writes before its arrival
        atomicAdd(&P.barrier->arrived, 1u);
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

// Copies chunk `chunk` of the tile's weight rows (and, if streamed, of the activation rows) into pipeline buffer `buf`.
template <int MT>
__device__ __forceinline__ void dt_issue_w(const DtGemm& g, uint32_t n0, uint32_t chunk, bf16* wbuf) {
    const uint32_t k0 = chunk * DT_KCH;
    const uint32_t pieces_per_row = DT_KCH / 8;
    for (uint32_t i = threadIdx.x; i < g.cols * pieces_per_row; i += DT_THREADS) {
        const uint32_t r = i / pieces_per_row, kk = (i % pieces_per_row) * 8;
        const bool valid = n0 + r < g.n && k0 + kk < g.k;
        dt_cp16(wbuf + (size_t)r * DT_PITCH + kk, g.w + (valid ? (size_t)(n0 + r) * g.k + k0 + kk : 0), valid);
    }
}
template <int MT>
__device__ __forceinline__ void dt_issue_a(const DtGemm& g, uint32_t rows, uint32_t chunk, bf16* abuf) {
    if (!g.act) return;
    const uint32_t k0 = chunk * DT_KCH;
    const uint32_t pieces_per_row = DT_KCH / 8;
    for (uint32_t i = threadIdx.x; i < MT * pieces_per_row; i += DT_THREADS) {
        const uint32_t r = i / pieces_per_row, kk = (i % pieces_per_row) * 8;
        const bool valid = r < rows && k0 + kk < g.k;
        dt_cp16(abuf + (size_t)r * DT_PITCH + kk, g.act + (valid ? (size_t)r * g.k + k0 + kk : 0), valid);
    }
}

// LayerNorm of the residual rows into `nbuf` ([MT][d + 8] bf16), one warp per row, the arithmetic of
// layernorm_warp_kernel (two passes over registers, rsqrt of the biased variance).  Rows past `rows` become zeros.
template <int MT>
__device__ __forceinline__ void dt_layernorm(const DtParams& P, const float* __restrict__ w, const float* __restrict__ b, bf16* nbuf) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t d = P.d, nvec = d >> 2, pitch = d + 8;
    for (uint32_t r = warp; r < (uint32_t)MT; r += DT_THREADS / 32) {
        uint2* out = reinterpret_cast<uint2*>(nbuf + (size_t)r * pitch);
        if (r >= P.rows) {
            for (uint32_t c = lane; c < nvec; c += 32) out[c] = make_uint2(0u, 0u);
            continue;
        }
        const float4* xr = reinterpret_cast<const float4*>(P.h + (size_t)r * d);
        float4 v[DT_MAX_D / 128];
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < DT_MAX_D / 128; ++i) {
            const uint32_t c = lane + i * 32;
            if (c < nvec) {
                v[i] = __ldcg(xr + c);
                sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float mean = sum / (float)d;
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < DT_MAX_D / 128; ++i) {
            const uint32_t c = lane + i * 32;
            if (c < nvec) {
                v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
                sq += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        const float inv = rsqrtf(sq / (float)d + P.eps);
        const float4* wr = reinterpret_cast<const float4*>(w);
        const float4* br = reinterpret_cast<const float4*>(b);
#pragma unroll
        for (int i = 0; i < DT_MAX_D / 128; ++i) {
            const uint32_t c = lane + i * 32;
            if (c < nvec) {
                const float4 ww = __ldg(wr + c), bb = __ldg(br + c);
                out[c] = make_uint2(pack_bf16x2(v[i].x * inv * ww.x + bb.x, v[i].y * inv * ww.y + bb.y),
                                    pack_bf16x2(v[i].z * inv * ww.z + bb.z, v[i].w * inv * ww.w + bb.w));
            }
        }
    }
}

// One tile of a projection: acc[c][m] for the tile's columns c and all MT session rows, left in `red` as
// red[c * MT + m] (f32).  The pipeline's first weight chunk may already be in flight (`w0_issued`).
//
// Warp w: k-group kp = w / 4 takes the k-steps kp, kp + 2, ... of every chunk; ng = w % 4 takes the session tiles
// ng and ng + 4 (8 sessions each).  The two k-groups are added as (group 0) + (group 1).
template <int MT>
__device__ __forceinline__ void dt_gemm_tile(const DtGemm& g, uint32_t rows, uint32_t n0, bf16* wbuf, bf16* abuf, const bf16* nbuf,
                                             uint32_t npitch, float* red, bool w0_issued) {
    constexpr int NT = MT / 8;                      // session tiles
    constexpr int NPW = (NT + 3) / 4;               // session tiles per warp: 1 (MT <= 32) or 2 (MT 64)
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t kp = warp >> 2, ng = warp & 3;
    const uint32_t chunks = (g.k + DT_KCH - 1) / DT_KCH;
    const uint32_t atiles = g.cols / 16;
    float acc[2][NPW][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int j = 0; j < NPW; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[a][j][e] = 0.0f;

    // every chunk is two cp.async groups: weights, then activations (empty when the rows are resident)
    if (!w0_issued) dt_issue_w<MT>(g, n0, 0, wbuf);
    dt_commit();
    dt_issue_a<MT>(g, rows, 0, abuf);
    dt_commit();
    for (uint32_t ch = 0; ch < chunks; ++ch) {
        const uint32_t cur = ch & 1, nxt = cur ^ 1;
        if (ch + 1 < chunks) {
            dt_issue_w<MT>(g, n0, ch + 1, wbuf + (size_t)nxt * DT_MAX_COLS * DT_PITCH);
            dt_commit();
            dt_issue_a<MT>(g, rows, ch + 1, abuf + (size_t)nxt * MT * DT_PITCH);
            dt_commit();
            dt_wait<2>();
        } else {
            dt_wait<0>();
        }
        __syncthreads();
        const bf16* wt = wbuf + (size_t)cur * DT_MAX_COLS * DT_PITCH;
        const bf16* at = g.act ? abuf + (size_t)cur * MT * DT_PITCH : nbuf + (size_t)ch * DT_KCH;
        const uint32_t apitch = g.act ? (uint32_t)DT_PITCH : npitch;
        const uint32_t ksteps = min((uint32_t)DT_KCH, g.k - ch * DT_KCH) / 16;
        for (uint32_t ks = kp; ks < ksteps; ks += 2) {
            uint32_t a[2][4];
            for (uint32_t t = 0; t < atiles; ++t)
                dt_ldmatrix_x4(a[t], wt + (size_t)(t * 16 + (lane & 15)) * DT_PITCH + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < NPW; ++j) {
                const uint32_t nt = ng + 4 * j;
                if (nt >= (uint32_t)NT) continue;
                uint32_t b[2];
                dt_ldmatrix_x2(b, at + (size_t)(nt * 8 + (lane & 7)) * apitch + ks * 16 + ((lane >> 3) & 1) * 8);
                for (uint32_t t = 0; t < atiles; ++t) dt_mma(acc[t][j], a[t], b);
            }
        }
        __syncthreads();        // the buffers of this chunk are free for the chunk after next
    }
    // (k-group 0) + (k-group 1), through shared memory: red[c * MT + m]
    const uint32_t row = lane >> 2, col = (lane & 3) * 2;
    if (kp == 1) {
#pragma unroll
        for (int j = 0; j < NPW; ++j) {
            const uint32_t nt = ng + 4 * j;
            if (nt >= (uint32_t)NT) continue;
            for (uint32_t t = 0; t < atiles; ++t) {
                const uint32_t c = t * 16 + row, m = nt * 8 + col;
                red[c * MT + m] = acc[t][j][0];
                red[c * MT + m + 1] = acc[t][j][1];
                red[(c + 8) * MT + m] = acc[t][j][2];
                red[(c + 8) * MT + m + 1] = acc[t][j][3];
            }
        }
    }
    __syncthreads();
    if (kp == 0) {
#pragma unroll
        for (int j = 0; j < NPW; ++j) {
            const uint32_t nt = ng + 4 * j;
            if (nt >= (uint32_t)NT) continue;
            for (uint32_t t = 0; t < atiles; ++t) {
                const uint32_t c = t * 16 + row, m = nt * 8 + col;
                red[c * MT + m] = acc[t][j][0] + red[c * MT + m];
                red[c * MT + m + 1] = acc[t][j][1] + red[c * MT + m + 1];
                red[(c + 8) * MT + m] = acc[t][j][2] + red[(c + 8) * MT + m];
                red[(c + 8) * MT + m + 1] = acc[t][j][3] + red[(c + 8) * MT + m + 1];
            }
        }
    }
    __syncthreads();
}

template <int MT>
__global__ void __launch_bounds__(DT_THREADS, 1)
decode_tail_kernel(DtParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    bf16* wbuf = reinterpret_cast<bf16*>(smem);                                   // [2][32][PITCH]
    bf16* abuf = wbuf + (size_t)2 * DT_MAX_COLS * DT_PITCH;                       // [2][MT][PITCH], or the resident rows
    bf16* nbuf = abuf;                                                            // [MT][d + 8] (phases GU and QKV)
    const size_t act_elems = max((size_t)2 * MT * DT_PITCH, (size_t)MT * (DT_MAX_D + 8));
    float* red = reinterpret_cast<float*>(abuf + act_elems);                      // [32 * MT]
    int* s_abort = reinterpret_cast<int*>(red + DT_MAX_COLS * MT);
    if (threadIdx.x == 0) *s_abort = 0;
    __syncthreads();

    const uint32_t d = P.d, f = P.f, rows = P.rows;
    const uint32_t npitch = d + 8;
    uint32_t barriers = 0;
    bool ok = true;

    DtGemm go = {P.wo, d, d, 16, P.att};
    DtGemm ggu = {P.wgu, 2 * f, d, 32, nullptr};
    DtGemm gdown = {P.wdown, d, f, 16, P.ff};
    DtGemm gqkv = {P.wqkv, 3 * d, d, 16, nullptr};

    // first weight chunk of the phase after `done`, for the tile this CTA will take there (if any)
    auto prefetch_next = [&](uint32_t done) -> bool {
        const DtGemm* g = nullptr;
        if (done < DT_PHASE_GU && (P.phases & DT_PHASE_GU)) g = &ggu;
        else if (done < DT_PHASE_DOWN && (P.phases & DT_PHASE_DOWN)) g = &gdown;
        else if (done < DT_PHASE_QKV && (P.phases & DT_PHASE_QKV)) g = &gqkv;
        if (!g) return false;
        const uint32_t n0 = blockIdx.x * g->cols;
        if (n0 >= g->n) return false;
        dt_issue_w<MT>(*g, n0, 0, wbuf);
        return true;
    };

    bool w0 = false;
    // ---------------- output projection: h += att . Wo^T + bo ----------------
    if (P.phases & DT_PHASE_O) {
        for (uint32_t n0 = blockIdx.x * 16; n0 < d; n0 += gridDim.x * 16) {
            dt_gemm_tile<MT>(go, rows, n0, wbuf, abuf, nullptr, 0, red, false);
            for (uint32_t o = threadIdx.x; o < 16u * MT; o += DT_THREADS) {
                const uint32_t c = o % 16, m = o / 16;
                if (m < rows && n0 + c < d) {
                    float* p = P.h + (size_t)m * d + n0 + c;
                    *p = __ldcg(p) + (red[c * MT + m] + __ldg(P.bo + n0 + c));
                }
            }
            __syncthreads();
        }
        w0 = prefetch_next(DT_PHASE_O);
        if (P.phases & ~(DT_PHASE_O | (DT_PHASE_O - 1))) ok = dt_grid_barrier(P, barriers++, s_abort);
    }
    // ---------------- LayerNorm, gate/up projection, SwiGLU -> ff ----------------
    if (ok && (P.phases & DT_PHASE_GU)) {
        // the LayerNorm output lives where the streamed activation chunks would: this phase streams none
        dt_layernorm<MT>(P, P.ln2w, P.ln2b, nbuf);
        __syncthreads();
        for (uint32_t n0 = blockIdx.x * 32; n0 < 2 * f; n0 += gridDim.x * 32) {
            dt_gemm_tile<MT>(ggu, rows, n0, wbuf, abuf, nbuf, npitch, red, w0);
            w0 = false;
            // packed columns [0, 16) are gate, [16, 32) the matching up columns -> 16 outputs
            for (uint32_t o = threadIdx.x; o < 16u * MT; o += DT_THREADS) {
                const uint32_t j = o % 16, m = o / 16;
                if (m < rows) {
                    const float gte = red[j * MT + m] + __ldg(P.bgu + n0 + j);
                    const float up = red[(16 + j) * MT + m] + __ldg(P.bgu + n0 + 16 + j);
                    P.ff[(size_t)m * f + n0 / 2 + j] = __float2bfloat16_rn(fast_silu(gte) * up);
                }
            }
            __syncthreads();
        }
        w0 = prefetch_next(DT_PHASE_GU);
        if (P.phases & (DT_PHASE_DOWN | DT_PHASE_QKV)) ok = dt_grid_barrier(P, barriers++, s_abort);
    }
    // ---------------- down projection: h += ff . Wdown^T + bdown ----------------
    if (ok && (P.phases & DT_PHASE_DOWN)) {
        for (uint32_t n0 = blockIdx.x * 16; n0 < d; n0 += gridDim.x * 16) {
            dt_gemm_tile<MT>(gdown, rows, n0, wbuf, abuf, nullptr, 0, red, w0);
            w0 = false;
            for (uint32_t o = threadIdx.x; o < 16u * MT; o += DT_THREADS) {
                const uint32_t c = o % 16, m = o / 16;
                if (m < rows && n0 + c < d) {
                    float* p = P.h + (size_t)m * d + n0 + c;
                    *p = __ldcg(p) + (red[c * MT + m] + __ldg(P.bdown + n0 + c));
                }
            }
            __syncthreads();
        }
        w0 = prefetch_next(DT_PHASE_DOWN);
        if (P.phases & DT_PHASE_QKV) ok = dt_grid_barrier(P, barriers++, s_abort);
    }
    // ---------------- next layer: LayerNorm, QKV projection, K/V rows into the cache ----------------
    if (ok && (P.phases & DT_PHASE_QKV)) {
        dt_layernorm<MT>(P, P.ln1w, P.ln1b, nbuf);
        __syncthreads();
        for (uint32_t n0 = blockIdx.x * 16; n0 < 3 * d; n0 += gridDim.x * 16) {
            dt_gemm_tile<MT>(gqkv, rows, n0, wbuf, abuf, nbuf, npitch, red, w0);
            w0 = false;
            for (uint32_t o = threadIdx.x; o < 16u * MT; o += DT_THREADS) {
                const uint32_t c = o % 16, m = o / 16, col = n0 + c;
                if (m < rows && col < 3 * d) {
                    const bf16 v = __float2bfloat16_rn(red[c * MT + m] + __ldg(P.bqkv + col));
                    const uint32_t which = col / d, cc = col % d;
                    if (which == 0) {
                        P.q[(size_t)m * d + cc] = v;
                    } else {
                        const uint32_t pos = P.d_position ? P.d_position[(size_t)m * P.position_stride] : P.position;
                        const size_t crow = kv_row(P.paging, P.first_session + m, pos, P.capacity);
                        (which == 1 ? P.k_cache : P.v_cache)[crow * d + cc] = v;
                    }
                }
            }
            __syncthreads();
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
    const size_t act = std::max((size_t)2 * MT * DT_PITCH, (size_t)MT * (DT_MAX_D + 8));
    return (size_t)2 * DT_MAX_COLS * DT_PITCH * 2 + act * 2 + (size_t)DT_MAX_COLS * MT * 4 + 16;
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
    return rows >= 1 && rows <= 64 && d % 16 == 0 && d <= DT_MAX_D && f % 16 == 0 && f >= 16;
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
    if (a.rows <= 32) return dt_launch<32>(P, stream);
    return dt_launch<64>(P, stream);
}

}  // namespace tb
