// HBM-bound kernels of the cached-GPT path: embedding gather-add, LayerNorm,
// SwiGLU, greedy pick, and the one-time weight repacking done at upload.
// All of them move 16 bytes per thread per access where alignment allows.
#include "common.cuh"

namespace tb {

thread_local bool t_single_token_step = false;


int launch_layernorm_strict(const float* x, const float* w, const float* b, float* out, uint32_t rows,
                            uint32_t width, float eps, cudaStream_t stream);

// ---------------------------------------------------------------------------
// Embedding: out[r, :] = tok[ids[r], :] + pos[position + r % chunk, :]
// (src/nn/kv_cache/graph.rs:30-41).  The gather is an exact copy and the sum one
// f32 add per element, so f32 tables reproduce the reference bit for bit.
// One block per row; 4 elements per thread per step.
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 load4<bf16>(const bf16* p) {
    uint2 v = *reinterpret_cast<const uint2*>(p);
    float2 a = bf16x2_to_f32(v.x), b = bf16x2_to_f32(v.y);
    return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T>
__device__ __forceinline__ float load1(const T* p);
template <>
__device__ __forceinline__ float load1<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load1<bf16>(const bf16* p) { return __bfloat162float(*p); }

template <typename T>
__global__ void __launch_bounds__(128)
embedding_kernel(const T* __restrict__ tok, const T* __restrict__ pos, const uint32_t* __restrict__ ids,
                 float* __restrict__ out, uint32_t chunk, uint32_t position0,
                 const uint32_t* __restrict__ d_position, uint32_t position_stride, uint32_t vocab, uint32_t width,
                 int* __restrict__ d_status) {
    pdl_wait();
    pdl_trigger();
    const uint32_t r = blockIdx.x;
    // position_stride 0: one position for all sessions; 1: d_position[session]
    const uint32_t position = (d_position ? d_position[(r / chunk) * position_stride] : position0) + r % chunk;
    uint32_t id = ids[r];
    float* o = out + (size_t)r * width;
    if (id >= vocab) {
        if (threadIdx.x == 0 && d_status) atomicCAS(d_status, DEV_OK, DEV_TOKEN_RANGE);
        for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) o[c] = 0.0f;
        return;
    }
    const T* tr = tok + (size_t)id * width;
    const T* pr = pos + (size_t)position * width;
    if (width % 4 == 0) {
        for (uint32_t c = threadIdx.x * 4; c < width; c += blockDim.x * 4) {
            float4 a = load4<T>(tr + c), b = load4<T>(pr + c);
            *reinterpret_cast<float4*>(o + c) =
                make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
        }
    } else {
        for (uint32_t c = threadIdx.x; c < width; c += blockDim.x)
            o[c] = __fadd_rn(load1<T>(tr + c), load1<T>(pr + c));
    }
}

int launch_embedding(const void* tok, const void* pos, const uint32_t* ids, float* out, uint32_t rows,
                     uint32_t chunk, uint32_t position0, const uint32_t* d_position, uint32_t vocab,
                     uint32_t width, int dtype, int* d_status, cudaStream_t stream, uint32_t position_stride) {
    if (rows == 0) return TNSR_B200_OK;
    if (chunk == 0) return TNSR_B200_ERR_INVALID_ARGUMENT;
    if (dtype == TNSR_B200_BF16)
        launch_kernel(embedding_kernel<bf16>, dim3(rows), dim3(128), 0, stream, (const bf16*)tok, (const bf16*)pos, ids, out,
                      chunk, position0, d_position, position_stride, vocab, width, d_status);
    else
        launch_kernel(embedding_kernel<float>, dim3(rows), dim3(128), 0, stream, (const float*)tok, (const float*)pos, ids, out,
                      chunk, position0, d_position, position_stride, vocab, width, d_status);
    count_launch();
    return check_launch("embedding");
}

// ---------------------------------------------------------------------------
// LayerNorm, fast form: one warp per row, the row kept in registers (up to
// 32 * 4 * LN_MAX_VEC columns), two-pass mean / variance with warp shuffles,
// rsqrt for the inverse deviation.  Reads 4 B/element, writes 2 B (bf16) or
// 4 B (f32): purely HBM-bound.
// ---------------------------------------------------------------------------
constexpr int LN_MAX_VEC = 8;  // float4 per lane -> rows up to 1024 columns stay in registers

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <bool OUT_BF16>
__global__ void __launch_bounds__(128)
layernorm_warp_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                      void* __restrict__ out, uint32_t rows, uint32_t width, float eps) {
    pdl_wait();
    pdl_trigger();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * width);
    const uint32_t nvec = width >> 2;
    float4 v[LN_MAX_VEC];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < LN_MAX_VEC; ++i) {
        uint32_t c = lane + i * 32;
        if (c < nvec) {
            v[i] = xr[c];
            sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
    }
    const float mean = warp_sum(sum) / (float)width;
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < LN_MAX_VEC; ++i) {
        uint32_t c = lane + i * 32;
        if (c < nvec) {
            v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
            sq += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
        }
    }
    const float inv = rsqrtf(warp_sum(sq) / (float)width + eps);
    const float4* wr = reinterpret_cast<const float4*>(w);
    const float4* br = reinterpret_cast<const float4*>(b);
#pragma unroll
    for (int i = 0; i < LN_MAX_VEC; ++i) {
        uint32_t c = lane + i * 32;
        if (c < nvec) {
            float4 ww = wr[c], bb = br[c];
            float4 y = make_float4(v[i].x * inv * ww.x + bb.x, v[i].y * inv * ww.y + bb.y,
                                   v[i].z * inv * ww.z + bb.z, v[i].w * inv * ww.w + bb.w);
            if (OUT_BF16) {
                uint2 p = make_uint2(pack_bf16x2(y.x, y.y), pack_bf16x2(y.z, y.w));
                reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + (size_t)row * width)[c] = p;
            } else {
                reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)row * width)[c] = y;
            }
        }
    }
}

// LayerNorm (bf16 out) of h + the partial sums of a split-K residual GEMM: the row is first completed (h + p0 + p1 +
// ..., in that order) and written back, then normalised (two passes, rsqrt of the biased variance).  One block per row,
// one float4 per thread: the row, its partial rows and the scale and shift are up to seven independent loads per thread,
// one L2 round trip in all (a warp per row with the partial rows fetched one after the other took 7.7 us per launch,
// and with all 40 loads of a lane written ahead of their uses 15 us: they came out one by one).
constexpr uint32_t LN_FOLD_MAX = 4;        // partial rows per call (gemm_split_k never asks for more)
constexpr uint32_t LN_FOLD_THREADS = 256;  // float4 per row: widths up to 1024

__device__ __forceinline__ float ln_fold_block_sum(float x, float* red) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    x = warp_sum(x);
    if (lane == 0) red[warp] = x;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (uint32_t i = 0; i < LN_FOLD_THREADS / 32; ++i) t += red[i];
    __syncthreads();           // `red` is reused by the next sum
    return t;
}

__global__ void __launch_bounds__(LN_FOLD_THREADS)
layernorm_fold_kernel(float* __restrict__ h, const float* __restrict__ partials, uint32_t split_k, uint32_t split_rows,
                      const float* __restrict__ w, const float* __restrict__ b, bf16* __restrict__ out, uint32_t rows,
                      uint32_t width, float eps) {
    __shared__ float red[LN_FOLD_THREADS / 32];
    pdl_wait();
    pdl_trigger();
    const uint32_t row = blockIdx.x, c = threadIdx.x;
    const bool live = c < (width >> 2);
    float4* xr = reinterpret_cast<float4*>(h + (size_t)row * width);
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 v = zero, ww = zero, bb = zero, p[LN_FOLD_MAX];
    if (live) {
        v = xr[c];
        ww = reinterpret_cast<const float4*>(w)[c];
        bb = reinterpret_cast<const float4*>(b)[c];
    }
#pragma unroll
    for (uint32_t s = 0; s < LN_FOLD_MAX; ++s)
        p[s] = (live && s < split_k) ? reinterpret_cast<const float4*>(partials + ((size_t)s * split_rows + row) * width)[c] : zero;
#pragma unroll
    for (uint32_t s = 0; s < LN_FOLD_MAX; ++s) {
        if (s < split_k) { v.x += p[s].x; v.y += p[s].y; v.z += p[s].z; v.w += p[s].w; }
    }
    if (live && split_k) xr[c] = v;
    const float mean = ln_fold_block_sum(live ? (v.x + v.y) + (v.z + v.w) : 0.0f, red) / (float)width;
    v.x -= mean; v.y -= mean; v.z -= mean; v.w -= mean;
    const float sq = ln_fold_block_sum(live ? (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w) : 0.0f, red);
    const float inv = rsqrtf(sq / (float)width + eps);
    if (live)
        reinterpret_cast<uint2*>(out + (size_t)row * width)[c] =
            make_uint2(pack_bf16x2(v.x * inv * ww.x + bb.x, v.y * inv * ww.y + bb.y),
                       pack_bf16x2(v.z * inv * ww.z + bb.z, v.w * inv * ww.w + bb.w));
    (void)rows;
}

// Any width: one block per row, three passes over global memory (L2-resident).
template <bool OUT_BF16>
__global__ void __launch_bounds__(256)
layernorm_block_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                       void* __restrict__ out, uint32_t width, float eps) {
    __shared__ float red[8];
    __shared__ float bc;
    pdl_wait();
    pdl_trigger();
    const float* xr = x + (size_t)blockIdx.x * width;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float sum = 0.0f;
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) sum += xr[c];
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int i = 0; i < 8; ++i) t += red[i];
        bc = t / (float)width;
    }
    __syncthreads();
    const float mean = bc;
    float sq = 0.0f;
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) {
        float d = xr[c] - mean;
        sq += d * d;
    }
    sq = warp_sum(sq);
    __syncthreads();
    if (lane == 0) red[warp] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int i = 0; i < 8; ++i) t += red[i];
        bc = rsqrtf(t / (float)width + eps);
    }
    __syncthreads();
    const float inv = bc;
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) {
        float y = (xr[c] - mean) * inv * w[c] + b[c];
        if (OUT_BF16) reinterpret_cast<bf16*>(out)[(size_t)blockIdx.x * width + c] = __float2bfloat16_rn(y);
        else reinterpret_cast<float*>(out)[(size_t)blockIdx.x * width + c] = y;
    }
}

int launch_layernorm(const float* x, const float* w, const float* b, void* out, uint32_t rows,
                     uint32_t width, float eps, int out_dtype, bool strict, cudaStream_t stream) {
    if (rows == 0) return TNSR_B200_OK;
    if (strict) {
        if (out_dtype != TNSR_B200_F32) {
            set_thread_error("strict LayerNorm writes f32 only");
            return TNSR_B200_ERR_UNSUPPORTED;
        }
        return launch_layernorm_strict(x, w, b, (float*)out, rows, width, eps, stream);
    }
    const bool vec_ok = width % 4 == 0 && width <= 32 * 4 * LN_MAX_VEC &&
                        (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(w) % 16 == 0) &&
                        (reinterpret_cast<uintptr_t>(b) % 16 == 0) && (reinterpret_cast<uintptr_t>(out) % 16 == 0);
    // Single-token steps (few rows): one block per row with every load of a thread issued at once (layernorm_fold_kernel
    // with nothing to fold); the row-per-warp kernel fetches scale and shift only after the statistics, a second round
    // trip that a launch of a few hundred rows has nothing to hide behind.  Many rows (prefill): row per warp, which
    // runs at 0.94 of the HBM copy rate.
    if (vec_ok && out_dtype == TNSR_B200_BF16 && t_single_token_step) {
        launch_kernel(layernorm_fold_kernel, dim3(rows), dim3(LN_FOLD_THREADS), 0, stream, const_cast<float*>(x),
                      static_cast<const float*>(nullptr), 0u, 0u, w, b, reinterpret_cast<bf16*>(out), rows, width, eps);
        count_launch();
        return check_launch("layernorm");
    }
    if (vec_ok) {
        dim3 grid(ceil_div(rows, 4));
        if (out_dtype == TNSR_B200_BF16)
            launch_kernel(layernorm_warp_kernel<true>, grid, dim3(128), 0, stream, x, w, b, out, rows, width, eps);
        else
            launch_kernel(layernorm_warp_kernel<false>, grid, dim3(128), 0, stream, x, w, b, out, rows, width, eps);
    } else {
        if (out_dtype == TNSR_B200_BF16)
            launch_kernel(layernorm_block_kernel<true>, dim3(rows), dim3(256), 0, stream, x, w, b, out, width, eps);
        else
            launch_kernel(layernorm_block_kernel<false>, dim3(rows), dim3(256), 0, stream, x, w, b, out, width, eps);
    }
    count_launch();
    return check_launch("layernorm");
}

bool layernorm_fold_supported(uint32_t width) { return width % 4 == 0 && width <= LN_FOLD_THREADS * 4; }

int launch_layernorm_fold(float* h, const float* partials, uint32_t split_k, uint32_t split_rows, const float* w, const float* b,
                          void* out, uint32_t rows, uint32_t width, float eps, cudaStream_t stream) {
    if (rows == 0) return TNSR_B200_OK;
    const bool aligned = (reinterpret_cast<uintptr_t>(h) % 16 == 0) && (reinterpret_cast<uintptr_t>(partials) % 16 == 0) &&
                         (reinterpret_cast<uintptr_t>(w) % 16 == 0) && (reinterpret_cast<uintptr_t>(b) % 16 == 0) &&
                         (reinterpret_cast<uintptr_t>(out) % 8 == 0);
    if (!layernorm_fold_supported(width) || !aligned || split_k == 0 || split_k > LN_FOLD_MAX || split_rows < rows) {
        set_thread_error("layernorm_fold: width, alignment or partial layout outside the kernel");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    launch_kernel(layernorm_fold_kernel, dim3(rows), dim3(LN_FOLD_THREADS), 0, stream, h, partials, split_k, split_rows, w, b,
                  reinterpret_cast<bf16*>(out), rows, width, eps);
    count_launch();
    return check_launch("layernorm_fold");
}

// ---------------------------------------------------------------------------
__global__ void gather_last_rows_kernel(const float* __restrict__ x, float* __restrict__ out, uint32_t chunk,
                                        uint32_t width) {
    pdl_wait();
    pdl_trigger();
    const float* src = x + ((size_t)blockIdx.x * chunk + chunk - 1) * width;
    float* dst = out + (size_t)blockIdx.x * width;
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
}

int launch_gather_last_rows(const float* x, float* out, uint32_t sessions, uint32_t chunk, uint32_t width,
                            cudaStream_t stream) {
    if (sessions == 0) return TNSR_B200_OK;
    launch_kernel(gather_last_rows_kernel, dim3(sessions), dim3(128), 0, stream, x, out, chunk, width);
    count_launch();
    return check_launch("gather_last_rows");
}

// ---------------------------------------------------------------------------
// Greedy pick: `max_by(total_cmp)` keeps the LAST index of the maximum under
// IEEE totalOrder (src/nn/kv_cache.rs:148-153).  Keys are the sign-folded bit
// patterns, compared as signed integers; ties prefer the larger index.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, uint32_t* __restrict__ out, uint32_t vocab, uint32_t row_stride) {
    __shared__ int keys[32];
    __shared__ uint32_t idxs[32];
    pdl_wait();
    pdl_trigger();
    const float* row = logits + (size_t)blockIdx.x * row_stride;
    int best = INT_MIN;
    uint32_t best_i = 0;
    bool have = false;
    auto take = [&](float v, uint32_t i) {
        const int key = total_order_key(v);
        if (!have || key >= best) { best = key; best_i = i; have = true; }
    };
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0 && vocab % 4 == 0) {
        // 16-byte loads, four in flight per thread before the first compare
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const uint32_t n4 = vocab >> 2, step = blockDim.x;
        uint32_t i = threadIdx.x;
        for (; i + 3 * step < n4; i += 4 * step) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = __ldcs(row4 + i + u * step);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t base = (i + u * step) << 2;
                take(v[u].x, base); take(v[u].y, base + 1); take(v[u].z, base + 2); take(v[u].w, base + 3);
            }
        }
        for (; i < n4; i += step) {
            const float4 v = __ldcs(row4 + i);
            take(v.x, 4 * i); take(v.y, 4 * i + 1); take(v.z, 4 * i + 2); take(v.w, 4 * i + 3);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < vocab; i += blockDim.x) take(row[i], i);
    }
    // per-thread scan visits indices in increasing order, so >= keeps the last; merge likewise
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        int ok = __shfl_xor_sync(0xffffffffu, best, o);
        uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        int oh = __shfl_xor_sync(0xffffffffu, (int)have, o);
        if (oh && (!have || ok > best || (ok == best && oi > best_i))) { best = ok; best_i = oi; have = true; }
    }
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { keys[warp] = have ? best : INT_MIN; idxs[warp] = have ? best_i : 0; }
    __syncthreads();
    if (threadIdx.x == 0) {
        int bk = INT_MIN;
        uint32_t bi = 0;
        bool any = false;
        for (int wi = 0; wi < (int)(blockDim.x >> 5); ++wi) {
            // a warp with no element reports INT_MIN at index 0; a real INT_MIN key can only
            // lose or tie against it, and ties resolve towards the larger index
            if (!any || keys[wi] > bk || (keys[wi] == bk && idxs[wi] > bi)) { bk = keys[wi]; bi = idxs[wi]; any = true; }
        }
        out[blockIdx.x] = bi;
    }
}

int launch_argmax(const float* logits, uint32_t* out, uint32_t rows, uint32_t vocab, uint32_t row_stride,
                  cudaStream_t stream) {
    if (rows == 0) return TNSR_B200_OK;
    launch_kernel(argmax_kernel, dim3(rows), dim3(vocab >= 8192 ? 1024 : 256), 0, stream, logits, out, vocab, row_stride);
    count_launch();
    return check_launch("argmax");
}

// ---------------------------------------------------------------------------
// SwiGLU elementwise: y = silu(gate) * up, bf16 in/out, 8 elements per thread.
// 6 bytes of traffic per element.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
swiglu_kernel(const bf16* __restrict__ gate, const bf16* __restrict__ up, bf16* __restrict__ out, uint64_t elems) {
    pdl_wait();
    pdl_trigger();
    const uint64_t nvec = elems >> 3;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (uint64_t)gridDim.x * blockDim.x) {
        uint4 g = reinterpret_cast<const uint4*>(gate)[i], u = reinterpret_cast<const uint4*>(up)[i], y;
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
        uint32_t yw[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 a = bf16x2_to_f32(gw[k]), b = bf16x2_to_f32(uw[k]);
            yw[k] = pack_bf16x2(fast_silu(a.x) * b.x, fast_silu(a.y) * b.y);
        }
        y = make_uint4(yw[0], yw[1], yw[2], yw[3]);
        reinterpret_cast<uint4*>(out)[i] = y;
    }
    // tail
    if (blockIdx.x == 0) {
        for (uint64_t i = (nvec << 3) + threadIdx.x; i < elems; i += blockDim.x)
            out[i] = __float2bfloat16_rn(fast_silu(__bfloat162float(gate[i])) * __bfloat162float(up[i]));
    }
}

int launch_swiglu(const bf16* gate, const bf16* up, bf16* out, uint64_t elems, cudaStream_t stream) {
    if (elems == 0) return TNSR_B200_OK;
    if ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(out)) % 16) {
        set_thread_error("swiglu: pointers must be 16-byte aligned");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    uint64_t want = ceil_div64(ceil_div64(elems, 8), 256);
    unsigned grid = (unsigned)(want < 148ull * 16 ? (want ? want : 1) : 148ull * 16);
    launch_kernel(swiglu_kernel, dim3(grid), dim3(256), 0, stream, gate, up, out, elems);
    count_launch();
    return check_launch("swiglu");
}

// ---------------------------------------------------------------------------
// Repacking (upload time, not on the hot path).
// ---------------------------------------------------------------------------
// in [k, n] row-major -> out rows of k bf16 each.  Output row of input column j:
//   row0 + (j / block) * block_stride + j % block
// (block = n, block_stride = n gives the plain transpose at row offset row0).
template <typename TIN>
__global__ void __launch_bounds__(256)
transpose_to_bf16_kernel(const TIN* __restrict__ in, bf16* __restrict__ out, uint32_t k, uint32_t n, uint32_t row0,
                         uint32_t block, uint32_t block_stride) {
    __shared__ float tile[32][33];
    const uint32_t bx = blockIdx.x * 32, by = blockIdx.y * 32;
    for (uint32_t r = threadIdx.y; r < 32; r += 8) {
        uint32_t p = by + r, j = bx + threadIdx.x;
        tile[r][threadIdx.x] = (p < k && j < n) ? load1<TIN>(in + (size_t)p * n + j) : 0.0f;
    }
    __syncthreads();
    for (uint32_t r = threadIdx.y; r < 32; r += 8) {
        uint32_t j = bx + r, p = by + threadIdx.x;
        if (j < n && p < k) {
            size_t orow = (size_t)row0 + (size_t)(j / block) * block_stride + j % block;
            out[orow * k + p] = __float2bfloat16_rn(tile[threadIdx.x][r]);
        }
    }
}

int launch_transpose_bf16(const bf16* in, bf16* out, uint32_t k, uint32_t n, cudaStream_t stream) {
    if (k == 0 || n == 0) return TNSR_B200_OK;
    dim3 grid(ceil_div(n, 32), ceil_div(k, 32)), block(32, 8);
    transpose_to_bf16_kernel<bf16><<<grid, block, 0, stream>>>(in, out, k, n, 0, n, n);
    count_launch();
    return check_launch("transpose_bf16");
}

int launch_transpose_f32_to_bf16_mapped(const float* in, bf16* out, uint32_t k, uint32_t n, uint32_t row0,
                                        uint32_t block, uint32_t block_stride, cudaStream_t stream) {
    if (k == 0 || n == 0) return TNSR_B200_OK;
    dim3 grid(ceil_div(n, 32), ceil_div(k, 32)), blk(32, 8);
    transpose_to_bf16_kernel<float><<<grid, blk, 0, stream>>>(in, out, k, n, row0, block ? block : n,
                                                              block ? block_stride : n);
    count_launch();
    return check_launch("transpose_f32_to_bf16");
}

int launch_transpose_f32_to_bf16(const float* in, bf16* out, uint32_t k, uint32_t n, cudaStream_t stream) {
    return launch_transpose_f32_to_bf16_mapped(in, out, k, n, 0, n, n, stream);
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, bf16* __restrict__ out, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void bf16_to_f32_kernel(const bf16* __restrict__ in, float* __restrict__ out, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        out[i] = __bfloat162float(in[i]);
}

static unsigned flat_grid(uint64_t n) {
    uint64_t want = ceil_div64(n, 256);
    return (unsigned)(want < 148ull * 32 ? (want ? want : 1) : 148ull * 32);
}

int launch_f32_to_bf16(const float* in, bf16* out, uint64_t elems, cudaStream_t stream) {
    if (elems == 0) return TNSR_B200_OK;
    f32_to_bf16_kernel<<<flat_grid(elems), 256, 0, stream>>>(in, out, elems);
    count_launch();
    return check_launch("f32_to_bf16");
}

int launch_bf16_to_f32(const bf16* in, float* out, uint64_t elems, cudaStream_t stream) {
    if (elems == 0) return TNSR_B200_OK;
    bf16_to_f32_kernel<<<flat_grid(elems), 256, 0, stream>>>(in, out, elems);
    count_launch();
    return check_launch("bf16_to_f32");
}

// Gate/up packing: row (32*g + i) of the packed [2f, d] matrix is gate row
// 16*g + i for i < 16 and up row 16*g + i - 16 otherwise; inputs are the
// reference's [d, f] row-major matrices, so this is also the transpose.
__global__ void __launch_bounds__(256)
pack_gate_up_kernel(const bf16* __restrict__ wg, const bf16* __restrict__ wu, const float* __restrict__ bg,
                    const float* __restrict__ bu, bf16* __restrict__ w_out, float* __restrict__ b_out,
                    uint32_t d, uint32_t f) {
    const uint64_t total = (uint64_t)2 * f * d;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t row = (uint32_t)(i / d), p = (uint32_t)(i % d);
        uint32_t g = row / 32, r = row % 32;
        uint32_t col = g * 16 + (r & 15);
        bf16 v = __float2bfloat16_rn(0.0f);
        if (col < f) v = (r < 16 ? wg : wu)[(size_t)p * f + col];
        w_out[i] = v;
        if (p == 0 && b_out) {
            float bv = 0.0f;
            if (col < f) {
                const float* src = (r < 16) ? bg : bu;
                bv = src ? src[col] : 0.0f;
            }
            b_out[row] = bv;
        }
    }
}

int launch_pack_gate_up(const bf16* wg, const bf16* wu, const float* bg, const float* bu, bf16* w_out,
                        float* b_out, uint32_t d, uint32_t f, cudaStream_t stream) {
    if (d == 0 || f == 0) return TNSR_B200_OK;
    if (f % 16 != 0) {
        set_thread_error("pack_gate_up: feed-forward width must be a multiple of 16");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    pack_gate_up_kernel<<<flat_grid((uint64_t)2 * f * d), 256, 0, stream>>>(wg, wu, bg, bu, w_out, b_out, d, f);
    count_launch();
    return check_launch("pack_gate_up");
}

__global__ void fill_u32_kernel(uint32_t* p, uint32_t value, uint32_t n) {
    pdl_wait();
    pdl_trigger();
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = value;
}
__global__ void add_u32_kernel(uint32_t* p, uint32_t delta) { *p += delta; }

int launch_fill_u32(uint32_t* p, uint32_t value, uint32_t n, cudaStream_t stream) {
    if (n == 0) return TNSR_B200_OK;
    launch_kernel(fill_u32_kernel, dim3(ceil_div(n, 256)), dim3(256), 0, stream, p, value, n);
    count_launch();
    return check_launch("fill_u32");
}

int launch_add_u32(uint32_t* p, uint32_t delta, cudaStream_t stream) {
    add_u32_kernel<<<1, 1, 0, stream>>>(p, delta);
    count_launch();
    return check_launch("add_u32");
}

}  // namespace tb
