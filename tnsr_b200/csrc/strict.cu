// Strict f32 kernels: the arithmetic of tnsr's CPU executor, operation by
// operation, for sessions created with weight_dtype = F32.
//
// This file is compiled with --fmad=false so that no multiply is fused into a
// following add: the reference rounds every product before adding it
// (src/lib.rs:1202-1208) and its own GPU decoder forces the same with
// MatMulPrecision::StrictF32 (src/nn/kv_cache/cuda.rs:480-486).  Reductions run
// in increasing index order from a zero start.  exp/ln go through the f64
// routines and are rounded once to f32, which is the nearest-f32 result the
// host libm delivers in all but rare last-bit cases.
#include "common.cuh"

namespace tb {

__device__ __forceinline__ float strict_expf(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float strict_logf(float x) { return (float)log((double)x); }

// nn::sigmoid op by op (src/nn/activations.rs:5-14).
__device__ __forceinline__ float strict_sigmoid(float x) {
    float negative = (-x > 0.0f) ? 1.0f : 0.0f;
    float nonnegative = 1.0f - negative;
    float magnitude = x * (1.0f - negative * 2.0f);
    float z = strict_expf(-magnitude);
    float denominator = z + 1.0f;
    float a = (nonnegative != 0.0f) ? (1.0f / denominator) : 0.0f;
    float b = (negative != 0.0f) ? (z / denominator) : 0.0f;
    return a + b;
}

// nn::gelu op by op (src/nn/activations.rs:29-47).
__device__ __forceinline__ float strict_gelu(float x) {
    float negative = (-x > 0.0f) ? 1.0f : 0.0f;
    float nonnegative = 1.0f - negative;
    float magnitude = (x * (1.0f - negative * 2.0f)) * 0.70710678118654752440f;
    float t = 1.0f / (magnitude * 0.3275911f + 1.0f);
    float polynomial =
        ((((t * 1.0614054f - 1.4531521f) * t + 1.4214138f) * t - 0.28449672f) * t + 0.2548296f) * t;
    float tail = (polynomial * strict_expf(-(magnitude * magnitude))) * 0.5f;
    float a = (nonnegative != 0.0f) ? (1.0f - tail) : 0.0f;
    float b = (negative != 0.0f) ? tail : 0.0f;
    return x * (a + b);
}

// ---------------------------------------------------------------------------
// GEMM: one thread per output element, K walked in order through 16-wide
// shared tiles.  The tiling changes which thread loads what, not the order in
// which any output's products are added.
// ---------------------------------------------------------------------------
constexpr int ST = 16;

template <bool BT>
__global__ void __launch_bounds__(ST* ST)
gemm_strict_kernel(const float* __restrict__ a, const float* __restrict__ b, void* __restrict__ out,
                   uint32_t ldc, uint32_t m, uint32_t k, uint32_t n, GemmEpilogue ep) {
    __shared__ float as[ST][ST + 1];
    __shared__ float bs[ST][ST + 1];
    const uint32_t tx = threadIdx.x, ty = threadIdx.y;
    const uint32_t row = blockIdx.y * ST + ty, col = blockIdx.x * ST + tx;
    float sum = 0.0f;
    for (uint32_t k0 = 0; k0 < k; k0 += ST) {
        uint32_t ka = k0 + tx;
        as[ty][tx] = (row < m && ka < k) ? a[(size_t)row * k + ka] : 0.0f;
        if (BT) {
            // b is [n, k]: element (p, j) lives at b[j * k + p]
            uint32_t j = blockIdx.x * ST + ty, p = k0 + tx;
            bs[tx][ty] = (j < n && p < k) ? b[(size_t)j * k + p] : 0.0f;
        } else {
            uint32_t p = k0 + ty;
            bs[ty][tx] = (p < k && col < n) ? b[(size_t)p * n + col] : 0.0f;
        }
        __syncthreads();
        const uint32_t lim = min((uint32_t)ST, k - k0);
        for (uint32_t p = 0; p < lim; ++p) sum = sum + as[ty][p] * bs[p][tx];
        __syncthreads();
    }
    if (row >= m || col >= n) return;
    float v = sum;
    if (ep.bias) v = v + ep.bias[col];
    if (ep.activation == ACT_RELU) v = fmaxf(v, 0.0f);
    else if (ep.activation == ACT_GELU) v = strict_gelu(v);
    if (ep.residual) v = ep.residual[(size_t)row * ep.ldr + col] + v;
    if (ep.round_bf16) v = round_to_bf16(v);
    size_t orow = row;
    if (ep.rows_per_session) {
        uint32_t off = ep.d_row_offset ? *ep.d_row_offset : ep.row_offset;
        orow = (size_t)(row / ep.rows_per_session) * ep.out_session_rows + off + row % ep.rows_per_session;
    }
    if (ep.out_dtype == TNSR_B200_BF16)
        reinterpret_cast<bf16*>(out)[orow * ldc + col] = __float2bfloat16_rn(v);
    else
        reinterpret_cast<float*>(out)[orow * ldc + col] = v;
}

// Few rows (decode steps, short prefills): one block per (row, 32 output columns).  The sum of an output is
// still ONE sequential chain in increasing k -- that is the reference's arithmetic -- but the terms are
// independent of the chain, so all 512 threads first form the rounded products a[row,p] * b[p,col] side by
// side into shared memory (every global load of the block is in flight at once), and then one lane per column
// walks its K products in order.  Same values, same order of additions as gemm_strict_kernel.
constexpr int SR_COLS = 32, SR_THREADS = 512;

template <bool BT>
__global__ void __launch_bounds__(SR_THREADS)
gemm_strict_rows_kernel(const float* __restrict__ a, const float* __restrict__ b, void* __restrict__ out,
                        uint32_t ldc, uint32_t m, uint32_t k, uint32_t n, GemmEpilogue ep) {
    extern __shared__ float prod[];   // [k][SR_COLS]
    const uint32_t row = blockIdx.y, col0 = blockIdx.x * SR_COLS;
    const float* ar = a + (size_t)row * k;
    if (BT) {
        // b is [n, k]: lanes run along p so that a warp reads one contiguous piece of a b row
        for (uint32_t e = threadIdx.x; e < k * SR_COLS; e += SR_THREADS) {
            const uint32_t c = e / k, p = e % k, col = col0 + c;
            prod[p * SR_COLS + c] = col < n ? ar[p] * b[(size_t)col * k + p] : 0.0f;
        }
    } else {
        for (uint32_t e = threadIdx.x; e < k * SR_COLS; e += SR_THREADS) {
            const uint32_t p = e / SR_COLS, c = e % SR_COLS, col = col0 + c;
            prod[e] = col < n ? ar[p] * b[(size_t)p * n + col] : 0.0f;
        }
    }
    __syncthreads();
    const uint32_t col = col0 + threadIdx.x;
    if (threadIdx.x >= SR_COLS || col >= n) return;
    float sum = 0.0f;
#pragma unroll 8
    for (uint32_t p = 0; p < k; ++p) sum = sum + prod[p * SR_COLS + threadIdx.x];
    float v = sum;
    if (ep.bias) v = v + ep.bias[col];
    if (ep.activation == ACT_RELU) v = fmaxf(v, 0.0f);
    else if (ep.activation == ACT_GELU) v = strict_gelu(v);
    if (ep.residual) v = ep.residual[(size_t)row * ep.ldr + col] + v;
    if (ep.round_bf16) v = round_to_bf16(v);
    size_t orow = row;
    if (ep.rows_per_session) {
        uint32_t off = ep.d_row_offset ? *ep.d_row_offset : ep.row_offset;
        orow = (size_t)(row / ep.rows_per_session) * ep.out_session_rows + off + row % ep.rows_per_session;
    }
    if (ep.out_dtype == TNSR_B200_BF16)
        reinterpret_cast<bf16*>(out)[orow * ldc + col] = __float2bfloat16_rn(v);
    else
        reinterpret_cast<float*>(out)[orow * ldc + col] = v;
}

int launch_gemm_strict(const float* a, const float* b, void* out, uint32_t ldc, uint32_t m, uint32_t k,
                       uint32_t n, bool b_transposed, const GemmEpilogue& ep, cudaStream_t stream) {
    if (m == 0 || n == 0) return TNSR_B200_OK;
    const size_t rows_smem = (size_t)k * SR_COLS * sizeof(float);
    if (m <= 64 && k > 0 && rows_smem <= 200 * 1024) {
        static bool configured[2] = {false, false};
        if (rows_smem > 48 * 1024 && !configured[b_transposed]) {
            cudaError_t e = b_transposed
                ? cudaFuncSetAttribute(gemm_strict_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                : cudaFuncSetAttribute(gemm_strict_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return check_launch("gemm_strict_rows attribute");
            configured[b_transposed] = true;
        }
        dim3 grid(ceil_div(n, SR_COLS), m);
        if (b_transposed)
            gemm_strict_rows_kernel<true><<<grid, SR_THREADS, rows_smem, stream>>>(a, b, out, ldc, m, k, n, ep);
        else
            gemm_strict_rows_kernel<false><<<grid, SR_THREADS, rows_smem, stream>>>(a, b, out, ldc, m, k, n, ep);
        count_launch();
        return check_launch("gemm_strict_rows");
    }
    dim3 grid(ceil_div(n, ST), ceil_div(m, ST)), block(ST, ST);
    if (grid.y > 65535u) {
        set_thread_error("strict GEMM: too many rows for one launch");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    if (b_transposed)
        gemm_strict_kernel<true><<<grid, block, 0, stream>>>(a, b, out, ldc, m, k, n, ep);
    else
        gemm_strict_kernel<false><<<grid, block, 0, stream>>>(a, b, out, ldc, m, k, n, ep);
    count_launch();
    return check_launch("gemm_strict");
}

// ---------------------------------------------------------------------------
// LayerNorm (src/nn.rs:199-212 on the interpreter's Mean reduction,
// src/lib.rs:1752-1754): mean = sum of x/n in order; var = sum of (c*c)/n in
// order; inv = exp(ln(var + eps) * -0.5); y = ((c * inv) * w) + b.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
layernorm_strict_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                        float* __restrict__ y, uint32_t width, float eps) {
    // The two sums are sequential chains in index order (the reference's arithmetic); their terms -- x/n and
    // (x - mean)^2/n -- do not depend on the chain, so all threads form them side by side and one thread adds them up.
    extern __shared__ float row[];     // [width] values, then [width] terms
    float* term = row + width;
    __shared__ float stats[2];
    const float* xr = x + (size_t)blockIdx.x * width;
    const float nf = (float)width;
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = xr[c];
        row[c] = v;
        term[c] = v / nf;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float mean = 0.0f;
#pragma unroll 8
        for (uint32_t c = 0; c < width; ++c) mean = mean + term[c];
        stats[0] = mean;
    }
    __syncthreads();
    {
        const float mean0 = stats[0];
        for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) {
            float d = row[c] - mean0;
            float sq = d * d;
            term[c] = sq / nf;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float var = 0.0f;
#pragma unroll 8
        for (uint32_t c = 0; c < width; ++c) var = var + term[c];
        stats[1] = strict_expf(strict_logf(var + eps) * -0.5f);
    }
    __syncthreads();
    const float mean = stats[0], inv = stats[1];
    float* yr = y + (size_t)blockIdx.x * width;
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) {
        float d = row[c] - mean;
        yr[c] = ((d * inv) * w[c]) + b[c];
    }
}

int launch_layernorm_strict(const float* x, const float* w, const float* b, float* out, uint32_t rows,
                            uint32_t width, float eps, cudaStream_t stream) {
    if (rows == 0) return TNSR_B200_OK;
    size_t smem = 2 * (size_t)width * sizeof(float);
    if (smem > 200 * 1024) {
        set_thread_error("strict LayerNorm: row does not fit shared memory");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(layernorm_strict_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    layernorm_strict_kernel<<<rows, 128, smem, stream>>>(x, w, b, out, width, eps);
    count_launch();
    return check_launch("layernorm_strict");
}

// ---------------------------------------------------------------------------
// Elementwise silu(gate) * up in the reference's op order.
// ---------------------------------------------------------------------------
__global__ void swiglu_strict_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                     float* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        float g = gate[i];
        out[i] = (g * strict_sigmoid(g)) * up[i];
    }
}

int launch_swiglu_strict(const float* gate, const float* up, float* out, size_t n, cudaStream_t stream) {
    if (n == 0) return TNSR_B200_OK;
    swiglu_strict_kernel<<<(unsigned)ceil_div64(n, 256), 256, 0, stream>>>(gate, up, out, n);
    count_launch();
    return check_launch("swiglu_strict");
}

// ---------------------------------------------------------------------------
// Attention over the live prefix in the order of the decode graph
// (src/nn/kv_cache/graph.rs:82-107, src/nn.rs:158-161): score_j = (q . k_j) *
// scale + 0; m = max_j; e_j = exp(score_j - m); S = e_0 + e_1 + ... in order;
// p_j = e_j / S; out_c = sum_j p_j * v[j, c] in order.  The new rows are already
// in the cache, so every key is read from it.  One block per (session, head,
// query).
// ---------------------------------------------------------------------------
template <typename KV>
__device__ __forceinline__ float kv_load(const KV* p, size_t i);
template <>
__device__ __forceinline__ float kv_load<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float kv_load<bf16>(const bf16* p, size_t i) { return __bfloat162float(p[i]); }

template <typename KV>
__global__ void __launch_bounds__(128)
attention_strict_kernel(const float* __restrict__ q, const KV* __restrict__ kc, const KV* __restrict__ vc,
                        float* __restrict__ out, uint32_t chunk, uint32_t position,
                        const uint32_t* __restrict__ d_position, uint32_t capacity, uint32_t heads,
                        uint32_t hd, float scale, int round_bf16) {
    extern __shared__ float smem[];
    __shared__ float red[128];
    const uint32_t t = blockIdx.x % chunk;
    const uint32_t h = (blockIdx.x / chunk) % heads;
    const uint32_t s = blockIdx.x / (chunk * heads);
    const uint32_t d = heads * hd;
    const uint32_t past = d_position ? *d_position : position;
    uint32_t total = past + t + 1;
    if (total > capacity) total = capacity;  // guarded by the host; never read past the cache
    float* qs = smem;            // [hd]
    float* sc = smem + hd;       // [total]
    const float* qr = q + ((size_t)s * chunk + t) * d + (size_t)h * hd;
    for (uint32_t c = threadIdx.x; c < hd; c += blockDim.x) qs[c] = qr[c];
    __syncthreads();
    const KV* kb = kc + (size_t)s * capacity * d + (size_t)h * hd;
    const KV* vb = vc + (size_t)s * capacity * d + (size_t)h * hd;
    float mx = -INFINITY;
    for (uint32_t j = threadIdx.x; j < total; j += blockDim.x) {
        float sum = 0.0f;
        for (uint32_t c = 0; c < hd; ++c) sum = sum + qs[c] * kv_load<KV>(kb, (size_t)j * d + c);
        float v = sum * scale;
        v = v + 0.0f;  // the mask term of visible keys
        sc[j] = v;
        mx = fmaxf(mx, v);
    }
    red[threadIdx.x] = mx;
    __syncthreads();
    for (uint32_t w = blockDim.x / 2; w > 0; w >>= 1) {
        if (threadIdx.x < w) red[threadIdx.x] = fmaxf(red[threadIdx.x], red[threadIdx.x + w]);
        __syncthreads();
    }
    mx = red[0];
    __syncthreads();
    for (uint32_t j = threadIdx.x; j < total; j += blockDim.x) sc[j] = strict_expf(sc[j] - mx);
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        for (uint32_t j = 0; j < total; ++j) sum = sum + sc[j];
        red[0] = sum;
    }
    __syncthreads();
    const float denom = red[0];
    __syncthreads();
    for (uint32_t j = threadIdx.x; j < total; j += blockDim.x) sc[j] = sc[j] / denom;
    __syncthreads();
    float* orow = out + ((size_t)s * chunk + t) * d + (size_t)h * hd;
    for (uint32_t c = threadIdx.x; c < hd; c += blockDim.x) {
        float acc = 0.0f;
        for (uint32_t j = 0; j < total; ++j) acc = acc + sc[j] * kv_load<KV>(vb, (size_t)j * d + c);
        orow[c] = round_bf16 ? round_to_bf16(acc) : acc;
    }
}

int launch_attention_strict(const float* q, const void* k_cache, const void* v_cache, float* out,
                            uint32_t sessions, uint32_t chunk, uint32_t position,
                            const uint32_t* d_position, uint32_t capacity, uint32_t heads,
                            uint32_t head_dim, int kv_dtype, int round_bf16, cudaStream_t stream) {
    if (sessions == 0 || chunk == 0) return TNSR_B200_OK;
    // (width as f32 / heads as f32).sqrt().recip()  -- src/nn/kv_cache/graph.rs:105
    const float scale = 1.0f / sqrtf((float)(heads * head_dim) / (float)heads);
    size_t smem = ((size_t)head_dim + capacity) * sizeof(float);
    if (smem > 200 * 1024) {
        set_thread_error("strict attention: context does not fit shared memory");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    uint64_t blocks = (uint64_t)sessions * heads * chunk;
    if (blocks > 0x7fffffffull) {
        set_thread_error("strict attention: too many queries for one launch");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    if (kv_dtype == TNSR_B200_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(attention_strict_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attention_strict_kernel<bf16><<<(unsigned)blocks, 128, smem, stream>>>(
            q, (const bf16*)k_cache, (const bf16*)v_cache, out, chunk, position, d_position, capacity, heads,
            head_dim, scale, round_bf16);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(attention_strict_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attention_strict_kernel<float><<<(unsigned)blocks, 128, smem, stream>>>(
            q, (const float*)k_cache, (const float*)v_cache, out, chunk, position, d_position, capacity, heads,
            head_dim, scale, round_bf16);
    }
    count_launch();
    return check_launch("attention_strict");
}

}  // namespace tb
