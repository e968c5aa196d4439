// The two operators the forty_five token encoder (tnsr examples/forty_five/mod.rs:329-407) needs beyond those of
// the GPT decoder: a three-table embedding with an input mask, and bidirectional attention with an additive key
// mask.  Strict f32 in the reference's CPU operation order, like strict.cu (this file is compiled with
// --fmad=false too); the encoder's projections, LayerNorms and SwiGLU reuse the decoder's strict operators.
#include "common.cuh"

namespace tb {

__device__ __forceinline__ float enc_expf(float x) { return (float)exp((double)x); }

// x[r, :] = mask[r] != 0 ? ((tok[ids[r]] + typ[kinds[r]]) + pos[pos_ids[r % seq]]) : 0
// (mod.rs:343-357: three `embedding_indices` gathers added left to right, then `mask`, src/lib.rs:315-329).
__global__ void __launch_bounds__(128)
encoder_embed_kernel(const float* __restrict__ tok, const float* __restrict__ typ, const float* __restrict__ pos,
                     const uint32_t* __restrict__ ids, const uint32_t* __restrict__ kinds,
                     const uint32_t* __restrict__ pos_ids, const float* __restrict__ mask, float* __restrict__ out,
                     uint32_t seq, uint32_t vocab, uint32_t kinds_vocab, uint32_t width, int* __restrict__ d_status) {
    const uint32_t r = blockIdx.x;
    const uint32_t id = ids[r], kind = kinds[r], p = pos_ids[r % seq];
    const bool valid = id < vocab && kind < kinds_vocab && p < seq;
    if (!valid && threadIdx.x == 0 && d_status) atomicCAS(d_status, DEV_OK, DEV_TOKEN_RANGE);
    const bool keep = valid && mask[r] != 0.0f;
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) {
        float v = 0.0f;
        if (keep) {
            v = tok[(size_t)id * width + c] + typ[(size_t)kind * width + c];
            v = v + pos[(size_t)p * width + c];
        }
        out[(size_t)r * width + c] = v;
    }
}

// One block per (sample, head, query).  score_j = (q . k_j) * scale + key_mask[sample, j] (mod.rs:368-382),
// softmax as src/nn.rs:158-161 (max, exp(x - max), sum in key order, divide), out_c = sum_j p_j * v[j, c] in key order.
// q, k, v are row-major with `ld` floats between rows (3 * width for a fused projection), heads are column slices.
__global__ void __launch_bounds__(128)
encoder_attention_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, uint32_t ld,
                         const float* __restrict__ key_mask, float* __restrict__ out, uint32_t seq, uint32_t heads,
                         uint32_t hd, float scale) {
    extern __shared__ float smem[];
    __shared__ float red[128];
    const uint32_t t = blockIdx.x % seq;
    const uint32_t h = (blockIdx.x / seq) % heads;
    const uint32_t s = blockIdx.x / (seq * heads);
    const uint32_t d = heads * hd;
    float* qs = smem;            // [hd]
    float* sc = smem + hd;       // [seq]
    const float* qr = q + ((size_t)s * seq + t) * ld + (size_t)h * hd;
    for (uint32_t c = threadIdx.x; c < hd; c += blockDim.x) qs[c] = qr[c];
    __syncthreads();
    const float* kb = k + (size_t)s * seq * ld + (size_t)h * hd;
    const float* vb = v + (size_t)s * seq * ld + (size_t)h * hd;
    const float* mk = key_mask + (size_t)s * seq;
    float mx = -INFINITY;
    for (uint32_t j = threadIdx.x; j < seq; j += blockDim.x) {
        float sum = 0.0f;
        for (uint32_t c = 0; c < hd; ++c) sum = sum + qs[c] * kb[(size_t)j * ld + c];
        float val = sum * scale;
        val = val + mk[j];
        sc[j] = val;
        mx = fmaxf(mx, val);
    }
    red[threadIdx.x] = mx;
    __syncthreads();
    for (uint32_t w = blockDim.x / 2; w > 0; w >>= 1) {
        if (threadIdx.x < w) red[threadIdx.x] = fmaxf(red[threadIdx.x], red[threadIdx.x + w]);
        __syncthreads();
    }
    mx = red[0];
    __syncthreads();
    for (uint32_t j = threadIdx.x; j < seq; j += blockDim.x) sc[j] = enc_expf(sc[j] - mx);
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        for (uint32_t j = 0; j < seq; ++j) sum = sum + sc[j];
        red[0] = sum;
    }
    __syncthreads();
    const float denom = red[0];
    __syncthreads();
    for (uint32_t j = threadIdx.x; j < seq; j += blockDim.x) sc[j] = sc[j] / denom;
    __syncthreads();
    float* orow = out + ((size_t)s * seq + t) * d + (size_t)h * hd;
    for (uint32_t c = threadIdx.x; c < hd; c += blockDim.x) {
        float acc = 0.0f;
        for (uint32_t j = 0; j < seq; ++j) acc = acc + sc[j] * vb[(size_t)j * ld + c];
        orow[c] = acc;
    }
}

__global__ void add_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
}

}  // namespace tb

using namespace tb;

extern "C" {

int tnsr_b200_encoder_embed(const float* token_table, const float* type_table, const float* position_table,
                            const uint32_t* ids, const uint32_t* type_ids, const uint32_t* position_ids, const float* mask,
                            float* out, uint32_t rows, uint32_t seq, uint32_t vocab, uint32_t type_vocab, uint32_t width,
                            int* d_status, void* stream) {
    if (!token_table || !type_table || !position_table || !ids || !type_ids || !position_ids || !mask || !out) {
        set_thread_error("encoder_embed: null pointer");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    if (seq == 0 || width == 0 || rows % seq != 0) {
        set_thread_error("encoder_embed: rows must be a multiple of a non-zero sequence length");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    if (rows == 0) return TNSR_B200_OK;
    encoder_embed_kernel<<<rows, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(token_table, type_table, position_table, ids,
                                                                                  type_ids, position_ids, mask, out, seq, vocab,
                                                                                  type_vocab, width, d_status);
    count_launch();
    return check_launch("encoder_embed");
}

int tnsr_b200_encoder_attention(const float* q, const float* k, const float* v, uint32_t row_stride, const float* key_mask,
                                float* out, uint32_t batch, uint32_t seq, uint32_t heads, uint32_t head_dim, void* stream) {
    if (!q || !k || !v || !key_mask || !out) {
        set_thread_error("encoder_attention: null pointer");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    if (seq == 0 || heads == 0 || head_dim == 0 || row_stride < heads * head_dim) {
        set_thread_error("encoder_attention: empty shape or a row stride below the width");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    if (batch == 0) return TNSR_B200_OK;
    const size_t smem = ((size_t)head_dim + seq) * sizeof(float);
    const uint64_t blocks = (uint64_t)batch * heads * seq;
    if (smem > 200 * 1024 || blocks > 0x7fffffffull) {
        set_thread_error("encoder_attention: sequence too long for shared memory or too many queries for one launch");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(encoder_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    // (head as f32).sqrt().recip()  -- examples/forty_five/mod.rs:377
    const float scale = 1.0f / sqrtf((float)head_dim);
    encoder_attention_kernel<<<(unsigned)blocks, 128, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
        q, k, v, row_stride, key_mask, out, seq, heads, head_dim, scale);
    count_launch();
    return check_launch("encoder_attention");
}

int tnsr_b200_add_f32(const float* a, const float* b, float* out, uint64_t elems, void* stream) {
    if (!a || !b || !out) {
        set_thread_error("add_f32: null pointer");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    if (elems == 0) return TNSR_B200_OK;
    add_f32_kernel<<<(unsigned)ceil_div64(elems, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a, b, out, elems);
    count_launch();
    return check_launch("add_f32");
}

int tnsr_b200_swiglu_f32(const float* gate, const float* up, float* out, uint64_t elems, void* stream) {
    if (!gate || !up || !out) {
        set_thread_error("swiglu_f32: null pointer");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    return launch_swiglu_strict(gate, up, out, (size_t)elems, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
