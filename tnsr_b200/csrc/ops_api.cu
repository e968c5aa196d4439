// extern "C" wrappers of the individual kernels (operator-level entry points of
// include/tnsr_b200.h).  They queue work on the caller's stream and never
// synchronise or allocate.
#include "common.cuh"

using namespace tb;

namespace {
inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline int bad(const char* msg) {
    set_thread_error(msg);
    return TNSR_B200_ERR_INVALID_ARGUMENT;
}
}  // namespace

extern "C" {

int tnsr_b200_embedding(const void* token_table, const void* position_table, const uint32_t* ids, float* out,
                        uint32_t rows, uint32_t chunk, uint32_t position0, uint32_t vocab, uint32_t width, int dtype,
                        int* d_status, void* stream) {
    if (!token_table || !position_table || !ids || !out) return bad("embedding: null pointer");
    if (dtype != TNSR_B200_F32 && dtype != TNSR_B200_BF16) return bad("embedding: dtype must be f32 or bf16");
    if (chunk == 0 || width == 0) return bad("embedding: chunk and width must be non-zero");
    return launch_embedding(token_table, position_table, ids, out, rows, chunk, position0, nullptr, vocab, width, dtype,
                            d_status, as_stream(stream));
}

int tnsr_b200_layernorm(const float* x, const float* weight, const float* bias, void* out, uint32_t rows, uint32_t width,
                        float epsilon, int out_dtype, int strict, void* stream) {
    if (!x || !weight || !bias || !out) return bad("layernorm: null pointer");
    if (width == 0 || !(epsilon > 0.0f)) return bad("layernorm: width and epsilon must be positive");
    if (out_dtype != TNSR_B200_F32 && out_dtype != TNSR_B200_BF16) return bad("layernorm: bad output dtype");
    return launch_layernorm(x, weight, bias, out, rows, width, epsilon, out_dtype, strict != 0, as_stream(stream));
}

int tnsr_b200_gemm_f32_strict(const float* a, const float* b, const float* bias, float* out, uint32_t m, uint32_t k,
                              uint32_t n, int b_transposed, void* stream) {
    if (!a || !b || !out) return bad("gemm_f32_strict: null pointer");
    GemmEpilogue ep;
    ep.bias = bias;
    return launch_gemm_strict(a, b, out, n, m, k, n, b_transposed != 0, ep, as_stream(stream));
}

int tnsr_b200_gemm_bf16(const void* a, const void* bt, const float* bias, const float* residual, void* out, uint32_t m,
                        uint32_t n, uint32_t k, int activation, int out_dtype, void* stream) {
    return tnsr_b200_gemm_bf16_ws(a, bt, bias, residual, out, m, n, k, activation, out_dtype, nullptr, 0, stream);
}

uint64_t tnsr_b200_gemm_workspace(void) { return gemm_skinny_workspace_bytes(); }

int tnsr_b200_gemm_bf16_ws(const void* a, const void* bt, const float* bias, const float* residual, void* out, uint32_t m,
                           uint32_t n, uint32_t k, int activation, int out_dtype, void* workspace, uint64_t workspace_bytes,
                           void* stream) {
    if (!a || !bt || !out) return bad("gemm_bf16: null pointer");
    if (out_dtype != TNSR_B200_F32 && out_dtype != TNSR_B200_BF16) return bad("gemm_bf16: bad output dtype");
    if (activation < -1 || activation > TNSR_B200_ACT_GELU) return bad("gemm_bf16: activation must be -1, RELU or GELU");
    if (residual && out_dtype != TNSR_B200_F32) return bad("gemm_bf16: a residual needs f32 output");
    GemmEpilogue ep;
    ep.bias = bias;
    ep.residual = residual;
    ep.ldr = n;
    ep.activation = activation;
    ep.out_dtype = out_dtype;
    if (workspace) {
        if (workspace_bytes < gemm_skinny_workspace_bytes() || (reinterpret_cast<uintptr_t>(workspace) & 15))
            return bad("gemm_bf16_ws: workspace too small or not 16-byte aligned");
        ep.skinny_ws = workspace;
        ep.skinny_ws_bytes = workspace_bytes;
    }
    return launch_gemm_bf16((const bf16*)a, (const bf16*)bt, out, n, m, n, k, GEMM_PLAIN, ep, nullptr, nullptr,
                            as_stream(stream));
}

int tnsr_b200_transpose_bf16(const void* in, void* out, uint32_t k, uint32_t n, void* stream) {
    if (!in || !out) return bad("transpose_bf16: null pointer");
    return launch_transpose_bf16((const bf16*)in, (bf16*)out, k, n, as_stream(stream));
}

int tnsr_b200_swiglu(const void* gate, const void* up, void* out, uint64_t elems, void* stream) {
    if (!gate || !up || !out) return bad("swiglu: null pointer");
    return launch_swiglu((const bf16*)gate, (const bf16*)up, (bf16*)out, elems, as_stream(stream));
}

int tnsr_b200_pack_gate_up(const void* w_gate, const void* w_up, const float* b_gate, const float* b_up, void* w_out,
                           float* b_out, uint32_t d, uint32_t f, void* stream) {
    if (!w_gate || !w_up || !w_out) return bad("pack_gate_up: null pointer");
    return launch_pack_gate_up((const bf16*)w_gate, (const bf16*)w_up, b_gate, b_up, (bf16*)w_out, b_out, d, f,
                               as_stream(stream));
}

int tnsr_b200_swiglu_mlp(const void* x, const void* w_gate_up_t, const float* b_gate_up, const void* w_down_t,
                         const float* b_down, void* hidden, void* out, uint32_t rows, uint32_t d, uint32_t f, void* stream) {
    if (!x || !w_gate_up_t || !w_down_t || !hidden || !out) return bad("swiglu_mlp: null pointer");
    if (f % 16 != 0) {
        set_thread_error("swiglu_mlp: feed-forward width must be a multiple of 16");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    GemmEpilogue eg;
    eg.bias = b_gate_up;
    eg.out_dtype = TNSR_B200_BF16;
    int rc = launch_gemm_bf16((const bf16*)x, (const bf16*)w_gate_up_t, hidden, f, rows, 2 * f, d, GEMM_SWIGLU, eg, nullptr,
                              nullptr, as_stream(stream));
    if (rc) return rc;
    GemmEpilogue ed;
    ed.bias = b_down;
    ed.out_dtype = TNSR_B200_BF16;
    return launch_gemm_bf16((const bf16*)hidden, (const bf16*)w_down_t, out, d, rows, d, f, GEMM_PLAIN, ed, nullptr, nullptr,
                            as_stream(stream));
}

uint64_t tnsr_b200_decode_attention_workspace(uint32_t batch, uint32_t capacity, uint32_t heads, uint32_t head_dim) {
    return decode_attention_workspace_bytes(batch, capacity, heads, head_dim);
}

int tnsr_b200_decode_attention(const void* q, const void* k_cache, const void* v_cache, const uint32_t* lengths, void* out,
                               void* workspace, uint64_t workspace_bytes, uint32_t batch, uint32_t capacity, uint32_t heads,
                               uint32_t head_dim, void* stream) {
    if (!q || !k_cache || !v_cache || !lengths || !out || !workspace) return bad("decode_attention: null pointer");
    // nothing may be written before the size is known to fit (the status word below lives inside the workspace)
    if (workspace_bytes < decode_attention_workspace_bytes(batch, capacity, heads, head_dim) || workspace_bytes < 256)
        return bad("decode_attention: workspace smaller than tnsr_b200_decode_attention_workspace() asks for");
    // bytes 64..67 of the workspace hold the kernel's status word
    int* d_status = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(workspace) + 64);
    cudaError_t e = cudaMemsetAsync(d_status, 0, 4, as_stream(stream));
    if (e != cudaSuccess) {
        set_thread_error(std::string("decode_attention: ") + cudaGetErrorString(e));
        return TNSR_B200_ERR_CUDA;
    }
    return launch_decode_attention((const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, lengths, (bf16*)out, workspace,
                                   workspace_bytes, batch, capacity, heads, head_dim, d_status, as_stream(stream));
}

int tnsr_b200_prefill_attention(const void* q, const void* k_cache, const void* v_cache, void* out, uint32_t batch,
                                uint32_t chunk, uint32_t position, uint32_t capacity, uint32_t heads, uint32_t head_dim,
                                void* stream) {
    if (!q || !k_cache || !v_cache || !out) return bad("prefill_attention: null pointer");
    if ((uint64_t)position + chunk > capacity) return bad("prefill_attention: position + chunk exceeds the capacity");
    if (prefill_attention_supported(head_dim))
        return launch_prefill_attention((const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, batch, chunk,
                                        position, nullptr, capacity, heads, head_dim, nullptr, as_stream(stream));
    return launch_attention_generic((const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, batch, chunk,
                                    position, nullptr, capacity, heads, head_dim, as_stream(stream));
}

int tnsr_b200_sample_top_k(const float* logits, uint32_t* out, uint32_t rows, uint32_t vocab, float temperature,
                           uint32_t top_k, uint64_t seed, uint32_t step, uint32_t first_session, void* stream) {
    if (!logits || !out) return bad("sample_top_k: null pointer");
    return launch_sample_top_k(logits, out, rows, vocab, vocab, temperature, top_k, seed, nullptr, 0, step, first_session,
                               as_stream(stream));
}

int tnsr_b200_argmax(const float* logits, uint32_t* out, uint32_t rows, uint32_t vocab, void* stream) {
    if (!logits || !out || vocab == 0) return bad("argmax: null pointer or empty vocabulary");
    return launch_argmax(logits, out, rows, vocab, vocab, as_stream(stream));
}

}  // extern "C"
