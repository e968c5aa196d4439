// The session object behind tnsr_b200_decoder_*: the B200 counterpart of
// cuda::CudaDecoder (tnsr src/nn/kv_cache/cuda.rs:47-596).  It owns a private
// stream, resident weights (repacked once at upload), the K/V cache, activation
// buffers sized for the largest chunk seen so far, and runs one decode step as a
// fixed sequence of kernels -- there is no graph to compile and no program
// cache to evict.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_set>
#include <vector>

#include "common.cuh"

namespace tb {
std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_wait_limit_ns{2000000000ull};
static thread_local std::string t_error;
void set_thread_error(const std::string& msg) { t_error = msg; }
const char* thread_error() { return t_error.c_str(); }
void prefer_max_shared_carveout(const void* kernel) {
    static std::mutex lock;
    static std::unordered_set<uint64_t> done;
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t key = (uint64_t)reinterpret_cast<uintptr_t>(kernel) ^ ((uint64_t)(uint32_t)dev << 56);
    std::lock_guard<std::mutex> guard(lock);
    if (!done.insert(key).second) return;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
        cudaGetLastError();   // a hint only: the launch itself does not depend on it
}
bool debug_sync_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("TNSR_B200_DEBUG_SYNC");
        return v && v[0] == '1';
    }();
    return on;
}
}  // namespace tb

using namespace tb;

namespace {

constexpr uint32_t kNoPage = 0xffffffffu;

struct Buffer {
    void* ptr = nullptr;
    size_t bytes = 0;
};

enum ParamKind { P_TOK, P_POS, P_VEC, P_QKV_W, P_QKV_B, P_O_W, P_FF_IN_W, P_FF_IN_B, P_FF_OUT_W, P_GATE_W, P_GATE_B, P_UP_W, P_UP_B };

struct ParamInfo {
    ParamKind kind;
    uint64_t elems;
    uint32_t rows, cols;  // [rows, cols] as the reference stores it ([in, out] for matrices)
    uint32_t layer;
    uint32_t slot;        // 0/1/2 = q/k/v for QKV params
    void* dev = nullptr;  // where the values live (f32 path: as given; bf16 path: see upload)
};

struct Layer {
    // f32 path: the reference layout, f32.  bf16 path: matrices are [out, in] bf16.
    void *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr;
    float *bq = nullptr, *bk = nullptr, *bv = nullptr, *bo = nullptr;
    float *ln1w = nullptr, *ln1b = nullptr, *ln2w = nullptr, *ln2b = nullptr;
    void *w_in = nullptr, *w_out = nullptr, *w_gate = nullptr, *w_up = nullptr;
    float *b_in = nullptr, *b_out = nullptr, *b_gate = nullptr, *b_up = nullptr;
    // bf16 path fused forms
    bf16* wqkv = nullptr;  // [3d, d]
    float* bqkv = nullptr; // [3d]
    bf16* wgu = nullptr;   // packed [2f, d] when f % 16 == 0
    float* bgu = nullptr;  // packed [2f]
    void *kcache = nullptr, *vcache = nullptr;
};

}  // namespace

struct tnsr_b200_decoder {
    tnsr_b200_config cfg;
    cudaStream_t stream = nullptr;
    bool bf16_path = false, kv_bf16 = false, swiglu = false, fused_gu = false;
    bool failed = false;
    std::string error;
    std::vector<ParamInfo> params;
    std::vector<Layer> layers;
    void *tok = nullptr, *pos = nullptr;
    float *fnw = nullptr, *fnb = nullptr;
    std::vector<void*> allocations;
    // activations (grow with the chunk)
    uint32_t rows_cap = 0, logit_rows_cap = 0;
    float* h = nullptr;      // residual stream [rows, d] f32
    void* n = nullptr;       // normalised rows: f32 (strict) or bf16
    void* q = nullptr;       // queries: f32 (strict) or bf16
    void* att = nullptr;     // attention output: f32 (strict) or bf16
    void* ff = nullptr;      // FFN hidden [rows, f]
    void* ff2 = nullptr;     // second FFN buffer (up projection) when gate/up are not fused
    float* hl = nullptr;     // last rows [batch, d] f32
    float* logits = nullptr; // [logit_rows, vocab]
    uint32_t* d_tokens = nullptr;
    uint32_t tokens_cap = 0;
    uint32_t* d_argmax = nullptr;
    int* d_status = nullptr;
    void* attn_ws = nullptr;
    // a single-token step may be divided into up to kMaxParts session ranges on as many streams (see step_bf16):
    // range 0 runs on `stream` with `attn_ws`, range i > 0 on side_stream[i - 1] with side_ws[i - 1]
    void* side_ws[3] = {nullptr, nullptr, nullptr};
    // partial sums of the split-K projections of an undivided single-token step: [4][split_rows][d] f32
    float* split_ws = nullptr;
    uint32_t split_rows = 0;
    uint32_t split_pending = 0;   // partial sums of the last layer's down projection, for the final LayerNorm to add
    uint64_t attn_ws_bytes = 0;
    cudaStream_t side_stream[3] = {nullptr, nullptr, nullptr};   // forked from and joined to `stream` by events
    cudaEvent_t ev_fork = nullptr, ev_join[3] = {nullptr, nullptr, nullptr};
    uint32_t parts = 1;
    // small batches: one persistent kernel per layer between the attention scans (decode_tail.cu); its barrier words
    void* tail_ws = nullptr;
    bool use_tail = true;
    // paged K/V: every cache tensor is a pool [pool_pages, page_rows, d]; h_table[s * pps + i] is the pool page of
    // session s's i-th page, kNoPage while unassigned (the device copy is refreshed before the step that needs it)
    bool paged = false;
    uint32_t page_rows = 0, pool_pages = 0, pps = 0;
    std::vector<uint32_t> h_table_shadow;   // the table as the host knows it
    std::vector<uint32_t> free_pages;       // stack of unassigned pool pages
    uint32_t* h_table = nullptr;            // pinned copy used for the upload
    uint32_t* d_table = nullptr;
    bool table_dirty = false;
    // next-token sampling instead of the greedy pick (temperature <= 0: greedy)
    float sample_temperature = 0.0f;
    uint32_t sample_top_k = 0;
    uint64_t sample_seed = 0;
    uint32_t* d_positions = nullptr;   // [batch] per-session positions of a ragged step
    uint32_t* h_positions = nullptr;   // pinned staging for them
    // pinned staging
    uint32_t* h_tokens = nullptr;
    uint32_t* h_argmax = nullptr;
    int* h_status = nullptr;
    float* h_stage = nullptr;  // upload staging (pinned)
    size_t h_stage_bytes = 0;
    float* d_stage = nullptr;  // upload staging (device, f32)
    size_t d_stage_bytes = 0;
    std::vector<float> host_bqkv, host_bgu;
    bool profile_attention = false;
    KernelTimer attention_timer;
    void* lm_candidates = nullptr;  // per (session, vocabulary tile) greedy candidates of the fused LM head
    // single-token steps are replayed from a captured CUDA graph; the position lives in d_pos
    uint32_t* d_pos = nullptr;
    struct StepGraph {
        const uint32_t* tokens;
        uint32_t* argmax;
        cudaGraphExec_t exec;
        uint64_t kernels;
    };
    std::vector<StepGraph> graphs;
    bool use_graphs = true;
    bool use_pdl = true;
    bool stepped_once = false;  // a plain (uncaptured) single-token step has run: buffers and attributes are set
};

namespace {

int fail(tnsr_b200_decoder* dec, int code, const std::string& msg) {
    if (dec) dec->error = msg;
    set_thread_error(msg);
    return code;
}

int cuda_fail(tnsr_b200_decoder* dec, cudaError_t e, const char* what) {
    std::string msg = std::string(what) + ": " + cudaGetErrorString(e);
    int code = (e == cudaErrorMemoryAllocation) ? TNSR_B200_ERR_OUT_OF_MEMORY : TNSR_B200_ERR_CUDA;
    if (dec && code == TNSR_B200_ERR_CUDA) dec->failed = true;
    cudaGetLastError();
    return fail(dec, code, msg);
}

#define CU(dec, call)                                                   \
    do {                                                                \
        cudaError_t e__ = (call);                                       \
        if (e__ != cudaSuccess) return cuda_fail(dec, e__, #call);      \
    } while (0)

#define RUN(dec, call)                                                  \
    do {                                                                \
        int rc__ = (call);                                              \
        if (rc__ != TNSR_B200_OK) {                                     \
            (dec)->error = thread_error();                              \
            if (rc__ == TNSR_B200_ERR_CUDA) (dec)->failed = true;       \
            return rc__;                                                \
        }                                                               \
    } while (0)

void drop_graphs(tnsr_b200_decoder* dec) {
    for (auto& g : dec->graphs) cudaGraphExecDestroy(g.exec);
    dec->graphs.clear();
}

int dev_alloc(tnsr_b200_decoder* dec, void** out, size_t bytes, bool zero) {
    if (bytes == 0) bytes = 16;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return cuda_fail(dec, e, "cudaMalloc");
    dec->allocations.push_back(p);
    if (zero) {
        e = cudaMemsetAsync(p, 0, bytes, dec->stream);
        if (e != cudaSuccess) return cuda_fail(dec, e, "cudaMemsetAsync");
    }
    *out = p;
    return TNSR_B200_OK;
}

void dev_free(tnsr_b200_decoder* dec, void* p) {
    if (!p) return;
    for (size_t i = 0; i < dec->allocations.size(); ++i)
        if (dec->allocations[i] == p) {
            dec->allocations.erase(dec->allocations.begin() + i);
            break;
        }
    cudaFree(p);
}

size_t elt(const tnsr_b200_decoder* dec) { return dec->bf16_path ? 2 : 4; }
size_t kv_elt(const tnsr_b200_decoder* dec) { return dec->kv_bf16 ? 2 : 4; }

bool mul_overflow(uint64_t a, uint64_t b, uint64_t* out) { return __builtin_mul_overflow(a, b, out); }

// model_parameters order (src/nn/kv_cache.rs:392-421) + the SwiGLU extension.
void describe_params(tnsr_b200_decoder* dec) {
    const tnsr_b200_config& c = dec->cfg;
    const uint32_t d = c.embed_dim, f = c.feed_forward_dim;
    auto add = [&](ParamKind k, uint32_t rows, uint32_t cols, uint32_t layer, uint32_t slot) {
        ParamInfo p;
        p.kind = k; p.rows = rows; p.cols = cols; p.elems = (uint64_t)rows * cols; p.layer = layer; p.slot = slot;
        dec->params.push_back(p);
    };
    add(P_TOK, c.vocab_size, d, 0, 0);
    add(P_POS, c.max_sequence_length, d, 0, 0);
    add(P_VEC, 1, d, 0, 100);  // final norm weight
    add(P_VEC, 1, d, 0, 101);  // final norm bias
    for (uint32_t l = 0; l < c.num_layers; ++l) {
        for (uint32_t s = 0; s < 3; ++s) { add(P_QKV_W, d, d, l, s); add(P_QKV_B, 1, d, l, s); }
        add(P_O_W, d, d, l, 0);
        add(P_VEC, 1, d, l, 0);   // o bias
        add(P_VEC, 1, d, l, 1);   // ln1 w
        add(P_VEC, 1, d, l, 2);   // ln1 b
        add(P_VEC, 1, d, l, 3);   // ln2 w
        add(P_VEC, 1, d, l, 4);   // ln2 b
        if (dec->swiglu) {
            add(P_GATE_W, d, f, l, 0); add(P_GATE_B, 1, f, l, 0);
            add(P_UP_W, d, f, l, 0);   add(P_UP_B, 1, f, l, 0);
            add(P_FF_OUT_W, f, d, l, 0); add(P_VEC, 1, d, l, 5);
        } else {
            add(P_FF_IN_W, d, f, l, 0); add(P_FF_IN_B, 1, f, l, 0);
            add(P_FF_OUT_W, f, d, l, 0); add(P_VEC, 1, d, l, 5);
        }
    }
}

int allocate_weights(tnsr_b200_decoder* dec) {
    const tnsr_b200_config& c = dec->cfg;
    const uint64_t d = c.embed_dim, f = c.feed_forward_dim;
    const size_t e = elt(dec);
    int rc;
    if ((rc = dev_alloc(dec, &dec->tok, (size_t)c.vocab_size * d * e, true))) return rc;
    if ((rc = dev_alloc(dec, &dec->pos, (size_t)c.max_sequence_length * d * e, true))) return rc;
    if ((rc = dev_alloc(dec, (void**)&dec->fnw, d * 4, true))) return rc;
    if ((rc = dev_alloc(dec, (void**)&dec->fnb, d * 4, true))) return rc;
    dec->layers.resize(c.num_layers);
    const size_t cache_bytes = dec->paged ? (size_t)dec->pool_pages * dec->page_rows * d * kv_elt(dec)
                                          : (size_t)c.batch * c.capacity * d * kv_elt(dec);
    for (Layer& L : dec->layers) {
        if (dec->bf16_path) {
            if ((rc = dev_alloc(dec, (void**)&L.wqkv, 3 * d * d * 2, true))) return rc;
            if ((rc = dev_alloc(dec, (void**)&L.bqkv, 3 * d * 4, true))) return rc;
            L.wq = L.wqkv; L.wk = L.wqkv + d * d; L.wv = L.wqkv + 2 * d * d;
            L.bq = L.bqkv; L.bk = L.bqkv + d; L.bv = L.bqkv + 2 * d;
        } else {
            if ((rc = dev_alloc(dec, &L.wq, d * d * 4, true))) return rc;
            if ((rc = dev_alloc(dec, &L.wk, d * d * 4, true))) return rc;
            if ((rc = dev_alloc(dec, &L.wv, d * d * 4, true))) return rc;
            if ((rc = dev_alloc(dec, (void**)&L.bq, d * 4, true))) return rc;
            if ((rc = dev_alloc(dec, (void**)&L.bk, d * 4, true))) return rc;
            if ((rc = dev_alloc(dec, (void**)&L.bv, d * 4, true))) return rc;
        }
        if ((rc = dev_alloc(dec, &L.wo, d * d * e, true))) return rc;
        if ((rc = dev_alloc(dec, (void**)&L.bo, d * 4, true))) return rc;
        if ((rc = dev_alloc(dec, (void**)&L.ln1w, d * 4, true))) return rc;
        if ((rc = dev_alloc(dec, (void**)&L.ln1b, d * 4, true))) return rc;
        if ((rc = dev_alloc(dec, (void**)&L.ln2w, d * 4, true))) return rc;
        if ((rc = dev_alloc(dec, (void**)&L.ln2b, d * 4, true))) return rc;
        if (dec->swiglu) {
            if (dec->fused_gu) {
                if ((rc = dev_alloc(dec, (void**)&L.wgu, 2 * f * d * 2, true))) return rc;
                if ((rc = dev_alloc(dec, (void**)&L.bgu, 2 * f * 4, true))) return rc;
            } else {
                if ((rc = dev_alloc(dec, &L.w_gate, d * f * e, true))) return rc;
                if ((rc = dev_alloc(dec, &L.w_up, d * f * e, true))) return rc;
                if ((rc = dev_alloc(dec, (void**)&L.b_gate, f * 4, true))) return rc;
                if ((rc = dev_alloc(dec, (void**)&L.b_up, f * 4, true))) return rc;
            }
        } else {
            if ((rc = dev_alloc(dec, &L.w_in, d * f * e, true))) return rc;
            if ((rc = dev_alloc(dec, (void**)&L.b_in, f * 4, true))) return rc;
        }
        if ((rc = dev_alloc(dec, &L.w_out, f * d * e, true))) return rc;
        if ((rc = dev_alloc(dec, (void**)&L.b_out, d * 4, true))) return rc;
        if ((rc = dev_alloc(dec, &L.kcache, cache_bytes, true))) return rc;
        if ((rc = dev_alloc(dec, &L.vcache, cache_bytes, true))) return rc;
    }
    return TNSR_B200_OK;
}

int ensure_rows(tnsr_b200_decoder* dec, uint32_t rows, uint32_t logit_rows) {
    const tnsr_b200_config& c = dec->cfg;
    const uint64_t d = c.embed_dim, f = c.feed_forward_dim;
    const size_t a = dec->bf16_path ? 2 : 4;
    int rc;
    if (rows > dec->rows_cap || logit_rows > dec->logit_rows_cap || rows > dec->tokens_cap) drop_graphs(dec);
    if (rows > dec->rows_cap) {
        CU(dec, cudaStreamSynchronize(dec->stream));
        dev_free(dec, dec->h); dev_free(dec, dec->n); dev_free(dec, dec->q); dev_free(dec, dec->att);
        dev_free(dec, dec->ff); dev_free(dec, dec->ff2);
        dec->h = nullptr; dec->n = dec->q = dec->att = dec->ff = dec->ff2 = nullptr;
        dec->rows_cap = 0;
        if ((rc = dev_alloc(dec, (void**)&dec->h, rows * d * 4, false))) return rc;
        if ((rc = dev_alloc(dec, &dec->n, rows * d * a, false))) return rc;
        if ((rc = dev_alloc(dec, &dec->q, rows * d * a, false))) return rc;
        if ((rc = dev_alloc(dec, &dec->att, rows * d * a, false))) return rc;
        if ((rc = dev_alloc(dec, &dec->ff, rows * f * a, false))) return rc;
        if (dec->swiglu && !dec->fused_gu)
            if ((rc = dev_alloc(dec, &dec->ff2, rows * f * a, false))) return rc;
        dec->rows_cap = rows;
    }
    if (logit_rows > dec->logit_rows_cap) {
        CU(dec, cudaStreamSynchronize(dec->stream));
        dev_free(dec, dec->logits);
        dec->logits = nullptr;
        dec->logit_rows_cap = 0;
        uint64_t bytes;
        if (mul_overflow((uint64_t)logit_rows * c.vocab_size, 4, &bytes)) return fail(dec, TNSR_B200_ERR_OUT_OF_MEMORY, "logits size overflow");
        if ((rc = dev_alloc(dec, (void**)&dec->logits, bytes, false))) return rc;
        dec->logit_rows_cap = logit_rows;
    }
    if (rows > dec->tokens_cap) {
        CU(dec, cudaStreamSynchronize(dec->stream));
        dev_free(dec, dec->d_tokens);
        if (dec->h_tokens) cudaFreeHost(dec->h_tokens);
        dec->d_tokens = nullptr; dec->h_tokens = nullptr; dec->tokens_cap = 0;
        if ((rc = dev_alloc(dec, (void**)&dec->d_tokens, (size_t)rows * 4, false))) return rc;
        CU(dec, cudaMallocHost((void**)&dec->h_tokens, (size_t)rows * 4));
        dec->tokens_cap = rows;
    }
    return TNSR_B200_OK;
}

// ---- paged K/V bookkeeping -------------------------------------------------------
// Makes sure session s owns pages for rows [0, rows_needed).  Pages are taken in one go per step: if the pool cannot
// cover the whole request nothing is assigned.
int reserve_pages(tnsr_b200_decoder* dec, const uint32_t* rows_needed /* [batch] */) {
    if (!dec->paged) return TNSR_B200_OK;
    const uint32_t B = dec->cfg.batch, pps = dec->pps;
    uint64_t want = 0;
    for (uint32_t s = 0; s < B; ++s) {
        const uint32_t pages = (rows_needed[s] + dec->page_rows - 1) / dec->page_rows;
        for (uint32_t i = 0; i < pages && i < pps; ++i)
            if (dec->h_table_shadow[(size_t)s * pps + i] == kNoPage) ++want;
    }
    if (want > dec->free_pages.size()) return fail(dec, TNSR_B200_ERR_CAPACITY, "K/V page pool exhausted");
    for (uint32_t s = 0; s < B; ++s) {
        const uint32_t pages = (rows_needed[s] + dec->page_rows - 1) / dec->page_rows;
        for (uint32_t i = 0; i < pages && i < pps; ++i) {
            uint32_t& slot = dec->h_table_shadow[(size_t)s * pps + i];
            if (slot == kNoPage) {
                slot = dec->free_pages.back();
                dec->free_pages.pop_back();
                dec->table_dirty = true;
            }
        }
    }
    return TNSR_B200_OK;
}

// Queues the upload of the page table if it changed.  Unassigned entries go up as page 0: they are never followed,
// because no kernel touches a row its session does not hold yet.
int upload_page_table(tnsr_b200_decoder* dec) {
    if (!dec->paged || !dec->table_dirty) return TNSR_B200_OK;
    // the pinned copy may still be the source of a queued upload
    CU(dec, cudaStreamSynchronize(dec->stream));
    for (size_t i = 0; i < dec->h_table_shadow.size(); ++i)
        dec->h_table[i] = dec->h_table_shadow[i] == kNoPage ? 0u : dec->h_table_shadow[i];
    CU(dec, cudaMemcpyAsync(dec->d_table, dec->h_table, dec->h_table_shadow.size() * 4, cudaMemcpyHostToDevice, dec->stream));
    dec->table_dirty = false;
    return TNSR_B200_OK;
}

int reserve_uniform(tnsr_b200_decoder* dec, uint32_t rows_needed) {
    if (!dec->paged) return TNSR_B200_OK;
    std::vector<uint32_t> need(dec->cfg.batch, rows_needed);
    int rc = reserve_pages(dec, need.data());
    return rc ? rc : upload_page_table(dec);
}

// ---- one step on the strict f32 path -----------------------------------------
// `d_position` (optional): the position as a device scalar, for replay from a captured graph.
int step_strict(tnsr_b200_decoder* dec, const uint32_t* d_tokens, uint32_t chunk, uint32_t position,
                const uint32_t* d_position, uint32_t logit_rows) {
    const tnsr_b200_config& c = dec->cfg;
    const uint32_t d = c.embed_dim, f = c.feed_forward_dim, H = c.num_heads, B = c.batch, rows = B * chunk;
    cudaStream_t st = dec->stream;
    const int kvdt = dec->kv_bf16 ? TNSR_B200_BF16 : TNSR_B200_F32;
    RUN(dec, launch_embedding(dec->tok, dec->pos, d_tokens, dec->h, rows, chunk, position, d_position, c.vocab_size, d,
                              TNSR_B200_F32, dec->d_status, st));
    float* n = (float*)dec->n; float* q = (float*)dec->q; float* att = (float*)dec->att; float* ff = (float*)dec->ff;
    for (Layer& L : dec->layers) {
        RUN(dec, launch_layernorm(dec->h, L.ln1w, L.ln1b, n, rows, d, c.layer_norm_epsilon, TNSR_B200_F32, true, st));
        GemmEpilogue eq;
        eq.bias = L.bq;
        eq.round_bf16 = dec->kv_bf16;
        RUN(dec, launch_gemm_strict(n, (const float*)L.wq, q, d, rows, d, d, false, eq, st));
        GemmEpilogue ek;
        ek.round_bf16 = dec->kv_bf16;
        ek.out_dtype = kvdt;
        ek.rows_per_session = chunk; ek.out_session_rows = c.capacity; ek.row_offset = position; ek.d_row_offset = d_position;
        ek.bias = L.bk;
        RUN(dec, launch_gemm_strict(n, (const float*)L.wk, L.kcache, d, rows, d, d, false, ek, st));
        ek.bias = L.bv;
        RUN(dec, launch_gemm_strict(n, (const float*)L.wv, L.vcache, d, rows, d, d, false, ek, st));
        RUN(dec, launch_attention_strict(q, L.kcache, L.vcache, att, B, chunk, position, d_position, c.capacity, H, d / H, kvdt,
                                         dec->kv_bf16, st));
        GemmEpilogue eo;
        eo.bias = L.bo; eo.residual = dec->h; eo.ldr = d;
        RUN(dec, launch_gemm_strict(att, (const float*)L.wo, dec->h, d, rows, d, d, false, eo, st));
        RUN(dec, launch_layernorm(dec->h, L.ln2w, L.ln2b, n, rows, d, c.layer_norm_epsilon, TNSR_B200_F32, true, st));
        if (dec->swiglu) {
            GemmEpilogue eg; eg.bias = L.b_gate;
            RUN(dec, launch_gemm_strict(n, (const float*)L.w_gate, ff, f, rows, d, f, false, eg, st));
            GemmEpilogue eu; eu.bias = L.b_up;
            RUN(dec, launch_gemm_strict(n, (const float*)L.w_up, dec->ff2, f, rows, d, f, false, eu, st));
            RUN(dec, launch_swiglu_strict(ff, (const float*)dec->ff2, ff, (size_t)rows * f, st));
        } else {
            GemmEpilogue ei; ei.bias = L.b_in;
            ei.activation = c.activation == TNSR_B200_ACT_GELU ? ACT_GELU : ACT_RELU;
            RUN(dec, launch_gemm_strict(n, (const float*)L.w_in, ff, f, rows, d, f, false, ei, st));
        }
        GemmEpilogue ef; ef.bias = L.b_out; ef.residual = dec->h; ef.ldr = d;
        RUN(dec, launch_gemm_strict(ff, (const float*)L.w_out, dec->h, d, rows, f, d, false, ef, st));
    }
    const float* src = dec->h;
    if (logit_rows != rows) {
        RUN(dec, launch_gather_last_rows(dec->h, dec->hl, B, chunk, d, st));
        src = dec->hl;
    }
    RUN(dec, launch_layernorm(src, dec->fnw, dec->fnb, n, logit_rows, d, c.layer_norm_epsilon, TNSR_B200_F32, true, st));
    GemmEpilogue el;
    RUN(dec, launch_gemm_strict(n, (const float*)dec->tok, dec->logits, c.vocab_size, logit_rows, d, c.vocab_size, true, el, st));
    return TNSR_B200_OK;
}

// Largest batch whose single-token step runs each layer's projections as one persistent kernel (decode_tail.cu): the
// kernel keeps 32 session rows per CTA (LayerNorm rows in registers, activation ring in shared memory).
// Measured on B200 with the 12-layer d768 model, ms per step fused / operator by operator: 32 sessions 0.55 / 0.74.
constexpr uint32_t kTailMaxSessions = 32;

// ---- one step on the bf16 tensor-core path -----------------------------------
// The part of a step that belongs to a range of sessions [s0, s0 + ns): embedding and all layers, on stream `st`.
// Nothing in it couples two sessions, so disjoint ranges may run on different streams at the same time.
// `d_position` (optional): the position as a device scalar, so that a captured graph of the step can be replayed
// while the position advances.  `ragged`: d_position is an array with one position per session (single-token steps).
// `ws`: decode-attention scratch of this range.  `lean`: take the decode-attention form that leaves room on every SM
// for the other range's projection kernels.
int layers_bf16(tnsr_b200_decoder* dec, const uint32_t* d_tokens, uint32_t chunk, uint32_t position,
                const uint32_t* d_position, bool ragged, uint32_t s0, uint32_t ns, void* ws, bool lean, cudaStream_t st) {
    const tnsr_b200_config& c = dec->cfg;
    const uint32_t d = c.embed_dim, f = c.feed_forward_dim, H = c.num_heads, hd = d / H;
    const uint32_t rows = ns * chunk;
    dec->split_pending = 0;
    const size_t r0 = (size_t)s0 * chunk;                       // first activation row of the range
    const size_t cache0 = dec->paged ? 0 : (size_t)s0 * c.capacity * d;   // first cache element of the range
    KvPaging pg;                                                // paged: the pools are shared, the table is per session
    if (dec->paged) { pg.table = dec->d_table + (size_t)s0 * dec->pps; pg.page_rows = dec->page_rows; pg.pages_per_session = dec->pps; }
    float* h = dec->h + r0 * d;
    bf16* n = (bf16*)dec->n + r0 * d; bf16* q = (bf16*)dec->q + r0 * d; bf16* att = (bf16*)dec->att + r0 * d;
    bf16* ff = (bf16*)dec->ff + r0 * f;
    bf16* ff2 = dec->ff2 ? (bf16*)dec->ff2 + r0 * f : nullptr;
    const uint32_t* pos_arg = ragged ? d_position + s0 : d_position;
    RUN(dec, launch_embedding(dec->tok, dec->pos, d_tokens + r0, h, rows, chunk, position, pos_arg, c.vocab_size, d,
                              TNSR_B200_BF16, dec->d_status, st, ragged ? 1u : 0u));
    const bool fast_decode = chunk == 1 && ws && decode_attention_supported(H, hd);
    if (ragged && !fast_decode) return fail(dec, TNSR_B200_ERR_UNSUPPORTED, "ragged decode needs the split-KV attention kernel (head width 32, 64 or 128)");
    bool planned = false;
    // Small batch: everything between two attention scans is one persistent kernel (decode_tail.cu).
    if (fast_decode && !lean && dec->fused_gu && dec->tail_ws && dec->use_tail && ns <= kTailMaxSessions &&
        decode_tail_supported(ns, d, f)) {
        const size_t layers = dec->layers.size();
        auto tail = [&](size_t prev, bool with_prev, bool with_next) -> int {
            DecodeTailArgs a;
            a.rows = ns; a.d = d; a.f = f; a.eps = c.layer_norm_epsilon;
            a.h = h; a.att = att; a.ff = ff; a.q = q;
            a.workspace = dec->tail_ws; a.d_status = dec->d_status;
            if (with_prev) {
                const Layer& L = dec->layers[prev];
                a.run_o = a.run_ffn = true;
                a.wo = (const bf16*)L.wo; a.bo = L.bo; a.ln2w = L.ln2w; a.ln2b = L.ln2b; a.wgu = L.wgu; a.bgu = L.bgu;
                a.wdown = (const bf16*)L.w_out; a.bdown = L.b_out;
            }
            if (with_next) {
                const Layer& N = dec->layers[with_prev ? prev + 1 : prev];
                a.run_qkv = true;
                a.ln1w = N.ln1w; a.ln1b = N.ln1b; a.wqkv = N.wqkv; a.bqkv = N.bqkv;
                a.k_cache = (bf16*)N.kcache + cache0; a.v_cache = (bf16*)N.vcache + cache0;
                a.capacity = c.capacity; a.d_position = pos_arg; a.position = position; a.position_stride = ragged ? 1u : 0u;
                a.paging = &pg;
            }
            return launch_decode_tail(a, st);
        };
        RUN(dec, tail(0, false, true));
        for (size_t l = 0; l < layers; ++l) {
            Layer& L = dec->layers[l];
            bf16* kcache = (bf16*)L.kcache + cache0;
            bf16* vcache = (bf16*)L.vcache + cache0;
            if (ragged)
                RUN(dec, launch_decode_attention_ex(q, kcache, vcache, pos_arg, nullptr, 1, att, ws, dec->attn_ws_bytes, ns,
                                                    c.capacity, H, hd, !planned, dec->d_status, st, false, &pg));
            else
                RUN(dec, launch_decode_attention_ex(q, kcache, vcache, nullptr, d_position, d_position ? 1 : position + 1, att,
                                                    ws, dec->attn_ws_bytes, ns, c.capacity, H, hd, !planned, dec->d_status,
                                                    st, false, &pg));
            planned = true;
            RUN(dec, tail(l, true, l + 1 < layers));
        }
        return TNSR_B200_OK;
    }
    // Single-token steps of up to 256 rows: the two narrow projections (attention output, FFN down) divide their K extent
    // over several CTAs per tile; the partial sums are added to the residual, in a fixed order, by the LayerNorm that
    // follows (for the last layer's down projection that is the final LayerNorm in step_bf16: dec->split_pending).
    // Measured on B200, 12 layers of d 768, ms per step without / with: 64 sessions 0.840 / 0.789, 128 sessions 1.007 /
    // 0.954.  Not in a divided step (`lean`): there four times as many projection CTAs take the room on the SMs that
    // the other range's attention CTAs are waiting for (256 sessions in two ranges: 1.365 without, 1.549 with).
    const bool splitk = chunk == 1 && !lean && dec->split_ws && layernorm_fold_supported(d);
    float* part_ws = splitk ? dec->split_ws + (size_t)(s0 + 31) / 32 * 32 * d : nullptr;
    uint32_t pending = 0;                                       // partial sums of the previous layer's down projection
    for (Layer& L : dec->layers) {
        bf16* kcache = (bf16*)L.kcache + cache0;
        bf16* vcache = (bf16*)L.vcache + cache0;
        if (pending)
            RUN(dec, launch_layernorm_fold(h, part_ws, pending, dec->split_rows, L.ln1w, L.ln1b, n, rows, d, c.layer_norm_epsilon, st));
        else
            RUN(dec, launch_layernorm(h, L.ln1w, L.ln1b, n, rows, d, c.layer_norm_epsilon, TNSR_B200_BF16, false, st));
        pending = 0;
        GemmEpilogue eq;
        eq.bias = L.bqkv;
        GemmQkvTargets tg;
        tg.q = q; tg.k_cache = kcache; tg.v_cache = vcache;
        tg.d = d; tg.chunk = chunk; tg.capacity = c.capacity; tg.position = position; tg.d_position = pos_arg;
        tg.position_stride = ragged ? 1u : 0u;
        tg.paging = pg;
        RUN(dec, launch_gemm_bf16(n, L.wqkv, nullptr, 0, rows, 3 * d, d, GEMM_QKV, eq, &tg, dec->d_status, st));
        if (fast_decode) {
            // every session holds position + 1 keys; the item list is the same for all layers of this step
            if (ragged)   // session b holds d_position[b] + 1 keys
                RUN(dec, launch_decode_attention_ex(q, kcache, vcache, pos_arg, nullptr, 1, att, ws, dec->attn_ws_bytes, ns,
                                                    c.capacity, H, hd, !planned, dec->d_status, st, lean, &pg));
            else
                RUN(dec, launch_decode_attention_ex(q, kcache, vcache, nullptr, d_position, d_position ? 1 : position + 1, att,
                                                    ws, dec->attn_ws_bytes, ns, c.capacity, H, hd, !planned, dec->d_status,
                                                    st, lean, &pg));
            planned = true;
        } else if (chunk > 1 && prefill_attention_supported(hd) && c.prefill_mode != TNSR_B200_PREFILL_SCALAR && !dec->paged) {
            RUN(dec, launch_prefill_attention(q, kcache, vcache, att, ns, chunk, position, d_position, c.capacity, H, hd,
                                              dec->d_status, st));
        } else {
            RUN(dec, launch_attention_generic(q, kcache, vcache, att, ns, chunk, position, d_position, c.capacity, H, hd, st, &pg));
        }
        GemmEpilogue eo;
        eo.bias = L.bo; eo.residual = h; eo.ldr = d; eo.out_dtype = TNSR_B200_F32;
        const uint32_t split_o = splitk ? gemm_split_k(att, (const bf16*)L.wo, rows, d, d) : 0;
        if (split_o) { eo.split_k = split_o; eo.split_partials = part_ws; eo.split_rows = dec->split_rows; }
        RUN(dec, launch_gemm_bf16(att, (const bf16*)L.wo, h, d, rows, d, d, GEMM_PLAIN, eo, nullptr, dec->d_status, st));
        if (split_o)
            RUN(dec, launch_layernorm_fold(h, part_ws, split_o, dec->split_rows, L.ln2w, L.ln2b, n, rows, d, c.layer_norm_epsilon, st));
        else
            RUN(dec, launch_layernorm(h, L.ln2w, L.ln2b, n, rows, d, c.layer_norm_epsilon, TNSR_B200_BF16, false, st));
        if (dec->swiglu) {
            if (dec->fused_gu) {
                GemmEpilogue eg; eg.bias = L.bgu; eg.out_dtype = TNSR_B200_BF16;
                RUN(dec, launch_gemm_bf16(n, L.wgu, ff, f, rows, 2 * f, d, GEMM_SWIGLU, eg, nullptr, dec->d_status, st));
            } else {
                GemmEpilogue eg; eg.bias = L.b_gate; eg.out_dtype = TNSR_B200_BF16;
                RUN(dec, launch_gemm_bf16(n, (const bf16*)L.w_gate, ff, f, rows, f, d, GEMM_PLAIN, eg, nullptr, dec->d_status, st));
                GemmEpilogue eu; eu.bias = L.b_up; eu.out_dtype = TNSR_B200_BF16;
                RUN(dec, launch_gemm_bf16(n, (const bf16*)L.w_up, ff2, f, rows, f, d, GEMM_PLAIN, eu, nullptr, dec->d_status, st));
                RUN(dec, launch_swiglu(ff, ff2, ff, (uint64_t)rows * f, st));
            }
        } else {
            GemmEpilogue ei; ei.bias = L.b_in; ei.out_dtype = TNSR_B200_BF16;
            ei.activation = c.activation == TNSR_B200_ACT_GELU ? ACT_GELU : ACT_RELU;
            RUN(dec, launch_gemm_bf16(n, (const bf16*)L.w_in, ff, f, rows, f, d, GEMM_PLAIN, ei, nullptr, dec->d_status, st));
        }
        GemmEpilogue ef; ef.bias = L.b_out; ef.residual = h; ef.ldr = d; ef.out_dtype = TNSR_B200_F32;
        const uint32_t split_d = splitk ? gemm_split_k(ff, (const bf16*)L.w_out, rows, d, f) : 0;
        if (split_d) { ef.split_k = split_d; ef.split_partials = part_ws; ef.split_rows = dec->split_rows; }
        RUN(dec, launch_gemm_bf16(ff, (const bf16*)L.w_out, h, d, rows, d, f, GEMM_PLAIN, ef, nullptr, dec->d_status, st));
        pending = split_d;
    }
    dec->split_pending = pending;   // only an undivided step (one range: all rows) gets here with partial sums left
    return TNSR_B200_OK;
}

// Smallest batch whose single-token step is divided over two streams unless the configuration says otherwise (see
// step_bf16).  Measured on B200 with the 12-layer d768 model: 256 sessions 1.35 ms per step divided in two against
// 1.48 ms undivided (three parts 1.46, four 1.53); at 128 sessions 1.02 against 1.01 and at 64 sessions 0.88 against
// 0.83, because a half batch no longer keeps every SM streaming during its attention.
constexpr uint32_t kSplitMinSessions = 192;

// One whole step.  `fused_ids` (optional): greedy ids come straight out of the LM-head GEMM and no logits are written
// (only when the logits mode is NONE).
//
// Single-token steps of at least kSplitMinSessions sessions (or as many parts as the configuration's step_parts asks
// for) run as two half-batches on two streams.  Inside one half
// the step is a chain of short, latency-bound kernels (LayerNorm, the four projections) around one long,
// bandwidth-bound kernel per layer (decode attention); sessions are independent, so while one half streams its K/V
// rows the other half's short kernels run beside it on the same SMs (the lean kernel forms leave room for that) and
// their latency is hidden instead of added.  The halves fork after the ids are in place and join before the final
// LayerNorm and the LM head, which read the token table once for the whole batch.
int step_bf16(tnsr_b200_decoder* dec, const uint32_t* d_tokens, uint32_t chunk, uint32_t position,
              const uint32_t* d_position, uint32_t logit_rows, uint32_t* fused_ids, bool ragged = false) {
    const tnsr_b200_config& c = dec->cfg;
    const uint32_t d = c.embed_dim, H = c.num_heads, hd = d / H, B = c.batch, rows = B * chunk;
    cudaStream_t st = dec->stream;
    const bool split = chunk == 1 && dec->parts > 1 && !dec->profile_attention && decode_attention_supported(H, hd) &&
                       !debug_sync_enabled();
    if (split) {
        const uint32_t parts = dec->parts;
        CU(dec, cudaEventRecord(dec->ev_fork, st));
        int rc = TNSR_B200_OK;
        cudaError_t e = cudaSuccess;
        for (uint32_t p = 1; p < parts; ++p) {
            const uint32_t s0 = (uint32_t)((uint64_t)B * p / parts), s1 = (uint32_t)((uint64_t)B * (p + 1) / parts);
            cudaStream_t side = dec->side_stream[p - 1];
            CU(dec, cudaStreamWaitEvent(side, dec->ev_fork, 0));
            int r = layers_bf16(dec, d_tokens, chunk, position, d_position, ragged, s0, s1 - s0, dec->side_ws[p - 1], true, side);
            cudaError_t er = cudaEventRecord(dec->ev_join[p - 1], side);   // every fork is joined, also after a failure
            if (r && !rc) rc = r;
            if (er != cudaSuccess && e == cudaSuccess) e = er;
        }
        int r0 = layers_bf16(dec, d_tokens, chunk, position, d_position, ragged, 0, (uint32_t)((uint64_t)B / parts), dec->attn_ws,
                             true, st);
        for (uint32_t p = 1; p < parts; ++p) {
            cudaError_t er = cudaStreamWaitEvent(st, dec->ev_join[p - 1], 0);
            if (er != cudaSuccess && e == cudaSuccess) e = er;
        }
        if (rc) return rc;
        if (r0) return r0;
        if (e != cudaSuccess) return cuda_fail(dec, e, "joining the parts of the step");
    } else {
        int rc = layers_bf16(dec, d_tokens, chunk, position, d_position, ragged, 0, B, dec->attn_ws, false, st);
        if (rc) return rc;
    }
    bf16* n = (bf16*)dec->n;
    const float* src = dec->h;
    if (logit_rows != rows) {
        RUN(dec, launch_gather_last_rows(dec->h, dec->hl, B, chunk, d, st));
        src = dec->hl;
    }
    const uint32_t pending = dec->split_pending;
    dec->split_pending = 0;
    if (pending && src == dec->h)   // split-K is for single-token steps, whose logit rows are all rows
        RUN(dec, launch_layernorm_fold(dec->h, dec->split_ws, pending, dec->split_rows, dec->fnw, dec->fnb, n, logit_rows, d,
                                       c.layer_norm_epsilon, st));
    else
        RUN(dec, launch_layernorm(src, dec->fnw, dec->fnb, n, logit_rows, d, c.layer_norm_epsilon, TNSR_B200_BF16, false, st));
    // the tied head: the token table [vocab, d] already is the K-major operand
    if (fused_ids) {
        RUN(dec, launch_lm_head_argmax(n, (const bf16*)dec->tok, logit_rows, c.vocab_size, d, dec->lm_candidates, fused_ids,
                                       dec->d_status, st));
        return TNSR_B200_OK;
    }
    GemmEpilogue el; el.out_dtype = TNSR_B200_F32;
    RUN(dec, launch_gemm_bf16(n, (const bf16*)dec->tok, dec->logits, c.vocab_size, logit_rows, c.vocab_size, d, GEMM_PLAIN, el,
                              nullptr, dec->d_status, st));
    return TNSR_B200_OK;
}

int run_step_direct(tnsr_b200_decoder* dec, const uint32_t* d_tokens, uint32_t chunk, uint32_t position,
                    const uint32_t* d_position, uint32_t* d_argmax_out) {
    const tnsr_b200_config& c = dec->cfg;
    const uint32_t rows = c.batch * chunk;
    const uint32_t logit_rows = c.logits_mode == TNSR_B200_LOGITS_ALL ? rows : c.batch;
    const bool sampling = dec->sample_temperature > 0.0f;
    const bool fuse_ids = dec->bf16_path && c.logits_mode == TNSR_B200_LOGITS_NONE && d_argmax_out && dec->lm_candidates && !sampling;
    t_attention_timer = dec->profile_attention ? &dec->attention_timer : nullptr;
    t_pdl = dec->use_pdl && dec->bf16_path && chunk == 1;
    t_single_token_step = chunk == 1;
    int rc = dec->bf16_path ? step_bf16(dec, d_tokens, chunk, position, d_position, logit_rows, fuse_ids ? d_argmax_out : nullptr)
                            : step_strict(dec, d_tokens, chunk, position, d_position, logit_rows);
    t_attention_timer = nullptr;
    if (rc) { t_pdl = t_single_token_step = false; return rc; }
    if (d_argmax_out && !fuse_ids) {
        // last position of every session
        const float* base = dec->logits;
        uint32_t stride = c.vocab_size;
        if (logit_rows == rows && chunk > 1) {
            base = dec->logits + (size_t)(chunk - 1) * c.vocab_size;
            stride = chunk * c.vocab_size;
        }
        // the new token of a step that starts at `position` with `chunk` rows will sit at position + chunk
        int arc = sampling ? launch_sample_top_k(base, d_argmax_out, c.batch, c.vocab_size, stride, dec->sample_temperature,
                                                 dec->sample_top_k, dec->sample_seed, d_position, 0,
                                                 (d_position ? 0 : position) + chunk, 0, dec->stream)
                           : launch_argmax(base, d_argmax_out, c.batch, c.vocab_size, stride, dec->stream);
        if (arc) {
            t_pdl = t_single_token_step = false;
            dec->error = thread_error();
            return arc;
        }
    }
    t_pdl = t_single_token_step = false;
    return TNSR_B200_OK;
}

// One step.  Single-token steps are captured once per (ids pointer, output pointer) pair and replayed: the
// kernels read the position from dec->d_pos, which a one-thread kernel sets before each replay.
int run_step(tnsr_b200_decoder* dec, const uint32_t* d_tokens, uint32_t chunk, uint32_t position, uint32_t* d_argmax_out) {
    const bool graphable = dec->use_graphs && chunk == 1 && !dec->profile_attention && dec->stepped_once && !debug_sync_enabled();
    if (!graphable) {
        int rc = run_step_direct(dec, d_tokens, chunk, position, nullptr, d_argmax_out);
        if (rc == TNSR_B200_OK && chunk == 1) dec->stepped_once = true;
        return rc;
    }
    tnsr_b200_decoder::StepGraph* found = nullptr;
    for (auto& g : dec->graphs)
        if (g.tokens == d_tokens && g.argmax == d_argmax_out) { found = &g; break; }
    if (!found) {
        if (dec->graphs.size() >= 8) drop_graphs(dec);
        const uint64_t before = g_launches.load();
        cudaGraph_t graph = nullptr;
        CU(dec, cudaStreamBeginCapture(dec->stream, cudaStreamCaptureModeThreadLocal));
        int rc = run_step_direct(dec, d_tokens, 1, 0, dec->d_pos, d_argmax_out);
        cudaError_t e = cudaStreamEndCapture(dec->stream, &graph);
        const uint64_t kernels = g_launches.load() - before;
        g_launches.fetch_sub(kernels);  // nothing ran yet; replays are counted below
        if (rc != TNSR_B200_OK || e != cudaSuccess || !graph) {
            if (graph) cudaGraphDestroy(graph);
            cudaGetLastError();
            dec->use_graphs = false;  // fall back to direct launches for the rest of this session
            dec->failed = false;      // a launch that capture refuses is not a device failure; a real one shows again below
            return run_step_direct(dec, d_tokens, chunk, position, nullptr, d_argmax_out);
        }
        cudaGraphExec_t exec = nullptr;
        e = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) {
            cudaGetLastError();
            dec->use_graphs = false;
            return run_step_direct(dec, d_tokens, chunk, position, nullptr, d_argmax_out);
        }
        dec->graphs.push_back({d_tokens, d_argmax_out, exec, kernels});
        found = &dec->graphs.back();
    }
    RUN(dec, launch_fill_u32(dec->d_pos, position, 1, dec->stream));
    CU(dec, cudaGraphLaunch(found->exec, dec->stream));
    count_launch(found->kernels);
    return TNSR_B200_OK;
}

int validate_config(const tnsr_b200_config* c, std::string& why) {
    if (!c) { why = "null configuration"; return TNSR_B200_ERR_INVALID_ARGUMENT; }
    if (c->vocab_size == 0 || c->max_sequence_length == 0 || c->embed_dim == 0 || c->num_layers == 0 ||
        c->feed_forward_dim == 0 || c->num_heads == 0 || c->embed_dim % c->num_heads != 0 ||
        !(c->layer_norm_epsilon > 0.0f) || !std::isfinite(c->layer_norm_epsilon)) {
        why = "invalid model configuration";
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    if (c->activation > TNSR_B200_ACT_SWIGLU || c->weight_dtype > TNSR_B200_BF16 || c->kv_dtype > TNSR_B200_BF16 ||
        c->logits_mode > TNSR_B200_LOGITS_NONE || c->prefill_mode > TNSR_B200_PREFILL_SCALAR || c->step_parts > 4 || c->small_batch_mode > 1) {
        why = "invalid enum value in configuration";
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    if (c->weight_dtype == TNSR_B200_BF16 && c->kv_dtype != TNSR_B200_BF16) {
        why = "bf16 weights require a bf16 K/V cache";
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    if (c->batch == 0) { why = "decoder batch size must be non-zero"; return TNSR_B200_ERR_INVALID_ARGUMENT; }
    if (c->kv_page_rows) {
        if (c->weight_dtype != TNSR_B200_BF16 || c->kv_page_rows % 16 != 0 || c->capacity % c->kv_page_rows != 0) {
            why = "paged K/V needs bf16 weights and a page size that is a multiple of 16 rows and divides the capacity";
            return TNSR_B200_ERR_INVALID_ARGUMENT;
        }
    } else if (c->kv_pool_pages) {
        why = "kv_pool_pages without kv_page_rows";
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    if (c->capacity == 0 || c->capacity > c->max_sequence_length) {
        why = "decoder capacity must fit the model context";
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    uint64_t elements, bytes, total;
    if (mul_overflow((uint64_t)c->batch * c->capacity, c->embed_dim, &elements) || mul_overflow(elements, 4, &bytes) ||
        mul_overflow(bytes, 2ull * c->num_layers, &total) || (uint64_t)c->batch * c->capacity > 0xffffffffull) {
        why = "decoder cache size overflow";
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    return TNSR_B200_OK;
}

}  // namespace

// ==============================================================================
// C ABI
// ==============================================================================
extern "C" {

const char* tnsr_b200_version(void) { return "tnsr_b200 0.1 (sm_100a)"; }

int tnsr_b200_device_count(void) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        set_thread_error(std::string("cudaGetDeviceCount: ") + cudaGetErrorString(e));
        return e == cudaErrorNoDevice ? 0 : TNSR_B200_ERR_NO_DEVICE;
    }
    return n;
}

const char* tnsr_b200_last_error(const tnsr_b200_decoder* dec) { return dec ? dec->error.c_str() : thread_error(); }

uint64_t tnsr_b200_kernel_launches(void) { return g_launches.load(); }

int tnsr_b200_set_wait_limit_ns(uint64_t ns) {
    if (ns < 1000ull || ns > 60000000000ull) return fail(nullptr, TNSR_B200_ERR_INVALID_ARGUMENT, "wait limit must lie between 1 us and 60 s");
    g_wait_limit_ns.store(ns);
    return TNSR_B200_OK;
}

int tnsr_b200_test_lose_gemm_stage(uint32_t k_block) {
    t_lose_gemm_stage = k_block + 1;
    return TNSR_B200_OK;
}

int tnsr_b200_set_gemm_engine(int engine) {
    if (engine < 0 || engine > 4) return TNSR_B200_ERR_INVALID_ARGUMENT;
    g_gemm_engine = engine;
    return TNSR_B200_OK;
}

int tnsr_b200_decoder_create(const tnsr_b200_config* config, tnsr_b200_decoder** out) {
    if (!out) return fail(nullptr, TNSR_B200_ERR_INVALID_ARGUMENT, "null output handle");
    *out = nullptr;
    std::string why;
    int rc = validate_config(config, why);
    if (rc) return fail(nullptr, rc, why);
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(nullptr, TNSR_B200_ERR_NO_DEVICE, "initialize CUDA decoder: no CUDA device");
    }
    if (config->device < 0 || config->device >= count)
        return fail(nullptr, TNSR_B200_ERR_NO_DEVICE, "initialize CUDA decoder: device ordinal out of range");
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, config->device) != cudaSuccess || prop.major < 10) {
        cudaGetLastError();
        return fail(nullptr, TNSR_B200_ERR_NO_DEVICE, "initialize CUDA decoder: an sm_100 class device is required");
    }
    tnsr_b200_decoder* dec = new (std::nothrow) tnsr_b200_decoder();
    if (!dec) return fail(nullptr, TNSR_B200_ERR_OUT_OF_MEMORY, "host allocation failed");
    dec->cfg = *config;
    dec->bf16_path = config->weight_dtype == TNSR_B200_BF16;
    dec->kv_bf16 = config->kv_dtype == TNSR_B200_BF16;
    dec->swiglu = config->activation == TNSR_B200_ACT_SWIGLU;
    dec->fused_gu = dec->bf16_path && dec->swiglu && config->feed_forward_dim % 16 == 0;
    auto bail = [&](int code) {
        std::string msg = dec->error;
        tnsr_b200_decoder_destroy(dec);
        set_thread_error(msg);
        return code;
    };
    if (cudaSetDevice(config->device) != cudaSuccess) return bail(cuda_fail(dec, cudaGetLastError(), "cudaSetDevice"));
    cudaError_t e = cudaStreamCreateWithFlags(&dec->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return bail(cuda_fail(dec, e, "cudaStreamCreate"));
    describe_params(dec);
    if (config->kv_page_rows) {
        dec->paged = true;
        dec->page_rows = config->kv_page_rows;
        dec->pps = config->capacity / config->kv_page_rows;
        const uint64_t worst = (uint64_t)config->batch * dec->pps;
        dec->pool_pages = config->kv_pool_pages ? config->kv_pool_pages : (uint32_t)std::min<uint64_t>(worst, 0xffffffffull);
        if (dec->pool_pages > worst) dec->pool_pages = (uint32_t)worst;
        dec->h_table_shadow.assign((size_t)config->batch * dec->pps, kNoPage);
        for (uint32_t p = dec->pool_pages; p > 0; --p) dec->free_pages.push_back(p - 1);
        if ((rc = dev_alloc(dec, (void**)&dec->d_table, dec->h_table_shadow.size() * 4, true))) return bail(rc);
        if (cudaMallocHost((void**)&dec->h_table, dec->h_table_shadow.size() * 4) != cudaSuccess)
            return bail(cuda_fail(dec, cudaGetLastError(), "cudaMallocHost"));
    }
    if ((rc = allocate_weights(dec))) return bail(rc);
    const uint64_t d = config->embed_dim;
    if ((rc = dev_alloc(dec, (void**)&dec->hl, (size_t)config->batch * d * 4, false))) return bail(rc);
    if ((rc = dev_alloc(dec, (void**)&dec->d_argmax, (size_t)config->batch * 4, true))) return bail(rc);
    if ((rc = dev_alloc(dec, (void**)&dec->d_status, 16, true))) return bail(rc);
    if ((rc = dev_alloc(dec, (void**)&dec->d_pos, 16, true))) return bail(rc);
    if (dec->bf16_path && config->logits_mode == TNSR_B200_LOGITS_NONE)
        if ((rc = dev_alloc(dec, &dec->lm_candidates, lm_head_argmax_scratch_bytes(config->batch, config->vocab_size), false)))
            return bail(rc);
    {
        const char* v = std::getenv("TNSR_B200_NO_GRAPH");
        if (v && v[0] == '1') dec->use_graphs = false;
        v = std::getenv("TNSR_B200_NO_PDL");
        if (v && v[0] == '1') dec->use_pdl = false;

    }
    if (cudaMallocHost((void**)&dec->h_argmax, (size_t)config->batch * 4) != cudaSuccess ||
        cudaMallocHost((void**)&dec->h_status, 16) != cudaSuccess)
        return bail(cuda_fail(dec, cudaGetLastError(), "cudaMallocHost"));
    *dec->h_status = 0;
    if (dec->bf16_path && decode_attention_supported(config->num_heads, config->embed_dim / config->num_heads)) {
        dec->attn_ws_bytes = decode_attention_workspace_bytes(config->batch, config->capacity, config->num_heads,
                                                              config->embed_dim / config->num_heads);
        if ((rc = dev_alloc(dec, &dec->attn_ws, dec->attn_ws_bytes, true))) return bail(rc);
        // ranges of about 128 sessions (one session per CTA of the 128-CTA attention grid), at most four of them.
        // Measured, ms per step: 320 sessions 1.786 in two ranges / 1.743 in three, 384 sessions 2.007 / 1.921,
        // 512 sessions 2.481 in two / 2.552 in three / 2.399 in four; 256 sessions 1.348 in two / 1.493 in three.
        uint32_t auto_parts = 1;
        if (config->batch >= kSplitMinSessions) auto_parts = std::min(4u, std::max(2u, (config->batch + 64) / 128));
        uint32_t parts = config->step_parts ? config->step_parts : auto_parts;
        if (parts > config->batch) parts = config->batch;
        if (parts > 1 && cudaEventCreateWithFlags(&dec->ev_fork, cudaEventDisableTiming) != cudaSuccess)
            return bail(cuda_fail(dec, cudaGetLastError(), "fork event of the divided step"));
        for (uint32_t p = 1; p < parts; ++p) {
            if ((rc = dev_alloc(dec, &dec->side_ws[p - 1], dec->attn_ws_bytes, true))) return bail(rc);
            if (cudaStreamCreateWithFlags(&dec->side_stream[p - 1], cudaStreamNonBlocking) != cudaSuccess ||
                cudaEventCreateWithFlags(&dec->ev_join[p - 1], cudaEventDisableTiming) != cudaSuccess)
                return bail(cuda_fail(dec, cudaGetLastError(), "side stream of the divided step"));
        }
        dec->parts = parts;
        if (config->batch <= 256) {
            dec->split_rows = (config->batch + 31) / 32 * 32 + 32;
            if ((rc = dev_alloc(dec, (void**)&dec->split_ws, (size_t)4 * dec->split_rows * config->embed_dim * sizeof(float), true)))
                return bail(rc);
        }
        if (config->batch <= kTailMaxSessions) {
            if ((rc = dev_alloc(dec, &dec->tail_ws, decode_tail_workspace_bytes(), true))) return bail(rc);
            dec->use_tail = config->small_batch_mode == 0;
        }
    }
    if (dec->bf16_path) {
        dec->host_bqkv.assign((size_t)config->num_layers * 3 * d, 0.0f);
        if (dec->fused_gu) dec->host_bgu.assign((size_t)config->num_layers * 2 * config->feed_forward_dim, 0.0f);
    }
    e = cudaStreamSynchronize(dec->stream);
    if (e != cudaSuccess) return bail(cuda_fail(dec, e, "cudaStreamSynchronize"));
    *out = dec;
    return TNSR_B200_OK;
}

void tnsr_b200_decoder_destroy(tnsr_b200_decoder* dec) {
    if (!dec) return;
    cudaSetDevice(dec->cfg.device);
    if (dec->stream) cudaStreamSynchronize(dec->stream);
    for (void* p : dec->allocations) cudaFree(p);
    if (dec->h_tokens) cudaFreeHost(dec->h_tokens);
    if (dec->h_argmax) cudaFreeHost(dec->h_argmax);
    if (dec->h_positions) cudaFreeHost(dec->h_positions);
    if (dec->h_status) cudaFreeHost(dec->h_status);
    if (dec->h_stage) cudaFreeHost(dec->h_stage);
    if (dec->h_table) cudaFreeHost(dec->h_table);
    drop_graphs(dec);
    for (int i = 0; i < 3; ++i) {
        if (dec->side_stream[i]) { cudaStreamSynchronize(dec->side_stream[i]); cudaStreamDestroy(dec->side_stream[i]); }
        if (dec->ev_join[i]) cudaEventDestroy(dec->ev_join[i]);
    }
    if (dec->ev_fork) cudaEventDestroy(dec->ev_fork);
    for (cudaEvent_t e : dec->attention_timer.events) cudaEventDestroy(e);
    if (dec->stream) cudaStreamDestroy(dec->stream);
    cudaGetLastError();
    delete dec;
}

uint32_t tnsr_b200_decoder_param_count(const tnsr_b200_decoder* dec) { return dec ? (uint32_t)dec->params.size() : 0; }

uint64_t tnsr_b200_decoder_param_elems(const tnsr_b200_decoder* dec, uint32_t index) {
    return (dec && index < dec->params.size()) ? dec->params[index].elems : 0;
}

int tnsr_b200_decoder_upload(tnsr_b200_decoder* dec, uint32_t index, const float* host, uint64_t elems) {
    if (!dec) return fail(nullptr, TNSR_B200_ERR_INVALID_ARGUMENT, "null decoder");
    if (index >= dec->params.size() || !host) return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "parameter index or pointer invalid");
    const ParamInfo& p = dec->params[index];
    if (elems != p.elems) return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "parameter length mismatch");
    CU(dec, cudaSetDevice(dec->cfg.device));
    const tnsr_b200_config& c = dec->cfg;
    const uint32_t d = c.embed_dim, f = c.feed_forward_dim;
    cudaStream_t st = dec->stream;
    Layer* L = p.kind == P_TOK || p.kind == P_POS ? nullptr : (p.layer < dec->layers.size() ? &dec->layers[p.layer] : nullptr);
    const size_t bytes = (size_t)elems * 4;
    // f32 destinations (vectors on both paths, everything on the strict path)
    auto vec_target = [&]() -> float* {
        if (p.slot == 100) return dec->fnw;
        if (p.slot == 101) return dec->fnb;
        switch (p.slot) {
            case 0: return L->bo;
            case 1: return L->ln1w;
            case 2: return L->ln1b;
            case 3: return L->ln2w;
            case 4: return L->ln2b;
            default: return L->b_out;
        }
    };
    auto copy_f32 = [&](void* dst) -> int {
        CU(dec, cudaMemcpyAsync(dst, host, bytes, cudaMemcpyHostToDevice, st));
        CU(dec, cudaStreamSynchronize(st));  // `host` is pageable and not retained
        return TNSR_B200_OK;
    };
    if (p.kind == P_VEC) return copy_f32(vec_target());
    if (!dec->bf16_path) {
        switch (p.kind) {
            case P_TOK: return copy_f32(dec->tok);
            case P_POS: return copy_f32(dec->pos);
            case P_QKV_W: return copy_f32(p.slot == 0 ? L->wq : p.slot == 1 ? L->wk : L->wv);
            case P_QKV_B: return copy_f32(p.slot == 0 ? L->bq : p.slot == 1 ? L->bk : L->bv);
            case P_O_W: return copy_f32(L->wo);
            case P_FF_IN_W: return copy_f32(L->w_in);
            case P_FF_IN_B: return copy_f32(L->b_in);
            case P_FF_OUT_W: return copy_f32(L->w_out);
            case P_GATE_W: return copy_f32(L->w_gate);
            case P_GATE_B: return copy_f32(L->b_gate);
            case P_UP_W: return copy_f32(L->w_up);
            case P_UP_B: return copy_f32(L->b_up);
            default: return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "unknown parameter kind");
        }
    }
    // bf16 path: biases stay f32 (possibly packed); matrices are staged in f32 on the device, then repacked
    if (p.kind == P_QKV_B) {
        float* hb = dec->host_bqkv.data() + ((size_t)p.layer * 3 + p.slot) * d;
        std::memcpy(hb, host, bytes);
        CU(dec, cudaMemcpyAsync(L->bqkv + (size_t)p.slot * d, hb, bytes, cudaMemcpyHostToDevice, st));
        CU(dec, cudaStreamSynchronize(st));
        return TNSR_B200_OK;
    }
    if (p.kind == P_FF_IN_B) return copy_f32(L->b_in);
    if (p.kind == P_GATE_B || p.kind == P_UP_B) {
        if (!dec->fused_gu) return copy_f32(p.kind == P_GATE_B ? L->b_gate : L->b_up);
        float* hb = dec->host_bgu.data() + (size_t)p.layer * 2 * f;
        const uint32_t off = p.kind == P_GATE_B ? 0 : 16;
        for (uint32_t cidx = 0; cidx < f; ++cidx) hb[(cidx / 16) * 32 + off + cidx % 16] = host[cidx];
        CU(dec, cudaMemcpyAsync(L->bgu, hb, (size_t)2 * f * 4, cudaMemcpyHostToDevice, st));
        CU(dec, cudaStreamSynchronize(st));
        return TNSR_B200_OK;
    }
    if (bytes > dec->d_stage_bytes) {
        CU(dec, cudaStreamSynchronize(st));
        dev_free(dec, dec->d_stage);
        dec->d_stage = nullptr;
        dec->d_stage_bytes = 0;
        int rc = dev_alloc(dec, (void**)&dec->d_stage, bytes, false);
        if (rc) return rc;
        dec->d_stage_bytes = bytes;
    }
    CU(dec, cudaMemcpyAsync(dec->d_stage, host, bytes, cudaMemcpyHostToDevice, st));
    int rc = TNSR_B200_OK;
    switch (p.kind) {
        case P_TOK: rc = launch_f32_to_bf16(dec->d_stage, (bf16*)dec->tok, elems, st); break;
        case P_POS: rc = launch_f32_to_bf16(dec->d_stage, (bf16*)dec->pos, elems, st); break;
        case P_QKV_W: rc = launch_transpose_f32_to_bf16_mapped(dec->d_stage, L->wqkv, d, d, p.slot * d, d, d, st); break;
        case P_O_W: rc = launch_transpose_f32_to_bf16(dec->d_stage, (bf16*)L->wo, d, d, st); break;
        case P_FF_IN_W: rc = launch_transpose_f32_to_bf16(dec->d_stage, (bf16*)L->w_in, d, f, st); break;
        case P_FF_OUT_W: rc = launch_transpose_f32_to_bf16(dec->d_stage, (bf16*)L->w_out, f, d, st); break;
        case P_GATE_W:
            rc = dec->fused_gu ? launch_transpose_f32_to_bf16_mapped(dec->d_stage, L->wgu, d, f, 0, 16, 32, st)
                               : launch_transpose_f32_to_bf16(dec->d_stage, (bf16*)L->w_gate, d, f, st);
            break;
        case P_UP_W:
            rc = dec->fused_gu ? launch_transpose_f32_to_bf16_mapped(dec->d_stage, L->wgu, d, f, 16, 16, 32, st)
                               : launch_transpose_f32_to_bf16(dec->d_stage, (bf16*)L->w_up, d, f, st);
            break;
        default: return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "unknown parameter kind");
    }
    if (rc) { dec->error = thread_error(); return rc; }
    CU(dec, cudaStreamSynchronize(st));
    return TNSR_B200_OK;
}

int tnsr_b200_decoder_reset(tnsr_b200_decoder* dec) {
    if (!dec) return fail(nullptr, TNSR_B200_ERR_INVALID_ARGUMENT, "null decoder");
    CU(dec, cudaSetDevice(dec->cfg.device));
    const size_t cache_bytes = dec->paged ? (size_t)dec->pool_pages * dec->page_rows * dec->cfg.embed_dim * kv_elt(dec)
                                          : (size_t)dec->cfg.batch * dec->cfg.capacity * dec->cfg.embed_dim * kv_elt(dec);
    if (dec->paged) {
        dec->free_pages.clear();
        for (uint32_t p = dec->pool_pages; p > 0; --p) dec->free_pages.push_back(p - 1);
        std::fill(dec->h_table_shadow.begin(), dec->h_table_shadow.end(), kNoPage);
        dec->table_dirty = true;
    }
    for (Layer& L : dec->layers) {
        CU(dec, cudaMemsetAsync(L.kcache, 0, cache_bytes, dec->stream));
        CU(dec, cudaMemsetAsync(L.vcache, 0, cache_bytes, dec->stream));
    }
    CU(dec, cudaMemsetAsync(dec->d_status, 0, 16, dec->stream));
    if (dec->tail_ws) CU(dec, cudaMemsetAsync(dec->tail_ws, 0, decode_tail_workspace_bytes(), dec->stream));
    CU(dec, cudaStreamSynchronize(dec->stream));
    dec->failed = false;
    return TNSR_B200_OK;
}

static int check_step_args(tnsr_b200_decoder* dec, uint32_t chunk, uint32_t position) {
    if (dec->failed) return fail(dec, TNSR_B200_ERR_FAILED_STATE, "decoder execution failed; reset the cache before reuse");
    if (chunk == 0) return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "tokens must be a nonempty rectangular [batch, sequence] chunk");
    if (position > dec->cfg.capacity || chunk > dec->cfg.capacity - position)
        return fail(dec, TNSR_B200_ERR_CAPACITY, "decoder context capacity exceeded");
    if ((uint64_t)dec->cfg.batch * chunk > 0x7fffffffull) return fail(dec, TNSR_B200_ERR_UNSUPPORTED, "chunk too large");
    return TNSR_B200_OK;
}

static int device_status_to_code(tnsr_b200_decoder* dec, int status) {
    switch (status) {
        case DEV_OK: return TNSR_B200_OK;
        case DEV_TOKEN_RANGE: return fail(dec, TNSR_B200_ERR_TOKEN_RANGE, "decoder token is outside the vocabulary");
        case DEV_TIMEOUT: dec->failed = true; return fail(dec, TNSR_B200_ERR_TIMEOUT, "a device-side wait timed out");
        default: dec->failed = true; return fail(dec, TNSR_B200_ERR_CUDA, "device reported an invalid session length");
    }
}

int tnsr_b200_decoder_decode(tnsr_b200_decoder* dec, const uint32_t* tokens, uint32_t chunk, uint32_t position,
                             float* logits_out, uint32_t* argmax_out) {
    if (!dec) return fail(nullptr, TNSR_B200_ERR_INVALID_ARGUMENT, "null decoder");
    int rc = check_step_args(dec, chunk, position);
    if (rc) return rc;
    const tnsr_b200_config& c = dec->cfg;
    if (!tokens) return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "null token pointer");
    if (c.logits_mode == TNSR_B200_LOGITS_NONE && logits_out)
        return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "logits_out must be NULL when logits_mode is NONE");
    const uint32_t rows = c.batch * chunk;
    for (uint32_t i = 0; i < rows; ++i)
        if (tokens[i] >= c.vocab_size) return fail(dec, TNSR_B200_ERR_TOKEN_RANGE, "decoder token is outside the vocabulary");
    CU(dec, cudaSetDevice(c.device));
    const uint32_t logit_rows = c.logits_mode == TNSR_B200_LOGITS_ALL ? rows : c.batch;
    if ((rc = ensure_rows(dec, rows, logit_rows))) return rc;
    if ((rc = reserve_uniform(dec, position + chunk))) return rc;
    dec->failed = true;  // poisoned until the step has completed (src/nn/kv_cache.rs:331)
    std::memcpy(dec->h_tokens, tokens, (size_t)rows * 4);
    CU(dec, cudaMemcpyAsync(dec->d_tokens, dec->h_tokens, (size_t)rows * 4, cudaMemcpyHostToDevice, dec->stream));
    if ((rc = run_step(dec, dec->d_tokens, chunk, position, argmax_out ? dec->d_argmax : nullptr))) return rc;
    if (logits_out)
        CU(dec, cudaMemcpyAsync(logits_out, dec->logits, (size_t)logit_rows * c.vocab_size * 4, cudaMemcpyDeviceToHost, dec->stream));
    if (argmax_out)
        CU(dec, cudaMemcpyAsync(dec->h_argmax, dec->d_argmax, (size_t)c.batch * 4, cudaMemcpyDeviceToHost, dec->stream));
    CU(dec, cudaMemcpyAsync(dec->h_status, dec->d_status, 4, cudaMemcpyDeviceToHost, dec->stream));
    CU(dec, cudaStreamSynchronize(dec->stream));
    if (*dec->h_status != DEV_OK) {
        int status = *dec->h_status;
        cudaMemsetAsync(dec->d_status, 0, 16, dec->stream);
        return device_status_to_code(dec, status);
    }
    if (argmax_out) std::memcpy(argmax_out, dec->h_argmax, (size_t)c.batch * 4);
    dec->failed = false;
    return TNSR_B200_OK;
}

// One new token per session, every session at its own position (no reference counterpart: the reference's
// sessions advance together).  Session b writes its K/V row at positions[b] and attends rows 0 .. positions[b].
int tnsr_b200_decoder_decode_ragged(tnsr_b200_decoder* dec, const uint32_t* tokens, const uint32_t* positions,
                                    float* logits_out, uint32_t* argmax_out) {
    if (!dec) return fail(nullptr, TNSR_B200_ERR_INVALID_ARGUMENT, "null decoder");
    if (dec->failed) return fail(dec, TNSR_B200_ERR_FAILED_STATE, "decoder execution failed; reset the cache before reuse");
    const tnsr_b200_config& c = dec->cfg;
    if (!dec->bf16_path) return fail(dec, TNSR_B200_ERR_UNSUPPORTED, "ragged decode is implemented for bf16 weights only");
    if (!tokens || !positions) return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "null token or position pointer");
    if (c.logits_mode == TNSR_B200_LOGITS_NONE && logits_out)
        return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "logits_out must be NULL when logits_mode is NONE");
    for (uint32_t b = 0; b < c.batch; ++b) {
        if (positions[b] >= c.capacity) return fail(dec, TNSR_B200_ERR_CAPACITY, "decoder context capacity exceeded");
        if (tokens[b] >= c.vocab_size) return fail(dec, TNSR_B200_ERR_TOKEN_RANGE, "decoder token is outside the vocabulary");
    }
    CU(dec, cudaSetDevice(c.device));
    int rc;
    if ((rc = ensure_rows(dec, c.batch, c.batch))) return rc;
    if (!dec->d_positions) {
        if ((rc = dev_alloc(dec, (void**)&dec->d_positions, (size_t)c.batch * 4, true))) return rc;
        CU(dec, cudaMallocHost((void**)&dec->h_positions, (size_t)c.batch * 4));
    }
    if (dec->paged) {
        std::vector<uint32_t> need(c.batch);
        for (uint32_t b = 0; b < c.batch; ++b) need[b] = positions[b] + 1;
        if ((rc = reserve_pages(dec, need.data()))) return rc;
        if ((rc = upload_page_table(dec))) return rc;
    }
    dec->failed = true;
    std::memcpy(dec->h_tokens, tokens, (size_t)c.batch * 4);
    std::memcpy(dec->h_positions, positions, (size_t)c.batch * 4);
    CU(dec, cudaMemcpyAsync(dec->d_tokens, dec->h_tokens, (size_t)c.batch * 4, cudaMemcpyHostToDevice, dec->stream));
    CU(dec, cudaMemcpyAsync(dec->d_positions, dec->h_positions, (size_t)c.batch * 4, cudaMemcpyHostToDevice, dec->stream));
    const bool sampling = dec->sample_temperature > 0.0f;
    const bool fuse_ids = c.logits_mode == TNSR_B200_LOGITS_NONE && argmax_out && dec->lm_candidates && !sampling;
    if ((rc = step_bf16(dec, dec->d_tokens, 1, 0, dec->d_positions, c.batch, fuse_ids ? dec->d_argmax : nullptr, true))) return rc;
    if (argmax_out && !fuse_ids) {
        // session b's new token will sit at positions[b] + 1
        rc = sampling ? launch_sample_top_k(dec->logits, dec->d_argmax, c.batch, c.vocab_size, c.vocab_size, dec->sample_temperature,
                                            dec->sample_top_k, dec->sample_seed, dec->d_positions, 1, 1, 0, dec->stream)
                      : launch_argmax(dec->logits, dec->d_argmax, c.batch, c.vocab_size, c.vocab_size, dec->stream);
        if (rc) { dec->error = thread_error(); return rc; }
    }
    if (logits_out)
        CU(dec, cudaMemcpyAsync(logits_out, dec->logits, (size_t)c.batch * c.vocab_size * 4, cudaMemcpyDeviceToHost, dec->stream));
    if (argmax_out)
        CU(dec, cudaMemcpyAsync(dec->h_argmax, dec->d_argmax, (size_t)c.batch * 4, cudaMemcpyDeviceToHost, dec->stream));
    CU(dec, cudaMemcpyAsync(dec->h_status, dec->d_status, 4, cudaMemcpyDeviceToHost, dec->stream));
    CU(dec, cudaStreamSynchronize(dec->stream));
    if (*dec->h_status != DEV_OK) {
        int status = *dec->h_status;
        cudaMemsetAsync(dec->d_status, 0, 16, dec->stream);
        return device_status_to_code(dec, status);
    }
    if (argmax_out) std::memcpy(argmax_out, dec->h_argmax, (size_t)c.batch * 4);
    dec->failed = false;
    return TNSR_B200_OK;
}

int tnsr_b200_decoder_decode_device(tnsr_b200_decoder* dec, const uint32_t* d_tokens, uint32_t chunk, uint32_t position,
                                    uint32_t* d_argmax_out) {
    if (!dec) return fail(nullptr, TNSR_B200_ERR_INVALID_ARGUMENT, "null decoder");
    int rc = check_step_args(dec, chunk, position);
    if (rc) return rc;
    if (!d_tokens) return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "null token pointer");
    const tnsr_b200_config& c = dec->cfg;
    CU(dec, cudaSetDevice(c.device));
    const uint32_t rows = c.batch * chunk;
    const uint32_t logit_rows = c.logits_mode == TNSR_B200_LOGITS_ALL ? rows : c.batch;
    if ((rc = ensure_rows(dec, rows, logit_rows))) return rc;
    if ((rc = reserve_uniform(dec, position + chunk))) return rc;
    return run_step(dec, d_tokens, chunk, position, d_argmax_out);
}

int tnsr_b200_decoder_set_sampler(tnsr_b200_decoder* dec, float temperature, uint32_t top_k, uint64_t seed) {
    if (!dec) return fail(nullptr, TNSR_B200_ERR_INVALID_ARGUMENT, "null decoder");
    if (temperature > 0.0f && (!std::isfinite(temperature) || top_k == 0 || top_k > 256))
        return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "sampling needs a finite temperature and 1 <= top_k <= 256");
    CU(dec, cudaSetDevice(dec->cfg.device));
    CU(dec, cudaStreamSynchronize(dec->stream));
    drop_graphs(dec);   // captured steps contain the previous pick
    dec->sample_temperature = temperature > 0.0f ? temperature : 0.0f;
    dec->sample_top_k = top_k;
    dec->sample_seed = seed;
    return TNSR_B200_OK;
}

int tnsr_b200_decoder_release(tnsr_b200_decoder* dec, uint32_t session) {
    if (!dec) return fail(nullptr, TNSR_B200_ERR_INVALID_ARGUMENT, "null decoder");
    if (!dec->paged) return fail(dec, TNSR_B200_ERR_UNSUPPORTED, "release applies to paged handles only");
    if (session >= dec->cfg.batch) return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "session index out of range");
    CU(dec, cudaSetDevice(dec->cfg.device));
    CU(dec, cudaStreamSynchronize(dec->stream));   // queued steps may still read the pages
    for (uint32_t i = 0; i < dec->pps; ++i) {
        uint32_t& slot = dec->h_table_shadow[(size_t)session * dec->pps + i];
        if (slot != kNoPage) {
            dec->free_pages.push_back(slot);
            slot = kNoPage;
            dec->table_dirty = true;
        }
    }
    return TNSR_B200_OK;
}

uint32_t tnsr_b200_decoder_free_pages(const tnsr_b200_decoder* dec) { return dec && dec->paged ? (uint32_t)dec->free_pages.size() : 0; }

int tnsr_b200_decoder_synchronize(tnsr_b200_decoder* dec) {
    if (!dec) return fail(nullptr, TNSR_B200_ERR_INVALID_ARGUMENT, "null decoder");
    CU(dec, cudaSetDevice(dec->cfg.device));
    CU(dec, cudaMemcpyAsync(dec->h_status, dec->d_status, 4, cudaMemcpyDeviceToHost, dec->stream));
    CU(dec, cudaStreamSynchronize(dec->stream));
    if (*dec->h_status != DEV_OK) {
        int status = *dec->h_status;
        cudaMemsetAsync(dec->d_status, 0, 16, dec->stream);
        return device_status_to_code(dec, status);
    }
    return TNSR_B200_OK;
}

int tnsr_b200_decoder_profile_attention(tnsr_b200_decoder* dec, int enable) {
    if (!dec) return fail(nullptr, TNSR_B200_ERR_INVALID_ARGUMENT, "null decoder");
    dec->profile_attention = enable != 0;
    return TNSR_B200_OK;
}

int tnsr_b200_decoder_attention_profile(tnsr_b200_decoder* dec, double* total_ms, uint64_t* launches) {
    if (!dec || !total_ms || !launches) return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "null argument");
    CU(dec, cudaSetDevice(dec->cfg.device));
    CU(dec, cudaStreamSynchronize(dec->stream));
    double sum = 0.0;
    KernelTimer& t = dec->attention_timer;
    for (size_t i = 0; i + 1 < t.used; i += 2) {
        float ms = 0.0f;
        CU(dec, cudaEventElapsedTime(&ms, t.events[i], t.events[i + 1]));
        sum += ms;
    }
    *total_ms = sum;
    *launches = t.used / 2;
    t.used = 0;
    return TNSR_B200_OK;
}

void* tnsr_b200_decoder_stream(tnsr_b200_decoder* dec) { return dec ? (void*)dec->stream : nullptr; }

int tnsr_b200_decoder_read_cache(tnsr_b200_decoder* dec, uint32_t index, float* host_out) {
    if (!dec || !host_out) return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "null argument");
    if (index >= 2 * dec->cfg.num_layers) return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "cache index out of range");
    CU(dec, cudaSetDevice(dec->cfg.device));
    const uint64_t elems = (uint64_t)dec->cfg.batch * dec->cfg.capacity * dec->cfg.embed_dim;
    Layer& L = dec->layers[index / 2];
    const void* src = (index & 1) ? L.vcache : L.kcache;
    if (dec->paged) {
        // the pool as f32 on the host, then every session's pages in logical order (rows of unassigned pages are zero)
        const uint64_t d = dec->cfg.embed_dim, page_elems = (uint64_t)dec->page_rows * d, pool_elems = dec->pool_pages * page_elems;
        float* tmp = nullptr;
        int rc = dev_alloc(dec, (void**)&tmp, pool_elems * 4, false);
        if (rc) return rc;
        std::vector<float> pool(pool_elems);
        rc = launch_bf16_to_f32((const bf16*)src, tmp, pool_elems, dec->stream);
        if (rc == TNSR_B200_OK) {
            cudaError_t e = cudaMemcpyAsync(pool.data(), tmp, pool_elems * 4, cudaMemcpyDeviceToHost, dec->stream);
            if (e == cudaSuccess) e = cudaStreamSynchronize(dec->stream);
            if (e != cudaSuccess) rc = cuda_fail(dec, e, "read_cache copy");
        } else {
            dec->error = thread_error();
        }
        cudaStreamSynchronize(dec->stream);
        dev_free(dec, tmp);
        if (rc) return rc;
        for (uint32_t s = 0; s < dec->cfg.batch; ++s)
            for (uint32_t i = 0; i < dec->pps; ++i) {
                float* dst = host_out + ((uint64_t)s * dec->cfg.capacity + (uint64_t)i * dec->page_rows) * d;
                const uint32_t page = dec->h_table_shadow[(size_t)s * dec->pps + i];
                if (page == kNoPage) std::memset(dst, 0, page_elems * 4);
                else std::memcpy(dst, pool.data() + page * page_elems, page_elems * 4);
            }
        return TNSR_B200_OK;
    }
    if (!dec->kv_bf16) {
        CU(dec, cudaMemcpyAsync(host_out, src, elems * 4, cudaMemcpyDeviceToHost, dec->stream));
        CU(dec, cudaStreamSynchronize(dec->stream));
        return TNSR_B200_OK;
    }
    float* tmp = nullptr;
    int rc = dev_alloc(dec, (void**)&tmp, elems * 4, false);
    if (rc) return rc;
    rc = launch_bf16_to_f32((const bf16*)src, tmp, elems, dec->stream);
    if (rc == TNSR_B200_OK) {
        cudaError_t e = cudaMemcpyAsync(host_out, tmp, elems * 4, cudaMemcpyDeviceToHost, dec->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(dec->stream);
        if (e != cudaSuccess) rc = cuda_fail(dec, e, "read_cache copy");
    } else {
        dec->error = thread_error();
    }
    cudaStreamSynchronize(dec->stream);
    dev_free(dec, tmp);
    return rc;
}

int tnsr_b200_decoder_write_cache(tnsr_b200_decoder* dec, uint32_t index, const float* host_in) {
    if (!dec || !host_in) return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "null argument");
    if (index >= 2 * dec->cfg.num_layers) return fail(dec, TNSR_B200_ERR_INVALID_ARGUMENT, "cache index out of range");
    CU(dec, cudaSetDevice(dec->cfg.device));
    const uint64_t elems = (uint64_t)dec->cfg.batch * dec->cfg.capacity * dec->cfg.embed_dim;
    Layer& L = dec->layers[index / 2];
    void* dst = (index & 1) ? L.vcache : L.kcache;
    if (dec->paged) {
        // writing whole tensors needs every page of every session; rows travel in pool order
        int rc = reserve_uniform(dec, dec->cfg.capacity);
        if (rc) return rc;
        const uint64_t d = dec->cfg.embed_dim, page_elems = (uint64_t)dec->page_rows * d, pool_elems = dec->pool_pages * page_elems;
        std::vector<float> pool(pool_elems, 0.0f);
        for (uint32_t s = 0; s < dec->cfg.batch; ++s)
            for (uint32_t i = 0; i < dec->pps; ++i)
                std::memcpy(pool.data() + dec->h_table_shadow[(size_t)s * dec->pps + i] * page_elems,
                            host_in + ((uint64_t)s * dec->cfg.capacity + (uint64_t)i * dec->page_rows) * d, page_elems * 4);
        float* tmp = nullptr;
        rc = dev_alloc(dec, (void**)&tmp, pool_elems * 4, false);
        if (rc) return rc;
        cudaError_t e = cudaMemcpyAsync(tmp, pool.data(), pool_elems * 4, cudaMemcpyHostToDevice, dec->stream);
        if (e != cudaSuccess) rc = cuda_fail(dec, e, "write_cache copy");
        if (rc == TNSR_B200_OK) {
            rc = launch_f32_to_bf16(tmp, (bf16*)dst, pool_elems, dec->stream);
            if (rc) dec->error = thread_error();
        }
        cudaStreamSynchronize(dec->stream);
        dev_free(dec, tmp);
        return rc;
    }
    if (!dec->kv_bf16) {
        CU(dec, cudaMemcpyAsync(dst, host_in, elems * 4, cudaMemcpyHostToDevice, dec->stream));
        CU(dec, cudaStreamSynchronize(dec->stream));
        return TNSR_B200_OK;
    }
    float* tmp = nullptr;
    int rc = dev_alloc(dec, (void**)&tmp, elems * 4, false);
    if (rc) return rc;
    cudaError_t e = cudaMemcpyAsync(tmp, host_in, elems * 4, cudaMemcpyHostToDevice, dec->stream);
    if (e != cudaSuccess) rc = cuda_fail(dec, e, "write_cache copy");
    if (rc == TNSR_B200_OK) {
        rc = launch_f32_to_bf16(tmp, (bf16*)dst, elems, dec->stream);
        if (rc) dec->error = thread_error();
    }
    cudaStreamSynchronize(dec->stream);
    dev_free(dec, tmp);
    return rc;
}

}  // extern "C"
