// Shared declarations of the sm_100a kernels behind the C ABI in include/tnsr_b200.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <string>
#include <vector>

#include "../../include/tnsr_b200.h"

namespace tb {

typedef __nv_bfloat16 bf16;

// ---- host-side plumbing ----------------------------------------------------

extern std::atomic<uint64_t> g_launches;       // kernels launched by this library
extern std::atomic<uint64_t> g_wait_limit_ns;  // bound of every device-side barrier wait; launchers copy it into kernel parameters
// Test hook: when non-zero, the next tcgen05 GEMM launched from this thread loses the copies of k-block (value - 1) of
// its first tile, so a bounded wait runs out and the kernel reports DEV_TIMEOUT; the launcher clears it.
extern thread_local uint32_t t_lose_gemm_stage;
void set_thread_error(const std::string& msg);  // message for calls without a handle
const char* thread_error();

inline void count_launch(uint64_t n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// Status of the last launch on the current thread's device, as a tnsr_b200 code.
// With TNSR_B200_DEBUG_SYNC=1 in the environment every launch is followed by a
// device synchronisation, so an asynchronous fault is attributed to its kernel.
bool debug_sync_enabled();
inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && debug_sync_enabled()) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        set_thread_error(std::string(what) + ": " + cudaGetErrorString(e));
        return TNSR_B200_ERR_CUDA;
    }
    return TNSR_B200_OK;
}

// Optional per-thread sink: when set, the decode-attention launcher records an
// event pair around its main kernel.
struct KernelTimer {
    std::vector<cudaEvent_t> events;  // start/stop pairs
    size_t used = 0;                  // events consumed so far
};
extern thread_local KernelTimer* t_attention_timer;

// Programmatic dependent launch: while t_pdl is set (the session sets it around single-token steps) kernels are
// launched with programmatic stream serialization, i.e. a kernel may be scheduled while its predecessor in the
// stream is still draining.  Every kernel launched this way starts with pdl_wait(), which blocks until the
// predecessor has completed and its writes are visible, so only launch latency overlaps, never data.
extern thread_local bool t_pdl;
// Set by the session around single-token steps: their LayerNorms have few rows and take the block-per-row kernel.  The
// choice follows the kind of step, never the row count, so that a session's LayerNorm bits do not depend on the batch it is in.
extern thread_local bool t_single_token_step;

// Asks (once per kernel and device) for the largest shared-memory carve-out whenever `kernel` runs.  The split between
// L1 and shared memory is a per-SM setting that can only change while the SM is empty, so two kernels can share an SM
// only if they agree on it; with every kernel of the library on the same setting, a CTA of one stream's kernel can
// move in beside a CTA of another stream's kernel as soon as threads, registers and shared memory allow.
void prefer_max_shared_carveout(const void* kernel);

template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    prefer_max_shared_carveout(reinterpret_cast<const void*>(kernel));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = t_pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }
inline uint64_t ceil_div64(uint64_t a, uint64_t b) { return (a + b - 1) / b; }

// FFN / epilogue activation codes shared by host and device.
enum : int { ACT_NONE = -1, ACT_RELU = 0, ACT_GELU = 1 };

// Device-side status word: kernels never trap; they record the first problem
// here and carry on with harmless values.
enum : int {
    DEV_OK = 0,
    DEV_TOKEN_RANGE = 1,    // an id >= vocab reached the gather
    DEV_TIMEOUT = 2,        // a bounded mbarrier wait gave up
    DEV_BAD_LENGTH = 3      // a session length beyond the cache capacity
};

// ---- operator launchers (one per kernel family) -----------------------------
// Every launcher queues work on `stream` and returns a tnsr_b200 status; none
// synchronises.  `d_position` arguments are device scalars so that one captured
// graph of a decode step can be replayed while the position advances.

struct GemmEpilogue {
    const float* bias = nullptr;      // [n] f32, added after accumulation
    const float* residual = nullptr;  // [m, ldr] f32, added last (f32 output only)
    uint32_t ldr = 0;
    int activation = ACT_NONE;        // applied to acc + bias
    int out_dtype = TNSR_B200_F32;    // f32 or bf16
    int round_bf16 = 0;               // strict path: round the f32 result to bf16 precision
    // Output row mapping: logical row r = s * rows_per_session + t lands at
    // out + ((s * out_session_rows + row_offset + t) * ldc).  rows_per_session == 0
    // means the identity mapping.  row_offset is *d_row_offset when that is set.
    uint32_t rows_per_session = 0;
    uint32_t out_session_rows = 0;
    uint32_t row_offset = 0;
    const uint32_t* d_row_offset = nullptr;
    // Optional scratch of the few-row engine (gemm_skinny_workspace_bytes(); zeroed once, then left zeroed by every
    // launch; not to be shared by launches that may overlap): lets it divide K over several CTAs per tile.
    void* skinny_ws = nullptr;
    uint64_t skinny_ws_bytes = 0;
    // Split-K for the in-place residual form (f32, residual == out) with few rows: the k-blocks are divided over
    // `split_k` CTAs per tile (gemm_split_k() says how many), CTA s stores its partial sums (the first one with the
    // bias) into split_partials[(s * split_rows + row) * ldc + col] and neither reads nor writes `out`; the caller adds
    // them to the residual in a fixed order (launch_layernorm_fold).  split_rows: a multiple of 32, >= m.
    float* split_partials = nullptr;
    uint32_t split_k = 0;
    uint32_t split_rows = 0;
};

// How many ways launch_gemm_bf16 can divide the k-blocks of a plain f32 residual GEMM with `m` rows (0: do not).  The
// answer depends on n and k only (not on m, as long as m is small enough to split at all), so that the partial sums of
// an output element, and with them its bits, are the same however the rows are batched.
uint32_t gemm_split_k(const bf16* a, const bf16* bt, uint32_t m, uint32_t n, uint32_t k);

// strict f32: out = a[m,k] . b (+bias)(act)(+residual), reference operation order.
int launch_gemm_strict(const float* a, const float* b, void* out, uint32_t ldc, uint32_t m, uint32_t k,
                       uint32_t n, bool b_transposed, const GemmEpilogue& ep, cudaStream_t stream);

// bf16 operands, f32 accumulation.  `bt` is [n, k] K-major.  `mode` selects the
// epilogue family.
enum GemmMode : int {
    GEMM_PLAIN = 0,   // out[m, n] (f32 or bf16) = act(acc + bias) (+ residual)
    GEMM_QKV = 1,     // n = 3*d: columns [0,d) -> q (bf16), [d,2d) -> K cache rows, [2d,3d) -> V cache rows
    GEMM_SWIGLU = 2,  // n = 2*f packed in blocks of 16: out[m, f] bf16 = silu(gate) * up
    GEMM_ARGMAX = 3   // no matrix leaves the kernel: per (row, column tile) the greedy candidate (key, index)
};
// Paged K/V: a cache tensor is a pool [pages, page_rows, d] shared by all sessions; logical row r of session s lives
// in page table[s * pages_per_session + r / page_rows] at row r % page_rows.  table == nullptr: the contiguous
// [sessions, capacity, d] layout of the reference.
struct KvPaging {
    const uint32_t* table = nullptr;
    uint32_t page_rows = 0, pages_per_session = 0;
};
#ifdef __CUDACC__
// Physical row of logical row `r` of session `s` (contiguous layout: s * capacity + r).
__device__ __forceinline__ size_t kv_row(const KvPaging& pg, uint32_t s, uint32_t r, uint32_t capacity) {
    if (!pg.table) return (size_t)s * capacity + r;
    return (size_t)pg.table[(size_t)s * pg.pages_per_session + r / pg.page_rows] * pg.page_rows + r % pg.page_rows;
}
#endif

struct GemmQkvTargets {
    bf16* q = nullptr;        // [m, d]
    bf16* k_cache = nullptr;  // [sessions, capacity, d]
    bf16* v_cache = nullptr;
    uint32_t d = 0, chunk = 0, capacity = 0;
    const uint32_t* d_position = nullptr;  // device scalar: first new row
    uint32_t position = 0;                 // used when d_position == nullptr
    uint32_t position_stride = 0;          // 1: d_position is an array with one entry per session (ragged batches)
    KvPaging paging;                       // paged caches: k_cache / v_cache are page pools
};
int launch_gemm_bf16(const bf16* a, const bf16* bt, void* out, uint32_t ldc, uint32_t m, uint32_t n,
                     uint32_t k, GemmMode mode, const GemmEpilogue& ep, const GemmQkvTargets* qkv,
                     int* d_status, cudaStream_t stream);
extern int g_gemm_engine;  // 0 auto, 1 CUDA-core only, 2 tcgen05 only, 3 auto + the tcgen05 few-row engine for every eligible shape, 4 auto + the streaming engine for every eligible shape
// Few rows (m <= 64): weights on the M side of the MMA, optional split-K (gemm_skinny.cu).
uint64_t gemm_skinny_workspace_bytes();
bool gemm_skinny_eligible(const bf16* a, const bf16* bt, uint32_t m, uint32_t n, uint32_t k, const GemmEpilogue& ep);
int launch_gemm_skinny(const bf16* a, const bf16* bt, void* out, uint32_t ldc, uint32_t m, uint32_t n, uint32_t k,
                       const GemmEpilogue& ep, void* scratch, uint64_t scratch_bytes, int* d_status, cudaStream_t stream);
// At most 16 rows: the weights stream once through a cp.async ring, no split-K and no scratch (gemm_stream.cu).
bool gemm_stream_eligible(const bf16* a, const bf16* bt, uint32_t m, uint32_t n, uint32_t k, const GemmEpilogue& ep);
int launch_gemm_stream(const bf16* a, const bf16* bt, void* out, uint32_t ldc, uint32_t m, uint32_t n, uint32_t k,
                       const GemmEpilogue& ep, int* d_status, cudaStream_t stream);
// Greedy ids straight from the LM-head GEMM: ids[r] = last index of the maximum of row r of a . bt^T
// under IEEE totalOrder.  `candidates` is scratch for rows * ceil(n / 32) uint2 values.
uint64_t lm_head_argmax_scratch_bytes(uint32_t rows, uint32_t n);
int launch_lm_head_argmax(const bf16* a, const bf16* bt, uint32_t m, uint32_t n, uint32_t k, void* candidates,
                          uint32_t* ids, int* d_status, cudaStream_t stream);

int launch_embedding(const void* tok, const void* pos, const uint32_t* ids, float* out, uint32_t rows,
                     uint32_t chunk, uint32_t position0, const uint32_t* d_position, uint32_t vocab,
                     uint32_t width, int dtype, int* d_status, cudaStream_t stream, uint32_t position_stride = 0);
int launch_layernorm(const float* x, const float* w, const float* b, void* out, uint32_t rows,
                     uint32_t width, float eps, int out_dtype, bool strict, cudaStream_t stream);
// Gathers row (s * chunk + chunk - 1) of x for every session s into out[s, :] (f32).
int launch_gather_last_rows(const float* x, float* out, uint32_t sessions, uint32_t chunk, uint32_t width,
                            cudaStream_t stream);
int launch_argmax(const float* logits, uint32_t* out, uint32_t rows, uint32_t vocab, uint32_t row_stride,
                  cudaStream_t stream);
// Next-token sampling (temperature, top-k, Philox per (session, step)); see sampler.cu for the exact rule.  The step
// of row r is (d_step[r * step_stride] if d_step is given, else 0) + step_add; row r belongs to session first_session + r.
int launch_sample_top_k(const float* logits, uint32_t* out, uint32_t rows, uint32_t vocab, uint32_t row_stride,
                        float temperature, uint32_t top_k, uint64_t seed, const uint32_t* d_step, uint32_t step_stride,
                        uint32_t step_add, uint32_t first_session, cudaStream_t stream);
int launch_swiglu(const bf16* gate, const bf16* up, bf16* out, uint64_t elems, cudaStream_t stream);
int launch_transpose_bf16(const bf16* in, bf16* out, uint32_t k, uint32_t n, cudaStream_t stream);
int launch_f32_to_bf16(const float* in, bf16* out, uint64_t elems, cudaStream_t stream);
int launch_bf16_to_f32(const bf16* in, float* out, uint64_t elems, cudaStream_t stream);
// in [k, n] f32 row-major -> out [n, k] bf16 (round to nearest even)
int launch_transpose_f32_to_bf16(const float* in, bf16* out, uint32_t k, uint32_t n, cudaStream_t stream);
int launch_transpose_f32_to_bf16_mapped(const float* in, bf16* out, uint32_t k, uint32_t n, uint32_t row0,
                                        uint32_t block, uint32_t block_stride, cudaStream_t stream);
// h[row] += partials[0][row] + partials[1][row] + ... (in that order; partial s of row r at (s * split_rows + r) * width),
// written back, then out = LayerNorm(h) as bf16: the other half of a split-K residual GEMM (GemmEpilogue::split_k).
bool layernorm_fold_supported(uint32_t width);
int launch_layernorm_fold(float* h, const float* partials, uint32_t split_k, uint32_t split_rows, const float* w, const float* b,
                          void* out, uint32_t rows, uint32_t width, float eps, cudaStream_t stream);
int launch_layernorm_strict(const float* x, const float* w, const float* b, float* out, uint32_t rows,
                            uint32_t width, float eps, cudaStream_t stream);
int launch_swiglu_strict(const float* gate, const float* up, float* out, size_t n, cudaStream_t stream);
int launch_decode_attention_ex(const bf16* q, const bf16* k_cache, const bf16* v_cache, const uint32_t* d_lengths,
                               const uint32_t* d_position, uint32_t extra, bf16* out, void* workspace,
                               uint64_t workspace_bytes, uint32_t batch, uint32_t capacity, uint32_t heads,
                               uint32_t head_dim, bool plan, int* d_status, cudaStream_t stream, bool lean = false,
                               const KvPaging* paging = nullptr);
int launch_pack_gate_up(const bf16* wg, const bf16* wu, const float* bg, const float* bu, bf16* w_out,
                        float* b_out, uint32_t d, uint32_t f, cudaStream_t stream);
int launch_fill_u32(uint32_t* p, uint32_t value, uint32_t n, cudaStream_t stream);
int launch_add_u32(uint32_t* p, uint32_t delta, cudaStream_t stream);

// Everything between two attention scans of a single-token step at small batch (<= 64 sessions) as one persistent
// kernel with grid-wide barriers (decode_tail.cu): [output projection + residual] -> [LayerNorm, gate/up, SwiGLU] ->
// [down projection + residual] -> [next layer's LayerNorm, QKV projection, K/V cache rows].  run_o / run_ffn / run_qkv
// select the parts; weights are the session's K-major bf16 matrices (gate/up packed in blocks of 16).
struct DecodeTailArgs {
    bool run_o = false, run_ffn = false, run_qkv = false;
    uint32_t rows = 0, d = 0, f = 0;
    float eps = 0.0f;
    float* h = nullptr;
    const bf16* att = nullptr;
    bf16* ff = nullptr;
    bf16* q = nullptr;
    const bf16* wo = nullptr; const float* bo = nullptr;
    const float* ln2w = nullptr; const float* ln2b = nullptr;
    const bf16* wgu = nullptr; const float* bgu = nullptr;
    const bf16* wdown = nullptr; const float* bdown = nullptr;
    const float* ln1w = nullptr; const float* ln1b = nullptr;
    const bf16* wqkv = nullptr; const float* bqkv = nullptr;
    bf16* k_cache = nullptr; bf16* v_cache = nullptr;
    uint32_t capacity = 0;
    const uint32_t* d_position = nullptr; uint32_t position = 0, position_stride = 0;
    uint32_t first_session = 0;
    const KvPaging* paging = nullptr;
    void* workspace = nullptr;     // decode_tail_workspace_bytes(), zeroed once; every completed launch leaves it zeroed
    int* d_status = nullptr;
};
uint64_t decode_tail_workspace_bytes();
bool decode_tail_supported(uint32_t rows, uint32_t d, uint32_t f);
int launch_decode_tail(const DecodeTailArgs& args, cudaStream_t stream);

// Strict f32 attention in the reference's order over a cache that already holds
// the new rows: q [sessions*chunk, d] f32; caches f32 or bf16 [sessions, capacity, d].
int launch_attention_strict(const float* q, const void* k_cache, const void* v_cache, float* out,
                            uint32_t sessions, uint32_t chunk, uint32_t position,
                            const uint32_t* d_position, uint32_t capacity, uint32_t heads,
                            uint32_t head_dim, int kv_dtype, int round_bf16, cudaStream_t stream);

// bf16 attention for any head_dim and chunk (online softmax, one warp per query/head).
int launch_attention_generic(const bf16* q, const bf16* k_cache, const bf16* v_cache, bf16* out,
                             uint32_t sessions, uint32_t chunk, uint32_t position,
                             const uint32_t* d_position, uint32_t capacity, uint32_t heads,
                             uint32_t head_dim, cudaStream_t stream, const KvPaging* paging = nullptr);

// Split-KV decode attention (one query per session/head) with per-session lengths.
uint64_t decode_attention_workspace_bytes(uint32_t batch, uint32_t capacity, uint32_t heads,
                                          uint32_t head_dim);
bool decode_attention_supported(uint32_t heads, uint32_t head_dim);
int launch_decode_attention(const bf16* q, const bf16* k_cache, const bf16* v_cache,
                            const uint32_t* d_lengths, bf16* out, void* workspace, uint64_t workspace_bytes,
                            uint32_t batch, uint32_t capacity, uint32_t heads, uint32_t head_dim,
                            int* d_status, cudaStream_t stream);

// Tiled causal prefill attention over the cache (tensor cores).  The tcgen05 kernel runs when the
// position is known on the host (d_position == nullptr), the head width is 64 and the chunk has at
// least 32 rows; otherwise the warp-level mma.sync kernel does.  d_status (may be null) receives
// DEV_TIMEOUT if a bounded wait of the tcgen05 kernel gives up.
bool prefill_attention_supported(uint32_t head_dim);
int launch_prefill_attention(const bf16* q, const bf16* k_cache, const bf16* v_cache, bf16* out,
                             uint32_t sessions, uint32_t chunk, uint32_t position,
                             const uint32_t* d_position, uint32_t capacity, uint32_t heads,
                             uint32_t head_dim, int* d_status, cudaStream_t stream);
bool prefill_attention_tc_eligible(uint32_t sessions, uint32_t chunk, uint32_t position, const uint32_t* d_position,
                                   uint32_t capacity, uint32_t heads, uint32_t head_dim);
int launch_prefill_attention_tc(const bf16* q, const bf16* k_cache, const bf16* v_cache, bf16* out, uint32_t sessions,
                                uint32_t chunk, uint32_t position, uint32_t capacity, uint32_t heads, int* d_status,
                                cudaStream_t stream);

// ---- device helpers ----------------------------------------------------------
#ifdef __CUDACC__

// Sign-folded bit pattern: integer order of the keys is IEEE totalOrder of the floats.
__device__ __forceinline__ int total_order_key(float x) {
    int bits = __float_as_int(x);
    return bits ^ (int)(((unsigned)(bits >> 31)) >> 1);
}
// First statement of every kernel that may be launched with programmatic stream serialization.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel in the stream be scheduled (it still waits for this one's completion in its own pdl_wait).
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t hi16) { return __uint_as_float(hi16 << 16); }
// Two packed bf16 (low half = element 0) -> two f32.
__device__ __forceinline__ float2 bf16x2_to_f32(uint32_t v) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
// Round to nearest even to bf16 and widen again; NaN stays a quiet NaN.
__device__ __forceinline__ float round_to_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// nn::sigmoid / nn::silu / nn::gelu (src/nn/activations.rs:5-47) for the fast
// path: same formulas, f32, with the hardware exponential.
__device__ __forceinline__ float fast_sigmoid(float x) {
    float z = __expf(-fabsf(x));
    float den = z + 1.0f;
    return (x < 0.0f) ? __fdividef(z, den) : __fdividef(1.0f, den);
}
__device__ __forceinline__ float fast_silu(float x) { return x * fast_sigmoid(x); }
__device__ __forceinline__ float fast_gelu(float x) {
    float mag = fabsf(x) * 0.70710678118654752440f;
    float t = __fdividef(1.0f, fmaf(mag, 0.3275911f, 1.0f));
    float poly = ((((t * 1.0614054f - 1.4531521f) * t + 1.4214138f) * t - 0.28449672f) * t + 0.2548296f) * t;
    float tail = poly * __expf(-mag * mag) * 0.5f;
    float cdf = (x < 0.0f) ? tail : 1.0f - tail;
    return x * cdf;
}
__device__ __forceinline__ float apply_activation(float x, int act) {
    if (act == ACT_RELU) return fmaxf(x, 0.0f);
    if (act == ACT_GELU) return fast_gelu(x);
    return x;
}

#endif  // __CUDACC__

}  // namespace tb
