/*
 * tnsr_b200.h -- C ABI of the B200-native replacement for tnsr's cached GPT
 * inference backend.
 *
 * The library takes the place of `DecoderBackend::Cuda(Box<cuda::CudaDecoder>)`
 * (tnsr src/nn/kv_cache.rs:60-64): everything below `GptDecoder::{new, reset,
 * decode}` on the GPU side.  Session guards that the reference keeps in
 * `GptDecoder` itself (failed flag, rectangular chunk, parameter revisions,
 * src/nn/kv_cache.rs:261-389) stay in the caller's wrapper; this ABI is what a
 * Rust `extern "C"` block, a ctypes module or C++ code binds.
 *
 * Conventions
 *  - plain pointers and sizes only; no exceptions, no aborts, no device traps;
 *  - every function returns TNSR_B200_OK (0) or a negative tnsr_b200_status;
 *    `tnsr_b200_last_error` gives the message of the last failure;
 *  - a handle is used by one host thread at a time (every reference method takes
 *    `&mut self`); distinct handles are independent, one per GPU if desired;
 *  - the library owns all device memory of a session; host buffers belong to
 *    the caller and are not retained after a call returns;
 *  - `stream` arguments of the operator entry points are `cudaStream_t` values
 *    passed as `void*` (NULL = the legacy default stream).
 */
#ifndef TNSR_B200_H
#define TNSR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define TNSR_B200_API
#else
#define TNSR_B200_API __attribute__((visibility("default")))
#endif

typedef enum tnsr_b200_status {
    TNSR_B200_OK = 0,
    TNSR_B200_ERR_INVALID_ARGUMENT = -1,
    TNSR_B200_ERR_CUDA = -2,          /* a CUDA runtime/driver call failed            */
    TNSR_B200_ERR_OUT_OF_MEMORY = -3,
    TNSR_B200_ERR_CAPACITY = -4,      /* "decoder context capacity exceeded"          */
    TNSR_B200_ERR_TOKEN_RANGE = -5,   /* "decoder token is outside the vocabulary"    */
    TNSR_B200_ERR_FAILED_STATE = -6,  /* a previous execution failed; reset first     */
    TNSR_B200_ERR_TIMEOUT = -7,       /* a bounded device-side wait gave up           */
    TNSR_B200_ERR_UNSUPPORTED = -8,   /* shape/dtype outside what the kernels cover   */
    TNSR_B200_ERR_NO_DEVICE = -9      /* no sm_100 device ("initialize CUDA decoder") */
} tnsr_b200_status;

/* FFN activation.  RELU is the only block `nn::Gpt` itself builds
 * (src/nn/kv_cache/graph.rs:133-138); GELU applies `nn::gelu`
 * (src/nn/activations.rs:29-47); SWIGLU is `down(silu(gate(x)) * up(x))`
 * (examples/forty_five/mod.rs:398-407, src/nn/activations.rs:5-20). */
typedef enum tnsr_b200_activation {
    TNSR_B200_ACT_RELU = 0,
    TNSR_B200_ACT_GELU = 1,
    TNSR_B200_ACT_SWIGLU = 2
} tnsr_b200_activation;

typedef enum tnsr_b200_dtype {
    TNSR_B200_F32 = 0,
    TNSR_B200_BF16 = 1
} tnsr_b200_dtype;

/* What `decode` hands back for a chunk of `chunk` new tokens per session. */
typedef enum tnsr_b200_logits_mode {
    TNSR_B200_LOGITS_ALL = 0,  /* [batch, chunk, vocab] f32 -- the reference contract */
    TNSR_B200_LOGITS_LAST = 1, /* [batch, vocab] f32 of the last position only        */
    TNSR_B200_LOGITS_NONE = 2  /* no logits leave the device, argmax ids only         */
} tnsr_b200_logits_mode;

/* `GptPrefillMode` (src/nn/kv_cache.rs:28-34).  AUTO lets multi-token chunks run
 * on the tiled tensor-core attention kernels; SCALAR keeps them on the
 * non-tiled scan (one warp per query and head, keys in order), which the
 * reference describes as "useful as a precision-matched reference".  It only
 * matters with bf16 weights: the strict f32 path has a single attention kernel. */
typedef enum tnsr_b200_prefill_mode {
    TNSR_B200_PREFILL_AUTO = 0,
    TNSR_B200_PREFILL_SCALAR = 1
} tnsr_b200_prefill_mode;

/* Session configuration: the seven `GptConfig` fields (src/nn.rs:543-552),
 * the `GptDecoder::new` arguments (src/nn/kv_cache.rs:161-167) and the
 * precision choices.
 *
 * weight_dtype = F32 keeps the reference's arithmetic: strict f32 projections
 * in increasing-K order with separately rounded multiply and add -- what
 * `MatMulPrecision::StrictF32` does in src/nn/kv_cache/cuda.rs:480-486.
 * kv_dtype = BF16 with F32 weights is `GptAttentionPrecision::Bf16`
 * (src/nn/kv_cache.rs:21-26).  weight_dtype = BF16 is the tensor-core path:
 * bf16 operands, f32 accumulation, bf16 K/V (kv_dtype must be BF16). */
typedef struct tnsr_b200_config {
    uint32_t vocab_size;
    uint32_t max_sequence_length;
    uint32_t embed_dim;
    uint32_t num_heads;
    uint32_t feed_forward_dim;
    uint32_t num_layers;
    float layer_norm_epsilon;
    uint32_t activation;   /* tnsr_b200_activation  */
    uint32_t weight_dtype; /* tnsr_b200_dtype       */
    uint32_t kv_dtype;     /* tnsr_b200_dtype       */
    uint32_t batch;        /* sessions held by this handle, all advancing together */
    uint32_t capacity;     /* K/V rows per session, <= max_sequence_length         */
    int32_t device;        /* CUDA ordinal (the reference always uses 0)           */
    uint32_t logits_mode;  /* tnsr_b200_logits_mode */
    uint32_t prefill_mode; /* tnsr_b200_prefill_mode */
    /* How many independent session ranges a single-token step of the bf16 path
     * is divided into, each on its own stream so that one range's short
     * projection kernels run while another range streams its K/V rows (no
     * reference counterpart; results differ from the undivided step only by
     * rounding).  0 = automatic (from 192 sessions up ranges of about 128
     * sessions, two to four of them; else 1), 1 = never divide, 2..4 = that
     * many parts. */
    uint32_t step_parts;
    /* Paged K/V (no reference counterpart; the reference's cache is one
     * [batch, capacity, width] slab per tensor and its documentation lists ragged
     * batches as future work, docs/kv-cache.md:94-95).  kv_page_rows > 0 stores
     * every cache tensor as a pool of kv_pool_pages pages of kv_page_rows rows
     * shared by all sessions of the handle; a session gets a page when one of
     * its rows is first written and gives its pages back through
     * tnsr_b200_decoder_release or reset, so memory follows the live tokens
     * instead of batch * capacity.  Requirements: bf16 weights, kv_page_rows a
     * multiple of 16 that divides capacity.  kv_pool_pages = 0 sizes the pool
     * for the worst case (batch * capacity / kv_page_rows).  A step that needs a
     * page when none is free fails with TNSR_B200_ERR_CAPACITY and changes
     * nothing.  Multi-token chunks run on the non-tiled attention scan in this
     * mode. */
    uint32_t kv_page_rows;
    uint32_t kv_pool_pages;
    /* Single-token steps of at most 32 sessions (bf16 weights, SwiGLU, width <=
     * 1024): 0 = everything between two attention scans runs as one persistent
     * kernel with grid-wide barriers (the default), 1 = one kernel per operator
     * as at larger batches.  No reference counterpart; the two differ by rounding
     * only. */
    uint32_t small_batch_mode;
} tnsr_b200_config;

typedef struct tnsr_b200_decoder tnsr_b200_decoder;

/* ---- library ------------------------------------------------------------ */

TNSR_B200_API const char* tnsr_b200_version(void);
/* Number of CUDA devices, or a negative status.  Never initialises a context. */
TNSR_B200_API int tnsr_b200_device_count(void);
/* Message of the last failure on `dec`, or (dec == NULL) of the last failed
 * call on this thread that had no handle yet.  Never NULL. */
TNSR_B200_API const char* tnsr_b200_last_error(const tnsr_b200_decoder* dec);
/* Total kernels this library has launched in this process (all handles and
 * operator calls); benchmarks report the difference across a timed region. */
TNSR_B200_API uint64_t tnsr_b200_kernel_launches(void);
/* GEMM engine of the bf16 path: 0 = tcgen05/TMEM kernel where the shape
 * allows it, else the CUDA-core kernel (default); 1 = always the CUDA-core
 * kernel; 2 = tcgen05 only (unsupported shapes fail); 3 = as 0, but products
 * of at most 64 rows always take the tcgen05 few-row engine with split-K (by
 * default only those shapes do for which it is the faster one); 4 = as 0, but
 * products of at most 16 rows always take the weight-streaming engine (by
 * default from 4 M weight elements up).  Process-wide.  Engine 1
 * also keeps prefill attention off tcgen05 (the warp-level mma.sync kernel
 * runs), which is how tests compare the two. */
TNSR_B200_API int tnsr_b200_set_gemm_engine(int engine);
/* Every wait inside a kernel (a producer/consumer barrier between the copy, MMA
 * and epilogue roles) is bounded: when it lasts longer than this limit the
 * kernel stops waiting, lets copies in flight land, releases what it holds and
 * records TNSR_B200_ERR_TIMEOUT in the caller's status word; a session then
 * enters the failed state until reset, like the `failed` flag of
 * src/nn/kv_cache.rs:262-265,331,387.  Default 2 s; accepted range 1 us .. 60 s.
 * Process-wide; it applies to kernels launched (or captured) afterwards. */
TNSR_B200_API int tnsr_b200_set_wait_limit_ns(uint64_t ns);
/* Test hook (no reference counterpart): the next tcgen05 GEMM launched from
 * the calling thread leaves out the operand copies of k-block `k_block` of its
 * first tile.  Nothing faults: the MMA role's bounded wait for that stage runs
 * out after the wait limit and the kernel returns through its time-out path,
 * which is the only way to exercise that path on healthy hardware. */
TNSR_B200_API int tnsr_b200_test_lose_gemm_stage(uint32_t k_block);

/* ---- session: replaces cuda::CudaDecoder -------------------------------- */

/* CudaDecoder::new (src/nn/kv_cache/cuda.rs:73-123): binds the device, makes a
 * private stream, allocates zeroed K/V [batch, capacity, embed_dim] for each of
 * the 2*num_layers cache tensors (src/nn/kv_cache.rs:188-195) and zeroed
 * parameters.  Size arithmetic is overflow-checked like src/nn/kv_cache.rs:173-187. */
TNSR_B200_API int tnsr_b200_decoder_create(const tnsr_b200_config* config, tnsr_b200_decoder** out);
/* Drop (src/nn/kv_cache/cuda.rs:56-62): waits for queued work, then frees. */
TNSR_B200_API void tnsr_b200_decoder_destroy(tnsr_b200_decoder* dec);

/* Parameters are addressed in `model_parameters` order
 * (src/nn/kv_cache.rs:392-421): token table, position table, final norm
 * weight, final norm bias, then per layer q_w, q_b, k_w, k_b, v_w, v_b, o_w,
 * o_b, ln1_w, ln1_b, ln2_w, ln2_b, ff_in_w, ff_in_b, ff_out_w, ff_out_b
 * (SWIGLU: ... ln2_b, gate_w, gate_b, up_w, up_b, down_w, down_b).  Matrices
 * are [in, out] row-major f32 exactly as `Parameter<f32>` holds them. */
TNSR_B200_API uint32_t tnsr_b200_decoder_param_count(const tnsr_b200_decoder* dec);
TNSR_B200_API uint64_t tnsr_b200_decoder_param_elems(const tnsr_b200_decoder* dec, uint32_t index);
/* CudaDecoder::refresh for one tensor (src/nn/kv_cache/cuda.rs:125-141): copies
 * host f32 values to the device (rounding to bf16 once, here, when
 * weight_dtype = BF16).  The caller decides when a tensor's revision changed. */
TNSR_B200_API int tnsr_b200_decoder_upload(tnsr_b200_decoder* dec, uint32_t index, const float* host,
                                           uint64_t elems);

/* CudaDecoder::reset (src/nn/kv_cache/cuda.rs:143-156): zero K/V, synchronise,
 * clear a failed state. */
TNSR_B200_API int tnsr_b200_decoder_reset(tnsr_b200_decoder* dec);

/* CudaDecoder::decode (src/nn/kv_cache/cuda.rs:159-218).  `tokens` is the
 * row-major [batch, chunk] id block, `position` the number of rows already
 * cached (`GptDecoder::length`).  Synchronous: on return the new K/V rows are
 * appended at `position` and the outputs are in host memory.
 *   logits_out: LOGITS_ALL [batch, chunk, vocab] f32, LOGITS_LAST [batch, vocab],
 *               must be NULL for LOGITS_NONE;
 *   argmax_out: optional [batch] greedy ids of the last position, chosen as
 *               `max_by(total_cmp)` does (src/nn/kv_cache.rs:148-153): the last
 *               index holding the maximum.
 * Invalid input (chunk 0, overflow, id >= vocab) is rejected before any device
 * work and leaves the session untouched.  A device failure puts the handle in
 * the failed state until reset. */
TNSR_B200_API int tnsr_b200_decoder_decode(tnsr_b200_decoder* dec, const uint32_t* tokens,
                                           uint32_t chunk, uint32_t position, float* logits_out,
                                           uint32_t* argmax_out);

/* Ragged single-token step (no reference counterpart: the reference's sessions
 * advance together; its documentation lists ragged batches as future work,
 * docs/kv-cache.md:94-95).  Session b consumes tokens[b] at its own position
 * positions[b] (< capacity): its K/V row is written there and it attends rows
 * 0 .. positions[b].  The caller keeps the per-session lengths; rows past a
 * session's position are never read.  bf16 weights only (weight_dtype BF16) and
 * head widths the split-KV attention kernel covers (32, 64, 128).  logits_out:
 * [batch, vocab] f32 or NULL; argmax_out: [batch] or NULL.  Synchronous like
 * tnsr_b200_decoder_decode. */
TNSR_B200_API int tnsr_b200_decoder_decode_ragged(tnsr_b200_decoder* dec, const uint32_t* tokens,
                                                  const uint32_t* positions, float* logits_out,
                                                  uint32_t* argmax_out);

/* Device-resident form of the same step for serving loops: ids are read from
 * and greedy ids written to device memory, nothing is copied and nothing is
 * synchronised; work is queued on the session's stream.  Ids are validated on
 * the device (an id >= vocab raises TNSR_B200_ERR_TOKEN_RANGE at the next
 * `synchronize`).  `d_argmax_out` may alias `d_tokens` when chunk == 1, which
 * turns repeated calls into a greedy decode loop. */
TNSR_B200_API int tnsr_b200_decoder_decode_device(tnsr_b200_decoder* dec, const uint32_t* d_tokens,
                                                  uint32_t chunk, uint32_t position,
                                                  uint32_t* d_argmax_out);
/* Replaces the greedy pick of `argmax_out` / `d_argmax_out` by
 * tnsr_b200_sample_top_k on the last position's logits: session b at a step
 * that ends at position p (its new token will sit at p) draws with counter
 * (p, 0, b, 0), so a run is reproducible from (seed, ids) whatever the chunking.
 * temperature <= 0 switches back to greedy.  Logits are materialised on the
 * device while a sampler is set, also with LOGITS_NONE. */
TNSR_B200_API int tnsr_b200_decoder_set_sampler(tnsr_b200_decoder* dec, float temperature, uint32_t top_k,
                                                uint64_t seed);
/* Paged handles only: returns the pages of session `session` to the pool (its
 * rows are gone; the caller restarts it at position 0).  Waits for queued work. */
TNSR_B200_API int tnsr_b200_decoder_release(tnsr_b200_decoder* dec, uint32_t session);
/* Paged handles only: pages currently not assigned to any session. */
TNSR_B200_API uint32_t tnsr_b200_decoder_free_pages(const tnsr_b200_decoder* dec);
/* Waits for the session's stream and reports any deferred device-side error. */
TNSR_B200_API int tnsr_b200_decoder_synchronize(tnsr_b200_decoder* dec);
/* The session's private stream as a cudaStream_t (for event timing). */
TNSR_B200_API void* tnsr_b200_decoder_stream(tnsr_b200_decoder* dec);

/* Cache tensor `index` (2*layer = keys, 2*layer+1 = values) as f32
 * [batch, capacity, embed_dim]; the counterpart of reading the reference's
 * `cache: Vec<Parameter<f32>>` (src/nn/kv_cache.rs:76).  `write` exists so
 * tests can poison unused slots the way src/nn/kv_cache/cuda/tests.rs:98-107 does. */
TNSR_B200_API int tnsr_b200_decoder_read_cache(tnsr_b200_decoder* dec, uint32_t index, float* host_out);
TNSR_B200_API int tnsr_b200_decoder_write_cache(tnsr_b200_decoder* dec, uint32_t index,
                                                const float* host_in);

/* Measurement aid (no reference counterpart; the reference times kernels from
 * outside with CUDA events, src/ptx/linear/mod.rs:425-437).  While enabled, the
 * session brackets every launch of its split-KV decode-attention kernel with a
 * pair of CUDA events on its stream.  `attention_profile` waits for the stream,
 * returns the summed device time in milliseconds and the number of launches
 * since the last call, and clears the record. */
TNSR_B200_API int tnsr_b200_decoder_profile_attention(tnsr_b200_decoder* dec, int enable);
TNSR_B200_API int tnsr_b200_decoder_attention_profile(tnsr_b200_decoder* dec, double* total_ms,
                                                      uint64_t* launches);

/* ---- operators on caller-owned device memory ---------------------------- */
/* The kernels of the session, exposed one by one for operator-level parity
 * tests and roofline measurement.  All pointers are device pointers. */

/* Embedding gather-add: out[r, :] = token_table[ids[r], :] + position_table[position0 + r % chunk, :]
 * (src/nn/kv_cache/graph.rs:30-41, src/lib.rs:868-909).  dtype is the tables'
 * element type; out is f32.  Ids >= vocab set *d_status (if non-NULL) to
 * TNSR_B200_ERR_TOKEN_RANGE and produce zeros. */
TNSR_B200_API int tnsr_b200_embedding(const void* token_table, const void* position_table,
                                      const uint32_t* ids, float* out, uint32_t rows, uint32_t chunk,
                                      uint32_t position0, uint32_t vocab, uint32_t width, int dtype,
                                      int* d_status, void* stream);

/* LayerNorm over the last axis (src/nn.rs:165-213).  strict != 0 reproduces the
 * reference's operation order (sequential mean of x/n, exp(ln(var+eps)*-0.5));
 * strict == 0 is the vectorised warp-shuffle kernel.  out_dtype selects f32 or
 * bf16 output. */
TNSR_B200_API int tnsr_b200_layernorm(const float* x, const float* weight, const float* bias, void* out,
                                      uint32_t rows, uint32_t width, float epsilon, int out_dtype,
                                      int strict, void* stream);

/* Strict f32 matmul, the reference's CPU order: out[i,j] = sum_p a[i,p]*b[p,j]
 * from a zero start in increasing p with a rounded product then a rounded add
 * (src/lib.rs:1202-1208; the GPU test that pins it is
 * tests/ptx_transformer.rs:1410-1465).  b is [k, n] row-major, or [n, k] when
 * b_transposed != 0.  bias (optional, [n]) is added after the sum. */
TNSR_B200_API int tnsr_b200_gemm_f32_strict(const float* a, const float* b, const float* bias,
                                            float* out, uint32_t m, uint32_t k, uint32_t n,
                                            int b_transposed, void* stream);

/* bf16 GEMM, f32 accumulation: out = act(a[m,k] . b^T + bias) (+ residual).
 * a is [m, k] row-major bf16; bt is the weight stored [n, k] row-major bf16
 * ("K-major": what a [k, n] `Parameter` becomes after the one-time transpose
 * at upload).  bias f32 [n] or NULL; residual f32 [m, n] or NULL (only with f32
 * output); activation: -1 none, else tnsr_b200_activation RELU/GELU;
 * out_dtype f32 or bf16.  This is "the tiled matmul path"
 * (src/tile/matmul_schedule.rs:487-646, src/ptx/graph/matmul.rs:4-129). */
TNSR_B200_API int tnsr_b200_gemm_bf16(const void* a, const void* bt, const float* bias,
                                      const float* residual, void* out, uint32_t m, uint32_t n,
                                      uint32_t k, int activation, int out_dtype, void* stream);
/* The same product with scratch lent by the caller (no reference counterpart).
 * It matters for m <= 64, where the weights are streamed once with the
 * operands of the MMA swapped: with scratch the K range of every 128-column
 * tile is divided over several CTAs so that all SMs pull on HBM, and the CTA
 * that finishes last adds the partial tiles in a fixed order (results do not
 * depend on timing).  `workspace`: tnsr_b200_gemm_workspace() bytes, 16-byte
 * aligned, zeroed once before the first use (every launch that completes leaves
 * it zeroed; zero it again if a launch was cut short by a device error);
 * launches that may overlap on the GPU must not share it. */
TNSR_B200_API uint64_t tnsr_b200_gemm_workspace(void);
TNSR_B200_API int tnsr_b200_gemm_bf16_ws(const void* a, const void* bt, const float* bias,
                                         const float* residual, void* out, uint32_t m, uint32_t n,
                                         uint32_t k, int activation, int out_dtype,
                                         void* workspace, uint64_t workspace_bytes, void* stream);
/* Transposes a [k, n] row-major bf16 matrix into the [n, k] layout above. */
TNSR_B200_API int tnsr_b200_transpose_bf16(const void* in, void* out, uint32_t k, uint32_t n,
                                           void* stream);

/* Elementwise SwiGLU, y = silu(gate) * up (src/tile/swiglu.rs:35-121,
 * src/nn/activations.rs:5-20), bf16 in and out, f32 arithmetic. */
TNSR_B200_API int tnsr_b200_swiglu(const void* gate, const void* up, void* out, uint64_t elems,
                                   void* stream);

/* Fused SwiGLU MLP block: out = (silu(x.Wg + bg) * (x.Wu + bu)) . Wd + bd
 * (examples/forty_five/mod.rs:398-407).  x [rows, d] bf16; w_gate_up_t is the
 * packed [2f, d] matrix made by tnsr_b200_pack_gate_up; w_down_t [d, f];
 * b_gate_up packed f32 [2f] or NULL; b_down f32 [d] or NULL; hidden is a
 * caller-provided [rows, f] bf16 scratch; out [rows, d] bf16. */
TNSR_B200_API int tnsr_b200_swiglu_mlp(const void* x, const void* w_gate_up_t, const float* b_gate_up,
                                       const void* w_down_t, const float* b_down, void* hidden,
                                       void* out, uint32_t rows, uint32_t d, uint32_t f, void* stream);
/* Packs gate and up weights ([d, f] row-major bf16 each) into one [2f, d]
 * K-major matrix whose rows alternate in blocks of 16 (16 gate rows, 16 up
 * rows, ...), so one accumulator tile holds matching (gate, up) columns;
 * biases (f32 [f], optional) are packed the same way into b_out [2f]. */
TNSR_B200_API int tnsr_b200_pack_gate_up(const void* w_gate, const void* w_up, const float* b_gate,
                                         const float* b_up, void* w_out, float* b_out, uint32_t d,
                                         uint32_t f, void* stream);

/* KV-cache decode attention over the live prefix only, one query per session
 * and head (the job of AttentionScan/MergeScan, src/nn/kv_cache/attention.rs,
 * src/tile/normalized_schedule.rs:173-353).  q, out: [batch, heads*head_dim]
 * bf16; k_cache, v_cache: [batch, capacity, heads*head_dim] bf16; lengths[b]
 * = live keys of session b including its newest row (1..capacity; 0 gives a
 * zero output row).  workspace: device scratch of at least
 * tnsr_b200_decode_attention_workspace(...) bytes (a smaller one is rejected
 * before anything is written); bytes 64..67 of it hold a status word once the
 * stream has passed the call: 0 = ok, 2 = a bounded wait inside the kernel gave
 * up, 3 = a length beyond the capacity was clamped.  The call clears the word
 * and the kernels re-arm their own counters at every launch, so a workspace can
 * be reused after an error status without zeroing it again.  Scores are scaled
 * by 1/sqrt(head_dim); softmax statistics and accumulation are f32. */
TNSR_B200_API uint64_t tnsr_b200_decode_attention_workspace(uint32_t batch, uint32_t capacity,
                                                            uint32_t heads, uint32_t head_dim);
TNSR_B200_API int tnsr_b200_decode_attention(const void* q, const void* k_cache, const void* v_cache,
                                             const uint32_t* lengths, void* out, void* workspace,
                                             uint64_t workspace_bytes, uint32_t batch,
                                             uint32_t capacity, uint32_t heads, uint32_t head_dim,
                                             void* stream);

/* The same decode attention for callers that cannot allocate device memory at
 * call time and so have no workspace to pass: processes that budget the whole
 * GPU at start-up, or latency-bound loops where cudaMalloc (a device-wide
 * synchronisation that may fail under fragmentation) is not allowed.  It has no
 * counterpart in the reference.  The scratch is a fixed array of
 * TNSR_B200_STATIC_SCRATCH_BYTES inside the library, present on every GPU that
 * loads it until the process exits; the call allocates and frees nothing.
 * Limit: tnsr_b200_decode_attention_workspace(batch, capacity, heads,
 * head_dim) must not exceed the array (it grows with batch * heads * head_dim,
 * not with capacity), otherwise TNSR_B200_ERR_UNSUPPORTED.  All calls
 * share the array, so calls that overlap on the GPU (different streams or host
 * threads) race: keep them on one stream.  The first call on each device looks
 * up the array's device address once and keeps it for the life of the process;
 * make that first call before any stream capture, and do not use this entry
 * point after cudaDeviceReset or under a context other than the device's primary
 * one (the remembered address belongs to the context that made the first call).
 * d_status (optional device int) receives 0 or a device-side error
 * code when the stream reaches the end of the call.  Arguments otherwise as
 * tnsr_b200_decode_attention. */
#define TNSR_B200_STATIC_SCRATCH_BYTES (32ull << 20)
TNSR_B200_API int tnsr_b200_decode_attention_static(const void* q, const void* k_cache, const void* v_cache,
                                                    const uint32_t* lengths, void* out, uint32_t batch,
                                                    uint32_t capacity, uint32_t heads, uint32_t head_dim,
                                                    int* d_status, void* stream);

/* Causal attention of `chunk` new queries per session over `position + chunk`
 * cached keys (the new rows are already in the cache), the job of the tiled
 * prefill (src/nn/kv_cache/prefill.rs:170-607).  q, out: [batch, chunk, width]
 * bf16; caches as above.  Head width 64 with at least 32 new rows runs on the
 * tcgen05 kernel (scores and outputs in TMEM); other shapes on the warp-level
 * tensor-core kernel (head width 64) or the generic one. */
TNSR_B200_API int tnsr_b200_prefill_attention(const void* q, const void* k_cache, const void* v_cache,
                                              void* out, uint32_t batch, uint32_t chunk,
                                              uint32_t position, uint32_t capacity, uint32_t heads,
                                              uint32_t head_dim, void* stream);

/* ---- the forty_five token encoder's extra operators ---------------------- */
/* tnsr's second model on this operator set is the token encoder of its
 * forty_five example (examples/forty_five/mod.rs:329-407): a bidirectional
 * pre-norm transformer with SwiGLU blocks over short token rows.  Its
 * projections, LayerNorms and SwiGLU are the strict f32 operators above; these
 * are the two operators it adds, plus two elementwise helpers.  All f32, in
 * the reference's CPU operation order. */

/* out[r, :] = mask[r] != 0 ? (token_table[ids[r]] + type_table[type_ids[r]])
 *                            + position_table[position_ids[r % seq]] : 0
 * (mod.rs:343-357).  rows = batch * seq.  Ids outside their table set *d_status
 * (if non-NULL) to 1 and give a zero row. */
TNSR_B200_API int tnsr_b200_encoder_embed(const float* token_table, const float* type_table,
                                          const float* position_table, const uint32_t* ids,
                                          const uint32_t* type_ids, const uint32_t* position_ids,
                                          const float* mask, float* out, uint32_t rows, uint32_t seq,
                                          uint32_t vocab, uint32_t type_vocab, uint32_t width,
                                          int* d_status, void* stream);
/* Bidirectional attention with an additive key mask (mod.rs:358-386):
 * score = (q . k) * 1/sqrt(head_dim) + key_mask[sample, key]; softmax over all
 * seq keys; out = weights . v.  q, k, v: [batch, seq, heads*head_dim] f32 rows
 * `row_stride` floats apart (3 * width when they are slices of one fused
 * projection); key_mask [batch, seq] f32 (0, or a large negative value such as
 * f32::MIN for padding); out [batch, seq, heads*head_dim] contiguous. */
TNSR_B200_API int tnsr_b200_encoder_attention(const float* q, const float* k, const float* v,
                                              uint32_t row_stride, const float* key_mask, float* out,
                                              uint32_t batch, uint32_t seq, uint32_t heads,
                                              uint32_t head_dim, void* stream);
/* out = a + b and out = silu(gate) * up (src/nn/activations.rs:5-20 op by op), f32. */
TNSR_B200_API int tnsr_b200_add_f32(const float* a, const float* b, float* out, uint64_t elems, void* stream);
TNSR_B200_API int tnsr_b200_swiglu_f32(const float* gate, const float* up, float* out, uint64_t elems,
                                       void* stream);

/* Next-token sampling on the device (no reference counterpart: tnsr's decode
 * loop is greedy, src/nn/kv_cache.rs:121-157).  Per row: the top_k entries
 * under IEEE totalOrder with ties towards the larger index (so top_k = 1 is
 * exactly tnsr_b200_argmax); walked in index order with weights
 * w_j = (float)exp((double)((l_j - l_max) / temperature)) summed in f32; one
 * uniform u = (x >> 8) * 2^-24 from Philox4x32-10 with counter (step, 0,
 * first_session + row, 0) and key (seed & 0xffffffff, seed >> 32); the pick is
 * the first candidate whose running sum exceeds u * sum.  temperature > 0,
 * 1 <= top_k <= 256.  The rule is stated operation by operation so that a CPU
 * restatement reproduces the ids exactly. */
TNSR_B200_API int tnsr_b200_sample_top_k(const float* logits, uint32_t* out, uint32_t rows, uint32_t vocab,
                                         float temperature, uint32_t top_k, uint64_t seed, uint32_t step,
                                         uint32_t first_session, void* stream);

/* Greedy pick per row: the last index holding the maximum under IEEE
 * totalOrder (src/nn/kv_cache.rs:148-153). */
TNSR_B200_API int tnsr_b200_argmax(const float* logits, uint32_t* out, uint32_t rows, uint32_t vocab,
                                   void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TNSR_B200_H */
