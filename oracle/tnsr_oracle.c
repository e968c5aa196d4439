/*
 * tnsr_oracle.c -- CPU restatement of tnsr's CPU executor for the cached-GPT
 * inference path.  TEST INFRASTRUCTURE ONLY: this file is the checker that the
 * CUDA library is compared against and the CPU baseline that the benchmark
 * reports beside it.  Nothing in the shipped library links, imports or calls it.
 *
 * Every function cites the reference file:line (paths relative to the tnsr
 * checkout) whose arithmetic it restates.  The rule that makes the results
 * reproducible is the one the reference's interpreter follows: every primitive
 * op is a separately rounded IEEE f32 operation, reductions run in increasing
 * index order from a zero (or -inf) start, products are rounded before they
 * are added (no FMA contraction) and nothing is reassociated.  Build with
 * -ffp-contract=off and without -ffast-math (see the Makefile).
 *
 * Parity status: the reference is Rust and cannot be built in this image, so
 * the oracle is pinned against the known-answer vectors of the reference's own
 * tests (gather, batched matmul, softmax, attention, activation bit patterns,
 * bf16 narrowing, the 17x65x19 cancellation matmul) and against its own
 * decode==forward / cached==uncached invariants.  expf/logf come from glibc,
 * the same libm Rust's f32::exp / f32::ln reach on linux-gnu; the reference's
 * tests pin those two only to tolerance, so bit-level agreement of exp/log with
 * a Rust build is "parity unpinned".
 *
 * Loop nests are ordered for cache friendliness (i, p, j with per-output
 * accumulators) but every output element still sees exactly the sequence
 *      s = 0; s = s + a[i,p]*b[p,j]   for p = 0..K-1
 * of src/lib.rs:1202-1208, so values are bit-identical to the j-inner order.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

enum { ACT_RELU = 0, ACT_GELU = 1, ACT_SWIGLU = 2 };

enum {
    ORACLE_OK = 0,
    ORACLE_ERR_ARG = -1,
    ORACLE_ERR_INDEX_FINITE = -2,      /* "index must be finite"        src/lib.rs:817 */
    ORACLE_ERR_INDEX_NEGATIVE = -3,    /* "index must be non-negative"  src/lib.rs:818 */
    ORACLE_ERR_INDEX_INTEGER = -4,     /* "index must be an integer"    src/lib.rs:819-822 */
    ORACLE_ERR_INDEX_USIZE = -5,       /* "cannot be represented as usize" src/lib.rs:823-829 */
    ORACLE_ERR_INDEX_RANGE = -6,       /* "is out of range for size"    src/lib.rs:830-833 */
    ORACLE_ERR_CAPACITY = -7,
    ORACLE_ERR_ALLOC = -8
};

static int g_threads = 1;

ORACLE_API void oracle_set_threads(int n) { g_threads = n < 1 ? 1 : n; }
ORACLE_API int oracle_get_threads(void) { return g_threads; }
ORACLE_API int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------- */
/* scalar pieces                                                             */
/* ------------------------------------------------------------------------- */

/* half::bf16::from_f32 (half 2.7.1) followed by to_f32: round to nearest even
 * on the upper 16 bits, NaN kept as a quiet NaN.  Call sites src/lib.rs:740,
 * src/nn/kv_cache.rs:351; pinned by src/graph/mixed.rs:113-136. */
ORACLE_API float oracle_bf16_round(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) {
        u = (u | 0x00400000u) & 0xffff0000u;
    } else {
        uint32_t bias = 0x7fffu + ((u >> 16) & 1u);
        u = (u + bias) & 0xffff0000u;
    }
    float r;
    memcpy(&r, &u, 4);
    return r;
}

ORACLE_API uint16_t oracle_bf16_bits(float x) {
    float r = oracle_bf16_round(x);
    uint32_t u;
    memcpy(&u, &r, 4);
    return (uint16_t)(u >> 16);
}

/* nn::sigmoid, op by op (src/nn/activations.rs:5-14): gt -> 1/0, mask(v,c) ->
 * c != 0 ? v : 0 (src/lib.rs:315-329). */
static inline float sigmoid_f(float x) {
    float negative = (-x > 0.0f) ? 1.0f : 0.0f;
    float nonnegative = 1.0f - negative;
    float magnitude = x * (1.0f - negative * 2.0f);
    float z = expf(-magnitude);
    float denominator = z + 1.0f;
    float a = (nonnegative != 0.0f) ? (1.0f / denominator) : 0.0f;
    float b = (negative != 0.0f) ? (z / denominator) : 0.0f;
    return a + b;
}

/* nn::silu = x * sigmoid(x) (src/nn/activations.rs:17-20). */
static inline float silu_f(float x) { return x * sigmoid_f(x); }

/* nn::gelu, Abramowitz-Stegun 7.1.26 form (src/nn/activations.rs:29-47).  The
 * f32 literals are the reference's (0.327_591_1 etc.) and FRAC_1_SQRT_2. */
static inline float gelu_f(float x) {
    float negative = (-x > 0.0f) ? 1.0f : 0.0f;
    float nonnegative = 1.0f - negative;
    float magnitude = (x * (1.0f - negative * 2.0f)) * 0.70710678118654752440f;
    float t = 1.0f / (magnitude * 0.3275911f + 1.0f);
    float polynomial =
        ((((t * 1.0614054f - 1.4531521f) * t + 1.4214138f) * t - 0.28449672f) * t + 0.2548296f) * t;
    float tail = (polynomial * expf(-(magnitude * magnitude))) * 0.5f;
    float a = (nonnegative != 0.0f) ? (1.0f - tail) : 0.0f;
    float b = (negative != 0.0f) ? tail : 0.0f;
    return x * (a + b);
}

ORACLE_API void oracle_sigmoid(const float* x, float* y, size_t n) {
    for (size_t i = 0; i < n; ++i) y[i] = sigmoid_f(x[i]);
}
ORACLE_API void oracle_silu(const float* x, float* y, size_t n) {
    for (size_t i = 0; i < n; ++i) y[i] = silu_f(x[i]);
}
ORACLE_API void oracle_gelu(const float* x, float* y, size_t n) {
    for (size_t i = 0; i < n; ++i) y[i] = gelu_f(x[i]);
}
/* The elementwise SwiGLU training kernel's forward, silu(gate) * up
 * (src/tile/swiglu.rs:35-121). */
ORACLE_API void oracle_swiglu(const float* gate, const float* up, float* y, size_t n) {
    for (size_t i = 0; i < n; ++i) y[i] = silu_f(gate[i]) * up[i];
}

/* ------------------------------------------------------------------------- */
/* tensor primitives                                                         */
/* ------------------------------------------------------------------------- */

/* checked_index for floating ids (src/lib.rs:816-835). */
static int check_index(float value, size_t upper, size_t* out) {
    if (!isfinite(value)) return ORACLE_ERR_INDEX_FINITE;
    if (!(value >= 0.0f)) return ORACLE_ERR_INDEX_NEGATIVE;
    if (value - truncf(value) != 0.0f) return ORACLE_ERR_INDEX_INTEGER;
    if (value >= 18446744073709551616.0f) return ORACLE_ERR_INDEX_USIZE;
    size_t index = (size_t)value;
    if ((float)index != value) return ORACLE_ERR_INDEX_USIZE;
    if (index >= upper) return ORACLE_ERR_INDEX_RANGE;
    *out = index;
    return ORACLE_OK;
}

/* embedding_forward (src/lib.rs:868-909): out[i,:] = weight[idx[i],:], exact
 * copy; ids arrive as f32 and are validated one by one. */
ORACLE_API int oracle_embedding(const float* weight, size_t vocabulary, size_t channels,
                                const float* indices, size_t count, float* out) {
    for (size_t i = 0; i < count; ++i) {
        size_t index = 0;
        int rc = check_index(indices[i], vocabulary, &index);
        if (rc != ORACLE_OK) return rc;
        memcpy(out + i * channels, weight + index * channels, channels * sizeof(float));
    }
    return ORACLE_OK;
}

/* matmul_forward for f32 (src/lib.rs:1179-1211): out[b,i,j] = sum_p a*b with a
 * zero start, increasing p, rounded product then rounded add.  `b_batches` is
 * 1 (broadcast right operand) or `batches`. */
static void matmul_rows(const float* a, const float* b, float* out, size_t m, size_t k, size_t n) {
#pragma omp parallel for schedule(static) num_threads(g_threads) if (g_threads > 1 && m > 1)
    for (size_t i = 0; i < m; ++i) {
        float* o = out + i * n;
        for (size_t j = 0; j < n; ++j) o[j] = 0.0f;
        const float* ar = a + i * k;
        for (size_t p = 0; p < k; ++p) {
            const float av = ar[p];
            const float* br = b + p * n;
            for (size_t j = 0; j < n; ++j) o[j] = o[j] + av * br[j];
        }
    }
}

ORACLE_API void oracle_matmul(const float* a, const float* b, float* out, size_t batches,
                              size_t b_batches, size_t m, size_t k, size_t n) {
    for (size_t batch = 0; batch < batches; ++batch) {
        const float* bb = b + (b_batches == 1 ? 0 : batch) * k * n;
        matmul_rows(a + batch * m * k, bb, out + batch * m * n, m, k, n);
    }
}

/* The interpreter's reference loop nest, kept verbatim in shape (i, j, p) so a
 * test can show the reordered nest above is bit-identical to it. */
ORACLE_API void oracle_matmul_naive(const float* a, const float* b, float* out, size_t m, size_t k,
                                    size_t n) {
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) {
            float sum = 0.0f;
            for (size_t p = 0; p < k; ++p) sum = sum + a[i * k + p] * b[p * n + j];
            out[i * n + j] = sum;
        }
}

/* A @ B^T with B stored [n,k]: what `x.matmul(w.transpose())` evaluates to
 * once the permute has been materialised (src/nn/kv_cache/graph.rs:156-158,
 * src/lib.rs:1609-1642): same increasing-p order. */
static void matmul_bt_rows(const float* a, const float* bt, float* out, size_t m, size_t k,
                           size_t n) {
#pragma omp parallel for schedule(static) num_threads(g_threads) if (g_threads > 1 && m * n > 64)
    for (size_t ij = 0; ij < m * n; ++ij) {
        size_t i = ij / n, j = ij % n;
        const float* ar = a + i * k;
        const float* br = bt + j * k;
        float sum = 0.0f;
        for (size_t p = 0; p < k; ++p) sum = sum + ar[p] * br[p];
        out[ij] = sum;
    }
}

/* Linear node (src/lib.rs:446-457): matmul, then `out[i] = out[i] + bias[i % width]`
 * as a second rounded op. */
static void linear(const float* x, const float* w, const float* bias, float* out, size_t m,
                   size_t k, size_t n) {
    matmul_rows(x, w, out, m, k, n);
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) out[i * n + j] = out[i * n + j] + bias[j];
}

ORACLE_API void oracle_linear(const float* x, const float* w, const float* bias, float* out,
                              size_t m, size_t k, size_t n) {
    if (bias) linear(x, w, bias, out, m, k, n);
    else matmul_rows(x, w, out, m, k, n);
}

/* nn::softmax over the last axis (src/nn.rs:149-162) on the interpreter's
 * reductions (src/lib.rs:1737-1759): max folds from -inf with f32::max
 * (IEEE maxNum -> fmaxf), exp(x - max), sum from 0 in index order, divide. */
static void softmax_row(const float* x, float* y, size_t n) {
    float mx = -INFINITY;
    for (size_t j = 0; j < n; ++j) mx = fmaxf(mx, x[j]);
    for (size_t j = 0; j < n; ++j) y[j] = expf(x[j] - mx);
    float sum = 0.0f;
    for (size_t j = 0; j < n; ++j) sum = sum + y[j];
    for (size_t j = 0; j < n; ++j) y[j] = y[j] / sum;
}

ORACLE_API void oracle_softmax(const float* x, float* y, size_t rows, size_t n) {
    for (size_t r = 0; r < rows; ++r) softmax_row(x + r * n, y + r * n, n);
}

/* nn::layer_norm over the last axis (src/nn.rs:165-213): Mean reduction adds
 * val / n element by element (src/lib.rs:1752-1754); inv_std is
 * exp(ln(var + eps) * -0.5); y = ((c * inv) * w) + b. */
static void layer_norm_row(const float* x, const float* w, const float* b, float eps, float* y,
                           size_t n) {
    const float nf = (float)n;
    float mean = 0.0f;
    for (size_t c = 0; c < n; ++c) mean = mean + x[c] / nf;
    float var = 0.0f;
    for (size_t c = 0; c < n; ++c) {
        float d = x[c] - mean;
        float sq = d * d;
        var = var + sq / nf;
    }
    float inv = expf(logf(var + eps) * -0.5f);
    for (size_t c = 0; c < n; ++c) {
        float d = x[c] - mean;
        y[c] = ((d * inv) * w[c]) + b[c];
    }
}

ORACLE_API void oracle_layer_norm(const float* x, const float* w, const float* b, float eps,
                                  float* y, size_t rows, size_t n) {
#pragma omp parallel for schedule(static) num_threads(g_threads) if (g_threads > 1 && rows > 1)
    for (size_t r = 0; r < rows; ++r) layer_norm_row(x + r * n, w, b, eps, y + r * n, n);
}

/* ------------------------------------------------------------------------- */
/* model                                                                     */
/* ------------------------------------------------------------------------- */

typedef struct {
    uint32_t vocab_size;
    uint32_t max_sequence_length;
    uint32_t embed_dim;
    uint32_t num_heads;
    uint32_t feed_forward_dim;
    uint32_t num_layers;
    float layer_norm_epsilon;
    uint32_t activation;      /* ACT_*: RELU is nn::Gpt's own block */
    uint32_t attention_bf16;  /* GptAttentionPrecision::Bf16 (src/nn/kv_cache.rs:21-26) */
} oracle_config;

typedef struct {
    oracle_config cfg;
    size_t count;
    float** params;
    size_t* elems;
} oracle_model;

static size_t per_layer(const oracle_config* c) { return c->activation == ACT_SWIGLU ? 18 : 16; }

/* Parameter order: model_parameters (src/nn/kv_cache.rs:392-421); the SwiGLU
 * extension replaces (ff_in_w, ff_in_b, ff_out_w, ff_out_b) with
 * (gate_w, gate_b, up_w, up_b, down_w, down_b), following the composition in
 * examples/forty_five/mod.rs:398-407. */
static size_t param_elems(const oracle_config* c, size_t index) {
    size_t d = c->embed_dim, f = c->feed_forward_dim;
    if (index == 0) return (size_t)c->vocab_size * d;
    if (index == 1) return (size_t)c->max_sequence_length * d;
    if (index < 4) return d;
    size_t k = (index - 4) % per_layer(c);
    if (k < 8) return (k % 2 == 0) ? d * d : d;
    if (k < 12) return d;
    if (c->activation == ACT_SWIGLU) {
        switch (k) {
            case 12: case 14: return d * f;
            case 13: case 15: return f;
            case 16: return f * d;
            default: return d;
        }
    }
    switch (k) {
        case 12: return d * f;
        case 13: return f;
        case 14: return f * d;
        default: return d;
    }
}

ORACLE_API oracle_model* oracle_model_create(const oracle_config* cfg) {
    if (!cfg || cfg->vocab_size == 0 || cfg->max_sequence_length == 0 || cfg->embed_dim == 0 ||
        cfg->num_layers == 0 || cfg->feed_forward_dim == 0 || cfg->num_heads == 0 ||
        cfg->embed_dim % cfg->num_heads != 0 || !(cfg->layer_norm_epsilon > 0.0f) ||
        !isfinite(cfg->layer_norm_epsilon) || cfg->activation > ACT_SWIGLU)
        return NULL;
    oracle_model* m = (oracle_model*)calloc(1, sizeof(*m));
    if (!m) return NULL;
    m->cfg = *cfg;
    m->count = 4 + per_layer(cfg) * cfg->num_layers;
    m->params = (float**)calloc(m->count, sizeof(float*));
    m->elems = (size_t*)calloc(m->count, sizeof(size_t));
    for (size_t i = 0; i < m->count; ++i) {
        m->elems[i] = param_elems(cfg, i);
        m->params[i] = (float*)calloc(m->elems[i], sizeof(float));
    }
    return m;
}

ORACLE_API void oracle_model_destroy(oracle_model* m) {
    if (!m) return;
    for (size_t i = 0; i < m->count; ++i) free(m->params[i]);
    free(m->params);
    free(m->elems);
    free(m);
}

ORACLE_API size_t oracle_model_param_count(const oracle_model* m) { return m->count; }
ORACLE_API size_t oracle_model_param_elems(const oracle_model* m, size_t i) {
    return i < m->count ? m->elems[i] : 0;
}
ORACLE_API int oracle_model_set_param(oracle_model* m, size_t i, const float* data, size_t n) {
    if (i >= m->count || n != m->elems[i]) return ORACLE_ERR_ARG;
    memcpy(m->params[i], data, n * sizeof(float));
    return ORACLE_OK;
}
ORACLE_API int oracle_model_get_param(const oracle_model* m, size_t i, float* data, size_t n) {
    if (i >= m->count || n != m->elems[i]) return ORACLE_ERR_ARG;
    memcpy(data, m->params[i], n * sizeof(float));
    return ORACLE_OK;
}

/* xavier_parameter (src/nn.rs:303-316): 64-bit LCG, 24 high bits -> unit. */
ORACLE_API void oracle_xavier(float* out, size_t rows, size_t columns, uint64_t seed) {
    float limit = sqrtf(6.0f / (float)(rows + columns));
    uint64_t state = seed;
    for (size_t i = 0; i < rows * columns; ++i) {
        state = state * 6364136223846793005ull + 1ull;
        float unit = (float)(state >> 40) / (float)(1u << 24);
        out[i] = (unit * 2.0f - 1.0f) * limit;
    }
}

/* Gpt::new defaults (src/nn.rs:597-612, :347-355, :478-499): seeds 101/102,
 * layer offset 1000 + 100*layer with +1..+4 q,k,v,o and +5/+6 the two FFN
 * matrices; biases 0; LayerNorm weight 1, bias 0.  SwiGLU extension: +5 gate,
 * +6 up, +7 down. */
ORACLE_API void oracle_model_init_reference(oracle_model* m) {
    const oracle_config* c = &m->cfg;
    size_t d = c->embed_dim, f = c->feed_forward_dim, pl = per_layer(c);
    oracle_xavier(m->params[0], c->vocab_size, d, 101);
    oracle_xavier(m->params[1], c->max_sequence_length, d, 102);
    for (size_t i = 0; i < d; ++i) { m->params[2][i] = 1.0f; m->params[3][i] = 0.0f; }
    for (size_t l = 0; l < c->num_layers; ++l) {
        float** p = m->params + 4 + l * pl;
        uint64_t off = 1000 + 100 * (uint64_t)l;
        for (size_t k = 0; k < 4; ++k) {
            oracle_xavier(p[2 * k], d, d, off + 1 + k);
            memset(p[2 * k + 1], 0, d * sizeof(float));
        }
        for (size_t i = 0; i < d; ++i) { p[8][i] = 1.0f; p[9][i] = 0.0f; p[10][i] = 1.0f; p[11][i] = 0.0f; }
        if (c->activation == ACT_SWIGLU) {
            oracle_xavier(p[12], d, f, off + 5); memset(p[13], 0, f * sizeof(float));
            oracle_xavier(p[14], d, f, off + 6); memset(p[15], 0, f * sizeof(float));
            oracle_xavier(p[16], f, d, off + 7); memset(p[17], 0, d * sizeof(float));
        } else {
            oracle_xavier(p[12], d, f, off + 5); memset(p[13], 0, f * sizeof(float));
            oracle_xavier(p[14], f, d, off + 6); memset(p[15], 0, d * sizeof(float));
        }
    }
}

/* ------------------------------------------------------------------------- */
/* one decode step = build_graph evaluated by the interpreter                 */
/* ------------------------------------------------------------------------- */

typedef struct {
    oracle_model* model;
    size_t batch, capacity, length;
    float** cache; /* 2 * layers tensors [batch, capacity, d]; K then V per layer */
} oracle_decoder;

ORACLE_API oracle_decoder* oracle_decoder_create(oracle_model* m, size_t batch, size_t capacity) {
    if (!m || batch == 0 || capacity == 0 || capacity > m->cfg.max_sequence_length) return NULL;
    oracle_decoder* dec = (oracle_decoder*)calloc(1, sizeof(*dec));
    if (!dec) return NULL;
    dec->model = m;
    dec->batch = batch;
    dec->capacity = capacity;
    size_t n = 2 * (size_t)m->cfg.num_layers;
    dec->cache = (float**)calloc(n, sizeof(float*));
    for (size_t i = 0; i < n; ++i) {
        dec->cache[i] = (float*)calloc(batch * capacity * m->cfg.embed_dim, sizeof(float));
        if (!dec->cache[i]) return NULL;
    }
    return dec;
}

ORACLE_API void oracle_decoder_destroy(oracle_decoder* dec) {
    if (!dec) return;
    size_t n = 2 * (size_t)dec->model->cfg.num_layers;
    for (size_t i = 0; i < n; ++i) free(dec->cache[i]);
    free(dec->cache);
    free(dec);
}

/* GptDecoder::reset, CPU arm (src/nn/kv_cache.rs:238-257). */
ORACLE_API void oracle_decoder_reset(oracle_decoder* dec) {
    size_t n = 2 * (size_t)dec->model->cfg.num_layers;
    for (size_t i = 0; i < n; ++i)
        memset(dec->cache[i], 0, dec->batch * dec->capacity * dec->model->cfg.embed_dim * sizeof(float));
    dec->length = 0;
}

ORACLE_API size_t oracle_decoder_len(const oracle_decoder* dec) { return dec->length; }

ORACLE_API int oracle_decoder_read_cache(const oracle_decoder* dec, size_t index, float* out) {
    if (index >= 2 * (size_t)dec->model->cfg.num_layers) return ORACLE_ERR_ARG;
    memcpy(out, dec->cache[index], dec->batch * dec->capacity * dec->model->cfg.embed_dim * sizeof(float));
    return ORACLE_OK;
}

/* Test hook: overwrite one cache tensor (used to poison unused slots). */
ORACLE_API int oracle_decoder_write_cache(oracle_decoder* dec, size_t index, const float* in) {
    if (index >= 2 * (size_t)dec->model->cfg.num_layers) return ORACLE_ERR_ARG;
    memcpy(dec->cache[index], in, dec->batch * dec->capacity * dec->model->cfg.embed_dim * sizeof(float));
    return ORACLE_OK;
}

ORACLE_API void oracle_decoder_set_len(oracle_decoder* dec, size_t length) { dec->length = length; }

static void round_bf16_inplace(float* x, size_t n) {
    for (size_t i = 0; i < n; ++i) x[i] = oracle_bf16_round(x[i]);
}

/* Attention of `chunk` new queries over `past + chunk` keys for one batch row
 * and head, as the decode graph spells it (src/nn/kv_cache/graph.rs:82-107):
 * keys = concat(cache[0..past], new); scores = (q . k) * scale + mask;
 * softmax; probabilities @ values.  `kc`/`vc` point at cache row 0 of this
 * batch row; q/k/v at this row's first new position; all with row stride d. */
static void attention_head(const float* q, const float* k, const float* v, const float* kc,
                           const float* vc, size_t past, size_t chunk, size_t d, size_t hd,
                           size_t head, float scale, float* out /* row stride d */,
                           float* scores /* scratch [past+chunk] */, float* acc /* [hd] */) {
    const size_t off = head * hd, total = past + chunk;
    for (size_t t = 0; t < chunk; ++t) {
        const float* qr = q + t * d + off;
        for (size_t j = 0; j < total; ++j) {
            const float* kr = (j < past) ? kc + j * d + off : k + (j - past) * d + off;
            float sum = 0.0f;
            for (size_t c = 0; c < hd; ++c) sum = sum + qr[c] * kr[c];
            float scaled = sum * scale;
            float mask = (j <= past + t) ? 0.0f : -INFINITY; /* src/nn/kv_cache.rs:323-330 */
            scores[j] = scaled + mask;
        }
        softmax_row(scores, scores, total);
        for (size_t c = 0; c < hd; ++c) acc[c] = 0.0f;
        for (size_t j = 0; j < total; ++j) {
            const float* vr = (j < past) ? vc + j * d + off : v + (j - past) * d + off;
            const float p = scores[j];
            for (size_t c = 0; c < hd; ++c) acc[c] = acc[c] + p * vr[c];
        }
        memcpy(out + t * d + off, acc, hd * sizeof(float));
    }
}

/* The feed-forward half of a block.  RELU is nn::Gpt's (graph.rs:126-147);
 * GELU swaps the activation for nn::gelu; SWIGLU follows
 * examples/forty_five/mod.rs:398-407: down(silu(gate(x)) * up(x)), all three
 * linears with bias. */
static int feed_forward(const oracle_config* c, float** p, const float* n2, float* r, size_t rows) {
    size_t d = c->embed_dim, f = c->feed_forward_dim;
    float* hidden = (float*)malloc(rows * f * sizeof(float));
    float* out = (float*)malloc(rows * d * sizeof(float));
    if (!hidden || !out) { free(hidden); free(out); return ORACLE_ERR_ALLOC; }
    if (c->activation == ACT_SWIGLU) {
        float* up = (float*)malloc(rows * f * sizeof(float));
        if (!up) { free(hidden); free(out); return ORACLE_ERR_ALLOC; }
        linear(n2, p[12], p[13], hidden, rows, d, f);
        linear(n2, p[14], p[15], up, rows, d, f);
        for (size_t i = 0; i < rows * f; ++i) hidden[i] = silu_f(hidden[i]) * up[i];
        free(up);
        linear(hidden, p[16], p[17], out, rows, f, d);
    } else {
        linear(n2, p[12], p[13], hidden, rows, d, f);
        if (c->activation == ACT_GELU)
            for (size_t i = 0; i < rows * f; ++i) hidden[i] = gelu_f(hidden[i]);
        else
            for (size_t i = 0; i < rows * f; ++i) hidden[i] = fmaxf(hidden[i], 0.0f); /* src/lib.rs:278 */
        linear(hidden, p[14], p[15], out, rows, f, d);
    }
    for (size_t i = 0; i < rows * d; ++i) r[i] = r[i] + out[i];
    free(hidden);
    free(out);
    return ORACLE_OK;
}

/* One step: `tokens` is row-major [batch, chunk]; positions start at `past`.
 * Writes logits [batch, chunk, vocab].  When `cache` is non-NULL the prefix is
 * read from it and the new K/V rows are appended after the whole step
 * (src/nn/kv_cache.rs:347-361); with cache == NULL and past == 0 this is
 * Gpt::forward (src/nn.rs:629-668), whose attention graph is the same
 * expression with a [seq, seq] causal mask (src/nn.rs:216-301). */
static int step(const oracle_model* m, float** cache, size_t capacity, size_t batch, size_t past,
                size_t chunk, const uint32_t* tokens, float* logits) {
    const oracle_config* c = &m->cfg;
    const size_t d = c->embed_dim, H = c->num_heads, hd = d / H, V = c->vocab_size;
    const size_t rows = batch * chunk, pl = per_layer(c);
    for (size_t i = 0; i < rows; ++i)
        if (tokens[i] >= V) return ORACLE_ERR_INDEX_RANGE;
    if (past + chunk > c->max_sequence_length) return ORACLE_ERR_CAPACITY;

    float* h = (float*)malloc(rows * d * sizeof(float));
    float* n = (float*)malloc(rows * d * sizeof(float));
    float* q = (float*)malloc(rows * d * sizeof(float));
    float* k = (float*)malloc(rows * d * sizeof(float));
    float* v = (float*)malloc(rows * d * sizeof(float));
    float* att = (float*)malloc(rows * d * sizeof(float));
    float* proj = (float*)malloc(rows * d * sizeof(float));
    float* newk = (float*)malloc((size_t)c->num_layers * rows * d * sizeof(float));
    float* newv = (float*)malloc((size_t)c->num_layers * rows * d * sizeof(float));
    int rc = ORACLE_OK;
    if (!h || !n || !q || !k || !v || !att || !proj || !newk || !newv) { rc = ORACLE_ERR_ALLOC; goto done; }

    /* graph.rs:30-41: token rows gathered exactly, position rows gathered and
     * broadcast over the batch, one add per element. */
    for (size_t b = 0; b < batch; ++b)
        for (size_t t = 0; t < chunk; ++t) {
            const float* tr = m->params[0] + (size_t)tokens[b * chunk + t] * d;
            const float* pr = m->params[1] + (past + t) * d;
            float* hr = h + (b * chunk + t) * d;
            for (size_t x = 0; x < d; ++x) hr[x] = tr[x] + pr[x];
        }

    /* graph.rs:104-105: (width as f32 / heads as f32).sqrt().recip() */
    const float scale = 1.0f / sqrtf((float)d / (float)H);

    for (size_t l = 0; l < c->num_layers; ++l) {
        float** p = m->params + 4 + l * pl;
        oracle_layer_norm(h, p[8], p[9], c->layer_norm_epsilon, n, rows, d);
        linear(n, p[0], p[1], q, rows, d, d);
        linear(n, p[2], p[3], k, rows, d, d);
        linear(n, p[4], p[5], v, rows, d, d);
        /* The cache receives the projected values, rounded at append time in
         * bf16 mode (kv_cache.rs:349-353); attention sees the same rounded
         * values through the Cast pair (graph.rs:95-104). */
        if (c->attention_bf16) {
            round_bf16_inplace(q, rows * d);
            round_bf16_inplace(k, rows * d);
            round_bf16_inplace(v, rows * d);
        }
        memcpy(newk + l * rows * d, k, rows * d * sizeof(float));
        memcpy(newv + l * rows * d, v, rows * d * sizeof(float));

#pragma omp parallel num_threads(g_threads) if (g_threads > 1 && batch * H > 1)
        {
            float* scores = (float*)malloc((past + chunk) * sizeof(float));
            float* acc = (float*)malloc(hd * sizeof(float));
#pragma omp for schedule(dynamic)
            for (size_t bh = 0; bh < batch * H; ++bh) {
                size_t b = bh / H, head = bh % H;
                const float* kc = cache ? cache[2 * l] + b * capacity * d : NULL;
                const float* vc = cache ? cache[2 * l + 1] + b * capacity * d : NULL;
                attention_head(q + b * chunk * d, k + b * chunk * d, v + b * chunk * d, kc, vc, past,
                               chunk, d, hd, head, scale, att + b * chunk * d, scores, acc);
            }
            free(scores);
            free(acc);
        }
        if (c->attention_bf16) round_bf16_inplace(att, rows * d); /* graph.rs:107 */

        /* graph.rs:116-125: residual = hidden + linear(attended) */
        linear(att, p[6], p[7], proj, rows, d, d);
        for (size_t i = 0; i < rows * d; ++i) h[i] = h[i] + proj[i];
        oracle_layer_norm(h, p[10], p[11], c->layer_norm_epsilon, n, rows, d);
        rc = feed_forward(c, p, n, h, rows);
        if (rc != ORACLE_OK) goto done;
    }

    /* graph.rs:149-159: final norm, tied head. */
    oracle_layer_norm(h, m->params[2], m->params[3], c->layer_norm_epsilon, n, rows, d);
    matmul_bt_rows(n, m->params[0], logits, rows, d, V);

    if (cache) {
        for (size_t l = 0; l < c->num_layers; ++l)
            for (size_t b = 0; b < batch; ++b) {
                size_t start = (b * capacity + past) * d;
                memcpy(cache[2 * l] + start, newk + l * rows * d + b * chunk * d, chunk * d * sizeof(float));
                memcpy(cache[2 * l + 1] + start, newv + l * rows * d + b * chunk * d, chunk * d * sizeof(float));
            }
    }
done:
    free(h); free(n); free(q); free(k); free(v); free(att); free(proj); free(newk); free(newv);
    return rc;
}

/* GptDecoder::decode, arithmetic only (src/nn/kv_cache.rs:261-389).  The
 * session guards (failed flag, rectangular chunk, revision check) live in the
 * wrapper that both the checker and the CUDA library share. */
ORACLE_API int oracle_decoder_decode(oracle_decoder* dec, const uint32_t* tokens, size_t chunk,
                                     float* logits) {
    if (chunk == 0) return ORACLE_ERR_ARG;
    if (chunk > dec->capacity - dec->length) return ORACLE_ERR_CAPACITY;
    int rc = step(dec->model, dec->cache, dec->capacity, dec->batch, dec->length, chunk, tokens, logits);
    if (rc == ORACLE_OK) dec->length += chunk;
    return rc;
}

/* Gpt::forward (src/nn.rs:629-668): logits [batch, sequence, vocab]. */
ORACLE_API int oracle_forward(const oracle_model* m, const uint32_t* tokens, size_t batch,
                              size_t sequence, float* logits) {
    if (batch == 0 || sequence == 0 || sequence > m->cfg.max_sequence_length) return ORACLE_ERR_ARG;
    return step(m, NULL, 0, batch, 0, sequence, tokens, logits);
}

/* `max_by(total_cmp)` over a logits row (src/nn/kv_cache.rs:148-153,
 * src/nn.rs:706-711): the LAST index attaining the maximum under IEEE
 * totalOrder (so +NaN sorts above +inf and -0 below +0). */
static int64_t total_order_key(float x) {
    int32_t bits;
    memcpy(&bits, &x, 4);
    bits ^= (int32_t)(((uint32_t)(bits >> 31)) >> 1);
    return bits;
}

ORACLE_API size_t oracle_argmax_last(const float* row, size_t n) {
    size_t best = 0;
    int64_t best_key = total_order_key(row[0]);
    for (size_t i = 1; i < n; ++i) {
        int64_t key = total_order_key(row[i]);
        if (key >= best_key) { best = i; best_key = key; }
    }
    return best;
}

/* Gpt::generate (src/nn.rs:680-715): re-run the whole retained context for
 * every new token.  `out` has room for prompt_len + max_new ids. */
ORACLE_API int oracle_generate(const oracle_model* m, const uint32_t* prompt, size_t prompt_len,
                               size_t max_new, uint32_t* out) {
    const size_t V = m->cfg.vocab_size, ctx = m->cfg.max_sequence_length;
    if (prompt_len == 0) return ORACLE_ERR_ARG;
    for (size_t i = 0; i < prompt_len; ++i) if (prompt[i] >= V) return ORACLE_ERR_INDEX_RANGE;
    memcpy(out, prompt, prompt_len * sizeof(uint32_t));
    size_t len = prompt_len;
    float* logits = (float*)malloc(ctx * V * sizeof(float));
    if (!logits) return ORACLE_ERR_ALLOC;
    for (size_t s = 0; s < max_new; ++s) {
        size_t start = len > ctx ? len - ctx : 0, n = len - start;
        int rc = oracle_forward(m, out + start, 1, n, logits);
        if (rc != ORACLE_OK) { free(logits); return rc; }
        out[len++] = (uint32_t)oracle_argmax_last(logits + (n - 1) * V, V);
    }
    free(logits);
    return ORACLE_OK;
}

/* Gpt::generate_cached (src/nn/kv_cache.rs:121-157): decoder of batch 1 and
 * full context; when empty or full, reset and re-prefill the last `capacity`
 * tokens from position 0, else decode the last token. */
ORACLE_API int oracle_generate_cached(oracle_model* m, const uint32_t* prompt, size_t prompt_len,
                                      size_t max_new, uint32_t* out) {
    const size_t V = m->cfg.vocab_size, ctx = m->cfg.max_sequence_length;
    if (prompt_len == 0) return ORACLE_ERR_ARG;
    for (size_t i = 0; i < prompt_len; ++i) if (prompt[i] >= V) return ORACLE_ERR_INDEX_RANGE;
    memcpy(out, prompt, prompt_len * sizeof(uint32_t));
    if (max_new == 0) return ORACLE_OK;
    size_t len = prompt_len;
    oracle_decoder* dec = oracle_decoder_create(m, 1, ctx);
    float* logits = (float*)malloc(ctx * V * sizeof(float));
    if (!dec || !logits) { oracle_decoder_destroy(dec); free(logits); return ORACLE_ERR_ALLOC; }
    int rc = ORACLE_OK;
    for (size_t s = 0; s < max_new; ++s) {
        size_t n;
        if (dec->length == 0 || dec->length == dec->capacity) {
            oracle_decoder_reset(dec);
            size_t start = len > ctx ? len - ctx : 0;
            n = len - start;
            rc = oracle_decoder_decode(dec, out + start, n, logits);
        } else {
            n = 1;
            rc = oracle_decoder_decode(dec, out + len - 1, 1, logits);
        }
        if (rc != ORACLE_OK) break;
        out[len++] = (uint32_t)oracle_argmax_last(logits + (n - 1) * V, V);
    }
    oracle_decoder_destroy(dec);
    free(logits);
    return rc;
}

/* ------------------------------------------------------------------------- */
/* standalone operators for the operator-level configurations                 */
/* ------------------------------------------------------------------------- */

/* Live-prefix decode attention over a [batch, capacity, heads*hd] cache with
 * per-session lengths: session b attends keys 0..lengths[b]-1 (its newest row
 * already stored at lengths[b]-1).  Same arithmetic as attention_head with
 * chunk = 1 and every key read from the cache. */
ORACLE_API void oracle_decode_attention(const float* q /* [batch, d] */, const float* kcache,
                                        const float* vcache, const uint32_t* lengths, size_t batch,
                                        size_t capacity, size_t heads, size_t hd, float* out) {
    const size_t d = heads * hd;
    const float scale = 1.0f / sqrtf((float)d / (float)heads);
#pragma omp parallel num_threads(g_threads) if (g_threads > 1)
    {
        float* scores = (float*)malloc(capacity * sizeof(float));
        float* acc = (float*)malloc(hd * sizeof(float));
#pragma omp for schedule(dynamic)
        for (size_t bh = 0; bh < batch * heads; ++bh) {
            size_t b = bh / heads, head = bh % heads, len = lengths[b];
            if (len == 0 || len > capacity) continue;
            /* keys 0..len-2 are the "past"; the newest row (len-1) plays the
             * part of the chunk's own key and is read from the same cache. */
            const float* kc = kcache + b * capacity * d;
            const float* vc = vcache + b * capacity * d;
            attention_head(q + b * d, kc + (len - 1) * d, vc + (len - 1) * d, kc, vc, len - 1, 1, d,
                           hd, head, scale, out + b * d, scores, acc);
        }
        free(scores);
        free(acc);
    }
}

/* Independent f64 attention reference in the style of the reference's own
 * kernel tests (src/nn/kv_cache/cuda/tests.rs:118-160): f64 dot, / sqrt(hd),
 * max, exp, sum, weighted average.  Keys 0..prefix-1 come from the cache,
 * prefix.. from the new chunk; query t sees keys 0..prefix+t. */
ORACLE_API void oracle_attention_f64(const float* q, const float* k, const float* v,
                                     const float* kcache, const float* vcache, size_t batch,
                                     size_t heads, size_t hd, size_t capacity, size_t prefix,
                                     size_t chunk, double* out /* [batch, heads, chunk, hd] */) {
    const size_t d = heads * hd;
    double* w = (double*)malloc((prefix + chunk) * sizeof(double));
    for (size_t b = 0; b < batch; ++b)
        for (size_t head = 0; head < heads; ++head)
            for (size_t t = 0; t < chunk; ++t) {
                size_t total = prefix + t + 1;
                double mx = -INFINITY;
                for (size_t j = 0; j < total; ++j) {
                    double s = 0.0;
                    for (size_t c = 0; c < hd; ++c) {
                        size_t f = head * hd + c;
                        double kv = j < prefix ? kcache[(b * capacity + j) * d + f]
                                               : k[(b * chunk + j - prefix) * d + f];
                        s += (double)q[(b * chunk + t) * d + f] * kv;
                    }
                    w[j] = s / sqrt((double)hd);
                    if (w[j] > mx) mx = w[j];
                }
                double den = 0.0;
                for (size_t j = 0; j < total; ++j) { w[j] = exp(w[j] - mx); den += w[j]; }
                for (size_t c = 0; c < hd; ++c) {
                    size_t f = head * hd + c;
                    double acc = 0.0;
                    for (size_t j = 0; j < total; ++j) {
                        double vv = j < prefix ? vcache[(b * capacity + j) * d + f]
                                               : v[(b * chunk + j - prefix) * d + f];
                        acc += w[j] * vv;
                    }
                    out[((b * heads + head) * chunk + t) * hd + c] = acc / den;
                }
            }
    free(w);
}

/* SwiGLU MLP block: down(silu(x.Wg + bg) * (x.Wu + bu)) + bd, the composition
 * of examples/forty_five/mod.rs:398-407 without the residual. */
ORACLE_API int oracle_swiglu_mlp(const float* x, const float* wg, const float* bg, const float* wu,
                                 const float* bu, const float* wd, const float* bd, float* out,
                                 size_t rows, size_t d, size_t f) {
    float* g = (float*)malloc(rows * f * sizeof(float));
    float* u = (float*)malloc(rows * f * sizeof(float));
    if (!g || !u) { free(g); free(u); return ORACLE_ERR_ALLOC; }
    linear(x, wg, bg, g, rows, d, f);
    linear(x, wu, bu, u, rows, d, f);
    for (size_t i = 0; i < rows * f; ++i) g[i] = silu_f(g[i]) * u[i];
    linear(g, wd, bd, out, rows, f, d);
    free(g);
    free(u);
    return ORACLE_OK;
}

/* SimpleExecutor<bf16> matmul (src/lib.rs:1111-1162, :1216-1218): operands are
 * bf16 values widened to f32, sequential f32 dot, result rounded to bf16.  The
 * caller passes f32 arrays that already hold bf16-representable values. */
ORACLE_API void oracle_matmul_bf16(const float* a, const float* b, float* out, size_t batches,
                                   size_t b_batches, size_t m, size_t k, size_t n) {
    oracle_matmul(a, b, out, batches, b_batches, m, k, n);
    round_bf16_inplace(out, batches * m * n);
}
