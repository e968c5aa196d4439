// KV-cache attention on bf16 caches.
//
//  * decode_attention_*: one query per (session, head) scanned over the live
//    prefix only, split over the key axis so that every SM streams a contiguous
//    slab of K and V rows (all heads) through a shared-memory ring filled by
//    bulk async copies (cp.async.bulk, mbarrier completion); f32 online softmax;
//    partials (max, sum, numerator) are merged inside the same kernel by whichever
//    warp stores the last partial of a (session, head) pair.  This is
//    the job of the reference's AttentionScan / MergeScan pair
//    (src/nn/kv_cache/attention.rs:31-239, :242-393; fixed 16/32 partitions,
//    src/nn/kv_cache/cuda.rs:31-32,110-116) with two differences: the split is
//    by fixed key-slab size chosen from the total live length, so ragged
//    per-session lengths balance across SMs, and K/V are read as whole cache
//    rows (all heads at once) so HBM sees only long contiguous bursts.
//  * attention_generic: any head width and chunk, one warp per query/head.
//
// HBM traffic per decode step is the live K and V rows once: 4 * d bytes per
// live key per session (d = heads * head_dim) plus q / out / partials.
#include "common.cuh"

namespace tb {

thread_local KernelTimer* t_attention_timer = nullptr;
thread_local bool t_pdl = false;

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ===========================================================================
// Generic kernel (bf16): one warp per (session, head, query); lane c owns dims
// c, c+32, ...; keys walked in order with a running max / sum / numerator.
// ===========================================================================
constexpr int GEN_MAX_SLOTS = 8;  // head_dim <= 256

__global__ void __launch_bounds__(128)
attention_generic_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                         bf16* __restrict__ out, uint32_t total_queries, uint32_t chunk, uint32_t position,
                         const uint32_t* __restrict__ d_position, uint32_t capacity, uint32_t heads, uint32_t hd,
                         float scale_log2, KvPaging paging) {
    pdl_wait();
    pdl_trigger();
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t idx = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (idx >= total_queries) return;
    const uint32_t t = idx % chunk, h = (idx / chunk) % heads, s = idx / (chunk * heads);
    const uint32_t d = heads * hd;
    const uint32_t past = d_position ? *d_position : position;
    uint32_t total = past + t + 1;
    if (total > capacity) total = capacity;
    float qv[GEN_MAX_SLOTS], acc[GEN_MAX_SLOTS];
    const bf16* qr = q + ((size_t)s * chunk + t) * d + (size_t)h * hd;
#pragma unroll
    for (int i = 0; i < GEN_MAX_SLOTS; ++i) {
        uint32_t c = lane + 32 * i;
        qv[i] = c < hd ? __bfloat162float(qr[c]) * scale_log2 : 0.0f;
        acc[i] = 0.0f;
    }
    const bf16* kb = kc + (size_t)h * hd;
    const bf16* vb = vc + (size_t)h * hd;
    float m = -INFINITY, l = 0.0f;
    for (uint32_t j0 = 0; j0 < total; ++j0) {
        const size_t j = kv_row(paging, s, j0, capacity);
        float part = 0.0f;
#pragma unroll
        for (int i = 0; i < GEN_MAX_SLOTS; ++i) {
            uint32_t c = lane + 32 * i;
            if (c < hd) part = fmaf(qv[i], __bfloat162float(kb[(size_t)j * d + c]), part);
        }
        const float sc = warp_sum_f(part);
        const float m_new = fmaxf(m, sc);
        const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;
        const float corr = ex2(m - m_safe), p = ex2(sc - m_safe);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < GEN_MAX_SLOTS; ++i) {
            uint32_t c = lane + 32 * i;
            if (c < hd) acc[i] = acc[i] * corr + p * __bfloat162float(vb[(size_t)j * d + c]);
        }
        m = m_new;
    }
    bf16* orow = out + ((size_t)s * chunk + t) * d + (size_t)h * hd;
#pragma unroll
    for (int i = 0; i < GEN_MAX_SLOTS; ++i) {
        uint32_t c = lane + 32 * i;
        if (c < hd) orow[c] = __float2bfloat16_rn(acc[i] / l);
    }
}

int launch_attention_generic(const bf16* q, const bf16* k_cache, const bf16* v_cache, bf16* out,
                             uint32_t sessions, uint32_t chunk, uint32_t position,
                             const uint32_t* d_position, uint32_t capacity, uint32_t heads,
                             uint32_t head_dim, cudaStream_t stream, const KvPaging* paging) {
    if (sessions == 0 || chunk == 0) return TNSR_B200_OK;
    if (head_dim > 32 * GEN_MAX_SLOTS) {
        set_thread_error("attention: head_dim above 256 is outside the bf16 kernels");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    uint64_t total = (uint64_t)sessions * heads * chunk;
    if (total > 0x7fffffffull) return TNSR_B200_ERR_UNSUPPORTED;
    const float scale_log2 = (1.0f / sqrtf((float)head_dim)) * 1.4426950408889634f;
    launch_kernel(attention_generic_kernel, dim3((unsigned)ceil_div64(total, 4)), dim3(128), 0, stream, q, k_cache, v_cache, out,
                  (uint32_t)total, chunk, position, d_position, capacity, heads, head_dim, scale_log2, paging ? *paging : KvPaging());
    count_launch();
    return check_launch("attention_generic");
}

// ===========================================================================
// Split-KV decode attention
// ===========================================================================
constexpr uint32_t DA_KS = 16;             // keys per ring stage (8 in the lean form, see launch_decode_attention_ex)
constexpr uint32_t DA_MAX_STAGES = 8;
constexpr uint32_t DA_SMEM_BUDGET = 200 * 1024;
// Lean form: half the shared memory, so that a CTA of another kernel (the projections of the other half of the batch)
// fits on the same SM while this one streams K/V.
constexpr uint32_t DA_KS_LEAN = 8;
constexpr uint32_t DA_SMEM_BUDGET_LEAN = 106 * 1024;
constexpr uint32_t DA_MAX_CTAS = 256;      // upper bound on the grid (one CTA per SM)

// A work item: keys [key0, key0 + nkeys) of one session, all heads.  `slot` is the index of its
// partial result, or DA_DIRECT when the item covers the whole session and writes the output row itself.
constexpr uint32_t DA_DIRECT = 0xffffffffu;
struct DaItem {
    uint32_t session, key0, nkeys, slot;
    uint32_t n_parts, first_slot;  // pieces of the session and the slot of its first piece (for the merge)
    uint32_t pad[2];
};

// Work is split by position in the concatenation of all sessions' live keys, counted in stages of
// DA_KS keys: CTA c owns stages [c * quota, (c + 1) * quota).  Every CTA therefore streams the same
// amount of K/V (+-1 stage) whatever the per-session lengths are, a session is cut only where a CTA
// boundary falls inside it, and there are at most batch + grid items.
//
// Workspace layout (all offsets 256-byte aligned):
//   header    : uint32 total_stages, quota, n_items
//   first     : uint32 [batch]          first partial slot of each session
//   count     : uint32 [batch]          number of pieces of each session (0 for an empty session)
//   done      : uint32 [batch * heads]  partials stored so far per (session, head); zero between launches
//   sstart    : uint32 [batch + 1]      first global stage of each session
//   cta_begin : uint32 [DA_MAX_CTAS + 1] first item of each CTA
//   items     : DaItem [batch + DA_MAX_CTAS]   (32 bytes each)
//   partial   : float  [batch + DA_MAX_CTAS][heads][head_dim + 2]   (numerator, then max, then sum)
struct DaLayout {
    uint64_t first, count, done, sstart, cta_begin, items, partial, bytes;
    uint32_t max_items;
};

static uint64_t align256(uint64_t x) { return (x + 255) & ~255ull; }

static DaLayout da_layout(uint32_t batch, uint32_t heads, uint32_t head_dim) {
    DaLayout L;
    const uint64_t per_item = (uint64_t)heads * (head_dim + 2) * 4;
    L.max_items = batch + DA_MAX_CTAS;
    L.first = 256;
    L.count = align256(L.first + 4ull * batch);
    L.done = align256(L.count + 4ull * batch);
    L.sstart = align256(L.done + 4ull * batch * heads);
    L.cta_begin = align256(L.sstart + 4ull * (batch + 1));
    L.items = align256(L.cta_begin + 4ull * (DA_MAX_CTAS + 1));
    L.partial = align256(L.items + sizeof(DaItem) * (uint64_t)L.max_items);
    L.bytes = L.partial + per_item * L.max_items;
    return L;
}

uint64_t decode_attention_workspace_bytes(uint32_t batch, uint32_t capacity, uint32_t heads, uint32_t head_dim) {
    (void)capacity;  // the scratch depends on the number of sessions, not on how long they may grow
    return da_layout(batch, heads, head_dim).bytes;
}

bool decode_attention_supported(uint32_t heads, uint32_t head_dim) {
    if (!(head_dim == 32 || head_dim == 64 || head_dim == 128)) return false;
    if (heads == 0 || heads > 32) return false;
    uint64_t stage = 2ull * DA_KS * heads * head_dim * 2 + (uint64_t)heads * head_dim * 2;
    return stage * 2 <= DA_SMEM_BUDGET;  // at least a double buffer
}

// ---- plan: one block ---------------------------------------------------------------
// Session b has lengths[b] + extra keys; lengths == nullptr means (d_position ? *d_position : 0) + extra for all.
__global__ void __launch_bounds__(1024)
da_plan_kernel(const uint32_t* __restrict__ lengths, const uint32_t* __restrict__ d_position, uint32_t extra,
               uint32_t batch, uint32_t heads, uint32_t capacity, uint32_t grid, uint32_t ks, uint32_t* __restrict__ header,
               uint32_t* __restrict__ first, uint32_t* __restrict__ count, uint32_t* __restrict__ done,
               uint32_t* __restrict__ sstart, uint32_t* __restrict__ cta_begin, DaItem* __restrict__ items,
               int* __restrict__ d_status) {
    __shared__ uint32_t s_carry, s_warp_tot[32], s_quota, s_total;
    pdl_wait();
    pdl_trigger();
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    auto len_of = [&](uint32_t b) -> uint32_t {
        uint32_t L = (lengths ? lengths[b] : (d_position ? *d_position : 0u)) + extra;
        if (L > capacity) {
            if (d_status) atomicCAS(d_status, DEV_OK, DEV_BAD_LENGTH);
            L = capacity;
        }
        return L;
    };
    // block-wide exclusive scan of f(b) over the sessions, 1024 at a time; returns the total
    auto scan = [&](auto f, uint32_t* out_excl) -> uint32_t {
        if (tid == 0) s_carry = 0;
        __syncthreads();
        for (uint32_t base = 0; base < batch; base += blockDim.x) {
            const uint32_t b = base + tid;
            const uint32_t v = b < batch ? f(b) : 0;
            uint32_t incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= (uint32_t)o) incl += t;
            }
            if (lane == 31) s_warp_tot[warp] = incl;
            __syncthreads();
            uint32_t before = s_carry;
            for (uint32_t w = 0; w < warp; ++w) before += s_warp_tot[w];
            if (b < batch) out_excl[b] = before + incl - v;
            __syncthreads();
            if (tid == blockDim.x - 1) s_carry = before + incl;
            __syncthreads();
        }
        return s_carry;
    };
    // the merge counters must be zero when the attention kernel starts
    for (uint32_t i = tid; i < batch * heads; i += blockDim.x) done[i] = 0;
    // 1. global stage offsets of the sessions
    const uint32_t total = scan([&](uint32_t b) { return (len_of(b) + ks - 1) / ks; }, sstart);
    if (tid == 0) {
        sstart[batch] = total;
        const uint32_t ctas = total < grid ? (total ? total : 1) : grid;
        s_quota = (total + ctas - 1) / ctas;
        if (s_quota == 0) s_quota = 1;
        s_total = total;
    }
    __syncthreads();
    const uint32_t quota = s_quota;
    // 2. pieces per session = CTAs its stage range touches; slots by exclusive scan
    auto pieces = [&](uint32_t b) -> uint32_t {
        const uint32_t s0 = sstart[b], n = (len_of(b) + ks - 1) / ks;
        return n ? (s0 + n - 1) / quota - s0 / quota + 1 : 0;
    };
    const uint32_t n_items = scan(pieces, first);
    // 3. items, one thread per session
    for (uint32_t b = tid; b < batch; b += blockDim.x) {
        const uint32_t L = len_of(b), s0 = sstart[b], n = (L + ks - 1) / ks;
        const uint32_t c = pieces(b), f = first[b];
        count[b] = c;
        const uint32_t cta0 = s0 / quota;
        for (uint32_t j = 0; j < c; ++j) {
            const uint32_t lo = max(s0, (cta0 + j) * quota), hi = min(s0 + n, (cta0 + j + 1) * quota);
            DaItem it;
            it.session = b;
            it.key0 = (lo - s0) * ks;
            it.nkeys = min(L, (hi - s0) * ks) - it.key0;
            it.slot = c == 1 ? DA_DIRECT : f + j;
            it.n_parts = c;
            it.first_slot = f;
            it.pad[0] = it.pad[1] = 0;
            items[f + j] = it;
        }
    }
    __syncthreads();
    // 4. first item of every CTA: the piece that contains global stage c * quota
    for (uint32_t c = tid; c <= grid; c += blockDim.x) {
        const uint32_t g = c * quota;
        uint32_t begin = n_items;
        if (g < s_total) {
            uint32_t lo = 0, hi = batch;  // last session with sstart <= g and at least one stage
            while (hi - lo > 1) {
                const uint32_t mid = (lo + hi) / 2;
                if (sstart[mid] <= g) lo = mid; else hi = mid;
            }
            begin = first[lo] + (g / quota - sstart[lo] / quota);
        }
        cta_begin[c] = begin;
    }
    if (tid == 0) {
        header[0] = s_total;
        header[1] = quota;
        header[2] = n_items;
    }
}

// ---- main kernel ------------------------------------------------------------------
__device__ __forceinline__ uint32_t da_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void da_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(da_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void da_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(da_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void da_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(da_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool da_mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(da_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t da_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool da_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint64_t limit_ns) {
    if (da_mbar_try_wait(bar, parity)) return true;
    const uint64_t start = da_timer_ns();
    for (uint32_t it = 1;; ++it) {
        if (da_mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 0) {
            if (*abort_flag) return false;
            if (da_timer_ns() - start > limit_ns) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}
// Plain (untiled) bulk copy global -> this CTA's shared memory; 16-byte aligned, size % 16 == 0.
__device__ __forceinline__ void da_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(da_smem_u32(dst)), "l"(src), "r"(bytes), "r"(da_smem_u32(bar))
                 : "memory");
}

// The same copy for data that is read exactly once (K/V rows): evict-first in L2, so that a long scan does not push out
// what other kernels keep there.
__device__ __forceinline__ void da_bulk_load_once(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(da_smem_u32(dst)), "l"(src), "r"(bytes), "r"(da_smem_u32(bar)), "l"(policy)
                 : "memory");
}

struct DaStageMeta {
    uint32_t slot;        // partial slot of the item, or DA_DIRECT
    uint32_t nk;          // valid keys in this stage (1..DA_KS)
    uint32_t flags;       // bit 0: first stage of the item, bit 1: last stage
    uint32_t session;
    uint32_t n_parts;     // pieces of this session (for the merge)
    uint32_t first_slot;  // partial slot of the session's first piece
    uint32_t pad[2];
};

struct DaParams {
    const bf16* q;
    const bf16* kc;
    const bf16* vc;
    const uint32_t* first;
    const uint32_t* count;
    uint32_t* done;
    const uint32_t* cta_begin;
    const DaItem* items;
    float* partial;
    bf16* out;
    uint32_t batch, capacity, heads;
    uint32_t stages;
    float scale_log2;
    int* d_status;
    uint64_t wait_limit_ns;   // bound of every mbarrier wait (tnsr_b200_set_wait_limit_ns)
    KvPaging paging;          // page pools instead of per-session slabs (page_rows is a multiple of the stage size)
};

// HD: head width; LPK = HD / 8 lanes share one (key, head) row slice, each lane
// owning 8 consecutive dims (one 16-byte shared-memory load); KPW = 32 / LPK keys
// are processed side by side in a warp.  HPW: heads per consumer warp.
template <int HD, int HPW, int KS>
__global__ void __launch_bounds__(576, 1)
decode_attention_kernel(DaParams P) {
    constexpr uint32_t LPK = HD / 8, KPW = 32 / LPK, ITERS = KS / KPW;
    static_assert(KS % KPW == 0, "stage must hold whole key groups");
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t d = P.heads * HD, row_bytes = d * 2;
    const uint32_t k_bytes = KS * row_bytes;
    const uint32_t stage_bytes = 2 * k_bytes + row_bytes;  // K slab, V slab, q row
    uint8_t* ring = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)P.stages * stage_bytes);
    uint64_t* empty_bar = full_bar + DA_MAX_STAGES;
    DaStageMeta* meta = reinterpret_cast<DaStageMeta*>(empty_bar + DA_MAX_STAGES);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(meta + DA_MAX_STAGES);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t consumers = (blockDim.x >> 5) - 1;  // last warp is the producer
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < P.stages; ++s) { da_mbar_init(full_bar + s, 1); da_mbar_init(empty_bar + s, consumers); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_wait();
    pdl_trigger();
    __syncthreads();
    const uint32_t item_begin = P.cta_begin[blockIdx.x], item_end = P.cta_begin[blockIdx.x + 1];

    if (warp == consumers) {
        // ---------------- producer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            uint64_t once;
            asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(once));
            // item records and the per-session piece counts are fetched one item ahead, so their latency
            // hides behind the copies of the current item
            DaItem nxt = {};
            if (item_begin < item_end) nxt = P.items[item_begin];
            for (uint32_t item = item_begin; ok && item < item_end; ++item) {
                const DaItem it = nxt;
                if (item + 1 < item_end) nxt = P.items[item + 1];
                const uint32_t n_stages = (it.nkeys + KS - 1) / KS;
                for (uint32_t s = 0; s < n_stages; ++s) {
                    if (!da_mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, P.wait_limit_ns)) { ok = false; break; }
                    const uint32_t nk = min((uint32_t)KS, it.nkeys - s * KS);
                    uint8_t* sk = ring + (size_t)stage * stage_bytes;
                    DaStageMeta mt;
                    mt.slot = it.slot;
                    mt.nk = nk;
                    mt.flags = (s == 0 ? 1u : 0u) | (s + 1 == n_stages ? 2u : 0u);
                    mt.session = it.session;
                    mt.n_parts = it.n_parts;
                    mt.first_slot = it.first_slot;
                    meta[stage] = mt;
                    const uint32_t bytes = nk * row_bytes;
                    da_mbar_expect_tx(full_bar + stage, 2 * bytes + (s == 0 ? row_bytes : 0));
                    // a stage never straddles pages: key0 and the page size are multiples of the stage size
                    const size_t base = kv_row(P.paging, it.session, it.key0 + s * KS, P.capacity) * d;
                    da_bulk_load_once(sk, P.kc + base, bytes, full_bar + stage, once);
                    da_bulk_load_once(sk + k_bytes, P.vc + base, bytes, full_bar + stage, once);
                    if (s == 0) da_bulk_load(sk + 2 * k_bytes, P.q + (size_t)it.session * d, row_bytes, full_bar + stage);
                    if (++stage == P.stages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else {
        // ---------------- consumers ----------------
        const uint32_t grp = lane / LPK;       // which of the KPW parallel keys
        const uint32_t sub = lane % LPK;       // which 8-dim slice of the head
        float qf[HPW][8], acc[HPW][8], m[HPW], l[HPW];
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (uint32_t item = item_begin; ok && item < item_end; ++item) {
            for (;;) {
                if (!da_mbar_wait(full_bar + stage, phase, abort_flag, P.wait_limit_ns)) { ok = false; break; }
                const DaStageMeta mt = meta[stage];
                const uint8_t* sk = ring + (size_t)stage * stage_bytes;
                const uint8_t* sv = sk + k_bytes;
                if (mt.flags & 1u) {
                    const uint8_t* sq = sk + 2 * k_bytes;
#pragma unroll
                    for (int hh = 0; hh < HPW; ++hh) {
                        const uint32_t h = warp + hh * consumers;
                        m[hh] = -INFINITY;
                        l[hh] = 0.0f;
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[hh][e] = 0.0f;
                        if (h < P.heads) {
                            const uint4 qq = *reinterpret_cast<const uint4*>(sq + ((size_t)h * HD + sub * 8) * 2);
                            const uint32_t w[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float2 f = bf16x2_to_f32(w[e]);
                                qf[hh][2 * e] = f.x * P.scale_log2;
                                qf[hh][2 * e + 1] = f.y * P.scale_log2;
                            }
                        }
                    }
                }
#pragma unroll
                for (int hh = 0; hh < HPW; ++hh) {
                    const uint32_t h = warp + hh * consumers;
                    if (h >= P.heads) continue;
                    const uint32_t col = (h * HD + sub * 8) * 2;
                    float sc[ITERS];
#pragma unroll
                    for (uint32_t itr = 0; itr < ITERS; ++itr) {
                        const uint32_t key = itr * KPW + grp;
                        const uint4 kk = *reinterpret_cast<const uint4*>(sk + (size_t)key * row_bytes + col);
                        const uint32_t w[4] = {kk.x, kk.y, kk.z, kk.w};
                        float part = 0.0f;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float2 f = bf16x2_to_f32(w[e]);
                            part = fmaf(qf[hh][2 * e], f.x, part);
                            part = fmaf(qf[hh][2 * e + 1], f.y, part);
                        }
#pragma unroll
                        for (uint32_t o = LPK / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                        sc[itr] = key < mt.nk ? part : -INFINITY;
                    }
                    float m_new = m[hh];
#pragma unroll
                    for (uint32_t itr = 0; itr < ITERS; ++itr) m_new = fmaxf(m_new, sc[itr]);
                    const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;
                    const float corr = ex2(m[hh] - m_safe);
                    m[hh] = m_new;
                    float lsum = l[hh] * corr;
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[hh][e] *= corr;
#pragma unroll
                    for (uint32_t itr = 0; itr < ITERS; ++itr) {
                        const uint32_t key = itr * KPW + grp;
                        const float p = ex2(sc[itr] - m_safe);  // 0 for masked keys
                        lsum += p;
                        if (key < mt.nk) {
                            const uint4 vv = *reinterpret_cast<const uint4*>(sv + (size_t)key * row_bytes + col);
                            const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float2 f = bf16x2_to_f32(w[e]);
                                acc[hh][2 * e] = fmaf(p, f.x, acc[hh][2 * e]);
                                acc[hh][2 * e + 1] = fmaf(p, f.y, acc[hh][2 * e + 1]);
                            }
                        }
                    }
                    l[hh] = lsum;
                }
                // the stage's shared memory is no longer needed: hand it back before any finishing work
                __syncwarp();
                if (lane == 0) da_mbar_arrive(empty_bar + stage);
                if (++stage == P.stages) { stage = 0; phase ^= 1; }
                const bool last = (mt.flags & 2u) != 0;
                if (!last) continue;
                // ---- end of the item: fold the KPW side-by-side key groups, then store or merge ----
#pragma unroll
                for (int hh = 0; hh < HPW; ++hh) {
                    const uint32_t h = warp + hh * consumers;
                    if (h >= P.heads) continue;
                    float mm = m[hh];
#pragma unroll
                    for (uint32_t o = LPK; o < 32; o <<= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
                    const float m_safe = (mm == -INFINITY) ? 0.0f : mm;
                    const float f = ex2(m[hh] - m_safe);
                    float ll = l[hh] * f;
                    float a[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) a[e] = acc[hh][e] * f;
#pragma unroll
                    for (uint32_t o = LPK; o < 32; o <<= 1) {
                        ll += __shfl_xor_sync(0xffffffffu, ll, o);
#pragma unroll
                        for (int e = 0; e < 8; ++e) a[e] += __shfl_xor_sync(0xffffffffu, a[e], o);
                    }
                    if (mt.slot == DA_DIRECT) {
                        // the item is the whole session: normalise and write the output row
                        if (grp == 0) {
                            const float inv = 1.0f / ll;
                            bf16* o = P.out + (size_t)mt.session * d + (size_t)h * HD + sub * 8;
                            *reinterpret_cast<uint4*>(o) = make_uint4(pack_bf16x2(a[0] * inv, a[1] * inv), pack_bf16x2(a[2] * inv, a[3] * inv),
                                                                      pack_bf16x2(a[4] * inv, a[5] * inv), pack_bf16x2(a[6] * inv, a[7] * inv));
                        }
                        continue;
                    }
                    if (grp == 0) {
                        float* dst = P.partial + ((size_t)mt.slot * P.heads + h) * (HD + 2);
                        // (HD + 2) floats per head keeps 8-byte alignment only: store as float2
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            *reinterpret_cast<float2*>(dst + sub * 8 + 2 * e) = make_float2(a[2 * e], a[2 * e + 1]);
                        if (sub == 0) *reinterpret_cast<float2*>(dst + HD) = make_float2(mm, ll);
                        __threadfence();
                    }
                    __syncwarp();
                    // whoever stores the last partial of (session, head) merges them
                    const uint32_t n_parts = mt.n_parts;
                    uint32_t seen = 0;
                    if (lane == 0) seen = atomicAdd(P.done + (size_t)mt.session * P.heads + h, 1u);
                    seen = __shfl_sync(0xffffffffu, seen, 0);
                    if (seen + 1 == n_parts) {
                        __threadfence();
                        constexpr int DPL = HD / 32;  // output dims per lane
                        const float* base = P.partial + ((size_t)mt.first_slot * P.heads + h) * (HD + 2);
                        const size_t step = (size_t)P.heads * (HD + 2);
                        float mx = -INFINITY;
                        float lt = 0.0f, o[DPL];
#pragma unroll
                        for (int e = 0; e < DPL; ++e) o[e] = 0.0f;
                        constexpr uint32_t FEW = 4;
                        if (n_parts <= FEW) {
                            // the usual case (a session cut in two to four pieces): every value of every piece is
                            // requested before the first is used, one L2 round trip instead of two dependent ones
                            float pm[FEW], pl[FEW], pn[FEW][DPL];
#pragma unroll
                            for (uint32_t i = 0; i < FEW; ++i) {
                                const float* pp = base + i * step;
                                const bool have = i < n_parts;
                                pm[i] = have ? __ldcg(pp + HD) : -INFINITY;
                                pl[i] = have ? __ldcg(pp + HD + 1) : 0.0f;
#pragma unroll
                                for (int e = 0; e < DPL; ++e) pn[i][e] = have ? __ldcg(pp + lane * DPL + e) : 0.0f;
                            }
#pragma unroll
                            for (uint32_t i = 0; i < FEW; ++i) mx = fmaxf(mx, pm[i]);
                            const float ms = (mx == -INFINITY) ? 0.0f : mx;
#pragma unroll
                            for (uint32_t i = 0; i < FEW; ++i) {
                                if (i < n_parts) {
                                    const float w = ex2(pm[i] - ms);
                                    lt = fmaf(pl[i], w, lt);
#pragma unroll
                                    for (int e = 0; e < DPL; ++e) o[e] = fmaf(pn[i][e], w, o[e]);
                                }
                            }
                        } else {
                            for (uint32_t i = 0; i < n_parts; ++i) mx = fmaxf(mx, __ldcg(base + i * step + HD));
                            const float ms = (mx == -INFINITY) ? 0.0f : mx;
                            for (uint32_t i = 0; i < n_parts; ++i) {
                                const float* pp = base + i * step;
                                const float w = ex2(__ldcg(pp + HD) - ms);
                                lt = fmaf(__ldcg(pp + HD + 1), w, lt);
#pragma unroll
                                for (int e = 0; e < DPL; ++e) o[e] = fmaf(__ldcg(pp + lane * DPL + e), w, o[e]);
                            }
                        }
                        const float inv = 1.0f / lt;
                        bf16* orow = P.out + (size_t)mt.session * d + (size_t)h * HD + lane * DPL;
#pragma unroll
                        for (int e = 0; e < DPL; ++e) orow[e] = __float2bfloat16_rn(o[e] * inv);
                        if (lane == 0) P.done[(size_t)mt.session * P.heads + h] = 0;
                    }
                }
                break;
            }
        }
        // sessions without any live key own no item: their output row is zero
        for (uint32_t b = blockIdx.x * consumers + warp; b < P.batch; b += gridDim.x * consumers) {
            if (P.count[b] != 0) continue;
            for (uint32_t c = lane * 8; c < d; c += 32 * 8)
                *reinterpret_cast<uint4*>(P.out + (size_t)b * d + c) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    __syncthreads();
    if (*abort_flag) {
        const uint64_t start = da_timer_ns();
        while (da_timer_ns() - start < 200000ull) __nanosleep(1000);
        if (threadIdx.x == 0 && P.d_status) atomicCAS(P.d_status, DEV_OK, DEV_TIMEOUT);
        __syncthreads();
    }
}

template <int HD, int HPW, int KS>
static int launch_da_t(const DaParams& P, uint32_t threads, size_t smem, uint32_t grid, cudaStream_t stream) {
    static size_t configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || configured[dev] < smem) {
        if (cudaFuncSetAttribute(decode_attention_kernel<HD, HPW, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return check_launch("decode_attention attribute");
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    KernelTimer* timer = t_attention_timer;
    cudaEvent_t start = nullptr, stop = nullptr;
    if (timer) {
        if (timer->used + 2 > timer->events.size()) {
            for (int i = 0; i < 2; ++i) {
                cudaEvent_t e;
                if (cudaEventCreate(&e) != cudaSuccess) return check_launch("decode_attention event");
                timer->events.push_back(e);
            }
        }
        start = timer->events[timer->used];
        stop = timer->events[timer->used + 1];
        timer->used += 2;
        cudaEventRecord(start, stream);
    }
    launch_kernel(decode_attention_kernel<HD, HPW, KS>, dim3(grid), dim3(threads), smem, stream, P);
    if (timer) cudaEventRecord(stop, stream);
    count_launch();
    return check_launch("decode_attention");
}

static int da_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// lengths may be nullptr: then every session holds (d_position ? *d_position : 0) + extra keys.
int launch_decode_attention_ex(const bf16* q, const bf16* k_cache, const bf16* v_cache, const uint32_t* d_lengths,
                               const uint32_t* d_position, uint32_t extra, bf16* out, void* workspace,
                               uint64_t workspace_bytes, uint32_t batch, uint32_t capacity, uint32_t heads,
                               uint32_t head_dim, bool plan, int* d_status, cudaStream_t stream, bool lean,
                               const KvPaging* paging) {
    if (batch == 0) return TNSR_B200_OK;
    if (!decode_attention_supported(heads, head_dim)) {
        set_thread_error("decode attention: head_dim must be 32, 64 or 128 and heads <= 32");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
         reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(workspace)) % 16) {
        set_thread_error("decode attention: pointers must be 16-byte aligned");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    const DaLayout L = da_layout(batch, heads, head_dim);
    if (L.bytes > workspace_bytes) {
        set_thread_error("decode attention: workspace too small");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    uint32_t* header = reinterpret_cast<uint32_t*>(ws);
    uint32_t* first = reinterpret_cast<uint32_t*>(ws + L.first);
    uint32_t* count = reinterpret_cast<uint32_t*>(ws + L.count);
    uint32_t* done = reinterpret_cast<uint32_t*>(ws + L.done);
    uint32_t* sstart = reinterpret_cast<uint32_t*>(ws + L.sstart);
    uint32_t* cta_begin = reinterpret_cast<uint32_t*>(ws + L.cta_begin);
    DaItem* items = reinterpret_cast<DaItem*>(ws + L.items);
    float* partial = reinterpret_cast<float*>(ws + L.partial);
    uint32_t grid = (uint32_t)da_sm_count();
    if (grid > DA_MAX_CTAS) grid = DA_MAX_CTAS;
    // keys per ring stage: 8 in the lean form if two such stages (the least a ring needs) fit its budget
    const uint32_t d = heads * head_dim, row_bytes = d * 2;
    if (lean && 2 * (2 * DA_KS_LEAN * row_bytes + row_bytes) > DA_SMEM_BUDGET_LEAN) lean = false;
    const uint32_t ks = lean ? DA_KS_LEAN : DA_KS;
    if (!d_lengths) {
        // Every session has the same length (the decoder's own steps).  If the grid divides the batch, or the batch
        // divides the grid, the equal key ranges of the CTAs line up with the sessions: whole sessions per CTA (no
        // partial results, no merge) or an even split of every session.  That is worth more than the SMs left idle:
        // 256 sessions on 128 CTAs take 81 us per launch against 86 us on 148 (measured), as long as at least three
        // quarters of the SMs stay in use.
        uint32_t aligned = 0;
        if (batch >= grid) {
            for (uint32_t g = grid; g >= 1 && 4 * g >= 3 * grid; --g)
                if (batch % g == 0) { aligned = g; break; }
        } else if (batch > 0) {
            aligned = batch * (grid / batch);
            if (4 * aligned < 3 * grid) aligned = 0;
        }
        if (aligned) grid = aligned;
    }
    if (plan) {
        launch_kernel(da_plan_kernel, dim3(1), dim3(1024), 0, stream, d_lengths, d_position, extra, batch, heads, capacity, grid,
                      ks, header, first, count, done, sstart, cta_begin, items, d_status);
        count_launch();
        int rc = check_launch("decode_attention plan");
        if (rc) return rc;
    }
    const uint32_t stage_bytes = 2 * ks * row_bytes + row_bytes;
    uint32_t stages = (lean ? DA_SMEM_BUDGET_LEAN : DA_SMEM_BUDGET) / stage_bytes;
    if (stages > DA_MAX_STAGES) stages = DA_MAX_STAGES;
    const size_t smem = (size_t)stages * stage_bytes + 2 * DA_MAX_STAGES * 8 + DA_MAX_STAGES * sizeof(DaStageMeta) + 16;
    const uint32_t hpw = heads > 16 ? 2 : 1;
    const uint32_t consumers = ceil_div(heads, hpw);
    DaParams P;
    P.q = q; P.kc = k_cache; P.vc = v_cache;
    P.first = first; P.count = count; P.done = done; P.cta_begin = cta_begin; P.items = items; P.partial = partial;
    P.out = out;
    P.batch = batch; P.capacity = capacity; P.heads = heads; P.stages = stages;
    P.scale_log2 = (1.0f / sqrtf((float)head_dim)) * 1.4426950408889634f;
    P.d_status = d_status;
    P.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
    if (paging && paging->table) {
        if (paging->page_rows == 0 || paging->page_rows % DA_KS != 0) {
            set_thread_error("decode attention: the page size must be a multiple of 16 rows");
            return TNSR_B200_ERR_INVALID_ARGUMENT;
        }
        P.paging = *paging;
    }
    const uint32_t threads = (consumers + 1) * 32;
    if (lean) {
        if (hpw == 1) {
            return head_dim == 32 ? launch_da_t<32, 1, DA_KS_LEAN>(P, threads, smem, grid, stream)
                 : head_dim == 64 ? launch_da_t<64, 1, DA_KS_LEAN>(P, threads, smem, grid, stream)
                                  : launch_da_t<128, 1, DA_KS_LEAN>(P, threads, smem, grid, stream);
        }
        return head_dim == 32 ? launch_da_t<32, 2, DA_KS_LEAN>(P, threads, smem, grid, stream)
             : head_dim == 64 ? launch_da_t<64, 2, DA_KS_LEAN>(P, threads, smem, grid, stream)
                              : launch_da_t<128, 2, DA_KS_LEAN>(P, threads, smem, grid, stream);
    }
    if (hpw == 1) {
        return head_dim == 32 ? launch_da_t<32, 1, DA_KS>(P, threads, smem, grid, stream)
             : head_dim == 64 ? launch_da_t<64, 1, DA_KS>(P, threads, smem, grid, stream)
                              : launch_da_t<128, 1, DA_KS>(P, threads, smem, grid, stream);
    }
    return head_dim == 32 ? launch_da_t<32, 2, DA_KS>(P, threads, smem, grid, stream)
         : head_dim == 64 ? launch_da_t<64, 2, DA_KS>(P, threads, smem, grid, stream)
                          : launch_da_t<128, 2, DA_KS>(P, threads, smem, grid, stream);
}

int launch_decode_attention(const bf16* q, const bf16* k_cache, const bf16* v_cache, const uint32_t* d_lengths,
                            bf16* out, void* workspace, uint64_t workspace_bytes, uint32_t batch,
                            uint32_t capacity, uint32_t heads, uint32_t head_dim, int* d_status,
                            cudaStream_t stream) {
    return launch_decode_attention_ex(q, k_cache, v_cache, d_lengths, nullptr, 0, out, workspace, workspace_bytes, batch,
                                      capacity, heads, head_dim, true, d_status, stream, false);
}

}  // namespace tb
