// tnsr_b200_decode_attention_static: the split-KV decode attention for callers
// that cannot hand the library a workspace because they cannot allocate one.
//
// Who that is: a process whose device memory is budgeted completely at start-up
// (a serving runtime that gives the whole GPU to its own pool, an embedding in
// another engine that forbids allocation after initialisation) or a latency-bound
// loop for which cudaMalloc is off limits because it synchronises the device and
// can fail when memory is fragmented.  Such a caller still owns its inputs and
// outputs (q, the K/V cache, lengths, out) but has nowhere to put the item list
// and the per-slab partial results the kernel needs between its two passes.
//
// What this file does about it: the scratch lives in a file-scope device array of
// fixed size that the CUDA module carries, so it exists on every GPU that loads
// the library, from load until the process exits, and nothing is allocated or
// freed by the call -- no cudaMalloc, no cudaFree, no library routine that
// allocates.
//
// Rules that follow from sharing one array:
//  * The array's name is only a host-side handle.  Its device address is looked up
//    once per device with cudaGetSymbolAddress (below, under a lock, with that
//    device current) and that address is what the kernels receive.  The first
//    call on a device performs this look-up; make that first call before any
//    stream capture begins.  The address is remembered per device ordinal for the
//    life of the process, so it is tied to the device's primary context: after
//    cudaDeviceReset, or under another context on the same ordinal, it is stale and
//    this entry point must not be used.
//  * Shapes whose workspace (tnsr_b200_decode_attention_workspace) exceeds the array are rejected with
//    TNSR_B200_ERR_UNSUPPORTED and a message that states both sizes.
//  * Every call reuses the same bytes and finds the previous call's contents in
//    them.  The words that must start at zero (item count, slab size, the
//    kernel's status word) are cleared on the caller's stream at the start of
//    each call; everything else is written before it is read.
//  * Two calls that overlap on the GPU -- different streams, or two host threads
//    -- race on the array and corrupt each other.  Serialise them (one stream),
//    or use tnsr_b200_decode_attention with separate workspaces.
#include <mutex>

#include "common.cuh"

using namespace tb;

namespace {

constexpr uint64_t kStaticScratchBytes = TNSR_B200_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// One-time set-up for the current device: resolve the device address of the array.
int scratch_for_current_device(void** out) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) {
        set_thread_error(std::string("decode_attention_static: cudaGetDevice: ") + cudaGetErrorString(e));
        return TNSR_B200_ERR_CUDA;
    }
    if (device < 0 || device >= kMaxDevices) {
        set_thread_error("decode_attention_static: device ordinal beyond the table of scratch addresses");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_address[device]) {
        void* address = nullptr;
        e = cudaGetSymbolAddress(&address, g_static_scratch);
        if (e != cudaSuccess || !address) {
            cudaGetLastError();
            set_thread_error(std::string("decode_attention_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
            return TNSR_B200_ERR_CUDA;
        }
        g_scratch_address[device] = address;
    }
    *out = g_scratch_address[device];
    return TNSR_B200_OK;
}

}  // namespace

extern "C" int tnsr_b200_decode_attention_static(const void* q, const void* k_cache, const void* v_cache,
                                                 const uint32_t* lengths, void* out, uint32_t batch, uint32_t capacity,
                                                 uint32_t heads, uint32_t head_dim, int* d_status, void* stream) {
    if (!q || !k_cache || !v_cache || !lengths || !out) {
        set_thread_error("decode_attention_static: null pointer");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    if (!decode_attention_supported(heads, head_dim)) {
        set_thread_error("decode_attention_static: head_dim must be 32, 64 or 128 and heads <= 32");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    const uint64_t need = decode_attention_workspace_bytes(batch, capacity, heads, head_dim);
    if (need > kStaticScratchBytes) {
        set_thread_error("decode_attention_static: this batch needs " + std::to_string(need) +
                         " bytes of scratch but the built-in array holds " + std::to_string(kStaticScratchBytes) +
                         "; use tnsr_b200_decode_attention with a caller-provided workspace");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    void* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc != TNSR_B200_OK) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // the previous call's header (item count, slab, status) must not be seen by this one
    cudaError_t e = cudaMemsetAsync(scratch, 0, 256, st);
    if (e == cudaSuccess && d_status) e = cudaMemsetAsync(d_status, 0, sizeof(int), st);
    if (e != cudaSuccess) {
        set_thread_error(std::string("decode_attention_static: cudaMemsetAsync: ") + cudaGetErrorString(e));
        return TNSR_B200_ERR_CUDA;
    }
    int* status = d_status ? d_status : reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(scratch) + 64);
    return launch_decode_attention((const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, lengths, (bf16*)out, scratch,
                                   kStaticScratchBytes, batch, capacity, heads, head_dim, status, st);
}
