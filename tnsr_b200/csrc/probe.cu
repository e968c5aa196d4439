// Measurement aid: how fast can one CTA per SM stream a buffer with bulk async copies and do nothing
// else?  This is the ceiling the decode-attention kernel's K/V ring can reach on a given GPU, the
// denominator that is fairer to it than a device-to-device copy (which also writes).
#include "common.cuh"

using namespace tb;

namespace {

__device__ __forceinline__ uint32_t pr_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool pr_wait(uint64_t* bar, uint32_t parity) {
    // bounded: ~2^26 polls, then give up
    for (uint32_t it = 0; it < (1u << 26); ++it) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                     : "=r"(ok) : "r"(pr_smem(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// Every CTA streams its own contiguous range through a ring of `stages` x `stage_bytes`, two copies per
// stage (like the K and V halves); three consumer warps touch each stage and hand it back.
__global__ void __launch_bounds__(128)
stream_read_kernel(const uint8_t* __restrict__ p, uint64_t bytes_per_cta, uint32_t stage_bytes, uint32_t stages, uint32_t* sink) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * stage_bytes);
    uint64_t* empty = full + 8;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pr_smem(full + s)), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pr_smem(empty + s)), "r"(3));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const uint8_t* base = p + (size_t)blockIdx.x * bytes_per_cta;
    const uint32_t n = (uint32_t)(bytes_per_cta / stage_bytes);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, half = stage_bytes / 2;
    if (warp == 3) {
        if (lane == 0) {
            uint32_t st = 0, ph = 0;
            for (uint32_t i = 0; i < n; ++i) {
                if (!pr_wait(empty + st, ph ^ 1)) break;
                uint8_t* dst = smem + (size_t)st * stage_bytes;
                const uint8_t* src = base + (size_t)i * stage_bytes;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pr_smem(full + st)), "r"(stage_bytes) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(pr_smem(dst)), "l"(src), "r"(half), "r"(pr_smem(full + st)) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(pr_smem(dst + half)), "l"(src + half), "r"(half), "r"(pr_smem(full + st)) : "memory");
                if (++st == stages) { st = 0; ph ^= 1; }
            }
        }
    } else {
        uint32_t st = 0, ph = 0, acc = 0;
        for (uint32_t i = 0; i < n; ++i) {
            if (!pr_wait(full + st, ph)) break;
            acc ^= *reinterpret_cast<const uint32_t*>(smem + (size_t)st * stage_bytes + threadIdx.x * 4);
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pr_smem(empty + st)) : "memory");
            if (++st == stages) { st = 0; ph ^= 1; }
        }
        if (acc == 0x12345678u && sink) sink[0] = acc;
    }
}

}  // namespace

extern "C" int tnsr_b200_stream_read_probe(const void* buffer, uint64_t bytes, uint32_t stage_bytes, uint32_t stages,
                                           uint64_t* bytes_read, void* stream) {
    if (!buffer || !bytes_read || stages < 2 || stages > 8 || stage_bytes < 1024 || stage_bytes % 32 != 0 ||
        (reinterpret_cast<uintptr_t>(buffer) & 15) != 0) {
        set_thread_error("stream_read_probe: need a 16-byte aligned buffer, 2..8 stages and a stage size that is a multiple of 32");
        return TNSR_B200_ERR_INVALID_ARGUMENT;
    }
    const size_t smem = (size_t)stages * stage_bytes + 256;
    if (smem > 220 * 1024) {
        set_thread_error("stream_read_probe: stages x stage_bytes exceeds shared memory");
        return TNSR_B200_ERR_UNSUPPORTED;
    }
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    const uint64_t per_cta = bytes / sms / stage_bytes * stage_bytes;
    *bytes_read = per_cta * sms;
    if (per_cta == 0) return TNSR_B200_OK;
    if (cudaFuncSetAttribute(stream_read_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return check_launch("stream_read_probe attribute");
    stream_read_kernel<<<sms, 128, smem, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const uint8_t*>(buffer), per_cta,
                                                                                   stage_bytes, stages, nullptr);
    count_launch();
    return check_launch("stream_read_probe");
}
