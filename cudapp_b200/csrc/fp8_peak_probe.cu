// fp8_peak_probe.cu: measures what the FP8 tensor pipe of this GPU sustains, as the denominator for "fraction of FP8 peak".
// Every SM runs one CTA whose elected thread issues `iters` x 4 tcgen05.mma.kind::f8f6f4 instructions (M 128, N 256, K 32, the
// largest single-CTA shape) on operands that stay in shared memory, accumulating into TMEM; nothing is loaded or stored while
// the clock runs. The figure is an upper bound for any kernel that also has to feed the operands.
#include "internal.h"
#include "mma_common.cuh"

namespace b200 {

constexpr uint32_t PROBE_SMEM = A_TILE + 256 * 128 + 1024;   // one 128 x 128-byte A tile, one 256 x 128-byte B tile

__global__ void __launch_bounds__(128, 1) fp8_peak_probe_kernel(uint32_t iters, uint32_t *err) {
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    extern __shared__ uint8_t dyn_smem[];
    __shared__ __align__(8) uint64_t s_bar;
    __shared__ uint32_t s_tmem, s_abort;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t smem_base = (smem_u32(dyn_smem) + 1023u) & ~1023u;
    uint8_t *gen = dyn_smem + (smem_base - smem_u32(dyn_smem));
    for (uint32_t i = threadIdx.x; i < (A_TILE + 256u * 128u) / 4u; i += 128u) reinterpret_cast<uint32_t *>(gen)[i] = ((i * 2654435761u) ^ (i >> 3) * 40503u) & 0x7e7e7e7eu;   // varied finite e4m3 codes (never 0x7F / 0xFF)
    if (threadIdx.x == 0) { s_abort = 0; mbar_init(smem_u32(&s_bar), 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the operands were written with ordinary stores
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    if (warp == 0 && lane == 0) {
        const uint64_t da = umma_desc(smem_base), db = umma_desc(smem_base + A_TILE);
        for (uint32_t it = 0; it < iters; it++) {
#pragma unroll
            for (uint32_t ks = 0; ks < 4; ks++) tc_mma_f8(tmem, da + 2u * ks, db + 2u * ks, IDESC, (it | ks) ? 1u : 0u);
        }
        tc_commit(smem_u32(&s_bar));
        // bounded: the MMAs above take iters x 4 x 128 clocks; each try below blocks for a while before it reports "not yet"
        bool done = false;
        for (uint32_t i = 0; i < (1u << 24) && !done; i++) done = mbar_try(smem_u32(&s_bar), 0u);
        if (!done) atomicCAS(err, 0u, 21u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
}

}  // namespace b200
using namespace b200;

extern "C" int omega_gpu_fp8_tensor_peak(uint32_t iters, uint32_t repeats, float *tflops, float *ms_out) {
    if (!tflops || !iters || iters > (1u << 20) || !repeats || repeats > 64) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = st().stream;
    uint32_t *err = nullptr; cudaEvent_t e0, e1;
    if (!cuda_ok(cudaFuncSetAttribute(fp8_peak_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PROBE_SMEM), "probe attribute") ||
        !cuda_ok(cudaMalloc(&err, 4), "cudaMalloc(probe)") || !cuda_ok(cudaMemsetAsync(err, 0, 4, s), "memset")) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    const int sms = st().sm_count ? st().sm_count : 148;
    fp8_peak_probe_kernel<<<sms, 128, PROBE_SMEM, s>>>(iters / 8u + 1u, err);   // warm-up
    float best = 0.0f; bool ok = true;
    for (uint32_t r = 0; r < repeats && ok; r++) {
        cudaEventRecord(e0, s);
        fp8_peak_probe_kernel<<<sms, 128, PROBE_SMEM, s>>>(iters, err);
        cudaEventRecord(e1, s);
        ok = cuda_ok(cudaStreamSynchronize(s), "fp8 peak probe");
        float ms = 0; if (ok) ok = cuda_ok(cudaEventElapsedTime(&ms, e0, e1), "event time");
        if (ok && (best == 0.0f || ms < best)) best = ms;
    }
    uint32_t code = 0;
    ok = ok && cuda_ok(cudaMemcpy(&code, err, 4, cudaMemcpyDeviceToHost), "copy probe status");
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaFree(err);
    if (!ok) return OMEGA_GPU_FP8_CHIP_FAIL;
    if (code) { set_error("fp8 peak probe: a bounded wait ran out (code %u)", code); return OMEGA_GPU_FP8_CHIP_FAIL; }
    *tflops = (float)((double)sms * iters * 4.0 * 2.0 * 128.0 * 256.0 * 32.0 / (best * 1e-3) / 1e12);
    if (ms_out) *ms_out = best;
    return OMEGA_GPU_FP8_OK;
}
