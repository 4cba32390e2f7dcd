// w4_gemm.cu: signed int4 group-scaled weights (two per byte along K, low nibble = even column; fp16 scale per 32
// columns) times bf16 activations, f32 accumulation, bf16 output. The reference has no integer-W4 arithmetic
// (docs/models/QUANT.md:62 of the reference: "integer W4 refuses"), so this follows the benchmark definition only:
// y[m][r] = sum over groups g of scale[r][g] * sum_{c in g} x[m][c] * q[r][c].
// Weight-streaming kernel: a warp owns RW output rows; lane l owns K groups l, l+32, ... (16 contiguous bytes each,
// 512 contiguous bytes per warp load); the activation panel sits in shared memory as bf16.
#include <cuda_fp16.h>
#include <stdlib.h>
#include "internal.h"

struct OmegaGpuW4Tensor { uint32_t n, k; uint8_t *w; uint16_t *s; };

namespace b200 {

constexpr int W4_RW = 2;    // output rows per warp task
constexpr int W4_MT = 16;   // activation rows per pass

__global__ void __launch_bounds__(256) w4_gemm_kernel(uint32_t m, uint32_t n, uint32_t k, const uint8_t *__restrict__ w, const uint16_t *__restrict__ sc,
                                                      const uint16_t *__restrict__ x, uint16_t *__restrict__ y16, float *__restrict__ y32) {
    extern __shared__ uint16_t xs[];   // [W4_MT][k] bf16
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, groups = k / 32u;
    for (uint32_t m0 = 0; m0 < m; m0 += W4_MT) {
        const uint32_t mt = min((uint32_t)W4_MT, m - m0);
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < W4_MT * k / 8; i += 256) {
            const uint32_t r = i / (k / 8), c8 = i - r * (k / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < mt) v = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)(m0 + r) * k) + c8);
            reinterpret_cast<uint4 *>(xs)[i] = v;
        }
        __syncthreads();
        for (uint32_t rb = (blockIdx.x * 8 + warp) * W4_RW; rb < n; rb += gridDim.x * 8 * W4_RW) {
            float acc[W4_RW][W4_MT];
#pragma unroll
            for (int j = 0; j < W4_RW; j++)
#pragma unroll
                for (int mm = 0; mm < W4_MT; mm++) acc[j][mm] = 0.0f;
            for (uint32_t g = lane; g < groups; g += 32) {
                float q[W4_RW][32]; float s[W4_RW];
#pragma unroll
                for (int j = 0; j < W4_RW; j++) {
                    const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(w + ((size_t)(rb + j) * k) / 2) + g);
                    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int i = 0; i < 32; i++) q[j][i] = (float)(((int32_t)(u[i >> 3] << (28 - 4 * (i & 7)))) >> 28);
                    s[j] = __half2float(__ushort_as_half(__ldg(sc + (size_t)(rb + j) * groups + g)));
                }
#pragma unroll 4
                for (int mm = 0; mm < W4_MT; mm++) {
                    float part[W4_RW];
#pragma unroll
                    for (int j = 0; j < W4_RW; j++) part[j] = 0.0f;
                    const uint4 *xp = reinterpret_cast<const uint4 *>(xs + (size_t)mm * k + g * 32u);
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const uint4 xv = xp[c];
                        const uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float x0 = __uint_as_float(xu[e] << 16), x1 = __uint_as_float(xu[e] & 0xffff0000u);
#pragma unroll
                            for (int j = 0; j < W4_RW; j++) { part[j] = fmaf(x0, q[j][c * 8 + e * 2], part[j]); part[j] = fmaf(x1, q[j][c * 8 + e * 2 + 1], part[j]); }
                        }
                    }
#pragma unroll
                    for (int j = 0; j < W4_RW; j++) acc[j][mm] = fmaf(part[j], s[j], acc[j][mm]);
                }
            }
#pragma unroll
            for (int j = 0; j < W4_RW; j++)
#pragma unroll
                for (int mm = 0; mm < W4_MT; mm++) {
                    float v = acc[j][mm];
                    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (lane == 0 && (uint32_t)mm < mt) {
                        const size_t at = (size_t)(m0 + mm) * n + rb + j;
                        if (y32) y32[at] = v;
                        if (y16) { const uint32_t b = __float_as_uint(v); y16[at] = (uint16_t)(((b & 0x7fffffffu) > 0x7f800000u) ? ((b >> 16) | 0x40u) : ((b + 0x7fffu + ((b >> 16) & 1u)) >> 16)); }
                    }
                }
        }
    }
}

}  // namespace b200
using namespace b200;

extern "C" {

int omega_gpu_w4_upload(uint32_t n, uint32_t k, const uint8_t *packed, const uint16_t *scale_f16, OmegaGpuW4Tensor **out) {
    if (out) *out = nullptr;
    if (!out || !packed || !scale_f16 || !n || !k || k % 32 || n % W4_RW) return OMEGA_GPU_FP8_BAD_ARGS;
    if ((size_t)W4_MT * k * 2 > 200 * 1024) return OMEGA_GPU_FP8_TOO_LARGE;
    for (size_t i = 0; i < (size_t)n * (k / 32); i++) if ((scale_f16[i] & 0x7c00u) == 0x7c00u) { set_error("w4 upload: NaN or inf scale"); return OMEGA_GPU_FP8_BAD_ARGS; }
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    OmegaGpuW4Tensor *t = (OmegaGpuW4Tensor *)calloc(1, sizeof *t);
    if (!t) return OMEGA_GPU_FP8_BAD_ARGS;
    t->n = n; t->k = k;
    const size_t wb = (size_t)n * k / 2, sb = (size_t)n * (k / 32) * 2;
    const bool ok = cuda_ok(cudaMalloc(&t->w, wb), "cudaMalloc(w4)") && cuda_ok(cudaMalloc(&t->s, sb), "cudaMalloc(w4 scales)") &&
                    cuda_ok(cudaMemcpy(t->w, packed, wb, cudaMemcpyHostToDevice), "copy w4") && cuda_ok(cudaMemcpy(t->s, scale_f16, sb, cudaMemcpyHostToDevice), "copy w4 scales");
    if (!ok) { if (t->w) cudaFree(t->w); if (t->s) cudaFree(t->s); free(t); return OMEGA_GPU_FP8_CHIP_FAIL; }
    *out = t;
    return OMEGA_GPU_FP8_OK;
}
void omega_gpu_w4_free(OmegaGpuW4Tensor *t) {
    if (!t) return;
    Lock l;
    if (t->w) cudaFree(t->w);
    if (t->s) cudaFree(t->s);
    free(t);
}
static cudaError_t w4_launch(const OmegaGpuW4Tensor *t, uint32_t m, const uint16_t *dx, uint16_t *d16, float *d32, cudaStream_t s) {
    const size_t smem = (size_t)W4_MT * t->k * 2;
    static bool attr = false;
    if (!attr) { const cudaError_t e = cudaFuncSetAttribute(w4_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); if (e != cudaSuccess) return e; attr = true; }
    uint32_t grid = (t->n / W4_RW + 7) / 8; const uint32_t cap = (uint32_t)(st().sm_count ? st().sm_count : 148); if (grid > cap) grid = cap;
    w4_gemm_kernel<<<grid, 256, smem, s>>>(m, t->n, t->k, t->w, t->s, dx, d16, d32);
    return cudaGetLastError();
}
int omega_gpu_w4_gemm_async(const OmegaGpuW4Tensor *t, uint32_t m, uint64_t x_bf16_va, uint64_t y_bf16_va, uint64_t y_f32_va, void *stream) {
    if (!t || !m || !x_bf16_va || (!y_bf16_va && !y_f32_va)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    return cuda_ok(w4_launch(t, m, (const uint16_t *)(uintptr_t)x_bf16_va, (uint16_t *)(uintptr_t)y_bf16_va, (float *)(uintptr_t)y_f32_va, (cudaStream_t)stream), "w4 launch")
               ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}
int omega_gpu_w4_gemm_bf16(const OmegaGpuW4Tensor *t, uint32_t m, const uint16_t *x, uint16_t *y16, float *y32) {
    if (!t || !m || !x || (!y16 && !y32)) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    const size_t xb = (size_t)m * t->k * 2, yb = (size_t)m * t->n;
    uint16_t *dx = (uint16_t *)stage(0, xb), *d16 = (uint16_t *)stage(1, yb * 2); float *d32 = (float *)stage(2, yb * 4);
    if (!dx || !d16 || !d32) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = st().stream;
    bool ok = cuda_ok(cudaMemcpyAsync(dx, x, xb, cudaMemcpyHostToDevice, s), "copy x") && cuda_ok(w4_launch(t, m, dx, d16, d32, s), "w4 launch");
    if (ok && y16) ok = cuda_ok(cudaMemcpyAsync(y16, d16, yb * 2, cudaMemcpyDeviceToHost, s), "copy y");
    if (ok && y32) ok = cuda_ok(cudaMemcpyAsync(y32, d32, yb * 4, cudaMemcpyDeviceToHost, s), "copy y");
    ok = ok && cuda_ok(cudaStreamSynchronize(s), "w4 gemm");
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

}  // extern "C"
