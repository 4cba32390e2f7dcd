// shim.cu: process state, error reporting, resident FP8 tensors and the weight quantiser of libb200moe.so.
// Mirrors the reference session's conventions (src/omega_gpu_session.h:27-29, src/omega_gpu_fp8_api.c:69-80,
// :433-482): one process-wide lock, a process-wide last-error text, a latch after an uncertain failure.
#include <stdarg.h>
#include <math.h>
#include <stdlib.h>
#include "internal.h"

namespace b200 {

State &st() { static State s; return s; }

void set_error(const char *fmt, ...) {
    va_list ap; va_start(ap, fmt);
    vsnprintf(st().err, sizeof st().err, fmt, ap);
    va_end(ap);
}

uint64_t now_ns() { timespec t; clock_gettime(CLOCK_MONOTONIC, &t); return (uint64_t)t.tv_sec * 1000000000ull + (uint64_t)t.tv_nsec; }

bool cuda_ok(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return true;
    set_error("%s: %s", what, cudaGetErrorString(e));
    // anything but a plain argument/allocation refusal leaves the context in an unknown state
    if (e != cudaErrorInvalidValue && e != cudaErrorMemoryAllocation && e != cudaErrorNoDevice && e != cudaErrorInsufficientDriver &&
        e != cudaErrorInvalidDevice) st().latched = true;
    (void)cudaGetLastError();
    return false;
}

bool dev_open() {
    State &g = st();
    if (g.latched) { if (!g.err[0]) set_error("process latched after a CUDA failure"); return false; }
    if (g.opened) return cudaSetDevice(g.device) == cudaSuccess;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) { set_error("no CUDA device: %s", e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e)); (void)cudaGetLastError(); return false; }
    int dev = 0;
    if (const char *v = getenv("B200MOE_DEVICE")) dev = atoi(v);
    else if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
    if (!cuda_ok(cudaSetDevice(dev), "cudaSetDevice")) return false;
    cudaDeviceProp p;
    if (!cuda_ok(cudaGetDeviceProperties(&p, dev), "cudaGetDeviceProperties")) return false;
    if (p.major != 10) { set_error("device %d is sm_%d%d; this library holds sm_100a code only", dev, p.major, p.minor); return false; }
    g.device = dev; g.sm_count = p.multiProcessorCount;
    snprintf(g.chip, sizeof g.chip, "%s", p.name);
    if (!cuda_ok(cudaStreamCreateWithFlags(&g.stream, cudaStreamNonBlocking), "cudaStreamCreate")) return false;
    if (!cuda_ok(cudaEventCreate(&g.ev0), "cudaEventCreate") || !cuda_ok(cudaEventCreate(&g.ev1), "cudaEventCreate")) return false;
    g.opened = true;
    return true;
}

void *stage(int i, size_t bytes) {
    State &g = st();
    if (bytes == 0) bytes = 16;
    if (g.stage_bytes[i] >= bytes) return g.stage[i];
    if (g.stage[i]) { cudaFree(g.stage[i]); g.stage[i] = nullptr; g.stage_bytes[i] = 0; }
    size_t want = bytes + (bytes >> 2) + 256;
    if (!cuda_ok(cudaMalloc(&g.stage[i], want), "cudaMalloc(staging)")) return nullptr;
    g.stage_bytes[i] = want;
    return g.stage[i];
}

__global__ void fill_f32_kernel(float *p, size_t n, float v) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}
void launch_fill_f32(float *p, size_t n, float v, cudaStream_t s) {
    if (!n) return;
    size_t blocks = (n + 255) / 256; if (blocks > 1184) blocks = 1184;
    fill_f32_kernel<<<(unsigned)blocks, 256, 0, s>>>(p, n, v);
}

// ---------------------------------------------------------------- e4m3 on the device (shared by the quantiser)
// Round to nearest even onto the e4m3 grid, saturating at 448, never the NaN code (the reference's host
// rule, src/omega_gpu_fp8_api.c:702-721). Hardware cvt.rn.satfinite.e4m3x2.f32 implements exactly this.
__device__ __forceinline__ uint8_t e4m3_encode_dev(float v) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(v));
    return (uint8_t)(r & 0xff);
}

// One CTA per 128 x 128 block: amax over |w|, scale = amax/448 rounded up to bf16, codes = encode(w / scale).
__global__ void __launch_bounds__(256) quantize_block_kernel(const uint16_t *__restrict__ w, uint8_t *__restrict__ w8,
                                                             uint16_t *__restrict__ scale, uint32_t k, uint32_t kb, int *bad) {
    __shared__ float red[8];
    __shared__ float s_scale;
    const uint32_t bn = blockIdx.y, bk = blockIdx.x, tid = threadIdx.x;
    const size_t base = (size_t)bn * 128 * k + (size_t)bk * 128;
    float amax = 0.0f; int nonfinite = 0;
    for (uint32_t i = tid; i < 128 * 128; i += 256) {
        const uint32_t r = i >> 7, c = i & 127;
        const float f = __uint_as_float((uint32_t)(w[base + (size_t)r * k + c] & 0x7fffu) << 16);
        if (!(f <= 3.0e38f)) nonfinite = 1;
        amax = fmaxf(amax, f);
    }
    if (nonfinite) atomicExch(bad, 1);
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((tid & 31) == 0) red[tid >> 5] = amax;
    __syncthreads();
    if (tid == 0) {
        float m = red[0];
        for (int i = 1; i < 8; i++) m = fmaxf(m, red[i]);
        uint16_t sb = 0x3f80u;
        if (m > 0.0f) { const uint32_t b = __float_as_uint(__fdiv_rn(m, 448.0f)); sb = (uint16_t)((b >> 16) + ((b & 0xffffu) ? 1u : 0u)); }
        scale[(size_t)bn * kb + bk] = sb;
        s_scale = __uint_as_float((uint32_t)sb << 16);
    }
    __syncthreads();
    const float sc = s_scale;
    for (uint32_t i = tid; i < 128 * 128; i += 256) {
        const uint32_t r = i >> 7, c = i & 127;
        const float f = __uint_as_float((uint32_t)w[base + (size_t)r * k + c] << 16);
        w8[base + (size_t)r * k + c] = e4m3_encode_dev(__fdiv_rn(f, sc));
    }
}

// counts e4m3 NaN codes and non-finite bf16 scales on the device (upload_dev's refusals)
__global__ void scan_codes_kernel(const uint8_t *w, size_t wbytes, const uint16_t *sc, size_t scount, float *sf, unsigned long long *first_nan, int *bad_scale) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < wbytes; i += (size_t)gridDim.x * blockDim.x)
        if ((w[i] & 0x7fu) == 0x7fu) atomicMin(first_nan, (unsigned long long)i);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < scount; i += (size_t)gridDim.x * blockDim.x) {
        const float f = __uint_as_float((uint32_t)sc[i] << 16);
        if (!(fabsf(f) <= 3.0e38f)) *bad_scale = 1;
        sf[i] = f;
    }
}

}  // namespace b200
using namespace b200;

extern "C" {

const char *omega_gpu_fp8_rc_name(int rc) {
    switch (rc) {
    case OMEGA_GPU_FP8_OK: return "OK";
    case OMEGA_GPU_FP8_BAD_ARGS: return "BAD_ARGS";
    case OMEGA_GPU_FP8_TOO_LARGE: return "TOO_LARGE";
    case OMEGA_GPU_FP8_CODEGEN_FAIL: return "CODEGEN_FAIL";
    case OMEGA_GPU_FP8_CHIP_FAIL: return "CHIP_FAIL";
    case OMEGA_GPU_FP8_NAN_WEIGHT: return "NAN_WEIGHT";
    default: return "UNKNOWN";
    }
}
const char *omega_gpu_fp8_last_error(void) { return st().err; }
const char *omega_gpu_fp8gemm_rc_name(int rc) { return rc == OMEGA_GPU_FP8_NAN_WEIGHT ? "UNKNOWN" : omega_gpu_fp8_rc_name(rc); }
const char *omega_gpu_fp8gemm_last_error(void) { return st().err; }
void omega_gpu_fp8_cache_clear(void) {}
void omega_gpu_fp8gemm_cache_clear(void) {}
void omega_gpu_fp8_seal(int on) { Lock l; st().sealed = on ? 1 : 0; }
void omega_gpu_fp8_set_cta_budget(uint32_t ctas) { Lock l; st().cta_budget = ctas; }
void omega_gpu_fp8_test_set_mutant(int mutant) { Lock l; st().gemv_mutant = mutant; }
void omega_gpu_fp8gemm_test_set_mutant(int mutant) { Lock l; st().gemm_mutant = mutant; }

static int prepare_k(uint32_t k) {
    if (k == 0 || k % OMEGA_FP8_BLOCK) return OMEGA_GPU_FP8_BAD_ARGS;
    if (k > OMEGA_FP8_MAX_K) return OMEGA_GPU_FP8_TOO_LARGE;
    Lock l;
    return dev_open() ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}
int omega_gpu_fp8_prepare(uint32_t k) { return prepare_k(k); }
int omega_gpu_fp8gemm_prepare(uint32_t k) { return prepare_k(k); }

// ---- host helpers (src/omega_gpu_fp8_pack.c:15-35, :59-76)
float omega_fp8_e4m3_ref(uint8_t b) {
    const int e = (b >> 3) & 15, m = b & 7;
    const float sgn = (b & 0x80) ? -1.0f : 1.0f;
    if (e == 15 && m == 7) return NAN;
    return e == 0 ? sgn * (float)m * 0.001953125f : sgn * (1.0f + (float)m * 0.125f) * ldexpf(1.0f, e - 7);
}
int omega_fp8_e4m3_is_nan(uint8_t b) { return (b & 0x7fu) == 0x7fu; }
size_t omega_fp8_pack_scan_nan(const uint8_t *w, size_t count, size_t *first) {
    size_t n = 0;
    for (size_t i = 0; i < count; i++) if ((w[i] & 0x7fu) == 0x7fu) { if (!n && first) *first = i; n++; }
    return n;
}
void omega_fp8_gemv_oracle(const uint8_t *w, const uint16_t *scale_bf16, uint32_t n, uint32_t k, const float *x, double *y, double *yscale) {
    const uint32_t kb = k / OMEGA_FP8_BLOCK;
    for (uint32_t r = 0; r < n; r++) {
        double acc = 0.0, mag = 0.0;
        for (uint32_t c = 0; c < k; c++) {
            uint32_t sb = (uint32_t)scale_bf16[(size_t)(r / OMEGA_FP8_BLOCK) * kb + c / OMEGA_FP8_BLOCK] << 16; float s; memcpy(&s, &sb, 4);
            const double p = (double)omega_fp8_e4m3_ref(w[(size_t)r * k + c]) * (double)x[c] * (double)s;
            acc += p; mag += fabs(p);
        }
        y[r] = acc; if (yscale) yscale[r] = mag;
    }
}
uint8_t omega_gpu_fp8_e4m3_rne(float v) {
    uint32_t u; memcpy(&u, &v, 4);
    const uint8_t sgn = (uint8_t)((u >> 24) & 0x80u);
    const float a = fabsf(v);
    if (!(a < 448.0f)) return (uint8_t)(sgn | 0x7eu);
    int e = a > 0.0f ? ilogbf(a) : -6;
    if (e < -6) e = -6;
    float r = nearbyintf(ldexpf(a, 3 - e));
    if (r >= 16.0f) { r = 8.0f; e++; }
    const uint32_t code = (e == -6 && r < 8.0f) ? (uint32_t)r : (((uint32_t)(e + 7) << 3) | ((uint32_t)r - 8u));
    return (uint8_t)(sgn | (code > 0x7eu ? 0x7eu : code));
}

// ---- resident tensors (src/omega_gpu_fp8_api.c:433-482, :679-684)
int omega_gpu_fp8_tensor_upload(uint32_t experts, uint32_t n, uint32_t k, const uint8_t *w, const uint16_t *scale, OmegaGpuFp8Tensor **out) {
    if (out) *out = nullptr;
    if (!w || !scale || !out || experts == 0 || n == 0 || k == 0 || n % OMEGA_FP8_BLOCK || k % OMEGA_FP8_BLOCK) return OMEGA_GPU_FP8_BAD_ARGS;
    if (k > OMEGA_FP8_MAX_K) return OMEGA_GPU_FP8_TOO_LARGE;
    const size_t wbytes = (size_t)experts * n * k, scount = (size_t)experts * (n / OMEGA_FP8_BLOCK) * (k / OMEGA_FP8_BLOCK);
    Lock l;
    size_t first = 0;
    if (omega_fp8_pack_scan_nan(w, wbytes, &first)) { set_error("fp8 upload: e4m3 NaN code at byte %zu", first); return OMEGA_GPU_FP8_NAN_WEIGHT; }
    float *sf = (float *)malloc(scount * sizeof(float));
    if (!sf) return OMEGA_GPU_FP8_BAD_ARGS;
    for (size_t i = 0; i < scount; i++) {
        uint32_t b = (uint32_t)scale[i] << 16; memcpy(&sf[i], &b, 4);
        if (!(fabsf(sf[i]) <= 3.0e38f)) { free(sf); set_error("fp8 upload: NaN, inf or overflowing scale"); return OMEGA_GPU_FP8_BAD_ARGS; }
    }
    if (!dev_open()) { free(sf); return OMEGA_GPU_FP8_CHIP_FAIL; }
    OmegaGpuFp8Tensor *t = (OmegaGpuFp8Tensor *)calloc(1, sizeof *t);
    if (!t) { free(sf); return OMEGA_GPU_FP8_BAD_ARGS; }
    t->experts = experts; t->n = n; t->k = k; t->device = st().device;
    bool ok = cuda_ok(cudaMalloc(&t->w, wbytes), "cudaMalloc(weights)") && cuda_ok(cudaMalloc(&t->s, scount * 4), "cudaMalloc(scales)") &&
              cuda_ok(cudaMemcpy(t->w, w, wbytes, cudaMemcpyHostToDevice), "copy weights") &&
              cuda_ok(cudaMemcpy(t->s, sf, scount * 4, cudaMemcpyHostToDevice), "copy scales");
    free(sf);
    if (!ok) { if (t->w) cudaFree(t->w); if (t->s) cudaFree(t->s); free(t); return OMEGA_GPU_FP8_CHIP_FAIL; }
    *out = t;
    return OMEGA_GPU_FP8_OK;
}
void omega_gpu_fp8_tensor_free(OmegaGpuFp8Tensor *t) {
    if (!t) return;
    Lock l;
    if (t->w) cudaFree(t->w);
    if (t->s) cudaFree(t->s);
    free(t);
}
void omega_gpu_fp8_tensor_shape(const OmegaGpuFp8Tensor *t, uint32_t *experts, uint32_t *n, uint32_t *k) {
    if (experts) *experts = t ? t->experts : 0;
    if (n) *n = t ? t->n : 0;
    if (k) *k = t ? t->k : 0;
}
int omega_gpu_fp8_tensor_entry(const OmegaGpuFp8Tensor *t, uint32_t expert, uint64_t *w_va, uint64_t *s_va) {
    if (!t || !t->w || expert >= t->experts || !w_va || !s_va) return OMEGA_GPU_FP8_BAD_ARGS;
    *w_va = (uint64_t)(uintptr_t)t->w + (uint64_t)expert * t->n * t->k;
    *s_va = (uint64_t)(uintptr_t)t->s + (uint64_t)expert * (t->n / OMEGA_FP8_BLOCK) * (t->k / OMEGA_FP8_BLOCK) * 4u;
    return OMEGA_GPU_FP8_OK;
}

int omega_gpu_fp8_tensor_upload_dev(uint32_t experts, uint32_t n, uint32_t k, uint64_t w_va, uint64_t scale_va, OmegaGpuFp8Tensor **out) {
    if (out) *out = nullptr;
    if (!w_va || !scale_va || !out || experts == 0 || n == 0 || k == 0 || n % OMEGA_FP8_BLOCK || k % OMEGA_FP8_BLOCK) return OMEGA_GPU_FP8_BAD_ARGS;
    if (k > OMEGA_FP8_MAX_K) return OMEGA_GPU_FP8_TOO_LARGE;
    const size_t wbytes = (size_t)experts * n * k, scount = (size_t)experts * (n / OMEGA_FP8_BLOCK) * (k / OMEGA_FP8_BLOCK);
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    OmegaGpuFp8Tensor *t = (OmegaGpuFp8Tensor *)calloc(1, sizeof *t);
    if (!t) return OMEGA_GPU_FP8_BAD_ARGS;
    t->experts = experts; t->n = n; t->k = k; t->device = st().device;
    unsigned long long *flags = (unsigned long long *)stage(7, 16);
    unsigned long long h[2] = {~0ull, 0};
    cudaStream_t s = st().stream;
    bool ok = flags && cuda_ok(cudaMalloc(&t->w, wbytes), "cudaMalloc(weights)") && cuda_ok(cudaMalloc(&t->s, scount * 4), "cudaMalloc(scales)") &&
              cuda_ok(cudaDeviceSynchronize(), "sync before upload") &&   // the caller's producer kernels may run on another stream
              cuda_ok(cudaMemcpyAsync(flags, h, 16, cudaMemcpyHostToDevice, s), "copy flags");
    if (ok) {
        scan_codes_kernel<<<1184, 256, 0, s>>>((const uint8_t *)(uintptr_t)w_va, wbytes, (const uint16_t *)(uintptr_t)scale_va, scount, t->s, flags, (int *)(flags + 1));
        ok = cuda_ok(cudaGetLastError(), "scan launch") &&
             cuda_ok(cudaMemcpyAsync(t->w, (const void *)(uintptr_t)w_va, wbytes, cudaMemcpyDeviceToDevice, s), "copy weights") &&
             cuda_ok(cudaMemcpyAsync(h, flags, 16, cudaMemcpyDeviceToHost, s), "copy flags") && cuda_ok(cudaStreamSynchronize(s), "upload");
    }
    int rc = ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
    if (ok && h[0] != ~0ull) { set_error("fp8 upload: e4m3 NaN code at byte %llu", h[0]); rc = OMEGA_GPU_FP8_NAN_WEIGHT; }
    else if (ok && (int)h[1]) { set_error("fp8 upload: NaN, inf or overflowing scale"); rc = OMEGA_GPU_FP8_BAD_ARGS; }
    if (rc != OMEGA_GPU_FP8_OK) { if (t->w) cudaFree(t->w); if (t->s) cudaFree(t->s); free(t); return rc; }
    *out = t;
    return OMEGA_GPU_FP8_OK;
}

int omega_gpu_fp8_quantize_bf16_dev(uint32_t n, uint32_t k, uint64_t w_va, uint64_t w8_va, uint64_t scale_va) {
    if (!w_va || !w8_va || !scale_va || n == 0 || k == 0 || n % OMEGA_FP8_BLOCK || k % OMEGA_FP8_BLOCK) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    int *bad = (int *)stage(7, 16); int hbad = 0;
    cudaStream_t s = st().stream;
    bool ok = bad && cuda_ok(cudaDeviceSynchronize(), "sync before quantize") && cuda_ok(cudaMemsetAsync(bad, 0, 4, s), "memset");
    if (ok) {
        quantize_block_kernel<<<dim3(k / 128, n / 128), 256, 0, s>>>((const uint16_t *)(uintptr_t)w_va, (uint8_t *)(uintptr_t)w8_va, (uint16_t *)(uintptr_t)scale_va, k, k / 128, bad);
        ok = cuda_ok(cudaGetLastError(), "quantize launch") && cuda_ok(cudaMemcpyAsync(&hbad, bad, 4, cudaMemcpyDeviceToHost, s), "copy flag") &&
             cuda_ok(cudaStreamSynchronize(s), "quantize");
    }
    if (!ok) return OMEGA_GPU_FP8_CHIP_FAIL;
    if (hbad) { set_error("fp8 quantize: inf or NaN weight"); return OMEGA_GPU_FP8_BAD_ARGS; }
    return OMEGA_GPU_FP8_OK;
}

// ---- weight quantiser on the GPU (semantics of src/omega_gpu_fp8_api.c:723-754)
int omega_gpu_fp8_quantize_bf16(uint32_t n, uint32_t k, const uint16_t *w, uint8_t *w8, uint16_t *scale_inv_bf16) {
    if (!w || !w8 || !scale_inv_bf16 || n == 0 || k == 0 || n % OMEGA_FP8_BLOCK || k % OMEGA_FP8_BLOCK) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    const size_t cnt = (size_t)n * k, sc = (size_t)(n / 128) * (k / 128);
    uint16_t *dw = (uint16_t *)stage(0, cnt * 2); uint8_t *d8 = (uint8_t *)stage(1, cnt); uint16_t *ds = (uint16_t *)stage(2, sc * 2 + 16);
    if (!dw || !d8 || !ds) return OMEGA_GPU_FP8_CHIP_FAIL;
    int *bad = (int *)((uint8_t *)ds + ((sc * 2 + 7) & ~(size_t)7));
    cudaStream_t s = st().stream;
    int hbad = 0;
    bool ok = cuda_ok(cudaMemcpyAsync(dw, w, cnt * 2, cudaMemcpyHostToDevice, s), "copy weights") &&
              cuda_ok(cudaMemsetAsync(bad, 0, 4, s), "memset");
    if (ok) {
        quantize_block_kernel<<<dim3(k / 128, n / 128), 256, 0, s>>>(dw, d8, ds, k, k / 128, bad);
        ok = cuda_ok(cudaGetLastError(), "quantize launch") &&
             cuda_ok(cudaMemcpyAsync(&hbad, bad, 4, cudaMemcpyDeviceToHost, s), "copy flag") &&
             cuda_ok(cudaStreamSynchronize(s), "quantize");
    }
    if (!ok) return OMEGA_GPU_FP8_CHIP_FAIL;
    if (hbad) { set_error("fp8 quantize: inf or NaN weight"); return OMEGA_GPU_FP8_BAD_ARGS; }
    ok = cuda_ok(cudaMemcpy(w8, d8, cnt, cudaMemcpyDeviceToHost), "copy codes") && cuda_ok(cudaMemcpy(scale_inv_bf16, ds, sc * 2, cudaMemcpyDeviceToHost), "copy scales");
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

}  // extern "C"
