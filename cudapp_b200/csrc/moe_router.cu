// moe_router.cu: the router front half in one launch for any number of residual rows: RMSNorm of the row with the layer's norm
// weight, router logits against the bf16 gate matrix, softmax top-k with the reference's tie rule, weights.
//
// What it computes is the reference's one-launch router in its ROWS form (src/omega_blackwell_codegen_router.h:15-33: phase 1
// RMSNorm and x' = xn * out_scale, phase 2 logits, phase 3 selection; API src/omega_gpu_router_api.h:74-110; double oracle
// tests/gpu_router_test.c:62-79). The reference's group tables (directory entries of the selected experts) are not produced: this
// library's routing plan reads the ids themselves.
//
// One CTA of 8 warps per row. The gate matrix (experts x hidden bf16, 512 KB at 128 x 2048) is shared by all rows and stays in L2;
// a warp streams whole expert rows with 16-byte loads against the normalised row held in shared memory.
#include "internal.h"
#include "route_common.cuh"

struct OmegaGpuMoeRouter {
    uint32_t experts, hidden;
    uint16_t *gate;      // device [experts][hidden] bf16
    float *norm_w;       // device [hidden]
    uint16_t *shared_gate;   // device [hidden] bf16 or null: the shared expert's gate vector (weight of the extra slot = sigmoid(gate . xn))
};

namespace b200 {

__device__ __forceinline__ uint32_t bf16_rne_bits(float f) {
    const uint32_t b = __float_as_uint(f);
    return ((b & 0x7fffffffu) > 0x7f800000u) ? ((b >> 16) | 0x40u) : ((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
}

// dynamic shared: xn f32 [ROUTER_TOK][hidden] | logits f32 [ROUTER_TOK][experts]
// A CTA takes ROUTER_TOK consecutive rows: every gate word it loads is multiplied into all of them (the gate matrix is read once per ROUTER_TOK rows
// instead of once per row), each row keeping its own accumulation chain in the order a one-row CTA would use, so the values do not depend on the grouping.
constexpr uint32_t ROUTER_TOK = 1;   // measured: 4 rows per CTA (64 CTAs for 256 rows) is slower, the kernel is bound by load latency, not by L2 traffic
__global__ void __launch_bounds__(256) router_rows_kernel(uint32_t rows, uint32_t hidden, uint32_t experts, uint32_t topk, int norm, float eps, float out_scale,
                                                          const float *__restrict__ x, size_t x_stride, const float *__restrict__ norm_w,
                                                          const uint16_t *__restrict__ gate, float *__restrict__ xn_out, uint16_t *__restrict__ xn16_out,
                                                          float *__restrict__ logits_out, uint32_t *__restrict__ ids, float *__restrict__ wts,
                                                          uint32_t slots, const uint16_t *__restrict__ shared_gate) {
    extern __shared__ __align__(16) float sm[];
    float *xn = sm, *lg = sm + (size_t)ROUTER_TOK * hidden;
    __shared__ double red[8];
    __shared__ float s_r;
    const uint32_t row0 = blockIdx.x * ROUTER_TOK, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t ntok = rows - row0 < ROUTER_TOK ? rows - row0 : ROUTER_TOK;
    // ---- phase 1, row by row: RMSNorm (sum of squares in double, one f32 factor, then (x * r) * w)
    for (uint32_t k = 0; k < ROUTER_TOK; k++) {
        float *xk = xn + (size_t)k * hidden;
        if (k >= ntok) { for (uint32_t i = tid * 4u; i < hidden; i += 1024u) *reinterpret_cast<float4 *>(xk + i) = make_float4(0.0f, 0.0f, 0.0f, 0.0f); continue; }
        const uint32_t row = row0 + k;
        const float *xr = x + (size_t)row * x_stride;
        double ss = 0.0;
        for (uint32_t i = tid * 4u; i < hidden; i += 1024u) {
            const float4 v = *reinterpret_cast<const float4 *>(xr + i);
            ss += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
        }
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (tid == 0) { double t = 0.0; for (int i = 0; i < 8; i++) t += red[i]; s_r = (float)(1.0 / sqrt(t / (double)hidden + (double)eps)); }
        __syncthreads();
        const float r = s_r;
        for (uint32_t i = tid * 4u; i < hidden; i += 1024u) {
            const float4 v = *reinterpret_cast<const float4 *>(xr + i), w = __ldg(reinterpret_cast<const float4 *>(norm_w + i));
            const float4 o = make_float4(v.x * r * w.x, v.y * r * w.y, v.z * r * w.z, v.w * r * w.w);
            *reinterpret_cast<float4 *>(xk + i) = o;
            if (xn_out) *reinterpret_cast<float4 *>(xn_out + (size_t)row * hidden + i) = make_float4(o.x * out_scale, o.y * out_scale, o.z * out_scale, o.w * out_scale);
            if (xn16_out) {
                uint2 pk; pk.x = bf16_rne_bits(o.x) | (bf16_rne_bits(o.y) << 16); pk.y = bf16_rne_bits(o.z) | (bf16_rne_bits(o.w) << 16);
                *reinterpret_cast<uint2 *>(xn16_out + (size_t)row * hidden + i) = pk;
            }
        }
    }
    __syncthreads();
    // ---- phase 2: logits; warp w takes experts w, w + 8, ...; a lane multiplies 8 consecutive bf16 weights per 16-byte load into every row's sum
    const uint32_t words = hidden / 8u;
    // two experts per pass (e and e + 8): twice the loads in flight per lane, each sum still in its own order
    for (uint32_t e = warp; e < experts; e += 16u) {
        const bool two = e + 8u < experts;
        const uint4 *g0 = reinterpret_cast<const uint4 *>(gate + (size_t)e * hidden), *g1 = reinterpret_cast<const uint4 *>(gate + (size_t)(two ? e + 8u : e) * hidden);
        float acc0[ROUTER_TOK], acc1[ROUTER_TOK];
#pragma unroll
        for (uint32_t k = 0; k < ROUTER_TOK; k++) { acc0[k] = 0.0f; acc1[k] = 0.0f; }
#pragma unroll 4
        for (uint32_t c = lane; c < words; c += 32u) {
            const uint4 u = __ldg(g0 + c), v = __ldg(g1 + c);
#pragma unroll
            for (uint32_t k = 0; k < ROUTER_TOK; k++) {
                const float *xk = xn + (size_t)k * hidden + c * 8u;
                const float4 a = *reinterpret_cast<const float4 *>(xk), b = *reinterpret_cast<const float4 *>(xk + 4u);
                float s0 = acc0[k], s1 = acc1[k];
                s0 = fmaf(__uint_as_float(u.x << 16), a.x, s0); s1 = fmaf(__uint_as_float(v.x << 16), a.x, s1);
                s0 = fmaf(__uint_as_float(u.x & 0xffff0000u), a.y, s0); s1 = fmaf(__uint_as_float(v.x & 0xffff0000u), a.y, s1);
                s0 = fmaf(__uint_as_float(u.y << 16), a.z, s0); s1 = fmaf(__uint_as_float(v.y << 16), a.z, s1);
                s0 = fmaf(__uint_as_float(u.y & 0xffff0000u), a.w, s0); s1 = fmaf(__uint_as_float(v.y & 0xffff0000u), a.w, s1);
                s0 = fmaf(__uint_as_float(u.z << 16), b.x, s0); s1 = fmaf(__uint_as_float(v.z << 16), b.x, s1);
                s0 = fmaf(__uint_as_float(u.z & 0xffff0000u), b.y, s0); s1 = fmaf(__uint_as_float(v.z & 0xffff0000u), b.y, s1);
                s0 = fmaf(__uint_as_float(u.w << 16), b.z, s0); s1 = fmaf(__uint_as_float(v.w << 16), b.z, s1);
                s0 = fmaf(__uint_as_float(u.w & 0xffff0000u), b.w, s0); s1 = fmaf(__uint_as_float(v.w & 0xffff0000u), b.w, s1);
                acc0[k] = s0; acc1[k] = s1;
            }
        }
#pragma unroll
        for (uint32_t k = 0; k < ROUTER_TOK; k++) {
            float s0 = acc0[k], s1 = acc1[k];
            for (int o = 16; o; o >>= 1) { s0 += __shfl_xor_sync(0xffffffffu, s0, o); s1 += __shfl_xor_sync(0xffffffffu, s1, o); }
            if (lane == 0 && k < ntok) {
                lg[(size_t)k * experts + e] = s0; if (logits_out) logits_out[(size_t)(row0 + k) * experts + e] = s0;
                if (two) { lg[(size_t)k * experts + e + 8u] = s1; if (logits_out) logits_out[(size_t)(row0 + k) * experts + e + 8u] = s1; }
            }
        }
    }
    __syncthreads();
    // ---- phase 3: selection and weights, one warp per row
    if (warp < ntok) warp_topk(lg + (size_t)warp * experts, experts, topk, norm, ids + (size_t)(row0 + warp) * slots, wts + (size_t)(row0 + warp) * slots);
    // ---- the shared expert's slot (slots = topk + 1): id = experts; weight = sigmoid(shared gate . xn), the reference's ninth group
    //      (src/omega_gpu_q36_graph.h:20), or 1 when the layer has no such gate; warps 4 .. 7, one per row
    if (slots > topk && warp >= ROUTER_TOK && warp - ROUTER_TOK < ntok) {
        const uint32_t k = warp - ROUTER_TOK, row = row0 + k;
        float acc = 0.0f;
        if (shared_gate) {
            for (uint32_t c = lane; c < hidden; c += 32u) acc = fmaf(__uint_as_float((uint32_t)shared_gate[c] << 16), xn[(size_t)k * hidden + c], acc);
            for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        }
        if (lane == 0) { ids[(size_t)row * slots + topk] = experts; wts[(size_t)row * slots + topk] = shared_gate ? __fdiv_rn(1.0f, 1.0f + expf(-acc)) : 1.0f; }
    }
}

// stream-ordered launch for callers inside the library (the layer stack): xn16 = bf16(RMSNorm(x) * norm weight), ids, weights
cudaError_t launch_router_rows(const OmegaGpuMoeRouter *r, uint32_t rows, const float *x, float eps, int norm_topk, uint32_t topk, uint16_t *xn16, uint32_t *ids, float *wts, cudaStream_t s, uint32_t slots) {
    const size_t smem = (size_t)ROUTER_TOK * ((size_t)r->hidden + r->experts) * 4;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(router_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    router_rows_kernel<<<(rows + ROUTER_TOK - 1) / ROUTER_TOK, 256, smem, s>>>(rows, r->hidden, r->experts, topk, norm_topk, eps, 1.0f, x, r->hidden, r->norm_w, r->gate, nullptr, xn16, nullptr, ids, wts, slots ? slots : topk, r->shared_gate);
    return cudaGetLastError();
}
void router_dims(const OmegaGpuMoeRouter *r, uint32_t *experts, uint32_t *hidden) { *experts = r->experts; *hidden = r->hidden; }

}  // namespace b200
using namespace b200;

extern "C" {

int omega_gpu_moe_router_create(uint32_t experts, uint32_t hidden, const uint16_t *gate_bf16, const float *norm_w, OmegaGpuMoeRouter **out) {
    if (out) *out = nullptr;
    if (!out || !gate_bf16 || !norm_w || !experts || experts > 1024 || !hidden || hidden % 8 || hidden > 8192) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    OmegaGpuMoeRouter *r = new OmegaGpuMoeRouter();
    r->experts = experts; r->hidden = hidden; r->gate = nullptr; r->norm_w = nullptr; r->shared_gate = nullptr;
    const size_t gb = (size_t)experts * hidden * 2, nb = (size_t)hidden * 4;
    const bool ok = cuda_ok(cudaMalloc(&r->gate, gb), "cudaMalloc(router gate)") && cuda_ok(cudaMalloc(&r->norm_w, nb), "cudaMalloc(router norm)") &&
                    cuda_ok(cudaMemcpy(r->gate, gate_bf16, gb, cudaMemcpyHostToDevice), "copy router gate") &&
                    cuda_ok(cudaMemcpy(r->norm_w, norm_w, nb, cudaMemcpyHostToDevice), "copy router norm");
    if (!ok) { if (r->gate) cudaFree(r->gate); if (r->norm_w) cudaFree(r->norm_w); delete r; return OMEGA_GPU_FP8_CHIP_FAIL; }
    *out = r;
    return OMEGA_GPU_FP8_OK;
}

void omega_gpu_moe_router_free(OmegaGpuMoeRouter *r) {
    if (!r) return;
    Lock l;
    if (r->gate) cudaFree(r->gate);
    if (r->norm_w) cudaFree(r->norm_w);
    if (r->shared_gate) cudaFree(r->shared_gate);
    delete r;
}

int omega_gpu_moe_router_set_shared_gate(OmegaGpuMoeRouter *r, const uint16_t *gate_bf16) {
    if (!r || !gate_bf16) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    if (!r->shared_gate && !cuda_ok(cudaMalloc(&r->shared_gate, (size_t)r->hidden * 2), "cudaMalloc(shared gate)")) return OMEGA_GPU_FP8_CHIP_FAIL;
    return cuda_ok(cudaMemcpy(r->shared_gate, gate_bf16, (size_t)r->hidden * 2, cudaMemcpyHostToDevice), "copy shared gate") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_router_rows_async(OmegaGpuMoeRouter *r, uint32_t rows, uint64_t x_va, uint32_t x_stride_bytes, float eps, int norm_topk, float out_scale,
                                    uint32_t topk, uint64_t xn_va, uint64_t xn_bf16_va, uint64_t logits_va, uint64_t ids_va, uint64_t wts_va, void *stream) {
    if (!r || !rows || !x_va || !ids_va || !wts_va || !topk || topk > 32 || topk > r->experts) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!x_stride_bytes) x_stride_bytes = r->hidden * 4u;
    if (x_stride_bytes % 16u || x_stride_bytes < r->hidden * 4u || (x_va & 15u)) { set_error("router: residual rows must be 16-byte aligned f32 rows of at least `hidden` values"); return OMEGA_GPU_FP8_BAD_ARGS; }
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    const size_t smem = (size_t)ROUTER_TOK * ((size_t)r->hidden + r->experts) * 4;
    if (smem > 48 * 1024) {
        if (!cuda_ok(cudaFuncSetAttribute(router_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "router attribute")) return OMEGA_GPU_FP8_CHIP_FAIL;
    }
    router_rows_kernel<<<(rows + ROUTER_TOK - 1) / ROUTER_TOK, 256, smem, (cudaStream_t)stream>>>(rows, r->hidden, r->experts, topk, norm_topk, eps, out_scale, (const float *)(uintptr_t)x_va, x_stride_bytes / 4u,
                                                                  r->norm_w, r->gate, (float *)(uintptr_t)xn_va, (uint16_t *)(uintptr_t)xn_bf16_va, (float *)(uintptr_t)logits_va,
                                                                  (uint32_t *)(uintptr_t)ids_va, (float *)(uintptr_t)wts_va, topk + (r->shared_gate ? 1u : 0u), r->shared_gate);
    return cuda_ok(cudaGetLastError(), "router launch") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_router_f32(OmegaGpuMoeRouter *r, uint32_t rows, const float *x, float eps, int norm_topk, float out_scale, uint32_t topk,
                             float *xn, float *logits, uint32_t *ids, float *wts) {
    if (!r || !rows || !x || !ids || !wts || !topk || topk > 32 || topk > r->experts) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    const size_t xb = (size_t)rows * r->hidden * 4, lb = (size_t)rows * r->experts * 4, kb = (size_t)rows * (topk + (r->shared_gate ? 1u : 0u)) * 4;   // ids / wts rows: topk (+ 1 with a shared gate)
    float *dx = (float *)stage(0, xb), *dxn = (float *)stage(1, xb), *dl = (float *)stage(2, lb + 2 * kb);
    if (!dx || !dxn || !dl) return OMEGA_GPU_FP8_CHIP_FAIL;
    uint32_t *di = (uint32_t *)(dl + (size_t)rows * r->experts); float *dw = (float *)(di + kb / 4);
    cudaStream_t s = st().stream;
    bool ok = cuda_ok(cudaMemcpyAsync(dx, x, xb, cudaMemcpyHostToDevice, s), "copy x");
    if (ok) {
        const int rc = omega_gpu_moe_router_rows_async(r, rows, (uint64_t)(uintptr_t)dx, 0, eps, norm_topk, out_scale, topk, (uint64_t)(uintptr_t)dxn, 0,
                                                       (uint64_t)(uintptr_t)dl, (uint64_t)(uintptr_t)di, (uint64_t)(uintptr_t)dw, s);
        if (rc != OMEGA_GPU_FP8_OK) return rc;
    }
    if (ok && xn) ok = cuda_ok(cudaMemcpyAsync(xn, dxn, xb, cudaMemcpyDeviceToHost, s), "copy xn");
    if (ok && logits) ok = cuda_ok(cudaMemcpyAsync(logits, dl, lb, cudaMemcpyDeviceToHost, s), "copy logits");
    ok = ok && cuda_ok(cudaMemcpyAsync(ids, di, kb, cudaMemcpyDeviceToHost, s), "copy ids") && cuda_ok(cudaMemcpyAsync(wts, dw, kb, cudaMemcpyDeviceToHost, s), "copy weights") &&
         cuda_ok(cudaStreamSynchronize(s), "router");
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

}  // extern "C"
