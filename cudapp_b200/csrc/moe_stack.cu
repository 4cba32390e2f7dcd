// moe_stack.cu: a stack of MoE layers on one residual stream, the MoE part of the reference's whole-token decode
// graph (src/omega_gpu_decode_graph.c:321-351: per layer RES COMBINE|NORM then router and experts). Per layer:
// xn = bf16(RMSNorm(h)), h = h + MoE_l(xn, logits_l). The residual add and the next layer's norm are one kernel,
// as in the reference's fused RES kernel (src/omega_blackwell_codegen_dec.c:226-286). The whole step is captured
// once per token count into a CUDA graph and replayed.
#include <stdlib.h>
#include <vector>
#include "internal.h"

namespace b200 {

// one CTA per token: h (+= m) ; xn = bf16(h * rsqrt(mean(h^2) + eps)). Sum of squares in double, one f32 factor,
// as the reference host glue does (tests/gpu_decode_graph_test.c:56-60). x16 != nullptr initialises h from bf16.
__global__ void __launch_bounds__(256) residual_norm_kernel(uint32_t hidden, float eps, const uint16_t *__restrict__ x16, const float *__restrict__ m,
                                                            float *__restrict__ h, uint16_t *__restrict__ xn, uint16_t *__restrict__ h16) {
    __shared__ double red[8];
    __shared__ float s_scale;
    const uint32_t t = blockIdx.x, tid = threadIdx.x;
    double sq = 0.0;
    for (uint32_t c = tid; c < hidden; c += 256) {
        const size_t i = (size_t)t * hidden + c;
        float v = x16 ? __uint_as_float((uint32_t)x16[i] << 16) : h[i];
        if (m) v = __fadd_rn(v, m[i]);
        h[i] = v;
        if (h16) { const uint32_t b = __float_as_uint(v); h16[i] = (uint16_t)(((b & 0x7fffffffu) > 0x7f800000u) ? ((b >> 16) | 0x40u) : ((b + 0x7fffu + ((b >> 16) & 1u)) >> 16)); }
        sq += (double)v * (double)v;
    }
    if (!xn) return;
    for (int o = 16; o; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if ((tid & 31) == 0) red[tid >> 5] = sq;
    __syncthreads();
    if (tid == 0) { double a = 0; for (int i = 0; i < 8; i++) a += red[i]; s_scale = (float)(1.0 / sqrt(a / (double)hidden + (double)eps)); }
    __syncthreads();
    const float sc = s_scale;
    for (uint32_t c = tid; c < hidden; c += 256) {
        const size_t i = (size_t)t * hidden + c;
        const uint32_t b = __float_as_uint(h[i] * sc);
        xn[i] = (uint16_t)(((b & 0x7fffffffu) > 0x7f800000u) ? ((b >> 16) | 0x40u) : ((b + 0x7fffu + ((b >> 16) & 1u)) >> 16));
    }
}

}  // namespace b200
using namespace b200;

struct OmegaGpuMoeStack {
    std::vector<OmegaGpuMoeLayer *> layers;
    float eps;
    uint32_t experts, hidden, max_tokens;
    float *h; uint16_t *xn, *logits, *x, *out16;      // device
    cudaGraphExec_t graph; uint32_t graph_tokens; cudaStream_t graph_stream;
    uint64_t g_logits, g_x, g_out32, g_out16;         // addresses the captured graph was built for
    uint32_t launches;
};

namespace b200 {
static bool stack_record(OmegaGpuMoeStack *S, uint32_t tokens, const uint16_t *logits, const uint16_t *x, float *out32, uint16_t *out16, cudaStream_t s) {
    const uint32_t H = S->hidden, E = S->experts, Ln = (uint32_t)S->layers.size();
    uint32_t n = 0;
    residual_norm_kernel<<<tokens, 256, 0, s>>>(H, S->eps, x, nullptr, S->h, S->xn, nullptr); n++;
    for (uint32_t l = 0; l < Ln; l++) {
        OmegaGpuMoeLayer *L = S->layers[l];
        float *m = layer_out32(L);
        if (!layer_forward(L, tokens, logits + (size_t)l * tokens * E, S->xn, m, nullptr, s)) return false;
        n += omega_gpu_moe_layer_launches(L);
        const bool last = l + 1 == Ln;
        residual_norm_kernel<<<tokens, 256, 0, s>>>(H, S->eps, nullptr, m, S->h, last ? nullptr : S->xn, last ? out16 : nullptr); n++;
    }
    if (out32 && !cuda_ok(cudaMemcpyAsync(out32, S->h, (size_t)tokens * H * 4, cudaMemcpyDeviceToDevice, s), "copy h")) return false;
    S->launches = n;
    return cuda_ok(cudaGetLastError(), "stack launch");
}

// replays (capturing first when the token count or a buffer address changed) the whole step on stream s
static bool stack_run(OmegaGpuMoeStack *S, uint32_t tokens, const uint16_t *logits, const uint16_t *x, float *out32, uint16_t *out16, cudaStream_t s) {
    const uint64_t a0 = (uint64_t)(uintptr_t)logits, a1 = (uint64_t)(uintptr_t)x, a2 = (uint64_t)(uintptr_t)out32, a3 = (uint64_t)(uintptr_t)out16;
    if (!S->graph || S->graph_tokens != tokens || S->g_logits != a0 || S->g_x != a1 || S->g_out32 != a2 || S->g_out16 != a3) {
        if (S->graph) { cudaGraphExecDestroy(S->graph); S->graph = nullptr; }
        cudaGraph_t g = nullptr;
        if (!cuda_ok(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal), "begin capture")) return false;
        const bool rec = stack_record(S, tokens, logits, x, out32, out16, s);
        const cudaError_t e = cudaStreamEndCapture(s, &g);
        if (!rec || !cuda_ok(e, "end capture")) { if (g) cudaGraphDestroy(g); return false; }
        const bool inst = cuda_ok(cudaGraphInstantiate(&S->graph, g, 0), "graph instantiate");
        cudaGraphDestroy(g);
        if (!inst) { S->graph = nullptr; return false; }
        S->graph_tokens = tokens; S->g_logits = a0; S->g_x = a1; S->g_out32 = a2; S->g_out16 = a3;
    }
    return cuda_ok(cudaGraphLaunch(S->graph, s), "graph launch");
}
}  // namespace b200

extern "C" {

int omega_gpu_residual_norm_async(uint32_t tokens, uint32_t hidden, float eps, uint64_t x16_va, uint64_t m_va, uint64_t h_va, uint64_t xn_va, uint64_t h16_va, void *stream) {
    if (!tokens || !hidden || !h_va) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    residual_norm_kernel<<<tokens, 256, 0, (cudaStream_t)stream>>>(hidden, eps, (const uint16_t *)(uintptr_t)x16_va, (const float *)(uintptr_t)m_va, (float *)(uintptr_t)h_va,
                                                                    (uint16_t *)(uintptr_t)xn_va, (uint16_t *)(uintptr_t)h16_va);
    return cuda_ok(cudaGetLastError(), "residual norm launch") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_stack_create(uint32_t layers, OmegaGpuMoeLayer *const *layer, float eps, OmegaGpuMoeStack **out) {
    if (out) *out = nullptr;
    if (!layers || !layer || !out || !(eps >= 0.0f)) return OMEGA_GPU_FP8_BAD_ARGS;
    for (uint32_t i = 0; i < layers; i++) if (!layer[i]) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    OmegaGpuMoeStack *S = new OmegaGpuMoeStack();
    S->eps = eps; S->graph = nullptr; S->graph_tokens = 0; S->launches = 0;
    layer_dims(layer[0], &S->experts, &S->hidden, &S->max_tokens);
    for (uint32_t i = 0; i < layers; i++) {
        uint32_t e, h, mt; layer_dims(layer[i], &e, &h, &mt);
        if (e != S->experts || h != S->hidden || mt != S->max_tokens || !layer_share_workspace(layer[i], layer[0])) {
            delete S; set_error("moe stack: layer %u does not match layer 0", i); return OMEGA_GPU_FP8_BAD_ARGS;
        }
        S->layers.push_back(layer[i]);
    }
    const size_t T = S->max_tokens, H = S->hidden;
    const size_t bytes = T * H * 4 + T * H * 2 * 3 + (size_t)layers * T * S->experts * 2;
    char *b = nullptr;
    if (!cuda_ok(cudaMalloc(&b, bytes), "cudaMalloc(stack)")) { delete S; return OMEGA_GPU_FP8_CHIP_FAIL; }
    S->h = (float *)b; S->xn = (uint16_t *)(b + T * H * 4); S->x = S->xn + T * H; S->out16 = S->x + T * H; S->logits = S->out16 + T * H;
    *out = S;
    return OMEGA_GPU_FP8_OK;
}

void omega_gpu_moe_stack_free(OmegaGpuMoeStack *S) {
    if (!S) return;
    Lock l;
    if (S->graph) cudaGraphExecDestroy(S->graph);
    if (S->h) cudaFree(S->h);
    delete S;
}

uint32_t omega_gpu_moe_stack_launches(const OmegaGpuMoeStack *S) { return S ? S->launches : 0; }

int omega_gpu_moe_stack_async(OmegaGpuMoeStack *S, uint32_t tokens, uint64_t logits_va, uint64_t x_va, uint64_t out_f32_va, uint64_t out_bf16_va, void *stream) {
    if (!S || !tokens || !logits_va || !x_va || (!out_f32_va && !out_bf16_va)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (tokens > S->max_tokens) return OMEGA_GPU_FP8_TOO_LARGE;
    Lock l;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    return stack_run(S, tokens, (const uint16_t *)(uintptr_t)logits_va, (const uint16_t *)(uintptr_t)x_va, (float *)(uintptr_t)out_f32_va,
                     (uint16_t *)(uintptr_t)out_bf16_va, (cudaStream_t)stream) ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_stack_bf16(OmegaGpuMoeStack *S, uint32_t tokens, const uint16_t *logits, const uint16_t *x, uint16_t *out_bf16, float *out_f32) {
    if (!S || !tokens || !logits || !x || (!out_bf16 && !out_f32)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (tokens > S->max_tokens) return OMEGA_GPU_FP8_TOO_LARGE;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = st().stream;
    const size_t xb = (size_t)tokens * S->hidden * 2, lb = S->layers.size() * (size_t)tokens * S->experts * 2;
    bool ok = cuda_ok(cudaMemcpyAsync(S->logits, logits, lb, cudaMemcpyHostToDevice, s), "copy logits") &&
              cuda_ok(cudaMemcpyAsync(S->x, x, xb, cudaMemcpyHostToDevice, s), "copy x") &&
              stack_run(S, tokens, S->logits, S->x, nullptr, S->out16, s);
    if (ok && out_bf16) ok = cuda_ok(cudaMemcpyAsync(out_bf16, S->out16, xb, cudaMemcpyDeviceToHost, s), "copy out");
    if (ok && out_f32) ok = cuda_ok(cudaMemcpyAsync(out_f32, S->h, xb * 2, cudaMemcpyDeviceToHost, s), "copy out");
    ok = ok && cuda_ok(cudaStreamSynchronize(s), "moe stack");
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

}  // extern "C"
