// moe_w4_layer.cu: one MoE layer whose expert weights are 4-bit (int4 + fp16 scales, MXFP4 or NVFP4: the formats of w4_gemm.cu; the last two are the
// reference's own 4-bit expert formats, docs/models/MXFP4.md and native/models/nvfp4.om). The same steps as the FP8 layer of moe_layer.cu
// (src/omega_gpu_decode_graph.c:341-351: router top-k, plan, gate|up, SiLU gate, down, combine), with the two grouped GEMMs run by the 4-bit
// tensor-core kernel over the plan's 16-row tiles: top-k -> plan (tile_rows 16) -> grouped gate|up (token rows gathered through xmap, f32 out in
// sorted-row order) -> SiLU gate, rounded to bf16 -> grouped down (results scattered to token * topk + slot through ymap) -> combine in slot order.
// Activations enter both GEMMs as bf16 (the GEMM's input type): x is bf16 already, the gated activation is rounded once.
#include <stdlib.h>
#include "internal.h"

namespace b200 {
static size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }
}
using namespace b200;

struct OmegaGpuMoeW4Layer {
    OmegaGpuW4Tensor *gu, *dn;     // not owned: experts x 2I rows of k = H; experts x H rows of k = I
    uint32_t experts, hidden, inter, topk, max_tokens, max_tiles; int norm_topk;
    char *base;
    uint16_t *logits, *x, *act16, *out16; uint32_t *ids, *counts, *starts, *xmap, *ymap, *tiles, *header, *scratch; size_t scratch_words;
    float *wts, *gu32, *dn32, *out32;
    uint32_t launches;
};

extern "C" {

int omega_gpu_moe_w4_layer_create(OmegaGpuW4Tensor *gate_up, OmegaGpuW4Tensor *down, uint32_t experts, uint32_t topk, uint32_t max_tokens, int norm_topk,
                                  OmegaGpuMoeW4Layer **out) {
    if (out) *out = nullptr;
    if (!out || !gate_up || !down || !experts || !topk || topk > 32 || topk > experts || !max_tokens) return OMEGA_GPU_FP8_BAD_ARGS;
    if (gate_up->n % experts || down->n % experts) { set_error("w4 layer: tensor rows are not a multiple of the expert count"); return OMEGA_GPU_FP8_BAD_ARGS; }
    const uint32_t H = gate_up->k, I = down->k;
    if (gate_up->n / experts != 2u * I || down->n / experts != H) { set_error("w4 layer: gate|up must be experts x 2I rows of H columns and down experts x H rows of I columns"); return OMEGA_GPU_FP8_BAD_ARGS; }
    if (gate_up->fmt != down->fmt) { set_error("w4 layer: both tensors must have one weight format"); return OMEGA_GPU_FP8_BAD_ARGS; }
    OmegaGpuMoeW4Layer *L = (OmegaGpuMoeW4Layer *)calloc(1, sizeof *L);
    if (!L) return OMEGA_GPU_FP8_BAD_ARGS;
    L->gu = gate_up; L->dn = down; L->experts = experts; L->hidden = H; L->inter = I; L->topk = topk; L->max_tokens = max_tokens; L->norm_topk = norm_topk;
    const size_t T = max_tokens, R = T * topk;
    L->max_tiles = (uint32_t)(R / 16 + experts + 8);
    // the per-tile scratch of the two grouped GEMMs (each call takes the library's lock itself)
    int rc = omega_gpu_w4_reserve_grouped(gate_up, 2u * I, L->max_tiles);
    if (rc == OMEGA_GPU_FP8_OK) rc = omega_gpu_w4_reserve_grouped(down, H, L->max_tiles);
    if (rc != OMEGA_GPU_FP8_OK) { free(L); return rc; }
    Lock l;
    if (!dev_open()) { free(L); return OMEGA_GPU_FP8_CHIP_FAIL; }
    L->scratch_words = plan_scratch_words((uint32_t)R, experts);
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off += up256(bytes); return o; };
    const size_t o_lg = take(T * experts * 2), o_x = take(T * H * 2), o_ids = take(R * 4), o_wts = take(R * 4), o_cnt = take((size_t)experts * 4), o_st = take((size_t)experts * 4),
                 o_xm = take((R + 8) * 4), o_ym = take((R + 8) * 4), o_tl = take((size_t)L->max_tiles * 16), o_hdr = take(64), o_sc = take(L->scratch_words * 4),
                 o_gu = take((R + 8) * 2 * I * 4), o_act = take((R + 8) * I * 2), o_dn = take((R + 8) * H * 4), o_o32 = take(T * H * 4), o_o16 = take(T * H * 2);
    if (!cuda_ok(cudaMalloc(&L->base, off), "cudaMalloc(w4 layer)") || !cuda_ok(cudaMemset(L->base, 0, off), "memset")) { if (L->base) cudaFree(L->base); free(L); return OMEGA_GPU_FP8_CHIP_FAIL; }
    char *b = L->base;
    L->logits = (uint16_t *)(b + o_lg); L->x = (uint16_t *)(b + o_x); L->ids = (uint32_t *)(b + o_ids); L->wts = (float *)(b + o_wts); L->counts = (uint32_t *)(b + o_cnt);
    L->starts = (uint32_t *)(b + o_st); L->xmap = (uint32_t *)(b + o_xm); L->ymap = (uint32_t *)(b + o_ym); L->tiles = (uint32_t *)(b + o_tl); L->header = (uint32_t *)(b + o_hdr);
    L->scratch = (uint32_t *)(b + o_sc); L->gu32 = (float *)(b + o_gu); L->act16 = (uint16_t *)(b + o_act); L->dn32 = (float *)(b + o_dn); L->out32 = (float *)(b + o_o32); L->out16 = (uint16_t *)(b + o_o16);
    *out = L;
    return OMEGA_GPU_FP8_OK;
}

void omega_gpu_moe_w4_layer_free(OmegaGpuMoeW4Layer *L) {
    if (!L) return;
    Lock l;
    if (L->base) cudaFree(L->base);
    free(L);
}

// device buffers, stream-ordered: logits bf16 [tokens][experts], x bf16 [tokens][hidden] -> out f32 [tokens][hidden] (required), out bf16 (optional)
int omega_gpu_moe_w4_layer_async(OmegaGpuMoeW4Layer *L, uint32_t tokens, uint64_t logits_va, uint64_t x_va, uint64_t out_f32_va, uint64_t out_bf16_va, void *stream) {
    if (!L || !tokens || !logits_va || !x_va || !out_f32_va) return OMEGA_GPU_FP8_BAD_ARGS;
    if (tokens > L->max_tokens) return OMEGA_GPU_FP8_TOO_LARGE;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t K = L->topk, E = L->experts, H = L->hidden, I = L->inter, R = tokens * K;
    OmegaGpuMoePlanOut o = {};
    o.counts_va = (uint64_t)(uintptr_t)L->counts; o.starts_va = (uint64_t)(uintptr_t)L->starts; o.xmap_va = (uint64_t)(uintptr_t)L->xmap; o.ymap_va = (uint64_t)(uintptr_t)L->ymap;
    o.tiles_va = (uint64_t)(uintptr_t)L->tiles; o.header_va = (uint64_t)(uintptr_t)L->header;
    const bool ok = cuda_ok(launch_topk(tokens, E, K, L->norm_topk, (const uint16_t *)(uintptr_t)logits_va, L->ids, L->wts, s), "top-k launch") &&
                    cuda_ok(launch_plan(tokens, K, E, K, 16, L->ids, o, s, L->scratch, L->scratch_words), "plan launch") &&
                    // gate|up: sorted row p = x[xmap[p]] against its expert's 2I x H matrix, f32 in sorted order
                    cuda_ok(launch_w4_grouped(L->gu, L->tiles, L->header, L->xmap, nullptr, (const uint16_t *)(uintptr_t)x_va, nullptr, L->gu32, s), "gate|up launch") &&
                    cuda_ok(launch_swiglu(R, I, L->gu32, nullptr, s, L->act16), "swiglu launch") &&
                    // down: sorted row p against its expert's H x I matrix, result to row ymap[p] = token * K + slot
                    cuda_ok(launch_w4_grouped(L->dn, L->tiles, L->header, nullptr, L->ymap, L->act16, nullptr, L->dn32, s), "down launch") &&
                    cuda_ok(launch_combine(tokens, K, H, L->wts, L->dn32, (float *)(uintptr_t)out_f32_va, (uint16_t *)(uintptr_t)out_bf16_va, s), "combine launch");
    L->launches = 6 + plan_launch_count(R, E, L->scratch, L->scratch_words, o) - 1u;
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

// host buffers: logits bf16 [tokens][E], x bf16 [tokens][H] -> out bf16 and / or f32 [tokens][H]; ids / wts optional ([tokens][topk])
int omega_gpu_moe_w4_layer_bf16(OmegaGpuMoeW4Layer *L, uint32_t tokens, const uint16_t *logits_bf16, const uint16_t *x_bf16, uint16_t *out_bf16, float *out_f32, uint32_t *ids, float *wts) {
    if (!L || !tokens || !logits_bf16 || !x_bf16 || (!out_bf16 && !out_f32)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (tokens > L->max_tokens) return OMEGA_GPU_FP8_TOO_LARGE;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = st().stream;
    const size_t lb = (size_t)tokens * L->experts * 2, xb = (size_t)tokens * L->hidden * 2, rb = (size_t)tokens * L->topk * 4;
    bool ok = cuda_ok(cudaMemcpyAsync(L->logits, logits_bf16, lb, cudaMemcpyHostToDevice, s), "copy logits") && cuda_ok(cudaMemcpyAsync(L->x, x_bf16, xb, cudaMemcpyHostToDevice, s), "copy x");
    if (!ok) return OMEGA_GPU_FP8_CHIP_FAIL;
    const int rc = omega_gpu_moe_w4_layer_async(L, tokens, (uint64_t)(uintptr_t)L->logits, (uint64_t)(uintptr_t)L->x, (uint64_t)(uintptr_t)L->out32, (uint64_t)(uintptr_t)L->out16, s);
    if (rc != OMEGA_GPU_FP8_OK) return rc;
    if (out_bf16) ok = ok && cuda_ok(cudaMemcpyAsync(out_bf16, L->out16, xb, cudaMemcpyDeviceToHost, s), "copy out");
    if (out_f32) ok = ok && cuda_ok(cudaMemcpyAsync(out_f32, L->out32, xb * 2, cudaMemcpyDeviceToHost, s), "copy out");
    if (ids) ok = ok && cuda_ok(cudaMemcpyAsync(ids, L->ids, rb, cudaMemcpyDeviceToHost, s), "copy ids");
    if (wts) ok = ok && cuda_ok(cudaMemcpyAsync(wts, L->wts, rb, cudaMemcpyDeviceToHost, s), "copy weights");
    uint32_t hdr[8] = {0};
    ok = ok && cuda_ok(cudaMemcpyAsync(hdr, L->header, 32, cudaMemcpyDeviceToHost, s), "copy status") && cuda_ok(cudaStreamSynchronize(s), "w4 layer");
    if (ok && hdr[3]) { set_error("w4 layer: routing plan refused (status %u)", hdr[3]); return OMEGA_GPU_FP8_BAD_ARGS; }
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

uint32_t omega_gpu_moe_w4_layer_launches(const OmegaGpuMoeW4Layer *L) { return L ? L->launches : 0; }

}  // extern "C"
