// moe_stack.cu: a stack of MoE layers on one residual stream, the MoE part of the reference's whole-token decode
// graph (src/omega_gpu_decode_graph.c:321-351: per layer RES COMBINE|NORM then router and experts). Per layer:
// xn = bf16(RMSNorm(h)), h = h + MoE_l(xn, logits_l). The residual add and the next layer's norm are one kernel,
// as in the reference's fused RES kernel (src/omega_blackwell_codegen_dec.c:226-286). The whole step is captured
// once per token count into a CUDA graph and replayed.
#include <stdlib.h>
#include <vector>
#include "internal.h"
#include "mma_common.cuh"

namespace b200 {

// one CTA per token: h (+= m) ; xn = bf16(h * rsqrt(mean(h^2) + eps)). Sum of squares in double, one f32 factor,
// as the reference host glue does (tests/gpu_decode_graph_test.c:56-60). x16 != nullptr initialises h from bf16.
__global__ void __launch_bounds__(256) residual_norm_kernel(uint32_t hidden, float eps, const uint16_t *__restrict__ x16, const float *__restrict__ m,
                                                            float *__restrict__ h, uint16_t *__restrict__ xn, uint16_t *__restrict__ h16, const float *__restrict__ nw) {
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
        const float v = __fmul_rn(h[i], sc);
        xn[i] = (uint16_t)bf16_rne_bits(nw ? __fmul_rn(v, nw[c]) : v);
    }
}


// Fused step between two layers on the tensor-core engine, one CTA per token:
//   m = sum over slots, in slot order, of w[t][s] * dn[t*K+s] (multiply then add, never fused: the reference's combine,
//   src/omega_blackwell_codegen_dec.c:226-255); h = (x16 ? f32(x16) : h) + m; then, when a next layer follows,
//   xn = bf16(RMSNorm(h)) is cut into e4m3 pieces per 128 columns (the activation quantiser of moe_glue.cu) and
//   written straight to the sorted rows the NEXT layer's plan assigns to this token's K picks (pos[t*K+s]).
// Same arithmetic, value for value, as combine_kernel -> residual_norm_kernel -> act_quant_kernel.
__global__ void __launch_bounds__(256) combine_norm_scatter_kernel(uint32_t hidden, uint32_t topk, float eps, const uint16_t *__restrict__ x16,
                                                                   const float *__restrict__ w, const float *__restrict__ dn, float *__restrict__ h,
                                                                   const uint32_t *__restrict__ pos, uint32_t pieces, size_t piece_stride, uint8_t *__restrict__ q,
                                                                   float *__restrict__ sx, uint16_t *__restrict__ h16, uint32_t *__restrict__ sched, uint32_t n_sched,
                                                                   const float *__restrict__ nw) {
    __shared__ double red[8];
    __shared__ float s_scale;
    __shared__ uint32_t s_pos[32];
    const uint32_t t = blockIdx.x, tid = threadIdx.x, lane = tid & 31u, kb_total = hidden / 128u;
    // the next layer's sorted rows of this token's picks and the norm weights come from step start, not from the kernel before: fetch them
    // before the dependency wait
    if (q && tid < topk) s_pos[tid] = pos[(size_t)t * topk + tid];
    float4 keep[4], wkeep[4];   // this thread's columns (tid * 4 + 1024 j) of h and of the norm weight: the quantiser below uses the same mapping
    const bool kept = hidden <= 4096u;
    if (q && kept) {
#pragma unroll
        for (int j = 0; j < 4; j++) { const uint32_t c = tid * 4u + 1024u * j; if (c < hidden) wkeep[j] = __ldg(reinterpret_cast<const float4 *>(nw + c)); }
    }
    // launched as a programmatic dependent: everything read below is the previous kernel's output
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // work-list words of the expert kernel that follows (its previous launch has completed: this kernel depends on it)
    if (sched && blockIdx.x == 0) for (uint32_t i = tid; i < n_sched; i += 256) sched[i] = 0;
    double sq = 0.0;
    auto add_row = [&](uint32_t c) -> float4 {
        const size_t i = (size_t)t * hidden + c;
        float4 v;
        if (x16) { const uint2 u = *reinterpret_cast<const uint2 *>(x16 + i); v = make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u)); }
        else v = *reinterpret_cast<const float4 *>(h + i);
        if (dn) {
            const float4 m = combine_slots<false>(topk, w, dn, (size_t)t * topk, hidden, c);
            v = make_float4(__fadd_rn(v.x, m.x), __fadd_rn(v.y, m.y), __fadd_rn(v.z, m.z), __fadd_rn(v.w, m.w));
        }
        *reinterpret_cast<float4 *>(h + i) = v;
        if (h16) {
            auto rne = [](float f) -> uint32_t { const uint32_t b = __float_as_uint(f); return ((b & 0x7fffffffu) > 0x7f800000u) ? ((b >> 16) | 0x40u) : ((b + 0x7fffu + ((b >> 16) & 1u)) >> 16); };
            uint2 pk; pk.x = rne(v.x) | (rne(v.y) << 16); pk.y = rne(v.z) | (rne(v.w) << 16);
            *reinterpret_cast<uint2 *>(h16 + i) = pk;
        }
        sq += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
        return v;
    };
    if (kept) {
#pragma unroll
        for (int j = 0; j < 4; j++) { const uint32_t c = tid * 4u + 1024u * j; if (c < hidden) keep[j] = add_row(c); }
    } else {
        for (uint32_t c = tid * 4; c < hidden; c += 1024) add_row(c);
    }
    if (!q) return;
    for (int o = 16; o; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if (lane == 0) red[tid >> 5] = sq;
    __syncthreads();
    if (tid == 0) { double acc = 0; for (int i = 0; i < 8; i++) acc += red[i]; s_scale = (float)(1.0 / sqrt(acc / (double)hidden + (double)eps)); }
    __syncthreads();
    const float sc = s_scale;
    // one warp per 128-column block, lane = 4 columns (the quantiser's own mapping): block warp + 8 j = columns tid * 4 + 1024 j, the ones this
    // thread summed above
    auto emit = [&](uint32_t kb, const float4 hv, const float4 wv) {
        const uint32_t c = kb * 128u + lane * 4u;
        // xn = h * s * w (the reference's RMSNorm, src/omega_blackwell_codegen_dec.c:261-286; host form tests/gpu_decode_graph_test.c:56-60);
        // xn is a bf16 tensor: round first, then quantise the rounded value
        float v[4] = {__fmul_rn(__fmul_rn(hv.x, sc), wv.x), __fmul_rn(__fmul_rn(hv.y, sc), wv.y), __fmul_rn(__fmul_rn(hv.z, sc), wv.z), __fmul_rn(__fmul_rn(hv.w, sc), wv.w)};
#pragma unroll
        for (int i = 0; i < 4; i++) v[i] = __uint_as_float(bf16_rne_bits(v[i]) << 16);
        uint32_t codes[4];
        const float qs = quant_pieces_warp(v, pieces, codes);
        for (uint32_t s = 0; s < topk; s++) {
            const uint32_t row = s_pos[s];
            for (uint32_t p = 0; p < pieces; p++) *reinterpret_cast<uint32_t *>(q + (size_t)p * piece_stride + (size_t)row * hidden + c) = codes[p];
            if (lane == 0) sx[(size_t)row * kb_total + kb] = qs;
        }
    };
    if (kept) {
#pragma unroll
        for (int j = 0; j < 4; j++) { const uint32_t kb = (tid >> 5) + 8u * j; if (kb < kb_total) emit(kb, keep[j], wkeep[j]); }
    } else {
        for (uint32_t kb = tid >> 5; kb < kb_total; kb += 8) {
            const uint32_t c = kb * 128u + lane * 4u;
            emit(kb, *reinterpret_cast<const float4 *>(h + (size_t)t * hidden + c), __ldg(reinterpret_cast<const float4 *>(nw + c)));
        }
    }
}

}  // namespace b200
using namespace b200;

struct OmegaGpuMoeStack {
    std::vector<OmegaGpuMoeLayer *> layers;
    std::vector<OmegaGpuMoeRouter *> routers;   // per layer, or null: when every layer has one the stack computes its own routing and takes no logits
    bool router_mode;
    float eps;
    uint32_t experts, hidden, max_tokens, shared;   // experts: what the tensors hold; shared 1: the last of them is the shared expert, logits cover experts - 1
    float *h; uint16_t *xn, *logits, *x, *out16;      // device
    float *norm_w;                                    // device [layers][hidden]: RMSNorm weight of each layer's input (ones until set)
    cudaGraphExec_t graph; uint32_t graph_tokens; cudaStream_t graph_stream;
    uint64_t g_logits, g_x, g_out32, g_out16;         // addresses the captured graph was built for
    uint32_t launches;
    // fused path (every layer on the tensor-core engine): routing of all layers up front, then per layer the expert kernel (one launch, or gate|up + down) and combine/norm/scatter
    bool fused;
    uint32_t topk, row_cap, x_pieces, tile_rows;
    uint32_t *ids_all; float *wts_all; PlanBatch pb; size_t map_stride, tile_stride;
    uint8_t *qx; float *sx; char *fused_base; uint32_t *sched; bool one_launch;
    cudaEvent_t *prof;   // when set (2 per layer): recorded before and after each layer's expert kernel(s)
    alignas(128) unsigned char tm_qx[128];
};

namespace b200 {
static bool stack_record(OmegaGpuMoeStack *S, uint32_t tokens, const uint16_t *logits, const uint16_t *x, float *out32, uint16_t *out16, cudaStream_t s) {
    const uint32_t H = S->hidden, E = S->experts, Ln = (uint32_t)S->layers.size();
    uint32_t n = 0;
    if (S->fused && S->router_mode) {
        // Router inside the stack (the reference's per-layer order, src/omega_gpu_decode_graph.c:341-351): residual (+ combine of the layer
        // before) -> router (RMSNorm with the layer's norm weight, gate GEMV, top-k) -> plan -> quantise the normalised rows into the plan's
        // sorted order -> experts. Five launches per layer instead of two; no logits input.
        const uint32_t K = S->topk, Px = S->x_pieces, R = tokens * K;
        LayerView v0; layer_view(S->layers[0], &v0);
        const size_t pstride = (size_t)S->row_cap * H;
        auto launch_res = [&](const uint16_t *x16, const float *w, const float *dn, uint16_t *h16) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(tokens); cfg.blockDim = dim3(256); cfg.stream = s;
            return cudaLaunchKernelEx(&cfg, combine_norm_scatter_kernel, H, K, S->eps, x16, w, dn, S->h, (const uint32_t *)nullptr, Px, pstride, (uint8_t *)nullptr, S->sx, h16, S->sched,
                                      (uint32_t)S->tile_stride + 1u, (const float *)S->norm_w);
        };
        for (uint32_t l = 0; l < Ln; l++) {
            LayerView v; layer_view(S->layers[l], &v);
            LayerView vp; if (l) layer_view(S->layers[l - 1], &vp);
            uint32_t *ids = S->ids_all + (size_t)l * R; float *wts = S->wts_all + (size_t)l * R;
            if (!cuda_ok(launch_res(l ? nullptr : x, l ? S->wts_all + (size_t)(l - 1) * R : nullptr, l ? vp.dn : nullptr, nullptr), "residual launch")) return false; n++;
            if (!cuda_ok(launch_router_rows(S->routers[l], tokens, S->h, S->eps, (int)v0.norm_topk, K - v0.shared, S->xn, ids, wts, s, K), "router launch")) return false; n++;
            uint32_t *hdr = S->pb.header + (size_t)l * 8;
            OmegaGpuMoePlanOut o = {};
            o.counts_va = (uint64_t)(uintptr_t)(S->pb.counts + (size_t)l * E); o.starts_va = (uint64_t)(uintptr_t)(S->pb.starts + (size_t)l * E);
            o.xmap_va = (uint64_t)(uintptr_t)(S->pb.xmap + (size_t)l * S->map_stride); o.ymap_va = (uint64_t)(uintptr_t)(S->pb.ymap + (size_t)l * S->map_stride);
            o.header_va = (uint64_t)(uintptr_t)hdr; o.tiles_va = (uint64_t)(uintptr_t)(S->pb.tiles + (size_t)l * S->tile_stride);
            if (!cuda_ok(launch_plan(tokens, K, E, K, S->tile_rows, ids, o, s), "plan launch")) return false; n++;
            if (!cuda_ok(launch_act_quant(R, H, Px, S->xn, 1, S->pb.xmap + (size_t)l * S->map_stride, hdr, S->qx, S->sx, s, 0, S->row_cap), "x quant launch")) return false; n++;
            if (S->prof) cudaEventRecord(S->prof[2 * l], s);
            if (S->one_launch) {
                FfnLaunch f = {};
                f.gu_scale = v.gu_scale; f.dn_scale = v.dn_scale; f.x_scale = S->sx; f.qa = v.qa; f.sa = v.sa; f.tiles = S->pb.tiles + (size_t)l * S->tile_stride; f.header = hdr;
                f.ymap = S->pb.ymap + (size_t)l * S->map_stride; f.out = v.dn; f.hidden = H; f.inter = v.inter; f.q_rows = S->row_cap; f.sched = S->sched; f.err = hdr + 4;
                if (!cuda_ok(launch_ffn(v.tm_gu, S->tm_qx, v.tm_dn, v.tm_qa, Px, v.act_pieces, f, s, true /* dependent of the quantiser just launched */), "expert ffn launch")) return false; n++;
            } else {
                MmaLaunch g = {};
                g.wscale = v.gu_scale; g.ascale = S->sx; g.tiles = S->pb.tiles + (size_t)l * S->tile_stride; g.header = hdr; g.q_out = v.qa; g.s_out = v.sa; g.q_rows = S->row_cap; g.q_pieces = v.act_pieces;
                g.n = 2 * v.inter; g.k = H; g.mode = 0; g.out_stride = v.inter; g.err = hdr + 4;
                if (!cuda_ok(launch_mma_grouped(v.tm_gu, S->tm_qx, Px, g, s, false), "gate|up mma launch")) return false; n++;
                MmaLaunch d = {};
                d.wscale = v.dn_scale; d.ascale = v.sa; d.tiles = g.tiles; d.header = hdr; d.ymap = S->pb.ymap + (size_t)l * S->map_stride; d.out = v.dn; d.q_rows = S->row_cap;
                d.n = H; d.k = v.inter; d.mode = 1; d.out_stride = H; d.err = g.err;
                if (!cuda_ok(launch_mma_grouped(v.tm_dn, v.tm_qa, v.act_pieces, d, s, false), "down mma launch")) return false; n++;
            }
            if (S->prof) cudaEventRecord(S->prof[2 * l + 1], s);
        }
        LayerView vl; layer_view(S->layers[Ln - 1], &vl);
        if (!cuda_ok(launch_res(nullptr, S->wts_all + (size_t)(Ln - 1) * R, vl.dn, out16), "combine launch")) return false; n++;
        if (out32 && !cuda_ok(cudaMemcpyAsync(out32, S->h, (size_t)tokens * H * 4, cudaMemcpyDeviceToDevice, s), "copy h")) return false;
        S->launches = n;
        return cuda_ok(cudaGetLastError(), "stack launch");
    }
    if (S->fused) {
        const uint32_t K = S->topk, Px = S->x_pieces;
        LayerView v0; layer_view(S->layers[0], &v0);
        if (!cuda_ok(launch_topk(Ln * tokens, E - v0.shared, K - v0.shared, (int)v0.norm_topk, logits, S->ids_all, S->wts_all, s, K), "topk launch")) return false; n++;
        if (!cuda_ok(launch_plan_batch(Ln, tokens, K, E, K, S->tile_rows, S->ids_all, S->pb, s), "plan launch")) return false; n++;
        const size_t pstride = (size_t)S->row_cap * H;
        auto launch_cns = [&](const uint16_t *x16, const float *w, const float *dn, const uint32_t *pos, uint8_t *q, uint16_t *h16, const float *nw) {
            cudaLaunchConfig_t cfg = {}; cudaLaunchAttribute at[1];
            cfg.gridDim = dim3(tokens); cfg.blockDim = dim3(256); cfg.stream = s;
            at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = at; cfg.numAttrs = 0;   // measured: launching this kernel (or the down GEMM) as a programmatic dependent is slower
            return cudaLaunchKernelEx(&cfg, combine_norm_scatter_kernel, H, K, S->eps, x16, w, dn, S->h, pos, Px, pstride, q, S->sx, h16, S->sched, (uint32_t)S->tile_stride + 1u, nw);
        };
        if (!cuda_ok(launch_cns(x, nullptr, nullptr, S->pb.pos, S->qx, nullptr, S->norm_w), "norm launch")) return false; n++;
        for (uint32_t l = 0; l < Ln; l++) {
            LayerView v; layer_view(S->layers[l], &v);
            const uint32_t *hdr = S->pb.header + (size_t)l * 8;
            if (S->prof) cudaEventRecord(S->prof[2 * l], s);
            if (S->one_launch) {
                FfnLaunch f = {};
                f.gu_scale = v.gu_scale; f.dn_scale = v.dn_scale; f.x_scale = S->sx; f.qa = v.qa; f.sa = v.sa; f.tiles = S->pb.tiles + (size_t)l * S->tile_stride; f.header = hdr;
                f.ymap = S->pb.ymap + (size_t)l * S->map_stride; f.out = v.dn; f.hidden = H; f.inter = v.inter; f.q_rows = S->row_cap; f.sched = S->sched;
                f.err = const_cast<uint32_t *>(hdr) + 4;
                if (!cuda_ok(launch_ffn(v.tm_gu, S->tm_qx, v.tm_dn, v.tm_qa, Px, v.act_pieces, f, s, true), "expert ffn launch")) return false; n++;
            } else {
                MmaLaunch g = {};
                g.wscale = v.gu_scale; g.ascale = S->sx; g.tiles = S->pb.tiles + (size_t)l * S->tile_stride; g.header = hdr; g.out = nullptr;
                g.q_out = v.qa; g.s_out = v.sa; g.q_rows = S->row_cap; g.q_pieces = v.act_pieces;
                g.n = 2 * v.inter; g.k = H; g.mode = 0; g.out_stride = v.inter; g.err = const_cast<uint32_t *>(hdr) + 4;
                if (!cuda_ok(launch_mma_grouped(v.tm_gu, S->tm_qx, Px, g, s, true /* weight tiles prefetched while the norm kernel runs */), "gate|up mma launch")) return false; n++;
                MmaLaunch d = {};
                d.wscale = v.dn_scale; d.ascale = v.sa; d.tiles = g.tiles; d.header = hdr; d.ymap = S->pb.ymap + (size_t)l * S->map_stride; d.out = v.dn; d.q_rows = S->row_cap;
                d.n = H; d.k = v.inter; d.mode = 1; d.out_stride = H; d.err = g.err;
                if (!cuda_ok(launch_mma_grouped(v.tm_dn, v.tm_qa, v.act_pieces, d, s, false), "down mma launch")) return false; n++;
            }
            if (S->prof) cudaEventRecord(S->prof[2 * l + 1], s);
            const bool last = l + 1 == Ln;
            if (!cuda_ok(launch_cns(nullptr, S->wts_all + (size_t)l * tokens * K, v.dn, last ? nullptr : S->pb.pos + (size_t)(l + 1) * S->map_stride,
                                    last ? nullptr : S->qx, last ? out16 : nullptr, S->norm_w + (size_t)(last ? 0 : l + 1) * H), "combine launch")) return false; n++;
        }
        if (out32 && !cuda_ok(cudaMemcpyAsync(out32, S->h, (size_t)tokens * H * 4, cudaMemcpyDeviceToDevice, s), "copy h")) return false;
        S->launches = n;
        return cuda_ok(cudaGetLastError(), "stack launch");
    }
    residual_norm_kernel<<<tokens, 256, 0, s>>>(H, S->eps, x, nullptr, S->h, S->xn, nullptr, S->norm_w); n++;
    for (uint32_t l = 0; l < Ln; l++) {
        OmegaGpuMoeLayer *L = S->layers[l];
        float *m = layer_out32(L);
        if (!layer_forward(L, tokens, logits + (size_t)l * tokens * (E - S->shared), S->xn, m, nullptr, s)) return false;
        n += omega_gpu_moe_layer_launches(L);
        const bool last = l + 1 == Ln;
        residual_norm_kernel<<<tokens, 256, 0, s>>>(H, S->eps, nullptr, m, S->h, last ? nullptr : S->xn, last ? out16 : nullptr, S->norm_w + (size_t)(last ? 0 : l + 1) * H); n++;
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

int omega_gpu_residual_norm_w_async(uint32_t tokens, uint32_t hidden, float eps, uint64_t x16_va, uint64_t m_va, uint64_t h_va, uint64_t xn_va, uint64_t h16_va,
                                    uint64_t norm_w_va, void *stream) {
    if (!tokens || !hidden || !h_va) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    residual_norm_kernel<<<tokens, 256, 0, (cudaStream_t)stream>>>(hidden, eps, (const uint16_t *)(uintptr_t)x16_va, (const float *)(uintptr_t)m_va, (float *)(uintptr_t)h_va,
                                                                    (uint16_t *)(uintptr_t)xn_va, (uint16_t *)(uintptr_t)h16_va, (const float *)(uintptr_t)norm_w_va);
    return cuda_ok(cudaGetLastError(), "residual norm launch") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}
int omega_gpu_residual_norm_async(uint32_t tokens, uint32_t hidden, float eps, uint64_t x16_va, uint64_t m_va, uint64_t h_va, uint64_t xn_va, uint64_t h16_va, void *stream) {
    return omega_gpu_residual_norm_w_async(tokens, hidden, eps, x16_va, m_va, h_va, xn_va, h16_va, 0, stream);
}

int omega_gpu_moe_stack_set_router(OmegaGpuMoeStack *S, uint32_t layer, OmegaGpuMoeRouter *router) {
    if (!S || layer >= S->layers.size()) return OMEGA_GPU_FP8_BAD_ARGS;
    if (router) {
        uint32_t e = 0, h = 0; router_dims(router, &e, &h);
        if (e != S->experts - S->shared || h != S->hidden) { set_error("moe stack: router of layer %u is %u experts x %u, the stack routes over %u x %u", layer, e, h, S->experts - S->shared, S->hidden); return OMEGA_GPU_FP8_BAD_ARGS; }
        if (!S->fused) { set_error("moe stack: the router runs inside the stack on the tensor-core engine only"); return OMEGA_GPU_FP8_BAD_ARGS; }
    }
    Lock l;
    S->routers[layer] = router;
    bool all = true;
    for (auto *r : S->routers) all = all && r != nullptr;
    S->router_mode = all;
    if (S->graph) { cudaGraphExecDestroy(S->graph); S->graph = nullptr; }   // another sequence of launches: capture again at the next step
    return OMEGA_GPU_FP8_OK;
}

int omega_gpu_moe_stack_set_norm(OmegaGpuMoeStack *S, uint32_t layer, const float *norm_w) {
    if (!S || !norm_w || layer >= S->layers.size()) return OMEGA_GPU_FP8_BAD_ARGS;
    for (uint32_t i = 0; i < S->hidden; i++) if (!(norm_w[i] == norm_w[i]) || norm_w[i] - norm_w[i] != 0.0f) { set_error("moe stack: norm weight %u of layer %u is not finite", i, layer); return OMEGA_GPU_FP8_BAD_ARGS; }
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    // the captured step reads this buffer, so new weights take effect at the next step without a new capture
    return cuda_ok(cudaMemcpy(S->norm_w + (size_t)layer * S->hidden, norm_w, (size_t)S->hidden * 4, cudaMemcpyHostToDevice), "copy norm weights") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_stack_create(uint32_t layers, OmegaGpuMoeLayer *const *layer, float eps, OmegaGpuMoeStack **out) {
    if (out) *out = nullptr;
    if (!layers || !layer || !out || !(eps >= 0.0f)) return OMEGA_GPU_FP8_BAD_ARGS;
    for (uint32_t i = 0; i < layers; i++) if (!layer[i]) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    OmegaGpuMoeStack *S = new OmegaGpuMoeStack();
    S->eps = eps; S->graph = nullptr; S->graph_tokens = 0; S->launches = 0; S->prof = nullptr; S->router_mode = false; S->routers.assign(layers, nullptr);
    layer_dims(layer[0], &S->experts, &S->hidden, &S->max_tokens);
    { LayerView vs; layer_view(layer[0], &vs); S->shared = vs.shared; }
    for (uint32_t i = 0; i < layers; i++) {
        uint32_t e, h, mt; layer_dims(layer[i], &e, &h, &mt);
        if (e != S->experts || h != S->hidden || mt != S->max_tokens || !layer_share_workspace(layer[i], layer[0])) {
            delete S; set_error("moe stack: layer %u does not match layer 0", i); return OMEGA_GPU_FP8_BAD_ARGS;
        }
        S->layers.push_back(layer[i]);
    }
    const size_t T = S->max_tokens, H = S->hidden;
    const size_t nw_off = (T * H * 4 + T * H * 2 * 3 + (size_t)layers * T * S->experts * 2 + 255) & ~(size_t)255, bytes = nw_off + (size_t)layers * H * 4;
    char *b = nullptr;
    if (!cuda_ok(cudaMalloc(&b, bytes), "cudaMalloc(stack)")) { delete S; return OMEGA_GPU_FP8_CHIP_FAIL; }
    S->h = (float *)b; S->xn = (uint16_t *)(b + T * H * 4); S->x = S->xn + T * H; S->out16 = S->x + T * H; S->logits = S->out16 + T * H;
    S->norm_w = (float *)(b + nw_off);
    {
        std::vector<float> ones((size_t)layers * H, 1.0f);
        if (!cuda_ok(cudaMemcpy(S->norm_w, ones.data(), ones.size() * 4, cudaMemcpyHostToDevice), "init norm weights")) { cudaFree(b); delete S; return OMEGA_GPU_FP8_CHIP_FAIL; }
    }
    // fused path when every layer runs the tensor-core engine with the same piece counts
    LayerView v0; layer_view(layer[0], &v0);
    S->fused = v0.engine == OMEGA_GPU_MOE_ENGINE_MMA && H % 128 == 0;
    for (uint32_t i = 0; i < layers && S->fused; i++) {
        LayerView v; layer_view(layer[i], &v);
        S->fused = v.engine == OMEGA_GPU_MOE_ENGINE_MMA && v.x_pieces == v0.x_pieces && v.topk == v0.topk && v.tile_rows == v0.tile_rows && v.norm_topk == v0.norm_topk;
    }
    S->fused_base = nullptr;
    if (S->fused) {
        const size_t K = v0.topk, R = T * K, Rp = v0.row_cap, E = S->experts, Ln = layers;
        S->topk = v0.topk; S->row_cap = v0.row_cap; S->x_pieces = v0.x_pieces; S->tile_rows = v0.tile_rows;
        S->map_stride = (R + 8 + 63) & ~(size_t)63; S->tile_stride = (R / 8 + E + 8 + 15) & ~(size_t)15;
        size_t off = 0;
        auto take = [&](size_t bytes) { const size_t o = off; off += (bytes + 255) & ~(size_t)255; return o; };
        const size_t o_ids = take(Ln * R * 4), o_w = take(Ln * R * 4), o_c = take(Ln * E * 4), o_s = take(Ln * E * 4), o_x = take(Ln * S->map_stride * 4),
                     o_y = take(Ln * S->map_stride * 4), o_p = take(Ln * S->map_stride * 4), o_h = take(Ln * 32), o_t = take(Ln * S->tile_stride * 16),
                     o_q = take((size_t)v0.x_pieces * Rp * H), o_sx = take(Rp * (H / 128) * 4), o_sched = take((S->tile_stride + 1) * 4);
        bool ok = cuda_ok(cudaMalloc(&S->fused_base, off), "cudaMalloc(stack routing)") && cuda_ok(cudaMemset(S->fused_base, 0, off), "memset");
        if (ok) {
            char *f = S->fused_base;
            S->ids_all = (uint32_t *)(f + o_ids); S->wts_all = (float *)(f + o_w);
            S->pb.counts = (uint32_t *)(f + o_c); S->pb.starts = (uint32_t *)(f + o_s); S->pb.xmap = (uint32_t *)(f + o_x); S->pb.ymap = (uint32_t *)(f + o_y);
            S->pb.pos = (uint32_t *)(f + o_p); S->pb.header = (uint32_t *)(f + o_h); S->pb.tiles = (uint4 *)(f + o_t);
            S->pb.map_stride = S->map_stride; S->pb.tile_stride = S->tile_stride;
            S->qx = (uint8_t *)(f + o_q); S->sx = (float *)(f + o_sx); S->sched = (uint32_t *)(f + o_sched);
            const bool pieces_ok = (v0.x_pieces == 2 && v0.act_pieces == 3) || (v0.x_pieces == 1 && v0.act_pieces == 1) || (v0.x_pieces == 2 && v0.act_pieces == 2);
            S->one_launch = pieces_ok && ffn_shape_ok((uint32_t)H, v0.inter) && !getenv("B200MOE_TWO_LAUNCH");
            ok = make_tmap_u8(S->tm_qx, S->qx, (uint64_t)v0.x_pieces * Rp, H, 32);
        }
        if (!ok) { if (S->fused_base) cudaFree(S->fused_base); cudaFree(S->h); delete S; return OMEGA_GPU_FP8_CHIP_FAIL; }
    }
    *out = S;
    return OMEGA_GPU_FP8_OK;
}

void omega_gpu_moe_stack_free(OmegaGpuMoeStack *S) {
    if (!S) return;
    Lock l;
    if (S->graph) cudaGraphExecDestroy(S->graph);
    if (S->h) cudaFree(S->h);
    if (S->fused_base) cudaFree(S->fused_base);
    delete S;
}

uint32_t omega_gpu_moe_stack_launches(const OmegaGpuMoeStack *S) { return S ? S->launches : 0; }

int omega_gpu_moe_stack_profile(OmegaGpuMoeStack *S, uint32_t tokens, uint64_t logits_va, uint64_t x_va, uint32_t cap, float *expert_ms, uint32_t *count, uint32_t *launches_per_layer) {
    if (!S || !tokens || (!logits_va && !S->router_mode) || !x_va || !expert_ms || !count || !cap) return OMEGA_GPU_FP8_BAD_ARGS;
    if (tokens > S->max_tokens) return OMEGA_GPU_FP8_TOO_LARGE;
    if (!S->fused) { set_error("moe stack profile: only the tensor-core path records per-layer times"); return OMEGA_GPU_FP8_BAD_ARGS; }
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    const uint32_t Ln = (uint32_t)S->layers.size();
    std::vector<cudaEvent_t> ev(2 * Ln);
    for (auto &e : ev) if (!cuda_ok(cudaEventCreate(&e), "cudaEventCreate")) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = st().stream;
    S->prof = ev.data();
    bool ok = stack_record(S, tokens, (const uint16_t *)(uintptr_t)logits_va, (const uint16_t *)(uintptr_t)x_va, nullptr, S->out16, s);
    S->prof = nullptr;
    ok = ok && cuda_ok(cudaStreamSynchronize(s), "moe stack profile");
    *count = 0;
    for (uint32_t i = 0; ok && i < Ln && i < cap; i++) { float t = 0; ok = cuda_ok(cudaEventElapsedTime(&t, ev[2 * i], ev[2 * i + 1]), "event time"); expert_ms[i] = t; *count = i + 1; }
    for (auto &e : ev) cudaEventDestroy(e);
    if (launches_per_layer) *launches_per_layer = S->one_launch ? 1u : 2u;
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_stack_async(OmegaGpuMoeStack *S, uint32_t tokens, uint64_t logits_va, uint64_t x_va, uint64_t out_f32_va, uint64_t out_bf16_va, void *stream) {
    if (!S || !tokens || (!logits_va && !S->router_mode) || !x_va || (!out_f32_va && !out_bf16_va)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (tokens > S->max_tokens) return OMEGA_GPU_FP8_TOO_LARGE;
    Lock l;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    return stack_run(S, tokens, (const uint16_t *)(uintptr_t)logits_va, (const uint16_t *)(uintptr_t)x_va, (float *)(uintptr_t)out_f32_va,
                     (uint16_t *)(uintptr_t)out_bf16_va, (cudaStream_t)stream) ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_stack_bf16(OmegaGpuMoeStack *S, uint32_t tokens, const uint16_t *logits, const uint16_t *x, uint16_t *out_bf16, float *out_f32) {
    if (!S || !tokens || (!logits && !S->router_mode) || !x || (!out_bf16 && !out_f32)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (tokens > S->max_tokens) return OMEGA_GPU_FP8_TOO_LARGE;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = st().stream;
    const size_t xb = (size_t)tokens * S->hidden * 2, lb = S->layers.size() * (size_t)tokens * (S->experts - S->shared) * 2;
    bool ok = (S->router_mode || cuda_ok(cudaMemcpyAsync(S->logits, logits, lb, cudaMemcpyHostToDevice, s), "copy logits")) &&
              cuda_ok(cudaMemcpyAsync(S->x, x, xb, cudaMemcpyHostToDevice, s), "copy x") &&
              stack_run(S, tokens, S->logits, S->x, nullptr, S->out16, s);
    if (ok && out_bf16) ok = cuda_ok(cudaMemcpyAsync(out_bf16, S->out16, xb, cudaMemcpyDeviceToHost, s), "copy out");
    if (ok && out_f32) ok = cuda_ok(cudaMemcpyAsync(out_f32, S->h, xb * 2, cudaMemcpyDeviceToHost, s), "copy out");
    std::vector<uint32_t> hdr;
    if (ok && S->fused) { hdr.resize(S->layers.size() * 8); ok = cuda_ok(cudaMemcpyAsync(hdr.data(), S->pb.header, hdr.size() * 4, cudaMemcpyDeviceToHost, s), "copy status"); }
    ok = ok && cuda_ok(cudaStreamSynchronize(s), "moe stack");
    for (size_t l = 0; ok && l * 8 < hdr.size(); l++) {
        if (hdr[l * 8 + 3]) { set_error("moe stack: routing plan of layer %zu refused (status %u)", l, hdr[l * 8 + 3]); return OMEGA_GPU_FP8_BAD_ARGS; }
        if (hdr[l * 8 + 4]) { set_error("moe stack: a bounded wait inside the tensor-core kernel ran out (layer %zu, code %u)", l, hdr[l * 8 + 4]); st().latched = true; return OMEGA_GPU_FP8_CHIP_FAIL; }
    }
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

}  // extern "C"
