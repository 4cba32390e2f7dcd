// moe_layer.cu: the quantized MoE layer and layer stack as host-side orchestration of this library's kernels.
// One layer = the MoE part of the reference decode graph (src/omega_gpu_decode_graph.c:341-351) and of its
// prefill recorder (src/omega_gpu_q36_graph.c:1147): router top-k, routing plan, gate|up grouped GEMM with the
// SiLU gate, down grouped GEMM, router-weighted combine. Everything between the input copy and the output copy
// stays on the device; the routing plan is never read back.
#include <stdlib.h>
#include <vector>
#include "internal.h"

namespace b200 {

struct Workspace {
    uint32_t max_tokens, topk, experts, hidden, inter;
    int refs;
    uint32_t *ids, *counts, *starts, *xmap, *ymap, *header, *plan_scratch, *sched; uint32_t sched_words;   // sched: work list of the one-launch expert kernel
    size_t plan_scratch_words;
    float *wts;
    Seg32 *seg_gu, *seg_dn;
    uint4 *tiles;
    float *gu, *act, *dn;          // [R][2I], [R][I], [R][H]
    uint8_t *qx, *qa;              // e4m3 pieces of x rows / act rows (tensor-core engine)
    float *sx, *sa;                // their per-128 scales
    uint8_t *qt; float *stt;       // x quantised once per token (prefill-sized calls): [piece][max_tokens][hidden], [max_tokens][hidden/128]
    uint16_t *logits, *x, *out16;  // staging for the host-buffer entry
    float *out32;
    char *base;
};

static size_t align_up(size_t v) { return (v + 255) & ~(size_t)255; }

static Workspace *workspace_create(uint32_t max_tokens, uint32_t topk, uint32_t experts, uint32_t hidden, uint32_t inter) {
    Workspace *w = (Workspace *)calloc(1, sizeof *w);
    if (!w) return nullptr;
    w->max_tokens = max_tokens; w->topk = topk; w->experts = experts; w->hidden = hidden; w->inter = inter; w->refs = 1;
    const size_t R = (size_t)max_tokens * topk, Rp = R + 8;
    const size_t max_tiles = R / 8 + experts + 8;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off += align_up(bytes); return o; };
    const size_t o_ids = take(R * 4), o_wts = take(R * 4), o_cnt = take((size_t)experts * 4), o_st = take((size_t)experts * 4),
                 o_xm = take(Rp * 4), o_ym = take(Rp * 4), o_hdr = take(64), o_sgu = take((size_t)experts * 32), o_sdn = take((size_t)experts * 32),
                 o_tiles = take(max_tiles * 16), o_gu = take(Rp * 2 * inter * 4), o_act = take(Rp * inter * 4), o_dn = take(Rp * hidden * 4),
                 o_qx = take(Rp * 4 * hidden), o_qa = take(Rp * 4 * inter), o_sx = take(Rp * (hidden / 128) * 4), o_sa = take(Rp * (inter / 128) * 4),
                 o_lg = take((size_t)max_tokens * experts * 2), o_x = take((size_t)max_tokens * hidden * 2), o_o16 = take((size_t)max_tokens * hidden * 2),
                 o_o32 = take((size_t)max_tokens * hidden * 4), o_ps = take(plan_scratch_words((uint32_t)R, experts) * 4),
                 o_qt = take((size_t)max_tokens * 4 * hidden), o_stt = take((size_t)max_tokens * (hidden / 128) * 4), o_sched = take((max_tiles + 1) * 4);
    if (!cuda_ok(cudaMalloc(&w->base, off), "cudaMalloc(workspace)")) { free(w); return nullptr; }
    if (!cuda_ok(cudaMemset(w->base, 0, off), "cudaMemset(workspace)")) { cudaFree(w->base); free(w); return nullptr; }
    char *b = w->base;
    w->ids = (uint32_t *)(b + o_ids); w->wts = (float *)(b + o_wts); w->counts = (uint32_t *)(b + o_cnt); w->starts = (uint32_t *)(b + o_st);
    w->xmap = (uint32_t *)(b + o_xm); w->ymap = (uint32_t *)(b + o_ym); w->header = (uint32_t *)(b + o_hdr);
    w->seg_gu = (Seg32 *)(b + o_sgu); w->seg_dn = (Seg32 *)(b + o_sdn); w->tiles = (uint4 *)(b + o_tiles);
    w->gu = (float *)(b + o_gu); w->act = (float *)(b + o_act); w->dn = (float *)(b + o_dn);
    w->qx = (uint8_t *)(b + o_qx); w->qa = (uint8_t *)(b + o_qa); w->sx = (float *)(b + o_sx); w->sa = (float *)(b + o_sa);
    w->qt = (uint8_t *)(b + o_qt); w->stt = (float *)(b + o_stt); w->sched = (uint32_t *)(b + o_sched); w->sched_words = (uint32_t)(max_tiles + 1);
    w->plan_scratch = (uint32_t *)(b + o_ps); w->plan_scratch_words = plan_scratch_words((uint32_t)R, experts);
    w->logits = (uint16_t *)(b + o_lg); w->x = (uint16_t *)(b + o_x); w->out16 = (uint16_t *)(b + o_o16); w->out32 = (float *)(b + o_o32);
    return w;
}
static void workspace_release(Workspace *w) {
    if (!w || --w->refs > 0) return;
    if (w->base) cudaFree(w->base);
    free(w);
}

}  // namespace b200

struct OmegaGpuMoeLayer {
    const OmegaGpuFp8Tensor *gu, *dn;
    OmegaGpuMoeConfig cfg;
    uint32_t experts, hidden, inter;   // experts: what the tensors hold (the shared expert included)
    uint32_t shared, routed_topk;      // shared 1: cfg.topk counts the slots (routed_topk + 1) and the router chooses among experts - 1
    uint64_t *dir_gu, *dir_dn;   // device {w_va, s_va} per expert
    b200::Workspace *ws;
    uint32_t launches, marks;    // kernels of the last forward; profile marks of the last forward (a mark may cover several launches)
    cudaEvent_t *prof;           // when set: prof[i] is recorded after the i-th launch of a forward
    const char *names[12];
    alignas(128) unsigned char tm_gu[128], tm_dn[128], tm_qx[128], tm_qa[128];   // TMA descriptors (tensor-core engine)
    uint32_t tile_rows;
    bool wide_ok;                // single-piece activations and shapes the 128-row-tile kernel takes
};

namespace b200 {

// one forward, device pointers, stream-ordered. out32 required; out16 optional.
// routing given (ids_in / wts_in, [tokens][topk] on the device) or computed from the logits
bool layer_forward(OmegaGpuMoeLayer *L, uint32_t tokens, const uint16_t *logits, const uint16_t *x, float *out32, uint16_t *out16, cudaStream_t s,
                   const uint32_t *ids_in, const float *wts_in) {
    Workspace *w = L->ws;
    const uint32_t K = L->cfg.topk, E = L->experts, H = L->hidden, I = L->inter, R = tokens * K;
    uint32_t n = 0;
#define MARK(name) do { L->names[n] = name; if (L->prof) cudaEventRecord(L->prof[n + 1], s); n++; } while (0)
    if (L->prof) cudaEventRecord(L->prof[0], s);
    if (ids_in) {
        if (!cuda_ok(cudaMemcpyAsync(w->ids, ids_in, (size_t)R * 4, cudaMemcpyDeviceToDevice, s), "copy ids") ||
            !cuda_ok(cudaMemcpyAsync(w->wts, wts_in, (size_t)R * 4, cudaMemcpyDeviceToDevice, s), "copy weights")) return false;
        MARK("routing_copy");
    } else {
        if (!cuda_ok(launch_topk(tokens, E - L->shared, L->routed_topk, (int)L->cfg.norm_topk, logits, w->ids, w->wts, s, K), "topk launch")) return false;
        MARK("topk");
    }
    OmegaGpuMoePlanOut o = {};
    o.counts_va = (uint64_t)(uintptr_t)w->counts; o.starts_va = (uint64_t)(uintptr_t)w->starts;
    o.xmap_va = (uint64_t)(uintptr_t)w->xmap; o.ymap_va = (uint64_t)(uintptr_t)w->ymap; o.header_va = (uint64_t)(uintptr_t)w->header;
    o.seg_a_va = (uint64_t)(uintptr_t)w->seg_gu; o.dir_a_va = (uint64_t)(uintptr_t)L->dir_gu;
    o.seg_b_va = (uint64_t)(uintptr_t)w->seg_dn; o.dir_b_va = (uint64_t)(uintptr_t)L->dir_dn;
    const bool mma = L->cfg.engine == OMEGA_GPU_MOE_ENGINE_MMA;
    // prefill-sized segments (64 rows per expert on average, or on request) take the 128-row-tile kernel
    const bool wide = mma && L->wide_ok && (L->cfg.tile_rows == 128u || (L->cfg.tile_rows == 0u && R >= 64u * E));
    o.tiles_va = mma ? (uint64_t)(uintptr_t)w->tiles : 0;
    if (!cuda_ok(launch_plan(tokens, K, E, K, mma ? (wide ? mma_wide_tile_rows() : L->tile_rows) : 0, w->ids, o, s, w->plan_scratch, w->plan_scratch_words), "plan launch")) return false;
    MARK("plan");
    const uint32_t extra = plan_launch_count(R, E, w->plan_scratch, w->plan_scratch_words, o) - 1u;   // launches behind that one mark
    if (mma) {
        // activations as e4m3 pieces in sorted-row order, then the two tensor-core grouped GEMMs
        const uint32_t Px = L->cfg.x_pieces, Pa = L->cfg.act_pieces, Rp = w->max_tokens * w->topk + 8;
        uint32_t extra_q = 0;
        if (!cuda_ok(cudaMemsetAsync(w->sched, 0, (size_t)w->sched_words * 4, s), "clear work list")) return false;   // the one-launch expert kernel's tickets and tile counters
        if (K >= 4u && tokens >= 512u) {
            // many picks per token: quantise every token row once, then copy codes and scales into sorted-row order (the same bytes as
            // quantising each sorted row, a fraction of the arithmetic)
            if (!cuda_ok(launch_act_quant(tokens, H, Px, x, 1, nullptr, nullptr, w->qt, w->stt, s, 0, w->max_tokens), "x quant launch") ||
                !cuda_ok(launch_gather_rows(R, H, Px, w->max_tokens, Rp, w->xmap, w->header, w->qt, w->stt, w->qx, w->sx, s), "x gather launch")) return false;
            extra_q = 1;
        } else if (!cuda_ok(launch_act_quant(R, H, Px, x, 1, w->xmap, w->header, w->qx, w->sx, s, 0, Rp), "x quant launch")) return false;
        MARK("x_quant");
        // decode-shaped calls: the whole expert FFN in one launch (gate|up units, then down units from a work list cleared just before)
        static const bool two_launches = getenv("B200MOE_TWO_LAUNCH") != nullptr;
        if (!wide && !two_launches && ffn_shape_ok(H, I) && ((Px == 2 && Pa == 3) || (Px == 1 && Pa == 1) || (Px == 2 && Pa == 2))) {
            FfnLaunch f = {};
            f.gu_scale = L->gu->s; f.dn_scale = L->dn->s; f.x_scale = w->sx; f.qa = w->qa; f.sa = w->sa; f.tiles = w->tiles; f.header = w->header; f.ymap = w->ymap;
            f.out = w->dn; f.hidden = H; f.inter = I; f.q_rows = Rp; f.sched = w->sched; f.err = w->header + 4;
            // programmatic dependent of the quantiser before it (the work list was cleared ahead of that kernel): set-up and first weight tiles overlap it
            if (!cuda_ok(launch_ffn(L->tm_gu, L->tm_qx, L->tm_dn, L->tm_qa, Px, Pa, f, s, true), "expert ffn launch")) return false;
            MARK("expert_ffn_mma");
            if (!cuda_ok(launch_combine(tokens, K, H, w->wts, w->dn, out32, out16, s), "combine launch")) return false; MARK("combine");
            L->launches = n + extra + extra_q; L->marks = n;
            return true;
        }
        MmaLaunch g = {};
        g.wscale = L->gu->s; g.ascale = w->sx; g.tiles = w->tiles; g.header = w->header; g.ymap = nullptr; g.out = nullptr;
        g.q_out = w->qa; g.s_out = w->sa; g.q_rows = Rp; g.q_pieces = Pa;
        g.n = 2 * I; g.k = H; g.mode = 0; g.out_stride = I; g.err = w->header + 4;
        if (!cuda_ok(wide ? launch_mma_wide(L->tm_gu, L->tm_qx, g, s) : launch_mma_grouped(L->tm_gu, L->tm_qx, Px, g, s), "gate|up mma launch")) return false;
        MARK(wide ? "gate_up_mma_wide" : "gate_up_mma");
        MmaLaunch dd = {};
        dd.wscale = L->dn->s; dd.ascale = w->sa; dd.tiles = w->tiles; dd.header = w->header; dd.ymap = w->ymap; dd.out = w->dn; dd.q_rows = Rp;
        dd.n = H; dd.k = I; dd.mode = 1; dd.out_stride = H; dd.err = w->header + 4;
        if (!cuda_ok(wide ? launch_mma_wide(L->tm_dn, L->tm_qa, dd, s) : launch_mma_grouped(L->tm_dn, L->tm_qa, Pa, dd, s), "down mma launch")) return false;
        MARK(wide ? "down_mma_wide" : "down_mma");
        if (!cuda_ok(launch_combine(tokens, K, H, w->wts, w->dn, out32, out16, s), "combine launch")) return false; MARK("combine");
        L->launches = n + extra + extra_q; L->marks = n;
        return true;
    }
    // gate|up: sorted row p reads x[xmap[p]], writes gu row p
    GemvArgs a = {};
    a.seg = w->seg_gu; a.x = x; a.x_bf16 = 1; a.x_rows = tokens; a.xmap = w->xmap; a.ymap = nullptr;
    a.y = w->gu; a.n = 2 * I; a.k = H; a.groups_or_segs = E; a.rows = R; a.out_mul = 1.0f;
    if (!cuda_ok(launch_gemm_rows(a, nullptr, nullptr, s), "gate|up launch")) return false; MARK("gate_up_gemm");
    if (!cuda_ok(launch_swiglu(R, I, w->gu, w->act, s), "swiglu launch")) return false; MARK("swiglu");
    // down: sorted row p reads act row p, writes dn row ymap[p] = token * topk + slot
    GemvArgs d = {};
    d.seg = w->seg_dn; d.x = w->act; d.x_bf16 = 0; d.x_rows = R; d.xmap = nullptr; d.ymap = w->ymap;
    d.y = w->dn; d.n = H; d.k = I; d.groups_or_segs = E; d.rows = R; d.out_mul = 1.0f;
    if (!cuda_ok(launch_gemm_rows(d, nullptr, nullptr, s), "down launch")) return false; MARK("down_gemm");
    if (!cuda_ok(launch_combine(tokens, K, H, w->wts, w->dn, out32, out16, s), "combine launch")) return false; MARK("combine");
#undef MARK
    L->launches = n + extra; L->marks = n;
    return true;
}

bool layer_forward_routed(OmegaGpuMoeLayer *L, uint32_t rows, const uint32_t *ids, const void *x, size_t x_stride_bytes, float *dn, cudaStream_t s) {
    Workspace *w = L->ws;
    const uint32_t E = L->experts, H = L->hidden, I = L->inter;
    if (rows > w->max_tokens * w->topk) return false;
    uint32_t n = 0;
    OmegaGpuMoePlanOut o = {};
    o.counts_va = (uint64_t)(uintptr_t)w->counts; o.starts_va = (uint64_t)(uintptr_t)w->starts;
    o.xmap_va = (uint64_t)(uintptr_t)w->xmap; o.ymap_va = (uint64_t)(uintptr_t)w->ymap; o.header_va = (uint64_t)(uintptr_t)w->header;
    o.seg_a_va = (uint64_t)(uintptr_t)w->seg_gu; o.dir_a_va = (uint64_t)(uintptr_t)L->dir_gu;
    o.seg_b_va = (uint64_t)(uintptr_t)w->seg_dn; o.dir_b_va = (uint64_t)(uintptr_t)L->dir_dn;
    const bool mma = L->cfg.engine == OMEGA_GPU_MOE_ENGINE_MMA;
    o.tiles_va = mma ? (uint64_t)(uintptr_t)w->tiles : 0;
    if (!cuda_ok(launch_plan(rows, 1, E, 1, mma ? L->tile_rows : 0, ids, o, s), "plan launch")) return false; n++;
    if (mma) {
        const uint32_t Px = L->cfg.x_pieces, Pa = L->cfg.act_pieces, Rp = w->max_tokens * w->topk + 8;
        if (!cuda_ok(launch_act_quant(rows, H, Px, x, 1, w->xmap, w->header, w->qx, w->sx, s, x_stride_bytes, Rp), "x quant launch")) return false; n++;
        MmaLaunch g = {};
        g.wscale = L->gu->s; g.ascale = w->sx; g.tiles = w->tiles; g.header = w->header; g.out = nullptr;
        g.q_out = w->qa; g.s_out = w->sa; g.q_rows = Rp; g.q_pieces = Pa;
        g.n = 2 * I; g.k = H; g.mode = 0; g.out_stride = I; g.err = w->header + 4;
        if (!cuda_ok(launch_mma_grouped(L->tm_gu, L->tm_qx, Px, g, s), "gate|up mma launch")) return false; n++;
        MmaLaunch dd = {};
        dd.wscale = L->dn->s; dd.ascale = w->sa; dd.tiles = w->tiles; dd.header = w->header; dd.ymap = w->ymap; dd.out = dn; dd.q_rows = Rp;
        dd.n = H; dd.k = I; dd.mode = 1; dd.out_stride = H; dd.err = w->header + 4;
        if (!cuda_ok(launch_mma_grouped(L->tm_dn, L->tm_qa, Pa, dd, s), "down mma launch")) return false; n++;
    } else {
        GemvArgs a = {};
        a.seg = w->seg_gu; a.x = x; a.x_bf16 = 1; a.x_rows = rows; a.x_stride_bytes = x_stride_bytes; a.xmap = w->xmap;
        a.y = w->gu; a.n = 2 * I; a.k = H; a.groups_or_segs = E; a.rows = rows; a.out_mul = 1.0f;
        if (!cuda_ok(launch_gemm_rows(a, nullptr, nullptr, s), "gate|up launch")) return false; n++;
        if (!cuda_ok(launch_swiglu(rows, I, w->gu, w->act, s), "swiglu launch")) return false; n++;
        GemvArgs d = {};
        d.seg = w->seg_dn; d.x = w->act; d.x_rows = rows; d.ymap = w->ymap;
        d.y = dn; d.n = H; d.k = I; d.groups_or_segs = E; d.rows = rows; d.out_mul = 1.0f;
        if (!cuda_ok(launch_gemm_rows(d, nullptr, nullptr, s), "down launch")) return false; n++;
    }
    L->launches = n;
    return true;
}

// TMA descriptors of the weights (fixed) and of the workspace's piece buffers (rebuilt when the workspace changes)
static bool layer_build_maps(OmegaGpuMoeLayer *L) {
    if (L->cfg.engine != OMEGA_GPU_MOE_ENGINE_MMA) return true;
    const uint64_t Rp = (uint64_t)L->ws->max_tokens * L->cfg.topk + 8;
    return make_tmap_u8(L->tm_gu, L->gu->w, (uint64_t)L->experts * 2 * L->inter, L->hidden, 128) &&
           make_tmap_u8(L->tm_dn, L->dn->w, (uint64_t)L->experts * L->hidden, L->inter, 128) &&
           make_tmap_u8(L->tm_qx, L->ws->qx, Rp * L->cfg.x_pieces, L->hidden, 32) &&
           make_tmap_u8(L->tm_qa, L->ws->qa, Rp * L->cfg.act_pieces, L->inter, 32);
}

// dst drops its own workspace and uses src's (same shape, at least as many tokens); calls on them must then be stream-ordered
bool layer_share_workspace(OmegaGpuMoeLayer *dst, OmegaGpuMoeLayer *src) {
    if (dst->ws == src->ws) return true;
    if (dst->experts != src->experts || dst->hidden != src->hidden || dst->inter != src->inter || dst->cfg.topk != src->cfg.topk || dst->shared != src->shared ||
        dst->cfg.max_tokens > src->cfg.max_tokens) return false;
    workspace_release(dst->ws);
    dst->ws = src->ws; src->ws->refs++;
    return layer_build_maps(dst);
}
void layer_dims(const OmegaGpuMoeLayer *L, uint32_t *experts, uint32_t *hidden, uint32_t *max_tokens) { *experts = L->experts; *hidden = L->hidden; *max_tokens = L->cfg.max_tokens; }
void layer_view(OmegaGpuMoeLayer *L, LayerView *v) {
    v->engine = L->cfg.engine; v->topk = L->cfg.topk; v->experts = L->experts; v->hidden = L->hidden; v->inter = L->inter;
    v->x_pieces = L->cfg.x_pieces; v->act_pieces = L->cfg.act_pieces; v->tile_rows = L->tile_rows; v->max_tokens = L->ws->max_tokens;
    v->row_cap = L->ws->max_tokens * L->ws->topk + 8; v->norm_topk = L->cfg.norm_topk; v->shared = L->shared;
    v->gu_scale = L->gu->s; v->dn_scale = L->dn->s; v->tm_gu = L->tm_gu; v->tm_dn = L->tm_dn; v->tm_qa = L->tm_qa;
    v->qa = L->ws->qa; v->sa = L->ws->sa; v->dn = L->ws->dn;
}
float *layer_out32(OmegaGpuMoeLayer *L) { return L->ws->out32; }
uint16_t *layer_stage_x(OmegaGpuMoeLayer *L) { return L->ws->x; }

}  // namespace b200
using namespace b200;

extern "C" {

int omega_gpu_moe_layer_create(const OmegaGpuFp8Tensor *gate_up, const OmegaGpuFp8Tensor *down, const OmegaGpuMoeConfig *cfg, OmegaGpuMoeLayer **out) {
    if (out) *out = nullptr;
    if (!gate_up || !down || !cfg || !out) return OMEGA_GPU_FP8_BAD_ARGS;
    if (gate_up->experts != down->experts || gate_up->n != 2 * down->k || gate_up->k != down->n) { set_error("moe layer: gate|up [E][2I][H] and down [E][H][I] do not match"); return OMEGA_GPU_FP8_BAD_ARGS; }
    if (cfg->topk == 0 || cfg->topk > 31 || cfg->topk > gate_up->experts || cfg->max_tokens == 0 || gate_up->experts > 1024 || cfg->shared_expert > 1) return OMEGA_GPU_FP8_BAD_ARGS;
    if (cfg->shared_expert && (gate_up->experts < 2 || cfg->topk > gate_up->experts - 1)) return OMEGA_GPU_FP8_BAD_ARGS;
    if ((uint64_t)cfg->max_tokens * (cfg->topk + cfg->shared_expert) > (1u << 24)) return OMEGA_GPU_FP8_TOO_LARGE;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    OmegaGpuMoeLayer *L = (OmegaGpuMoeLayer *)calloc(1, sizeof *L);
    if (!L) return OMEGA_GPU_FP8_BAD_ARGS;
    L->gu = gate_up; L->dn = down; L->cfg = *cfg; L->experts = gate_up->experts; L->hidden = gate_up->k; L->inter = down->k;
    L->shared = cfg->shared_expert; L->routed_topk = cfg->topk; L->cfg.topk = cfg->topk + cfg->shared_expert;   // from here on topk = slots per token
    if (!L->cfg.x_pieces) L->cfg.x_pieces = 2;
    if (!L->cfg.act_pieces) L->cfg.act_pieces = 3;
    if (L->cfg.x_pieces > 4 || L->cfg.act_pieces > 4) { free(L); return OMEGA_GPU_FP8_BAD_ARGS; }
    const bool mma_ok = mma_shape_ok(2 * L->inter, L->hidden, 0) && mma_shape_ok(L->hidden, L->inter, 1);
    if (L->cfg.engine == OMEGA_GPU_MOE_ENGINE_AUTO) L->cfg.engine = mma_ok ? OMEGA_GPU_MOE_ENGINE_MMA : OMEGA_GPU_MOE_ENGINE_FMA;
    if (L->cfg.engine == OMEGA_GPU_MOE_ENGINE_MMA && !mma_ok) { free(L); set_error("moe layer: shape outside the tensor-core engine (k <= 4096, even number of 128-row blocks)"); return OMEGA_GPU_FP8_BAD_ARGS; }
    L->tile_rows = mma_tile_rows(L->cfg.x_pieces > L->cfg.act_pieces ? L->cfg.x_pieces : L->cfg.act_pieces);
    L->wide_ok = L->cfg.engine == OMEGA_GPU_MOE_ENGINE_MMA && L->cfg.x_pieces == 1 && L->cfg.act_pieces == 1 && mma_wide_shape_ok(2 * L->inter, L->hidden, 0) &&
                 mma_wide_shape_ok(L->hidden, L->inter, 1);
    if ((L->cfg.tile_rows != 0 && L->cfg.tile_rows != 32 && L->cfg.tile_rows != 128) || (L->cfg.tile_rows == 128 && !L->wide_ok)) {
        free(L); set_error("moe layer: tile_rows must be 0, 32 or 128; 128 needs the tensor-core engine, x_pieces = act_pieces = 1 and k <= 2048"); return OMEGA_GPU_FP8_BAD_ARGS;
    }
    const uint32_t E = L->experts;
    std::vector<uint64_t> dir((size_t)E * 4);
    for (uint32_t e = 0; e < E; e++) {
        (void)omega_gpu_fp8_tensor_entry(gate_up, e, &dir[2 * e], &dir[2 * e + 1]);
        (void)omega_gpu_fp8_tensor_entry(down, e, &dir[2 * E + 2 * e], &dir[2 * E + 2 * e + 1]);
    }
    bool ok = cuda_ok(cudaMalloc(&L->dir_gu, (size_t)E * 32), "cudaMalloc(directory)");
    if (ok) { L->dir_dn = L->dir_gu + 2 * E; ok = cuda_ok(cudaMemcpy(L->dir_gu, dir.data(), (size_t)E * 32, cudaMemcpyHostToDevice), "copy directory"); }
    if (ok) { L->ws = workspace_create(cfg->max_tokens, L->cfg.topk, E, L->hidden, L->inter); ok = L->ws != nullptr; }
    if (ok) ok = layer_build_maps(L);
    if (!ok) { if (L->dir_gu) cudaFree(L->dir_gu); free(L); return OMEGA_GPU_FP8_CHIP_FAIL; }
    *out = L;
    return OMEGA_GPU_FP8_OK;
}

void omega_gpu_moe_layer_free(OmegaGpuMoeLayer *L) {
    if (!L) return;
    Lock l;
    workspace_release(L->ws);
    if (L->dir_gu) cudaFree(L->dir_gu);
    free(L);
}

uint32_t omega_gpu_moe_layer_launches(const OmegaGpuMoeLayer *L) { return L ? L->launches : 0; }

int omega_gpu_moe_layer_async(OmegaGpuMoeLayer *L, uint32_t tokens, uint64_t logits_va, uint64_t x_va, uint64_t out_f32_va, uint64_t out_bf16_va, void *stream) {
    if (!L || !tokens || !logits_va || !x_va || !out_f32_va) return OMEGA_GPU_FP8_BAD_ARGS;
    if (tokens > L->cfg.max_tokens) return OMEGA_GPU_FP8_TOO_LARGE;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    return layer_forward(L, tokens, (const uint16_t *)(uintptr_t)logits_va, (const uint16_t *)(uintptr_t)x_va, (float *)(uintptr_t)out_f32_va,
                         (uint16_t *)(uintptr_t)out_bf16_va, (cudaStream_t)stream) ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_layer_routed_async(OmegaGpuMoeLayer *L, uint32_t tokens, uint64_t ids_va, uint64_t wts_va, uint64_t x_va, uint64_t out_f32_va, uint64_t out_bf16_va,
                                     void *stream) {
    if (!L || !tokens || !ids_va || !wts_va || !x_va || !out_f32_va) return OMEGA_GPU_FP8_BAD_ARGS;
    if (tokens > L->cfg.max_tokens) return OMEGA_GPU_FP8_TOO_LARGE;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    return layer_forward(L, tokens, nullptr, (const uint16_t *)(uintptr_t)x_va, (float *)(uintptr_t)out_f32_va, (uint16_t *)(uintptr_t)out_bf16_va, (cudaStream_t)stream,
                         (const uint32_t *)(uintptr_t)ids_va, (const float *)(uintptr_t)wts_va) ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_layer_profile(OmegaGpuMoeLayer *L, uint32_t tokens, uint64_t logits_va, uint64_t x_va, uint64_t out_f32_va, uint32_t cap,
                                float *ms, const char **names, uint32_t *count) {
    if (!L || !tokens || !logits_va || !x_va || !out_f32_va || !ms || !count || cap == 0) return OMEGA_GPU_FP8_BAD_ARGS;
    if (tokens > L->cfg.max_tokens) return OMEGA_GPU_FP8_TOO_LARGE;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaEvent_t ev[13];
    for (auto &e : ev) if (!cuda_ok(cudaEventCreate(&e), "cudaEventCreate")) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = st().stream;
    L->prof = ev;
    bool ok = layer_forward(L, tokens, (const uint16_t *)(uintptr_t)logits_va, (const uint16_t *)(uintptr_t)x_va, (float *)(uintptr_t)out_f32_va, nullptr, s);
    L->prof = nullptr;
    ok = ok && cuda_ok(cudaStreamSynchronize(s), "moe layer profile");
    *count = 0;
    for (uint32_t i = 0; ok && i < L->marks && i < cap; i++) {
        float t = 0; ok = cuda_ok(cudaEventElapsedTime(&t, ev[i], ev[i + 1]), "event time");
        ms[i] = t; if (names) names[i] = L->names[i]; *count = i + 1;
    }
    for (auto &e : ev) cudaEventDestroy(e);
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_layer_bf16(OmegaGpuMoeLayer *L, uint32_t tokens, const uint16_t *logits, const uint16_t *x, uint16_t *out_bf16, float *out_f32,
                             uint32_t *ids, float *wts) {
    if (!L || !tokens || !logits || !x || (!out_bf16 && !out_f32)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (tokens > L->cfg.max_tokens) return OMEGA_GPU_FP8_TOO_LARGE;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    Workspace *w = L->ws; cudaStream_t s = st().stream;
    const size_t lb = (size_t)tokens * (L->experts - L->shared) * 2, xb = (size_t)tokens * L->hidden * 2, rb = (size_t)tokens * L->cfg.topk * 4;
    bool ok = cuda_ok(cudaMemcpyAsync(w->logits, logits, lb, cudaMemcpyHostToDevice, s), "copy logits") &&
              cuda_ok(cudaMemcpyAsync(w->x, x, xb, cudaMemcpyHostToDevice, s), "copy x") &&
              layer_forward(L, tokens, w->logits, w->x, w->out32, w->out16, s);
    if (ok && out_bf16) ok = cuda_ok(cudaMemcpyAsync(out_bf16, w->out16, xb, cudaMemcpyDeviceToHost, s), "copy out");
    if (ok && out_f32) ok = cuda_ok(cudaMemcpyAsync(out_f32, w->out32, xb * 2, cudaMemcpyDeviceToHost, s), "copy out");
    if (ok && ids) ok = cuda_ok(cudaMemcpyAsync(ids, w->ids, rb, cudaMemcpyDeviceToHost, s), "copy ids");
    if (ok && wts) ok = cuda_ok(cudaMemcpyAsync(wts, w->wts, rb, cudaMemcpyDeviceToHost, s), "copy weights");
    uint32_t hdr[8] = {0};
    ok = ok && cuda_ok(cudaMemcpyAsync(hdr, w->header, 32, cudaMemcpyDeviceToHost, s), "copy status") && cuda_ok(cudaStreamSynchronize(s), "moe layer");
    if (ok && hdr[3]) { set_error("moe layer: routing plan refused (status %u)", hdr[3]); return OMEGA_GPU_FP8_BAD_ARGS; }
    if (ok && hdr[4]) { set_error("moe layer: a bounded wait inside the tensor-core kernel ran out (code %u)", hdr[4]); st().latched = true; return OMEGA_GPU_FP8_CHIP_FAIL; }
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

// Status of the stream-ordered entries (which never block): waits for `stream`, then returns 0, 100 + the routing plan's refusal, or the
// code of a bounded wait that ran out inside a tensor-core kernel (that word is sticky: the process latches, as the blocking entry does).
int omega_gpu_moe_layer_status(OmegaGpuMoeLayer *L, void *stream) {
    if (!L) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    uint32_t hdr[8] = {0};
    if (!cuda_ok(cudaMemcpyAsync(hdr, L->ws->header, 32, cudaMemcpyDeviceToHost, (cudaStream_t)stream), "copy status") ||
        !cuda_ok(cudaStreamSynchronize((cudaStream_t)stream), "moe layer status")) return OMEGA_GPU_FP8_CHIP_FAIL;
    if (hdr[4]) { set_error("moe layer: a bounded wait inside the tensor-core kernel ran out (code %u)", hdr[4]); st().latched = true; return (int)hdr[4]; }
    return hdr[3] ? 100 + (int)hdr[3] : 0;
}

}  // extern "C"
