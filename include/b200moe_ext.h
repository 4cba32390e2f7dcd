/*
 * b200moe_ext.h: entry points with no same-named counterpart in the reference: the router top-k on given logits,
 * the device-resident routing plan at any token count, the glue operators as single calls, the W4 GEMM, and the
 * whole quantized MoE layer / layer stack. Each cites the reference operator whose arithmetic it carries.
 *
 * Forms: a name ending in _async takes device addresses and a cudaStream_t (as void *) and neither copies nor
 * synchronises; every other entry takes HOST buffers, stages them, runs the kernels and copies the result back.
 * Return codes are the OMEGA_GPU_FP8_* values of b200moe_fp8.h; the failing stage is in omega_gpu_fp8_last_error().
 */
#ifndef B200MOE_EXT_H
#define B200MOE_EXT_H
#include "b200moe_fp8gemm.h"
#ifdef __cplusplus
extern "C" {
#endif

/* ---- device-resident forms of upload and quantise (weights produced on the GPU, e.g. synthetic benchmark data).
 * Same rules as omega_gpu_fp8_tensor_upload / omega_gpu_fp8_quantize_bf16; the sources are device addresses and are
 * copied, so the caller may free them afterwards. Synchronous. */
int omega_gpu_fp8_tensor_upload_dev(uint32_t experts, uint32_t n, uint32_t k, uint64_t w_va, uint64_t scale_inv_bf16_va,
                                    OmegaGpuFp8Tensor **out);
int omega_gpu_fp8_quantize_bf16_dev(uint32_t n, uint32_t k, uint64_t w_bf16_va, uint64_t w8_va, uint64_t scale_inv_bf16_va);

/* ---- router top-k on given logits: k rounds of "largest remaining, lowest index on ties", ids in selection order,
 * weights = softmax over the selected logits (norm_topk) or over all experts (src/omega_blackwell_codegen_router.c:298-401,
 * oracle tests/gpu_router_test.c:62-79). logits bf16 [tokens][experts], experts <= 1024, topk <= 32. */
int omega_gpu_moe_topk_bf16(uint32_t tokens, uint32_t experts, uint32_t topk, int norm_topk, const uint16_t *logits_bf16,
                            uint32_t *ids, float *wts);
int omega_gpu_moe_topk_async(uint32_t tokens, uint32_t experts, uint32_t topk, int norm_topk, uint64_t logits_va,
                             uint64_t ids_va, uint64_t wts_va, void *stream);

/* ---- routing plan, device u32 form, any token count (the on-chip GROUP of src/omega_blackwell_codegen_dec.c:534-651
 * and the host GROUP of src/omega_gpu_q36_graph.c:1107-1144, same ordering rule: expert, token, slot).
 * ids u32 [tokens][slots] (0xFFFFFFFF = absent). Outputs: counts[experts], starts[experts] (exclusive scan),
 * xmap[rows+8] = token, ymap[rows+8] = token*ystride+slot (8 zero pads), seg: 32-byte records for the non-empty
 * experts in ascending id built from the two directories ({w_va, s_va} per expert), records past the last
 * non-empty expert up to `experts` zeroed; tiles: one {expert, row0, cnt} u32 x4 entry per `tile_rows` slice of
 * a segment (tile_rows 0 = none); header u32[8] = {rows, segments, tiles, status, w, 0, 0, 0}; status 2 = id out of range; word w is
 * left as it is (the kernels that consume a plan record an expired bounded wait there: zero it once, when the buffer is made). */
typedef struct {
    uint64_t counts_va, starts_va, xmap_va, ymap_va;
    uint64_t seg_a_va, dir_a_va; /* first projection's segment records and {w_va, s_va} directory (may be 0) */
    uint64_t seg_b_va, dir_b_va; /* second projection's (may be 0) */
    uint64_t tiles_va;           /* u32 x4 per tile (may be 0) */
    uint64_t header_va;          /* u32[8] */
} OmegaGpuMoePlanOut;
int omega_gpu_moe_plan_async(uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, uint32_t tile_rows,
                             uint64_t ids_va, const OmegaGpuMoePlanOut *out, void *stream);
/* host form for tests: returns rows/segments through the arrays; seg3 = {expert, row0, cnt} per segment */
int omega_gpu_moe_plan_u32(uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, const uint32_t *ids,
                           uint32_t *counts, uint32_t *starts, uint32_t *xmap, uint32_t *ymap, uint32_t *seg3,
                           uint32_t *rows, uint32_t *segments);

/* ---- glue operators as single host calls (parity with the reference's separate launches) */
/* act[r][c] = silu(gu[r][c]) * gu[r][inter + c] (src/omega_blackwell_codegen_dec.c:291-324) */
int omega_gpu_swiglu_f32(uint32_t rows, uint32_t inter, const float *gu, float *act);
/* out[t] = sum over slots of w[t][s] * d[t][s], multiply then add in slot order, never fused
 * (src/omega_blackwell_codegen_dec.c:226-255) */
int omega_gpu_moe_combine_f32(uint32_t tokens, uint32_t slots, uint32_t hidden, const float *w, const float *d, float *out);
/* per row, per 128 columns: power-of-two scale, e4m3 codes (src/omega_blackwell_codegen_qg.h:7-19). pieces > 1
 * adds residual pieces at scale/16^p (this library's exact-activation format). q: [pieces][rows][k] (piece-major). */
int omega_gpu_act_quant_f32(uint32_t rows, uint32_t k, uint32_t pieces, const float *x, uint8_t *q, float *s);

/* ---- W4: signed int4 weights, two per byte along K (low nibble = even column), fp16 scale per 32 columns.
 * The reference has no integer-W4 arithmetic (docs/models/QUANT.md:62); this follows the benchmark definition. */
typedef struct OmegaGpuW4Tensor OmegaGpuW4Tensor;
int omega_gpu_w4_upload(uint32_t n, uint32_t k, const uint8_t *packed, const uint16_t *scale_f16, OmegaGpuW4Tensor **out);
void omega_gpu_w4_free(OmegaGpuW4Tensor *t);
/* ---- MXFP4 weights: E2M1 nibbles (two per byte along K, low nibble = even column) with one E8M0 scale byte per 32 columns, the format of the
 * reference's docs/models/MXFP4.md; every element's value is what its scalar decoder native/models/mxfp4.om returns (checked against that unit's
 * own verification oracle). packed [n][k/2], scale_e8m0 [n][k/32]; scale 255 (a NaN block) is refused with NAN_WEIGHT. n a multiple of 128,
 * k 768, 1024, 2048 or 4096. The tensor is used with omega_gpu_w4_gemm_bf16 / _async and freed with omega_gpu_w4_free. The product y = x W^T: per
 * group the sum of x * element, times 2^(scale - 127), accumulated in f32; with activations that are themselves MXFP4 values (element x scale, exact in
 * bf16) this is the reference's block-scaled product (native/models/mxdot.om `mxmm`) up to the rounding of the f32 running sum. */
int omega_gpu_mxfp4_upload(uint32_t n, uint32_t k, const uint8_t *packed, const uint8_t *scale_e8m0, OmegaGpuW4Tensor **out);
/* NVFP4 weights: E2M1 nibbles [n][k/2] (low nibble = even column) and one unsigned E4M3 scale per 16 columns [n][k/16], the reference's
 * native/models/nvfp4.om (docs/models/MXFMT.md); an element's value is what its nvfp4bits returns; no second-level per-tensor scale, as there.
 * Scale 127 (NaN) -> NAN_WEIGHT, a scale with the sign bit set -> BAD_ARGS (that unit refuses both); n % 128 == 0, k 768, 1024, 2048 or 4096.
 * The tensor runs through omega_gpu_w4_gemm_bf16 / _async. */
int omega_gpu_nvfp4_upload(uint32_t n, uint32_t k, const uint8_t *packed, const uint8_t *scale_ue4m3, OmegaGpuW4Tensor **out);
/* bf16 rows [rows][k] (host, k % 16 == 0) -> NVFP4 codes and scales on the GPU, bit for bit what the reference's block encoder gives (native/models/nvfp4.om
 * nvfp4nib: scale = e4m3(amax / 6) nearest even and saturating, element = nearest even E2M1 of x / scale, above 6 and infinity saturate). A NaN value refuses
 * the call with NAN_WEIGHT and writes nothing. packed [rows][k / 2] (element 2i in the low nibble), scale_ue4m3 [rows][k / 16]. */
int omega_gpu_nvfp4_quantize_bf16(uint32_t rows, uint32_t k, const uint16_t *w_bf16, uint8_t *packed, uint8_t *scale_ue4m3);
/* y bf16 [m][n] = x bf16 [m][k] * W^T, f32 accumulation; yf32 (optional) receives the unrounded values */
int omega_gpu_w4_gemm_bf16(const OmegaGpuW4Tensor *t, uint32_t m, const uint16_t *x_bf16, uint16_t *y_bf16, float *y_f32);
/* the same on device buffers, stream-ordered (one of y_bf16_va / y_f32_va may be 0) */
int omega_gpu_w4_gemm_async(const OmegaGpuW4Tensor *t, uint32_t m, uint64_t x_bf16_va, uint64_t y_bf16_va, uint64_t y_f32_va, void *stream);
/* Grouped by expert (4-bit expert weights): the tensor was uploaded as experts x n_per_expert rows (expert e's matrix = rows [e n, (e + 1) n)). The rows to
 * multiply are described by a routing plan made with tile_rows = 16 (omega_gpu_moe_plan_async): tiles u32 x4 {expert, first sorted row, rows <= 16, -},
 * header[2] = number of tiles. Activation row i of a tile is x[xmap[first + i]] (xmap_va 0: x[first + i]), bf16 [.][k]; its result row (n_per_expert wide) is
 * y[ymap[first + i]] (ymap_va 0: y[first + i]). omega_gpu_w4_reserve_grouped allocates the per-tile scratch once for at most max_tiles tiles (blocking);
 * the async entry queues one launch of max_tiles x n / 128 x 4 CTAs (tiles past header[2] return at once) and allocates nothing. */
int omega_gpu_w4_reserve_grouped(OmegaGpuW4Tensor *t, uint32_t n_per_expert, uint32_t max_tiles);
int omega_gpu_w4_gemm_grouped_async(const OmegaGpuW4Tensor *t, uint64_t tiles_va, uint64_t header_va, uint64_t xmap_va, uint64_t ymap_va,
                                    uint64_t x_bf16_va, uint64_t y_bf16_va, uint64_t y_f32_va, void *stream);

/* ---- one MoE layer with 4-bit expert weights (any of the three formats above; MXFP4 and NVFP4 are the reference's own 4-bit expert formats).
 * gate_up: experts x 2I rows of k = hidden (gate rows first, then up rows, per expert); down: experts x hidden rows of k = I; both uploaded with the
 * upload entry of their format, not owned by the layer and not usable by another layer at the same time (the layer reserves their grouped scratch).
 * hidden and I in {768, 1024, 2048, 4096}. Steps: top-k of the bf16 logits (the reference's selection rule), routing plan, grouped gate|up, SiLU gate
 * rounded to bf16, grouped down, slot-order combine; 6 launches. */
typedef struct OmegaGpuMoeW4Layer OmegaGpuMoeW4Layer;
int omega_gpu_moe_w4_layer_create(OmegaGpuW4Tensor *gate_up, OmegaGpuW4Tensor *down, uint32_t experts, uint32_t topk, uint32_t max_tokens, int norm_topk,
                                  OmegaGpuMoeW4Layer **out);
void omega_gpu_moe_w4_layer_free(OmegaGpuMoeW4Layer *l);
int omega_gpu_moe_w4_layer_bf16(OmegaGpuMoeW4Layer *l, uint32_t tokens, const uint16_t *logits_bf16, const uint16_t *x_bf16, uint16_t *out_bf16, float *out_f32,
                                uint32_t *ids, float *wts);
int omega_gpu_moe_w4_layer_async(OmegaGpuMoeW4Layer *l, uint32_t tokens, uint64_t logits_va, uint64_t x_va, uint64_t out_f32_va, uint64_t out_bf16_va, void *stream);
uint32_t omega_gpu_moe_w4_layer_launches(const OmegaGpuMoeW4Layer *l);

/* ---- the MoE layer: top-k -> plan -> gate|up grouped GEMM + SiLU gate -> down grouped GEMM -> weighted combine
 * (the MoE part of src/omega_gpu_decode_graph.c:341-351 for decode, src/omega_gpu_q36_graph.c:1147 for prefill). */
typedef struct OmegaGpuMoeLayer OmegaGpuMoeLayer;
enum { OMEGA_GPU_MOE_ENGINE_AUTO = 0, OMEGA_GPU_MOE_ENGINE_FMA = 1, OMEGA_GPU_MOE_ENGINE_MMA = 2 };
typedef struct {
    uint32_t topk;        /* 8 */
    uint32_t max_tokens;  /* scratch is sized for this many tokens per call */
    uint32_t engine;      /* AUTO, FMA (CUDA-core, reference summation order) or MMA (tcgen05 FP8 tensor cores) */
    uint32_t x_pieces;    /* MMA: e4m3 pieces per bf16 input value (2 = exact, 1 = plain FP8 activations); 0 = 2 */
    uint32_t act_pieces;  /* MMA: pieces per f32 SwiGLU output (0 = 3) */
    uint32_t norm_topk;   /* 1: weights renormalised over the selected experts */
    uint32_t first_expert, local_experts; /* expert-parallel shard held here; 0, 0 = all */
    uint32_t tile_rows;   /* tensor-core engine, rows per routed-row tile: 0 = chosen per call (128 once a call brings 64 rows per expert on average and
                             x_pieces = act_pieces = 1, else 32), 32 = always 32, 128 = always 128 (refused unless x_pieces = act_pieces = 1, k <= 2048) */
    uint32_t shared_expert; /* 1: the two tensors hold one expert more than the router routes over, the LAST one being the shared expert every token
                             goes through (the reference's ninth group: src/omega_gpu_q36_graph.h:7-21, :53-55, :87). A token then has topk + 1
                             slots: logits are [tokens][experts - 1], ids / wts are [tokens][topk + 1], slot topk holds id experts - 1; its weight is 1
                             from the logits entries, or what the caller / the router's shared gate supplies through the routed entry. The routing
                             plan puts the shared rows in the last segment (om/moe/moe_plan.om:112-117) and the combine runs over topk + 1 slots. */
} OmegaGpuMoeConfig;
/* gate_up: [E][2I][H] (gate rows first), down: [E][H][I]; both stay owned by the caller and must outlive the layer */
int omega_gpu_moe_layer_create(const OmegaGpuFp8Tensor *gate_up, const OmegaGpuFp8Tensor *down, const OmegaGpuMoeConfig *cfg,
                               OmegaGpuMoeLayer **out);
void omega_gpu_moe_layer_free(OmegaGpuMoeLayer *l);
/* host buffers: logits bf16 [tokens][E], x bf16 [tokens][H] -> out bf16 [tokens][H]; out_f32, ids, wts optional */
int omega_gpu_moe_layer_bf16(OmegaGpuMoeLayer *l, uint32_t tokens, const uint16_t *logits_bf16, const uint16_t *x_bf16,
                             uint16_t *out_bf16, float *out_f32, uint32_t *ids, float *wts);
/* device buffers, stream-ordered: out_f32_va f32 [tokens][H] (required), out_bf16_va optional (0 = skip) */
int omega_gpu_moe_layer_async(OmegaGpuMoeLayer *l, uint32_t tokens, uint64_t logits_va, uint64_t x_va, uint64_t out_f32_va,
                              uint64_t out_bf16_va, void *stream);
/* the same forward with the routing given: ids_va u32 [tokens][topk] and wts_va f32 [tokens][topk] on the device (the outputs of
 * omega_gpu_moe_router_rows_async), x_va the bf16 input rows; an id outside the layer's experts makes the plan refuse (header status) */
int omega_gpu_moe_layer_routed_async(OmegaGpuMoeLayer *l, uint32_t tokens, uint64_t ids_va, uint64_t wts_va, uint64_t x_va, uint64_t out_f32_va,
                                     uint64_t out_bf16_va, void *stream);
/* status of the two stream-ordered entries above: waits for `stream`; 0, 100 + the routing plan's status, or the code of a bounded wait
 * that ran out inside a kernel (sticky; the process is latched, as by the blocking entry) */
int omega_gpu_moe_layer_status(OmegaGpuMoeLayer *l, void *stream);
/* One forward on the library's stream with a CUDA event between consecutive launches: ms[i] = device time of the i-th
 * kernel (launch order), names[i] = its static name; *count entries (at most cap). For measurement. */
int omega_gpu_moe_layer_profile(OmegaGpuMoeLayer *l, uint32_t tokens, uint64_t logits_va, uint64_t x_va, uint64_t out_f32_va,
                                uint32_t cap, float *ms, const char **names, uint32_t *count);
/* number of kernels the last forward of this layer launched */
uint32_t omega_gpu_moe_layer_launches(const OmegaGpuMoeLayer *l);

/* ---- a stack of MoE layers, the MoE part of the reference's whole-token decode graph (src/omega_gpu_decode_graph.c:321-351):
 * h = x; per layer: xn = bf16(RMSNorm(h) * norm weight of the layer) (sum of squares in double as the reference host glue,
 * tests/gpu_decode_graph_test.c:56-60), h = h + MoE_l(xn, logits_l). Router logits are inputs (one [tokens][E] block per
 * layer). Layers of one stack share one scratch workspace and run as one CUDA graph per token count. */
typedef struct OmegaGpuMoeStack OmegaGpuMoeStack;
typedef struct OmegaGpuMoeRouter OmegaGpuMoeRouter;   /* the router front half, further down */
int omega_gpu_moe_stack_create(uint32_t layers, OmegaGpuMoeLayer *const *layer, float eps, OmegaGpuMoeStack **out);
void omega_gpu_moe_stack_free(OmegaGpuMoeStack *s);
/* host buffers: logits bf16 [layers][tokens][E], x bf16 [tokens][H] -> out bf16 [tokens][H] (final h), out_f32 optional */
int omega_gpu_moe_stack_bf16(OmegaGpuMoeStack *s, uint32_t tokens, const uint16_t *logits_bf16, const uint16_t *x_bf16,
                             uint16_t *out_bf16, float *out_f32);
/* device buffers, stream-ordered (captures and replays a graph on `stream`) */
int omega_gpu_moe_stack_async(OmegaGpuMoeStack *s, uint32_t tokens, uint64_t logits_va, uint64_t x_va, uint64_t out_f32_va,
                              uint64_t out_bf16_va, void *stream);
uint32_t omega_gpu_moe_stack_launches(const OmegaGpuMoeStack *s);
/* RMSNorm weight of layer `layer`'s input, f32 [hidden] on the host (copied): xn = bf16(h * rsqrt(mean(h^2) + eps) * norm_w), the
 * reference's RES COMBINE|NORM with the layer's norm weight (src/omega_blackwell_codegen_dec.c:261-286; host form
 * tests/gpu_decode_graph_test.c:56-60). Every layer starts with unit weights. Takes effect at the next step. */
int omega_gpu_moe_stack_set_norm(OmegaGpuMoeStack *s, uint32_t layer, const float *norm_w);
/* Router inside the stack, the reference's own per-layer order (src/omega_gpu_decode_graph.c:341-351: router -> experts -> RES COMBINE|NORM).
 * Once EVERY layer has a router (omega_gpu_moe_router_create: the layer's gate matrix and the norm weight of its input), the stack takes no
 * logits (pass NULL / 0): per layer it adds the combine of the layer before to the residual stream, runs the router on it (RMSNorm with
 * the router's norm weight -> bf16 xn, logits, top-k), plans, quantises xn into the plan's sorted rows and runs the experts. The routers
 * stay owned by the caller and must outlive the stack; router NULL takes a layer's router away again (the stack then wants logits).
 * Tensor-core engine only. Weights set with omega_gpu_moe_stack_set_norm are not used in this mode (the router carries the norm weight). */
int omega_gpu_moe_stack_set_router(OmegaGpuMoeStack *s, uint32_t layer, OmegaGpuMoeRouter *router);
/* One step launched without the graph, a CUDA event before and after each layer's expert kernel(s): expert_ms[l] = device
 * time of layer l's gate|up + down work (one launch when *launches_per_layer is 1). Tensor-core path only. For measurement. */
int omega_gpu_moe_stack_profile(OmegaGpuMoeStack *s, uint32_t tokens, uint64_t logits_va, uint64_t x_va, uint32_t cap, float *expert_ms,
                                uint32_t *count, uint32_t *launches_per_layer);

/* ---- residual stream step as one call (the stack uses it; exposed for callers that drive layers themselves):
 * h = (x16 ? bf16->f32(x16) : h) + (m ? m : 0); xn = bf16(RMSNorm(h)) when xn_va != 0; h16 = bf16(h) when h16_va != 0 */
int omega_gpu_residual_norm_async(uint32_t tokens, uint32_t hidden, float eps, uint64_t x16_va, uint64_t m_va, uint64_t h_va,
                                  uint64_t xn_va, uint64_t h16_va, void *stream);
/* the same with the norm weight vector: norm_w_va f32 [hidden] on the device (0 = unit weights); xn = bf16(h * s * w) */
int omega_gpu_residual_norm_w_async(uint32_t tokens, uint32_t hidden, float eps, uint64_t x16_va, uint64_t m_va, uint64_t h_va,
                                    uint64_t xn_va, uint64_t h16_va, uint64_t norm_w_va, void *stream);

/* ---- expert parallelism over the GPUs of one node (no counterpart in the reference, which runs one device).
 * Rank r of `world` holds experts [r*E/world, (r+1)*E/world) as an ordinary OmegaGpuMoeLayer over its local tensors
 * (created with max_tokens >= world * tokens_local_max + 1) and a slice of the tokens. One OmegaGpuMoeEp per rank holds
 * the exchange buffers, shared by all layers. Per layer the caller runs dispatch -> [all-to-all send->recv] -> experts
 * -> [all-to-all dn->back] -> combine; the two collectives (equal chunks of buffers[4] and buffers[5] bytes per rank)
 * are the caller's (NCCL). After omega_gpu_moe_ep_connect the rows instead travel by direct peer stores inside
 * dispatch/experts and no collective is needed. Outputs equal the single-GPU layer's. */
typedef struct OmegaGpuMoeEp OmegaGpuMoeEp;
int omega_gpu_moe_ep_create(uint32_t world, uint32_t rank, uint32_t experts, uint32_t topk, uint32_t hidden, uint32_t tokens_local_max,
                            OmegaGpuMoeEp **out);
void omega_gpu_moe_ep_free(OmegaGpuMoeEp *ep);
/* out[0..7] = send_va, recv_va, dn_va, back_va, activation chunk bytes, result chunk bytes, comm block va, comm block bytes */
int omega_gpu_moe_ep_buffers(const OmegaGpuMoeEp *ep, uint64_t *out);
/* 64-byte inter-process handle of this rank's comm block; connect takes world x 64 bytes in rank order */
int omega_gpu_moe_ep_export(const OmegaGpuMoeEp *ep, uint8_t *handle64);
int omega_gpu_moe_ep_connect(OmegaGpuMoeEp *ep, const uint8_t *handles);
int omega_gpu_moe_ep_dispatch_async(OmegaGpuMoeEp *ep, uint32_t tokens_local, uint64_t logits_va, uint64_t x_va, void *stream);
int omega_gpu_moe_ep_experts_async(OmegaGpuMoeEp *ep, OmegaGpuMoeLayer *local, void *stream);
int omega_gpu_moe_ep_combine_async(OmegaGpuMoeEp *ep, uint32_t tokens_local, uint64_t out_f32_va, uint64_t out_bf16_va, void *stream);
/* synchronises `stream`; 0, or the code of a bounded cross-GPU wait that ran out (11 dispatch, 12 return) */
int omega_gpu_moe_ep_status(OmegaGpuMoeEp *ep, void *stream);

/* ---- fused expert-parallel stack: two launches per layer and rank (three with the two-launch expert path), rows and results travel by peer stores, waits are
 * counters advanced with system-scope atomics (bounded). local[l]: rank's layer l over its experts/world experts, tensor-core
 * engine, max_tokens >= tokens (all ranks' tokens). After create: export this rank's handle, gather all ranks' handles,
 * connect (world 1 needs neither). Per step the caller gathers the router logits of ALL tokens ([layers][tokens][experts]
 * bf16) and calls step_async on every rank; outputs are bit-identical to the single-GPU stack. */
typedef struct OmegaGpuMoeEpStack OmegaGpuMoeEpStack;
int omega_gpu_moe_epstack_create(uint32_t world, uint32_t rank, uint32_t layers, OmegaGpuMoeLayer *const *local, uint32_t experts,
                                 uint32_t tokens, float eps, OmegaGpuMoeEpStack **out);
void omega_gpu_moe_epstack_free(OmegaGpuMoeEpStack *s);
int omega_gpu_moe_epstack_export(const OmegaGpuMoeEpStack *s, uint8_t *handle64);
int omega_gpu_moe_epstack_connect(OmegaGpuMoeEpStack *s, const uint8_t *handles);
int omega_gpu_moe_epstack_step_async(OmegaGpuMoeEpStack *s, uint64_t logits_all_va, uint64_t x_va, uint64_t out_bf16_va, void *stream);
int omega_gpu_moe_epstack_status(OmegaGpuMoeEpStack *s, void *stream);
uint32_t omega_gpu_moe_epstack_launches(const OmegaGpuMoeEpStack *s);
/* synchronises `stream`; 0, 100 + a routing-plan status, or the code of a bounded wait that ran out inside a kernel (13 / 14 input rows of a
 * layer, 16 result rows, 17 buffer credit, 1-10, 20-22 the kernel's own pipeline). On such a code the kernels of the step have returned by
 * themselves, the later ones did nothing, and the process LATCHES: every later compute call returns CHIP_FAIL and nothing is freed,
 * the reference's contract for a completion of unknown outcome (src/omega_gpu_session.h:27-29, src/omega_gpu_wait.h:20-24). */
/* TEST ONLY: the iteration limit of those waits (0 = default, about a second), and a host-made failure: expect `rows` input rows more
 * than any peer will deliver. */
void omega_gpu_moe_test_set_wait_limit(uint32_t iterations);
int omega_gpu_moe_epstack_test_expect_extra(OmegaGpuMoeEpStack *s, uint32_t rows);
int omega_gpu_moe_epstack_set_norm(OmegaGpuMoeEpStack *s, uint32_t layer, const float *norm_w);   /* as omega_gpu_moe_stack_set_norm; every rank sets the same weights */
uint64_t omega_gpu_moe_epstack_h(const OmegaGpuMoeEpStack *s);   /* device address of the f32 residual stream [tokens_local][hidden] */
/* ---- router front half: RMSNorm of a residual row with the layer's norm weight, router logits against the bf16 gate matrix,
 * softmax top-k (lowest index on ties, ids in descending-logit order), weights renormalised over the selected when norm_topk.
 * Replaces omega_gpu_router / omega_gpu_router_record_rows (src/omega_gpu_router_api.h:74-110; kernel contract
 * src/omega_blackwell_codegen_router.h:15-33) for any number of rows in one launch. The reference's group tables (directory
 * entries of the selected experts) are not produced: this library's routing plan reads the ids themselves.
 * gate_bf16: [experts][hidden] bf16 bits (the checkpoint's mlp.gate.weight), norm_w: f32 [hidden]; both are copied. */
int omega_gpu_moe_router_create(uint32_t experts, uint32_t hidden, const uint16_t *gate_bf16, const float *norm_w, OmegaGpuMoeRouter **out);
void omega_gpu_moe_router_free(OmegaGpuMoeRouter *r);
/* The shared expert's gate vector, bf16 [hidden] (copied). Once set, every row gets one more slot after its topk routed ones: id = experts
 * (the shared expert's index in a tensor of experts + 1), weight = sigmoid(gate . xn) (src/omega_gpu_q36_graph.h:20); ids_va / wts_va of the
 * calls below are then [rows][topk + 1]. */
int omega_gpu_moe_router_set_shared_gate(OmegaGpuMoeRouter *r, const uint16_t *gate_bf16);
/* device buffers, stream-ordered. x_va: f32 rows, x_stride_bytes apart (0 = dense; a multiple of 16). Outputs: xn_va f32
 * [rows][hidden] = RMSNorm(x) * out_scale (0 = skip), xn_bf16_va bf16 [rows][hidden] = RMSNorm(x) rounded to nearest even (0 = skip;
 * the input rows of omega_gpu_moe_layer_async), logits_va f32 [rows][experts] (0 = skip), ids_va u32 [rows][topk], wts_va f32 [rows][topk]. */
int omega_gpu_moe_router_rows_async(OmegaGpuMoeRouter *r, uint32_t rows, uint64_t x_va, uint32_t x_stride_bytes, float eps, int norm_topk,
                                    float out_scale, uint32_t topk, uint64_t xn_va, uint64_t xn_bf16_va, uint64_t logits_va, uint64_t ids_va,
                                    uint64_t wts_va, void *stream);
/* host buffers; xn and logits optional */
int omega_gpu_moe_router_f32(OmegaGpuMoeRouter *r, uint32_t rows, const float *x, float eps, int norm_topk, float out_scale, uint32_t topk,
                             float *xn, float *logits, uint32_t *ids, float *wts);

/* Measurement aid, no reference counterpart: the FP8 tensor throughput this GPU sustains when nothing has to be loaded (every SM
 * issues iters x 4 tcgen05 MMAs of M 128, N 256, K 32 on operands resident in shared memory). *tflops = best of `repeats` timed
 * launches (CUDA events), *ms_out (optional) that launch's duration. The denominator for "fraction of FP8 tensor peak". */
int omega_gpu_fp8_tensor_peak(uint32_t iters, uint32_t repeats, float *tflops, float *ms_out);
/* Measurement aid, no reference counterpart: HBM bandwidth of this GPU as this process sees it. Two buffers of `bytes` each (256 MiB to
 * 4 GiB, larger than L2) are allocated for the call: *copy_gbs = (bytes read + bytes written) / time of a plain copy kernel, *read_gbs =
 * bytes / time of a read-only stream; best of `repeats` timed launches each (CUDA events). */
int omega_gpu_hbm_peak(uint64_t bytes, uint32_t repeats, float *copy_gbs, float *read_gbs);

#ifdef __cplusplus
}
#endif
#endif
