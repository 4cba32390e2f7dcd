// internal.h: shared state and helpers of libb200moe.so (not installed; the public surface is include/*.h).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <time.h>
#include <mutex>

#include "../../include/b200moe_ext.h"
#include "../../include/b200moe_plan.h"

static_assert(sizeof(OmegaGpuFp8Info) == 160 && offsetof(OmegaGpuFp8Info, weight_bytes) == 48 &&
              offsetof(OmegaGpuFp8Info, elapsed_ns) == 64 && offsetof(OmegaGpuFp8Info, call_ns) == 72 &&
              offsetof(OmegaGpuFp8Info, kernel_cache_hit) == 84 && offsetof(OmegaGpuFp8Info, target_chip) == 85 &&
              offsetof(OmegaGpuFp8Info, sm_architecture) == 152 && offsetof(OmegaGpuFp8Info, general) == 156,
              "OmegaGpuFp8Info must keep the reference's binary layout");
static_assert(sizeof(OmegaGpuFp8GemmInfo) == 88 && offsetof(OmegaGpuFp8GemmInfo, streamed_bytes) == 48 &&
              offsetof(OmegaGpuFp8GemmInfo, elapsed_ns) == 56 && offsetof(OmegaGpuFp8GemmInfo, call_ns) == 64 &&
              offsetof(OmegaGpuFp8GemmInfo, general) == 80,
              "OmegaGpuFp8GemmInfo must keep the reference's binary layout");

struct OmegaGpuFp8Tensor {
    uint32_t experts, n, k;
    uint8_t *w;   // device, [experts][n][k] e4m3, checkpoint order
    float *s;     // device, [experts][n/128][k/128] f32
    int device;
};

struct Seg32 { uint64_t w_va, s_va; uint32_t row0, cnt; uint64_t pad; };
static_assert(sizeof(Seg32) == OMEGA_GEMM_SEG_BYTES, "segment record layout");

// 4-bit weight tensor (w4_gemm.cu): int4 + fp16 scales, MXFP4 or NVFP4; one matrix, or the matrices of several experts one after the other
struct OmegaGpuW4Tensor {
    uint32_t n, k; uint8_t *w; uint16_t *s;   // s: fp16 scales (int4 format) or, viewed as bytes, E8M0 scales (MXFP4 format)
    uint32_t fmt;                              // 0: signed int4 + fp16 scale per 32; 1: MXFP4 = E2M1 + E8M0 scale per 32
    float *part; uint32_t *counters;   // scratch of the tensor-core kernel: K-quarter partial sums [4][16][n] f32 and one arrival counter per 128 output rows
    float *gpart; uint32_t *gcounters; uint32_t gtiles, gn;   // the same for the grouped form: per row tile [4][16][gn]; set by omega_gpu_w4_reserve_grouped
};

namespace b200 {

#define POISON_F32 (-999.0f)

struct State {
    std::recursive_mutex mu;        // one process-wide lock, as the reference session has
    char err[256] = {0};
    bool latched = false;           // a CUDA failure of unknown outcome: every later call is refused
    bool opened = false;
    int device = 0;
    int sm_count = 0;
    char chip[64] = {0};
    cudaStream_t stream = nullptr;  // the library's own stream for host-staged calls
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int gemv_mutant = 0, gemm_mutant = 0;
    uint32_t cta_budget = 0;
    uint32_t wait_limit = 1u << 22;   // iterations of a bounded cross-GPU wait before it gives up (each iteration sleeps about 100 ns); tests shorten it
    int sealed = 0;
    // grow-only staging buffers for host-staged calls
    void *stage[8] = {nullptr}; size_t stage_bytes[8] = {0};
};
State &st();

void set_error(const char *fmt, ...);
// true when the device is open (opens it on first use); false + last_error otherwise
bool dev_open();
// records a failing CUDA call; sticky errors latch the process
bool cuda_ok(cudaError_t e, const char *what);
// staging slot `i` with at least `bytes` (device memory); nullptr on failure
void *stage(int i, size_t bytes);
uint64_t now_ns();

struct Lock { Lock() { st().mu.lock(); } ~Lock() { st().mu.unlock(); } };

// ---- launchers implemented across the .cu files (all stream-ordered, device pointers)
// y poison / generic fill
void launch_fill_f32(float *p, size_t n, float v, cudaStream_t s);

struct GemvArgs {
    const Seg32 *seg;        // grouped GEMM form: segment records (nullptr for the GEMV forms)
    const uint64_t *tab;     // GEMV forms: {w_va, s_va} per group
    const void *x; int x_bf16; uint32_t x_rows;  // activation rows
    size_t x_stride_bytes;                       // 0 = rows are dense (k elements apart)
    const uint32_t *xmap, *ymap;                 // optional row maps (grouped GEMM form)
    float *y;
    uint32_t n, k, groups_or_segs, rows;
    float out_mul;           // exact power of two applied to the result (removes a caller-side fold)
    int mutant;
};
cudaError_t launch_gemv_grouped(const GemvArgs &a, uint32_t cta_budget, uint32_t *grid_x, uint32_t *warps, cudaStream_t s);
cudaError_t launch_gemm_rows(const GemvArgs &a, uint32_t *grid_x, uint32_t *mt, cudaStream_t s);

// slots: entries per token in ids / wts (0 = topk); topk + 1 appends the shared expert (id = experts, weight 1)
cudaError_t launch_topk(uint32_t tokens, uint32_t experts, uint32_t topk, int norm, const uint16_t *logits, uint32_t *ids, float *wts, cudaStream_t s, uint32_t slots = 0);
// scratch (optional, zero-filled once, plan_scratch_words(picks, experts) u32): lets a plan of 4096 picks or more run as three launches over many SMs
cudaError_t launch_plan(uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, uint32_t tile_rows, const uint32_t *ids,
                        const OmegaGpuMoePlanOut &o, cudaStream_t s, uint32_t *scratch = nullptr, size_t scratch_words = 0);
size_t plan_scratch_words(uint32_t picks, uint32_t experts);
uint32_t plan_launch_count(uint32_t picks, uint32_t experts, const uint32_t *scratch, size_t scratch_words, const OmegaGpuMoePlanOut &o);
// routing plans of several layers in one launch (one CTA per layer); element strides between layers
struct PlanBatch { uint32_t *counts, *starts, *xmap, *ymap, *pos, *header; uint4 *tiles; size_t map_stride, tile_stride; };
cudaError_t launch_plan_batch(uint32_t layers, uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, uint32_t tile_rows, const uint32_t *ids,
                              const PlanBatch &b, cudaStream_t s);
cudaError_t launch_swiglu(uint32_t rows, uint32_t inter, const float *gu, float *act, cudaStream_t s, uint16_t *act_bf16 = nullptr);   // act_bf16: the same values rounded to bf16 (either output may be null)
cudaError_t launch_combine(uint32_t tokens, uint32_t slots, uint32_t hidden, const float *w, const float *d, float *out_f32, uint16_t *out_bf16, cudaStream_t s);
// quantise rows of x (f32 or bf16; gathered through xmap when given) into e4m3 pieces: q [rows][pieces][k], s [rows][k/128]
cudaError_t launch_act_quant(uint32_t rows, uint32_t k, uint32_t pieces, const void *x, int x_bf16, const uint32_t *xmap,
                             const uint32_t *rows_dev, uint8_t *q, float *sc, cudaStream_t s, size_t x_stride_bytes = 0, uint32_t q_rows = 0);
// sorted row r <- codes (all pieces, piece-major with src_rows / dst_rows rows per piece) and scales of source row xmap[r]
cudaError_t launch_gather_rows(uint32_t rows, uint32_t k, uint32_t pieces, uint32_t src_rows, uint32_t dst_rows, const uint32_t *xmap, const uint32_t *rows_dev,
                               const uint8_t *q_src, const float *s_src, uint8_t *q_dst, float *s_dst, cudaStream_t s);
// tcgen05 grouped GEMM (fp8_mma_sm100.cu)
struct MmaLaunch {
    const float *wscale, *ascale;      // weight scales [E][n/128][k/128]; activation scales [rows][k/128]
    const void *tiles;                 // uint4 {expert, row0, cnt, segment} per row tile
    const uint32_t *header, *ymap;     // header[2] = tile count; ymap: destination rows (mode 1)
    float *out; uint32_t n, k, mode, out_stride;   // mode 1: out[ymap[row]][n]; mode 0: gate|up + SiLU gate, f32 copy to out[row][n/2] when out != null
    uint8_t *q_out; float *s_out; uint32_t q_rows, q_pieces;   // mode 0 result as e4m3 pieces [piece][q_rows][n/2] + scales [row][n/256]; q_rows also = row capacity of the input pieces
    uint32_t *err;                     // device word: non-zero = a bounded wait inside the kernel ran out
    // expert parallelism (null / 0 otherwise): wait for `*gate >= header[0]` delivered input rows; mode 1 results go to out_peers[row / rows_per_rank]
    const unsigned long long *gate; const uint64_t *out_peers, *ret_counters; uint32_t rows_per_rank, ret_index; const unsigned long long *gate_base; unsigned long long *bump;
    uint32_t wait_limit;               // iterations of the bounded wait on `gate` (0 = the default)
};
bool make_tmap_u8(void *out_map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows);
uint32_t mma_tile_rows(uint32_t pieces);
bool mma_shape_ok(uint32_t n, uint32_t k, uint32_t mode);
cudaError_t launch_mma_grouped(const void *tm_w, const void *tm_q, uint32_t pieces, const MmaLaunch &m, cudaStream_t s, bool pdl = false);
// the same GEMM on 128-row tiles for prefill-sized segments (fp8_mma_wide_sm100.cu); single-piece activations only, no expert-parallel fields
uint32_t mma_wide_tile_rows();
bool mma_wide_shape_ok(uint32_t n, uint32_t k, uint32_t mode);
cudaError_t launch_mma_wide(const void *tm_w, const void *tm_q, const MmaLaunch &m, cudaStream_t s);
// whole expert FFN of a layer in one launch (fp8_ffn_sm100.cu); piece counts (2,3), (1,1) or (2,2)
struct FfnLaunch {
    const float *gu_scale, *dn_scale, *x_scale; uint8_t *qa; float *sa; const void *tiles; const uint32_t *header, *ymap; float *out;
    uint32_t hidden, inter, q_rows; uint32_t *sched, *err;   // sched: [0] next down unit, [1 + tile] finished gate|up units; zeroed before the launch
    const unsigned long long *gate, *gate_base; const uint64_t *out_peers, *ret_counters; uint32_t rows_per_rank, ret_index;   // expert parallelism, as in MmaLaunch
    uint32_t wait_limit;
};
// grouped 4-bit GEMM over a plan's 16-row tiles (the tensor must have been given its per-tile scratch by omega_gpu_w4_reserve_grouped)
cudaError_t launch_w4_grouped(const OmegaGpuW4Tensor *t, const void *tiles, const uint32_t *header, const uint32_t *xmap, const uint32_t *ymap,
                              const uint16_t *x_bf16, uint16_t *y_bf16, float *y_f32, cudaStream_t s);
bool ffn_shape_ok(uint32_t hidden, uint32_t inter);
cudaError_t launch_ffn(const void *tm_gu, const void *tm_qx, const void *tm_dn, const void *tm_qa, uint32_t px, uint32_t pa, const FfnLaunch &m, cudaStream_t s, bool pdl);
bool layer_forward(OmegaGpuMoeLayer *L, uint32_t tokens, const uint16_t *logits, const uint16_t *x, float *out32, uint16_t *out16, cudaStream_t s,
                   const uint32_t *ids_in = nullptr, const float *wts_in = nullptr);
// expert side only (expert-parallel receive path): `rows` candidate rows, ids[row] = local expert or 0xFFFFFFFF,
// x row r at x + r * x_stride_bytes (bf16); writes dn[row][hidden] f32 for the present rows
bool layer_forward_routed(OmegaGpuMoeLayer *L, uint32_t rows, const uint32_t *ids, const void *x, size_t x_stride_bytes, float *dn, cudaStream_t s);
// what the stack needs from a layer to drive the tensor-core kernels itself
struct LayerView {
    uint32_t engine, topk, experts, hidden, inter, x_pieces, act_pieces, tile_rows, max_tokens, row_cap, norm_topk;   // topk = slots per token, experts = what the tensors hold
    uint32_t shared;   // 1: the last expert is the shared one, slot topk - 1 of every token
    const float *gu_scale, *dn_scale; const void *tm_gu, *tm_dn, *tm_qa;
    uint8_t *qa; float *sa, *dn;
};
void layer_view(OmegaGpuMoeLayer *L, LayerView *v);
bool layer_share_workspace(OmegaGpuMoeLayer *dst, OmegaGpuMoeLayer *src);
void layer_dims(const OmegaGpuMoeLayer *L, uint32_t *experts, uint32_t *hidden, uint32_t *max_tokens);
cudaError_t launch_router_rows(const OmegaGpuMoeRouter *r, uint32_t rows, const float *x, float eps, int norm_topk, uint32_t topk, uint16_t *xn16, uint32_t *ids, float *wts, cudaStream_t s, uint32_t slots = 0);
void router_dims(const OmegaGpuMoeRouter *r, uint32_t *experts, uint32_t *hidden);
float *layer_out32(OmegaGpuMoeLayer *L);
uint16_t *layer_stage_x(OmegaGpuMoeLayer *L);
}  // namespace b200
