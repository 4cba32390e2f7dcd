/*
 * b200moe_fp8gemm.h: grouped GEMM over FP8 e4m3 block-scaled expert weights (rows sorted by expert).
 *
 * Drop-in for the reference's grouped GEMM interface (src/omega_gpu_fp8gemm_api.h:68-110). The weights are
 * the OmegaGpuFp8Tensor of b200moe_fp8.h. Host pointers throughout.
 *
 *   row i (0 <= i < M) applies expert expert_ids[i] to activation row x[token_rows[i]]; expert_ids must be
 *   non-decreasing; y is M x n f32 in row-table order, each row bit-identical to one omega_gpu_fp8_gemv call.
 *
 * Unlike the reference kernel (M <= 1024, 256 segments) any M and segment count runs on the tuned path.
 */
#ifndef B200MOE_FP8GEMM_H
#define B200MOE_FP8GEMM_H
#include "b200moe_fp8.h"
#ifdef __cplusplus
extern "C" {
#endif

enum { /* src/omega_gpu_fp8gemm_api.h:45-51 */
    OMEGA_GPU_FP8GEMM_OK = 0,
    OMEGA_GPU_FP8GEMM_BAD_ARGS = -1,
    OMEGA_GPU_FP8GEMM_TOO_LARGE = -2,
    OMEGA_GPU_FP8GEMM_CODEGEN_FAIL = -3,
    OMEGA_GPU_FP8GEMM_CHIP_FAIL = -4
};
#define OMEGA_GEMM_SEG_BYTES 32u /* {w_va u64, s_va u64, row0 u32, cnt u32, 0 u64}: src/omega_gpu_fp8gemm_api.c:290 */

/* 88 bytes, field for field src/omega_gpu_fp8gemm_api.h:55-66 */
typedef struct {
    uint32_t rows, segments, n, k, mt, warps_per_cta, lane_bytes, grid_x, grid_y, passes_max;
    uint64_t weight_bytes;   /* e4m3 bytes of the distinct experts */
    uint64_t streamed_bytes; /* bytes the launch reads from the weights (each segment once per pass of mt rows) */
    uint64_t elapsed_ns;
    uint64_t call_ns;
    uint32_t completion_marker;
    bool kernel_cache_hit;
    uint32_t general;
} OmegaGpuFp8GemmInfo;

int omega_gpu_fp8gemm_f32(const OmegaGpuFp8Tensor *t, uint32_t M, const uint32_t *expert_ids, const uint32_t *token_rows,
                          const float *x, uint32_t x_rows, float *y, OmegaGpuFp8GemmInfo *info);    /* :68 */
int omega_gpu_fp8gemm_bf16(const OmegaGpuFp8Tensor *t, uint32_t M, const uint32_t *expert_ids, const uint32_t *token_rows,
                           const uint16_t *x, uint32_t x_rows, float *y, OmegaGpuFp8GemmInfo *info); /* :70 */
int omega_gpu_fp8gemm_prepare(uint32_t k);         /* :72 */
const char *omega_gpu_fp8gemm_rc_name(int rc);     /* :73 */
const char *omega_gpu_fp8gemm_last_error(void);    /* :74 */
void omega_gpu_fp8gemm_cache_clear(void);          /* :75 */
/* TEST ONLY (:87): 1 scale dropped, 2 scale pointer never advances, 3 the neighbouring row's x. */
void omega_gpu_fp8gemm_test_set_mutant(int mutant);

/* Stream-ordered device form of the reference's record entry (src/omega_gpu_fp8gemm_api.h:103): seg_va: `segs`
 * 32-byte segment records (a cnt of 0 is skipped); x_va: activation rows (f32, or bf16 when x_bf16), natural
 * column order, no fold; xmap_va / ymap_va: both 0, or u32 tables: activation row XMAP[p] feeds sorted row p and its
 * output lands in y row YMAP[p]. stream is a cudaStream_t as void *. */
int omega_gpu_fp8gemm_async(const OmegaGpuFp8Tensor *t, uint32_t rows, uint32_t segs, uint64_t seg_va, uint64_t x_va,
                            int x_bf16, uint64_t y_va, uint64_t xmap_va, uint64_t ymap_va, void *stream);
/* No counterpart in the reference. The row-table GEMM for callers that must not allocate device memory: an
 * embedder that has given all device memory to its own arena, or a host in a section where cudaMalloc (which can
 * synchronise the whole device) is not allowed. Inputs and the output are the caller's DEVICE buffers: expert_ids
 * (u32 [M], non-decreasing), token_rows (u32 [M], each below x_rows), x (f32 or bf16 [x_rows][k]), y (f32 [M][n]).
 * The segment table, which the other entries keep in a staging buffer they allocate, lives in one fixed device array
 * inside the library (about 33 KB per GPU that loads the library, held until the process exits). Limits: at most
 * OMEGA_GPU_FP8GEMM_NOALLOC_MAX_SEGMENTS experts in the tensor and OMEGA_GPU_FP8GEMM_NOALLOC_MAX_ROWS rows; more is
 * refused with TOO_LARGE and a message. The call runs on `stream` (a cudaStream_t as void *) and EVERY call blocks
 * once on that stream for its small table-building kernel, so an unsorted or out-of-range id table, or a token row at
 * or past x_rows, is reported (BAD_ARGS) before the GEMM is queued; y is complete when work queued on `stream` after
 * the call runs. Because of that wait no call may be made while `stream` is being captured: it is refused with
 * BAD_ARGS, nothing is queued and the capture stays valid. The first call on a device also looks up the array's device
 * address. All calls share the one array: calls that overlap on the GPU (two
 * streams, two threads) race on it; calls ordered on one stream do not. Results are bit-identical to
 * omega_gpu_fp8gemm_f32 / _bf16 on the same table. */
#define OMEGA_GPU_FP8GEMM_NOALLOC_MAX_SEGMENTS 1024u
#define OMEGA_GPU_FP8GEMM_NOALLOC_MAX_ROWS 1048576u
int omega_gpu_fp8gemm_noalloc(const OmegaGpuFp8Tensor *t, uint32_t M, uint64_t expert_ids_va, uint64_t token_rows_va, uint64_t x_va,
                              int x_bf16, uint32_t x_rows, uint64_t y_va, void *stream);
#ifdef __cplusplus
}
#endif
#endif
