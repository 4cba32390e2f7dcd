/*
 * b200moe_fp8.h: FP8 e4m3, 128 x 128 block-scaled weight tensors and the decode GEMV on B200 (sm_100a).
 *
 * Drop-in surface: every function in the first section has the name, argument list, return codes and error
 * behaviour of the reference operator library's FP8 GEMV interface (src/omega_gpu_fp8_api.h:101-241 of the
 * reference project; the line each entry replaces is cited beside it). A C caller written against that header
 * links against libb200moe.so unchanged. All pointers are HOST pointers unless a name ends in _va (a device
 * address held in a uint64_t). No CPU fallback exists: with no usable CUDA device every compute entry returns
 * OMEGA_GPU_FP8_CHIP_FAIL and says why in omega_gpu_fp8_last_error().
 *
 * Semantics kept from the reference: weights [expert][n][k] e4m3 row-major, unchanged on the device; one f32
 * scale per 128 x 128 block taken from bf16 `weight_scale_inv`; y[r] = sum_c W[r][c] * x[c] * scale[r/128][c/128]
 * with f32 accumulation in the reference kernel's own summation order (lane-owned 8/16-byte chunks, one scale
 * FMA per K step, shuffle-down tree), so results are bit-identical to that kernel's host emulation
 * (tests/gpu_fp8gemm_test.c:48-69). Every output word is poisoned (-999.0f) before the launch and a result
 * that still holds poison is refused. A CUDA error of unknown outcome latches the process: later calls fail.
 */
#ifndef B200MOE_FP8_H
#define B200MOE_FP8_H
#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* return codes: src/omega_gpu_fp8_api.h:68-75 */
enum {
    OMEGA_GPU_FP8_OK = 0,
    OMEGA_GPU_FP8_BAD_ARGS = -1,
    OMEGA_GPU_FP8_TOO_LARGE = -2,
    OMEGA_GPU_FP8_CODEGEN_FAIL = -3, /* kept for ABI compatibility: kernels here are compiled ahead of time */
    OMEGA_GPU_FP8_CHIP_FAIL = -4,
    OMEGA_GPU_FP8_NAN_WEIGHT = -5
};
#define OMEGA_GPU_FP8_MAX_GROUPS 64u /* src/omega_gpu_fp8_api.h:77 */
#define OMEGA_FP8_BLOCK 128u         /* src/omega_blackwell_codegen_moe.h:62 */
#define OMEGA_FP8_MAX_K 32768u       /* src/omega_blackwell_codegen_moe.h:63 */

/* 160 bytes, 8-byte aligned, field for field the reference's record (src/omega_gpu_fp8_api.h:83-97;
 * docs/runtime/omega_runtime_api.manifest:642-680). target_chip names the CUDA device; sm_architecture is 100. */
typedef struct {
    uint32_t experts, n, k, groups;
    uint32_t lane_bytes, rows_per_warp, warps_per_cta;
    uint32_t depth;
    uint32_t grid_x, grid_y, steps;
    uint64_t weight_bytes;
    uint64_t scale_bytes;
    uint64_t elapsed_ns; /* device time of the kernel (CUDA events) */
    uint64_t call_ns;    /* whole call on the host clock */
    uint32_t completion_marker;
    bool kernel_cache_hit;
    char target_chip[64];
    uint32_t sm_architecture;
    uint32_t general;
} OmegaGpuFp8Info;

typedef struct OmegaGpuFp8Tensor OmegaGpuFp8Tensor;

/* src/omega_gpu_fp8_api.h:101-102. n, k multiples of 128, k <= 32768, experts >= 1. NaN codes (0x7f, 0xff) in w
 * give NAN_WEIGHT, a NaN/inf scale BAD_ARGS; *out is NULL on every failure. */
int omega_gpu_fp8_tensor_upload(uint32_t experts, uint32_t n, uint32_t k, const uint8_t *w,
                                const uint16_t *scale_inv_bf16, OmegaGpuFp8Tensor **out);
/* src/omega_gpu_fp8_api.h:106. bf16 [n][k] -> e4m3 [n][k] + bf16 scales [n/128][k/128]; scale = amax/448 rounded up
 * to bf16 (1.0 for a zero block), round to nearest even, saturating. Runs on the GPU; bit-identical to the
 * reference's host quantiser. BAD_ARGS on an inf/NaN weight. */
int omega_gpu_fp8_quantize_bf16(uint32_t n, uint32_t k, const uint16_t *w_bf16, uint8_t *w8, uint16_t *scale_inv_bf16);
uint8_t omega_gpu_fp8_e4m3_rne(float v);                                  /* src/omega_gpu_fp8_api.h:107 */
void omega_gpu_fp8_tensor_free(OmegaGpuFp8Tensor *t);                     /* src/omega_gpu_fp8_api.h:108 */
void omega_gpu_fp8_tensor_shape(const OmegaGpuFp8Tensor *t, uint32_t *experts, uint32_t *n, uint32_t *k); /* :109 */

/* src/omega_gpu_fp8_api.h:111-114. x: k values (f32, or bf16 bits); y: n f32 per group. grouped: x_rows is 1 (one
 * row shared by every group) or `groups` (one row each); ids may repeat; groups <= OMEGA_GPU_FP8_MAX_GROUPS on the
 * tuned path, any count otherwise (info->general = 1). */
int omega_gpu_fp8_gemv_f32(const OmegaGpuFp8Tensor *t, uint32_t expert, const float *x, float *y, OmegaGpuFp8Info *info);
int omega_gpu_fp8_gemv_bf16(const OmegaGpuFp8Tensor *t, uint32_t expert, const uint16_t *x, float *y, OmegaGpuFp8Info *info);
int omega_gpu_fp8_gemv_grouped_f32(const OmegaGpuFp8Tensor *t, uint32_t groups, const uint32_t *expert_ids,
                                   const float *x, uint32_t x_rows, float *y, OmegaGpuFp8Info *info);
/* src/omega_gpu_fp8_api.h:118. tab_va: `groups` {w_va, s_va} pairs in device memory (omega_gpu_fp8_tensor_entry
 * values); x_va: one device row of k f32 that already carries the reference's 2^64 fold (its router writes it that
 * way); the fold is removed exactly inside the kernel. y is a host buffer. */
int omega_gpu_fp8_gemv_grouped_dev(const OmegaGpuFp8Tensor *t, uint32_t groups, uint64_t tab_va, uint64_t x_va, float *y, OmegaGpuFp8Info *info);
int omega_gpu_fp8_tensor_entry(const OmegaGpuFp8Tensor *t, uint32_t expert, uint64_t *w_va, uint64_t *s_va); /* :132 */

/* src/omega_gpu_fp8_api.h:135-141. Kernels are ahead-of-time compiled, so prepare only validates k and opens the
 * device, seal and cache_clear keep their meaning trivially. */
int omega_gpu_fp8_prepare(uint32_t k);
void omega_gpu_fp8_seal(int on);
const char *omega_gpu_fp8_rc_name(int rc);
const char *omega_gpu_fp8_last_error(void);
void omega_gpu_fp8_cache_clear(void);
/* src/omega_gpu_fp8_api.h:165: CTAs per group (0 = automatic: enough to fill the 148 SMs). */
void omega_gpu_fp8_set_cta_budget(uint32_t ctas);
/* src/omega_gpu_fp8_api.h:211: TEST ONLY, deliberately wrong kernels: 1 scale dropped, 2 scale block never
 * advances, 3 group g reads the weights of group g ^ 1. The parity tests must catch each. */
void omega_gpu_fp8_test_set_mutant(int mutant);

/* host helpers, no device (src/omega_gpu_fp8_api.h:224-238) */
float omega_fp8_e4m3_ref(uint8_t b);
int omega_fp8_e4m3_is_nan(uint8_t b);
size_t omega_fp8_pack_scan_nan(const uint8_t *w, size_t count, size_t *first);
/* double-precision reference for a caller's own checks; no compute entry point of this library calls it */
void omega_fp8_gemv_oracle(const uint8_t *w, const uint16_t *scale_bf16, uint32_t n, uint32_t k,
                           const float *x, double *y, double *yscale);

/* ---- stream-ordered device forms (no counterpart in the reference: its record path appends to a command list,
 * which has no CUDA meaning). Every pointer is a device address; nothing is staged, poisoned or read back.
 * stream is a cudaStream_t passed as void *. x_bf16 != 0: x holds bf16 bits. */
int omega_gpu_fp8_gemv_grouped_async(const OmegaGpuFp8Tensor *t, uint32_t groups, uint64_t tab_va, uint64_t x_va,
                                     uint32_t x_rows, int x_bf16, uint64_t y_va, void *stream);

#ifdef __cplusplus
}
#endif
#endif
