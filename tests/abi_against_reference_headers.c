/* Link test of the drop-in boundary: a C translation unit written against THE REFERENCE'S OWN headers (found through -I <reference>/src,
 * nothing copied), linked with this library instead of the reference's. It checks what a C caller sees: the prototypes compile against
 * this library's symbols, the two info records have the reference's sizes and field offsets (the reference's own compiled probe checks
 * the same numbers, docs/runtime/omega_runtime_api.manifest:642-680), return-code names agree, and the argument and NaN-weight
 * refusals come back before any device work. Built and run by tests/test_abi_host.py where the reference tree is present. */
#include "omega_gpu_fp8_api.h"
#include "omega_gpu_fp8gemm_api.h"
#include "cudapp_native.h"
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

_Static_assert(sizeof(OmegaGpuFp8Info) == 160, "OmegaGpuFp8Info size");
_Static_assert(offsetof(OmegaGpuFp8Info, weight_bytes) == 48 && offsetof(OmegaGpuFp8Info, elapsed_ns) == 64 && offsetof(OmegaGpuFp8Info, call_ns) == 72, "OmegaGpuFp8Info offsets");
_Static_assert(offsetof(OmegaGpuFp8Info, kernel_cache_hit) == 84 && offsetof(OmegaGpuFp8Info, target_chip) == 85 && offsetof(OmegaGpuFp8Info, sm_architecture) == 152 &&
               offsetof(OmegaGpuFp8Info, general) == 156, "OmegaGpuFp8Info offsets");
_Static_assert(sizeof(OmegaGpuFp8GemmInfo) == 88 && offsetof(OmegaGpuFp8GemmInfo, streamed_bytes) == 48 && offsetof(OmegaGpuFp8GemmInfo, elapsed_ns) == 56 &&
               offsetof(OmegaGpuFp8GemmInfo, call_ns) == 64 && offsetof(OmegaGpuFp8GemmInfo, general) == 80, "OmegaGpuFp8GemmInfo layout");

static int fails;
#define CHECK(c) do { if (!(c)) { fails++; printf("FAIL line %d: %s\n", __LINE__, #c); } } while (0)

int main(void) {
    CHECK(strcmp(omega_gpu_fp8_rc_name(OMEGA_GPU_FP8_OK), "OK") == 0 && strcmp(omega_gpu_fp8_rc_name(OMEGA_GPU_FP8_NAN_WEIGHT), "NAN_WEIGHT") == 0);
    CHECK(strcmp(omega_gpu_fp8gemm_rc_name(OMEGA_GPU_FP8GEMM_BAD_ARGS), omega_gpu_fp8_rc_name(OMEGA_GPU_FP8_BAD_ARGS)) == 0);
    CHECK(omega_fp8_e4m3_ref(0x38) == 1.0f && omega_fp8_e4m3_ref(0x7E) == 448.0f && omega_fp8_e4m3_is_nan(0x7F) && omega_fp8_e4m3_is_nan(0xFF) && !omega_fp8_e4m3_is_nan(0x7E));
    CHECK(omega_gpu_fp8_e4m3_rne(1.0f) == 0x38 && omega_gpu_fp8_e4m3_rne(1e9f) == 0x7E && omega_gpu_fp8_e4m3_rne(-1e9f) == 0xFE);
    /* upload refusals: shape, then a NaN code, all before a device is touched; *out is NULL afterwards */
    static uint8_t w[128 * 128]; uint16_t s = 0x3F80;
    OmegaGpuFp8Tensor *t = (OmegaGpuFp8Tensor *)(uintptr_t)123;
    CHECK(omega_gpu_fp8_tensor_upload(1, 128, 100, w, &s, &t) == OMEGA_GPU_FP8_BAD_ARGS && t == NULL);
    w[5 * 128 + 7] = 0xFF;
    t = (OmegaGpuFp8Tensor *)(uintptr_t)123;
    CHECK(omega_gpu_fp8_tensor_upload(1, 128, 128, w, &s, &t) == OMEGA_GPU_FP8_NAN_WEIGHT && t == NULL && strstr(omega_gpu_fp8_last_error(), "NaN") != NULL);
    /* argument refusals of the compute entries */
    float x[128] = {0}, y[128];
    uint32_t ids[2] = {0, 0}, rows[2] = {0, 0};
    OmegaGpuFp8Info info; memset(&info, 0xAA, sizeof info);
    CHECK(omega_gpu_fp8_gemv_f32(NULL, 0, x, y, &info) == OMEGA_GPU_FP8_BAD_ARGS && info.n == 0 && info.elapsed_ns == 0);      /* info zeroed at entry */
    OmegaGpuFp8GemmInfo ginfo; memset(&ginfo, 0xAA, sizeof ginfo);
    CHECK(omega_gpu_fp8gemm_f32(NULL, 2, ids, rows, x, 1, y, &ginfo) == OMEGA_GPU_FP8GEMM_BAD_ARGS && ginfo.rows == 0);
    omega_gpu_fp8_tensor_free(NULL);                                                                                             /* NULL is a no-op */
    /* a plan unit through its ABI1 signature: a bad argument (wrong configuration length) is status 32 and writes nothing */
    static uint64_t cfg[8], pid[1024], work[10368], seg[1028], maps[2320], meta[8]; uint64_t result = 77;
    CHECK(omega_moe_plan(&result, cfg, 7, pid, 1024, work, 10368, seg, 1028, maps, 2320, meta, 8) == 32 && result == 77);
    printf("abi_against_reference_headers: %s\n", fails ? "FAIL" : "PASS");
    return fails ? 1 : 0;
}
