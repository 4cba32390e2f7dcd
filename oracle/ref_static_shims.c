/* Test infrastructure only: exposes three reference functions that the reference keeps `static` inside its own test
 * files, by compiling each test file where it lies with its main renamed (the trick of ref_router_shim.c). One shim
 * per macro so that the three test files, which share helper names, never meet in one translation unit:
 *   -DSHIM_EMU  tests/gpu_fp8gemm_test.c  -> emu_row  (:48-69), the kernels' exact f32 summation order
 *   -DSHIM_PQ   tests/gpu_qgemm_test.c    -> pq_ref   (:24-35) and its input generator rand_act (:36-40)
 *   -DSHIM_MC   tests/gpu_pfhost_test.c   -> mc_ref   (:38-49), compiled with -ffp-contract=off as that test is
 * Built by `make ref` into _ref/libref_emu.so, libref_pq.so, libref_mc.so; nothing of the reference is copied. */
#define EXPORT __attribute__((visibility("default")))
#if defined(SHIM_EMU)
#define main omega_fp8gemm_test_main_unused
#include "gpu_fp8gemm_test.c"
#undef main
/* lb = the lane's bytes per K step (16 when k % 512 == 0, else 8), as the kernel chooses it */
EXPORT float ref_emu_row(const uint8_t *w, const uint16_t *s, const float *x, uint32_t k, uint32_t lb) { return emu_row(w, s, x, k, lb); }
#elif defined(SHIM_PQ)
#define main omega_qgemm_test_main_unused
#include "gpu_qgemm_test.c"
#undef main
EXPORT void ref_pq(const float *x, uint32_t k, uint8_t *q, float *s) { pq_ref(x, k, q, s, 0); }
/* n activations from the reference test's own generator, from its own start state */
EXPORT void ref_pq_rand_act(float *out, uint32_t n) { rng = 0x243f6a8885a308d3ull; for (uint32_t i = 0; i < n; i++) out[i] = rand_act(); }
#elif defined(SHIM_MC)
#define main omega_pfhost_test_main_unused
#include "gpu_pfhost_test.c"
#undef main
EXPORT void ref_mc(const float *down, const uint32_t *inv, const float *wt, uint32_t rows, uint32_t h, uint32_t K, float *out) { mc_ref(down, inv, wt, rows, h, K, out, 0); }
#else
#error "define SHIM_EMU, SHIM_PQ or SHIM_MC"
#endif
