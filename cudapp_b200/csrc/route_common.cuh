// route_common.cuh: the router's selection rule as one warp-wide device function, shared by the top-k kernel (given logits) and the
// router front half (logits computed in the same launch).
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace b200 {

// l: `experts` f32 logits in shared memory, visible to the whole warp; selected entries are overwritten. topk <= 32.
// k rounds of "largest remaining logit, lowest expert index on ties" (src/omega_blackwell_codegen_router.c:298-401; oracle
// tests/gpu_router_test.c:62-79); ids in selection order; weights = exp(l_i - l_0) / sum over the selected (norm) or
// exp(l_i - max) / sum over all experts.
__device__ __forceinline__ void warp_topk(float *l, uint32_t experts, uint32_t topk, int norm, uint32_t *__restrict__ ids, float *__restrict__ wts) {
    const uint32_t lane = threadIdx.x & 31u;
    float lmax = -INFINITY;
    for (uint32_t e = lane; e < experts; e += 32) lmax = fmaxf(lmax, l[e]);
    float denom_all = 0.0f;
    if (!norm) {
        for (int o = 16; o; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
        for (uint32_t e = lane; e < experts; e += 32) denom_all += expf(l[e] - lmax);
        for (int o = 16; o; o >>= 1) denom_all += __shfl_xor_sync(0xffffffffu, denom_all, o);
    }
    float my_logit = 0.0f, l0 = 0.0f, sum = 0.0f;   // lane r keeps the r-th selected logit
    uint32_t my_id = 0;
    for (uint32_t r = 0; r < topk; r++) {
        float best = -INFINITY; uint32_t bi = 0xffffffffu;
        for (uint32_t e = lane; e < experts; e += 32) { const float v = l[e]; if (bi == 0xffffffffu || v > best) { best = v; bi = e; } }
        // ascending scan with strict > keeps the lowest index inside a lane; across lanes prefer larger value, then lower index
        for (int o = 16; o; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o); const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == r) { my_logit = best; my_id = bi; }
        if (r == 0) l0 = best;
        if (lane == 0) l[bi] = -INFINITY;   // taken
        __syncwarp();
    }
    const float e_i = lane < topk ? expf(my_logit - (norm ? l0 : lmax)) : 0.0f;
    sum = e_i;
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane < topk) {
        ids[lane] = my_id;
        wts[lane] = __fdiv_rn(e_i, norm ? sum : denom_all);
    }
}

}  // namespace b200
