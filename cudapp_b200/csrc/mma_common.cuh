// mma_common.cuh: PTX wrappers and small device helpers shared by the tcgen05 kernels of this library
// (TMA loads, mbarriers with bounded waits, tcgen05 MMA / commit / TMEM load, programmatic dependent launch, e4m3 pieces).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int MMA_TOK = 32;                     // routed rows per tile; accumulator columns = 32 per activation piece
constexpr uint32_t A_TILE = 128 * 128, B_PIECE = MMA_TOK * 128;
constexpr int KB_MAX = 32;                      // k <= 4096 on this engine
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr uint32_t Q_STAGE_BYTES = 2 * 4 * MMA_TOK * 128;   // per epilogue group: up to 4 pieces x 32 rows x 128 bytes of output codes

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false (and *err = code) when the limit runs out or another role already gave up
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, uint32_t *err, uint32_t code) {
    for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1; atomicCAS(err, 0u, code);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// the same load with an L2 eviction policy (weights are read once per launch: evict-first keeps them from displacing the activation tiles,
// scales and result rows that are read again); the policy word comes from createpolicy
__device__ __forceinline__ uint64_t l2_policy_evict_first() { uint64_t p; asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p)); return p; }
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy) : "memory");
}
// programmatic dependent launch: wait = the grids this one depends on have completed and their writes are visible;
// launch_dependents = the next grid in the stream may start occupying free SMs (it blocks in its own wait)
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// bounded wait until a counter that peers advance with system-scope atomics reaches `want`
__device__ __forceinline__ bool gate_wait(const unsigned long long *gate, unsigned long long want, uint32_t *err, uint32_t code, uint32_t limit = 1u << 22) {
    for (uint32_t i = 0; i < limit; i++) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(gate) : "memory");
        if (v >= want) { asm volatile("fence.proxy.async;" ::: "memory"); return true; }
        if ((i & 63u) == 63u && *reinterpret_cast<volatile uint32_t *>(err)) return false;   // somebody already gave up: do not wait out the limit again
        __nanosleep(100);
    }
    atomicCAS(err, 0u, code);
    return false;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) { asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p; }"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// K-major operand tile, rows of 128 bytes, SWIZZLE_128B: 8-row groups 1024 bytes apart (stride offset), version 1
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3ffffu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

#define TMEM_LD32(taddr, r)                                                                                                              \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];" \
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),       \
                   "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),           \
                   "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]) \
                 : "r"(taddr))

// acc += Sw * Sa * partial for the 32 routed rows of one half (one 128-feature block) of a K block: the reference's promotion
// (src/omega_blackwell_codegen_qg.h:24-26); sc = 32 floats in shared memory, 16-byte aligned
__device__ __forceinline__ void promote_half(const uint32_t (&v)[MMA_TOK], const float *sc, float (&acc)[MMA_TOK]) {
#pragma unroll
    for (int i = 0; i < MMA_TOK; i += 4) {
        const float4 c = *reinterpret_cast<const float4 *>(sc + i);
        acc[i] = fmaf(__uint_as_float(v[i]), c.x, acc[i]); acc[i + 1] = fmaf(__uint_as_float(v[i + 1]), c.y, acc[i + 1]);
        acc[i + 2] = fmaf(__uint_as_float(v[i + 2]), c.z, acc[i + 2]); acc[i + 3] = fmaf(__uint_as_float(v[i + 3]), c.w, acc[i + 3]);
    }
}
// pieces of one half folded last to first (x 1/16 each): r[P-1] / 16 + r[P-2], ... ; the result replaces r[0]
template <int P>
__device__ __forceinline__ void fold_pieces(uint32_t (&r)[P][MMA_TOK]) {
#pragma unroll
    for (int i = 0; i < MMA_TOK; i++) {
        float v = __uint_as_float(r[P - 1][i]);
#pragma unroll
        for (int p = P - 2; p >= 0; p--) v = fmaf(v, 0.0625f, __uint_as_float(r[p][i]));
        r[0][i] = __float_as_uint(v);
    }
}
// One K block's partial sums of a promotion thread (its TMEM lane, 2 halves x P pieces x 32 columns at taddr) into the two accumulators.
// The TMEM loads are what costs time (a few hundred cycles per dependent round trip), so as much as the registers hold is requested at once:
// both halves in one round trip for P <= 2; one half per round trip for P = 3, the second half in flight while the first is promoted; two pieces
// per round trip for P = 4. The partial buffer goes back to the MMA issuer (accempty) as soon as its last load has landed.
template <int P>
__device__ __forceinline__ void promote_kblock(uint32_t taddr, uint32_t accempty, const float *sc0, const float *sc1, float (&acc0)[MMA_TOK], float (&acc1)[MMA_TOK]) {
    if constexpr (P <= 2) {
        uint32_t h0[P][MMA_TOK], h1[P][MMA_TOK];
#pragma unroll
        for (int p = P - 1; p >= 0; p--) { TMEM_LD32(taddr + p * MMA_TOK, h0[p]); TMEM_LD32(taddr + P * MMA_TOK + p * MMA_TOK, h1[p]); }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        tc_fence_before(); mbar_arrive(accempty);
        fold_pieces<P>(h0); fold_pieces<P>(h1);
        promote_half(h0[0], sc0, acc0);
        promote_half(h1[0], sc1, acc1);
    } else if constexpr (P == 3) {
        uint32_t r[P][MMA_TOK], da[MMA_TOK];
#pragma unroll
        for (int p = P - 1; p >= 0; p--) TMEM_LD32(taddr + p * MMA_TOK, r[p]);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        fold_pieces<P>(r);
#pragma unroll
        for (int i = 0; i < MMA_TOK; i++) da[i] = r[0][i];
#pragma unroll
        for (int p = P - 1; p >= 0; p--) TMEM_LD32(taddr + P * MMA_TOK + p * MMA_TOK, r[p]);
        promote_half(da, sc0, acc0);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        tc_fence_before(); mbar_arrive(accempty);
        fold_pieces<P>(r);
        promote_half(r[0], sc1, acc1);
    } else {
        static_assert(P == 4, "at most four pieces");
#pragma unroll
        for (int half = 0; half < 2; half++) {
            uint32_t hi[2][MMA_TOK], lo[2][MMA_TOK];
            TMEM_LD32(taddr + half * P * MMA_TOK + 3 * MMA_TOK, hi[1]); TMEM_LD32(taddr + half * P * MMA_TOK + 2 * MMA_TOK, hi[0]);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            TMEM_LD32(taddr + half * P * MMA_TOK + MMA_TOK, lo[1]); TMEM_LD32(taddr + half * P * MMA_TOK, lo[0]);
            fold_pieces<2>(hi);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (half == 1) { tc_fence_before(); mbar_arrive(accempty); }
#pragma unroll
            for (int i = 0; i < MMA_TOK; i++)
                lo[0][i] = __float_as_uint(fmaf(fmaf(__uint_as_float(hi[0][i]), 0.0625f, __uint_as_float(lo[1][i])), 0.0625f, __uint_as_float(lo[0][i])));
            if (half) promote_half(lo[0], sc1, acc1); else promote_half(lo[0], sc0, acc0);
        }
    }
}

#define TMEM_LD16(taddr, r, o)                                                                                                           \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"                   \
                 : "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7]),      \
                   "=r"(r[o + 8]), "=r"(r[o + 9]), "=r"(r[o + 10]), "=r"(r[o + 11]), "=r"(r[o + 12]), "=r"(r[o + 13]), "=r"(r[o + 14]), "=r"(r[o + 15]) \
                 : "r"(taddr))

// SiLU gate with the fast exponential and division (the reference kernel itself uses EX2 / RCP approximations here,
// src/omega_blackwell_codegen_dec.c:291-324)
__device__ __forceinline__ float silu_mul_dev(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// activation-piece helpers (same arithmetic as act_quant_kernel in moe_glue.cu)
__device__ __forceinline__ float pq_scale_mma(float amax) {
    amax = fmaxf(amax, 7.888609052210118e-31f /* 2^-100 */);
    const uint32_t mb = __float_as_uint(amax), E = mb >> 23, M = mb & 0x7fffffu, c = (M + 0x1fffffu) >> 23;
    return __uint_as_float((E + c - 8u) << 23);
}
__device__ __forceinline__ uint32_t enc2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float2 dec2(uint32_t v) {
    uint32_t h2; float2 f;
    asm("{ .reg .b16 a; cvt.u16.u32 a, %1; cvt.rn.f16x2.e4m3x2 %0, a; }" : "=r"(h2) : "r"(v));
    asm("{ .reg .b16 a, b; mov.b32 {a, b}, %2; cvt.f32.f16 %0, a; cvt.f32.f16 %1, b; }" : "=f"(f.x), "=f"(f.y) : "r"(h2));
    return f;
}

__device__ __forceinline__ uint32_t enc4(float a, float b, float c, float d) { return enc2(a, b) | (enc2(c, d) << 16); }
__device__ __forceinline__ void dec4(uint32_t v, float *o) {
    const float2 lo = dec2(v & 0xffffu), hi = dec2(v >> 16);
    o[0] = lo.x; o[1] = lo.y; o[2] = hi.x; o[3] = hi.y;
}
// f32 -> bf16 bits, round to nearest even, NaN kept quiet
__device__ __forceinline__ uint32_t bf16_rne_bits(float f) {
    const uint32_t b = __float_as_uint(f);
    return ((b & 0x7fffffffu) > 0x7f800000u) ? ((b >> 16) | 0x40u) : ((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
}
// THE activation quantiser of this library (src/omega_blackwell_codegen_qg.h:7-19 in the reference), one call per warp and
// 128-column group, lane = 4 consecutive columns: amax over the group floored at 2^-100, scale = the smallest power of two with
// amax / scale <= 448, code = e4m3 round-to-nearest-even, saturating. pieces > 1 (this library's exact-activation format): piece
// p re-encodes the residual the earlier pieces left, scaled by 16^p; every step is exact in f32. Every kernel that produces
// activation pieces calls this one function, so the stand-alone quantiser, the fused stack step and the expert-parallel stack step
// cannot drift apart. Returns the scale; codes[p] = this lane's four codes of piece p.
__device__ __forceinline__ float quant_pieces_warp(const float *v, uint32_t pieces, uint32_t *codes) {
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = pq_scale_mma(amax);
    const float inv = __uint_as_float((254u - (__float_as_uint(s) >> 23)) << 23);   // s is a power of two: exact reciprocal, v * inv == v / s
    float res[4];
#pragma unroll
    for (int i = 0; i < 4; i++) res[i] = v[i] * inv;
    for (uint32_t p = 0; p < pieces; p++) {
        codes[p] = enc4(res[0], res[1], res[2], res[3]);
        if (p + 1 == pieces) break;
        float d[4]; dec4(codes[p], d);
#pragma unroll
        for (int i = 0; i < 4; i++) res[i] = (res[i] - d[i]) * 16.0f;
    }
    return s;
}

// Router-weighted sum of one token's K result rows at columns c .. c + 3, in slot order, multiply then add, never fused: the reference's combine
// (src/omega_blackwell_codegen_dec.c:226-255). All K row loads are issued before the first one is used: with a run-time slot count the loop
// serialises K dependent memory round trips per thread (measured: 14 us per layer for this step at 8 slots, against 4 with the loads in flight).
// VOLATILE: rows written by peer GPUs are read past L1.
template <int K, bool VOLATILE>
__device__ __forceinline__ float4 combine_slots_k(const float *__restrict__ w, const float *__restrict__ dn, size_t first_row, uint32_t hidden, uint32_t c) {
    float ws[K]; float4 d[K];
#pragma unroll
    for (int s = 0; s < K; s++) {
        ws[s] = __ldg(w + first_row + s);
        const float4 *p = reinterpret_cast<const float4 *>(dn + (first_row + s) * hidden + c);
        d[s] = VOLATILE ? __ldcv(p) : __ldg(p);
    }
    float4 m = make_float4(__fmul_rn(ws[0], d[0].x), __fmul_rn(ws[0], d[0].y), __fmul_rn(ws[0], d[0].z), __fmul_rn(ws[0], d[0].w));
#pragma unroll
    for (int s = 1; s < K; s++)
        m = make_float4(__fadd_rn(m.x, __fmul_rn(ws[s], d[s].x)), __fadd_rn(m.y, __fmul_rn(ws[s], d[s].y)), __fadd_rn(m.z, __fmul_rn(ws[s], d[s].z)), __fadd_rn(m.w, __fmul_rn(ws[s], d[s].w)));
    return m;
}
template <bool VOLATILE>
__device__ __forceinline__ float4 combine_slots(uint32_t topk, const float *__restrict__ w, const float *__restrict__ dn, size_t first_row, uint32_t hidden, uint32_t c) {
    switch (topk) {
        case 8: return combine_slots_k<8, VOLATILE>(w, dn, first_row, hidden, c);
        case 9: return combine_slots_k<9, VOLATILE>(w, dn, first_row, hidden, c);
        case 4: return combine_slots_k<4, VOLATILE>(w, dn, first_row, hidden, c);
        case 5: return combine_slots_k<5, VOLATILE>(w, dn, first_row, hidden, c);
        case 2: return combine_slots_k<2, VOLATILE>(w, dn, first_row, hidden, c);
        default: break;
    }
    float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t s = 0; s < topk; s++) {
        const float ws = __ldg(w + first_row + s);
        const float4 *p = reinterpret_cast<const float4 *>(dn + (first_row + s) * hidden + c);
        const float4 d = VOLATILE ? __ldcv(p) : __ldg(p);
        const float4 q = make_float4(__fmul_rn(ws, d.x), __fmul_rn(ws, d.y), __fmul_rn(ws, d.z), __fmul_rn(ws, d.w));
        m = s == 0 ? q : make_float4(__fadd_rn(m.x, q.x), __fadd_rn(m.y, q.y), __fadd_rn(m.z, q.z), __fadd_rn(m.w, q.w));
    }
    return m;
}

}  // namespace b200
