// w4_gemm.cu: signed int4 group-scaled weights (two per byte along K, low nibble = even column; fp16 scale per 32
// columns) times bf16 activations, f32 accumulation, bf16 output. The reference has no integer-W4 arithmetic
// (docs/models/QUANT.md:62 of the reference: "integer W4 refuses"), so this follows the benchmark definition only:
// y[m][r] = sum over groups g of scale[r][g] * sum_{c in g} x[m][c] * q[r][c].
// Two kernels. The tensor-core kernel takes the shapes it is written for (n a multiple of 128; k 1024, 2048 or 4096); the
// CUDA-core kernel takes every other shape: a warp owns RW output rows; lane l owns K groups l, l+32, ... (16 contiguous bytes
// each, 512 contiguous bytes per warp load); the activation panel sits in shared memory as bf16.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdlib.h>
#include "internal.h"


namespace b200 {

constexpr int W4_RW = 2;    // output rows per warp task
constexpr int W4_MT = 16;   // activation rows per pass

__global__ void __launch_bounds__(256) w4_gemm_kernel(uint32_t m, uint32_t n, uint32_t k, const uint8_t *__restrict__ w, const uint16_t *__restrict__ sc,
                                                      const uint16_t *__restrict__ x, uint16_t *__restrict__ y16, float *__restrict__ y32) {
    extern __shared__ uint16_t xs[];   // [W4_MT][k] bf16
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, groups = k / 32u;
    for (uint32_t m0 = 0; m0 < m; m0 += W4_MT) {
        const uint32_t mt = min((uint32_t)W4_MT, m - m0);
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < W4_MT * k / 8; i += 256) {
            const uint32_t r = i / (k / 8), c8 = i - r * (k / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < mt) v = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)(m0 + r) * k) + c8);
            reinterpret_cast<uint4 *>(xs)[i] = v;
        }
        __syncthreads();
        for (uint32_t rb = (blockIdx.x * 8 + warp) * W4_RW; rb < n; rb += gridDim.x * 8 * W4_RW) {
            float acc[W4_RW][W4_MT];
#pragma unroll
            for (int j = 0; j < W4_RW; j++)
#pragma unroll
                for (int mm = 0; mm < W4_MT; mm++) acc[j][mm] = 0.0f;
            for (uint32_t g = lane; g < groups; g += 32) {
                float q[W4_RW][32]; float s[W4_RW];
#pragma unroll
                for (int j = 0; j < W4_RW; j++) {
                    const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(w + ((size_t)(rb + j) * k) / 2) + g);
                    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int i = 0; i < 32; i++) q[j][i] = (float)(((int32_t)(u[i >> 3] << (28 - 4 * (i & 7)))) >> 28);
                    s[j] = __half2float(__ushort_as_half(__ldg(sc + (size_t)(rb + j) * groups + g)));
                }
#pragma unroll 4
                for (int mm = 0; mm < W4_MT; mm++) {
                    float part[W4_RW];
#pragma unroll
                    for (int j = 0; j < W4_RW; j++) part[j] = 0.0f;
                    const uint4 *xp = reinterpret_cast<const uint4 *>(xs + (size_t)mm * k + g * 32u);
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const uint4 xv = xp[c];
                        const uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float x0 = __uint_as_float(xu[e] << 16), x1 = __uint_as_float(xu[e] & 0xffff0000u);
#pragma unroll
                            for (int j = 0; j < W4_RW; j++) { part[j] = fmaf(x0, q[j][c * 8 + e * 2], part[j]); part[j] = fmaf(x1, q[j][c * 8 + e * 2 + 1], part[j]); }
                        }
                    }
#pragma unroll
                    for (int j = 0; j < W4_RW; j++) acc[j][mm] = fmaf(part[j], s[j], acc[j][mm]);
                }
            }
#pragma unroll
            for (int j = 0; j < W4_RW; j++)
#pragma unroll
                for (int mm = 0; mm < W4_MT; mm++) {
                    float v = acc[j][mm];
                    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (lane == 0 && (uint32_t)mm < mt) {
                        const size_t at = (size_t)(m0 + mm) * n + rb + j;
                        if (y32) y32[at] = v;
                        if (y16) { const uint32_t b = __float_as_uint(v); y16[at] = (uint16_t)(((b & 0x7fffffffu) > 0x7f800000u) ? ((b >> 16) | 0x40u) : ((b + 0x7fffu + ((b >> 16) & 1u)) >> 16)); }
                    }
                }
        }
    }
}

// ---------------------------------------------------------------- tensor-core kernel
// The activation panel has at most 16 rows per pass: exactly the M of the warp-level mma.sync m16n8k16 (the tcgen05 MMA starts at M 64 and
// takes its operands from shared or tensor memory, so the int4 -> bf16 expansion would have to go through shared memory; here it stays
// in registers, and the kernel is a weight stream whose tensor work is a few percent of the memory time either way).
// int4 values are exact in bf16; a scale group is 32 columns = two k16 MMAs into a fresh accumulator, then acc += scale * partial in f32:
// the definition's own order of operations (group sums first, then the scale). Work split: grid (n / 128, 4 K quarters), 16 warps, a warp owns
// 8 output rows (one n8 tile) over its quarter's groups; every weight word a thread needs is requested before the first one is used (the whole
// matrix is in flight at once). Inside a group the 32 columns are dealt to the MMA's k slots so that thread t of a quad uses exactly the 8
// nibbles of its own 32-bit word (columns 8t .. 8t+7): k slots {2t, 2t+1, 2t+8, 2t+9} of the first MMA are columns 8t .. 8t+3, of the second
// 8t+4 .. 8t+7; the activation fragments follow the same dealing, so each product meets its own weight. The four K quarters of an output block
// meet in a scratch buffer; the CTA that arrives last adds them in quarter order (a fixed order: same bits every run).
__device__ __forceinline__ void mma_bf16_16816(float *d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// byte j of v (two signed nibbles: low = even column) -> two bf16 values. 0x4300 | (nibble ^ 8) is the bf16 number 128 + (q + 8); minus 136 gives q exactly.
__device__ __forceinline__ uint32_t nib2_bf16(uint32_t v, int j) {
    const uint32_t b = v >> (8 * j);
    uint32_t u = (((b & 0xFu) | ((b << 12) & 0xF0000u)) ^ 0x00080008u) | 0x43004300u;
    __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162 *>(&u);
    h = __hsub2(h, __floats2bfloat162_rn(136.0f, 136.0f));
    return *reinterpret_cast<uint32_t *>(&h);
}

// Eight E2M1 nibbles of v -> four bf16 pairs (b[j] = the two nibbles of byte j, low nibble = even column = low half). The seven magnitudes
// 0.5, 1, 1.5, 2, 3, 4, 6 are exact in bf16; a byte-permute looks the low and the high byte of each up in 8-entry tables, the sign bit moves to bit 15
// (the reference's scalar decoder: native/models/mxfp4.om, docs/models/MXFP4.md:4-9; signed zero kept).
__device__ __forceinline__ void e2m1x8_bf16(uint32_t v, uint32_t *b) {
    const uint32_t m = v & 0x77777777u;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint32_t sel = h ? (m >> 16) : (m & 0xffffu), sg = h ? (v >> 16) : (v & 0xffffu);
        uint32_t lo, hi, p01, p23;
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(lo) : "r"(0xC0800000u), "r"(0xC0804000u), "r"(sel));   // low bytes of bf16(0, .5, 1, 1.5 | 2, 3, 4, 6)
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(0x3F3F3F00u), "r"(0x40404040u), "r"(sel));   // high bytes
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(p01) : "r"(lo), "r"(hi), "r"(0x5140u));
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(p23) : "r"(lo), "r"(hi), "r"(0x7362u));
        b[2 * h] = p01 | ((sg & 0x8u) << 12) | ((sg & 0x80u) << 24);
        b[2 * h + 1] = p23 | ((sg & 0x800u) << 4) | ((sg & 0x8000u) << 16);
    }
}

// FMT 2 (NVFP4: E2M1 + one unsigned E4M3 scale per 16 columns): a 32-column group holds two scale groups, so its two MMAs must be columns 0..15 and
// 16..31. Thread t of a quad then feeds columns 4t .. 4t+3 to the first MMA and 16+4t .. 16+4t+3 to the second: the two 16-bit halves it needs sit in
// the words of quad threads t/2 and 2 + t/2 (one shuffle each); each MMA goes into its own fresh accumulator and is scaled by its own scale.
template <int GQ, int FMT>   // 32-column groups per K quarter: k = 128 * GQ; FMT 0: int4 + fp16 scales, 1: E2M1 + E8M0 scales (MXFP4), 2: E2M1 + UE4M3 per 16 (NVFP4)
__global__ void __launch_bounds__(512, GQ <= 16 ? 2 : 1) w4_mma_kernel(uint32_t m0, uint32_t m, uint32_t n, uint32_t k, const uint8_t *__restrict__ w, const uint16_t *__restrict__ sc,
                                                        const uint16_t *__restrict__ x, uint16_t *__restrict__ y16, float *__restrict__ y32, float *part, uint32_t *counters,
                                                        const uint4 *__restrict__ tiles, const uint32_t *__restrict__ header, const uint32_t *__restrict__ xmap, const uint32_t *__restrict__ ymap) {
    constexpr uint32_t KQ = GQ * 32u, XS = KQ * 2u + 64u;   // columns per quarter; bytes between panel rows (the 64 keep a quarter-warp's 16-byte reads on separate banks)
    extern __shared__ __align__(16) uint8_t xq[];
    __shared__ uint32_t s_last;
    const uint32_t nb = blockIdx.x, kq = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, r = lane >> 2, t = lane & 3u;
    // grouped form (tiles != null): blockIdx.z is a row tile {expert, first sorted row, rows <= 16} of a routing plan; the tensor holds the experts' matrices
    // one after the other (n rows each); activation row i of the tile is x[xmap[row0 + i]] (or row0 + i), its result goes to row ymap[row0 + i] (or row0 + i)
    uint32_t mt = 0, row0 = m0;
    if (tiles) {
        if (blockIdx.z >= header[2]) return;
        const uint4 tl = tiles[blockIdx.z];
        w += (size_t)tl.x * n * (k / 2u); sc = reinterpret_cast<const uint16_t *>(reinterpret_cast<const uint8_t *>(sc) + (size_t)tl.x * n * (k / 32u) * (FMT == 1 ? 1u : 2u));
        row0 = tl.y; mt = min(16u, tl.z);
        part += (size_t)blockIdx.z * 4u * 16u * n; counters += (size_t)blockIdx.z * (n / 128u);
    } else mt = min(16u, m - m0);
    // this thread's weight words: output row n0 + r, word t of every group of the quarter; all requested before anything else
    const uint32_t n0 = nb * 128u + warp * 8u;
    const uint32_t *wrow = reinterpret_cast<const uint32_t *>(w + (size_t)(n0 + r) * (k / 2u) + (size_t)kq * (KQ / 2u));
    uint32_t wq[GQ];
#pragma unroll
    for (int g = 0; g < GQ; g++) wq[g] = __ldcs(wrow + g * 4 + t);
    // scales of the two output columns this thread's accumulators belong to (n0 + 2t, n0 + 2t + 1): GQ values each, fp16 (FMT 0) or E8M0 bytes (FMT 1)
    constexpr int SB = FMT == 1 ? 1 : 2, SV = (GQ * SB + 15) / 16;   // bytes per scale; 16-byte vectors per row (GQ = 8 bytes of E8M0: half a vector, loaded as 8 bytes)
    const uint8_t *scb = reinterpret_cast<const uint8_t *>(sc);
    const uint8_t *s0b = scb + ((size_t)(n0 + 2u * t) * (k / 32u) + kq * GQ) * SB, *s1b = scb + ((size_t)(n0 + 2u * t + 1u) * (k / 32u) + kq * GQ) * SB;   // FMT 2: two scale bytes per 32 columns
    uint4 sv0[SV], sv1[SV];
    if (GQ * SB % 16 == 0) {
#pragma unroll
        for (int i = 0; i < SV; i++) { sv0[i] = __ldg(reinterpret_cast<const uint4 *>(s0b) + i); sv1[i] = __ldg(reinterpret_cast<const uint4 *>(s1b) + i); }
    } else if (GQ * SB == 8) {
        const uint2 a0 = __ldg(reinterpret_cast<const uint2 *>(s0b)), a1 = __ldg(reinterpret_cast<const uint2 *>(s1b));
        sv0[0] = make_uint4(a0.x, a0.y, 0, 0); sv1[0] = make_uint4(a1.x, a1.y, 0, 0);
    } else {   // k = 768: 6 or 12 scale bytes per quarter, two-byte aligned
        sv0[0] = make_uint4(0, 0, 0, 0); sv1[0] = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < GQ * SB / 2; i++) {
            reinterpret_cast<uint16_t *>(&sv0[0])[i] = __ldg(reinterpret_cast<const uint16_t *>(s0b) + i);
            reinterpret_cast<uint16_t *>(&sv1[0])[i] = __ldg(reinterpret_cast<const uint16_t *>(s1b) + i);
        }
    }
    // the quarter of the activation panel: rows m0 .. m0 + 15 (zero past m), columns kq * KQ ..
    for (uint32_t i = threadIdx.x; i < 16u * (KQ / 8u); i += 512u) {
        const uint32_t row = i / (KQ / 8u), c8 = i - row * (KQ / 8u);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < mt) v = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)(xmap ? xmap[row0 + row] : row0 + row) * k + (size_t)kq * KQ) + c8);
        *reinterpret_cast<uint4 *>(xq + row * XS + c8 * 16u) = v;
    }
    __syncthreads();
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int g = 0; g < GQ; g++) {
        float p[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        uint32_t bq[4];
        if (FMT == 2) {
            const uint32_t wa = __shfl_sync(0xffffffffu, wq[g], (lane & ~3u) | (t >> 1)), wb = __shfl_sync(0xffffffffu, wq[g], (lane & ~3u) | 2u | (t >> 1));
            const uint32_t v = (t & 1u) ? ((wa >> 16) | (wb & 0xffff0000u)) : ((wa & 0xffffu) | (wb << 16));   // nibbles 0..3: columns 4t..4t+3, nibbles 4..7: columns 16+4t..
            e2m1x8_bf16(v, bq);
            const uint2 xa = *reinterpret_cast<const uint2 *>(xq + r * XS + g * 64 + t * 8u), xb = *reinterpret_cast<const uint2 *>(xq + (r + 8u) * XS + g * 64 + t * 8u);
            const uint2 xc = *reinterpret_cast<const uint2 *>(xq + r * XS + g * 64 + 32u + t * 8u), xd = *reinterpret_cast<const uint2 *>(xq + (r + 8u) * XS + g * 64 + 32u + t * 8u);
            float p2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            mma_bf16_16816(p, xa.x, xb.x, xa.y, xb.y, bq[0], bq[1]);
            mma_bf16_16816(p2, xc.x, xd.x, xc.y, xd.y, bq[2], bq[3]);
            const uint32_t *u0 = reinterpret_cast<const uint32_t *>(&sv0[g >> 3]), *u1 = reinterpret_cast<const uint32_t *>(&sv1[g >> 3]);
            const uint32_t h0 = (u0[(g & 7) >> 1] >> (16 * (g & 1))) & 0xffffu, h1 = (u1[(g & 7) >> 1] >> (16 * (g & 1))) & 0xffffu;
            // unsigned E4M3: (8 + m) * 2^(e - 10) for e > 0 (binary32 exponent field e + 120), m * 2^-9 for e = 0
            auto ue4m3 = [](uint32_t c) -> float { return (c >> 3) ? __uint_as_float((((c >> 3) + 120u) << 23) | ((c & 7u) << 20)) : (float)(c & 7u) * 0.001953125f; };
            const float a0 = ue4m3(h0 & 0xffu), a1 = ue4m3(h0 >> 8), c0 = ue4m3(h1 & 0xffu), c1 = ue4m3(h1 >> 8);
            acc[0] = fmaf(p[0], a0, acc[0]); acc[1] = fmaf(p[1], c0, acc[1]); acc[2] = fmaf(p[2], a0, acc[2]); acc[3] = fmaf(p[3], c0, acc[3]);
            acc[0] = fmaf(p2[0], a1, acc[0]); acc[1] = fmaf(p2[1], c1, acc[1]); acc[2] = fmaf(p2[2], a1, acc[2]); acc[3] = fmaf(p2[3], c1, acc[3]);
            continue;
        }
        const uint4 xa = *reinterpret_cast<const uint4 *>(xq + r * XS + g * 64 + t * 16u);          // panel row r, columns 8t .. 8t+7 of group g
        const uint4 xb = *reinterpret_cast<const uint4 *>(xq + (r + 8u) * XS + g * 64 + t * 16u);   // panel row r + 8
        if (FMT) e2m1x8_bf16(wq[g], bq);
        else { bq[0] = nib2_bf16(wq[g], 0); bq[1] = nib2_bf16(wq[g], 1); bq[2] = nib2_bf16(wq[g], 2); bq[3] = nib2_bf16(wq[g], 3); }
        mma_bf16_16816(p, xa.x, xb.x, xa.y, xb.y, bq[0], bq[1]);
        mma_bf16_16816(p, xa.z, xb.z, xa.w, xb.w, bq[2], bq[3]);
        float sl, sh;
        if (FMT) {   // E8M0: 2^(byte - 127); byte 0 is 2^-127, a subnormal f32
            const uint32_t e0 = (reinterpret_cast<const uint32_t *>(&sv0[g >> 4])[(g & 15) >> 2] >> (8 * (g & 3))) & 0xffu, e1 = (reinterpret_cast<const uint32_t *>(&sv1[g >> 4])[(g & 15) >> 2] >> (8 * (g & 3))) & 0xffu;
            sl = __uint_as_float(e0 ? e0 << 23 : 0x00400000u); sh = __uint_as_float(e1 ? e1 << 23 : 0x00400000u);
        } else {
            const uint32_t *u0 = reinterpret_cast<const uint32_t *>(&sv0[g >> 3]), *u1 = reinterpret_cast<const uint32_t *>(&sv1[g >> 3]);
            const uint32_t h0 = (u0[(g & 7) >> 1] >> (16 * (g & 1))) & 0xffffu, h1 = (u1[(g & 7) >> 1] >> (16 * (g & 1))) & 0xffffu;
            sl = __half2float(__ushort_as_half((unsigned short)h0)); sh = __half2float(__ushort_as_half((unsigned short)h1));
        }
        acc[0] = fmaf(p[0], sl, acc[0]); acc[1] = fmaf(p[1], sh, acc[1]); acc[2] = fmaf(p[2], sl, acc[2]); acc[3] = fmaf(p[3], sh, acc[3]);
    }
    // this quarter's share of the block: part[kq][row][n]
    *reinterpret_cast<float2 *>(part + ((size_t)kq * 16u + r) * n + n0 + 2u * t) = make_float2(acc[0], acc[1]);
    *reinterpret_cast<float2 *>(part + ((size_t)kq * 16u + r + 8u) * n + n0 + 2u * t) = make_float2(acc[2], acc[3]);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(counters + nb, 1u) == 3u ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (uint32_t i = threadIdx.x; i < 16u * 128u; i += 512u) {
        const uint32_t row = i >> 7, col = nb * 128u + (i & 127u);
        if (row >= mt) continue;
        float v = __ldcg(part + (size_t)row * n + col);
#pragma unroll
        for (uint32_t q = 1; q < 4; q++) v = __fadd_rn(v, __ldcg(part + ((size_t)q * 16u + row) * n + col));
        const size_t at = (size_t)(ymap ? ymap[row0 + row] : row0 + row) * n + col;
        if (y32) y32[at] = v;
        if (y16) { const uint32_t b = __float_as_uint(v); y16[at] = (uint16_t)(((b & 0x7fffffffu) > 0x7f800000u) ? ((b >> 16) | 0x40u) : ((b + 0x7fffu + ((b >> 16) & 1u)) >> 16)); }
    }
    if (threadIdx.x == 0) counters[nb] = 0;   // ready for the next launch (launches on one tensor are stream-ordered)
}

// NVFP4 block quantiser (the reference's native/models/nvfp4.om: nvfp4nib = nvfp4scale + nvfp4enc per element). One thread per 16-element block of a
// bf16 row: amax over the magnitudes, scale = e4m3 (nearest even, saturating) of the binary32 quotient amax / 6, then every element's nibble by comparing
// its magnitude with scale x {1, 3, 5, 7, 10, 14, 20} / 4 (exact binary32 products), a tie going to the even code, above 6 saturating. NaN sets *bad.
__global__ void __launch_bounds__(256) nvfp4_quantize_kernel(size_t blocks, const uint16_t *__restrict__ w, uint8_t *__restrict__ packed, uint8_t *__restrict__ scales, int *bad) {
    const size_t b = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (b >= blocks) return;
    const uint4 lo = __ldg(reinterpret_cast<const uint4 *>(w + b * 16)), hi = __ldg(reinterpret_cast<const uint4 *>(w + b * 16) + 1);
    const uint32_t v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    uint32_t amax = 0; bool nan = false;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t a0 = (v[i] & 0x7fffu) << 16, a1 = v[i] & 0x7fff0000u;
        nan |= a0 > 0x7f800000u || a1 > 0x7f800000u;
        amax = max(amax, max(a0, a1));
    }
    if (nan) { atomicExch(bad, 1); return; }
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(__fdiv_rn(__uint_as_float(amax), 6.0f)));
    const uint32_t sc = r & 0x7fu, se = sc >> 3, sig = se ? ((sc & 7u) | 8u) : (sc & 7u);
    const float unit = __uint_as_float((uint32_t)((se ? (int)se - 10 : -9) - 2 + 127) << 23);   // 2^(exponent of the scale - 2)
    const float t0 = (float)(sig * 1u) * unit, t1 = (float)(sig * 3u) * unit, t2 = (float)(sig * 5u) * unit, t3 = (float)(sig * 7u) * unit,
                t4 = (float)(sig * 10u) * unit, t5 = (float)(sig * 14u) * unit, t6 = (float)(sig * 20u) * unit;
    auto enc = [&](uint32_t bits) -> uint32_t {   // bits: a binary32 pattern
        const uint32_t sign = (bits >> 28) & 8u;
        if (sig == 0) return sign;
        const float a = __uint_as_float(bits & 0x7fffffffu);
        // codes 0..7; thresholds between k and k + 1; a tie stays at k when k is even, goes to k + 1 when k is odd
        uint32_t c = (a > t0) + (a >= t1) + (a > t2) + (a >= t3) + (a > t4) + (a >= t5) + (a > t6);
        return sign | c;
    };
    uint32_t out[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t byte = enc(v[i] << 16) | (enc(v[i] & 0xffff0000u) << 4);   // element 2i in the low nibble
        out[i >> 2] |= byte << (8 * (i & 3));
    }
    *reinterpret_cast<uint2 *>(packed + b * 8) = make_uint2(out[0], out[1]);
    scales[b] = (uint8_t)sc;
}

cudaError_t launch_w4_grouped(const OmegaGpuW4Tensor *t, const void *tiles, const uint32_t *header, const uint32_t *xmap, const uint32_t *ymap,
                              const uint16_t *dx, uint16_t *d16, float *d32, cudaStream_t s) {
    const dim3 grid(t->gn / 128u, 4, t->gtiles);
#define W4_GROUPED(GQV, FMTV) w4_mma_kernel<GQV, FMTV><<<grid, 512, 16 * (GQV * 64 + 64), s>>>(0u, 0u, t->gn, t->k, t->w, t->s, dx, d16, d32, t->gpart, t->gcounters, \
        (const uint4 *)tiles, header, xmap, ymap)
    if (t->fmt == 2) { if (t->k == 4096u) W4_GROUPED(32, 2); else if (t->k == 2048u) W4_GROUPED(16, 2); else if (t->k == 1024u) W4_GROUPED(8, 2); else W4_GROUPED(6, 2); }
    else if (t->fmt) { if (t->k == 4096u) W4_GROUPED(32, 1); else if (t->k == 2048u) W4_GROUPED(16, 1); else if (t->k == 1024u) W4_GROUPED(8, 1); else W4_GROUPED(6, 1); }
    else { if (t->k == 4096u) W4_GROUPED(32, 0); else if (t->k == 2048u) W4_GROUPED(16, 0); else if (t->k == 1024u) W4_GROUPED(8, 0); else W4_GROUPED(6, 0); }
#undef W4_GROUPED
    return cudaGetLastError();
}

}  // namespace b200
using namespace b200;

extern "C" {

int omega_gpu_w4_upload(uint32_t n, uint32_t k, const uint8_t *packed, const uint16_t *scale_f16, OmegaGpuW4Tensor **out) {
    if (out) *out = nullptr;
    if (!out || !packed || !scale_f16 || !n || !k || k % 32 || n % W4_RW) return OMEGA_GPU_FP8_BAD_ARGS;
    if ((size_t)W4_MT * k * 2 > 200 * 1024) return OMEGA_GPU_FP8_TOO_LARGE;
    for (size_t i = 0; i < (size_t)n * (k / 32); i++) if ((scale_f16[i] & 0x7c00u) == 0x7c00u) { set_error("w4 upload: NaN or inf scale"); return OMEGA_GPU_FP8_BAD_ARGS; }
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    OmegaGpuW4Tensor *t = (OmegaGpuW4Tensor *)calloc(1, sizeof *t);
    if (!t) return OMEGA_GPU_FP8_BAD_ARGS;
    t->n = n; t->k = k;
    const size_t wb = (size_t)n * k / 2, sb = (size_t)n * (k / 32) * 2;
    bool ok = cuda_ok(cudaMalloc(&t->w, wb), "cudaMalloc(w4)") && cuda_ok(cudaMalloc(&t->s, sb), "cudaMalloc(w4 scales)") &&
              cuda_ok(cudaMemcpy(t->w, packed, wb, cudaMemcpyHostToDevice), "copy w4") && cuda_ok(cudaMemcpy(t->s, scale_f16, sb, cudaMemcpyHostToDevice), "copy w4 scales");
    if (ok && n % 128u == 0 && (k == 768u || k == 1024u || k == 2048u || k == 4096u)) {   // the tensor-core kernel's scratch
        const size_t pb = (size_t)4 * 16 * n * 4, cb = (size_t)(n / 128u) * 4;
        ok = cuda_ok(cudaMalloc(&t->part, pb), "cudaMalloc(w4 partials)") && cuda_ok(cudaMalloc(&t->counters, cb), "cudaMalloc(w4 counters)") &&
             cuda_ok(cudaMemset(t->counters, 0, cb), "memset");
    }
    if (!ok) { if (t->w) cudaFree(t->w); if (t->s) cudaFree(t->s); if (t->part) cudaFree(t->part); if (t->counters) cudaFree(t->counters); free(t); return OMEGA_GPU_FP8_CHIP_FAIL; }
    *out = t;
    return OMEGA_GPU_FP8_OK;
}
/* MXFP4 weights (E2M1 nibbles, low nibble = even column, E8M0 scale per 32 columns: the format of docs/models/MXFP4.md in the reference, whose
 * scalar decoder native/models/mxfp4.om defines every element's value). The tensor runs through omega_gpu_w4_gemm_bf16 / _async like an int4 one. */
int omega_gpu_mxfp4_upload(uint32_t n, uint32_t k, const uint8_t *packed, const uint8_t *scale_e8m0, OmegaGpuW4Tensor **out) {
    if (out) *out = nullptr;
    if (!out || !packed || !scale_e8m0 || !n || !k) return OMEGA_GPU_FP8_BAD_ARGS;
    if (n % 128u || !(k == 768u || k == 1024u || k == 2048u || k == 4096u)) { set_error("mxfp4 upload: n must be a multiple of 128 and k 768, 1024, 2048 or 4096"); return OMEGA_GPU_FP8_BAD_ARGS; }
    for (size_t i = 0; i < (size_t)n * (k / 32); i++) if (scale_e8m0[i] == 0xffu) { set_error("mxfp4 upload: scale 255 (a NaN block) at group %zu", i); return OMEGA_GPU_FP8_NAN_WEIGHT; }
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    OmegaGpuW4Tensor *t = (OmegaGpuW4Tensor *)calloc(1, sizeof *t);
    if (!t) return OMEGA_GPU_FP8_BAD_ARGS;
    t->n = n; t->k = k; t->fmt = 1;
    const size_t wb = (size_t)n * k / 2, sb = (size_t)n * (k / 32), pb = (size_t)4 * 16 * n * 4, cb = (size_t)(n / 128u) * 4;
    const bool ok = cuda_ok(cudaMalloc(&t->w, wb), "cudaMalloc(mxfp4)") && cuda_ok(cudaMalloc((void **)&t->s, sb), "cudaMalloc(mxfp4 scales)") &&
                    cuda_ok(cudaMemcpy(t->w, packed, wb, cudaMemcpyHostToDevice), "copy mxfp4") && cuda_ok(cudaMemcpy(t->s, scale_e8m0, sb, cudaMemcpyHostToDevice), "copy mxfp4 scales") &&
                    cuda_ok(cudaMalloc(&t->part, pb), "cudaMalloc(mxfp4 partials)") && cuda_ok(cudaMalloc(&t->counters, cb), "cudaMalloc(mxfp4 counters)") &&
                    cuda_ok(cudaMemset(t->counters, 0, cb), "memset");
    if (!ok) { if (t->w) cudaFree(t->w); if (t->s) cudaFree(t->s); if (t->part) cudaFree(t->part); if (t->counters) cudaFree(t->counters); free(t); return OMEGA_GPU_FP8_CHIP_FAIL; }
    *out = t;
    return OMEGA_GPU_FP8_OK;
}
/* NVFP4 weights (E2M1 nibbles, low nibble = even column, one unsigned E4M3 scale per 16 columns, no second-level scale: the reference's
 * native/models/nvfp4.om, docs/models/MXFMT.md). Scale codes 0..126 only: 127 is NaN and 128..255 carry a sign bit, both refused as that unit does. */
int omega_gpu_nvfp4_upload(uint32_t n, uint32_t k, const uint8_t *packed, const uint8_t *scale_ue4m3, OmegaGpuW4Tensor **out) {
    if (out) *out = nullptr;
    if (!out || !packed || !scale_ue4m3 || !n || !k) return OMEGA_GPU_FP8_BAD_ARGS;
    if (n % 128u || !(k == 768u || k == 1024u || k == 2048u || k == 4096u)) { set_error("nvfp4 upload: n must be a multiple of 128 and k 768, 1024, 2048 or 4096"); return OMEGA_GPU_FP8_BAD_ARGS; }
    for (size_t i = 0; i < (size_t)n * (k / 16); i++) {
        if (scale_ue4m3[i] == 0x7fu) { set_error("nvfp4 upload: scale 127 (NaN) at group %zu", i); return OMEGA_GPU_FP8_NAN_WEIGHT; }
        if (scale_ue4m3[i] > 0x7fu) { set_error("nvfp4 upload: scale code %u at group %zu has the sign bit set", (unsigned)scale_ue4m3[i], i); return OMEGA_GPU_FP8_BAD_ARGS; }
    }
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    OmegaGpuW4Tensor *t = (OmegaGpuW4Tensor *)calloc(1, sizeof *t);
    if (!t) return OMEGA_GPU_FP8_BAD_ARGS;
    t->n = n; t->k = k; t->fmt = 2;
    const size_t wb = (size_t)n * k / 2, sb = (size_t)n * (k / 16), pb = (size_t)4 * 16 * n * 4, cb = (size_t)(n / 128u) * 4;
    const bool ok = cuda_ok(cudaMalloc(&t->w, wb), "cudaMalloc(nvfp4)") && cuda_ok(cudaMalloc((void **)&t->s, sb), "cudaMalloc(nvfp4 scales)") &&
                    cuda_ok(cudaMemcpy(t->w, packed, wb, cudaMemcpyHostToDevice), "copy nvfp4") && cuda_ok(cudaMemcpy(t->s, scale_ue4m3, sb, cudaMemcpyHostToDevice), "copy nvfp4 scales") &&
                    cuda_ok(cudaMalloc(&t->part, pb), "cudaMalloc(nvfp4 partials)") && cuda_ok(cudaMalloc(&t->counters, cb), "cudaMalloc(nvfp4 counters)") &&
                    cuda_ok(cudaMemset(t->counters, 0, cb), "memset");
    if (!ok) { if (t->w) cudaFree(t->w); if (t->s) cudaFree(t->s); if (t->part) cudaFree(t->part); if (t->counters) cudaFree(t->counters); free(t); return OMEGA_GPU_FP8_CHIP_FAIL; }
    *out = t;
    return OMEGA_GPU_FP8_OK;
}
/* bf16 rows [rows][k] (k a multiple of 16) -> NVFP4: packed [rows][k / 2] and scales [rows][k / 16], bit for bit what the reference's block encoder
 * (native/models/nvfp4.om nvfp4nib) gives for the same values; a NaN anywhere refuses the call (NAN_WEIGHT), infinities saturate as there. */
int omega_gpu_nvfp4_quantize_bf16(uint32_t rows, uint32_t k, const uint16_t *w_bf16, uint8_t *packed, uint8_t *scale_ue4m3) {
    if (!w_bf16 || !packed || !scale_ue4m3 || !rows || !k || k % 16u) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    const size_t cnt = (size_t)rows * k, blocks = cnt / 16;
    uint16_t *dw = (uint16_t *)stage(0, cnt * 2); uint8_t *dp = (uint8_t *)stage(1, cnt / 2); uint8_t *ds = (uint8_t *)stage(2, blocks + 16);
    if (!dw || !dp || !ds) return OMEGA_GPU_FP8_CHIP_FAIL;
    int *bad = (int *)(ds + ((blocks + 7) & ~(size_t)7));
    cudaStream_t s = st().stream;
    int hbad = 0;
    bool ok = cuda_ok(cudaMemcpyAsync(dw, w_bf16, cnt * 2, cudaMemcpyHostToDevice, s), "copy weights") && cuda_ok(cudaMemsetAsync(bad, 0, 4, s), "memset");
    if (ok) {
        nvfp4_quantize_kernel<<<(unsigned)((blocks + 255) / 256), 256, 0, s>>>(blocks, dw, dp, ds, bad);
        ok = cuda_ok(cudaGetLastError(), "nvfp4 quantize launch") && cuda_ok(cudaMemcpyAsync(&hbad, bad, 4, cudaMemcpyDeviceToHost, s), "copy flag") &&
             cuda_ok(cudaStreamSynchronize(s), "nvfp4 quantize");
    }
    if (!ok) return OMEGA_GPU_FP8_CHIP_FAIL;
    if (hbad) { set_error("nvfp4 quantize: NaN value"); return OMEGA_GPU_FP8_NAN_WEIGHT; }
    ok = cuda_ok(cudaMemcpy(packed, dp, cnt / 2, cudaMemcpyDeviceToHost), "copy codes") && cuda_ok(cudaMemcpy(scale_ue4m3, ds, blocks, cudaMemcpyDeviceToHost), "copy scales");
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}
void omega_gpu_w4_free(OmegaGpuW4Tensor *t) {
    if (!t) return;
    Lock l;
    if (t->w) cudaFree(t->w);
    if (t->s) cudaFree(t->s);
    if (t->part) cudaFree(t->part);
    if (t->counters) cudaFree(t->counters);
    if (t->gpart) cudaFree(t->gpart);
    if (t->gcounters) cudaFree(t->gcounters);
    free(t);
}
static cudaError_t w4_launch(const OmegaGpuW4Tensor *t, uint32_t m, const uint16_t *dx, uint16_t *d16, float *d32, cudaStream_t s) {
    if (t->part && (t->fmt || !getenv("B200MOE_W4_FMA"))) {   // tensor-core kernel: one launch per 16 activation rows (they share the tensor's scratch, in stream order)
        const dim3 grid(t->n / 128u, 4);
        for (uint32_t m0 = 0; m0 < m; m0 += 16u) {
#define W4_LAUNCH(GQV, FMTV) w4_mma_kernel<GQV, FMTV><<<grid, 512, 16 * (GQV * 64 + 64), s>>>(m0, m, t->n, t->k, t->w, t->s, dx, d16, d32, t->part, t->counters, nullptr, nullptr, nullptr, nullptr)
            if (t->fmt == 2) { if (t->k == 4096u) W4_LAUNCH(32, 2); else if (t->k == 2048u) W4_LAUNCH(16, 2); else if (t->k == 1024u) W4_LAUNCH(8, 2); else W4_LAUNCH(6, 2); }
            else if (t->fmt) { if (t->k == 4096u) W4_LAUNCH(32, 1); else if (t->k == 2048u) W4_LAUNCH(16, 1); else if (t->k == 1024u) W4_LAUNCH(8, 1); else W4_LAUNCH(6, 1); }
            else { if (t->k == 4096u) W4_LAUNCH(32, 0); else if (t->k == 2048u) W4_LAUNCH(16, 0); else if (t->k == 1024u) W4_LAUNCH(8, 0); else W4_LAUNCH(6, 0); }
#undef W4_LAUNCH
        }
        return cudaGetLastError();
    }
    const size_t smem = (size_t)W4_MT * t->k * 2;
    static bool attr = false;
    if (!attr) { const cudaError_t e = cudaFuncSetAttribute(w4_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); if (e != cudaSuccess) return e; attr = true; }
    uint32_t grid = (t->n / W4_RW + 7) / 8; const uint32_t cap = (uint32_t)(st().sm_count ? st().sm_count : 148); if (grid > cap) grid = cap;
    w4_gemm_kernel<<<grid, 256, smem, s>>>(m, t->n, t->k, t->w, t->s, dx, d16, d32);
    return cudaGetLastError();
}
/* Grouped form: the tensor holds `experts` matrices of n_per_expert rows one after the other (uploaded as one tensor of experts x n_per_expert rows);
 * the rows to multiply come sorted by expert with a tile table of a routing plan made with tile_rows = 16 (omega_gpu_moe_plan_async: tiles {expert, first
 * row, rows}, header[2] = tiles). reserve allocates the per-tile scratch once (blocking); the async entry queues one launch and allocates nothing. */
int omega_gpu_w4_reserve_grouped(OmegaGpuW4Tensor *t, uint32_t n_per_expert, uint32_t max_tiles) {
    if (!t || !n_per_expert || !max_tiles || n_per_expert % 128u || t->n % n_per_expert || !(t->k == 768u || t->k == 1024u || t->k == 2048u || t->k == 4096u)) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    if (t->gpart) { cudaFree(t->gpart); t->gpart = nullptr; }
    if (t->gcounters) { cudaFree(t->gcounters); t->gcounters = nullptr; }
    const size_t pb = (size_t)max_tiles * 4 * 16 * n_per_expert * 4, cb = (size_t)max_tiles * (n_per_expert / 128u) * 4;
    const bool ok = cuda_ok(cudaMalloc(&t->gpart, pb), "cudaMalloc(w4 grouped partials)") && cuda_ok(cudaMalloc(&t->gcounters, cb), "cudaMalloc(w4 grouped counters)") &&
                    cuda_ok(cudaMemset(t->gcounters, 0, cb), "memset");
    if (!ok) { if (t->gpart) cudaFree(t->gpart); if (t->gcounters) cudaFree(t->gcounters); t->gpart = nullptr; t->gcounters = nullptr; return OMEGA_GPU_FP8_CHIP_FAIL; }
    t->gtiles = max_tiles; t->gn = n_per_expert;
    return OMEGA_GPU_FP8_OK;
}
int omega_gpu_w4_gemm_grouped_async(const OmegaGpuW4Tensor *t, uint64_t tiles_va, uint64_t header_va, uint64_t xmap_va, uint64_t ymap_va,
                                    uint64_t x_bf16_va, uint64_t y_bf16_va, uint64_t y_f32_va, void *stream) {
    if (!t || !tiles_va || !header_va || !x_bf16_va || (!y_bf16_va && !y_f32_va)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!t->gpart || !t->gtiles) { set_error("w4 grouped gemm: call omega_gpu_w4_reserve_grouped first"); return OMEGA_GPU_FP8_BAD_ARGS; }
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    return cuda_ok(launch_w4_grouped(t, (const void *)(uintptr_t)tiles_va, (const uint32_t *)(uintptr_t)header_va, (const uint32_t *)(uintptr_t)xmap_va, (const uint32_t *)(uintptr_t)ymap_va,
                                     (const uint16_t *)(uintptr_t)x_bf16_va, (uint16_t *)(uintptr_t)y_bf16_va, (float *)(uintptr_t)y_f32_va, (cudaStream_t)stream), "w4 grouped launch")
               ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}
int omega_gpu_w4_gemm_async(const OmegaGpuW4Tensor *t, uint32_t m, uint64_t x_bf16_va, uint64_t y_bf16_va, uint64_t y_f32_va, void *stream) {
    if (!t || !m || !x_bf16_va || (!y_bf16_va && !y_f32_va)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    return cuda_ok(w4_launch(t, m, (const uint16_t *)(uintptr_t)x_bf16_va, (uint16_t *)(uintptr_t)y_bf16_va, (float *)(uintptr_t)y_f32_va, (cudaStream_t)stream), "w4 launch")
               ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}
int omega_gpu_w4_gemm_bf16(const OmegaGpuW4Tensor *t, uint32_t m, const uint16_t *x, uint16_t *y16, float *y32) {
    if (!t || !m || !x || (!y16 && !y32)) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    const size_t xb = (size_t)m * t->k * 2, yb = (size_t)m * t->n;
    uint16_t *dx = (uint16_t *)stage(0, xb), *d16 = (uint16_t *)stage(1, yb * 2); float *d32 = (float *)stage(2, yb * 4);
    if (!dx || !d16 || !d32) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = st().stream;
    bool ok = cuda_ok(cudaMemcpyAsync(dx, x, xb, cudaMemcpyHostToDevice, s), "copy x") && cuda_ok(w4_launch(t, m, dx, d16, d32, s), "w4 launch");
    if (ok && y16) ok = cuda_ok(cudaMemcpyAsync(y16, d16, yb * 2, cudaMemcpyDeviceToHost, s), "copy y");
    if (ok && y32) ok = cuda_ok(cudaMemcpyAsync(y32, d32, yb * 4, cudaMemcpyDeviceToHost, s), "copy y");
    ok = ok && cuda_ok(cudaStreamSynchronize(s), "w4 gemm");
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

}  // extern "C"
