// moe_glue.cu: the small operators between the expert GEMMs: SiLU gate, router-weighted combine, and the
// activation quantiser that feeds the FP8 tensor-core GEMM.
#include "internal.h"
#include "mma_common.cuh"

namespace b200 {

// act[r][c] = g / (1 + exp(-g)) * u with g = gu[r][c], u = gu[r][inter + c]: the reference host glue's form
// (tests/gpu_decode_graph_test.c:61-66); its kernel computes the same with EX2/RCP approximations
// (src/omega_blackwell_codegen_dec.c:291-324).
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdiv_rn(g, 1.0f + expf(-g)) * u; }

__global__ void __launch_bounds__(256) swiglu_kernel(uint32_t rows, uint32_t inter, const float *__restrict__ gu, float *__restrict__ act, uint16_t *__restrict__ act16) {
    const size_t total = (size_t)rows * inter;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / inter, c = i - r * inter;
        const float v = silu_mul(gu[r * 2 * inter + c], gu[r * 2 * inter + inter + c]);
        if (act) act[i] = v;
        if (act16) act16[i] = (uint16_t)bf16_rne_bits(v);
    }
}
cudaError_t launch_swiglu(uint32_t rows, uint32_t inter, const float *gu, float *act, cudaStream_t s, uint16_t *act_bf16) {
    const size_t total = (size_t)rows * inter;
    if (!total) return cudaSuccess;
    size_t blocks = (total + 255) / 256; if (blocks > 148 * 8) blocks = 148 * 8;
    swiglu_kernel<<<(unsigned)blocks, 256, 0, s>>>(rows, inter, gu, act, act_bf16);
    return cudaGetLastError();
}

// out[t][c] = w0*d0 ; then m = m + w_s*d_s for s = 1.. in slot order, multiply and add kept separate
// (src/omega_blackwell_codegen_dec.c:226-255: FMUL then FADD, never FFMA).
__global__ void __launch_bounds__(256) combine_kernel(uint32_t tokens, uint32_t slots, uint32_t hidden, const float *__restrict__ w,
                                                      const float *__restrict__ d, float *__restrict__ out, uint16_t *__restrict__ out_bf16) {
    const uint32_t t = blockIdx.x;
    for (uint32_t c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
        const float4 m = combine_slots<false>(slots, w, d, (size_t)t * slots, hidden, c);
        if (out) *reinterpret_cast<float4 *>(out + (size_t)t * hidden + c) = m;
        if (out_bf16) {
            const uint32_t lo = __float_as_uint(m.x), hi = __float_as_uint(m.y), lo2 = __float_as_uint(m.z), hi2 = __float_as_uint(m.w);
            auto rne = [](uint32_t x) -> uint32_t { return ((x & 0x7fffffffu) > 0x7f800000u) ? ((x >> 16) | 0x40u) : ((x + 0x7fffu + ((x >> 16) & 1u)) >> 16); };
            uint2 pk; pk.x = rne(lo) | (rne(hi) << 16); pk.y = rne(lo2) | (rne(hi2) << 16);
            *reinterpret_cast<uint2 *>(out_bf16 + (size_t)t * hidden + c) = pk;
        }
    }
}
cudaError_t launch_combine(uint32_t tokens, uint32_t slots, uint32_t hidden, const float *w, const float *d, float *out_f32, uint16_t *out_bf16, cudaStream_t s) {
    if (!tokens) return cudaSuccess;
    combine_kernel<<<tokens, 256, 0, s>>>(tokens, slots, hidden, w, d, out_f32, out_bf16);
    return cudaGetLastError();
}

// Activation quantiser: quant_pieces_warp (mma_common.cuh) applied to rows of x. One warp per (row, 128-column group); lane = 4 columns.
__global__ void __launch_bounds__(256) act_quant_kernel(uint32_t rows, uint32_t k, uint32_t pieces, size_t piece_stride, const void *__restrict__ x, int x_bf16, size_t x_stride,
                                                        const uint32_t *__restrict__ xmap, const uint32_t *__restrict__ rows_dev,
                                                        uint8_t *__restrict__ q, float *__restrict__ sc) {
    // a kernel launched as a programmatic dependent of this one (the expert kernel: it fetches weights and waits for this grid before it reads a row) may start now
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t lane = threadIdx.x & 31u, kb = k / 128u;
    const uint32_t nrows = rows_dev ? min(rows, *rows_dev) : rows;
    const uint32_t tasks = nrows * kb, stride = gridDim.x * (blockDim.x >> 5);   // rows <= 2^24 and kb <= 32 on every caller's path
    constexpr int U = 4;   // tasks in flight per warp: their loads are issued before the first value is used
    for (uint32_t task0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); task0 < tasks; task0 += U * stride) {
        float v[U][4]; uint32_t rr[U], bb[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint32_t task = task0 + (uint32_t)u * stride;
            if (task >= tasks) { rr[u] = 0xffffffffu; bb[u] = 0; v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0.0f; continue; }   // warp-uniform
            const uint32_t r = task / kb, b = task - r * kb;
            rr[u] = r; bb[u] = b;
            const uint32_t src = xmap ? xmap[r] : r;
            if (x_bf16) {
                const uint2 w = __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const uint8_t *>(x) + (size_t)src * x_stride + (b * 128u + lane * 4u) * 2u));
                v[u][0] = __uint_as_float(w.x << 16); v[u][1] = __uint_as_float(w.x & 0xffff0000u); v[u][2] = __uint_as_float(w.y << 16); v[u][3] = __uint_as_float(w.y & 0xffff0000u);
            } else {
                const float4 w = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const uint8_t *>(x) + (size_t)src * x_stride + (b * 128u + lane * 4u) * 4u));
                v[u][0] = w.x; v[u][1] = w.y; v[u][2] = w.z; v[u][3] = w.w;
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (rr[u] == 0xffffffffu) continue;
            const uint32_t r = rr[u], b = bb[u];
            uint32_t codes[4];
            const float s = quant_pieces_warp(v[u], pieces, codes);
            if (lane == 0) sc[(size_t)r * kb + b] = s;
            for (uint32_t p = 0; p < pieces; p++) *reinterpret_cast<uint32_t *>(q + (size_t)p * piece_stride + (size_t)r * k + b * 128u + lane * 4u) = codes[p];
        }
    }
}
// q: piece p of row r at q[p * q_rows * k + r * k] (piece-major; q_rows = row capacity, 0 = rows)
cudaError_t launch_act_quant(uint32_t rows, uint32_t k, uint32_t pieces, const void *x, int x_bf16, const uint32_t *xmap, const uint32_t *rows_dev,
                             uint8_t *q, float *sc, cudaStream_t s, size_t x_stride_bytes, uint32_t q_rows) {
    if (!q_rows) q_rows = rows;
    if (!x_stride_bytes) x_stride_bytes = (size_t)k * (x_bf16 ? 2 : 4);
    const size_t tasks = (size_t)rows * (k / 128u);
    if (!tasks) return cudaSuccess;
    if (tasks >= ((size_t)1 << 32)) return cudaErrorInvalidValue;
    size_t blocks = (tasks + 7) / 8; if (blocks > 148 * 8) blocks = 148 * 8;
    act_quant_kernel<<<(unsigned)blocks, 256, 0, s>>>(rows, k, pieces, (size_t)q_rows * k, x, x_bf16, x_stride_bytes, xmap, rows_dev, q, sc);
    return cudaGetLastError();
}

// Sorted-row copies of rows that were quantised once per source row: sorted row r takes the codes (every piece) and the scales of
// source row xmap[r]. One warp per (sorted row, piece); k is a multiple of 128, so a row is k / 16 16-byte words.
__global__ void __launch_bounds__(256) gather_rows_kernel(uint32_t rows, uint32_t k, uint32_t pieces, size_t src_piece_stride, size_t dst_piece_stride,
                                                          const uint32_t *__restrict__ xmap, const uint32_t *__restrict__ rows_dev,
                                                          const uint8_t *__restrict__ q_src, const float *__restrict__ s_src, uint8_t *__restrict__ q_dst, float *__restrict__ s_dst) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // as in act_quant_kernel
    const uint32_t lane = threadIdx.x & 31u, kb = k / 128u, words = k / 16u;
    const uint32_t nrows = rows_dev ? min(rows, *rows_dev) : rows;
    const uint32_t tasks = nrows * pieces, stride = gridDim.x * (blockDim.x >> 5);
    for (uint32_t task = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); task < tasks; task += stride) {
        const uint32_t r = task / pieces, p = task - r * pieces, src = xmap[r];
        const uint4 *from = reinterpret_cast<const uint4 *>(q_src + (size_t)p * src_piece_stride + (size_t)src * k);
        uint4 *to = reinterpret_cast<uint4 *>(q_dst + (size_t)p * dst_piece_stride + (size_t)r * k);
        for (uint32_t w0 = 0; w0 < words; w0 += 128u) {   // four independent 16-byte loads per lane before the first store
            uint4 v[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { const uint32_t w = w0 + lane + 32u * i; v[i] = w < words ? __ldg(from + w) : make_uint4(0, 0, 0, 0); }
#pragma unroll
            for (int i = 0; i < 4; i++) { const uint32_t w = w0 + lane + 32u * i; if (w < words) to[w] = v[i]; }
        }
        if (p == 0) for (uint32_t b = lane; b < kb; b += 32u) s_dst[(size_t)r * kb + b] = s_src[(size_t)src * kb + b];
    }
}
cudaError_t launch_gather_rows(uint32_t rows, uint32_t k, uint32_t pieces, uint32_t src_rows, uint32_t dst_rows, const uint32_t *xmap, const uint32_t *rows_dev,
                               const uint8_t *q_src, const float *s_src, uint8_t *q_dst, float *s_dst, cudaStream_t s) {
    const size_t tasks = (size_t)rows * pieces;
    if (!tasks) return cudaSuccess;
    if (tasks >= ((size_t)1 << 32)) return cudaErrorInvalidValue;
    size_t blocks = (tasks + 7) / 8; if (blocks > 148 * 8) blocks = 148 * 8;
    gather_rows_kernel<<<(unsigned)blocks, 256, 0, s>>>(rows, k, pieces, (size_t)src_rows * k, (size_t)dst_rows * k, xmap, rows_dev, q_src, s_src, q_dst, s_dst);
    return cudaGetLastError();
}

}  // namespace b200
using namespace b200;

extern "C" {

int omega_gpu_swiglu_f32(uint32_t rows, uint32_t inter, const float *gu, float *act) {
    if (!rows || !inter || !gu || !act) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    const size_t ib = (size_t)rows * inter * 8, ob = (size_t)rows * inter * 4;
    float *dg = (float *)stage(0, ib), *da = (float *)stage(1, ob);
    if (!dg || !da) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = st().stream;
    const bool ok = cuda_ok(cudaMemcpyAsync(dg, gu, ib, cudaMemcpyHostToDevice, s), "copy gu") && cuda_ok(launch_swiglu(rows, inter, dg, da, s), "swiglu launch") &&
                    cuda_ok(cudaMemcpyAsync(act, da, ob, cudaMemcpyDeviceToHost, s), "copy act") && cuda_ok(cudaStreamSynchronize(s), "swiglu");
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_combine_f32(uint32_t tokens, uint32_t slots, uint32_t hidden, const float *w, const float *d, float *out) {
    if (!tokens || !slots || !hidden || hidden % 4 || !w || !d || !out) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    const size_t wb = (size_t)tokens * slots * 4, db = wb * hidden, ob = (size_t)tokens * hidden * 4;
    float *dw = (float *)stage(0, wb), *dd = (float *)stage(1, db), *dout = (float *)stage(2, ob);
    if (!dw || !dd || !dout) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = st().stream;
    const bool ok = cuda_ok(cudaMemcpyAsync(dw, w, wb, cudaMemcpyHostToDevice, s), "copy w") && cuda_ok(cudaMemcpyAsync(dd, d, db, cudaMemcpyHostToDevice, s), "copy d") &&
                    cuda_ok(launch_combine(tokens, slots, hidden, dw, dd, dout, nullptr, s), "combine launch") &&
                    cuda_ok(cudaMemcpyAsync(out, dout, ob, cudaMemcpyDeviceToHost, s), "copy out") && cuda_ok(cudaStreamSynchronize(s), "combine");
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_act_quant_f32(uint32_t rows, uint32_t k, uint32_t pieces, const float *x, uint8_t *q, float *sc) {
    if (!rows || !k || k % 128 || !pieces || pieces > 4 || !x || !q || !sc) return OMEGA_GPU_FP8_BAD_ARGS;
    if ((uint64_t)rows * (k / 128) >= (1ull << 32)) return OMEGA_GPU_FP8_TOO_LARGE;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    const size_t xb = (size_t)rows * k * 4, qb = (size_t)rows * pieces * k, sb = (size_t)rows * (k / 128) * 4;
    float *dx = (float *)stage(0, xb); uint8_t *dq = (uint8_t *)stage(1, qb); float *ds = (float *)stage(2, sb);
    if (!dx || !dq || !ds) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = st().stream;
    const bool ok = cuda_ok(cudaMemcpyAsync(dx, x, xb, cudaMemcpyHostToDevice, s), "copy x") &&
                    cuda_ok(launch_act_quant(rows, k, pieces, dx, 0, nullptr, nullptr, dq, ds, s), "act quant launch") &&
                    cuda_ok(cudaMemcpyAsync(q, dq, qb, cudaMemcpyDeviceToHost, s), "copy q") && cuda_ok(cudaMemcpyAsync(sc, ds, sb, cudaMemcpyDeviceToHost, s), "copy s") &&
                    cuda_ok(cudaStreamSynchronize(s), "act quant");
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

}  // extern "C"
