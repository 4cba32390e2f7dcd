// fp8_gemv.cu: FP8 e4m3 block-scaled GEMV / grouped GEMV / grouped row-table GEMM on the CUDA cores.
//
// This is the exactness engine: it keeps the summation order of the reference kernels
// (src/omega_blackwell_codegen_moe.h:13-29, src/omega_blackwell_codegen_gemm.h:5-14; host emulation
// tests/gpu_fp8gemm_test.c:48-69) so every output is bit-identical to them: lane L of a warp owns LB contiguous
// columns per K step of 32*LB columns; dot = FMA chain over those LB bytes; acc = fma(dot, scale, acc) once per
// step; lanes are summed by a shuffle-down tree 16, 8, 4, 2, 1. The reference folds 2^-120 / 2^64 / 2^56 into
// w / x / scale because its integer byte decode yields e4m3 * 2^-120; here cvt.f16x2.e4m3x2 decodes exactly, so
// no fold is stored (the folds are exact powers of two whose product is 1: same bits).
//
// Weight bytes are streamed once with 16/8/4-byte loads per lane (512/256/128 contiguous bytes per warp) and
// decoded in registers; R output rows per warp share each x chunk, MT activation rows share each weight chunk.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "internal.h"

namespace b200 {

template <int LB> struct WVec;
template <> struct WVec<16> { using T = uint4; };
template <> struct WVec<8> { using T = uint2; };
template <> struct WVec<4> { using T = uint32_t; };

__device__ __forceinline__ void decode4(uint32_t v, float *o) {
    uint32_t lo, hi;
    asm("{ .reg .b16 a, b; mov.b32 {a, b}, %2; cvt.rn.f16x2.e4m3x2 %0, a; cvt.rn.f16x2.e4m3x2 %1, b; }" : "=r"(lo), "=r"(hi) : "r"(v));
    const float2 f0 = __half22float2(*reinterpret_cast<__half2 *>(&lo)), f1 = __half22float2(*reinterpret_cast<__half2 *>(&hi));
    o[0] = f0.x; o[1] = f0.y; o[2] = f1.x; o[3] = f1.y;
}
template <int LB> __device__ __forceinline__ void load_w(const uint8_t *p, float *o) {
    typename WVec<LB>::T v = __ldcs(reinterpret_cast<const typename WVec<LB>::T *>(p));  // streaming: read once
    const uint32_t *u = reinterpret_cast<const uint32_t *>(&v);
#pragma unroll
    for (int i = 0; i < LB / 4; i++) decode4(u[i], o + 4 * i);
}
template <int LB> __device__ __forceinline__ void load_x(const void *x, int bf16, uint32_t c0, float *o) {
    if (bf16) {
        const uint16_t *p = reinterpret_cast<const uint16_t *>(x) + c0;
#pragma unroll
        for (int i = 0; i < LB / 4; i++) {
            const uint2 v = __ldg(reinterpret_cast<const uint2 *>(p) + i);
            o[4 * i] = __uint_as_float(v.x << 16); o[4 * i + 1] = __uint_as_float(v.x & 0xffff0000u);
            o[4 * i + 2] = __uint_as_float(v.y << 16); o[4 * i + 3] = __uint_as_float(v.y & 0xffff0000u);
        }
    } else {
        const float4 *p = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + c0);
#pragma unroll
        for (int i = 0; i < LB / 4; i++) { const float4 v = __ldg(p + i); o[4 * i] = v.x; o[4 * i + 1] = v.y; o[4 * i + 2] = v.z; o[4 * i + 3] = v.w; }
    }
}

// grid (ctas, groups or segments); block 256 (8 warps). Warp task: R consecutive output rows x one pass of MT activation rows.
template <int LB, int R, int MT>
__global__ void __launch_bounds__(256) fp8_rows_kernel(const GemvArgs a) {
    const uint32_t g = blockIdx.y, lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    uint64_t w_va, s_va; uint32_t row0, cnt;
    if (a.seg) {
        const Seg32 sg = a.seg[g];
        w_va = sg.w_va; s_va = sg.s_va; row0 = sg.row0; cnt = sg.cnt;
        if (cnt == 0) return;
    } else {
        const uint32_t gg = (a.mutant == 3 && (g ^ 1u) < a.groups_or_segs) ? (g ^ 1u) : g;
        w_va = a.tab[2 * gg]; s_va = a.tab[2 * gg + 1]; row0 = g; cnt = 1;
    }
    const uint8_t *W = reinterpret_cast<const uint8_t *>(w_va);
    const float *S = reinterpret_cast<const float *>(s_va);
    const uint32_t n = a.n, k = a.k, kb = k / 128u, steps = k / (32u * LB);
    const size_t xstride = a.x_stride_bytes ? a.x_stride_bytes : (size_t)k * (a.x_bf16 ? 2 : 4);
    for (uint32_t rb = (blockIdx.x * nw + warp) * R; rb < n; rb += gridDim.x * nw * R) {
        const uint8_t *wrow = W + (size_t)rb * k + lane * LB;
        const float *srow = S + (size_t)(rb / 128u) * kb;   // R divides 128: the R rows share a scale row
        for (uint32_t i0 = 0; i0 < cnt; i0 += MT) {
            float acc[R][MT];
            const uint8_t *xr[MT];
#pragma unroll
            for (int m = 0; m < MT; m++) {
                uint32_t p = row0 + (i0 + m < cnt ? i0 + m : i0);
                if (a.seg && a.mutant == 3 && (p ^ 1u) < a.rows) p ^= 1u;
                const uint32_t xi = a.seg ? (a.xmap ? a.xmap[p] : p) : (a.x_rows == 1 ? 0u : p);
                xr[m] = reinterpret_cast<const uint8_t *>(a.x) + (size_t)xi * xstride;
#pragma unroll
                for (int j = 0; j < R; j++) acc[j][m] = 0.0f;
            }
#pragma unroll(R == 1 && MT == 1 ? 4 : 2)   // one row per warp: all four 16-byte weight loads of a 2048-wide row in flight
            for (uint32_t st = 0; st < steps; st++) {
                const uint32_t c0 = st * 32u * LB + lane * LB;
                float wv[R][LB];
#pragma unroll
                for (int j = 0; j < R; j++) load_w<LB>(wrow + (size_t)j * k + (size_t)st * 32u * LB, wv[j]);
                const float sc = a.mutant == 1 ? 1.0f : __ldg(srow + (a.mutant == 2 ? 0u : c0 / 128u));
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    float xv[LB];
                    load_x<LB>(xr[m], a.x_bf16, c0, xv);
#pragma unroll
                    for (int j = 0; j < R; j++) {
                        float dot = 0.0f;
#pragma unroll
                        for (int b = 0; b < LB; b++) dot = fmaf(wv[j][b], xv[b], dot);
                        acc[j][m] = fmaf(dot, sc, acc[j][m]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < R; j++)
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    float v = acc[j][m];
#pragma unroll
                    for (int o = 16; o >= 1; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
                    if (lane == 0 && i0 + m < cnt) {
                        const uint32_t p = row0 + i0 + m;
                        const uint32_t yi = (a.seg && a.ymap) ? a.ymap[p] : p;
                        a.y[(size_t)yi * n + rb + j] = v * a.out_mul;
                    }
                }
        }
    }
}

template <int R, int MT>
static cudaError_t launch_lb(const GemvArgs &a, dim3 grid, cudaStream_t s) {
    const uint32_t k = a.k;
    if (k % 512u == 0) fp8_rows_kernel<16, R, MT><<<grid, 256, 0, s>>>(a);
    else if (k % 256u == 0) fp8_rows_kernel<8, R, MT><<<grid, 256, 0, s>>>(a);
    else fp8_rows_kernel<4, R, MT><<<grid, 256, 0, s>>>(a);
    return cudaGetLastError();
}

// GEMV forms: one activation row per group. CTAs per group chosen to put about four 8-warp CTAs on every SM.
cudaError_t launch_gemv_grouped(const GemvArgs &a, uint32_t cta_budget, uint32_t *grid_x, uint32_t *warps, cudaStream_t s) {
    const uint32_t sms = st().sm_count ? st().sm_count : 148u;
    const uint32_t row_groups = a.n / 4u;                    // R = 4 rows per warp task
    uint32_t gx = (row_groups + 7u) / 8u;                    // one task per warp
    uint32_t want = cta_budget ? cta_budget : (sms * 4u + a.groups_or_segs - 1u) / a.groups_or_segs;
    if (want == 0) want = 1;
    if (gx > want) gx = want;
    if (warps) *warps = 8;
    if (gx * a.groups_or_segs < sms && !cta_budget) {
        // few groups (the single-projection call): four rows per warp would leave most SMs without a CTA; one row per warp gives
        // four times the CTAs. A row's arithmetic does not depend on how rows are dealt to warps: same bits.
        gx = (a.n + 7u) / 8u;
        if (gx > want) gx = want;
        if (grid_x) *grid_x = gx;
        return launch_lb<1, 1>(a, dim3(gx, a.groups_or_segs), s);
    }
    if (grid_x) *grid_x = gx;
    return launch_lb<4, 1>(a, dim3(gx, a.groups_or_segs), s);
}
// Row-table form: MT = 4 activation rows per pass of a segment's weights.
cudaError_t launch_gemm_rows(const GemvArgs &a, uint32_t *grid_x, uint32_t *mt, cudaStream_t s) {
    const uint32_t sms = st().sm_count ? st().sm_count : 148u;
    uint32_t gx = (a.n + 7u) / 8u;
    uint32_t want = (sms * 4u + a.groups_or_segs - 1u) / a.groups_or_segs;
    if (want == 0) want = 1;
    if (gx > want) gx = want;
    if (grid_x) *grid_x = gx;
    if (mt) *mt = 4;
    return launch_lb<1, 4>(a, dim3(gx, a.groups_or_segs), s);
}

// ---------------------------------------------------------------- host-staged API cores
static void fill_info(OmegaGpuFp8Info *info, const OmegaGpuFp8Tensor *t, uint32_t groups, uint32_t gx, uint32_t warps) {
    if (!info) return;
    const uint32_t lb = t->k % 512u == 0 ? 16u : t->k % 256u == 0 ? 8u : 4u;
    info->experts = t->experts; info->n = t->n; info->k = t->k; info->groups = groups;
    info->lane_bytes = lb; info->rows_per_warp = 4; info->warps_per_cta = warps; info->depth = 0;
    info->grid_x = gx; info->grid_y = groups; info->steps = t->k / (32u * lb);
    info->weight_bytes = (uint64_t)groups * t->n * t->k;
    info->scale_bytes = (uint64_t)groups * (t->n / 128u) * (t->k / 128u) * 4u;
    info->kernel_cache_hit = true;
    snprintf(info->target_chip, sizeof info->target_chip, "%s", st().chip);
    info->sm_architecture = 100;
    info->general = lb == 4u || groups > OMEGA_GPU_FP8_MAX_GROUPS;
}

// ids / x on the host, or tab / x on the device (dev form). y always a host buffer here.
static int gemv_core(const OmegaGpuFp8Tensor *t, uint32_t groups, const uint32_t *ids, const float *x32, const uint16_t *x16,
                     uint32_t x_rows, float *y, OmegaGpuFp8Info *info, uint64_t dev_tab, uint64_t dev_x) {
    const uint64_t t0 = now_ns();
    if (info) memset(info, 0, sizeof *info);
    if (!t || !t->w || (!ids && !dev_tab) || (!x32 && !x16 && !dev_x) || !y || groups == 0 || (x_rows != 1 && x_rows != groups)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!dev_tab) for (uint32_t g = 0; g < groups; g++) if (ids[g] >= t->experts) return OMEGA_GPU_FP8_BAD_ARGS;
    if (dev_tab && groups > OMEGA_GPU_FP8_MAX_GROUPS) return OMEGA_GPU_FP8_TOO_LARGE;
    Lock l;
    State &g = st();
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    const uint32_t n = t->n, k = t->k;
    const size_t xbytes = (size_t)x_rows * k * (x16 ? 2 : 4), ybytes = (size_t)groups * n * 4;
    uint64_t *tab = (uint64_t *)stage(0, (size_t)groups * 16);
    void *xd = stage(1, xbytes); float *yd = (float *)stage(2, ybytes);
    if (!tab || !xd || !yd) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = g.stream;
    bool ok = true;
    if (!dev_tab) {
        uint64_t *ht = (uint64_t *)malloc((size_t)groups * 16);
        if (!ht) return OMEGA_GPU_FP8_BAD_ARGS;
        for (uint32_t i = 0; i < groups; i++) (void)omega_gpu_fp8_tensor_entry(t, ids[i], &ht[2 * i], &ht[2 * i + 1]);
        ok = cuda_ok(cudaMemcpyAsync(tab, ht, (size_t)groups * 16, cudaMemcpyHostToDevice, s), "copy group table") && cuda_ok(cudaStreamSynchronize(s), "copy group table");
        free(ht);
    }
    if (ok && !dev_x) ok = cuda_ok(cudaMemcpyAsync(xd, x32 ? (const void *)x32 : (const void *)x16, xbytes, cudaMemcpyHostToDevice, s), "copy x");
    if (!ok) return OMEGA_GPU_FP8_CHIP_FAIL;
    launch_fill_f32(yd, (size_t)groups * n, POISON_F32, s);
    GemvArgs a = {};
    a.tab = dev_tab ? (const uint64_t *)(uintptr_t)dev_tab : tab;
    a.x = dev_x ? (const void *)(uintptr_t)dev_x : xd; a.x_bf16 = (!dev_x && x16) ? 1 : 0; a.x_rows = x_rows;
    a.y = yd; a.n = n; a.k = k; a.groups_or_segs = groups; a.rows = groups;
    a.out_mul = dev_x ? 5.421010862427522e-20f /* 2^-64: the reference router's fold on x' */ : 1.0f;
    a.mutant = g.gemv_mutant;
    uint32_t gx = 0, warps = 0;
    cudaEventRecord(g.ev0, s);
    ok = cuda_ok(launch_gemv_grouped(a, g.cta_budget, &gx, &warps, s), "gemv launch");
    cudaEventRecord(g.ev1, s);
    float *yh = (float *)malloc(ybytes);
    if (!yh) return OMEGA_GPU_FP8_BAD_ARGS;
    ok = ok && cuda_ok(cudaMemcpyAsync(yh, yd, ybytes, cudaMemcpyDeviceToHost, s), "copy y") && cuda_ok(cudaStreamSynchronize(s), "gemv");
    int rc = ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
    if (ok) {
        size_t unchanged = 0;
        for (size_t i = 0; i < (size_t)groups * n; i++) if (yh[i] == POISON_F32) unchanged++;
        if (unchanged) { set_error("output poison survived"); rc = OMEGA_GPU_FP8_CHIP_FAIL; }
        else memcpy(y, yh, ybytes);
    }
    free(yh);
    fill_info(info, t, groups, gx, warps);
    if (info && ok) { float ms = 0; if (cudaEventElapsedTime(&ms, g.ev0, g.ev1) == cudaSuccess) info->elapsed_ns = (uint64_t)(ms * 1e6); info->completion_marker = 1; }
    if (info) info->call_ns = now_ns() - t0;
    return rc;
}

static int gemm_core(const OmegaGpuFp8Tensor *t, uint32_t M, const uint32_t *ids, const uint32_t *trow, const float *x32, const uint16_t *x16,
                     uint32_t x_rows, float *y, OmegaGpuFp8GemmInfo *info) {
    const uint64_t t0 = now_ns();
    if (info) memset(info, 0, sizeof *info);
    if (!t || !t->experts || !ids || !trow || (!x32 && !x16) || !y || M == 0 || x_rows == 0) return OMEGA_GPU_FP8GEMM_BAD_ARGS;
    uint32_t segs = 0;
    for (uint32_t i = 0; i < M; i++) {
        if (ids[i] >= t->experts || trow[i] >= x_rows || (i && ids[i] < ids[i - 1])) return OMEGA_GPU_FP8GEMM_BAD_ARGS;
        if (i == 0 || ids[i] != ids[i - 1]) segs++;
    }
    Lock l;
    State &g = st();
    if (!dev_open()) return OMEGA_GPU_FP8GEMM_CHIP_FAIL;
    const uint32_t n = t->n, k = t->k;
    const size_t xbytes = (size_t)x_rows * k * (x16 ? 2 : 4), ybytes = (size_t)M * n * 4;
    Seg32 *hseg = (Seg32 *)calloc(segs, sizeof(Seg32));
    if (!hseg) return OMEGA_GPU_FP8GEMM_BAD_ARGS;
    uint32_t sg = 0, passes_max = 0; uint64_t streamed = 0;
    for (uint32_t i = 0; i < M;) {
        uint32_t j = i; while (j < M && ids[j] == ids[i]) j++;
        (void)omega_gpu_fp8_tensor_entry(t, ids[i], &hseg[sg].w_va, &hseg[sg].s_va);
        hseg[sg].row0 = i; hseg[sg].cnt = j - i;
        const uint32_t passes = (j - i + 3u) / 4u; if (passes > passes_max) passes_max = passes;
        streamed += (uint64_t)passes * n * k;
        sg++; i = j;
    }
    Seg32 *dseg = (Seg32 *)stage(0, (size_t)segs * sizeof(Seg32));
    void *xd = stage(1, xbytes); float *yd = (float *)stage(2, ybytes); uint32_t *dmap = (uint32_t *)stage(3, (size_t)M * 4);
    if (!dseg || !xd || !yd || !dmap) { free(hseg); return OMEGA_GPU_FP8GEMM_CHIP_FAIL; }
    cudaStream_t s = g.stream;
    bool ok = cuda_ok(cudaMemcpyAsync(dseg, hseg, (size_t)segs * sizeof(Seg32), cudaMemcpyHostToDevice, s), "copy segments") &&
              cuda_ok(cudaMemcpyAsync(dmap, trow, (size_t)M * 4, cudaMemcpyHostToDevice, s), "copy row table") &&
              cuda_ok(cudaMemcpyAsync(xd, x32 ? (const void *)x32 : (const void *)x16, xbytes, cudaMemcpyHostToDevice, s), "copy x") &&
              cuda_ok(cudaStreamSynchronize(s), "stage");
    free(hseg);
    if (!ok) return OMEGA_GPU_FP8GEMM_CHIP_FAIL;
    launch_fill_f32(yd, (size_t)M * n, POISON_F32, s);
    GemvArgs a = {};
    a.seg = dseg; a.x = xd; a.x_bf16 = x16 ? 1 : 0; a.x_rows = x_rows; a.xmap = dmap; a.ymap = nullptr;
    a.y = yd; a.n = n; a.k = k; a.groups_or_segs = segs; a.rows = M; a.out_mul = 1.0f; a.mutant = g.gemm_mutant;
    uint32_t gx = 0, mt = 0;
    cudaEventRecord(g.ev0, s);
    ok = cuda_ok(launch_gemm_rows(a, &gx, &mt, s), "fp8gemm launch");
    cudaEventRecord(g.ev1, s);
    float *yh = (float *)malloc(ybytes);
    if (!yh) return OMEGA_GPU_FP8GEMM_BAD_ARGS;
    ok = ok && cuda_ok(cudaMemcpyAsync(yh, yd, ybytes, cudaMemcpyDeviceToHost, s), "copy y") && cuda_ok(cudaStreamSynchronize(s), "fp8gemm");
    int rc = ok ? OMEGA_GPU_FP8GEMM_OK : OMEGA_GPU_FP8GEMM_CHIP_FAIL;
    if (ok) {
        size_t unchanged = 0;
        for (size_t i = 0; i < (size_t)M * n; i++) if (yh[i] == POISON_F32) unchanged++;
        if (unchanged) { set_error("output poison survived"); rc = OMEGA_GPU_FP8GEMM_CHIP_FAIL; }
        else memcpy(y, yh, ybytes);
    }
    free(yh);
    if (info) {
        const uint32_t lb = k % 512u == 0 ? 16u : k % 256u == 0 ? 8u : 4u;
        info->rows = M; info->segments = segs; info->n = n; info->k = k; info->mt = mt; info->warps_per_cta = 8; info->lane_bytes = lb;
        info->grid_x = gx; info->grid_y = segs; info->passes_max = passes_max;
        info->weight_bytes = (uint64_t)segs * n * k; info->streamed_bytes = streamed; info->kernel_cache_hit = true;
        info->general = lb == 4u;
        if (ok) { float ms = 0; if (cudaEventElapsedTime(&ms, g.ev0, g.ev1) == cudaSuccess) info->elapsed_ns = (uint64_t)(ms * 1e6); info->completion_marker = 1; }
        info->call_ns = now_ns() - t0;
    }
    return rc;
}


// ---------------------------------------------------------------- allocation-free row-table GEMM
// The segment table the grouped GEMM kernel reads normally lives in a cudaMalloc'ed staging buffer. This variant
// keeps it in a fixed device array instead, so the whole call touches no allocator. Layout of the array:
// [0, 32 * NOALLOC_MAX_SEGMENTS) segment records, then one 16-byte header {segments, status, 0, 0}.
constexpr uint32_t NOALLOC_MAX_SEGMENTS = OMEGA_GPU_FP8GEMM_NOALLOC_MAX_SEGMENTS;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_MAX_SEGMENTS * 32 + 256];
static void *g_noalloc_ptr[64];   // per device: the array's DEVICE address (the symbol itself is only a host-side stand-in)

// One CTA. Turns M sorted expert ids into segment records {w_va, s_va, row0, cnt}. status: 0 ok, 1 ids not sorted or
// out of range, 2 more segments than the table holds, 3 an activation row index at or past x_rows (the GEMM kernel would
// read x out of bounds). Everything a previous call left behind is overwritten: the header is rewritten, records
// [segments, max) are zeroed.
__global__ void __launch_bounds__(1024) noalloc_segments_kernel(unsigned char *scratch, uint32_t M, uint32_t experts, const uint32_t *__restrict__ ids,
                                                                const uint32_t *__restrict__ token_rows, uint32_t x_rows,
                                                                uint64_t w_base, uint64_t s_base, uint64_t w_stride, uint64_t s_stride) {
    __shared__ uint32_t warp_sum[32];
    __shared__ uint32_t s_run, s_bad, s_bad_row;
    Seg32 *seg = reinterpret_cast<Seg32 *>(scratch);
    uint32_t *hdr = reinterpret_cast<uint32_t *>(scratch + NOALLOC_MAX_SEGMENTS * 32);
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    if (tid == 0) { s_run = 0; s_bad = 0; s_bad_row = 0; }
    __syncthreads();
    for (uint32_t base = 0; base < M; base += 1024) {
        const uint32_t i = base + tid;
        uint32_t flag = 0, e = 0;
        if (i < M) {
            e = ids[i];
            if (token_rows[i] >= x_rows) s_bad_row = 1;
            const uint32_t prev = i ? ids[i - 1] : 0xffffffffu;
            if (e >= experts || (i && e < prev)) s_bad = 1;
            flag = (i == 0 || e != prev) ? 1u : 0u;
        }
        uint32_t inc = flag;
        for (int o = 1; o < 32; o <<= 1) { const uint32_t u = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= (uint32_t)o) inc += u; }
        if (lane == 31) warp_sum[warp] = inc;
        __syncthreads();
        uint32_t before = s_run;
        for (uint32_t w = 0; w < warp; w++) before += warp_sum[w];
        const uint32_t si = before + inc - flag;
        if (flag && si < NOALLOC_MAX_SEGMENTS && e < experts) {
            Seg32 r; r.w_va = w_base + (uint64_t)e * w_stride; r.s_va = s_base + (uint64_t)e * s_stride; r.row0 = i; r.cnt = 0; r.pad = 0;
            seg[si] = r;
        }
        __syncthreads();
        if (tid == 0) { uint32_t tot = 0; for (int w = 0; w < 32; w++) tot += warp_sum[w]; s_run += tot; }
        __syncthreads();
    }
    const uint32_t S = s_run, kept = min(S, NOALLOC_MAX_SEGMENTS);
    for (uint32_t z = tid; z < kept; z += 1024) seg[z].cnt = (z + 1 < kept ? seg[z + 1].row0 : M) - seg[z].row0;
    for (uint32_t z = kept + tid; z < NOALLOC_MAX_SEGMENTS; z += 1024) { const Seg32 zero = {0, 0, 0, 0, 0}; seg[z] = zero; }
    if (tid == 0) { hdr[0] = kept; hdr[1] = s_bad ? 1u : (s_bad_row ? 3u : (S > NOALLOC_MAX_SEGMENTS ? 2u : 0u)); hdr[2] = 0; hdr[3] = 0; }
}

}  // namespace b200
using namespace b200;

extern "C" {
int omega_gpu_fp8_gemv_f32(const OmegaGpuFp8Tensor *t, uint32_t expert, const float *x, float *y, OmegaGpuFp8Info *info) {
    return gemv_core(t, 1, &expert, x, nullptr, 1, y, info, 0, 0);
}
int omega_gpu_fp8_gemv_bf16(const OmegaGpuFp8Tensor *t, uint32_t expert, const uint16_t *x, float *y, OmegaGpuFp8Info *info) {
    return gemv_core(t, 1, &expert, nullptr, x, 1, y, info, 0, 0);
}
int omega_gpu_fp8_gemv_grouped_f32(const OmegaGpuFp8Tensor *t, uint32_t groups, const uint32_t *ids, const float *x, uint32_t x_rows, float *y, OmegaGpuFp8Info *info) {
    return gemv_core(t, groups, ids, x, nullptr, x_rows, y, info, 0, 0);
}
int omega_gpu_fp8_gemv_grouped_dev(const OmegaGpuFp8Tensor *t, uint32_t groups, uint64_t tab_va, uint64_t x_va, float *y, OmegaGpuFp8Info *info) {
    if (!tab_va || !x_va) return OMEGA_GPU_FP8_BAD_ARGS;
    return gemv_core(t, groups, nullptr, nullptr, nullptr, 1, y, info, tab_va, x_va);
}
int omega_gpu_fp8_gemv_grouped_async(const OmegaGpuFp8Tensor *t, uint32_t groups, uint64_t tab_va, uint64_t x_va, uint32_t x_rows, int x_bf16,
                                     uint64_t y_va, void *stream) {
    if (!t || !tab_va || !x_va || !y_va || groups == 0 || (x_rows != 1 && x_rows != groups)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    GemvArgs a = {};
    a.tab = (const uint64_t *)(uintptr_t)tab_va; a.x = (const void *)(uintptr_t)x_va; a.x_bf16 = x_bf16; a.x_rows = x_rows;
    a.y = (float *)(uintptr_t)y_va; a.n = t->n; a.k = t->k; a.groups_or_segs = groups; a.rows = groups; a.out_mul = 1.0f;
    return cuda_ok(launch_gemv_grouped(a, 0, nullptr, nullptr, (cudaStream_t)stream), "gemv launch") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}
int omega_gpu_fp8gemm_f32(const OmegaGpuFp8Tensor *t, uint32_t M, const uint32_t *ids, const uint32_t *trow, const float *x, uint32_t x_rows, float *y, OmegaGpuFp8GemmInfo *info) {
    return gemm_core(t, M, ids, trow, x, nullptr, x_rows, y, info);
}
int omega_gpu_fp8gemm_bf16(const OmegaGpuFp8Tensor *t, uint32_t M, const uint32_t *ids, const uint32_t *trow, const uint16_t *x, uint32_t x_rows, float *y, OmegaGpuFp8GemmInfo *info) {
    return gemm_core(t, M, ids, trow, nullptr, x, x_rows, y, info);
}
int omega_gpu_fp8gemm_async(const OmegaGpuFp8Tensor *t, uint32_t rows, uint32_t segs, uint64_t seg_va, uint64_t x_va, int x_bf16, uint64_t y_va,
                            uint64_t xmap_va, uint64_t ymap_va, void *stream) {
    if (!t || !seg_va || !x_va || !y_va || rows == 0 || segs == 0 || (!xmap_va != !ymap_va)) return OMEGA_GPU_FP8GEMM_BAD_ARGS;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8GEMM_CHIP_FAIL;
    GemvArgs a = {};
    a.seg = (const Seg32 *)(uintptr_t)seg_va; a.x = (const void *)(uintptr_t)x_va; a.x_bf16 = x_bf16; a.x_rows = rows;
    a.xmap = (const uint32_t *)(uintptr_t)xmap_va; a.ymap = (const uint32_t *)(uintptr_t)ymap_va;
    a.y = (float *)(uintptr_t)y_va; a.n = t->n; a.k = t->k; a.groups_or_segs = segs; a.rows = rows; a.out_mul = 1.0f;
    return cuda_ok(launch_gemm_rows(a, nullptr, nullptr, (cudaStream_t)stream), "fp8gemm launch") ? OMEGA_GPU_FP8GEMM_OK : OMEGA_GPU_FP8GEMM_CHIP_FAIL;
}

// Allocation-free entry (declared in b200moe_fp8gemm.h). Some hosts of this library may not allocate device memory
// at all once they are running: a serving process that has handed every byte to its own arena, a caller inside a
// latency-critical section, a plugin whose embedder forbids cudaMalloc after start-up. The host-staged calls above
// grow staging buffers on demand, so they are closed to such callers; this one is not. Every call blocks once on
// `stream` (it reads the table builder's status word back), so no call may be made while `stream` is being captured:
// such a call is refused with BAD_ARGS and queues nothing.
int omega_gpu_fp8gemm_noalloc(const OmegaGpuFp8Tensor *t, uint32_t M, uint64_t expert_ids_va, uint64_t token_rows_va, uint64_t x_va, int x_bf16,
                              uint32_t x_rows, uint64_t y_va, void *stream) {
    if (!t || !t->w || !M || !expert_ids_va || !token_rows_va || !x_va || !y_va || !x_rows) return OMEGA_GPU_FP8GEMM_BAD_ARGS;
    if (t->experts > NOALLOC_MAX_SEGMENTS) {
        set_error("fp8gemm_noalloc: the tensor has %u experts but the fixed segment table holds %u segments", t->experts, NOALLOC_MAX_SEGMENTS);
        return OMEGA_GPU_FP8GEMM_TOO_LARGE;
    }
    if (M > OMEGA_GPU_FP8GEMM_NOALLOC_MAX_ROWS) {
        set_error("fp8gemm_noalloc: %u rows is past the stated maximum of %u", M, OMEGA_GPU_FP8GEMM_NOALLOC_MAX_ROWS);
        return OMEGA_GPU_FP8GEMM_TOO_LARGE;
    }
    Lock l;
    State &g = st();
    if (!g.opened || g.latched) { set_error("fp8gemm_noalloc: the device is not open (upload a tensor first)"); return OMEGA_GPU_FP8GEMM_CHIP_FAIL; }
    if (t->device < 0 || t->device >= 64) return OMEGA_GPU_FP8GEMM_BAD_ARGS;
    cudaStream_t s = (cudaStream_t)stream;
    // every call waits once on `stream` for its table-building kernel, which a capturing stream cannot do: refuse before
    // anything is queued, so the caller's capture stays valid and nothing latches
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess) { (void)cudaGetLastError(); set_error("fp8gemm_noalloc: not a usable stream"); return OMEGA_GPU_FP8GEMM_BAD_ARGS; }
    if (cap != cudaStreamCaptureStatusNone) { set_error("fp8gemm_noalloc: the stream is being captured; this entry synchronises the stream once per call and cannot be captured"); return OMEGA_GPU_FP8GEMM_BAD_ARGS; }
    if (!cuda_ok(cudaSetDevice(t->device), "cudaSetDevice")) return OMEGA_GPU_FP8GEMM_CHIP_FAIL;
    if (!g_noalloc_ptr[t->device]) {   // set-up, once per device, with that device current
        void *p = nullptr;
        if (!cuda_ok(cudaGetSymbolAddress(&p, g_noalloc_scratch), "cudaGetSymbolAddress(noalloc scratch)") || !p) return OMEGA_GPU_FP8GEMM_CHIP_FAIL;
        g_noalloc_ptr[t->device] = p;
    }
    unsigned char *scratch = (unsigned char *)g_noalloc_ptr[t->device];
    uint64_t w0 = 0, s0 = 0;
    (void)omega_gpu_fp8_tensor_entry(t, 0, &w0, &s0);
    noalloc_segments_kernel<<<1, 1024, 0, s>>>(scratch, M, t->experts, (const uint32_t *)(uintptr_t)expert_ids_va,
                                               (const uint32_t *)(uintptr_t)token_rows_va, x_rows, w0, s0, (uint64_t)t->n * t->k,
                                               (uint64_t)(t->n / 128u) * (t->k / 128u) * 4u);
    if (!cuda_ok(cudaGetLastError(), "noalloc segments launch")) return OMEGA_GPU_FP8GEMM_CHIP_FAIL;
    uint32_t hdr[4] = {0, 0, 0, 0};
    if (!cuda_ok(cudaMemcpyAsync(hdr, scratch + NOALLOC_MAX_SEGMENTS * 32, 16, cudaMemcpyDeviceToHost, s), "copy status") ||
        !cuda_ok(cudaStreamSynchronize(s), "noalloc segments")) return OMEGA_GPU_FP8GEMM_CHIP_FAIL;
    if (hdr[1] == 1) { set_error("fp8gemm_noalloc: expert ids must be non-decreasing and below the expert count"); return OMEGA_GPU_FP8GEMM_BAD_ARGS; }
    if (hdr[1] == 3) { set_error("fp8gemm_noalloc: a token row index is at or past x_rows (%u)", x_rows); return OMEGA_GPU_FP8GEMM_BAD_ARGS; }
    if (hdr[1] == 2) { set_error("fp8gemm_noalloc: more segments than the fixed table holds"); return OMEGA_GPU_FP8GEMM_TOO_LARGE; }
    GemvArgs a = {};
    a.seg = (const Seg32 *)scratch; a.x = (const void *)(uintptr_t)x_va; a.x_bf16 = x_bf16; a.x_rows = x_rows;
    a.xmap = (const uint32_t *)(uintptr_t)token_rows_va; a.ymap = nullptr;
    a.y = (float *)(uintptr_t)y_va; a.n = t->n; a.k = t->k; a.groups_or_segs = hdr[0]; a.rows = M; a.out_mul = 1.0f;
    return cuda_ok(launch_gemm_rows(a, nullptr, nullptr, s), "fp8gemm_noalloc launch") ? OMEGA_GPU_FP8GEMM_OK : OMEGA_GPU_FP8GEMM_CHIP_FAIL;
}
}  // extern "C"
