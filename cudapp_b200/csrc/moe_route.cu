// moe_route.cu: router top-k on given logits and the routing plan (token-to-expert grouping) on the GPU.
//
// Top-k follows the reference router's selection phase (src/omega_blackwell_codegen_router.c:298-401; oracle
// tests/gpu_router_test.c:62-79): k rounds of "largest remaining logit, lowest expert index on ties"; ids in
// selection order; weights = exp(l_i - l_0) / sum over the selected (or over all experts).
//
// The plan is the stable counting sort of the reference's host units (om/moe/moe_plan.om:139-159,
// src/omega_gpu_q36_graph.c:1107-1144) and its one-CTA GROUP kernel (src/omega_blackwell_codegen_dec.c:534-651):
// order = expert, then token, then slot. Here it is histogram -> block exclusive scan -> stable scatter built from
// warp match/ballot primitives, for any row count (the reference kernel ranks <= 128 rows with an O(R^2) loop).
#include "internal.h"
#include "route_common.cuh"

namespace b200 {

// ------------------------------------------------------------------ top-k: one warp per token
// slots = entries per token in ids / wts: topk, or topk + 1 when a shared expert follows the routed picks (its id = experts, weight 1:
// the reference's ninth group, src/omega_gpu_q36_graph.h:7-21; a caller with a shared-expert gate supplies the weight through the router)
__global__ void __launch_bounds__(256) topk_kernel(uint32_t tokens, uint32_t experts, uint32_t topk, int norm, uint32_t slots,
                                                   const uint16_t *__restrict__ logits, uint32_t *__restrict__ ids, float *__restrict__ wts) {
    extern __shared__ float sm[];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= tokens) return;
    float *l = sm + (size_t)warp * experts;
    for (uint32_t e = lane; e < experts; e += 32) l[e] = __uint_as_float((uint32_t)logits[(size_t)t * experts + e] << 16);
    __syncwarp();
    warp_topk(l, experts, topk, norm, ids + (size_t)t * slots, wts + (size_t)t * slots);
    if (slots > topk && lane == 0) { ids[(size_t)t * slots + topk] = experts; wts[(size_t)t * slots + topk] = 1.0f; }
}

cudaError_t launch_topk(uint32_t tokens, uint32_t experts, uint32_t topk, int norm, const uint16_t *logits, uint32_t *ids, float *wts, cudaStream_t s, uint32_t slots) {
    const uint32_t warps = experts <= 512 ? 8u : 4u;
    topk_kernel<<<(tokens + warps - 1) / warps, warps * 32, (size_t)warps * experts * 4, s>>>(tokens, experts, topk, norm, slots ? slots : topk, logits, ids, wts);
    return cudaGetLastError();
}

// ------------------------------------------------------------------ plan: one CTA of 1024 threads
// Exclusive scan of one value per thread over the block (Hillis-Steele in shared memory). buf: 1024 u32.
__device__ __forceinline__ uint32_t block_excl_scan(uint32_t v, uint32_t *buf, uint32_t *total) {
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    uint32_t inc = v;
    for (int o = 1; o < 32; o <<= 1) { const uint32_t u = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= (uint32_t)o) inc += u; }
    if (lane == 31) buf[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = buf[lane], wi = w;
        for (int o = 1; o < 32; o <<= 1) { const uint32_t u = __shfl_up_sync(0xffffffffu, wi, o); if (lane >= (uint32_t)o) wi += u; }
        buf[32 + lane] = wi - w;           // exclusive warp offsets
        if (lane == 31) buf[64] = wi;      // block total
    }
    __syncthreads();
    const uint32_t r = buf[32 + warp] + inc - v;
    if (total) *total = buf[64];
    __syncthreads();
    return r;
}

// Everything of a plan that follows from the per-expert counts (in shared memory): row starts, segment records, row tiles, header,
// the zero pads after the maps. One CTA of 1024 threads; false = refused (only the status word is written).
__device__ __forceinline__ bool plan_tables(uint32_t experts, uint32_t tile_rows, const uint32_t *counts, uint32_t *starts, uint32_t *sbuf,
                                            const OmegaGpuMoePlanOut &o, bool bad) {
    const uint32_t tid = threadIdx.x;
    uint32_t *hdr = reinterpret_cast<uint32_t *>(o.header_va);
    if (bad) {   // refuse: nothing but the status word is written
        if (tid == 0) { hdr[0] = 0; hdr[1] = 0; hdr[2] = 0; hdr[3] = 2; }
        return false;
    }
    // 2. exclusive scans over experts (one expert per thread, passes of 1024): row starts, segment index, tile index
    uint32_t rows_total = 0, segs_total = 0, tiles_total = 0;
    for (uint32_t e0 = 0; e0 < experts; e0 += 1024) {
        const uint32_t e = e0 + tid, c = e < experts ? counts[e] : 0;
        uint32_t tot;
        const uint32_t st_ = rows_total + block_excl_scan(c, sbuf, &tot);
        uint32_t nz;
        const uint32_t si = segs_total + block_excl_scan(c ? 1u : 0u, sbuf, &nz);
        const uint32_t nt = tile_rows ? (c + tile_rows - 1) / tile_rows : 0;
        uint32_t ttot;
        const uint32_t ti = tiles_total + block_excl_scan(nt, sbuf, &ttot);
        rows_total += tot; tiles_total += ttot;
        if (e < experts) {
            starts[e] = st_;
            if (o.counts_va) reinterpret_cast<uint32_t *>(o.counts_va)[e] = c;
            if (o.starts_va) reinterpret_cast<uint32_t *>(o.starts_va)[e] = st_;
            if (c) {
                if (o.seg_a_va) { const uint64_t *d = reinterpret_cast<const uint64_t *>(o.dir_a_va) + 2 * e; Seg32 r = {d[0], d[1], st_, c, 0}; reinterpret_cast<Seg32 *>(o.seg_a_va)[si] = r; }
                if (o.seg_b_va) { const uint64_t *d = reinterpret_cast<const uint64_t *>(o.dir_b_va) + 2 * e; Seg32 r = {d[0], d[1], st_, c, 0}; reinterpret_cast<Seg32 *>(o.seg_b_va)[si] = r; }
                if (o.tiles_va) for (uint32_t j = 0; j < nt; j++) {
                    uint4 tv; tv.x = e; tv.y = st_ + j * tile_rows; tv.z = min(tile_rows, c - j * tile_rows); tv.w = si;
                    reinterpret_cast<uint4 *>(o.tiles_va)[ti + j] = tv;
                }
            }
        }
        segs_total += nz;
    }
    // records past the last non-empty expert: zero count, skipped by the consumers
    for (uint32_t z = segs_total + tid; z < experts; z += 1024) {
        const Seg32 zero = {0, 0, 0, 0, 0};
        if (o.seg_a_va) reinterpret_cast<Seg32 *>(o.seg_a_va)[z] = zero;
        if (o.seg_b_va) reinterpret_cast<Seg32 *>(o.seg_b_va)[z] = zero;
    }
    // word 4 belongs to the kernels that consume the plan (an expired bounded wait is recorded there): it is zero from the owner's allocation and
    // stays set once written, so a later plan does not erase a timeout that nobody has read yet
    if (tid == 0) { hdr[0] = rows_total; hdr[1] = segs_total; hdr[2] = tiles_total; hdr[3] = 0; hdr[5] = hdr[6] = hdr[7] = 0; }
    uint32_t *xmap = reinterpret_cast<uint32_t *>(o.xmap_va), *ymap = reinterpret_cast<uint32_t *>(o.ymap_va);
    if (tid < 8) { xmap[rows_total + tid] = 0; ymap[rows_total + tid] = 0; }
    __syncthreads();
    return true;
}

// dynamic shared: counts[E] | starts[E] | run[E] | scan buf[96] | wcnt u16 [32][E]
// pos (optional): inverse of the Y map, pos[token * slots + slot] = sorted row of that pick
__device__ __forceinline__ void plan_body(uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, uint32_t tile_rows,
                                          const uint32_t *__restrict__ ids, const OmegaGpuMoePlanOut &o, uint32_t *__restrict__ pos) {
    extern __shared__ uint32_t smem[];
    uint32_t *counts = smem, *starts = smem + experts, *run = smem + 2 * experts, *sbuf = smem + 3 * experts;
    uint16_t *wcnt = reinterpret_cast<uint16_t *>(sbuf + 96);
    __shared__ uint32_t s_bad;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, R = tokens * slots;
    for (uint32_t e = tid; e < experts; e += 1024) { counts[e] = 0; run[e] = 0; }
    if (tid == 0) s_bad = 0;
    __syncthreads();
    // 1. histogram (shared-memory integer atomics: the result does not depend on their order)
    for (uint32_t i = tid; i < R; i += 1024) {
        const uint32_t e = ids[i];
        if (e == 0xffffffffu) continue;
        if (e >= experts) { s_bad = 1; continue; }
        atomicAdd(&counts[e], 1u);
    }
    __syncthreads();
    if (!plan_tables(experts, tile_rows, counts, starts, sbuf, o, s_bad != 0)) return;
    uint32_t *xmap = reinterpret_cast<uint32_t *>(o.xmap_va), *ymap = reinterpret_cast<uint32_t *>(o.ymap_va);
    // 3. stable scatter, 1024 rows per chunk in row order: rank = rows of the same expert before this one.
    //    run[e] = rows of expert e in earlier chunks; counts[] is reused for this chunk's per-expert total.
    for (uint32_t base = 0; base < R; base += 1024) {
        for (uint32_t j = tid; j < 32u * experts; j += 1024) wcnt[j] = 0;
        __syncthreads();
        const uint32_t i = base + tid;
        const uint32_t e = i < R ? ids[i] : 0xffffffffu;
        const uint32_t peers = __match_any_sync(0xffffffffu, e);
        const uint32_t rank_w = __popc(peers & ((1u << lane) - 1u));
        if (e != 0xffffffffu && rank_w == 0) wcnt[warp * experts + e] = (uint16_t)__popc(peers);
        __syncthreads();
        for (uint32_t ee = tid; ee < experts; ee += 1024) {   // per expert: exclusive scan over the 32 warps
            uint32_t acc = 0;
            for (uint32_t w = 0; w < 32; w++) { const uint32_t c = wcnt[w * experts + ee]; wcnt[w * experts + ee] = (uint16_t)acc; acc += c; }
            counts[ee] = acc;
        }
        __syncthreads();
        if (e != 0xffffffffu) {
            const uint32_t p = starts[e] + run[e] + wcnt[warp * experts + e] + rank_w;
            const uint32_t t = i / slots, s = i - t * slots;
            xmap[p] = t; ymap[p] = t * ystride + s;
            if (pos) pos[i] = p;
        }
        __syncthreads();
        for (uint32_t ee = tid; ee < experts; ee += 1024) run[ee] += counts[ee];
        __syncthreads();
    }
}

__global__ void __launch_bounds__(1024) plan_kernel(uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, uint32_t tile_rows,
                                                    const uint32_t *__restrict__ ids, const OmegaGpuMoePlanOut o) {
    plan_body(tokens, slots, experts, ystride, tile_rows, ids, o, nullptr);
}
// one CTA per layer: layer l's picks at ids + l * tokens * slots, its outputs at the PlanBatch strides
__global__ void __launch_bounds__(1024) plan_batch_kernel(uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, uint32_t tile_rows,
                                                          const uint32_t *__restrict__ ids, const PlanBatch b) {
    const uint32_t l = blockIdx.x;
    OmegaGpuMoePlanOut o = {};
    o.counts_va = (uint64_t)(uintptr_t)(b.counts + (size_t)l * experts); o.starts_va = (uint64_t)(uintptr_t)(b.starts + (size_t)l * experts);
    o.xmap_va = (uint64_t)(uintptr_t)(b.xmap + (size_t)l * b.map_stride); o.ymap_va = (uint64_t)(uintptr_t)(b.ymap + (size_t)l * b.map_stride);
    o.tiles_va = (uint64_t)(uintptr_t)(b.tiles + (size_t)l * b.tile_stride); o.header_va = (uint64_t)(uintptr_t)(b.header + (size_t)l * 8);
    plan_body(tokens, slots, experts, ystride, tile_rows, ids + (size_t)l * tokens * slots, o, b.pos + (size_t)l * b.map_stride);
}
cudaError_t launch_plan_batch(uint32_t layers, uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, uint32_t tile_rows, const uint32_t *ids,
                              const PlanBatch &b, cudaStream_t s) {
    const size_t smem = (size_t)experts * 12 + 96 * 4 + (size_t)32 * experts * 2;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(plan_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    plan_batch_kernel<<<layers, 1024, smem, s>>>(tokens, slots, experts, ystride, tile_rows, ids, b);
    return cudaGetLastError();
}

// ------------------------------------------------------------------ plan of many picks: three launches, one CTA per 1024 picks in the first and the last
// The same stable order as plan_kernel (sorted row = rows of lower experts + earlier picks of the same expert), split so that the
// per-chunk work runs on as many SMs as there are chunks: (1) per-chunk histograms, (2) one CTA turns them into per-chunk
// offsets and builds the tables, (3) every chunk scatters its picks. scratch: u32 [chunks][experts] + 1 flag word.
__global__ void __launch_bounds__(1024) plan_hist_kernel(uint32_t R, uint32_t experts, const uint32_t *__restrict__ ids, uint32_t *__restrict__ scratch, uint32_t chunks) {
    extern __shared__ uint32_t smem[];
    const uint32_t tid = threadIdx.x;
    for (uint32_t e = tid; e < experts; e += 1024) smem[e] = 0;
    __syncthreads();
    const uint32_t i = blockIdx.x * 1024u + tid;
    if (i < R) {
        const uint32_t e = ids[i];
        if (e != 0xffffffffu) { if (e >= experts) atomicOr(scratch + (size_t)chunks * experts, 1u); else atomicAdd(&smem[e], 1u); }
    }
    __syncthreads();
    for (uint32_t e = tid; e < experts; e += 1024) scratch[(size_t)blockIdx.x * experts + e] = smem[e];
}
// dynamic shared: counts[E] | starts[E] | scan buf[96]
__global__ void __launch_bounds__(1024) plan_scan_kernel(uint32_t experts, uint32_t tile_rows, uint32_t *__restrict__ scratch, uint32_t chunks, const OmegaGpuMoePlanOut o) {
    extern __shared__ uint32_t smem[];
    uint32_t *counts = smem, *starts = smem + experts, *sbuf = smem + 2 * experts;
    const uint32_t tid = threadIdx.x;
    const bool bad = scratch[(size_t)chunks * experts] != 0;
    __syncthreads();
    if (tid == 0) scratch[(size_t)chunks * experts] = 0;   // the flag is clear again for the next plan
    for (uint32_t e = tid; e < experts; e += 1024) {        // per expert: counts of earlier chunks
        uint32_t acc = 0;
        for (uint32_t c = 0; c < chunks; c++) { const uint32_t v = scratch[(size_t)c * experts + e]; scratch[(size_t)c * experts + e] = acc; acc += v; }
        counts[e] = acc;
    }
    __syncthreads();
    (void)plan_tables(experts, tile_rows, counts, starts, sbuf, o, bad);
}
// dynamic shared: wcnt u16 [32][E]
__global__ void __launch_bounds__(1024) plan_scatter_kernel(uint32_t R, uint32_t slots, uint32_t experts, uint32_t ystride, const uint32_t *__restrict__ ids,
                                                            const uint32_t *__restrict__ scratch, const OmegaGpuMoePlanOut o, uint32_t *__restrict__ pos) {
    extern __shared__ uint32_t smem[];
    uint16_t *wcnt = reinterpret_cast<uint16_t *>(smem);
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    if (reinterpret_cast<const uint32_t *>(o.header_va)[3]) return;   // refused: nothing is written
    const uint32_t *starts = reinterpret_cast<const uint32_t *>(o.starts_va);
    uint32_t *xmap = reinterpret_cast<uint32_t *>(o.xmap_va), *ymap = reinterpret_cast<uint32_t *>(o.ymap_va);
    for (uint32_t j = tid; j < 32u * experts; j += 1024) wcnt[j] = 0;
    __syncthreads();
    const uint32_t i = blockIdx.x * 1024u + tid;
    const uint32_t e = i < R ? ids[i] : 0xffffffffu;
    const uint32_t peers = __match_any_sync(0xffffffffu, e);
    const uint32_t rank_w = __popc(peers & ((1u << lane) - 1u));
    if (e != 0xffffffffu && rank_w == 0) wcnt[warp * experts + e] = (uint16_t)__popc(peers);
    __syncthreads();
    for (uint32_t ee = tid; ee < experts; ee += 1024) {   // per expert: exclusive scan over the 32 warps
        uint32_t acc = 0;
        for (uint32_t w = 0; w < 32; w++) { const uint32_t c = wcnt[w * experts + ee]; wcnt[w * experts + ee] = (uint16_t)acc; acc += c; }
    }
    __syncthreads();
    if (e != 0xffffffffu) {
        const uint32_t p = starts[e] + scratch[(size_t)blockIdx.x * experts + e] + wcnt[warp * experts + e] + rank_w;
        const uint32_t t = i / slots, sl = i - t * slots;
        xmap[p] = t; ymap[p] = t * ystride + sl;
        if (pos) pos[i] = p;
    }
}
size_t plan_scratch_words(uint32_t picks, uint32_t experts) { return (size_t)((picks + 1023u) / 1024u) * experts + 1; }
static bool plan_split(uint32_t picks, uint32_t experts, const uint32_t *scratch, size_t scratch_words, const OmegaGpuMoePlanOut &o) {
    return scratch && picks >= 4096u && o.starts_va && plan_scratch_words(picks, experts) <= scratch_words && (size_t)32 * experts * 2 <= 48 * 1024;
}
uint32_t plan_launch_count(uint32_t picks, uint32_t experts, const uint32_t *scratch, size_t scratch_words, const OmegaGpuMoePlanOut &o) {
    return plan_split(picks, experts, scratch, scratch_words, o) ? 3u : 1u;
}

cudaError_t launch_plan(uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, uint32_t tile_rows, const uint32_t *ids,
                        const OmegaGpuMoePlanOut &o, cudaStream_t s, uint32_t *scratch, size_t scratch_words) {
    const uint32_t R = tokens * slots, chunks = (R + 1023u) / 1024u;
    if (plan_split(R, experts, scratch, scratch_words, o)) {
        plan_hist_kernel<<<chunks, 1024, (size_t)experts * 4, s>>>(R, experts, ids, scratch, chunks);
        plan_scan_kernel<<<1, 1024, (size_t)experts * 8 + 96 * 4, s>>>(experts, tile_rows, scratch, chunks, o);
        plan_scatter_kernel<<<chunks, 1024, (size_t)32 * experts * 2, s>>>(R, slots, experts, ystride, ids, scratch, o, nullptr);
        return cudaGetLastError();
    }

    const size_t smem = (size_t)experts * 12 + 96 * 4 + (size_t)32 * experts * 2;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    plan_kernel<<<1, 1024, smem, s>>>(tokens, slots, experts, ystride, tile_rows, ids, o);
    return cudaGetLastError();
}

}  // namespace b200
using namespace b200;

// ------------------------------------------------------------------ host-buffer forms
extern "C" {

int omega_gpu_moe_topk_async(uint32_t tokens, uint32_t experts, uint32_t topk, int norm_topk, uint64_t logits_va, uint64_t ids_va, uint64_t wts_va, void *stream) {
    if (!tokens || !experts || experts > 1024 || !topk || topk > 32 || topk > experts || !logits_va || !ids_va || !wts_va) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    return cuda_ok(launch_topk(tokens, experts, topk, norm_topk, (const uint16_t *)(uintptr_t)logits_va, (uint32_t *)(uintptr_t)ids_va, (float *)(uintptr_t)wts_va,
                               (cudaStream_t)stream), "topk launch") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_topk_bf16(uint32_t tokens, uint32_t experts, uint32_t topk, int norm_topk, const uint16_t *logits, uint32_t *ids, float *wts) {
    if (!tokens || !experts || experts > 1024 || !topk || topk > 32 || topk > experts || !logits || !ids || !wts) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    const size_t lb = (size_t)tokens * experts * 2, ib = (size_t)tokens * topk * 4;
    uint16_t *dl = (uint16_t *)stage(0, lb); uint32_t *di = (uint32_t *)stage(1, ib); float *dw = (float *)stage(2, ib);
    if (!dl || !di || !dw) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = st().stream;
    bool ok = cuda_ok(cudaMemcpyAsync(dl, logits, lb, cudaMemcpyHostToDevice, s), "copy logits") &&
              cuda_ok(launch_topk(tokens, experts, topk, norm_topk, dl, di, dw, s), "topk launch") &&
              cuda_ok(cudaMemcpyAsync(ids, di, ib, cudaMemcpyDeviceToHost, s), "copy ids") &&
              cuda_ok(cudaMemcpyAsync(wts, dw, ib, cudaMemcpyDeviceToHost, s), "copy weights") && cuda_ok(cudaStreamSynchronize(s), "topk");
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_plan_async(uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, uint32_t tile_rows, uint64_t ids_va,
                             const OmegaGpuMoePlanOut *out, void *stream) {
    if (!experts || experts > 1024 || !out || !out->xmap_va || !out->ymap_va || !out->header_va || (tokens && slots && !ids_va)) return OMEGA_GPU_FP8_BAD_ARGS;
    if ((out->seg_a_va && !out->dir_a_va) || (out->seg_b_va && !out->dir_b_va)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    return cuda_ok(launch_plan(tokens, slots, experts, ystride, tile_rows, (const uint32_t *)(uintptr_t)ids_va, *out, (cudaStream_t)stream), "plan launch")
               ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

// staged plan: device buffers in staging slots 4..7; returns host copies. rows/segs through hdr.
static int plan_staged(uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, const uint32_t *ids, uint32_t *counts, uint32_t *starts,
                       uint32_t *xmap, uint32_t *ymap, uint32_t hdr[8]) {
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    const size_t R = (size_t)tokens * slots;
    uint32_t *dids = (uint32_t *)stage(4, R * 4), *dmaps = (uint32_t *)stage(5, (R + 8) * 8), *dcs = (uint32_t *)stage(6, (size_t)experts * 8 + 32);
    if (!dids || !dmaps || !dcs) return OMEGA_GPU_FP8_CHIP_FAIL;
    OmegaGpuMoePlanOut o = {};
    o.counts_va = (uint64_t)(uintptr_t)dcs; o.starts_va = (uint64_t)(uintptr_t)(dcs + experts); o.header_va = (uint64_t)(uintptr_t)(dcs + 2 * experts);
    o.xmap_va = (uint64_t)(uintptr_t)dmaps; o.ymap_va = (uint64_t)(uintptr_t)(dmaps + R + 8);
    cudaStream_t s = st().stream;
    bool ok = (R == 0 || cuda_ok(cudaMemcpyAsync(dids, ids, R * 4, cudaMemcpyHostToDevice, s), "copy ids")) &&
              cuda_ok(launch_plan(tokens, slots, experts, ystride, 0, dids, o, s), "plan launch") &&
              cuda_ok(cudaMemcpyAsync(hdr, dcs + 2 * experts, 32, cudaMemcpyDeviceToHost, s), "copy header") && cuda_ok(cudaStreamSynchronize(s), "plan");
    if (!ok) return OMEGA_GPU_FP8_CHIP_FAIL;
    if (hdr[3] != 0) return OMEGA_GPU_FP8_OK;   // refused by the kernel: nothing else was written
    ok = cuda_ok(cudaMemcpy(counts, dcs, (size_t)experts * 4, cudaMemcpyDeviceToHost), "copy counts") &&
         cuda_ok(cudaMemcpy(starts, dcs + experts, (size_t)experts * 4, cudaMemcpyDeviceToHost), "copy starts") &&
         cuda_ok(cudaMemcpy(xmap, dmaps, ((size_t)hdr[0] + 8) * 4, cudaMemcpyDeviceToHost), "copy xmap") &&
         cuda_ok(cudaMemcpy(ymap, dmaps + R + 8, ((size_t)hdr[0] + 8) * 4, cudaMemcpyDeviceToHost), "copy ymap");
    return ok ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

int omega_gpu_moe_plan_u32(uint32_t tokens, uint32_t slots, uint32_t experts, uint32_t ystride, const uint32_t *ids, uint32_t *counts, uint32_t *starts,
                           uint32_t *xmap, uint32_t *ymap, uint32_t *seg3, uint32_t *rows, uint32_t *segments) {
    if (!experts || experts > 1024 || !counts || !starts || !xmap || !ymap || !rows || !segments || (tokens && slots && !ids)) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    uint32_t hdr[8];
    const int rc = plan_staged(tokens, slots, experts, ystride, ids, counts, starts, xmap, ymap, hdr);
    if (rc != OMEGA_GPU_FP8_OK) return rc;
    if (hdr[3] != 0) { set_error("plan: expert id out of range"); return OMEGA_GPU_FP8_BAD_ARGS; }
    *rows = hdr[0]; *segments = hdr[1];
    if (seg3) { uint32_t z = 0; for (uint32_t e = 0; e < experts; e++) if (counts[e]) { seg3[z * 3] = e; seg3[z * 3 + 1] = starts[e]; seg3[z * 3 + 2] = counts[e]; z++; } }
    return OMEGA_GPU_FP8_OK;
}

// ------------------------------------------------------------------ ABI1 plan units (src/cudapp_native.h:33-38)
static bool view_ok(const void *p, uint64_t n, uint64_t want, uint64_t elem) { return p && n == want && ((uintptr_t)p % elem) == 0; }
static bool overlap(const void *a, uint64_t an, const void *b, uint64_t bn) { const uintptr_t x = (uintptr_t)a, y = (uintptr_t)b; return x < y + bn && y < x + an; }
struct View { const void *p; uint64_t bytes; };
static bool views_ok(uint64_t *result, const View *v, int nv) {
    if (!result || ((uintptr_t)result % 8)) return false;
    for (int i = 0; i < nv; i++) {
        if (overlap(result, 8, v[i].p, v[i].bytes)) return false;
        for (int j = 0; j < i; j++) if (overlap(v[i].p, v[i].bytes, v[j].p, v[j].bytes)) return false;
    }
    return true;
}
static thread_local int unit_busy = 0;
struct Busy { bool ok; Busy() : ok(!unit_busy) { if (ok) unit_busy = 1; } ~Busy() { if (ok) unit_busy = 0; } };

uint32_t omega_moe_plan(uint64_t *result, const void *cfg_, uint64_t cfg_n, const void *ids_, uint64_t ids_n, void *work_, uint64_t work_n,
                        void *seg_, uint64_t seg_n, void *maps_, uint64_t maps_n, void *meta_, uint64_t meta_n) {
    if (!view_ok(cfg_, cfg_n, 8, 8) || !view_ok(ids_, ids_n, 1024, 8) || !view_ok(work_, work_n, 10368, 8) || !view_ok(seg_, seg_n, 1028, 8) ||
        !view_ok(maps_, maps_n, 2320, 8) || !view_ok(meta_, meta_n, 8, 8)) return OMEGA_BAD_ARG;
    const View v[6] = {{cfg_, 64}, {ids_, 8192}, {work_, 82944}, {seg_, 8224}, {maps_, 18560}, {meta_, 64}};
    if (!views_ok(result, v, 6)) return OMEGA_BAD_ARG;
    Busy b; if (!b.ok) return OMEGA_REENTRY;
    const uint64_t *c = (const uint64_t *)cfg_, *ids = (const uint64_t *)ids_;
    uint64_t *work = (uint64_t *)work_, *seg = (uint64_t *)seg_, *maps = (uint64_t *)maps_, *meta = (uint64_t *)meta_;
    const uint64_t T = c[1], S = c[2], E = c[3];
    if (c[0] != 1 || T > 128 || S > 8 || E == 0 || E > 256 || c[4] != E || c[5] > 1152 || c[6] > 257 || c[7] > 1160) { *result = 1; return OMEGA_OK; }
    // The grouping runs on the GPU over u32 picks, the shared expert's rows included: every token gets one more pick, slot S, for expert E
    // (the unit's shared id), so the device plan itself puts them last (E is the largest id) in token order with destination t * (S + 1) + S
    // (om/moe/moe_plan.om:112-117). An id that does not fit 32 bits, or a routed pick at or past E that is not the "absent" mark, is invalid.
    const uint64_t S1 = S + 1;
    uint32_t id32[128 * 9], counts[257], starts[257], xmap[128 * 9 + 8], ymap[128 * 9 + 8], hdr[8];
    for (uint64_t t = 0; t < T; t++) {
        for (uint64_t sl = 0; sl < S; sl++) {
            const uint64_t v = ids[t * S + sl];
            if (v > 0xffffffffull || (v >= E && v != 0xffffffffull)) { *result = 2; return OMEGA_OK; }
            id32[t * S1 + sl] = (uint32_t)v;
        }
        id32[t * S1 + S] = (uint32_t)E;
    }
    {
        Lock l;
        if (plan_staged((uint32_t)T, (uint32_t)S1, (uint32_t)E + 1u, (uint32_t)S1, id32, counts, starts, xmap, ymap, hdr) != OMEGA_GPU_FP8_OK) return 14; /* trap: no device */
    }
    if (hdr[3] != 0) { *result = 2; return OMEGA_OK; }
    const uint64_t nw = hdr[0], routed = nw - T, ns = hdr[1];
    if (nw > c[5] || ns > c[6] || nw + 8 > c[7]) { *result = 3; return OMEGA_OK; }
    uint64_t z = 0;
    for (uint64_t e = 0; e <= E; e++) if (counts[e]) {
        seg[z * 4] = e; seg[z * 4 + 1] = starts[e]; seg[z * 4 + 2] = counts[e]; seg[z * 4 + 3] = e == E ? 1 : 0; z++;
        for (uint64_t p = starts[e]; p < (uint64_t)starts[e] + counts[e]; p++) {
            uint64_t *r = work + p * 9; const uint64_t t = xmap[p], sl = ymap[p] - t * S1;
            r[0] = e; r[1] = t; r[2] = t; r[3] = sl; r[4] = sl; r[5] = starts[e]; r[6] = counts[e]; r[7] = ymap[p]; r[8] = sl;
        }
    }
    for (uint64_t p = 0; p < nw; p++) { maps[p] = work[p * 9 + 1]; maps[1160 + p] = work[p * 9 + 7]; }
    for (uint64_t p = 0; p < 8; p++) { maps[nw + p] = 0; maps[1160 + nw + p] = 0; }
    meta[0] = nw; meta[1] = ns; meta[2] = routed; meta[3] = T; meta[4] = 1; meta[5] = meta[6] = meta[7] = 0;
    *result = 0;
    return OMEGA_OK;
}

uint32_t omega_moe_ids32(uint64_t *result, const void *src_, uint64_t src_n, uint64_t n, void *ids_, uint64_t ids_n) {
    if (!view_ok(src_, src_n, 4096, 1) || !view_ok(ids_, ids_n, 1024, 8)) return OMEGA_BAD_ARG;
    const View v[2] = {{src_, 4096}, {ids_, 8192}};
    if (!views_ok(result, v, 2)) return OMEGA_BAD_ARG;
    Busy b; if (!b.ok) return OMEGA_REENTRY;
    if (n > 1024) { *result = 1; return OMEGA_OK; }
    const uint8_t *s = (const uint8_t *)src_; uint64_t *ids = (uint64_t *)ids_;
    for (uint64_t i = 0; i < n; i++) ids[i] = (uint64_t)s[4 * i] | (uint64_t)s[4 * i + 1] << 8 | (uint64_t)s[4 * i + 2] << 16 | (uint64_t)s[4 * i + 3] << 24;
    *result = 0; return OMEGA_OK;
}

uint32_t omega_moe_maps32(uint64_t *result, const void *meta_, uint64_t meta_n, const void *maps_, uint64_t maps_n, void *out_, uint64_t out_n) {
    if (!view_ok(meta_, meta_n, 8, 8) || !view_ok(maps_, maps_n, 2320, 8) || !view_ok(out_, out_n, 9280, 1)) return OMEGA_BAD_ARG;
    const View v[3] = {{meta_, 64}, {maps_, 18560}, {out_, 9280}};
    if (!views_ok(result, v, 3)) return OMEGA_BAD_ARG;
    Busy b; if (!b.ok) return OMEGA_REENTRY;
    const uint64_t *m = (const uint64_t *)meta_, *mp = (const uint64_t *)maps_; uint8_t *o = (uint8_t *)out_;
    if (m[0] > 1152) { *result = 1; return OMEGA_OK; }
    const uint64_t n = m[0] + 8;
    for (int zz = 0; zz < 2; zz++) for (uint64_t i = 0; i < n; i++) if (mp[zz * 1160 + i] > 0xffffffffull) { *result = 2; return OMEGA_OK; }
    for (int zz = 0; zz < 2; zz++) for (uint64_t i = 0; i < n; i++) { const uint64_t p = zz * 1160 + i; for (int q = 0; q < 4; q++) o[p * 4 + q] = (uint8_t)(mp[p] >> (8 * q)); }
    *result = 0; return OMEGA_OK;
}

uint32_t omega_moe_segs32(uint64_t *result, const void *seg_, uint64_t seg_n, const void *meta_, uint64_t meta_n, const void *dir_, uint64_t dir_n, void *out_, uint64_t out_n) {
    if (!view_ok(seg_, seg_n, 1028, 8) || !view_ok(meta_, meta_n, 8, 8) || !view_ok(dir_, dir_n, 514, 8) || !view_ok(out_, out_n, 8224, 1)) return OMEGA_BAD_ARG;
    const View v[4] = {{seg_, 8224}, {meta_, 64}, {dir_, 4112}, {out_, 8224}};
    if (!views_ok(result, v, 4)) return OMEGA_BAD_ARG;
    Busy b; if (!b.ok) return OMEGA_REENTRY;
    const uint64_t *sg = (const uint64_t *)seg_, *m = (const uint64_t *)meta_, *dir = (const uint64_t *)dir_; uint8_t *o = (uint8_t *)out_;
    if (m[1] > 257 || m[0] > 1152) { *result = 1; return OMEGA_OK; }
    uint64_t pos = 0;
    for (uint64_t z = 0; z < m[1]; z++) {
        const uint64_t e = sg[z * 4], cnt = sg[z * 4 + 2];
        if (e > 256 || sg[z * 4 + 1] != pos || cnt == 0 || cnt > m[0]) { *result = 2; return OMEGA_OK; }
        pos += cnt;
        if (pos > m[0]) { *result = 2; return OMEGA_OK; }
        for (int q = 0; q < 2; q++) if (dir[e * 2 + q] == 0 || dir[e * 2 + q] % 8) { *result = 3; return OMEGA_OK; }
    }
    if (pos != m[0]) { *result = 2; return OMEGA_OK; }
    for (uint64_t z = 0; z < m[1]; z++) {
        const uint64_t e = sg[z * 4];
        const uint64_t rec[4] = {dir[e * 2], dir[e * 2 + 1], sg[z * 4 + 1] | sg[z * 4 + 2] << 32, 0};
        for (int q = 0; q < 4; q++) for (int bb = 0; bb < 8; bb++) o[z * 32 + q * 8 + bb] = (uint8_t)(rec[q] >> (8 * bb));
    }
    *result = 0; return OMEGA_OK;
}

uint32_t omega_moe_windows(uint64_t *result, const void *cfg_, uint64_t cfg_n, void *win_, uint64_t win_n, void *meta_, uint64_t meta_n) {
    if (!view_ok(cfg_, cfg_n, 8, 8) || !view_ok(win_, win_n, 1024, 8) || !view_ok(meta_, meta_n, 4, 8)) return OMEGA_BAD_ARG;
    const View v[3] = {{cfg_, 64}, {win_, 8192}, {meta_, 32}};
    if (!views_ok(result, v, 3)) return OMEGA_BAD_ARG;
    Busy b; if (!b.ok) return OMEGA_REENTRY;
    const uint64_t *c = (const uint64_t *)cfg_; uint64_t *o = (uint64_t *)win_, *m = (uint64_t *)meta_;
    if (c[0] != 1 || c[1] > 128 || c[2] != 2048 || c[3] != 512 || c[4] != 9 || c[5] == 0 || c[5] > 0xffffffffull || c[5] % 16 || c[6] > 128 || c[7] != 0) { *result = 1; return OMEGA_OK; }
    const uint64_t take = 128 / 9, nwin = (c[1] + take - 1) / take;
    if (nwin > c[6]) { *result = 2; return OMEGA_OK; }
    uint64_t first = 0;
    for (uint64_t z = 0; z < nwin; z++) {
        const uint64_t count = c[1] - first > take ? take : c[1] - first; uint64_t *w = o + z * 8;
        w[0] = first; w[1] = count; w[2] = count * c[4]; w[3] = first * c[2] * 4; w[4] = first * c[4] * c[3] * 8; w[5] = first * c[4] * c[3] * 4;
        w[6] = first * c[4] * c[2] * 4; w[7] = first * c[5];
        first += count;
    }
    m[0] = nwin; m[1] = c[1]; m[2] = c[1] * 9; m[3] = 1;
    *result = 0; return OMEGA_OK;
}

static uint64_t group_extent(const uint64_t *r, uint64_t i) {
    if (i < 3) return (r[8] - 1) * r[7] + (i == 0 ? 32u : 144u);
    if (i < 5) return r[8] * 9 * 32;
    return (r[8] * 9 + 8) * 4;
}
uint32_t omega_moe_group(uint64_t *result, const void *req_, uint64_t req_n, void *words_, uint64_t words_n) {
    if (!view_ok(req_, req_n, 16, 8) || !view_ok(words_, words_n, 64, 1)) return OMEGA_BAD_ARG;
    const View v[2] = {{req_, 128}, {words_, 64}};
    if (!views_ok(result, v, 2)) return OMEGA_BAD_ARG;
    Busy b; if (!b.ok) return OMEGA_REENTRY;
    const uint64_t *r = (const uint64_t *)req_; uint8_t *o = (uint8_t *)words_;
    uint64_t rc = 0;
    const uint64_t rows = r[8] * 9;
    if (r[8] > 128 || r[8] == 0 || rows > 128 || r[11] != 9 || r[15] != 256) rc = 1;
    else if (r[9] < rows || r[10] < rows + 8 || r[7] == 0 || r[7] > 0xffffffffull || r[7] < 144) rc = 2;
    else if (r[7] % 16) rc = 3;
    if (!rc) for (int i = 0; i < 7; i++) if (r[i] == 0 || r[i] % 8) { rc = 3; break; }
    if (!rc && (r[12] != r[13] || r[14] != 1)) rc = 4;
    if (!rc) for (uint64_t i = 0; i < 7; i++) if (r[i] > UINT64_MAX - group_extent(r, i)) { rc = 5; break; }
    if (!rc) for (uint64_t j = 0; j < 4 && !rc; j++) for (uint64_t i = 0; i < j + 3; i++) {
        const uint64_t a = r[i], al = group_extent(r, i), bb = r[j + 3], bl = group_extent(r, j + 3);
        if (a < bb + bl && bb < a + al) { rc = 5; break; }
    }
    if (rc) { *result = rc; return OMEGA_OK; }
    uint32_t w[16];
    for (int i = 0; i < 7; i++) { w[2 * i] = (uint32_t)r[i]; w[2 * i + 1] = (uint32_t)(r[i] >> 32); }
    w[14] = (uint32_t)r[7]; w[15] = (uint32_t)r[8];
    for (int i = 0; i < 16; i++) for (int q = 0; q < 4; q++) o[i * 4 + q] = (uint8_t)(w[i] >> (8 * q));
    *result = 0; return OMEGA_OK;
}

}  // extern "C"
