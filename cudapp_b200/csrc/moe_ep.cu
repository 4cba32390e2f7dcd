// moe_ep.cu: expert-parallel execution of the MoE layer over the GPUs of one node. The reference runs one device
// only (docs/runtime/API.md:125 of the reference), so there is no reference behaviour to mirror beyond "the same
// numbers as one GPU": each routed row goes through exactly the kernels of the single-GPU layer and the combine
// keeps the reference's slot order (src/omega_blackwell_codegen_dec.c:226-255), so outputs equal the 1-GPU run.
//
// Rank r of G owns experts [r*E/G, (r+1)*E/G) and a slice of the tokens. Per layer:
//   dispatch  top-k on the local tokens; picks grouped by destination rank (the routing-plan kernel with G "experts");
//             each pick's activation row + {local expert id, token*topk+slot} is written into region (r -> d);
//   experts   the receiver plans over every region's rows and runs gate|up, SiLU gate, down on its local experts;
//   return    each result row goes back to the same region position on the owner;
//   combine   the owner sums its token's slots in slot order.
// Regions have fixed capacity (tokens_local*topk rows, the worst case) so no count ever has to reach the host.
// Two transports share these kernels: (1) NCCL all-to-all of whole regions, issued by the caller between the
// three calls; (2) direct peer stores over NVLink into the destination's receive memory (only the rows that
// exist move) with a release/acquire flag per (source, destination); waits on those flags are bounded.
// No TMA load reads peer memory anywhere: remote rows are written by plain stores and read locally.
#include <stdlib.h>
#include "internal.h"

struct OmegaGpuMoeEp {
    uint32_t world, rank, topk, experts, experts_local, hidden, tokens_local_max, cap, region_rows;
    size_t row_bytes;
    uint32_t *ids, *dest, *cnt, *starts, *xmap, *ymap, *hdr, *slot_pos, *rids, *err;
    float *wts;
    uint8_t *comm;                       // one allocation: recv | back | flags (what peers write into)
    uint8_t *send, *recv; float *dn, *back; uint32_t *flag_disp, *flag_ret;
    uint64_t *peer_tab;                  // device: [4][G] addresses of the peers' recv, back, flag_disp, flag_ret
    int p2p; uint32_t epoch;
    size_t comm_bytes, off_back, off_flags;
    void *opened[64]; int n_opened;
};

namespace b200 {

// also advances the device-resident epoch (one per dispatch), so a replayed CUDA graph still gets a fresh value
__global__ void ep_dest_kernel(uint32_t n, uint32_t experts_local, const uint32_t *__restrict__ ids, uint32_t *__restrict__ dest, uint32_t *epoch) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0) *epoch += 1u;
    if (i < n) dest[i] = ids[i] / experts_local;
}

// one warp per sorted pick: copy the token's bf16 row and its meta into region (rank -> d)
__global__ void __launch_bounds__(256) ep_pack_kernel(uint32_t world, uint32_t rank, uint32_t topk, uint32_t experts_local, uint32_t hidden, uint32_t region_rows,
                                                      size_t row_bytes, int p2p, const uint32_t *__restrict__ epoch_dev, const uint32_t *__restrict__ hdr, const uint32_t *__restrict__ cnt,
                                                      const uint32_t *__restrict__ starts, const uint32_t *__restrict__ xmap, const uint32_t *__restrict__ ymap,
                                                      const uint32_t *__restrict__ ids, const uint16_t *__restrict__ x, uint8_t *send, const uint64_t *__restrict__ peer_recv,
                                                      uint32_t *__restrict__ slot_pos) {
    const uint32_t lane = threadIdx.x & 31u, gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), rows = hdr[0];
    if (gw < world && lane == 0) {   // region headers: {count, epoch}
        uint8_t *base = p2p ? reinterpret_cast<uint8_t *>(peer_recv[gw]) + (size_t)rank * region_rows * row_bytes : send + (size_t)gw * region_rows * row_bytes;
        uint4 h; h.x = cnt[gw]; h.y = *epoch_dev; h.z = 0; h.w = 0;
        *reinterpret_cast<uint4 *>(base) = h;
    }
    if (gw >= rows) return;
    uint32_t d = 0;
    while (d + 1 < world && starts[d + 1] <= gw) d++;
    const uint32_t j = gw - starts[d], t = xmap[gw], slot = ymap[gw];
    uint8_t *base = p2p ? reinterpret_cast<uint8_t *>(peer_recv[d]) + (size_t)rank * region_rows * row_bytes : send + (size_t)d * region_rows * row_bytes;
    uint8_t *dst = base + (size_t)(1 + j) * row_bytes;
    const uint4 *src = reinterpret_cast<const uint4 *>(x + (size_t)t * hidden);
    for (uint32_t c = lane; c < hidden / 8; c += 32) reinterpret_cast<uint4 *>(dst)[c] = __ldg(src + c);
    if (lane == 0) {
        uint4 m; m.x = ids[slot] - d * experts_local; m.y = slot; m.z = 0; m.w = 0;
        *reinterpret_cast<uint4 *>(dst + (size_t)hidden * 2) = m;
        slot_pos[slot] = d * region_rows + 1 + j;
    }
}

// after a kernel that stored into peers: publish the epoch in every peer's flag word for this rank
__global__ void ep_signal_kernel(uint32_t world, uint32_t rank, const uint32_t *__restrict__ epoch_dev, const uint64_t *__restrict__ peer_flags) {
    const uint32_t d = threadIdx.x;
    if (d >= world) return;
    const uint32_t epoch = *epoch_dev;
    __threadfence_system();
    uint32_t *f = reinterpret_cast<uint32_t *>(peer_flags[d]) + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
}
// bounded wait until every source has published `epoch`; on expiry *err = code and the kernel returns
__global__ void ep_wait_kernel(uint32_t world, const uint32_t *__restrict__ epoch_dev, const uint32_t *flags, uint32_t *err, uint32_t code) {
    const uint32_t r = threadIdx.x;
    if (r >= world) return;
    const uint32_t epoch = *epoch_dev;
    for (uint32_t i = 0; i < (1u << 22); i++) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + r) : "memory");
        if ((int32_t)(v - epoch) >= 0) return;
        __nanosleep(200);
    }
    atomicCAS(err, 0u, code);
}

// candidate ids over every region row: header rows and rows past a region's count are absent
__global__ void ep_ids_kernel(uint32_t world, uint32_t region_rows, size_t row_bytes, uint32_t hidden, const uint8_t *__restrict__ recv, uint32_t *__restrict__ rids) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= world * region_rows) return;
    const uint32_t r = i / region_rows, jj = i - r * region_rows;
    const uint32_t count = *reinterpret_cast<const uint32_t *>(recv + (size_t)r * region_rows * row_bytes);
    uint32_t id = 0xffffffffu;
    if (jj >= 1 && jj - 1 < count) id = *reinterpret_cast<const uint32_t *>(recv + (size_t)i * row_bytes + (size_t)hidden * 2);
    rids[i] = id;
}

// push the present result rows to their owners: region (source r, row jj) -> owner r's back buffer, region `rank`
__global__ void __launch_bounds__(256) ep_return_kernel(uint32_t world, uint32_t rank, uint32_t region_rows, uint32_t hidden, const uint32_t *__restrict__ rids,
                                                        const float *__restrict__ dn, const uint64_t *__restrict__ peer_back) {
    const uint32_t lane = threadIdx.x & 31u, i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= world * region_rows || rids[i] == 0xffffffffu) return;
    const uint32_t r = i / region_rows, jj = i - r * region_rows;
    float *dst = reinterpret_cast<float *>(peer_back[r]) + ((size_t)rank * region_rows + jj) * hidden;
    const float4 *src = reinterpret_cast<const float4 *>(dn + (size_t)i * hidden);
    for (uint32_t c = lane; c < hidden / 4; c += 32) reinterpret_cast<float4 *>(dst)[c] = src[c];
}

// out[t] = sum over slots, in slot order, multiply then add (never fused), of w[t][s] * back[slot_pos[t*topk+s]]
__global__ void __launch_bounds__(256) ep_combine_kernel(uint32_t topk, uint32_t hidden, const float *__restrict__ w, const float *__restrict__ back,
                                                         const uint32_t *__restrict__ slot_pos, float *__restrict__ out, uint16_t *__restrict__ out16) {
    const uint32_t t = blockIdx.x;
    for (uint32_t c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
        float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t s = 0; s < topk; s++) {
            const float ws = __ldg(w + (size_t)t * topk + s);
            const float4 v = *reinterpret_cast<const float4 *>(back + (size_t)slot_pos[t * topk + s] * hidden + c);
            const float4 p = make_float4(__fmul_rn(ws, v.x), __fmul_rn(ws, v.y), __fmul_rn(ws, v.z), __fmul_rn(ws, v.w));
            m = s == 0 ? p : make_float4(__fadd_rn(m.x, p.x), __fadd_rn(m.y, p.y), __fadd_rn(m.z, p.z), __fadd_rn(m.w, p.w));
        }
        if (out) *reinterpret_cast<float4 *>(out + (size_t)t * hidden + c) = m;
        if (out16) {
            auto rne = [](float f) -> uint32_t { const uint32_t x = __float_as_uint(f); return ((x & 0x7fffffffu) > 0x7f800000u) ? ((x >> 16) | 0x40u) : ((x + 0x7fffu + ((x >> 16) & 1u)) >> 16); };
            uint2 pk; pk.x = rne(m.x) | (rne(m.y) << 16); pk.y = rne(m.z) | (rne(m.w) << 16);
            *reinterpret_cast<uint2 *>(out16 + (size_t)t * hidden + c) = pk;
        }
    }
}

}  // namespace b200
using namespace b200;

extern "C" {

int omega_gpu_moe_ep_create(uint32_t world, uint32_t rank, uint32_t experts, uint32_t topk, uint32_t hidden, uint32_t tokens_local_max, OmegaGpuMoeEp **out) {
    if (out) *out = nullptr;
    if (!out || !world || world > 64 || rank >= world || !experts || experts % world || !topk || topk > 32 || !hidden || hidden % 8 || !tokens_local_max) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    OmegaGpuMoeEp *ep = (OmegaGpuMoeEp *)calloc(1, sizeof *ep);
    if (!ep) return OMEGA_GPU_FP8_BAD_ARGS;
    ep->world = world; ep->rank = rank; ep->topk = topk; ep->experts = experts; ep->experts_local = experts / world; ep->hidden = hidden;
    ep->tokens_local_max = tokens_local_max; ep->cap = tokens_local_max * topk; ep->region_rows = ep->cap + 1; ep->row_bytes = (size_t)hidden * 2 + 16;
    const size_t R = ep->cap, cand = (size_t)world * ep->region_rows;
    const size_t xb = (cand * ep->row_bytes + 255) & ~(size_t)255, db = (cand * hidden * 4 + 255) & ~(size_t)255;
    ep->off_back = xb; ep->off_flags = xb + db; ep->comm_bytes = xb + db + 1024;
    uint8_t *loc = nullptr;
    const size_t loc_bytes = (R + 8) * 4 * 6 + (size_t)world * 8 + 256 + cand * 4 + R * 4 + 4096;
    bool ok = cuda_ok(cudaMalloc(&ep->comm, ep->comm_bytes), "cudaMalloc(ep comm)") && cuda_ok(cudaMemset(ep->comm, 0, ep->comm_bytes), "memset") &&
              cuda_ok(cudaMalloc(&ep->send, xb), "cudaMalloc(ep send)") && cuda_ok(cudaMalloc(&ep->dn, db), "cudaMalloc(ep dn)") &&
              cuda_ok(cudaMalloc(&loc, loc_bytes), "cudaMalloc(ep scratch)") && cuda_ok(cudaMemset(loc, 0, loc_bytes), "memset") &&
              cuda_ok(cudaMalloc(&ep->peer_tab, (size_t)world * 8 * 4), "cudaMalloc(ep peers)");
    if (!ok) { if (ep->comm) cudaFree(ep->comm); if (ep->send) cudaFree(ep->send); if (ep->dn) cudaFree(ep->dn); if (loc) cudaFree(loc); if (ep->peer_tab) cudaFree(ep->peer_tab); free(ep); return OMEGA_GPU_FP8_CHIP_FAIL; }
    ep->recv = ep->comm; ep->back = (float *)(ep->comm + ep->off_back);
    ep->flag_disp = (uint32_t *)(ep->comm + ep->off_flags); ep->flag_ret = ep->flag_disp + 64;
    uint32_t *p = (uint32_t *)loc;
    ep->ids = p; p += R + 8; ep->wts = (float *)p; p += R + 8; ep->dest = p; p += R + 8; ep->xmap = p; p += R + 8; ep->ymap = p; p += R + 8; ep->slot_pos = p; p += R + 8;
    ep->cnt = p; p += world; ep->starts = p; p += world; ep->hdr = p; p += 16; ep->err = p; p += 16; ep->rids = p;
    *out = ep;
    return OMEGA_GPU_FP8_OK;
}

void omega_gpu_moe_ep_free(OmegaGpuMoeEp *ep) {
    if (!ep) return;
    Lock l;
    for (int i = 0; i < ep->n_opened; i++) cudaIpcCloseMemHandle(ep->opened[i]);
    if (ep->comm) cudaFree(ep->comm);
    if (ep->send) cudaFree(ep->send);
    if (ep->dn) cudaFree(ep->dn);
    if (ep->ids) cudaFree(ep->ids);
    if (ep->peer_tab) cudaFree(ep->peer_tab);
    free(ep);
}

/* out[0..7] = {send_va, recv_va, dn_va, back_va, activation region bytes, result region bytes, comm_va, comm_bytes} */
int omega_gpu_moe_ep_buffers(const OmegaGpuMoeEp *ep, uint64_t *out) {
    if (!ep || !out) return OMEGA_GPU_FP8_BAD_ARGS;
    out[0] = (uint64_t)(uintptr_t)ep->send; out[1] = (uint64_t)(uintptr_t)ep->recv; out[2] = (uint64_t)(uintptr_t)ep->dn; out[3] = (uint64_t)(uintptr_t)ep->back;
    out[4] = (uint64_t)ep->region_rows * ep->row_bytes; out[5] = (uint64_t)ep->region_rows * ep->hidden * 4; out[6] = (uint64_t)(uintptr_t)ep->comm; out[7] = ep->comm_bytes;
    return OMEGA_GPU_FP8_OK;
}

/* 64-byte CUDA IPC handle of this rank's comm block (what its peers map) */
int omega_gpu_moe_ep_export(const OmegaGpuMoeEp *ep, uint8_t *handle64) {
    if (!ep || !handle64) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    cudaIpcMemHandle_t h;
    if (!cuda_ok(cudaIpcGetMemHandle(&h, ep->comm), "cudaIpcGetMemHandle")) return OMEGA_GPU_FP8_CHIP_FAIL;
    memcpy(handle64, &h, 64);
    return OMEGA_GPU_FP8_OK;
}

/* handles: world x 64 bytes, rank order (this rank's own entry is ignored). Switches the object to direct peer stores. */
int omega_gpu_moe_ep_connect(OmegaGpuMoeEp *ep, const uint8_t *handles) {
    if (!ep || !handles) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    uint64_t tab[4 * 64];
    for (uint32_t r = 0; r < ep->world; r++) {
        uint8_t *base = ep->comm;
        if (r != ep->rank) {
            cudaIpcMemHandle_t h; memcpy(&h, handles + (size_t)r * 64, 64);
            void *p = nullptr;
            if (!cuda_ok(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) return OMEGA_GPU_FP8_CHIP_FAIL;
            ep->opened[ep->n_opened++] = p; base = (uint8_t *)p;
        }
        tab[r] = (uint64_t)(uintptr_t)base; tab[ep->world + r] = (uint64_t)(uintptr_t)(base + ep->off_back);
        tab[2 * ep->world + r] = (uint64_t)(uintptr_t)(base + ep->off_flags); tab[3 * ep->world + r] = (uint64_t)(uintptr_t)(base + ep->off_flags + 256);
    }
    if (!cuda_ok(cudaMemcpy(ep->peer_tab, tab, (size_t)ep->world * 32, cudaMemcpyHostToDevice), "copy peer table")) return OMEGA_GPU_FP8_CHIP_FAIL;
    ep->p2p = 1;
    return OMEGA_GPU_FP8_OK;
}

/* top-k, grouping by destination rank and packing of the local tokens' picks (plus, with peer stores, the signal) */
int omega_gpu_moe_ep_dispatch_async(OmegaGpuMoeEp *ep, uint32_t tokens_local, uint64_t logits_va, uint64_t x_va, void *stream) {
    if (!ep || !tokens_local || tokens_local > ep->tokens_local_max || !logits_va || !x_va) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t R = tokens_local * ep->topk, G = ep->world;
    if (!cuda_ok(launch_topk(tokens_local, ep->experts, ep->topk, 1, (const uint16_t *)(uintptr_t)logits_va, ep->ids, ep->wts, s), "topk launch")) return OMEGA_GPU_FP8_CHIP_FAIL;
    ep_dest_kernel<<<(R + 255) / 256, 256, 0, s>>>(R, ep->experts_local, ep->ids, ep->dest, ep->err + 4);
    OmegaGpuMoePlanOut o = {};
    o.counts_va = (uint64_t)(uintptr_t)ep->cnt; o.starts_va = (uint64_t)(uintptr_t)ep->starts; o.xmap_va = (uint64_t)(uintptr_t)ep->xmap;
    o.ymap_va = (uint64_t)(uintptr_t)ep->ymap; o.header_va = (uint64_t)(uintptr_t)ep->hdr;
    if (!cuda_ok(launch_plan(tokens_local, ep->topk, G, ep->topk, 0, ep->dest, o, s), "destination plan launch")) return OMEGA_GPU_FP8_CHIP_FAIL;
    const uint32_t warps = R > G ? R : G;
    ep_pack_kernel<<<(warps + 7) / 8, 256, 0, s>>>(G, ep->rank, ep->topk, ep->experts_local, ep->hidden, ep->region_rows, ep->row_bytes, ep->p2p, ep->err + 4, ep->hdr, ep->cnt,
                                                   ep->starts, ep->xmap, ep->ymap, ep->ids, (const uint16_t *)(uintptr_t)x_va, ep->send, ep->peer_tab, ep->slot_pos);
    if (ep->p2p) ep_signal_kernel<<<1, 64, 0, s>>>(G, ep->rank, ep->err + 4, ep->peer_tab + 2 * G);
    return cuda_ok(cudaGetLastError(), "ep dispatch launch") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

/* expert side: (wait for every source,) plan over the received rows, run the local experts, (push results back) */
int omega_gpu_moe_ep_experts_async(OmegaGpuMoeEp *ep, OmegaGpuMoeLayer *local, void *stream) {
    if (!ep || !local) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t G = ep->world, cand = G * ep->region_rows;
    if (ep->p2p) ep_wait_kernel<<<1, 64, 0, s>>>(G, ep->err + 4, ep->flag_disp, ep->err, 11);
    ep_ids_kernel<<<(cand + 255) / 256, 256, 0, s>>>(G, ep->region_rows, ep->row_bytes, ep->hidden, ep->recv, ep->rids);
    if (!cuda_ok(cudaGetLastError(), "ep ids launch")) return OMEGA_GPU_FP8_CHIP_FAIL;
    if (!layer_forward_routed(local, cand, ep->rids, ep->recv, ep->row_bytes, ep->dn, s)) return OMEGA_GPU_FP8_CHIP_FAIL;
    if (ep->p2p) {
        ep_return_kernel<<<(cand + 7) / 8, 256, 0, s>>>(G, ep->rank, ep->region_rows, ep->hidden, ep->rids, ep->dn, ep->peer_tab + G);
        ep_signal_kernel<<<1, 64, 0, s>>>(G, ep->rank, ep->err + 4, ep->peer_tab + 3 * G);
    }
    return cuda_ok(cudaGetLastError(), "ep experts launch") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

/* owner side: (wait for every expert rank,) slot-order weighted sum of the returned rows */
int omega_gpu_moe_ep_combine_async(OmegaGpuMoeEp *ep, uint32_t tokens_local, uint64_t out_f32_va, uint64_t out_bf16_va, void *stream) {
    if (!ep || !tokens_local || tokens_local > ep->tokens_local_max || (!out_f32_va && !out_bf16_va)) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = (cudaStream_t)stream;
    if (ep->p2p) ep_wait_kernel<<<1, 64, 0, s>>>(ep->world, ep->err + 4, ep->flag_ret, ep->err, 12);
    ep_combine_kernel<<<tokens_local, 256, 0, s>>>(ep->topk, ep->hidden, ep->wts, ep->back, ep->slot_pos, (float *)(uintptr_t)out_f32_va, (uint16_t *)(uintptr_t)out_bf16_va);
    return cuda_ok(cudaGetLastError(), "ep combine launch") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

/* 0, or the code of a bounded wait that ran out (11 dispatch flags, 12 return flags); synchronises the stream */
int omega_gpu_moe_ep_status(OmegaGpuMoeEp *ep, void *stream) {
    if (!ep) return OMEGA_GPU_FP8_BAD_ARGS;
    uint32_t v = 0;
    if (!cuda_ok(cudaMemcpyAsync(&v, ep->err, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream), "copy status") || !cuda_ok(cudaStreamSynchronize((cudaStream_t)stream), "ep status")) return OMEGA_GPU_FP8_CHIP_FAIL;
    return (int)v;
}

}  // extern "C"
