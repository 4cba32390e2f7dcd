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
#include "mma_common.cuh"

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
    // the transport's word, then the word the local tensor-core kernels record an expired wait in (word 4 of the plan header)
    uint32_t v = 0, k = 0;
    if (!cuda_ok(cudaMemcpyAsync(&v, ep->err, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream), "copy status") ||
        !cuda_ok(cudaMemcpyAsync(&k, ep->hdr + 4, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream), "copy status") ||
        !cuda_ok(cudaStreamSynchronize((cudaStream_t)stream), "ep status")) return OMEGA_GPU_FP8_CHIP_FAIL;
    return (int)(v ? v : k);
}

}  // extern "C"

// =====================================================================================================================
// Fused expert-parallel stack: the same launches per layer and rank as on one GPU (expert kernel(s) + combine/norm/scatter).
//
// Every rank first gathers the router logits of all tokens (they are small) and computes the routing of every layer for
// all tokens: the global plan tells a sender the sorted row each of its picks has on the rank that owns the expert
// (global sorted row minus the start of that rank's first expert); the plan over the rank's own experts gives its
// row tiles. Per layer a rank then runs
//   combine+norm+quantise: its tokens' next-layer activation pieces are stored straight into the owning ranks' piece
//       buffers (peer stores), one system-scope atomic per delivered row on the receiver's counter;
//   gate|up GEMM: waits (bounded) until the counter shows every row of its plan, then runs as on one GPU;
//   down GEMM: stores every result row straight into its token owner's buffer and advances the owner's counter;
// and the next combine waits for its tokens' 8 x (hidden/256) result slices. Counters only grow; counters, piece buffers and
// scale buffers alternate by layer parity: a peer that already has all its results of layer l may deliver rows of layer l+1
// while this rank still reads rows of layer l. Rows of layer l+2 go into the buffers layer l used, so a sender first waits for
// the destination's buffer credit: every rank tells every other, after its expert kernel of a layer has completed, how many layers of
// that parity it has consumed (one store per peer and layer), and a sender compares its local copy of that number with the
// number of same-parity layers before the one it sends for. No collective and no host round trip per layer.
#include <vector>

struct OmegaGpuMoeEpStack {
    uint32_t world, rank, layers, topk, experts, experts_local, hidden, tokens, tokens_local, row_cap, x_pieces, tile_rows;
    float eps;
    std::vector<OmegaGpuMoeLayer *> local;
    char *route;                         // routing scratch (ids, weights, two plan batches)
    uint32_t *ids_g, *ids_l; float *wts_g;
    b200::PlanBatch pg, pl; size_t map_stride, tile_stride;
    uint8_t *comm; size_t comm_bytes, q_par, off_sx, sx_par, off_dn, off_cnt, off_credit;   // peers map this block: pieces x2 | scales x2 | results | counters (x2: by layer parity)
    uint64_t *peer_tab;                  // device [5][world]: pieces, scales, results, counters, buffer credits of every rank
    float *h, *norm_w; uint32_t *err, *sched; bool one_launch;   // norm_w: device [layers][hidden], RMSNorm weight of each layer's input (ones until set)
    void *opened[64]; int n_opened; int connected;
    alignas(128) unsigned char tm_qx[2][128];
    uint32_t launches;
};

namespace b200 {

// also counts the steps on the device (a replayed graph cannot carry a host counter)
__global__ void ep_localise_kernel(size_t n, uint32_t e0, uint32_t e1, const uint32_t *__restrict__ ids, uint32_t *__restrict__ out, uint32_t *step) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0) *step += 1u;
    if (i < n) { const uint32_t e = ids[i]; out[i] = (e >= e0 && e < e1) ? e - e0 : 0xffffffffu; }
}

// One CTA per local token. dn/w != null: wait until this rank's result buffer is complete, combine in slot order and add to h.
// q_peers != null: quantise xn = bf16(RMSNorm(h)) into pieces and store them into the owners' piece buffers.
__global__ void __launch_bounds__(256) ep_combine_norm_scatter_kernel(
        uint32_t hidden, uint32_t topk, float eps, const uint16_t *__restrict__ x16, const float *__restrict__ w, const float *__restrict__ dn, float *__restrict__ h,
        const unsigned long long *ret_gate, unsigned long long ret_unit, const uint32_t *step, uint32_t uses_per_step, uint32_t uses_before,
        const uint32_t *__restrict__ ids_next, const uint32_t *__restrict__ pos_next, const uint32_t *__restrict__ starts_next, uint32_t experts_local,
        uint32_t pieces, size_t piece_stride, size_t q_off, size_t sx_off, const uint64_t *__restrict__ q_peers, const uint64_t *__restrict__ sx_peers, const uint64_t *__restrict__ cnt_peers,
        uint32_t parity, uint16_t *__restrict__ h16, uint32_t *err, uint32_t *__restrict__ sched, uint32_t n_sched,
        unsigned long long *bump, const uint32_t *bump_rows,
        uint32_t world, uint32_t rank, const uint64_t *__restrict__ credit_peers, const unsigned long long *credit_local,
        uint32_t done_parity, uint32_t done_uses_per_step, uint32_t done_uses_before, uint32_t next_uses_per_step, uint32_t next_uses_before,
        const float *__restrict__ nw, uint32_t wait_limit) {
    __shared__ double red[8];
    __shared__ float s_scale;
    __shared__ uint32_t s_d[32], s_row[32], s_fail;
    __shared__ uint8_t *s_q[32]; __shared__ float *s_sx[32];   // per pick: the destination rank's piece and scale buffers of the next layer's parity
    const uint32_t t = blockIdx.x, tid = threadIdx.x, lane = tid & 31u, kb_total = hidden / 128u;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next gate|up GEMM may start fetching weights
    // the expert kernel before this one has completed: clear its work-list words for the next launch, and count the input rows its
    // layer consumed (the delivery counters only grow)
    if (blockIdx.x == 0) {
        if (sched) for (uint32_t i = tid; i < n_sched; i += 256) sched[i] = 0;
        if (bump && tid == 0) *bump += *bump_rows;
        // Buffer credit: this rank's expert kernel of the layer before this kernel has completed, so the piece and scale buffers of that
        // layer's parity may be overwritten (by rows of the layer two ahead). Tell every rank how many layers of that parity this rank
        // has consumed since the stack was made; a sender waits on its own copy of that number before it stores into this rank.
        if (done_parity < 2u && tid < world) {
            const unsigned long long v = (unsigned long long)(*step - 1u) * done_uses_per_step + done_uses_before + 1ull;
            unsigned long long *dst = reinterpret_cast<unsigned long long *>(credit_peers[tid]) + 2u * rank + done_parity;
            asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(v) : "memory");
        }
    }
    if (tid == 0) {
        s_fail = *reinterpret_cast<volatile uint32_t *>(err) ? 1u : 0u;
        if (!s_fail && dn && ret_gate) {
            // the counter only grows: this layer's results are complete at (uses so far + 1) x slices per use
            const unsigned long long ret_want = ((unsigned long long)(*step - 1u) * uses_per_step + uses_before + 1ull) * ret_unit;
            bool ok = false;
            for (uint32_t i = 0; i < wait_limit && !ok; i++) {
                unsigned long long v;
                asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(ret_gate) : "memory");
                ok = v >= ret_want;
                if (!ok && (i & 63u) == 63u && *reinterpret_cast<volatile uint32_t *>(err)) break;   // a failure is already recorded: give up at once
                if (!ok) __nanosleep(100);
            }
            if (!ok) { atomicCAS(err, 0u, 16u); s_fail = 1; }
        }
    }
    if (q_peers && tid < topk) {
        const size_t i = (size_t)t * topk + tid;        // ids_next / pos_next are already offset to this rank's first token
        const uint32_t d = ids_next[i] / experts_local;
        s_d[tid] = d; s_row[tid] = pos_next[i] - starts_next[d * experts_local];
        s_q[tid] = reinterpret_cast<uint8_t *>(q_peers[d]) + q_off; s_sx[tid] = reinterpret_cast<float *>(sx_peers[d] + sx_off);
    }
    __syncthreads();
    if (q_peers && tid < topk && !s_fail) {
        // the destination's buffers of the next layer's parity still hold the rows of the layer two back until that rank's expert kernel
        // for it has completed: wait (bounded) for its credit. Data dependence through routed rows usually implies it, but not for every routing.
        const unsigned long long want = (unsigned long long)(*step - 1u) * next_uses_per_step + next_uses_before;
        const unsigned long long *c = credit_local + 2u * s_d[tid] + parity;
        bool ok = want == 0ull;
        for (uint32_t i = 0; i < wait_limit && !ok; i++) {
            unsigned long long v;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(c) : "memory");
            ok = v >= want;
            if (!ok && (i & 63u) == 63u && *reinterpret_cast<volatile uint32_t *>(err)) break;
            if (!ok) __nanosleep(100);
        }
        if (!ok) { atomicCAS(err, 0u, 17u); s_fail = 1; }
    }
    __syncthreads();
    if (s_fail) return;
    double sq = 0.0;
    float4 k0 = make_float4(0, 0, 0, 0), k1 = k0;   // this thread's columns of h (tid * 4 and 1024 + tid * 4): the quantiser below uses the same mapping
    for (uint32_t c = tid * 4; c < hidden; c += 1024) {
        const size_t i = (size_t)t * hidden + c;
        float4 v;
        if (x16) { const uint2 u = *reinterpret_cast<const uint2 *>(x16 + i); v = make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u)); }
        else v = *reinterpret_cast<const float4 *>(h + i);
        if (dn) {
            const float4 m = combine_slots<true>(topk, w, dn, (size_t)t * topk, hidden, c);
            v = make_float4(__fadd_rn(v.x, m.x), __fadd_rn(v.y, m.y), __fadd_rn(v.z, m.z), __fadd_rn(v.w, m.w));
        }
        *reinterpret_cast<float4 *>(h + i) = v;
        if (c < 1024u) k0 = v; else if (c < 2048u) k1 = v;
        if (h16) {
            auto rne = [](float f) -> uint32_t { const uint32_t b = __float_as_uint(f); return ((b & 0x7fffffffu) > 0x7f800000u) ? ((b >> 16) | 0x40u) : ((b + 0x7fffu + ((b >> 16) & 1u)) >> 16); };
            uint2 pk; pk.x = rne(v.x) | (rne(v.y) << 16); pk.y = rne(v.z) | (rne(v.w) << 16);
            *reinterpret_cast<uint2 *>(h16 + i) = pk;
        }
        sq += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
    }
    if (!q_peers) return;
    for (int o = 16; o; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if (lane == 0) red[tid >> 5] = sq;
    __syncthreads();
    if (tid == 0) { double acc = 0; for (int i = 0; i < 8; i++) acc += red[i]; s_scale = (float)(1.0 / sqrt(acc / (double)hidden + (double)eps)); }
    __syncthreads();
    const float sc = s_scale;
    for (uint32_t kb = tid >> 5; kb < kb_total; kb += 8) {
        const uint32_t c = kb * 128u + lane * 4u;
        const float4 hv = c < 1024u ? k0 : c < 2048u ? k1 : *reinterpret_cast<const float4 *>(h + (size_t)t * hidden + c);   // c = tid * 4 + 1024 j: this thread's own columns
        const float4 wv = __ldg(reinterpret_cast<const float4 *>(nw + c));
        // the same arithmetic, value for value, as combine_norm_scatter_kernel of the single-GPU stack: xn = bf16(h * s * w), then the shared quantiser
        float v[4] = {__fmul_rn(__fmul_rn(hv.x, sc), wv.x), __fmul_rn(__fmul_rn(hv.y, sc), wv.y), __fmul_rn(__fmul_rn(hv.z, sc), wv.z), __fmul_rn(__fmul_rn(hv.w, sc), wv.w)};
#pragma unroll
        for (int i = 0; i < 4; i++) v[i] = __uint_as_float(bf16_rne_bits(v[i]) << 16);
        uint32_t codes[4];
        const float qs = quant_pieces_warp(v, pieces, codes);
        for (uint32_t s = 0; s < topk; s++) {
            uint8_t *q = s_q[s];
            for (uint32_t p = 0; p < pieces; p++) *reinterpret_cast<uint32_t *>(q + (size_t)p * piece_stride + (size_t)s_row[s] * hidden + c) = codes[p];
            if (lane == 0) s_sx[s][(size_t)s_row[s] * kb_total + kb] = qs;
        }
    }
    // publish: every thread's stores are ordered before the barrier; the few publishing threads then fence at system scope (a fence is
    // cumulative: it covers what the barrier made visible to them) and count the row in. One fence by one warp, not one per thread.
    __syncthreads();
    if (tid < topk) {
        __threadfence_system();
        atomicAdd_system(reinterpret_cast<unsigned long long *>(cnt_peers[s_d[tid]]) + parity, 1ull);
    }
}

}  // namespace b200

extern "C" {

int omega_gpu_moe_epstack_create(uint32_t world, uint32_t rank, uint32_t layers, OmegaGpuMoeLayer *const *local, uint32_t experts, uint32_t tokens, float eps,
                                 OmegaGpuMoeEpStack **out) {
    if (out) *out = nullptr;
    if (!out || !local || !layers || !world || world > 64 || rank >= world || !experts || experts % world || !tokens || tokens % world) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    LayerView v0; layer_view(local[0], &v0);
    if (v0.shared) { set_error("ep stack: layers with a shared expert are not sharded by this stack"); return OMEGA_GPU_FP8_BAD_ARGS; }
    if (v0.engine != OMEGA_GPU_MOE_ENGINE_MMA || v0.experts != experts / world || v0.max_tokens < tokens || v0.topk > 32) { set_error("ep stack: local layers must run the tensor-core engine over experts/world experts with max_tokens >= tokens"); return OMEGA_GPU_FP8_BAD_ARGS; }
    OmegaGpuMoeEpStack *S = new OmegaGpuMoeEpStack();
    S->world = world; S->rank = rank; S->layers = layers; S->topk = v0.topk; S->experts = experts; S->experts_local = experts / world; S->hidden = v0.hidden;
    S->tokens = tokens; S->tokens_local = tokens / world; S->row_cap = v0.row_cap; S->x_pieces = v0.x_pieces; S->tile_rows = v0.tile_rows; S->eps = eps;
    S->n_opened = 0; S->connected = 0; S->launches = 0; S->route = nullptr; S->comm = nullptr; S->peer_tab = nullptr; S->h = nullptr;
    for (uint32_t i = 0; i < layers; i++) {
        if (!local[i] || !layer_share_workspace(local[i], local[0])) { delete S; set_error("ep stack: layer %u does not match layer 0", i); return OMEGA_GPU_FP8_BAD_ARGS; }
        S->local.push_back(local[i]);
    }
    const size_t K = S->topk, T = tokens, R = T * K, H = S->hidden, E = experts, Ln = layers, Rp = S->row_cap;
    S->map_stride = (R + 8 + 63) & ~(size_t)63; S->tile_stride = (R / 8 + E + 8 + 15) & ~(size_t)15;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off += (bytes + 255) & ~(size_t)255; return o; };
    const size_t o_ig = take(Ln * R * 4), o_il = take(Ln * R * 4), o_w = take(Ln * R * 4);
    size_t o_pb[2][7];
    for (int b = 0; b < 2; b++) {
        o_pb[b][0] = take(Ln * E * 4); o_pb[b][1] = take(Ln * E * 4); o_pb[b][2] = take(Ln * S->map_stride * 4); o_pb[b][3] = take(Ln * S->map_stride * 4);
        o_pb[b][4] = take(Ln * S->map_stride * 4); o_pb[b][5] = take(Ln * 32); o_pb[b][6] = take(Ln * S->tile_stride * 16);
    }
    const size_t o_h = take((size_t)S->tokens_local * H * 4), o_err = take(64), o_sched = take((S->tile_stride + 1) * 4), o_nw = take(Ln * H * 4);
    bool ok = cuda_ok(cudaMalloc(&S->route, off), "cudaMalloc(ep routing)") && cuda_ok(cudaMemset(S->route, 0, off), "memset");
    if (ok) {
        char *f = S->route;
        S->ids_g = (uint32_t *)(f + o_ig); S->ids_l = (uint32_t *)(f + o_il); S->wts_g = (float *)(f + o_w);
        PlanBatch *pb[2] = {&S->pg, &S->pl};
        for (int b = 0; b < 2; b++) {
            pb[b]->counts = (uint32_t *)(f + o_pb[b][0]); pb[b]->starts = (uint32_t *)(f + o_pb[b][1]); pb[b]->xmap = (uint32_t *)(f + o_pb[b][2]);
            pb[b]->ymap = (uint32_t *)(f + o_pb[b][3]); pb[b]->pos = (uint32_t *)(f + o_pb[b][4]); pb[b]->header = (uint32_t *)(f + o_pb[b][5]);
            pb[b]->tiles = (uint4 *)(f + o_pb[b][6]); pb[b]->map_stride = S->map_stride; pb[b]->tile_stride = S->tile_stride;
        }
        S->h = (float *)(f + o_h); S->err = (uint32_t *)(f + o_err); S->sched = (uint32_t *)(f + o_sched); S->norm_w = (float *)(f + o_nw);
        { std::vector<float> ones(Ln * H, 1.0f); ok = cuda_ok(cudaMemcpy(S->norm_w, ones.data(), ones.size() * 4, cudaMemcpyHostToDevice), "init norm weights"); }
        S->one_launch = ((v0.x_pieces == 2 && v0.act_pieces == 3) || (v0.x_pieces == 1 && v0.act_pieces == 1) || (v0.x_pieces == 2 && v0.act_pieces == 2)) &&
                        ffn_shape_ok(v0.hidden, v0.inter) && !getenv("B200MOE_TWO_LAUNCH");
        // the block peers write into: activation pieces | their scales | result rows of the local tokens | counters
        const size_t qb = ((size_t)S->x_pieces * Rp * H + 255) & ~(size_t)255, sb = (Rp * (H / 128) * 4 + 255) & ~(size_t)255, db = ((size_t)S->tokens_local * K * H * 4 + 255) & ~(size_t)255;
        S->q_par = qb; S->off_sx = 2 * qb; S->sx_par = sb; S->off_dn = 2 * qb + 2 * sb; S->off_cnt = S->off_dn + db; S->off_credit = S->off_cnt + 256; S->comm_bytes = S->off_credit + 64 * 2 * 8;   // counters, then credits [source rank][layer parity]
        ok = cuda_ok(cudaMalloc(&S->comm, S->comm_bytes), "cudaMalloc(ep comm)") && cuda_ok(cudaMemset(S->comm, 0, S->comm_bytes), "memset") &&
             cuda_ok(cudaMalloc(&S->peer_tab, (size_t)world * 40), "cudaMalloc(ep peers)") && make_tmap_u8(S->tm_qx[0], S->comm, (uint64_t)S->x_pieces * Rp, H, 32) &&
             make_tmap_u8(S->tm_qx[1], S->comm + S->q_par, (uint64_t)S->x_pieces * Rp, H, 32);
    }
    if (ok && world == 1) {
        uint64_t tab[5] = {(uint64_t)(uintptr_t)S->comm, (uint64_t)(uintptr_t)(S->comm + S->off_sx), (uint64_t)(uintptr_t)(S->comm + S->off_dn), (uint64_t)(uintptr_t)(S->comm + S->off_cnt),
                           (uint64_t)(uintptr_t)(S->comm + S->off_credit)};
        ok = cuda_ok(cudaMemcpy(S->peer_tab, tab, 40, cudaMemcpyHostToDevice), "copy peer table"); S->connected = 1;
    }
    if (!ok) { if (S->route) cudaFree(S->route); if (S->comm) cudaFree(S->comm); if (S->peer_tab) cudaFree(S->peer_tab); delete S; return OMEGA_GPU_FP8_CHIP_FAIL; }
    *out = S;
    return OMEGA_GPU_FP8_OK;
}

void omega_gpu_moe_epstack_free(OmegaGpuMoeEpStack *S) {
    if (!S) return;
    Lock l;
    for (int i = 0; i < S->n_opened; i++) cudaIpcCloseMemHandle(S->opened[i]);
    if (S->route) cudaFree(S->route);
    if (S->comm) cudaFree(S->comm);
    if (S->peer_tab) cudaFree(S->peer_tab);
    delete S;
}

int omega_gpu_moe_epstack_export(const OmegaGpuMoeEpStack *S, uint8_t *handle64) {
    if (!S || !handle64) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    cudaIpcMemHandle_t h;
    if (!cuda_ok(cudaIpcGetMemHandle(&h, S->comm), "cudaIpcGetMemHandle")) return OMEGA_GPU_FP8_CHIP_FAIL;
    memcpy(handle64, &h, 64);
    return OMEGA_GPU_FP8_OK;
}

int omega_gpu_moe_epstack_connect(OmegaGpuMoeEpStack *S, const uint8_t *handles) {
    if (!S || !handles) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    uint64_t tab[5 * 64];
    for (uint32_t r = 0; r < S->world; r++) {
        uint8_t *base = S->comm;
        if (r != S->rank) {
            cudaIpcMemHandle_t h; memcpy(&h, handles + (size_t)r * 64, 64);
            void *p = nullptr;
            if (!cuda_ok(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) return OMEGA_GPU_FP8_CHIP_FAIL;
            S->opened[S->n_opened++] = p; base = (uint8_t *)p;
        }
        tab[r] = (uint64_t)(uintptr_t)base; tab[S->world + r] = (uint64_t)(uintptr_t)(base + S->off_sx);
        tab[2 * S->world + r] = (uint64_t)(uintptr_t)(base + S->off_dn); tab[3 * S->world + r] = (uint64_t)(uintptr_t)(base + S->off_cnt);
        tab[4 * S->world + r] = (uint64_t)(uintptr_t)(base + S->off_credit);
    }
    if (!cuda_ok(cudaMemcpy(S->peer_tab, tab, (size_t)S->world * 40, cudaMemcpyHostToDevice), "copy peer table")) return OMEGA_GPU_FP8_CHIP_FAIL;
    S->connected = 1;
    return OMEGA_GPU_FP8_OK;
}

uint32_t omega_gpu_moe_epstack_launches(const OmegaGpuMoeEpStack *S) { return S ? S->launches : 0; }
int omega_gpu_moe_epstack_set_norm(OmegaGpuMoeEpStack *S, uint32_t layer, const float *norm_w) {
    if (!S || !norm_w || layer >= S->layers) return OMEGA_GPU_FP8_BAD_ARGS;
    for (uint32_t i = 0; i < S->hidden; i++) if (!(norm_w[i] == norm_w[i]) || norm_w[i] - norm_w[i] != 0.0f) { set_error("ep stack: norm weight %u of layer %u is not finite", i, layer); return OMEGA_GPU_FP8_BAD_ARGS; }
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    return cuda_ok(cudaMemcpy(S->norm_w + (size_t)layer * S->hidden, norm_w, (size_t)S->hidden * 4, cudaMemcpyHostToDevice), "copy norm weights") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}
uint64_t omega_gpu_moe_epstack_h(const OmegaGpuMoeEpStack *S) { return S ? (uint64_t)(uintptr_t)S->h : 0; }

/* one whole step for this rank. logits_all_va: bf16 [layers][tokens][experts] of ALL tokens (gathered by the caller);
 * x_va: bf16 [tokens_local][hidden]; out_bf16_va: bf16 [tokens_local][hidden] (final h); the f32 h stays readable through
 * omega_gpu_moe_epstack_h. Stream-ordered; every rank must enqueue the same number of steps. */
int omega_gpu_moe_epstack_step_async(OmegaGpuMoeEpStack *S, uint64_t logits_all_va, uint64_t x_va, uint64_t out_bf16_va, void *stream) {
    if (!S || !logits_all_va || !x_va || !out_bf16_va) return OMEGA_GPU_FP8_BAD_ARGS;
    if (!S->connected) { set_error("ep stack: not connected to its peers"); return OMEGA_GPU_FP8_BAD_ARGS; }
    if (!st().opened || st().latched) return OMEGA_GPU_FP8_CHIP_FAIL;
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t G = S->world, K = S->topk, E = S->experts, El = S->experts_local, H = S->hidden, T = S->tokens, Tl = S->tokens_local, Ln = S->layers, Px = S->x_pieces;
    const size_t R = (size_t)T * K, pstride = (size_t)S->row_cap * H;
    const uint64_t *tab = S->peer_tab;
    unsigned long long *cnt = (unsigned long long *)(S->comm + S->off_cnt);   // [0..1] delivered input rows by layer parity, [2..3] delivered result slices
    float *dn_local = (float *)(S->comm + S->off_dn);
    const unsigned long long *credit = (const unsigned long long *)(S->comm + S->off_credit);   // [source rank][parity], written by that rank
    uint32_t n = 0;
    LayerView v0; layer_view(S->local[0], &v0);
    bool ok = cuda_ok(launch_topk(Ln * T, E, K, (int)v0.norm_topk, (const uint16_t *)(uintptr_t)logits_all_va, S->ids_g, S->wts_g, s), "topk launch"); n++;
    if (ok) { ep_localise_kernel<<<(unsigned)((Ln * R + 255) / 256), 256, 0, s>>>(Ln * R, S->rank * El, (S->rank + 1) * El, S->ids_g, S->ids_l, S->err + 4); n++; }
    ok = ok && cuda_ok(launch_plan_batch(Ln, T, K, E, K, 0, S->ids_g, S->pg, s), "global plan launch") &&
         cuda_ok(launch_plan_batch(Ln, T, K, El, K, S->tile_rows, S->ids_l, S->pl, s), "local plan launch"); n += 2;
    if (!ok) return OMEGA_GPU_FP8_CHIP_FAIL;
    const size_t tok0 = (size_t)S->rank * Tl * K;
    const unsigned long long ret_unit = (unsigned long long)Tl * K * (H / 256u);
    unsigned long long *base = (unsigned long long *)(S->err + 8);   // [0..1]: input rows already consumed through the even / odd layer counter
    ep_combine_norm_scatter_kernel<<<Tl, 256, 0, s>>>(H, K, S->eps, (const uint16_t *)(uintptr_t)x_va, nullptr, nullptr, S->h, nullptr, 0ull, S->err + 4, 0u, 0u,
                                                      S->ids_g + tok0, S->pg.pos + tok0, S->pg.starts, El, Px, pstride, (size_t)0, (size_t)0, tab, tab + G, tab + 3 * G, 0u, nullptr, S->err,
                                                      S->sched, (uint32_t)S->tile_stride + 1u, nullptr, nullptr,
                                                      G, S->rank, tab + 4 * G, credit, 0xffffffffu, 0u, 0u, (Ln + 1u) / 2u, 0u, S->norm_w, st().wait_limit); n++;
    for (uint32_t l = 0; l < Ln && ok; l++) {
        LayerView v; layer_view(S->local[l], &v);
        const uint32_t par = l & 1u;
        const uint32_t *hdr = S->pl.header + (size_t)l * 8;
        if (S->one_launch) {
            FfnLaunch f = {};
            f.gu_scale = v.gu_scale; f.dn_scale = v.dn_scale; f.x_scale = (const float *)(S->comm + S->off_sx + par * S->sx_par); f.qa = v.qa; f.sa = v.sa;
            f.tiles = S->pl.tiles + (size_t)l * S->tile_stride; f.header = hdr; f.ymap = S->pl.ymap + (size_t)l * S->map_stride; f.out = dn_local;
            f.hidden = H; f.inter = v.inter; f.q_rows = S->row_cap; f.sched = S->sched; f.err = S->err;
            f.wait_limit = st().wait_limit; f.gate = cnt + par; f.gate_base = base + par; f.out_peers = tab + 2 * G; f.ret_counters = tab + 3 * G; f.rows_per_rank = Tl * K; f.ret_index = 2 + par;
            ok = cuda_ok(launch_ffn(v.tm_gu, S->tm_qx[par], v.tm_dn, v.tm_qa, Px, v.act_pieces, f, s, true), "expert ffn launch"); n++;
        } else {
            MmaLaunch g = {};
            g.wscale = v.gu_scale; g.ascale = (const float *)(S->comm + S->off_sx + par * S->sx_par); g.tiles = S->pl.tiles + (size_t)l * S->tile_stride; g.header = hdr;
            g.q_out = v.qa; g.s_out = v.sa; g.q_rows = S->row_cap; g.q_pieces = v.act_pieces;
            g.n = 2 * v.inter; g.k = H; g.mode = 0; g.out_stride = v.inter; g.err = S->err;   // one failure word for the whole step: later kernels see it and do nothing
            g.gate = cnt + par; g.gate_base = base + par; g.wait_limit = st().wait_limit;
            ok = cuda_ok(launch_mma_grouped(v.tm_gu, S->tm_qx[par], Px, g, s, true), "gate|up mma launch"); n++;
            MmaLaunch d = {};
            d.wscale = v.dn_scale; d.ascale = v.sa; d.tiles = g.tiles; d.header = hdr; d.ymap = S->pl.ymap + (size_t)l * S->map_stride; d.out = dn_local; d.q_rows = S->row_cap;
            d.n = H; d.k = v.inter; d.mode = 1; d.out_stride = H; d.err = g.err;
            d.out_peers = tab + 2 * G; d.ret_counters = tab + 3 * G; d.ret_index = 2 + par; d.rows_per_rank = Tl * K; d.bump = base + par;
            ok = ok && cuda_ok(launch_mma_grouped(v.tm_dn, v.tm_qa, v.act_pieces, d, s, false), "down mma launch"); n++;
        }
        const bool last = l + 1 == Ln;
        const size_t nx = (size_t)(l + 1) * S->map_stride;
        if (ok) ep_combine_norm_scatter_kernel<<<Tl, 256, 0, s>>>(H, K, S->eps, nullptr, S->wts_g + (size_t)l * R + tok0, dn_local, S->h, cnt + 2 + par, ret_unit, S->err + 4, (Ln + 1u - par) / 2u, l / 2u,
                                                                  last ? nullptr : S->ids_g + (size_t)(l + 1) * R + tok0, last ? nullptr : S->pg.pos + nx + tok0,
                                                                  last ? nullptr : S->pg.starts + (size_t)(l + 1) * E, El, Px, pstride, (par ^ 1u) * S->q_par, (par ^ 1u) * S->sx_par, last ? nullptr : tab, tab + G, tab + 3 * G,
                                                                  par ^ 1u, last ? (uint16_t *)(uintptr_t)out_bf16_va : nullptr, S->err,
                                                                  S->sched, (uint32_t)S->tile_stride + 1u, S->one_launch ? base + par : nullptr, hdr,
                                                                  G, S->rank, tab + 4 * G, credit, par, (Ln + 1u - par) / 2u, l / 2u, (Ln + par) / 2u, (l + 1u) / 2u,
                                                                  S->norm_w + (size_t)(last ? 0 : l + 1) * H, st().wait_limit);
        n++;
    }
    S->launches = n;
    return ok && cuda_ok(cudaGetLastError(), "ep stack launch") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

/* synchronises `stream`; 0, or a non-zero code when a bounded wait ran out anywhere in the step */
int omega_gpu_moe_epstack_status(OmegaGpuMoeEpStack *S, void *stream) {
    if (!S) return OMEGA_GPU_FP8_BAD_ARGS;
    std::vector<uint32_t> hdr(S->layers * 8); uint32_t e = 0;
    if (!cuda_ok(cudaMemcpyAsync(&e, S->err, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream), "copy status") ||
        !cuda_ok(cudaMemcpyAsync(hdr.data(), S->pl.header, hdr.size() * 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream), "copy status") ||
        !cuda_ok(cudaStreamSynchronize((cudaStream_t)stream), "ep stack status")) return OMEGA_GPU_FP8_CHIP_FAIL;
    for (size_t l = 0; l < S->layers && !e; l++) if (hdr[l * 8 + 4]) e = hdr[l * 8 + 4];
    if (e) {
        // a bounded wait gave up: the step's outcome is unknown, peers may still be storing into this rank. As the reference does on a
        // timeout (src/omega_gpu_session.h:27-29), the process latches: every later compute call is refused, nothing is freed.
        Lock l;
        set_error("ep stack: a bounded wait inside a kernel ran out (code %u); the process is latched", e);
        st().latched = true;
        return (int)e;
    }
    for (size_t l = 0; l < S->layers; l++) if (hdr[l * 8 + 3]) return 100 + (int)hdr[l * 8 + 3];
    return 0;
}

/* TEST ONLY. Shortens (or restores, 0) the iteration limit of the bounded cross-GPU waits of kernels launched from now on. */
void omega_gpu_moe_test_set_wait_limit(uint32_t iterations) { Lock l; st().wait_limit = iterations ? iterations : (1u << 22); }
/* TEST ONLY. Makes this rank expect `rows` more delivered input rows than its peers will ever store (layers of even index), so the next
 * step's first expert kernel waits for a row that never comes: the host-made failure for the timeout test. Synchronous. */
int omega_gpu_moe_epstack_test_expect_extra(OmegaGpuMoeEpStack *S, uint32_t rows) {
    if (!S) return OMEGA_GPU_FP8_BAD_ARGS;
    Lock l;
    if (!dev_open()) return OMEGA_GPU_FP8_CHIP_FAIL;
    unsigned long long v = 0;
    unsigned long long *base = (unsigned long long *)(S->err + 8);
    if (!cuda_ok(cudaMemcpy(&v, base, 8, cudaMemcpyDeviceToHost), "read base")) return OMEGA_GPU_FP8_CHIP_FAIL;
    v += rows;
    return cuda_ok(cudaMemcpy(base, &v, 8, cudaMemcpyHostToDevice), "write base") ? OMEGA_GPU_FP8_OK : OMEGA_GPU_FP8_CHIP_FAIL;
}

}  // extern "C"
