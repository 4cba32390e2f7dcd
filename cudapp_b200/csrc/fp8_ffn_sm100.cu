// fp8_ffn_sm100.cu: the whole expert FFN of one MoE layer in ONE persistent tcgen05 kernel:
//   gate|up grouped GEMM + SiLU gate + activation pieces  ->  down grouped GEMM,
// the two reference launches of src/omega_gpu_decode_graph.c:343-347 (gate|up GEMV group, SWIGLU, down GEMV group).
// Same MMA pipeline, operand layout and epilogues as fp8_mma_sm100.cu (see there for the mapping); what is new is the
// work list: every CTA first takes its share of the gate|up units (row tile x 128-feature pair), then down units are
// handed out through one atomic counter, so the partly filled last round of gate|up work is filled with down work and
// the kernel boundary (pipeline drain, launch, pipeline fill) between the two GEMMs is gone. A down unit of a row tile
// may start when all gate|up units of that tile have published their activation pieces: a per-tile counter in global
// memory (release by the producing epilogue, acquire + proxy fence before the TMA load that reads the pieces).
// Gate|up units never wait on down units, so the dependency cannot cycle; every wait is bounded.
#include <type_traits>
#include "internal.h"
#include "mma_common.cuh"

namespace b200 {

struct FfnArgs {
    const float *gu_scale, *dn_scale, *x_scale;   // weight scales [E][n/128][k/128]; input row scales [rows][hidden/128]
    uint8_t *qa; float *sa;                        // gated activations: pieces [PA][q_rows][inter] + scales [rows][inter/128] (written, then read)
    const uint4 *tiles; const uint32_t *header, *ymap;
    float *out;                                    // down results, row ymap[p], `hidden` floats each
    uint32_t hidden, inter, q_rows;
    uint32_t *sched;                               // [0]: next down unit; [1 + tile]: gate|up units of that tile finished (zeroed by the plan kernel)
    uint32_t *err;
    // expert parallelism (null / 0 on one GPU): wait until peers have delivered header[0] input rows past *gate_base; down results go to the
    // owning rank's buffer (row y -> rank y / rows_per_rank) and each owner's counter [ret_index] is advanced once per delivered 256-feature slice
    const unsigned long long *gate, *gate_base; const uint64_t *out_peers, *ret_counters; uint32_t rows_per_rank, ret_index; uint32_t wait_limit;
};

constexpr int FFN_THREADS = 32 * 12;              // warp group 0: TMA, MMA, scale loader, scheduler of the down units; warp groups 1 and 2: the two promotion / epilogue groups
constexpr uint32_t FFN_AHEAD = 6;                 // the scheduler takes the next down unit when the producer has this many K blocks left to issue
constexpr uint32_t FFN_RING = 64;                 // ring of published down-unit ids; the producer is never more than a few units ahead of the slowest role

template <int PX, int PA>
__global__ void __launch_bounds__(FFN_THREADS, 1) fp8_ffn_kernel(const __grid_constant__ CUtensorMap tm_gu, const __grid_constant__ CUtensorMap tm_qx,
                                                                   const __grid_constant__ CUtensorMap tm_dn, const __grid_constant__ CUtensorMap tm_qa, const FfnArgs a) {
    constexpr int PMAX = PX > PA ? PX : PA, NMAX = MMA_TOK * PMAX;
    constexpr int STAGES = PMAX <= 3 ? 4 : 3;
    constexpr uint32_t STAGE_BYTES = 2 * A_TILE + PMAX * B_PIECE;
    // TMEM partial buffers: one buffer = both 128-feature blocks of a K block (2 x 32 x pieces columns). All 512 columns are taken, so a
    // gate|up K block (narrower: PX pieces) has up to four buffers and the MMA issuer can run that far ahead of the promotion warps; the
    // buffers of the two kinds of unit overlap, so the issuer drains the gate|up buffers once, before its first down unit.
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t NBX = 512 / (64 * PX) >= 4 ? 4 : 512 / (64 * PX), NBD = 512 / (64 * PA) >= 4 ? 4 : 512 / (64 * PA);
    static_assert(NBX >= 2 && NBD >= 2, "two partial buffers at least");
    constexpr uint32_t Q_GROUP_BYTES = PA * MMA_TOK * 128;   // per epilogue group: PA pieces x 32 rows x 128 bytes of output codes
    extern __shared__ uint8_t dyn_smem[];
    __shared__ __align__(8) uint64_t s_bar[2 * STAGES + 16];
    __shared__ uint32_t s_tmem, s_abort;
    __shared__ __align__(16) float s_sc[2][2][KB_MAX][MMA_TOK];
    __shared__ float s_red[2][4][MMA_TOK];
    __shared__ uint32_t s_ymap[2][MMA_TOK];
    __shared__ volatile uint32_t s_units[FFN_RING];   // down units this CTA took, in order (slot = index % FFN_RING); 0xffffffff = no more
    __shared__ uint4 s_tile[FFN_RING];                // their tile records; an entry is published once its tile's gate|up units have all finished
    __shared__ volatile uint32_t s_published, s_prog; // entries published by the scheduler; K blocks the producer has issued
    __shared__ uint32_t s_ret[2][64];             // [epilogue group][rank]: result slices stored into that rank's buffer (expert parallel)
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t smem_base = (smem_u32(dyn_smem) + 1023u) & ~1023u;
    const uint32_t bar0 = smem_u32(s_bar);
    auto full_bar = [&](uint32_t s) { return bar0 + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar0 + 8u * (STAGES + s); };
    auto accfull_bar = [&](uint32_t b) { return bar0 + 8u * (2 * STAGES + b); };
    auto accempty_bar = [&](uint32_t b) { return bar0 + 8u * (2 * STAGES + 4 + b); };
    auto scfull_bar = [&](uint32_t b) { return bar0 + 8u * (2 * STAGES + 8 + b); };
    auto scempty_bar = [&](uint32_t b) { return bar0 + 8u * (2 * STAGES + 10 + b); };
    auto group_bar = [&](uint32_t g) { return bar0 + 8u * (2 * STAGES + 12 + g); };
    auto turn_bar = [&](uint32_t g) { return bar0 + 8u * (2 * STAGES + 14 + g); };
    volatile uint32_t *abort_flag = &s_abort;

    if (threadIdx.x < 128) s_ret[threadIdx.x >> 6][threadIdx.x & 63u] = 0;
    if (threadIdx.x == 0) {
        s_abort = 0; s_published = 0; s_prog = 0;
        for (uint32_t s = 0; s < STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (uint32_t b = 0; b < 4; b++) { mbar_init(accfull_bar(b), 1); mbar_init(accempty_bar(b), 128); }
        for (uint32_t b = 0; b < 2; b++) {
            mbar_init(scfull_bar(b), 32); mbar_init(scempty_bar(b), 128); mbar_init(group_bar(b), 128); mbar_init(turn_bar(b), 128);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    // Registers go where the promotion needs them: the three single-thread roles give theirs up, the promotion threads hold a whole K block of
    // partial sums at once, so a K block costs one TMEM round trip (two with three pieces) instead of one per piece pair.
    // 128 x 56 + 256 x 224 = 384 x 168 registers. Each warp group changes its own count inside its own branch.
    const uint32_t H = a.hidden, I = a.inter, KBX = H / 128u, KBA = I / 128u, PG = I / 128u, PD = H / 256u;
    const bool dead = *reinterpret_cast<volatile uint32_t *>(a.err) != 0;   // a failure is already recorded: do nothing
    const uint32_t n_tiles = dead ? 0u : a.header[2], n_gu = n_tiles * PG, n_dn = n_tiles * PD;
    const uint32_t my_gu = blockIdx.x < n_gu ? (n_gu - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;   // gate|up units of this CTA (static round-robin)
    // The partial buffer of this CTA's it-th K block (its gate|up K blocks come first: it < gu_kbs): buffer index, how often that buffer was
    // used before (its mbarrier phase) and its first TMEM column. Every role walks the same sequence, so all compute the same slots.
    const uint32_t gu_kbs = my_gu * KBX;
    struct Slot { uint32_t buf, use, col, half; };
    auto acc_slot = [&](uint32_t it) -> Slot {
        Slot sl;
        if (it < gu_kbs) { sl.buf = it % NBX; sl.use = it / NBX; sl.col = sl.buf * (64u * PX); sl.half = 32u * PX; }
        else { const uint32_t j = it - gu_kbs; sl.buf = j % NBD; sl.use = (gu_kbs + NBX - 1u - sl.buf) / NBX + j / NBD; sl.col = sl.buf * (64u * PA); sl.half = 32u * PA; }
        return sl;
    };

    // The n-th unit of this CTA: gate|up units first (unit id u < n_gu), then the down units the producer publishes.
    // Returns false when the CTA has no n-th unit. Only the producer fetches; the other roles read what it published.
    auto unit_at = [&](uint32_t n, uint32_t &u) -> bool {
        if (n < my_gu) { u = blockIdx.x + n * gridDim.x; return true; }
        const uint32_t i = n - my_gu;
        for (uint32_t spin = 0; s_published <= i; spin++) {
            if (spin > SPIN_LIMIT || *abort_flag) { if (!*abort_flag) { *abort_flag = 1; atomicCAS(a.err, 0u, 20u); } return false; }
            __nanosleep(20);
        }
        __threadfence_block();   // the entry (and, through the scheduler's acquire, the tile's pieces and scales) is read after the count
        const uint32_t v = s_units[i % FFN_RING];
        if (v == 0xffffffffu) return false;
        u = n_gu + v;
        return true;
    };
    // tile record of this CTA's n-th unit (after unit_at(n) returned true)
    auto tile_at = [&](uint32_t n, uint32_t tile) -> uint4 { return n < my_gu ? a.tiles[tile] : s_tile[(n - my_gu) % FFN_RING]; };
    struct Unit { uint32_t mode, tile, j, KB, r0, r1; };
    auto decode = [&](uint32_t u) -> Unit {
        Unit q;
        if (u < n_gu) { q.mode = 0; q.tile = u / PG; q.j = u % PG; q.KB = KBX; q.r0 = q.j * 128u; q.r1 = I + q.j * 128u; }
        else { const uint32_t v = u - n_gu; q.mode = 1; q.tile = v / PD; q.j = v % PD; q.KB = KBA; q.r0 = 2u * q.j * 128u; q.r1 = q.r0 + 128u; }
        return q;
    };
    // wait (bounded) until every gate|up unit of `tile` has published its activation pieces
    auto tile_ready = [&](uint32_t tile, uint32_t code) -> bool {
        const uint32_t *p = a.sched + 1 + tile;
        for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
            if (v >= PG) { asm volatile("fence.proxy.async;" ::: "memory"); return true; }
            if ((i & 255u) == 255u && *abort_flag) return false;
            __nanosleep(40);
        }
        *abort_flag = 1; atomicCAS(a.err, 0u, code);
        return false;
    };

    if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;" ::: "memory");
    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (and scheduler of the down units)
        if (lane == 0) {
            uint32_t it = 0, n = 0; bool ok = true, first = true;
            const uint64_t pol_w = l2_policy_evict_first();   // weights are read once: keep them from displacing the rows that are read again (measured: 3 % of the step)
            while (ok) {
                uint32_t u;
                if (n >= my_gu && first) { first = false; griddep_wait(); griddep_launch(); }   // no gate|up unit here: the down units come from the scheduler, which waits for the same grid
                if (!unit_at(n, u)) break;
                const Unit q = decode(u);
                const uint4 t = tile_at(n, q.tile);
                if (q.mode) asm volatile("fence.proxy.async;" ::: "memory");   // the tile's pieces were written by other SMs: the scheduler acquired them, this thread reads them through TMA
                n++;
                const CUtensorMap *mw = q.mode ? &tm_dn : &tm_gu, *mq = q.mode ? &tm_qa : &tm_qx;
                const uint32_t wn = q.mode ? H : 2u * I, P = q.mode ? (uint32_t)PA : (uint32_t)PX, bytes = 2 * A_TILE + P * B_PIECE;
                const int wy0 = (int)(t.x * wn + q.r0), wy1 = (int)(t.x * wn + q.r1);
                uint32_t kb0 = 0;
                if (first) {
                    // weights do not depend on the previous kernel: start the pipeline with weight tiles, then wait for the producer grid
                    first = false;
                    const uint32_t npre = q.KB < (uint32_t)STAGES ? q.KB : (uint32_t)STAGES;
                    for (uint32_t kb = 0; kb < npre; kb++) {
                        const uint32_t dst = smem_base + kb * STAGE_BYTES;
                        mbar_expect_tx(full_bar(kb), bytes);
                        tma_load_2d_hint(dst, mw, full_bar(kb), (int)(kb * 128u), wy0, pol_w);
                        tma_load_2d_hint(dst + A_TILE, mw, full_bar(kb), (int)(kb * 128u), wy1, pol_w);
                    }
                    griddep_wait(); griddep_launch();
                    if (a.gate && !(ok = gate_wait(a.gate, *a.gate_base + a.header[0], a.err, 13, a.wait_limit))) { *abort_flag = 1; break; }
                    for (uint32_t kb = 0; kb < npre; kb++)
                        for (uint32_t p = 0; p < P; p++)
                            tma_load_2d(smem_base + kb * STAGE_BYTES + 2 * A_TILE + p * B_PIECE, mq, full_bar(kb), (int)(kb * 128u), (int)(p * a.q_rows + t.y));
                    it = npre; kb0 = npre; s_prog = it;
                }
                for (uint32_t kb = kb0; kb < q.KB && ok; kb++, it++) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    if (!(ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, a.err, 1))) break;
                    const uint32_t dst = smem_base + s * STAGE_BYTES;
                    mbar_expect_tx(full_bar(s), bytes);
                    tma_load_2d_hint(dst, mw, full_bar(s), (int)(kb * 128u), wy0, pol_w);
                    tma_load_2d_hint(dst + A_TILE, mw, full_bar(s), (int)(kb * 128u), wy1, pol_w);
                    for (uint32_t p = 0; p < P; p++)
                        tma_load_2d(dst + 2 * A_TILE + p * B_PIECE, mq, full_bar(s), (int)(kb * 128u), (int)(p * a.q_rows + t.y));
                    s_prog = it + 1;
                }
            }
            if (first) { griddep_wait(); griddep_launch(); }   // a CTA without work still takes part in the launch chain
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t it = 0; bool ok = true;
            for (uint32_t n = 0; ok; n++) {
                uint32_t u;
                if (!unit_at(n, u)) break;
                const Unit q = decode(u);
                const uint32_t N = q.mode ? (uint32_t)(MMA_TOK * PA) : (uint32_t)(MMA_TOK * PX);
                const uint32_t idesc = (1u << 4) | ((N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);   // f8f6f4, D f32, A = B = e4m3 K-major, M 128
                if (it == gu_kbs && it != 0) {   // first down unit: its buffers overlap the gate|up ones, which must all be drained (once per launch)
                    for (uint32_t b = 0; b < NBX && ok; b++) ok = mbar_wait(accempty_bar(b), (((gu_kbs + NBX - 1u - b) / NBX) & 1u) ^ 1u, abort_flag, a.err, 2);
                    if (!ok) break;
                }
                for (uint32_t kb = 0; kb < q.KB; kb++, it++) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                    const Slot sl = acc_slot(it);
                    if (!(ok = mbar_wait(accempty_bar(sl.buf), (sl.use & 1u) ^ 1u, abort_flag, a.err, 2))) break;
                    if (!(ok = mbar_wait(full_bar(s), ph, abort_flag, a.err, 3))) break;
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * STAGE_BYTES;
                    const uint64_t da0 = umma_desc(sa), da1 = umma_desc(sa + A_TILE), db = umma_desc(sa + 2 * A_TILE);
                    const uint32_t d0 = tmem + sl.col, d1 = d0 + sl.half;
#pragma unroll
                    for (uint32_t ks = 0; ks < 4; ks++) {
                        tc_mma_f8(d0, da0 + 2u * ks, db + 2u * ks, idesc, ks);
                        tc_mma_f8(d1, da1 + 2u * ks, db + 2u * ks, idesc, ks);
                    }
                    tc_commit(empty_bar(s));
                    tc_commit(accfull_bar(sl.buf));
                }
            }
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------------- scale loader
        bool ok = true;
        griddep_wait();
        if (a.gate) { if (lane == 0 && !gate_wait(a.gate, *a.gate_base + a.header[0], a.err, 14, a.wait_limit)) *abort_flag = 1; __syncwarp(); if (*abort_flag) ok = false; }
        for (uint32_t n = 0; ok; n++) {
            uint32_t u = 0, have = 0;
            if (lane == 0) have = unit_at(n, u) ? 1u : 0u;
            have = __shfl_sync(0xffffffffu, have, 0); u = __shfl_sync(0xffffffffu, u, 0);
            __syncwarp();
            if (!have) break;
            const Unit q = decode(u);
            const uint4 t = tile_at(n, q.tile); const uint32_t b = n & 1u;
            if (!(ok = mbar_wait(scempty_bar(b), ((n >> 1) & 1u) ^ 1u, abort_flag, a.err, 7))) break;
            // the row scales of a down unit are written by this launch's gate|up units: its entry is published only after they have finished
            if (q.mode) s_ymap[b][lane] = lane < t.z ? a.ymap[t.y + lane] : 0u;
            const float *ws = q.mode ? a.dn_scale : a.gu_scale, *as = q.mode ? a.sa : a.x_scale;
            const uint32_t nb = (q.mode ? H : 2u * I) / 128u;
            const float *w0 = ws + ((size_t)t.x * nb + q.r0 / 128u) * q.KB, *w1 = ws + ((size_t)t.x * nb + q.r1 / 128u) * q.KB;
            for (uint32_t kb = 0; kb < q.KB; kb++) {
                const float cs = lane < t.z ? __ldcg(as + (size_t)(t.y + lane) * q.KB + kb) : 0.0f;
                s_sc[b][0][kb][lane] = __ldg(w0 + kb) * cs;
                s_sc[b][1][kb][lane] = __ldg(w1 + kb) * cs;
            }
            mbar_arrive(scfull_bar(b));
        }
    } else if (warp == 3) {
        // ---------------------------------------------------------------- scheduler of the down units: takes the next ticket of the layer's work list a
        // few K blocks before the producer runs out of work, fetches the tile record, waits until the tile's gate|up units have published their pieces
        // and only then publishes the entry, so that no other role pays these round trips
        if (lane == 0) {
            griddep_wait();   // the work-list words are cleared by the kernel this one depends on
            for (uint32_t i = 0;; i++) {
                const uint32_t need = gu_kbs + i * KBA;   // K blocks the producer has issued when it asks for entry i
                bool ok = true;
                for (uint32_t spin = 0; s_prog + FFN_AHEAD < need; spin++) {
                    if (spin > SPIN_LIMIT || *abort_flag) { ok = false; break; }
                    __nanosleep(64);
                }
                uint32_t v = 0xffffffffu;
                if (ok && n_dn) { v = atomicAdd(a.sched, 1u); if (v >= n_dn) v = 0xffffffffu; }
                if (v != 0xffffffffu) {
                    const uint32_t tile = v / PD;
                    const uint4 t = a.tiles[tile];
                    if (tile_ready(tile, 21)) s_tile[i % FFN_RING] = t; else v = 0xffffffffu;
                }
                s_units[i % FFN_RING] = v;
                __threadfence_block();
                s_published = i + 1;
                if (v == 0xffffffffu) break;
            }
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- promotion + epilogue: two groups of 4 warps take alternate units
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;" ::: "memory");
        const uint32_t g = (warp - 4u) >> 2, q4 = warp & 3u, row = q4 * 32u + lane, et = row;
        uint32_t it = 0, gsync = 0, turns = 0; bool ok = true;
        for (uint32_t n = 0; ok; n++) {
            uint32_t u = 0, have = 0;
            if (lane == 0) have = unit_at(n, u) ? 1u : 0u;
            have = __shfl_sync(0xffffffffu, have, 0); u = __shfl_sync(0xffffffffu, u, 0);
            if (!have) break;
            const Unit q = decode(u);
            if ((n & 1u) != g) { it += q.KB; continue; }
            if (n > 0 && !(ok = mbar_wait(turn_bar(g), turns++ & 1u, abort_flag, a.err, 9))) break;
            const uint4 t = tile_at(n, q.tile); const uint32_t cnt = t.z, b = n & 1u;
            if (!(ok = mbar_wait(scfull_bar(b), (n >> 1) & 1u, abort_flag, a.err, 8))) break;
            float acc0[MMA_TOK], acc1[MMA_TOK];
#pragma unroll
            for (int i = 0; i < MMA_TOK; i++) { acc0[i] = 0.0f; acc1[i] = 0.0f; }
            auto kloop = [&](auto pc) {
                constexpr int P = decltype(pc)::value;
                for (uint32_t kb = 0; kb < q.KB; kb++, it++) {
                    const Slot sl = acc_slot(it);
                    if (!(ok = mbar_wait(accfull_bar(sl.buf), sl.use & 1u, abort_flag, a.err, 4))) return;
                    tc_fence_after();
                    promote_kblock<P>(tmem + ((q4 * 32u) << 16) + sl.col, accempty_bar(sl.buf), &s_sc[b][0][kb][0], &s_sc[b][1][kb][0], acc0, acc1);
                }
            };
            if (q.mode) kloop(std::integral_constant<int, PA>{}); else kloop(std::integral_constant<int, PX>{});
            if (!ok) break;
            mbar_arrive(turn_bar(g ^ 1u));
            if (q.mode == 0) {
                float m[MMA_TOK];
#pragma unroll
                for (int i = 0; i < MMA_TOK; i++) { acc0[i] = silu_mul_dev(acc0[i], acc1[i]); m[i] = fabsf(acc0[i]); }
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) {
                    const bool up = (lane & (uint32_t)o) != 0;
#pragma unroll
                    for (int jj = 0; jj < o; jj++) {
                        const float keep = up ? m[jj + o] : m[jj], send = up ? m[jj] : m[jj + o];
                        m[jj] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, o));
                    }
                }
                s_red[g][q4][lane] = m[0];
                mbar_arrive(group_bar(g));
                if (!(ok = mbar_wait(group_bar(g), gsync++ & 1u, abort_flag, a.err, 5))) break;
                const float sc = pq_scale_mma(fmaxf(fmaxf(s_red[g][0][lane], s_red[g][1][lane]), fmaxf(s_red[g][2][lane], s_red[g][3][lane])));
                const float inv = __uint_as_float((254u - (__float_as_uint(sc) >> 23)) << 23);
                if (q4 == 0 && lane < cnt) a.sa[(size_t)(t.y + lane) * KBA + q.j] = sc;
                uint8_t *sq = dyn_smem + (smem_base - smem_u32(dyn_smem)) + STAGES * STAGE_BYTES + g * Q_GROUP_BYTES;
#pragma unroll
                for (int i = 0; i < MMA_TOK; i += 2) {
                    float ra = acc0[i] * __shfl_sync(0xffffffffu, inv, i), rb = acc0[i + 1] * __shfl_sync(0xffffffffu, inv, i + 1);
#pragma unroll
                    for (int p = 0; p < PA; p++) {
                        const uint32_t code = enc2(ra, rb);
                        sq[(p * MMA_TOK + i) * 128u + row] = (uint8_t)(code & 0xffu);
                        sq[(p * MMA_TOK + i + 1) * 128u + row] = (uint8_t)(code >> 8);
                        const float2 dv = dec2(code);
                        ra = (ra - dv.x) * 16.0f; rb = (rb - dv.y) * 16.0f;
                    }
                }
                mbar_arrive(group_bar(g));
                if (!(ok = mbar_wait(group_bar(g), gsync++ & 1u, abort_flag, a.err, 6))) break;
                for (uint32_t c = et; c < (uint32_t)PA * MMA_TOK * 8u; c += 128u) {
                    const uint32_t r = c >> 3, p = r / MMA_TOK, i = r - p * MMA_TOK;
                    if (i < cnt) *reinterpret_cast<uint4 *>(a.qa + ((size_t)p * a.q_rows + t.y + i) * I + q.j * 128u + (c & 7u) * 16u) = *reinterpret_cast<const uint4 *>(sq + (size_t)c * 16u);
                }
                // publish: the pieces and scales of this unit are in global memory for every SM
                __threadfence();
                mbar_arrive(group_bar(g));
                if (!(ok = mbar_wait(group_bar(g), gsync++ & 1u, abort_flag, a.err, 10))) break;
                if (et == 0) atomicAdd(a.sched + 1 + q.tile, 1u);
            } else if (!a.out_peers) {
#pragma unroll
                for (int i = 0; i < MMA_TOK; i++)
                    if ((uint32_t)i < cnt) {
                        float *o = a.out + (size_t)s_ymap[b][i] * H;
                        o[q.r0 + row] = acc0[i]; o[q.r1 + row] = acc1[i];
                    }
            } else {
#pragma unroll
                for (int i = 0; i < MMA_TOK; i++)
                    if ((uint32_t)i < cnt) {
                        const uint32_t y = s_ymap[b][i], owner = y / a.rows_per_rank;
                        float *o = reinterpret_cast<float *>(a.out_peers[owner]) + (size_t)(y - owner * a.rows_per_rank) * H;
                        o[q.r0 + row] = acc0[i]; o[q.r1 + row] = acc1[i];
                    }
                if (et < cnt) atomicAdd(&s_ret[g][s_ymap[b][et] / a.rows_per_rank], 1u);   // published once, after the last unit
            }
            mbar_arrive(scempty_bar(b));
        }
        if (a.out_peers && ok) {
            // the group's result stores are ordered before its barrier; the publishing threads fence once at system scope (cumulative) and count
            mbar_arrive(group_bar(g));
            if (mbar_wait(group_bar(g), gsync++ & 1u, abort_flag, a.err, 15) && et < 64u && s_ret[g][et]) {
                __threadfence_system();
                atomicAdd_system(reinterpret_cast<unsigned long long *>(a.ret_counters[et]) + a.ret_index, (unsigned long long)s_ret[g][et]);
            }
        }
    }
    if (*abort_flag) { for (int i = 0; i < 64; i++) __nanosleep(1000); }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

bool ffn_shape_ok(uint32_t hidden, uint32_t inter) { return hidden % 256u == 0 && inter % 128u == 0 && hidden <= 128u * KB_MAX && inter <= 128u * KB_MAX; }

cudaError_t launch_ffn(const void *tm_gu, const void *tm_qx, const void *tm_dn, const void *tm_qa, uint32_t px, uint32_t pa, const FfnLaunch &m, cudaStream_t s, bool pdl) {
    FfnArgs a = {};
    a.gu_scale = m.gu_scale; a.dn_scale = m.dn_scale; a.x_scale = m.x_scale; a.qa = m.qa; a.sa = m.sa; a.tiles = (const uint4 *)m.tiles; a.header = m.header; a.ymap = m.ymap;
    a.out = m.out; a.hidden = m.hidden; a.inter = m.inter; a.q_rows = m.q_rows; a.sched = m.sched; a.err = m.err;
    a.gate = m.gate; a.gate_base = m.gate_base; a.out_peers = m.out_peers; a.ret_counters = m.ret_counters; a.rows_per_rank = m.rows_per_rank; a.ret_index = m.ret_index; a.wait_limit = m.wait_limit ? m.wait_limit : (1u << 22);
    const int sms = st().sm_count ? st().sm_count : 148;
    const CUtensorMap *w0 = (const CUtensorMap *)tm_gu, *q0 = (const CUtensorMap *)tm_qx, *w1 = (const CUtensorMap *)tm_dn, *q1 = (const CUtensorMap *)tm_qa;
#define LAUNCH(PXV, PAV)                                                                                                                \
    do {                                                                                                                                \
        constexpr int PM = (PXV) > (PAV) ? (PXV) : (PAV);                                                                               \
        const size_t smem = (size_t)(PM <= 3 ? 4 : 3) * (2 * A_TILE + PM * B_PIECE) + 2 * (PAV) * MMA_TOK * 128 + 1024;                             \
        static bool attr = false;                                                                                                       \
        if (!attr) {                                                                                                                    \
            /* the register hand-over inside the kernel (56 / 224) balances only if every thread starts with 168: refuse anything else */ \
            cudaFuncAttributes fa; cudaError_t e = cudaFuncGetAttributes(&fa, fp8_ffn_kernel<PXV, PAV>); if (e != cudaSuccess) return e;                 \
            if (fa.numRegs != 168) { set_error("expert kernel: %d registers per thread at launch, 168 expected", fa.numRegs); return cudaErrorInvalidConfiguration; } \
            e = cudaFuncSetAttribute(fp8_ffn_kernel<PXV, PAV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; attr = true; \
        }                                                                                                                               \
        cudaLaunchConfig_t cfg = {}; cudaLaunchAttribute at[1];                                                                         \
        cfg.gridDim = dim3(sms); cfg.blockDim = dim3(FFN_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = s;                        \
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;           \
        cfg.attrs = at; cfg.numAttrs = pdl ? 1 : 0;                                                                                     \
        cudaError_t le = cudaLaunchKernelEx(&cfg, fp8_ffn_kernel<PXV, PAV>, *w0, *q0, *w1, *q1, a);                                     \
        if (le != cudaSuccess) return le;                                                                                               \
    } while (0)
    if (px == 2 && pa == 3) LAUNCH(2, 3);
    else if (px == 1 && pa == 1) LAUNCH(1, 1);
    else if (px == 2 && pa == 2) LAUNCH(2, 2);
    else return cudaErrorInvalidValue;
#undef LAUNCH
    return cudaGetLastError();
}

}  // namespace b200
