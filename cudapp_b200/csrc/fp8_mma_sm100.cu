// fp8_mma_sm100.cu: grouped FP8 GEMM on the B200 tensor cores (tcgen05, kind::f8f6f4) for the MoE expert path.
//
// What it computes is the reference's grouped GEMM (src/omega_blackwell_codegen_gemm.h:5-14; block-scale promotion
// as its QMMA path does it, src/omega_blackwell_codegen_qg.h:24-37): for a segment of rows routed to one expert,
//   y[row][f] = sum over 128-column blocks kb of  Sw[f/128][kb] * Sa[row][kb] * sum_c W[f][c] * A[row][c]
// with W the e4m3 weights exactly as uploaded (no repack, no conversion) and A the activations as e4m3 "pieces".
//
// Mapping ("swap-AB"): the weight tile is the MMA's M operand (128 output features x 128 K bytes straight from a
// TMA load of the checkpoint-order tensor, SWIZZLE_128B), the routed rows are the N operand (up to 64 columns of
// activation pieces). So the work per weight byte does not depend on how few rows an expert received: decode is a
// pure weight stream. An activation value is held as P e4m3 pieces (piece p = the residual left by pieces < p,
// scaled by 16^p; P = 2 represents a bf16 value exactly, P = 3 gives 12 significant bits of an f32), each piece a
// separate MMA column; columns are folded back (Horner, factor 1/16) when the accumulator is read.
//
// One persistent CTA per SM, 12 warps in three warp groups: warp 0 = TMA producer, warp 1 = MMA issuer (one elected lane each, the
// tcgen05 model), warp 2 = scale loader, warp 3 idle; warps 4-11 = two promotion/epilogue groups of four warps (one TMEM lane quarter
// each) that take alternate units. After the set-up the first warp group gives registers to the other two (setmaxnreg 56 / 224), so that a
// promotion thread can hold a whole K block of partial sums and fetch it from TMEM in one round trip. A unit of work is (row tile, pair of
// 128-feature blocks): gate block j with up block j (SiLU gate fused in the epilogue) or two adjacent down blocks.
// Per 128-wide K block: 2 x 4 MMAs (K = 32 each) into a double-buffered TMEM partial, tcgen05.commit, then the
// epilogue warps tcgen05.ld the partial and add scale * partial into register accumulators while the next block's
// MMAs run. Shared memory: 4 stages x (2 weight tiles 16 KB + activation tile 8 KB).
//
// Every mbarrier wait is bounded; on expiry the kernel records a code in *err, lets its own copies land, frees its
// TMEM and returns (no trap, no endless spin).
#include "internal.h"
#include "mma_common.cuh"

namespace b200 {

struct MmaArgs {
    const float *wscale, *ascale;
    const uint4 *tiles; const uint32_t *header;
    const uint32_t *ymap;
    float *out;                      // mode 1: y rows; mode 0: optional f32 copy of the gated activations (may be null)
    uint8_t *q_out; float *s_out;    // mode 0: gated activations as e4m3 pieces [piece][q_rows][inter] + scales [row][inter/128]
    uint32_t n, k, pairs, mode, inter, out_stride, q_rows, q_pieces;
    uint32_t *err;
    // expert parallelism (all null / 0 on one GPU)
    const unsigned long long *gate;     // rows that peers have delivered into the input pieces; the kernel waits for header[0] of them
    const uint64_t *out_peers;          // mode 1: base address of every rank's result buffer; row y belongs to rank y / rows_per_rank
    const uint64_t *ret_counters;       // mode 1: address of every rank's "result slices delivered" counter
    uint32_t rows_per_rank, ret_index;  // ret_index: which counter of the owner's counter block this launch advances
    const unsigned long long *gate_base; // rows delivered through `gate` before this layer (counters only ever grow)
    unsigned long long *bump;           // a base to advance by header[0] (the gate|up GEMM of this layer has consumed those rows)
    uint32_t wait_limit;                // iterations of the bounded wait on `gate`
};

constexpr int GRP_THREADS = 32 * 12;   // warp group 0: TMA, MMA, scale loader, one idle warp; warp groups 1 and 2: the two promotion / epilogue groups

template <int P>
__global__ void __launch_bounds__(GRP_THREADS, 1) fp8_mma_grouped_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_q, const MmaArgs a) {
    constexpr int N = MMA_TOK * P;                                   // accumulator columns per weight tile
    constexpr int STAGES = P <= 3 ? 4 : 3;
    constexpr uint32_t STAGE_BYTES = 2 * A_TILE + P * B_PIECE;
    constexpr uint32_t TMEM_COLS = 4 * N <= 128 ? 128 : 4 * N <= 256 ? 256 : 512;   // 2 buffers x 2 accumulators x N
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);   // f8f6f4, D f32, A = B = e4m3 K-major, M 128
    extern __shared__ uint8_t dyn_smem[];
    __shared__ __align__(8) uint64_t s_bar[2 * STAGES + 12];
    __shared__ uint32_t s_tmem, s_abort;
    __shared__ __align__(16) float s_sc[2][2][KB_MAX][MMA_TOK]; // [scale buffer][weight tile][k block][row] = weight scale x row scale
    __shared__ float s_red[2][4][MMA_TOK];        // [epilogue group][warp][row]: amax exchange
    __shared__ uint32_t s_ymap[2][MMA_TOK];       // [scale buffer][row]: destination rows (mode 1)
    __shared__ uint32_t s_ret[2][64];             // [epilogue group][rank]: result slices stored into that rank's buffer (expert parallel)
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t smem_base = (smem_u32(dyn_smem) + 1023u) & ~1023u;
    const uint32_t bar0 = smem_u32(s_bar);
    auto full_bar = [&](uint32_t s) { return bar0 + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar0 + 8u * (STAGES + s); };
    auto accfull_bar = [&](uint32_t b) { return bar0 + 8u * (2 * STAGES + b); };
    auto accempty_bar = [&](uint32_t b) { return bar0 + 8u * (2 * STAGES + 2 + b); };
    auto scfull_bar = [&](uint32_t b) { return bar0 + 8u * (2 * STAGES + 4 + b); };
    auto scempty_bar = [&](uint32_t b) { return bar0 + 8u * (2 * STAGES + 6 + b); };
    auto group_bar = [&](uint32_t g) { return bar0 + 8u * (2 * STAGES + 8 + g); };
    auto turn_bar = [&](uint32_t g) { return bar0 + 8u * (2 * STAGES + 10 + g); };   // "the other group has drained its unit's partials"
    volatile uint32_t *abort_flag = &s_abort;

    if (threadIdx.x < 128) s_ret[threadIdx.x >> 6][threadIdx.x & 63u] = 0;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (uint32_t s = 0; s < STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (uint32_t b = 0; b < 2; b++) {
            mbar_init(accfull_bar(b), 1); mbar_init(accempty_bar(b), 128);
            mbar_init(scfull_bar(b), 32); mbar_init(scempty_bar(b), 128); mbar_init(group_bar(b), 128); mbar_init(turn_bar(b), 128);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // TMEM allocation by one whole warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t KB = a.k / 128u, n_tiles = a.header[2], total = *reinterpret_cast<volatile uint32_t *>(a.err) ? 0u : n_tiles * a.pairs;   // after a recorded failure: no work

    // registers go where the promotion needs them (128 x 56 + 256 x 224 = 384 x 168); each warp group changes its own count inside its own branch
    if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;" ::: "memory");
    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            // The weights do not depend on the previous kernel, the activation pieces do: fill the pipeline with weight tiles
            // first, then wait for the producer grid, then add the activation tiles of those same stages.
            uint32_t it = 0; bool ok = true;
            const uint64_t pol_w = l2_policy_evict_first();   // weights are read once per launch
            for (int phase = 0; phase < 3 && ok; phase++) {
                if (phase == 1) {
                    griddep_wait(); griddep_launch();
                    if (a.bump && blockIdx.x == 0) *a.bump += a.header[0];
                    if (a.gate && !(ok = gate_wait(a.gate, *a.gate_base + a.header[0], a.err, 13, a.wait_limit))) { *abort_flag = 1; break; }
                }
                it = phase == 2 ? STAGES : 0;
                uint32_t seen = 0;
                for (uint32_t u = blockIdx.x; u < total && ok; u += gridDim.x) {
                    if (phase < 2 && seen >= STAGES) break;
                    if (phase == 2 && seen + KB <= STAGES) { seen += KB; continue; }
                    const uint4 t = a.tiles[u / a.pairs]; const uint32_t j = u % a.pairs;
                    const uint32_t r0 = a.mode == 0 ? j * 128u : 2u * j * 128u, r1 = a.mode == 0 ? a.inter + j * 128u : (2u * j + 1u) * 128u;
                    const int wy0 = (int)(t.x * a.n + r0), wy1 = (int)(t.x * a.n + r1);
                    for (uint32_t kb = 0; kb < KB; kb++, seen++) {
                        if (phase < 2 && seen >= STAGES) break;
                        if (phase == 2 && seen < STAGES) continue;
                        const uint32_t g_it = seen, s = g_it % STAGES, ph = (g_it / STAGES) & 1u;
                        const uint32_t dst = smem_base + s * STAGE_BYTES;
                        if (phase == 2 && !(ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, a.err, 1))) break;
                        if (phase != 1) {
                            mbar_expect_tx(full_bar(s), STAGE_BYTES);
                            tma_load_2d_hint(dst, &tm_w, full_bar(s), (int)(kb * 128u), wy0, pol_w);
                            tma_load_2d_hint(dst + A_TILE, &tm_w, full_bar(s), (int)(kb * 128u), wy1, pol_w);
                        }
                        if (phase != 0) {
#pragma unroll
                            for (int p = 0; p < P; p++)   // piece p of the tile's rows: 32 rows x 128 bytes
                                tma_load_2d(dst + 2 * A_TILE + p * B_PIECE, &tm_q, full_bar(s), (int)(kb * 128u), (int)(p * a.q_rows + t.y));
                        }
                    }
                }
            }
            (void)it;
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t it = 0; bool ok = true;
            for (uint32_t u = blockIdx.x; u < total && ok; u += gridDim.x) {
                for (uint32_t kb = 0; kb < KB; kb++, it++) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u, buf = it & 1u, bph = (it >> 1) & 1u;
                    if (!(ok = mbar_wait(accempty_bar(buf), bph ^ 1u, abort_flag, a.err, 2))) break;
                    if (!(ok = mbar_wait(full_bar(s), ph, abort_flag, a.err, 3))) break;
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * STAGE_BYTES;
                    const uint64_t da0 = umma_desc(sa), da1 = umma_desc(sa + A_TILE), db = umma_desc(sa + 2 * A_TILE);
                    const uint32_t d0 = tmem + buf * 2u * N, d1 = d0 + N;
#pragma unroll
                    for (uint32_t ks = 0; ks < 4; ks++) {   // 32 K bytes per MMA: advance the start address inside the swizzle row
                        tc_mma_f8(d0, da0 + 2u * ks, db + 2u * ks, IDESC, ks);
                        tc_mma_f8(d1, da1 + 2u * ks, db + 2u * ks, IDESC, ks);
                    }
                    tc_commit(empty_bar(s));       // the stage is free once these MMAs have read it
                    tc_commit(accfull_bar(buf));   // the partial is complete
                }
            }
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------------- scale loader: next unit's scales while this one runs
        uint32_t n = 0; bool ok = true;
        griddep_wait();   // the row scales below are the previous kernel's output
        if (a.gate) { if (lane == 0 && !gate_wait(a.gate, *a.gate_base + a.header[0], a.err, 14, a.wait_limit)) *abort_flag = 1; __syncwarp(); if (*abort_flag) ok = false; }
        for (uint32_t u = blockIdx.x; u < total && ok; u += gridDim.x, n++) {
            const uint4 t = a.tiles[u / a.pairs]; const uint32_t j = u % a.pairs, b = n & 1u;
            const uint32_t r0 = a.mode == 0 ? j * 128u : 2u * j * 128u, r1 = a.mode == 0 ? a.inter + j * 128u : (2u * j + 1u) * 128u;
            if (!(ok = mbar_wait(scempty_bar(b), ((n >> 1) & 1u) ^ 1u, abort_flag, a.err, 7))) break;
            if (a.mode == 1) s_ymap[b][lane] = lane < t.z ? a.ymap[t.y + lane] : 0u;
            const float *w0 = a.wscale + ((size_t)t.x * (a.n / 128u) + r0 / 128u) * KB, *w1 = a.wscale + ((size_t)t.x * (a.n / 128u) + r1 / 128u) * KB;
            for (uint32_t kb = 0; kb < KB; kb++) {
                const float cs = lane < t.z ? a.ascale[(size_t)(t.y + lane) * KB + kb] : 0.0f;
                s_sc[b][0][kb][lane] = __ldg(w0 + kb) * cs;
                s_sc[b][1][kb][lane] = __ldg(w1 + kb) * cs;
            }
            mbar_arrive(scfull_bar(b));
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- promotion + epilogue: two groups of 4 warps take alternate units
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;" ::: "memory");
        const uint32_t g = (warp - 4u) >> 2, q = warp & 3u, row = q * 32u + lane;   // q: the TMEM lane quarter this warp may read
        uint32_t n = 0, gsync = 0, turns = 0; bool ok = true;
        for (uint32_t u = blockIdx.x; u < total && ok; u += gridDim.x, n++) {
            if ((n & 1u) != g) continue;
            // partial sums are consumed strictly in order: start only when the other group has taken the last partial of unit n-1
            // (a parity wait can only tell the next phase from the current one, never a later one)
            if (n > 0 && !(ok = mbar_wait(turn_bar(g), turns++ & 1u, abort_flag, a.err, 9))) break;
            const uint4 t = a.tiles[u / a.pairs]; const uint32_t j = u % a.pairs, cnt = t.z, b = n & 1u;
            const uint32_t r0 = a.mode == 0 ? j * 128u : 2u * j * 128u, r1 = a.mode == 0 ? a.inter + j * 128u : (2u * j + 1u) * 128u;
            if (!(ok = mbar_wait(scfull_bar(b), (n >> 1) & 1u, abort_flag, a.err, 8))) break;
            float acc0[MMA_TOK], acc1[MMA_TOK];
#pragma unroll
            for (int i = 0; i < MMA_TOK; i++) { acc0[i] = 0.0f; acc1[i] = 0.0f; }
            for (uint32_t kb = 0; kb < KB; kb++) {
                const uint32_t it = n * KB + kb, buf = it & 1u, bph = (it >> 1) & 1u;
                if (!(ok = mbar_wait(accfull_bar(buf), bph, abort_flag, a.err, 4))) break;
                tc_fence_after();
                promote_kblock<P>(tmem + ((q * 32u) << 16) + buf * 2u * N, accempty_bar(buf), &s_sc[b][0][kb][0], &s_sc[b][1][kb][0], acc0, acc1);
            }
            if (!ok) break;
            mbar_arrive(turn_bar(g ^ 1u));   // the other group may start on the next unit's partials
            if (a.mode == 0) {
                // ---- SiLU gate, then the gated activations leave as e4m3 pieces with one scale per (row, this unit's 128 features)
                float m[MMA_TOK];
#pragma unroll
                for (int i = 0; i < MMA_TOK; i++) { acc0[i] = silu_mul_dev(acc0[i], acc1[i]); m[i] = fabsf(acc0[i]); }
                // per-row maximum over the warp's 32 features: butterfly that halves the rows kept per lane (31 shuffles, lane l ends with row l)
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) {
                    const bool up = (lane & (uint32_t)o) != 0;
#pragma unroll
                    for (int jj = 0; jj < o; jj++) {
                        const float keep = up ? m[jj + o] : m[jj], send = up ? m[jj] : m[jj + o];
                        m[jj] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, o));
                    }
                }
                s_red[g][q][lane] = m[0];
                mbar_arrive(group_bar(g));
                if (!(ok = mbar_wait(group_bar(g), gsync++ & 1u, abort_flag, a.err, 5))) break;
                // lane = row: maximum over the four warps, power-of-two scale and its exact reciprocal
                const float sc = pq_scale_mma(fmaxf(fmaxf(s_red[g][0][lane], s_red[g][1][lane]), fmaxf(s_red[g][2][lane], s_red[g][3][lane])));
                const float inv = __uint_as_float((254u - (__float_as_uint(sc) >> 23)) << 23);
                if (q == 0 && lane < cnt) a.s_out[(size_t)(t.y + lane) * (a.inter / 128u) + j] = sc;
                uint8_t *sq = dyn_smem + (smem_base - smem_u32(dyn_smem)) + STAGES * STAGE_BYTES + g * (Q_STAGE_BYTES / 2);   // [piece][row][128]
#pragma unroll
                for (int i = 0; i < MMA_TOK; i += 2) {
                    float ra = acc0[i] * __shfl_sync(0xffffffffu, inv, i), rb = acc0[i + 1] * __shfl_sync(0xffffffffu, inv, i + 1);
                    for (uint32_t p = 0; p < a.q_pieces; p++) {
                        const uint32_t code = enc2(ra, rb);
                        sq[(p * MMA_TOK + i) * 128u + row] = (uint8_t)(code & 0xffu);
                        sq[(p * MMA_TOK + i + 1) * 128u + row] = (uint8_t)(code >> 8);
                        const float2 dv = dec2(code);
                        ra = (ra - dv.x) * 16.0f; rb = (rb - dv.y) * 16.0f;
                    }
                }
                mbar_arrive(group_bar(g));
                if (!(ok = mbar_wait(group_bar(g), gsync++ & 1u, abort_flag, a.err, 6))) break;
                // copy out: every (piece, row) is 128 consecutive bytes in memory; 16 bytes per thread per step
                const uint32_t et = row;
                for (uint32_t c = et; c < a.q_pieces * MMA_TOK * 8u; c += 128u) {
                    const uint32_t r = c >> 3, p = r / MMA_TOK, i = r - p * MMA_TOK;
                    if (i < cnt) *reinterpret_cast<uint4 *>(a.q_out + ((size_t)p * a.q_rows + t.y + i) * a.inter + j * 128u + (c & 7u) * 16u) = *reinterpret_cast<const uint4 *>(sq + (size_t)c * 16u);
                }
                if (a.out) {
#pragma unroll
                    for (int i = 0; i < MMA_TOK; i++) if ((uint32_t)i < cnt) a.out[(size_t)(t.y + i) * a.out_stride + j * 128u + row] = acc0[i];
                }
            } else if (!a.out_peers) {
#pragma unroll
                for (int i = 0; i < MMA_TOK; i++)
                    if ((uint32_t)i < cnt) {
                        float *o = a.out + (size_t)s_ymap[b][i] * a.out_stride;
                        o[r0 + row] = acc0[i]; o[r1 + row] = acc1[i];
                    }
            } else {
                // expert parallel: every result row goes straight into its owner's buffer (peer stores), then the owner's counter
                // is advanced once per delivered 256-feature slice
#pragma unroll
                for (int i = 0; i < MMA_TOK; i++)
                    if ((uint32_t)i < cnt) {
                        const uint32_t y = s_ymap[b][i], owner = y / a.rows_per_rank;
                        float *o = reinterpret_cast<float *>(a.out_peers[owner]) + (size_t)(y - owner * a.rows_per_rank) * a.out_stride;
                        o[r0 + row] = acc0[i]; o[r1 + row] = acc1[i];
                    }
                const uint32_t et = row;
                if (et < cnt) atomicAdd(&s_ret[g][s_ymap[b][et] / a.rows_per_rank], 1u);   // published once, after the last unit
            }
            mbar_arrive(scempty_bar(b));   // this unit's scales and destination rows may be overwritten
        }
        if (a.out_peers && ok) {
            // all result rows of this group are stored and ordered before the group's barrier: the publishing threads fence once at system scope
            // (a fence is cumulative) and advance each owner's counter once
            mbar_arrive(group_bar(g));
            if (mbar_wait(group_bar(g), gsync++ & 1u, abort_flag, a.err, 15)) {
                const uint32_t et = row;
                if (et < 64u && s_ret[g][et]) __threadfence_system();
                if (et < 64u && s_ret[g][et]) atomicAdd_system(reinterpret_cast<unsigned long long *>(a.ret_counters[et]) + a.ret_index, (unsigned long long)s_ret[g][et]);
            }
        }
    }
    // ---------------------------------------------------------------- teardown
    if (*abort_flag) { for (int i = 0; i < 64; i++) __nanosleep(1000); }   // let copies already issued land before the CTA goes away
    tc_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr; cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
    }
    return fn;
}
// 2-D map over a row-major u8 matrix [rows][cols], box [box_rows][128 bytes], 128-byte swizzle
bool make_tmap_u8(void *out_map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return false; }
    const cuuint64_t dims[2] = {cols, rows}, strides[1] = {cols};
    const cuuint32_t box[2] = {128, box_rows}, estr[2] = {1, 1};
    const CUresult r = fn((CUtensorMap *)out_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return false; }
    return true;
}

uint32_t mma_tile_rows(uint32_t) { return MMA_TOK; }
bool mma_shape_ok(uint32_t n, uint32_t k, uint32_t mode) { return k % 128u == 0 && k <= 128u * KB_MAX && n % 128u == 0 && (mode == 0 || (n / 128u) % 2u == 0); }

cudaError_t launch_mma_grouped(const void *tm_w, const void *tm_q, uint32_t pieces, const MmaLaunch &m, cudaStream_t s, bool pdl) {
    MmaArgs a = {};
    a.wscale = m.wscale; a.ascale = m.ascale; a.tiles = (const uint4 *)m.tiles; a.header = m.header; a.ymap = m.ymap; a.out = m.out;
    a.q_out = m.q_out; a.s_out = m.s_out; a.q_rows = m.q_rows; a.q_pieces = m.q_pieces;
    a.gate = m.gate; a.out_peers = m.out_peers; a.ret_counters = m.ret_counters; a.rows_per_rank = m.rows_per_rank; a.ret_index = m.ret_index; a.gate_base = m.gate_base; a.bump = m.bump; a.wait_limit = m.wait_limit ? m.wait_limit : (1u << 22);
    a.n = m.n; a.k = m.k; a.mode = m.mode; a.inter = m.n / 2u; a.pairs = m.n / 256u; a.out_stride = m.out_stride; a.err = m.err;
    const int sms = st().sm_count ? st().sm_count : 148;
    const CUtensorMap *w = (const CUtensorMap *)tm_w, *q = (const CUtensorMap *)tm_q;
#define LAUNCH(PV)                                                                                                                      \
    do {                                                                                                                                \
        const size_t smem = (size_t)((PV) <= 3 ? 4 : 3) * (2 * A_TILE + (PV) * B_PIECE) + Q_STAGE_BYTES + 1024;                                        \
        static bool attr = false;                                                                                                       \
        if (!attr) {                                                                                                                    \
            /* the register hand-over inside the kernel (56 / 224) balances only if every thread starts with 168: refuse anything else */ \
            cudaFuncAttributes fa; cudaError_t e = cudaFuncGetAttributes(&fa, fp8_mma_grouped_kernel<PV>); if (e != cudaSuccess) return e;                 \
            if (fa.numRegs != 168) { set_error("grouped kernel: %d registers per thread at launch, 168 expected", fa.numRegs); return cudaErrorInvalidConfiguration; } \
            e = cudaFuncSetAttribute(fp8_mma_grouped_kernel<PV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; attr = true; \
        }                                                                                                                               \
        cudaLaunchConfig_t cfg = {}; cudaLaunchAttribute at[1];                                                                         \
        cfg.gridDim = dim3(sms); cfg.blockDim = dim3(GRP_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = s;                        \
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;           \
        cfg.attrs = at; cfg.numAttrs = pdl ? 1 : 0;                                                                                     \
        cudaError_t le = cudaLaunchKernelEx(&cfg, fp8_mma_grouped_kernel<PV>, *w, *q, a);                                              \
        if (le != cudaSuccess) return le;                                                                                               \
    } while (0)
    switch (pieces) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 3: LAUNCH(3); break;
    case 4: LAUNCH(4); break;
    default: return cudaErrorInvalidValue;
    }
#undef LAUNCH
    return cudaGetLastError();
}

}  // namespace b200
