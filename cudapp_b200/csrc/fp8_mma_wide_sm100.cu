// fp8_mma_wide_sm100.cu: the grouped FP8 GEMM of fp8_mma_sm100.cu shaped for prefill-sized segments.
//
// Same arithmetic (weights as uploaded, activations as plain e4m3 with one power-of-two scale per (row, 128 columns), block-scale
// promotion per 128-wide K block in f32 registers; src/omega_blackwell_codegen_qg.h:7-37 in the reference), but the operand roles
// are the ordinary ones: a tile of 128 routed rows is the MMA's M operand, 256 weight rows (gate block j with up block j, or two
// adjacent down blocks) are the N operand. Every weight byte that reaches shared memory is used for 128 rows, and an epilogue
// thread owns one routed row: its promotion scale is one register per weight block (row scale x weight-block scale), the row
// maximum for the output quantiser needs no shuffles, and its output bytes are contiguous in memory.
//
// One persistent CTA per SM, 19 warps: TMA producer, MMA issuer, scale loader, and four groups of four promotion/epilogue warps;
// warp q of a group reads TMEM lanes [32q, 32q+32) (rows of the tile), group g owns accumulator columns [32g, 32g+32) of both weight
// blocks. A unit of work is (row tile, pair of 128-feature blocks); per 128-wide K block 4 MMAs (M 128, N 256, K 32) go into a
// double-buffered TMEM partial (2 x 256 columns = all 512), and all four groups drain it. Only single-piece activations
// (x_pieces = act_pieces = 1) take this path; k <= 2048.
//
// Every mbarrier wait is bounded; on expiry the kernel records a code in *err, lets its own copies land, frees its TMEM and returns.
#include "internal.h"
#include "mma_common.cuh"

namespace b200 {

constexpr int WIDE_GROUPS = 4;
constexpr int WIDE_ROWS = 128;                                    // routed rows per tile = TMEM lanes
constexpr int WIDE_COLS = 256;                                    // weight rows per unit = accumulator columns
constexpr int WIDE_THREADS = 32 * (3 + 4 * WIDE_GROUPS);          // 608
constexpr int WIDE_STAGES = 4;
constexpr int WIDE_KB_MAX = 16;
constexpr uint32_t WIDE_STAGE_BYTES = 2 * A_TILE + WIDE_ROWS * 128;        // 48 KB: two weight blocks + 128 activation rows
constexpr uint32_t WIDE_SA_FLOATS = 2 * WIDE_KB_MAX * WIDE_ROWS;           // [scale buffer][k block][row]
constexpr size_t WIDE_SMEM = (size_t)WIDE_STAGES * WIDE_STAGE_BYTES + WIDE_SA_FLOATS * 4 + 1024;

// one 32-byte store (sm_100: 256-bit vector access); p must be 32-byte aligned
__device__ __forceinline__ void st_v8(void *p, const uint32_t *v) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

struct WideArgs {
    const float *wscale, *ascale;
    const uint4 *tiles; const uint32_t *header;
    const uint32_t *ymap;
    float *out;                      // mode 1: y rows
    uint8_t *q_out; float *s_out;    // mode 0: gated activations as e4m3 [q_rows][inter] + scales [row][inter/128]
    uint32_t n, k, pairs, mode, inter, out_stride, q_rows;
    uint32_t *err;
};

__global__ void __launch_bounds__(WIDE_THREADS, 1) fp8_mma_wide_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_q, const WideArgs a) {
    constexpr uint32_t TMEM_COLS = 512;                                   // 2 buffers x 256 columns
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(WIDE_COLS >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);   // f8f6f4, D f32, A = B = e4m3 K-major, M 128, N 256
    extern __shared__ uint8_t dyn_smem[];
    __shared__ __align__(8) uint64_t s_bar[2 * WIDE_STAGES + 9];
    __shared__ uint32_t s_tmem, s_abort;
    __shared__ float s_sw[2][2][WIDE_KB_MAX];          // [scale buffer][weight block][k block]
    __shared__ float s_red[2][WIDE_GROUPS][WIDE_ROWS]; // [unit parity][group][row]: amax exchange between the groups of a row
    __shared__ uint32_t s_ymap[2][WIDE_ROWS];          // [scale buffer][row]: destination rows (mode 1)
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t smem_base = (smem_u32(dyn_smem) + 1023u) & ~1023u;
    uint8_t *smem_gen = dyn_smem + (smem_base - smem_u32(dyn_smem));
    float *s_sa = reinterpret_cast<float *>(smem_gen + WIDE_STAGES * WIDE_STAGE_BYTES);
    auto sa_at = [&](uint32_t b, uint32_t kb) { return s_sa + (b * WIDE_KB_MAX + kb) * WIDE_ROWS; };
    const uint32_t bar0 = smem_u32(s_bar);
    auto full_bar = [&](uint32_t s) { return bar0 + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar0 + 8u * (WIDE_STAGES + s); };
    auto accfull_bar = [&](uint32_t b) { return bar0 + 8u * (2 * WIDE_STAGES + b); };
    auto accempty_bar = [&](uint32_t b) { return bar0 + 8u * (2 * WIDE_STAGES + 2 + b); };
    auto scfull_bar = [&](uint32_t b) { return bar0 + 8u * (2 * WIDE_STAGES + 4 + b); };
    auto scempty_bar = [&](uint32_t b) { return bar0 + 8u * (2 * WIDE_STAGES + 6 + b); };
    const uint32_t all_bar = bar0 + 8u * (2 * WIDE_STAGES + 8);   // every epilogue thread
    volatile uint32_t *abort_flag = &s_abort;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (uint32_t s = 0; s < WIDE_STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (uint32_t b = 0; b < 2; b++) {
            mbar_init(accfull_bar(b), 1); mbar_init(accempty_bar(b), 128 * WIDE_GROUPS);
            mbar_init(scfull_bar(b), 32); mbar_init(scempty_bar(b), 128 * WIDE_GROUPS);
        }
        mbar_init(all_bar, 128 * WIDE_GROUPS);
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

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t it = 0; bool ok = true;
            for (uint32_t u = blockIdx.x; u < total && ok; u += gridDim.x) {
                const uint4 t = a.tiles[u / a.pairs]; const uint32_t j = u % a.pairs;
                const uint32_t r0 = a.mode == 0 ? j * 128u : 2u * j * 128u, r1 = a.mode == 0 ? a.inter + j * 128u : (2u * j + 1u) * 128u;
                const int wy0 = (int)(t.x * a.n + r0), wy1 = (int)(t.x * a.n + r1);
                for (uint32_t kb = 0; kb < KB; kb++, it++) {
                    const uint32_t s = it % WIDE_STAGES, ph = (it / WIDE_STAGES) & 1u;
                    const uint32_t dst = smem_base + s * WIDE_STAGE_BYTES;
                    if (!(ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, a.err, 1))) break;
                    mbar_expect_tx(full_bar(s), WIDE_STAGE_BYTES);
                    tma_load_2d(dst, &tm_w, full_bar(s), (int)(kb * 128u), wy0);
                    tma_load_2d(dst + A_TILE, &tm_w, full_bar(s), (int)(kb * 128u), wy1);
#pragma unroll
                    for (int g = 0; g < WIDE_ROWS / MMA_TOK; g++)   // 32 rows x 128 bytes each; rows past the segment belong to nobody and are never stored
                        tma_load_2d(dst + 2 * A_TILE + g * B_PIECE, &tm_q, full_bar(s), (int)(kb * 128u), (int)(t.y + g * MMA_TOK));
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t it = 0; bool ok = true;
            for (uint32_t u = blockIdx.x; u < total && ok; u += gridDim.x) {
                for (uint32_t kb = 0; kb < KB; kb++, it++) {
                    const uint32_t s = it % WIDE_STAGES, ph = (it / WIDE_STAGES) & 1u, buf = it & 1u, bph = (it >> 1) & 1u;
                    if (!(ok = mbar_wait(accempty_bar(buf), bph ^ 1u, abort_flag, a.err, 2))) break;
                    if (!(ok = mbar_wait(full_bar(s), ph, abort_flag, a.err, 3))) break;
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * WIDE_STAGE_BYTES;
                    const uint64_t dw = umma_desc(sa), dx = umma_desc(sa + 2 * A_TILE);   // 256 weight rows (N), 128 routed rows (M)
                    const uint32_t d = tmem + buf * WIDE_COLS;
#pragma unroll
                    for (uint32_t ks = 0; ks < 4; ks++)   // 32 K bytes per MMA: advance the start address inside the swizzle row
                        tc_mma_f8(d, dx + 2u * ks, dw + 2u * ks, IDESC, ks);
                    tc_commit(empty_bar(s));       // the stage is free once these MMAs have read it
                    tc_commit(accfull_bar(buf));   // the partial is complete
                }
            }
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------------- scale loader: next unit's scales while this one runs
        uint32_t n = 0; bool ok = true;
        const uint32_t kb_magic = 65536u / KB + 1u;
        for (uint32_t u = blockIdx.x; u < total && ok; u += gridDim.x, n++) {
            const uint4 t = a.tiles[u / a.pairs]; const uint32_t j = u % a.pairs, b = n & 1u;
            const uint32_t r0 = a.mode == 0 ? j * 128u : 2u * j * 128u, r1 = a.mode == 0 ? a.inter + j * 128u : (2u * j + 1u) * 128u;
            if (!(ok = mbar_wait(scempty_bar(b), ((n >> 1) & 1u) ^ 1u, abort_flag, a.err, 7))) break;
            // every global load of the unit is issued before the first one is used
            uint32_t ym[WIDE_ROWS / 32];
            if (a.mode == 1) {
#pragma unroll
                for (int i = 0; i < WIDE_ROWS / 32; i++) { const uint32_t r = lane + 32u * i; ym[i] = r < t.z ? a.ymap[t.y + r] : 0u; }
            }
            const float *w0 = a.wscale + ((size_t)t.x * (a.n / 128u) + r0 / 128u) * KB, *w1 = a.wscale + ((size_t)t.x * (a.n / 128u) + r1 / 128u) * KB;
            if (lane < KB) { s_sw[b][0][lane] = __ldg(w0 + lane); s_sw[b][1][lane] = __ldg(w1 + lane); }
            // the tile's row scales are one contiguous block [row][k block]: read it coalesced, store it as [k block][row]
            const float *as = a.ascale + (size_t)t.y * KB;
            const uint32_t total_sc = WIDE_ROWS * KB;
            if (a.mode == 1) {
#pragma unroll
                for (int i = 0; i < WIDE_ROWS / 32; i++) s_ymap[b][lane + 32u * i] = ym[i];
            }
            for (uint32_t base = 0; base < total_sc; base += 32u * 2u * WIDE_KB_MAX) {   // at most two passes of 32 loads per lane
                float v[2 * WIDE_KB_MAX];
#pragma unroll
                for (int i = 0; i < 2 * WIDE_KB_MAX; i++) {
                    const uint32_t idx = base + lane + 32u * i, r = (idx * kb_magic) >> 16;   // r = idx / KB (exact for idx < 2048, KB <= 16)
                    v[i] = (idx < total_sc && r < t.z) ? as[idx] : 0.0f;
                }
#pragma unroll
                for (int i = 0; i < 2 * WIDE_KB_MAX; i++) {
                    const uint32_t idx = base + lane + 32u * i, r = (idx * kb_magic) >> 16, kb = idx - r * KB;
                    if (idx < total_sc) sa_at(b, kb)[r] = v[i];
                }
            }
            mbar_arrive(scfull_bar(b));
        }
    } else {
        // ---------------------------------------------------------------- promotion + epilogue: one routed row per thread, 32 + 32 accumulator columns
        const uint32_t g = (warp - 3u) >> 2, q = warp & 3u, row = q * 32u + lane;   // q: the TMEM lane quarter this warp may read
        const uint32_t col0 = g * 32u;
        uint32_t n = 0, async = 0; bool ok = true;
        for (uint32_t u = blockIdx.x; u < total && ok; u += gridDim.x, n++) {
            const uint4 t = a.tiles[u / a.pairs]; const uint32_t j = u % a.pairs, b = n & 1u;
            const bool valid = row < t.z;
            const uint32_t r0 = a.mode == 0 ? j * 128u : 2u * j * 128u, r1 = a.mode == 0 ? a.inter + j * 128u : (2u * j + 1u) * 128u;
            if (!(ok = mbar_wait(scfull_bar(b), (n >> 1) & 1u, abort_flag, a.err, 8))) break;
            float acc0[32], acc1[32];
#pragma unroll
            for (int i = 0; i < 32; i++) { acc0[i] = 0.0f; acc1[i] = 0.0f; }
            for (uint32_t kb = 0; kb < KB; kb++) {
                const uint32_t it = n * KB + kb, buf = it & 1u, bph = (it >> 1) & 1u;
                const float rs = sa_at(b, kb)[row];                 // 0 for rows past the segment
                const float s0 = rs * s_sw[b][0][kb], s1 = rs * s_sw[b][1][kb];
                if (!(ok = mbar_wait(accfull_bar(buf), bph, abort_flag, a.err, 4))) break;
                tc_fence_after();
                const uint32_t taddr = tmem + ((q * 32u) << 16) + buf * WIDE_COLS + col0;
#pragma unroll
                for (int part = 0; part < 4; part++) {   // (weight block, 16-column half of this group's columns)
                    const int half = part >> 1, c0 = (part & 1) * 16;
                    uint32_t da[16];
                    TMEM_LD16(taddr + half * 128 + c0, da, 0);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (part == 3) { tc_fence_before(); mbar_arrive(accempty_bar(buf)); }   // this thread's share of the partial is in registers
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        if (half) acc1[c0 + i] = fmaf(__uint_as_float(da[i]), s1, acc1[c0 + i]);
                        else acc0[c0 + i] = fmaf(__uint_as_float(da[i]), s0, acc0[c0 + i]);
                    }
                }
            }
            if (!ok) break;
            if (a.mode == 0) {
                // ---- SiLU gate, then the gated activations leave as e4m3 with one scale per (row, this unit's 128 features)
                float m = 0.0f;
#pragma unroll
                for (int i = 0; i < 32; i++) { acc0[i] = silu_mul_dev(acc0[i], acc1[i]); m = fmaxf(m, fabsf(acc0[i])); }
                s_red[b][g][row] = m;
                mbar_arrive(all_bar);
                if (!(ok = mbar_wait(all_bar, async++ & 1u, abort_flag, a.err, 5))) break;
                const float sc = pq_scale_mma(fmaxf(fmaxf(s_red[b][0][row], s_red[b][1][row]), fmaxf(s_red[b][2][row], s_red[b][3][row])));
                const float inv = __uint_as_float((254u - (__float_as_uint(sc) >> 23)) << 23);
                if (valid) {
                    if (g == 0) a.s_out[(size_t)(t.y + row) * (a.inter / 128u) + j] = sc;
                    uint32_t w[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) w[i] = enc2(acc0[4 * i] * inv, acc0[4 * i + 1] * inv) | (enc2(acc0[4 * i + 2] * inv, acc0[4 * i + 3] * inv) << 16);
                    st_v8(a.q_out + (size_t)(t.y + row) * a.inter + j * 128u + col0, w);   // 32 consecutive bytes of this row: one full sector
                }
            } else if (valid) {
                float *o = a.out + (size_t)s_ymap[b][row] * a.out_stride;
                // a thread's 32 + 32 results are two runs of 128 consecutive bytes of its destination row: whole 32-byte sectors per store
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    st_v8(o + r0 + col0 + 8 * i, reinterpret_cast<const uint32_t *>(acc0 + 8 * i));
                    st_v8(o + r1 + col0 + 8 * i, reinterpret_cast<const uint32_t *>(acc1 + 8 * i));
                }
            }
            mbar_arrive(scempty_bar(b));   // this unit's scales and destination rows may be overwritten
        }
    }
    // ---------------------------------------------------------------- teardown
    if (*abort_flag) { for (int i = 0; i < 64; i++) __nanosleep(1000); }   // let copies already issued land before the CTA goes away
    tc_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

uint32_t mma_wide_tile_rows() { return WIDE_ROWS; }
bool mma_wide_shape_ok(uint32_t n, uint32_t k, uint32_t mode) { return k % 128u == 0 && k <= 128u * WIDE_KB_MAX && n % 256u == 0 && (mode == 1 || (n / 2u) % 128u == 0); }

cudaError_t launch_mma_wide(const void *tm_w, const void *tm_q, const MmaLaunch &m, cudaStream_t s) {
    WideArgs a = {};
    a.wscale = m.wscale; a.ascale = m.ascale; a.tiles = (const uint4 *)m.tiles; a.header = m.header; a.ymap = m.ymap; a.out = m.out;
    a.q_out = m.q_out; a.s_out = m.s_out; a.q_rows = m.q_rows;
    a.n = m.n; a.k = m.k; a.mode = m.mode; a.inter = m.n / 2u; a.pairs = m.n / 256u; a.out_stride = m.out_stride; a.err = m.err;
    static bool attr = false;
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(fp8_mma_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WIDE_SMEM);
        if (e != cudaSuccess) return e;
        attr = true;
    }
    const int sms = st().sm_count ? st().sm_count : 148;
    fp8_mma_wide_kernel<<<sms, WIDE_THREADS, WIDE_SMEM, s>>>(*(const CUtensorMap *)tm_w, *(const CUtensorMap *)tm_q, a);
    return cudaGetLastError();
}

}  // namespace b200
