// fp8_mma_wide8_sm100.cu: a variant of the prefill-shaped grouped GEMM (fp8_mma_wide_sm100.cu, same arithmetic, same operand roles, same
// tiles) with eight promotion warps instead of sixteen. The promotion is what bounds that kernel: at 96 registers a thread stages 16
// accumulator columns per tcgen05.ld and pays four dependent TMEM round trips per 128-wide K block. Here the CTA has three warpgroups
// (roles: TMA producer, MMA issuer, scale loader, one idle warp; two promotion warpgroups) and reallocates registers between them
// (setmaxnreg: 64 for the role warps, 216 for the promotion warps; a register-file quarter then holds 64 + 2 x 216 per lane), so a promotion thread holds 64 + 64 accumulators and stages 64
// columns at once: two round trips per K block. Selected only on request (B200MOE_WIDE8 in the environment when the layer is created); not the default: it matches the sixteen-warp
// kernel's results on a B200 but has not been timed against it.
#include "internal.h"
#include "mma_common.cuh"

namespace b200 {

constexpr int WIDE8_GROUPS = 2;
constexpr int WIDE8_ROWS = 128;                                    // routed rows per tile = TMEM lanes
constexpr int WIDE8_COLS = 256;                                    // weight rows per unit = accumulator columns
constexpr int WIDE8_THREADS = 32 * (4 + 4 * WIDE8_GROUPS);          // 384: role warpgroup (TMA, MMA, scales, idle) + two promotion warpgroups
constexpr int WIDE8_GCOLS = 128 / WIDE8_GROUPS;                     // columns of each weight block per promotion thread
constexpr int WIDE8_STAGES = 4;
constexpr int WIDE8_KB_MAX = 16;
constexpr uint32_t WIDE8_STAGE_BYTES = 2 * A_TILE + WIDE8_ROWS * 128;        // 48 KB: two weight blocks + 128 activation rows
constexpr uint32_t WIDE8_SA_FLOATS = 2 * WIDE8_KB_MAX * WIDE8_ROWS;           // [scale buffer][k block][row]
constexpr size_t WIDE8_SMEM = (size_t)WIDE8_STAGES * WIDE8_STAGE_BYTES + WIDE8_SA_FLOATS * 4 + 1024;

// one 32-byte store (sm_100: 256-bit vector access); p must be 32-byte aligned
__device__ __forceinline__ void st8_v8(void *p, const uint32_t *v) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

#define TMEM8_LD64(taddr, r)                                                                                                              \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"          \
                 "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"                                  \
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),  \
                   "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),      \
                   "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),      \
                   "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]),      \
                   "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])                                   \
                 : "r"(taddr))

struct Wide8Args {
    const float *wscale, *ascale;
    const uint4 *tiles; const uint32_t *header;
    const uint32_t *ymap;
    float *out;                      // mode 1: y rows
    uint8_t *q_out; float *s_out;    // mode 0: gated activations as e4m3 [q_rows][inter] + scales [row][inter/128]
    uint32_t n, k, pairs, mode, inter, out_stride, q_rows;
    uint32_t *err;
};

__global__ void __launch_bounds__(WIDE8_THREADS, 1) fp8_mma_wide8_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_q, const Wide8Args a) {
    constexpr uint32_t TMEM_COLS = 512;                                   // 2 buffers x 256 columns
    constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(WIDE8_COLS >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);   // f8f6f4, D f32, A = B = e4m3 K-major, M 128, N 256
    extern __shared__ uint8_t dyn_smem[];
    __shared__ __align__(8) uint64_t s_bar[2 * WIDE8_STAGES + 9];
    __shared__ uint32_t s_tmem, s_abort;
    __shared__ float s_sw[2][2][WIDE8_KB_MAX];          // [scale buffer][weight block][k block]
    __shared__ float s_red[2][WIDE8_GROUPS][WIDE8_ROWS]; // [unit parity][group][row]: amax exchange between the groups of a row
    __shared__ uint32_t s_ymap[2][WIDE8_ROWS];          // [scale buffer][row]: destination rows (mode 1)
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t smem_base = (smem_u32(dyn_smem) + 1023u) & ~1023u;
    uint8_t *smem_gen = dyn_smem + (smem_base - smem_u32(dyn_smem));
    float *s_sa = reinterpret_cast<float *>(smem_gen + WIDE8_STAGES * WIDE8_STAGE_BYTES);
    auto sa_at = [&](uint32_t b, uint32_t kb) { return s_sa + (b * WIDE8_KB_MAX + kb) * WIDE8_ROWS; };
    const uint32_t bar0 = smem_u32(s_bar);
    auto full_bar = [&](uint32_t s) { return bar0 + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar0 + 8u * (WIDE8_STAGES + s); };
    auto accfull_bar = [&](uint32_t b) { return bar0 + 8u * (2 * WIDE8_STAGES + b); };
    auto accempty_bar = [&](uint32_t b) { return bar0 + 8u * (2 * WIDE8_STAGES + 2 + b); };
    auto scfull_bar = [&](uint32_t b) { return bar0 + 8u * (2 * WIDE8_STAGES + 4 + b); };
    auto scempty_bar = [&](uint32_t b) { return bar0 + 8u * (2 * WIDE8_STAGES + 6 + b); };
    const uint32_t all_bar = bar0 + 8u * (2 * WIDE8_STAGES + 8);   // every epilogue thread
    volatile uint32_t *abort_flag = &s_abort;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (uint32_t s = 0; s < WIDE8_STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (uint32_t b = 0; b < 2; b++) {
            mbar_init(accfull_bar(b), 1); mbar_init(accempty_bar(b), 128 * WIDE8_GROUPS);
            mbar_init(scfull_bar(b), 32); mbar_init(scempty_bar(b), 128 * WIDE8_GROUPS);
        }
        mbar_init(all_bar, 128 * WIDE8_GROUPS);
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

    // register reallocation between the warpgroups: the role warps need few, a promotion thread holds 128 accumulators + 64 staged columns
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t it = 0; bool ok = true;
            for (uint32_t u = blockIdx.x; u < total && ok; u += gridDim.x) {
                const uint4 t = a.tiles[u / a.pairs]; const uint32_t j = u % a.pairs;
                const uint32_t r0 = a.mode == 0 ? j * 128u : 2u * j * 128u, r1 = a.mode == 0 ? a.inter + j * 128u : (2u * j + 1u) * 128u;
                const int wy0 = (int)(t.x * a.n + r0), wy1 = (int)(t.x * a.n + r1);
                for (uint32_t kb = 0; kb < KB; kb++, it++) {
                    const uint32_t s = it % WIDE8_STAGES, ph = (it / WIDE8_STAGES) & 1u;
                    const uint32_t dst = smem_base + s * WIDE8_STAGE_BYTES;
                    if (!(ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, a.err, 1))) break;
                    mbar_expect_tx(full_bar(s), WIDE8_STAGE_BYTES);
                    tma_load_2d(dst, &tm_w, full_bar(s), (int)(kb * 128u), wy0);
                    tma_load_2d(dst + A_TILE, &tm_w, full_bar(s), (int)(kb * 128u), wy1);
#pragma unroll
                    for (int g = 0; g < WIDE8_ROWS / MMA_TOK; g++)   // 32 rows x 128 bytes each; rows past the segment belong to nobody and are never stored
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
                    const uint32_t s = it % WIDE8_STAGES, ph = (it / WIDE8_STAGES) & 1u, buf = it & 1u, bph = (it >> 1) & 1u;
                    if (!(ok = mbar_wait(accempty_bar(buf), bph ^ 1u, abort_flag, a.err, 2))) break;
                    if (!(ok = mbar_wait(full_bar(s), ph, abort_flag, a.err, 3))) break;
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * WIDE8_STAGE_BYTES;
                    const uint64_t dw = umma_desc(sa), dx = umma_desc(sa + 2 * A_TILE);   // 256 weight rows (N), 128 routed rows (M)
                    const uint32_t d = tmem + buf * WIDE8_COLS;
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
            uint32_t ym[WIDE8_ROWS / 32];
            if (a.mode == 1) {
#pragma unroll
                for (int i = 0; i < WIDE8_ROWS / 32; i++) { const uint32_t r = lane + 32u * i; ym[i] = r < t.z ? a.ymap[t.y + r] : 0u; }
            }
            const float *w0 = a.wscale + ((size_t)t.x * (a.n / 128u) + r0 / 128u) * KB, *w1 = a.wscale + ((size_t)t.x * (a.n / 128u) + r1 / 128u) * KB;
            if (lane < KB) { s_sw[b][0][lane] = __ldg(w0 + lane); s_sw[b][1][lane] = __ldg(w1 + lane); }
            // the tile's row scales are one contiguous block [row][k block]: read it coalesced, store it as [k block][row]
            const float *as = a.ascale + (size_t)t.y * KB;
            const uint32_t total_sc = WIDE8_ROWS * KB;
            if (a.mode == 1) {
#pragma unroll
                for (int i = 0; i < WIDE8_ROWS / 32; i++) s_ymap[b][lane + 32u * i] = ym[i];
            }
            for (uint32_t base = 0; base < total_sc; base += 32u * 2u * WIDE8_KB_MAX) {   // at most two passes of 32 loads per lane
                float v[2 * WIDE8_KB_MAX];
#pragma unroll
                for (int i = 0; i < 2 * WIDE8_KB_MAX; i++) {
                    const uint32_t idx = base + lane + 32u * i, r = (idx * kb_magic) >> 16;   // r = idx / KB (exact for idx < 2048, KB <= 16)
                    v[i] = (idx < total_sc && r < t.z) ? as[idx] : 0.0f;
                }
#pragma unroll
                for (int i = 0; i < 2 * WIDE8_KB_MAX; i++) {
                    const uint32_t idx = base + lane + 32u * i, r = (idx * kb_magic) >> 16, kb = idx - r * KB;
                    if (idx < total_sc) sa_at(b, kb)[r] = v[i];
                }
            }
            mbar_arrive(scfull_bar(b));
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        // ---------------------------------------------------------------- promotion + epilogue: one routed row per thread, 64 + 64 accumulator columns
        const uint32_t g = (warp - 4u) >> 2, q = warp & 3u, row = q * 32u + lane;   // q: the TMEM lane quarter this warp may read
        const uint32_t col0 = g * WIDE8_GCOLS;
        uint32_t n = 0, async = 0; bool ok = true;
        for (uint32_t u = blockIdx.x; u < total && ok; u += gridDim.x, n++) {
            const uint4 t = a.tiles[u / a.pairs]; const uint32_t j = u % a.pairs, b = n & 1u;
            const bool valid = row < t.z;
            const uint32_t r0 = a.mode == 0 ? j * 128u : 2u * j * 128u, r1 = a.mode == 0 ? a.inter + j * 128u : (2u * j + 1u) * 128u;
            if (!(ok = mbar_wait(scfull_bar(b), (n >> 1) & 1u, abort_flag, a.err, 8))) break;
            float acc0[WIDE8_GCOLS], acc1[WIDE8_GCOLS];
#pragma unroll
            for (int i = 0; i < WIDE8_GCOLS; i++) { acc0[i] = 0.0f; acc1[i] = 0.0f; }
            for (uint32_t kb = 0; kb < KB; kb++) {
                const uint32_t it = n * KB + kb, buf = it & 1u, bph = (it >> 1) & 1u;
                const float rs = sa_at(b, kb)[row];                 // 0 for rows past the segment
                const float s0 = rs * s_sw[b][0][kb], s1 = rs * s_sw[b][1][kb];
                if (!(ok = mbar_wait(accfull_bar(buf), bph, abort_flag, a.err, 4))) break;
                tc_fence_after();
                const uint32_t taddr = tmem + ((q * 32u) << 16) + buf * WIDE8_COLS + col0;
                uint32_t da[WIDE8_GCOLS];
                TMEM8_LD64(taddr, da);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < WIDE8_GCOLS; i++) acc0[i] = fmaf(__uint_as_float(da[i]), s0, acc0[i]);
                TMEM8_LD64(taddr + 128u, da);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                tc_fence_before(); mbar_arrive(accempty_bar(buf));   // this thread's share of the partial is in registers
#pragma unroll
                for (int i = 0; i < WIDE8_GCOLS; i++) acc1[i] = fmaf(__uint_as_float(da[i]), s1, acc1[i]);
            }
            if (!ok) break;
            if (a.mode == 0) {
                // ---- SiLU gate, then the gated activations leave as e4m3 with one scale per (row, this unit's 128 features)
                float m = 0.0f;
#pragma unroll
                for (int i = 0; i < WIDE8_GCOLS; i++) { acc0[i] = silu_mul_dev(acc0[i], acc1[i]); m = fmaxf(m, fabsf(acc0[i])); }
                s_red[b][g][row] = m;
                mbar_arrive(all_bar);
                if (!(ok = mbar_wait(all_bar, async++ & 1u, abort_flag, a.err, 5))) break;
                const float sc = pq_scale_mma(fmaxf(s_red[b][0][row], s_red[b][1][row]));
                const float inv = __uint_as_float((254u - (__float_as_uint(sc) >> 23)) << 23);
                if (valid) {
                    if (g == 0) a.s_out[(size_t)(t.y + row) * (a.inter / 128u) + j] = sc;
                    uint32_t w[WIDE8_GCOLS / 4];
#pragma unroll
                    for (int i = 0; i < WIDE8_GCOLS / 4; i++) w[i] = enc2(acc0[4 * i] * inv, acc0[4 * i + 1] * inv) | (enc2(acc0[4 * i + 2] * inv, acc0[4 * i + 3] * inv) << 16);
#pragma unroll
                    for (int i = 0; i < WIDE8_GCOLS / 32; i++) st8_v8(a.q_out + (size_t)(t.y + row) * a.inter + j * 128u + col0 + 32 * i, w + 8 * i);   // whole 32-byte sectors of this row
                }
            } else if (valid) {
                float *o = a.out + (size_t)s_ymap[b][row] * a.out_stride;
                // a thread's 64 + 64 results are two runs of 256 consecutive bytes of its destination row: whole 32-byte sectors per store
#pragma unroll
                for (int i = 0; i < WIDE8_GCOLS / 8; i++) {
                    st8_v8(o + r0 + col0 + 8 * i, reinterpret_cast<const uint32_t *>(acc0 + 8 * i));
                    st8_v8(o + r1 + col0 + 8 * i, reinterpret_cast<const uint32_t *>(acc1 + 8 * i));
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

uint32_t mma_wide8_tile_rows() { return WIDE8_ROWS; }
bool mma_wide8_shape_ok(uint32_t n, uint32_t k, uint32_t mode) { return k % 128u == 0 && k <= 128u * WIDE8_KB_MAX && n % 256u == 0 && (mode == 1 || (n / 2u) % 128u == 0); }

cudaError_t launch_mma_wide8(const void *tm_w, const void *tm_q, const MmaLaunch &m, cudaStream_t s) {
    Wide8Args a = {};
    a.wscale = m.wscale; a.ascale = m.ascale; a.tiles = (const uint4 *)m.tiles; a.header = m.header; a.ymap = m.ymap; a.out = m.out;
    a.q_out = m.q_out; a.s_out = m.s_out; a.q_rows = m.q_rows;
    a.n = m.n; a.k = m.k; a.mode = m.mode; a.inter = m.n / 2u; a.pairs = m.n / 256u; a.out_stride = m.out_stride; a.err = m.err;
    static bool attr = false;
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(fp8_mma_wide8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WIDE8_SMEM);
        if (e != cudaSuccess) return e;
        attr = true;
    }
    const int sms = st().sm_count ? st().sm_count : 148;
    fp8_mma_wide8_kernel<<<sms, WIDE8_THREADS, WIDE8_SMEM, s>>>(*(const CUtensorMap *)tm_w, *(const CUtensorMap *)tm_q, a);
    return cudaGetLastError();
}

}  // namespace b200
