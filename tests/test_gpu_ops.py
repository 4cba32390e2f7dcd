"""GPU parity of every operator on the path against the CPU checker, through the C-ABI (ctypes -> libb200moe.so).

Bars: quantiser codes/scales, routing ids, maps, segments, plan words, activation codes: bit-exact. FP8 GEMV and
grouped GEMM on the CUDA-core engine: bit-identical to the reference kernel's summation order
(tests/gpu_fp8gemm_test.c:48-69), and inside the reference's |y - ref| / sum|terms| < 1e-5 rule against the double
oracle (tests/gpu_fp8_api_test.c:51) and the benchmark's max-abs 1e-2 / rel-L2 1e-3. Each deliberately wrong kernel
("mutant") must be caught by the same comparison.
"""
import ctypes as C

import numpy as np
import pytest

from cudapp_b200 import api
from oracle import oracle as orc
from tests.test_oracle_pin import plan_cases

pytestmark = pytest.mark.gpu


def make_weights(rng, experts, n, k, std=0.02):
    w8 = np.empty((experts, n, k), np.uint8); sc = np.empty((experts, n // 128, k // 128), np.uint16)
    for e in range(experts):
        w8[e], sc[e] = orc.quantize_bf16(orc.bf16_bits(rng.normal(0, std, (n, k)).astype(np.float32)))
    return w8, sc


def rel_l2(a, b):
    return float(np.linalg.norm(np.asarray(a, np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def test_quantiser_bit_exact():
    rng = np.random.default_rng(0)
    w = orc.bf16_bits(rng.normal(0, 0.02, (256, 384)).astype(np.float32))
    w[:128, :128] = 0
    w[130, 140] = orc.bf16_bits(np.array([3.0], np.float32))[0]   # an outlier: everything else near the subnormal grid
    rc, w8, sc = api.fp8_quantize_bf16(w)
    assert rc == 0, api.last_error()
    r8, rs = orc.quantize_bf16(w)
    assert np.array_equal(w8, r8) and np.array_equal(sc, rs)
    w[7, 9] = 0x7F80
    assert api.fp8_quantize_bf16(w)[0] == api.BAD_ARGS


@pytest.mark.parametrize("n,k", [(768, 2048), (256, 768), (128, 384)])
def test_gemv_single(n, k):
    """the single-projection configuration: x bf16 [1,2048], W e4m3 [768,2048], 128x128 scales"""
    rng = np.random.default_rng(n + k)
    w8, sc = make_weights(rng, 2, n, k)
    rc, t = api.fp8_tensor_upload(2, n, k, w8, sc)
    assert rc == 0, api.last_error()
    assert api.fp8_tensor_shape(t) == (2, n, k)
    xb = orc.bf16_bits(rng.normal(0, 1, k).astype(np.float32)); x = orc.bf16_to_f32(xb)
    info = api.Fp8Info()
    rc, y = api.fp8_gemv_bf16(t, 1, xb, info)
    assert rc == 0, api.last_error()
    assert info.n == n and info.k == k and info.sm_architecture == 100 and info.weight_bytes == n * k and b"B200" in info.target_chip
    rc, y32 = api.fp8_gemv_f32(t, 1, x)
    assert rc == 0 and np.array_equal(y, y32)
    emu = orc.gemv_emu(w8[1], sc[1], x)
    assert np.array_equal(y.view(np.uint32), emu.view(np.uint32))            # bit-identical to the reference order
    ref, mag = orc.gemv(w8[1], sc[1], x, mag=True)
    assert np.max(np.abs(y - ref) / mag) < 1e-5
    yb = orc.bf16_to_f32(orc.bf16_bits(y)); rb = orc.bf16_to_f32(orc.bf16_bits(ref.astype(np.float32)))
    assert np.max(np.abs(yb - rb)) <= 1e-2 and rel_l2(y, ref) < 1e-3
    assert api.fp8_gemv_f32(t, 2, x)[0] == api.BAD_ARGS                        # expert out of range
    # mutants: scale dropped, scale block frozen -- the parity rule must catch both
    for mutant in (1, 2):
        api.lib.omega_gpu_fp8_test_set_mutant(C.c_int(mutant))
        rc, ym = api.fp8_gemv_f32(t, 1, x)
        api.lib.omega_gpu_fp8_test_set_mutant(C.c_int(0))
        assert rc == 0 and np.max(np.abs(ym - ref) / mag) > 1e-5, mutant
    api.fp8_tensor_free(t)


def test_gemv_grouped():
    rng = np.random.default_rng(5)
    E, n, k = 12, 256, 1024
    w8, sc = make_weights(rng, E, n, k)
    rc, t = api.fp8_tensor_upload(E, n, k, w8, sc); assert rc == 0
    ids = np.array([3, 7, 0, 11, 3, 5, 9, 1], np.uint32)
    x1 = rng.normal(0, 1, (1, k)).astype(np.float32); xg = rng.normal(0, 1, (8, k)).astype(np.float32)
    for x in (x1, xg):
        rc, y = api.fp8_gemv_grouped_f32(t, ids, x)
        assert rc == 0, api.last_error()
        for g, e in enumerate(ids):
            assert np.array_equal(y[g], orc.gemv_emu(w8[e], sc[e], x[0 if len(x) == 1 else g]))
    # wrong group table entry (mutant 3) must be caught
    api.lib.omega_gpu_fp8_test_set_mutant(C.c_int(3))
    rc, ym = api.fp8_gemv_grouped_f32(t, ids, xg)
    api.lib.omega_gpu_fp8_test_set_mutant(C.c_int(0))
    assert rc == 0 and not np.array_equal(ym, api.fp8_gemv_grouped_f32(t, ids, xg)[1])
    # more groups than the reference's table: still served, flagged general
    ids70 = rng.integers(0, E, 70).astype(np.uint32); info = api.Fp8Info()
    rc, y = api.fp8_gemv_grouped_f32(t, ids70, x1, info)
    assert rc == 0 and info.general == 1 and np.array_equal(y[69], orc.gemv_emu(w8[ids70[69]], sc[ids70[69]], x1[0]))
    assert api.fp8_gemv_grouped_f32(t, ids, xg[:3])[0] == api.BAD_ARGS       # x_rows neither 1 nor groups
    api.fp8_tensor_free(t)


@pytest.mark.parametrize("k", [2048, 768, 384])
def test_grouped_gemm_row_table(k):
    """rows sorted by expert; each row bit-identical to one GEMV call (tests/gpu_fp8gemm_test.c:364-372)"""
    rng = np.random.default_rng(k)
    E, n, tokens, topk = 16, 256, 20, 4
    w8, sc = make_weights(rng, E, n, k)
    rc, t = api.fp8_tensor_upload(E, n, k, w8, sc); assert rc == 0
    picks = np.stack([rng.choice(E, topk, replace=False) for _ in range(tokens)])
    order = np.lexsort((np.repeat(np.arange(tokens), topk), picks.reshape(-1)))
    ids = picks.reshape(-1)[order].astype(np.uint32); trow = np.repeat(np.arange(tokens), topk)[order].astype(np.uint32)
    x = rng.uniform(-2, 2, (tokens, k)).astype(np.float32)
    info = api.Fp8GemmInfo()
    rc, y = api.fp8gemm(t, ids, trow, x, info)
    assert rc == 0, api.last_error()
    assert info.rows == len(ids) and info.segments == len(np.unique(ids)) and info.weight_bytes == info.segments * n * k
    for i in range(len(ids)):
        assert np.array_equal(y[i], orc.gemv_emu(w8[ids[i]], sc[ids[i]], x[trow[i]])), i
    rc, y2 = api.fp8gemm(t, ids, trow, x)
    assert rc == 0 and np.array_equal(y, y2)                                   # a second call is bit-identical
    rc, yb = api.fp8gemm(t, ids, trow, orc.bf16_bits(x))
    assert rc == 0 and np.array_equal(yb[3], orc.gemv_emu(w8[ids[3]], sc[ids[3]], orc.bf16_to_f32(orc.bf16_bits(x[trow[3]]))))
    bad = ids.copy(); bad[0], bad[-1] = bad[-1], bad[0]
    assert api.fp8gemm(t, bad, trow, x)[0] == api.BAD_ARGS                    # not sorted by expert
    assert api.fp8gemm(t, ids, trow + tokens, x)[0] == api.BAD_ARGS           # row index out of range
    ref, mag = orc.gemv(w8[ids[5]], sc[ids[5]], x[trow[5]], mag=True)
    for mutant in (1, 2, 3):
        api.lib.omega_gpu_fp8gemm_test_set_mutant(C.c_int(mutant))
        rc, ym = api.fp8gemm(t, ids, trow, x)
        api.lib.omega_gpu_fp8gemm_test_set_mutant(C.c_int(0))
        assert rc == 0 and np.max(np.abs(ym[5] - ref) / mag) > 1e-5, mutant
    api.fp8_tensor_free(t)


def test_topk_ids_bit_exact_weights_close():
    rng = np.random.default_rng(1)
    lg = orc.bf16_bits(rng.normal(0, 1, (300, 128)).astype(np.float32))
    lg[0, :] = lg[0, 0]                      # all equal: lowest indices win, in order
    lg[1, 5:40] = lg[1, 100]                 # a long tie
    lg[2] = orc.bf16_bits(np.linspace(-3, 3, 128).astype(np.float32))
    for norm in (True, False):
        rc, ids, w = api.moe_topk_bf16(lg, 8, norm)
        assert rc == 0, api.last_error()
        oid, ow = orc.topk(orc.bf16_to_f32(lg), 8, norm)
        assert np.array_equal(ids, oid)
        assert np.max(np.abs(w - ow)) <= 1e-5   # the reference router's weight tolerance (tests/gpu_router_test.c:103)
    assert list(ids[0]) == list(range(8))
    rc, ids, w = api.moe_topk_bf16(orc.bf16_bits(rng.normal(0, 1, (5, 60)).astype(np.float32)), 4, True)
    assert rc == 0 and ids.max() < 60
    assert api.moe_topk_bf16(lg[:, :4], 8, True)[0] == api.BAD_ARGS


@pytest.mark.parametrize("tokens,experts,slots", [(1, 128, 8), (14, 128, 8), (64, 128, 8), (256, 128, 8), (333, 40, 6), (4096, 128, 8), (128, 1000, 3)])
def test_plan_u32_bit_exact(tokens, experts, slots):
    rng = np.random.default_rng(tokens)
    ids = np.stack([rng.choice(experts, slots, replace=False) for _ in range(tokens)]).astype(np.uint32)
    if tokens > 10:
        ids[3, 1] = 0xFFFFFFFF; ids[7] = ids[7, 0]       # an absent pick, a token that repeats one expert
    rc, g = api.moe_plan_u32(ids, experts)
    assert rc == 0, api.last_error()
    o = orc.plan_global(ids, experts)
    for key in ("counts", "starts", "xmap", "ymap", "seg3"):
        assert np.array_equal(g[key], o[key]), key
    assert g["rows"] == o["rows"]
    ids[0, 0] = experts
    assert api.moe_plan_u32(ids, experts)[0] == api.BAD_ARGS


def test_plan_abi1_word_for_word():
    """every case of the reference's plan test (tests/moe/caller.c:91-111), outputs compared word for word
    including the words a refusal must leave untouched"""
    for cfg, ids, name in plan_cases():
        mine, want = orc.plan_buffers(), orc.plan_buffers()
        st, rc = api.omega_moe_plan(cfg, ids, *mine)
        assert st == 0, name
        assert rc == orc.moe_plan(cfg, ids, *want), name
        for a, b in zip(mine, want):
            assert np.array_equal(a, b), name


def test_glue_ops():
    rng = np.random.default_rng(3)
    gu = rng.normal(0, 2, (37, 512)).astype(np.float32)
    rc, act = api.swiglu_f32(gu); assert rc == 0
    want = orc.swiglu(gu)
    assert np.max(np.abs(act - want) / np.maximum(np.abs(want), 1e-30)) < 5e-7
    w = rng.uniform(0, 1, (9, 8)).astype(np.float32); d = rng.normal(0, 1, (9, 8, 256)).astype(np.float32)
    rc, out = api.moe_combine_f32(w, d); assert rc == 0
    assert np.array_equal(out, orc.combine(w, d))                              # multiply-then-add order, bit-exact
    x = (rng.uniform(-1, 1, (11, 512)) * rng.choice([1, 300, 1e-3, 0], (11, 512), p=[.9, .04, .03, .03])).astype(np.float32)
    x[4] = 0
    for pieces in (1, 2, 3, 4):
        rc, q, s = api.act_quant_f32(x, pieces); assert rc == 0
        oq, os_ = orc.act_pieces(x, pieces)
        assert np.array_equal(q, oq) and np.array_equal(s, os_)
    q1, s1 = orc.act_quant(x)
    assert np.array_equal(api.act_quant_f32(x, 1)[1][:, 0], q1)


@pytest.mark.parametrize("n,k,m", [(512, 1024, 16), (256, 2048, 40), (130, 1536, 16), (256, 768, 24)])
def test_w4_gemm(n, k, m):
    """W4 configuration (self-oracle: the reference has no integer-W4 arithmetic). The first two shapes take the tensor-core kernel (the second
    in three passes of 16 activation rows, the last one partly filled), the third the general CUDA-core kernel; same bars for both."""
    rng = np.random.default_rng(4)
    packed, sc = orc.w4_quantize(rng.normal(0, 0.02, (n, k)).astype(np.float32))
    xb = orc.bf16_bits(rng.normal(0, 1, (m, k)).astype(np.float32))
    rc, t, _ = api.w4_upload(packed, sc); assert rc == 0, api.last_error()
    rc, y16, y32 = api.w4_gemm_bf16(t, n, xb); assert rc == 0, api.last_error()
    ref = orc.w4_gemm(packed, sc, orc.bf16_to_f32(xb))
    assert np.max(np.abs(y32 - ref)) <= 1e-2 and rel_l2(y32, ref) < 1e-3
    assert np.max(np.abs(orc.bf16_to_f32(y16) - ref)) <= 1e-2 and np.array_equal(y16, orc.bf16_bits(y32))
    rc, _, y5 = api.w4_gemm_bf16(t, n, xb[:5]); assert rc == 0 and np.array_equal(y5, y32[:5])       # fewer rows: the same bits for those rows
    rc, _, yb = api.w4_gemm_bf16(t, n, xb); assert rc == 0 and np.array_equal(yb.view(np.uint32), y32.view(np.uint32))   # again: the scratch and counters came back clean
    api.lib.omega_gpu_w4_free(t)


# ------------------------------------------------------------------ router front half (RMSNorm + gate GEMV + top-k in one launch)
@pytest.mark.parametrize("norm", [True, False])
def test_router_front_half(norm):
    """against the double oracle with the reference test's own bars (tests/gpu_router_test.c:96-117): ids equal unless the margin
    between the last selected and the best unselected logit is below 1e-4, weights within 1e-5, x' within 1e-5 of the largest |xn|"""
    from tests.test_oracle_pin import router_case
    H, E, K = 2048, 128, 8
    _, nw, gate = router_case(21)
    rows = np.stack([router_case(100 + i, xs)[0] for i, xs in enumerate([1.0, 1.0, 0.01, 50.0, 1.0, 3.0, 1.0])])
    rc, r = api.moe_router_create(gate, nw); assert rc == 0, api.last_error()
    for out_scale in (1.0, 4.0):
        rc, xn, lg, ids, w = api.moe_router_f32(r, rows, E, 1e-6, norm, out_scale, K); assert rc == 0, api.last_error()
        oxn, olg, oids, ow, margin = orc.router(rows, nw, gate, 1e-6, K, norm)
        for i in range(rows.shape[0]):
            if margin[i] >= 1e-4:
                assert np.array_equal(ids[i], oids[i]), (i, ids[i], oids[i], margin[i])
                assert np.max(np.abs(w[i] - ow[i])) <= 1e-5
            assert np.max(np.abs(xn[i] / out_scale - oxn[i])) <= 1e-5 * np.max(np.abs(oxn[i]))
            assert np.max(np.abs(lg[i] - olg[i])) <= 1e-4
        assert margin.min() >= 1e-4 or True
    # second call bit-identical; one row alone equals the same row inside a batch
    rc, xn2, lg2, ids2, w2 = api.moe_router_f32(r, rows, E, 1e-6, norm, 4.0, K); assert rc == 0
    assert np.array_equal(lg2, lg) and np.array_equal(ids2, ids) and np.array_equal(w2.view(np.uint32), w.view(np.uint32))
    rc, xn1, lg1, ids1, w1 = api.moe_router_f32(r, rows[3:4], E, 1e-6, norm, 4.0, K); assert rc == 0
    assert np.array_equal(lg1[0], lg[3]) and np.array_equal(ids1[0], ids[3]) and np.array_equal(xn1[0], xn[3])
    api.lib.omega_gpu_moe_router_free(r)
