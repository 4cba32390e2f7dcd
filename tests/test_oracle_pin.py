"""Pins the CPU checker (oracle/moe_oracle.c) to the reference's own host code.

Two anchors: (1) where the reference build is present (oracle/_ref, made by `make -C oracle ref` from the
reference sources), every function is compared with it directly on seeded inputs and on the cases the
reference's own tests use (tests/gpu_fp8_api_test.c:250-339, tests/moe/caller.c:91-157); (2) everywhere,
the committed vectors in tests/golden/, which tests/golden/make_golden.py produced from that build.
"""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import oracle as orc

REF = orc.ref_lib()
REFG = orc.ref_group_lib()
REFR = orc.ref_router_lib()
REF_EMU, REF_PQ, REF_MC = orc.ref_static_lib("emu"), orc.ref_static_lib("pq"), orc.ref_static_lib("mc")
need_ref = pytest.mark.skipif(REF is None, reason="reference build (oracle/_ref) not present")
U8P, U16P, U32P, U64P, F32P, F64P = orc.U8P, orc.U16P, orc.U32P, orc.U64P, orc.F32P, orc.F64P
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def ptr(a, t):
    return a.ctypes.data_as(t)


# ------------------------------------------------------------------ e4m3 known answers (tests/gpu_fp8_api_test.c:313-339)
def test_e4m3_known_answers():
    L = orc.lib()
    assert L.orc_e4m3_decode(0x38) == 1.0
    assert L.orc_e4m3_decode(0x7E) == 448.0
    assert L.orc_e4m3_decode(0x01) == 2.0 ** -9
    assert L.orc_e4m3_decode(0x07) == 7 * 2.0 ** -9
    assert L.orc_e4m3_decode(0x08) == 2.0 ** -6
    assert L.orc_e4m3_decode(0xB8) == -1.0
    assert np.isnan(L.orc_e4m3_decode(0x7F)) and np.isnan(L.orc_e4m3_decode(0xFF))
    # every finite code survives encode(decode(code)); -0 keeps its sign
    for c in range(256):
        if c & 0x7F == 0x7F:
            continue
        assert L.orc_e4m3_encode(L.orc_e4m3_decode(c)) == c
    assert L.orc_e4m3_encode(1e9) == 0x7E and L.orc_e4m3_encode(-1e9) == 0xFE
    assert L.orc_e4m3_encode(float("nan")) & 0x7F == 0x7E
    assert L.orc_e4m3_encode(448.0) == 0x7E and L.orc_e4m3_encode(464.0) == 0x7E


def test_e4m3_encode_brute_force():
    """nearest code, ties to the even code, saturating (the reference's rule, tests/gpu_fp8_api_test.c:250-288)"""
    L = orc.lib()
    tab = orc.e4m3_table()[:0x7F].astype(np.float64)  # non-negative finite codes, ascending
    rng = np.random.default_rng(11)
    vals = np.concatenate([rng.normal(0, 100, 4000), rng.normal(0, 0.05, 3000), rng.uniform(-500, 500, 2000),
                           (tab[:-1] + tab[1:]) / 2, -(tab[:-1] + tab[1:]) / 2, tab, [0.0, -0.0, 2.0 ** -10, 3 * 2.0 ** -10]]).astype(np.float32)
    for v in vals:
        a = abs(float(v))
        d = np.abs(tab - a)
        best = int(np.argmin(d))
        ties = np.nonzero(d == d[best])[0]
        if len(ties) > 1:
            best = int([t for t in ties if t % 2 == 0][0])
        if a >= 448.0:
            best = 0x7E
        want = best | (0x80 if np.signbit(v) else 0)
        assert L.orc_e4m3_encode(C.c_float(float(v))) == want, (v, want)


@need_ref
def test_formats_against_reference():
    L = orc.lib()
    for c in range(256):
        a, b = L.orc_e4m3_decode(c), REF.omega_fp8_e4m3_ref(c)
        assert (np.isnan(a) and np.isnan(b)) or a == b
    rng = np.random.default_rng(5)
    vals = np.concatenate([rng.normal(0, 120, 20000), rng.normal(0, 0.02, 20000), rng.uniform(-460, 460, 5000),
                           [0.0, -0.0, 448.0, 447.99, 1e-30, -1e-30, np.inf, -np.inf]]).astype(np.float32)
    for v in vals:
        assert L.orc_e4m3_encode(C.c_float(float(v))) == REF.omega_gpu_fp8_e4m3_rne(C.c_float(float(v))), v
        assert L.orc_f32_to_bf16(C.c_float(float(v))) == REF.omega_fp32_to_bf16(C.c_float(float(v))), v


@need_ref
def test_quantiser_and_gemv_against_reference():
    rng = np.random.default_rng(0)
    n, k = 256, 384
    w = orc.bf16_bits(rng.normal(0, 0.02, (n, k)).astype(np.float32))
    w[0:128, 0:128] = 0  # an all-zero block: scale 1.0
    w8, sc = orc.quantize_bf16(w)
    r8 = np.empty_like(w8); rs = np.empty_like(sc)
    assert REF.omega_gpu_fp8_quantize_bf16(C.c_uint32(n), C.c_uint32(k), ptr(w, U16P), ptr(r8, U8P), ptr(rs, U16P)) == 0
    assert np.array_equal(w8, r8) and np.array_equal(sc, rs)
    assert sc[0, 0] == 0x3F80
    x = rng.normal(0, 1, k).astype(np.float32)
    y, m = orc.gemv(w8, sc, x, mag=True)
    ry = np.empty(n, np.float64); rm = np.empty(n, np.float64)
    REF.omega_fp8_gemv_oracle(ptr(w8, U8P), ptr(sc, U16P), C.c_uint32(n), C.c_uint32(k), ptr(x, F32P), ptr(ry, F64P), ptr(rm, F64P))
    assert np.array_equal(y, ry) and np.array_equal(m, rm)
    # inf weight refused by both
    w[3, 3] = 0x7F80
    assert REF.omega_gpu_fp8_quantize_bf16(C.c_uint32(n), C.c_uint32(k), ptr(w, U16P), ptr(r8, U8P), ptr(rs, U16P)) == -1
    with pytest.raises(ValueError):
        orc.quantize_bf16(w)


def _ref_plan(cfg, ids, bufs):
    r = C.c_uint64(99)
    rc = REF.omega_moe_plan(C.byref(r), ptr(cfg, U64P), C.c_uint64(8), ptr(ids, U64P), C.c_uint64(1024), ptr(bufs[0], U64P), C.c_uint64(10368),
                            ptr(bufs[1], U64P), C.c_uint64(1028), ptr(bufs[2], U64P), C.c_uint64(2320), ptr(bufs[3], U64P), C.c_uint64(8))
    assert rc == 0
    return r.value


def plan_cases():
    """the id patterns and sizes of tests/moe/caller.c:34-50, :91-111"""
    for n in (0, 1, 2, 3, 7, 14, 15, 31, 127, 128):
        for mode in range(5):
            ids = np.zeros(1024, np.uint64)
            for t in range(n):
                for s in range(8):
                    ids[t * 8 + s] = [7, (t * 8 + s) % 256, s % 3, 255 if t % 2 else s, (t * 17 + s * 13) % 256][mode]
            yield np.array([1, n, 8, 256, 256, 1152, 257, 1160], np.uint64), ids, "dense n=%d mode=%d" % (n, mode)
    ids = np.zeros(1024, np.uint64)
    for j in range(24):
        ids[j] = 0xFFFFFFFF if j % 4 else j
    yield np.array([1, 3, 8, 256, 256, 1152, 257, 1160], np.uint64), ids, "sparse"
    yield np.array([1, 128, 8, 256, 256, 1152, 257, 1160], np.uint64), np.full(1024, 0xFFFFFFFF, np.uint64), "all absent"
    yield np.array([1, 5, 0, 256, 256, 1152, 257, 1160], np.uint64), np.zeros(1024, np.uint64), "zero slots"
    yield np.array([1, 64, 8, 128, 128, 1152, 257, 1160], np.uint64), (np.arange(1024) * 37 % 128).astype(np.uint64), "128 experts"
    # refusals (tests/moe/caller.c:98-107)
    base = [1, 1, 8, 256, 256, 1152, 257, 1160]
    z = np.zeros(1024, np.uint64)
    for field, val in ((5, 1151), (7, 1159)):
        c = np.array([1, 128, 8, 256, 256, 1152, 257, 1160], np.uint64); c[field] = val
        yield c, z, "capacity %d" % field
    for field, val in ((6, 1), (0, 2), (1, 129), (2, 9), (4, 255), (5, 1153), (6, 258), (7, 1161), (3, 0), (3, 257)):
        c = np.array(base, np.uint64); c[field] = val
        yield c, z, "cfg %d=%d" % (field, val)
    for bad in (256, 0xFFFFFFFE):
        ids = np.zeros(1024, np.uint64); ids[3] = bad
        yield np.array(base, np.uint64), ids, "bad id"


@need_ref
def test_plan_against_reference():
    for cfg, ids, name in plan_cases():
        mine, theirs = orc.plan_buffers(), orc.plan_buffers()
        rc = orc.moe_plan(cfg, ids, *mine)
        assert rc == _ref_plan(cfg, ids, theirs), name
        for a, b in zip(mine, theirs):  # word for word, including every untouched (0x5a) word
            assert np.array_equal(a, b), name


@need_ref
def test_serialisers_against_reference():
    L = orc.lib()
    cfg = np.array([1, 31, 8, 256, 256, 1152, 257, 1160], np.uint64)
    ids = (np.arange(1024) * 29 % 256).astype(np.uint64)
    work, seg, maps, meta = orc.plan_buffers()
    assert orc.moe_plan(cfg, ids, work, seg, maps, meta) == 0
    dirs = np.zeros(514, np.uint64)
    for j in range(257):
        dirs[2 * j] = j * 256 + 4096; dirs[2 * j + 1] = dirs[2 * j] + 128
    r = C.c_uint64(0)
    for mut in ("ok", "map", "dir", "seg"):
        mp, sg, dr = maps.copy(), seg.copy(), dirs.copy()
        if mut == "map": mp[0] = 2 ** 64 - 1
        if mut == "dir": dr[0] = 0
        if mut == "seg": sg[2] = 2 ** 64 - 1
        a = np.full(9280, 90, np.uint8); b = a.copy()
        rc = L.orc_moe_maps32(ptr(meta, U64P), ptr(mp, U64P), ptr(a, U8P))
        assert REF.omega_moe_maps32(C.byref(r), ptr(meta, U64P), C.c_uint64(8), ptr(mp, U64P), C.c_uint64(2320), ptr(b, U8P), C.c_uint64(9280)) == 0
        assert rc == r.value and np.array_equal(a, b), mut
        a = np.full(8224, 90, np.uint8); b = a.copy()
        rc = L.orc_moe_segs32(ptr(sg, U64P), ptr(meta, U64P), ptr(dr, U64P), ptr(a, U8P))
        assert REF.omega_moe_segs32(C.byref(r), ptr(sg, U64P), C.c_uint64(1028), ptr(meta, U64P), C.c_uint64(8), ptr(dr, U64P), C.c_uint64(514), ptr(b, U8P), C.c_uint64(8224)) == 0
        assert rc == r.value and np.array_equal(a, b), mut
    wire = np.zeros(4096, np.uint8)
    wire.view(np.uint32)[:] = np.arange(1024) % 257
    for n in (0, 5, 1024, 1025):
        a = np.full(1024, 7, np.uint64); b = a.copy()
        rc = L.orc_moe_ids32(ptr(wire, U8P), C.c_uint64(n), ptr(a, U64P))
        assert REF.omega_moe_ids32(C.byref(r), ptr(wire, U8P), C.c_uint64(4096), C.c_uint64(n), ptr(b, U64P), C.c_uint64(1024)) == 0
        assert rc == r.value and np.array_equal(a, b)
    for n in list(range(0, 129)) + [129]:
        for cap, flush in ((128, 0), (1, 0), (128, 1)):
            c = np.array([1, n, 2048, 512, 9, 512, cap, flush], np.uint64)
            a = np.full(1024, 3, np.uint64); am = np.full(4, 3, np.uint64); b = a.copy(); bm = am.copy()
            rc = L.orc_moe_windows(ptr(c, U64P), ptr(a, U64P), ptr(am, U64P))
            assert REF.omega_moe_windows(C.byref(r), ptr(c, U64P), C.c_uint64(8), ptr(b, U64P), C.c_uint64(1024), ptr(bm, U64P), C.c_uint64(4)) == 0
            assert rc == r.value and np.array_equal(a, b) and np.array_equal(am, bm), (n, cap, flush)
    q = [4096, 8192, 12288, 65536, 131072, 196608, 262144, 512, 14, 126, 134, 9, 1, 1, 1, 256]
    bads = [(None, None)] + [(8, 15), (8, 0), (11, 8), (15, 255), (9, 125), (10, 133), (7, 0), (7, 513), (0, 4097), (12, 0), (13, 2), (14, 0),
                             (3, 4096), (4, 65536), (5, 65536), (6, 196608), (0, 2 ** 64 - 8), (3, 2 ** 64 - 8), (7, 128), (8, 2 ** 64 - 1)]
    for f, v in bads:
        req = np.array(q, np.uint64)
        if f is not None: req[f] = v
        a = np.full(64, 9, np.uint8); b = a.copy()
        rc = L.orc_moe_group(ptr(req, U64P), ptr(a, U8P))
        assert REF.omega_moe_group(C.byref(r), ptr(req, U64P), C.c_uint64(16), ptr(b, U8P), C.c_uint64(64)) == 0
        assert rc == r.value and np.array_equal(a, b), (f, v)


@pytest.mark.skipif(REFG is None, reason="reference build (oracle/_ref) not present")
def test_global_plan_against_incumbent_group():
    """the u32 form against the reference's unchanged host GROUP (tests/moe/incumbent.c; 9-wide Y rows)"""
    rng = np.random.default_rng(3)
    for n in (1, 2, 7, 14, 64, 128):
        ids = np.stack([rng.choice(128, 8, replace=False) for _ in range(n)]).astype(np.uint32)
        ox = np.zeros(1152 + 16, np.uint32); oy = np.zeros(1152 + 16, np.uint32); os_ = np.zeros(1028, np.uint32)
        ns = REFG.moe_incumbent(C.c_uint32(n), ptr(ids, U32P), ptr(ox, U32P), ptr(oy, U32P), ptr(os_, U32P))
        g = orc.plan_global(ids, 128, ystride=9)
        assert g["rows"] == n * 8 and len(g["seg3"]) == ns - 1  # the incumbent appends the shared segment
        assert np.array_equal(g["xmap"][: n * 8], ox[: n * 8]) and np.array_equal(g["ymap"][: n * 8], oy[: n * 8])
        assert np.array_equal(g["seg3"].reshape(-1), os_.reshape(-1, 4)[: ns - 1, :3].reshape(-1))


def test_global_plan_rank_rule():
    """independent check of the ordering rule: rank = #{(e',t',s') < (e,t,s)} (tests/moe/caller.c:66-73)"""
    rng = np.random.default_rng(4)
    ids = rng.integers(0, 16, (40, 8)).astype(np.uint32)
    ids[5, 2] = 0xFFFFFFFF
    g = orc.plan_global(ids, 16)
    key = [(int(ids[t, s]), t * 8 + s) for t in range(40) for s in range(8) if ids[t, s] != 0xFFFFFFFF]
    for (e, i) in key:
        rank = sum(1 for (f, j) in key if f < e or (f == e and j < i))
        assert g["xmap"][rank] == i // 8 and g["ymap"][rank] == i
    assert np.all(g["xmap"][g["rows"]:] == 0) and g["rows"] == len(key)


def test_emu_order_is_close_to_double():
    rng = np.random.default_rng(8)
    for k in (512, 768, 2048):
        w8, sc = orc.quantize_bf16(orc.bf16_bits(rng.normal(0, 0.02, (128, k)).astype(np.float32)))
        x = rng.normal(0, 1, k).astype(np.float32)
        y, m = orc.gemv(w8, sc, x, mag=True)
        e = orc.gemv_emu(w8, sc, x)
        assert np.max(np.abs(e - y) / m) < 1e-5  # the reference's parity rule (tests/gpu_fp8_api_test.c:51)


def test_act_quant_and_pieces():
    rng = np.random.default_rng(9)
    x = (rng.uniform(-1, 1, (6, 256)) * rng.choice([1, 300, 1e-3, 0], (6, 256), p=[.9, .04, .03, .03])).astype(np.float32)
    x[5] = 0
    q, s = orc.act_quant(x)
    tab = orc.e4m3_table()
    amax = np.abs(x.reshape(6, 2, 128)).max(-1)
    assert np.all(np.log2(s) == np.round(np.log2(s)))  # powers of two
    nz = amax > 0
    assert np.all(amax[nz] / s[nz] <= 448) and np.all(amax[nz] / s[nz] > 224)
    assert np.all(s[~nz] == 2.0 ** -108)
    q3, s3 = orc.act_pieces(x, 3)
    assert np.array_equal(q3[:, 0], q) and np.array_equal(s3, s)
    bf = orc.bf16_to_f32(orc.bf16_bits(x))
    q2, s2 = orc.act_pieces(bf, 2)
    back = orc.act_pieces_decode(q2, s2)
    big = np.abs(bf) >= np.repeat(s2, 128, axis=1) * 2.0 ** -6
    assert np.array_equal(back[big], bf[big].astype(np.float64))  # two pieces hold a bf16 value exactly
    assert np.max(np.abs(back - bf)) <= np.max(s2) * 2.0 ** -14
    back3 = orc.act_pieces_decode(q3, s3)
    rel = np.abs(back3 - x)[np.abs(x) > 0] / np.abs(x)[np.abs(x) > 0]
    assert np.median(rel) < 2.0 ** -13


def test_w4_self_consistency():
    rng = np.random.default_rng(1)
    w = rng.normal(0, 0.02, (64, 128)).astype(np.float32); w[0, :32] = 0
    p, sc = orc.w4_quantize(w)
    L = orc.lib()
    scf = np.array([L.orc_f16_to_f32(int(v)) for v in sc.reshape(-1)], np.float32).reshape(sc.shape)
    assert scf[0, 0] == 1.0
    assert np.array_equal(sc.view(np.float16).astype(np.float32), scf)
    lo = (p & 15).astype(np.int8); hi = (p >> 4).astype(np.int8)
    q = np.stack([lo, hi], -1).reshape(64, 128); q[q > 7] -= 16
    deq = q * np.repeat(scf, 32, axis=1)
    assert np.max(np.abs(deq - w)) <= np.max(scf) * 0.5 + 1e-7
    x = rng.normal(0, 1, (3, 128)).astype(np.float32)
    y = orc.w4_gemm(p, sc, x, threads=2)
    assert np.allclose(y, x.astype(np.float64) @ deq.astype(np.float64).T, rtol=1e-12, atol=1e-12)
    h = rng.normal(0, 30, 2000).astype(np.float32)
    mine = np.array([L.orc_f32_to_f16(C.c_float(float(v))) for v in h], np.uint16)
    assert np.array_equal(mine, h.astype(np.float16).view(np.uint16))


# ------------------------------------------------------------------ router front half (tests/gpu_router_test.c:62-79)
def router_case(seed, xscale=1.0, hidden=2048, experts=128):
    """seeded inputs in the ranges the reference's router test draws from: x in [-2, 2) * xscale, norm weight in [0.8, 1.2),
    gate rows in [-0.05, 0.05) rounded to bf16"""
    rng = np.random.default_rng([77, seed])
    x = (rng.uniform(-2.0, 2.0, hidden) * xscale).astype(np.float32)
    nw = rng.uniform(0.8, 1.2, hidden).astype(np.float32)
    gate = orc.bf16_bits(rng.uniform(-0.05, 0.05, (experts, hidden)).astype(np.float32))
    return x, nw, gate


@pytest.mark.skipif(REFR is None, reason="reference router oracle (oracle/_ref/libref_router.so) not present")
def test_router_against_reference():
    REFR.ref_router_eps.restype = C.c_float
    H, E, K = REFR.ref_router_hidden(), REFR.ref_router_experts(), REFR.ref_router_topk()
    assert (H, E, K) == (2048, 128, 8)
    eps = float(REFR.ref_router_eps())
    for seed, xscale in [(1, 1.0), (2, 1.0), (3, 0.01), (4, 50.0), (5, 1.0)]:
        x, nw, gate = router_case(seed, xscale)
        for norm in (1, 0):
            xn = np.empty(H, np.float64); lg = np.empty(E, np.float64); ids = np.empty(K, np.uint32); w = np.empty(K, np.float64); m = C.c_double(0)
            REFR.ref_router_oracle(ptr(x, F32P), ptr(nw, F32P), ptr(gate, U16P), C.c_int(norm), ptr(xn, F64P), ptr(lg, F64P), ptr(ids, U32P), ptr(w, F64P), C.byref(m))
            mxn, mlg, mids, mw, mm = orc.router(x[None], nw, gate, eps, K, bool(norm))
            assert np.array_equal(mids[0], ids)
            assert np.array_equal(mxn[0], xn) and np.array_equal(mlg[0], lg)          # the same double arithmetic in the same order
            assert np.max(np.abs(mw[0] - w)) <= 1e-15 and abs(mm[0] - m.value) <= 1e-15
            assert abs(w.sum() - 1.0) < 1e-12 if norm else w.sum() < 1.0


@need_ref
def test_plan_against_reference_random():
    """seeded random plans beyond the reference test's own patterns: any token / slot / expert count inside the caps, absent picks
    sprinkled in, with and without the shared expert; word for word against the reference's emitted unit"""
    rng = np.random.default_rng(404)
    for trial in range(300):
        tokens = int(rng.integers(0, 129)); slots = int(rng.integers(0, 9)); experts = int(rng.integers(1, 257))
        shared = int(rng.integers(0, 2))
        cfg = np.array([shared, tokens, slots, experts, 256 if shared else int(rng.choice([experts, 256])), 1152, 257, 1160], np.uint64)
        ids = np.zeros(1024, np.uint64)
        n = tokens * slots
        ids[:n] = rng.integers(0, experts, n)
        if n and trial % 3 == 0:
            ids[rng.integers(0, n, max(1, n // 5))] = 0xFFFFFFFF
        if n and trial % 50 == 7:
            ids[int(rng.integers(0, n))] = experts          # one id out of range: both must refuse the same way
        mine, theirs = orc.plan_buffers(), orc.plan_buffers()
        rc = orc.moe_plan(cfg, ids, *mine)
        assert rc == _ref_plan(cfg, ids, theirs), (trial, cfg.tolist())
        for a, b in zip(mine, theirs):
            assert np.array_equal(a, b), (trial, cfg.tolist())


# ------------------------------------------------------------------ static functions of the reference's own tests, compiled in place
def emu_case(seed, n, k):
    """weights and scales drawn as the reference test draws them (any non-NaN code, bf16 scales of either sign: tests/gpu_fp8gemm_test.c:40-47)"""
    rng = np.random.default_rng(seed)
    w8 = rng.integers(0, 256, (n, k)).astype(np.uint8); w8[(w8 & 0x7F) == 0x7F] -= 1
    sc = orc.bf16_bits((rng.uniform(0.001, 0.1, (n // 128, k // 128)) * rng.choice([-1.0, 1.0], (n // 128, k // 128))).astype(np.float32))
    x = rng.uniform(-2, 2, k).astype(np.float32)
    return w8, sc, x


def ref_emu(w8, sc, x):
    n, k = w8.shape
    lb = 16 if k % 512 == 0 else 8
    return np.array([REF_EMU.ref_emu_row(ptr(w8[r], U8P), ptr(sc[r // 128], U16P), ptr(x, F32P), C.c_uint32(k), C.c_uint32(lb)) for r in range(n)], np.float32)


@pytest.mark.skipif(REF_EMU is None, reason="reference emu_row (oracle/_ref/libref_emu.so) not present")
def test_gemv_emulation_against_reference():
    """the kernels' exact f32 summation order: the checker's restatement against emu_row of tests/gpu_fp8gemm_test.c:48-69, bit for bit
    (the reference folds 2^64 / 2^56 / 2^-120 into x / scale / weight; exact powers of two whose product is 1)"""
    for seed, n, k in ((1, 128, 512), (2, 256, 768), (3, 128, 2048), (4, 128, 256), (5, 256, 1024)):
        w8, sc, x = emu_case(seed, n, k)
        assert np.array_equal(orc.gemv_emu(w8, sc, x).view(np.uint32), ref_emu(w8, sc, x).view(np.uint32)), (seed, n, k)


def pq_case(rows, k):
    """activations from the reference test's own generator (rand_act, tests/gpu_qgemm_test.c:36-40), row 3 zero, one huge outlier in row 5 (:43-47)"""
    x = np.empty(rows * k, np.float32)
    REF_PQ.ref_pq_rand_act(ptr(x, F32P), C.c_uint32(rows * k))
    x = x.reshape(rows, k)
    x[3] = 0
    x[5, 77] = 3.0e4
    return x


@pytest.mark.skipif(REF_PQ is None, reason="reference pq_ref (oracle/_ref/libref_pq.so) not present")
def test_act_quant_against_reference():
    """activation quantiser (per row, per 128 columns: power-of-two scale, e4m3 RNE sat-finite) against pq_ref of tests/gpu_qgemm_test.c:24-35"""
    for rows, k in ((8, 256), (16, 2048), (7, 768)):
        x = pq_case(rows, k)
        q, s = orc.act_quant(x)
        for r in range(rows):
            rq = np.empty(k, np.uint8); rs = np.empty(k // 128, np.float32)
            REF_PQ.ref_pq(ptr(x[r], F32P), C.c_uint32(k), ptr(rq, U8P), ptr(rs, F32P))
            assert np.array_equal(q[r], rq) and np.array_equal(s[r].view(np.uint32), rs.view(np.uint32)), (rows, k, r)


def mc_case(seed, rows, h, K):
    rng = np.random.default_rng(seed)
    down = (rng.uniform(-1, 1, (rows * K, h)) * rng.choice([1.0, 40.0, 0.0], (rows * K, h), p=[0.96, 0.02, 0.02])).astype(np.float32)
    wt = rng.uniform(0, 1, (rows, K)).astype(np.float32)
    inv = rng.permutation(rows * K).astype(np.uint32).reshape(rows, K)
    return down, inv, wt


@pytest.mark.skipif(REF_MC is None, reason="reference mc_ref (oracle/_ref/libref_mc.so) not present")
def test_combine_against_reference():
    """slot-order multiply-then-add combine against mc_ref of tests/gpu_pfhost_test.c:38-49, bit for bit; the decode form (accumulator
    starts at the first product) differs from it in the sign of an exact zero at most"""
    for seed, rows, h, K in ((1, 5, 256, 8), (2, 33, 2048, 8), (3, 4, 128, 9), (4, 9, 512, 1)):
        down, inv, wt = mc_case(seed, rows, h, K)
        ref = np.empty((rows, h), np.float32)
        REF_MC.ref_mc(ptr(down, F32P), ptr(inv, U32P), ptr(wt, F32P), C.c_uint32(rows), C.c_uint32(h), C.c_uint32(K), ptr(ref, F32P))
        assert np.array_equal(orc.combine_mc(down, inv, wt).view(np.uint32), ref.view(np.uint32))
        dec = orc.combine(wt, down[inv.reshape(-1)].reshape(rows, K, h))
        assert np.array_equal(dec, ref)                                        # equal as numbers everywhere ...
        nz = ref != 0
        assert np.array_equal(dec.view(np.uint32)[nz], ref.view(np.uint32)[nz])   # ... and as bits wherever the sum is not an exact zero


# ------------------------------------------------------------------ MXFP4 element decoder (native/models/mxfp4.om; oracle tests/models/mxfp4-check.py)
MXFP4_ORACLE_SHA256 = "665ce3b50c419456c447dc8eabf300d79f20d38dfdbd6e5b3fd6b97308f0bf04"   # docs/models/MXFP4.md: oracle_sha256 of the 130 560 records


def mxfp4_all_records():
    import struct
    return b"".join(struct.pack("<I", orc.mxfp4_bits((p >> (4 * l)) & 15, s)) for s in range(255) for p in range(256) for l in range(2))


def test_mxfp4_decoder_against_published_digest():
    """every (scale, byte, lane) record of the reference's own check, in its order: the digest the reference publishes for its oracle's output"""
    import hashlib
    assert hashlib.sha256(mxfp4_all_records()).hexdigest() == MXFP4_ORACLE_SHA256
    for nib, scale, want in ((2, 127, 1.0), (7, 127, 6.0), (9, 127, -0.5), (1, 128, 1.0), (7, 254, np.inf), (15, 254, -np.inf), (8, 5, -0.0)):
        got = np.array([orc.mxfp4_bits(nib, scale)], np.uint32).view(np.float32)[0]
        assert got == np.float32(want) and np.signbit(got) == np.signbit(np.float32(want))
    assert orc.mxfp4_bits(1, 0) == 1 << 21                                     # 0.5 * 2^-127 = 2^-128: a subnormal, not flushed


MXCHECK = os.path.join(os.environ.get("B200MOE_REFERENCE", os.path.normpath(os.path.join(os.path.dirname(__file__), "..", "..", "reference"))), "tests", "models", "mxfp4-check.py")


@pytest.mark.skipif(not os.path.exists(MXCHECK), reason="the reference tree is not on this machine")
def test_mxfp4_decoder_against_reference_oracle():
    """the same records against the reference's verification oracle itself (imported from its test script where the tree is present)"""
    import importlib.util
    spec = importlib.util.spec_from_file_location("mxfp4_check", MXCHECK); m = importlib.util.module_from_spec(spec); spec.loader.exec_module(m)
    want = b"".join(m.oracle(p, l, s) for s in range(255) for p in range(256) for l in range(2))
    assert want == mxfp4_all_records()


# ------------------------------------------------------------------ NVFP4 element x scale decoder (native/models/nvfp4.om; oracle tests/models/mxfmt-check.py:278-300)
def nvfp4_all_pairs():
    """bits of every element x valid scale pair, element-major: the order of the reference's own decode check"""
    return np.array([orc.nvfp4_bits(n, c) for n in range(16) for c in range(127)], np.uint32)


def test_nvfp4_decoder_against_ml_dtypes():
    """the comparison the reference's check makes (tests/models/mxfmt-check.py:289-295): the binary32 product of the ml_dtypes values, exact"""
    ml = pytest.importorskip("ml_dtypes")
    nib = np.repeat(np.arange(16, dtype=np.uint8), 127); sc = np.tile(np.arange(127, dtype=np.uint8), 16)
    f4 = nib.view(ml.float4_e2m1fn).astype(np.float64); f8 = sc.view(ml.float8_e4m3fn).astype(np.float64)
    prod = (f4 * f8).astype(np.float32)
    assert np.all(prod.astype(np.float64) == f4 * f8)                          # exact in binary32
    assert np.array_equal(nvfp4_all_pairs(), prod.view(np.uint32))             # signed zeros included
    for bad in (127, 128, 255):                                                # NaN scale and sign-set scales: refused by the unit (trap 5)
        assert orc.nvfp4_bits(3, bad) == 0xffffffff
    assert orc.nvfp4_bits(7, 126) == np.array([6.0 * 448.0], np.float32).view(np.uint32)[0]
    assert orc.nvfp4_bits(1, 1) == np.array([2.0 ** -10], np.float32).view(np.uint32)[0]


MXFMT = os.path.join(os.path.dirname(MXCHECK), "mxfmt-check.py")


@pytest.mark.skipif(not os.path.exists(MXFMT), reason="the reference tree is not on this machine")
def test_nvfp4_decoder_against_reference_oracle():
    """every pair against the exact rationals of the reference's verification script itself (its e2m1 and ue4m3 functions)"""
    pytest.importorskip("ml_dtypes")                                           # the script imports it at load
    import importlib.util
    from fractions import Fraction
    spec = importlib.util.spec_from_file_location("mxfmt_check", MXFMT); m = importlib.util.module_from_spec(spec); spec.loader.exec_module(m)
    got = nvfp4_all_pairs().view(np.float32).reshape(16, 127)
    for n in range(16):
        for c in range(127):
            assert Fraction(float(got[n, c])) == m.e2m1(n) * m.ue4m3(c), (n, c)
            assert bool(np.signbit(got[n, c])) == bool(n & 8)


# ------------------------------------------------------------------ block-scaled product of two quantised operands (native/models/mxdot.om; oracle tests/models/mxfmt-check.py:392-411)
MX_SHAPES = ((1, 1, 1), (4, 4, 8), (16, 16, 1), (2, 3, 4), (1, 1, 64))   # (m, n, k in blocks)


def mx_cases(m, rounds=4, seed=1026):
    """seeded cases from the reference script's own generator: all three formats, narrow and wide scale ranges"""
    rng = np.random.default_rng(seed)
    for rnd in range(rounds):
        for fmt in (0, 1, 2):
            for (mm, nn, kblocks) in MX_SHAPES:
                yield m.mx_case(rng, fmt, mm, nn, kblocks * m.BS[fmt], wide=(rnd % 2 == 0))[1]


@pytest.mark.skipif(not os.path.exists(MXFMT), reason="the reference tree is not on this machine")
def test_mxmm_against_reference_oracle():
    """every entry bit-equal to the left-to-right binary64 sum of exact block terms that the reference's verification script computes with rationals,
    and the sum of |terms| equal to its value; then the refusals of the unit"""
    pytest.importorskip("ml_dtypes")
    import importlib.util
    spec = importlib.util.spec_from_file_location("mxfmt_check", MXFMT); m = importlib.util.module_from_spec(spec); spec.loader.exec_module(m)
    dots = 0
    for (fmt, mm, nn, k, A, SA, B, SB) in mx_cases(m):
        exact, seq, babs, kb = m.mx_reference(fmt, mm, nn, k, A, SA, B, SB)
        rc, got, mag = orc.mxmm(fmt, mm, nn, k, A, SA, B, SB)
        assert rc == 0
        assert got.reshape(-1).tolist() == [float(v) for v in seq]                 # bit-equal (== on floats; no NaN occurs)
        assert np.allclose(mag.reshape(-1), [float(v) for v in babs], rtol=1e-15, atol=0)
        dots += mm * nn
    assert dots >= 3000
    z = np.zeros(64, np.uint8)
    assert orc.mxmm(3, 1, 1, 32, z, z, z, z)[0] == 5 and orc.mxmm(0, 1, 1, 0, z, z, z, z)[0] == 5 and orc.mxmm(1, 1, 1, 48, z, z, z, z)[0] == 5
    bad = z.copy(); bad[0] = 255
    assert orc.mxmm(1, 1, 1, 32, z, bad, z, z)[0] == 5 and orc.mxmm(2, 1, 1, 32, z, z, z, bad)[0] == 5     # E8M0 255
    bad[0] = 127
    assert orc.mxmm(0, 1, 1, 16, z, bad, z, z)[0] == 5 and orc.mxmm(2, 1, 1, 32, bad, z, z, z)[0] == 5     # UE4M3 NaN scale, E4M3 NaN element


# ------------------------------------------------------------------ NVFP4 encoder (native/models/nvfp4.om: nvfp4enc, nvfp4scale; checked as tests/models/mxfmt-check.py:302-352 checks the unit)
def test_nvfp4_encoder_against_quotient_oracle_and_ml_dtypes():
    """every non-NaN bfloat16 value under every valid scale against the binary64 quotient placed among the E2M1 midpoints (ties to the even code, above 6
    saturating); +-1 ulp around every threshold against exact rationals; round trip of every element; the block scale against ml_dtypes' e4m3 cast"""
    ml = pytest.importorskip("ml_dtypes")
    from fractions import Fraction
    F4 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
    bf = np.arange(65536, dtype=np.uint32) << 16
    bf = bf[(bf & 0x7FFFFFFF) <= 0x7F800000]
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    sval = np.arange(127, dtype=np.uint8).view(ml.float8_e4m3fn).astype(np.float64)
    x = bf.view(np.float32).astype(np.float64); neg = (bf >> 31).astype(np.uint32)
    for s in range(127):
        got = orc.nvfp4_enc(bf, s)
        if sval[s] == 0:
            want = neg << 3
        else:
            q = np.abs(x) / sval[s]
            c = np.searchsorted(mids, q, side="left").astype(np.uint32)
            c = np.minimum(np.where(np.isin(q, mids) & (c % 2 == 1), c + 1, c), 7)
            want = (neg << 3) | c
        assert np.array_equal(got, want.astype(np.uint8)), s
    f32 = lambda v: np.array([v], np.float32).view(np.uint32)[0]
    for s in range(1, 127):
        sv = Fraction(float(sval[s])); pts = []
        for m in (Fraction(1, 4), Fraction(3, 4), Fraction(5, 4), Fraction(7, 4), Fraction(5, 2), Fraction(7, 2), Fraction(5), Fraction(6), Fraction(7)):
            b = int(f32(float(m * sv))); pts += [b - 1, b, b + 1]
        got = orc.nvfp4_enc(np.array(pts, np.uint32), s)
        for b, g in zip(pts, got):
            xq = Fraction(float(np.array([b], np.uint32).view(np.float32)[0])) / sv
            assert int(g) == min(range(8), key=lambda k: (abs(xq - Fraction(F4[k])), k % 2)), (s, hex(b))
        dec = np.array([orc.nvfp4_bits(n, s) for n in range(16)], np.uint32)
        assert orc.nvfp4_enc(dec, s).tolist() == list(range(16))                  # round trip
    assert orc.nvfp4_enc(np.array([0x7fc00000], np.uint32), 5)[0] == 0xff and orc.nvfp4_enc(np.array([0], np.uint32), 127)[0] == 0xff   # NaN input, NaN scale: the unit traps
    rng = np.random.default_rng(20261026)
    am = np.concatenate([(np.arange(65536, dtype=np.uint32) << 16)[:0x7F81], rng.integers(0, 0x7F800001, 200000, dtype=np.uint32)]).astype(np.uint32)
    q = (am.view(np.float32) / np.float32(6.0)).astype(np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        c = q.astype(ml.float8_e4m3fn).view(np.uint8).astype(np.uint32)
    c = np.where((c & 127) == 0x7F, 0x7E, c)                                       # saturating mode: what overflows becomes the largest finite code
    assert np.array_equal(orc.nvfp4_scale(am), c.astype(np.uint8))
