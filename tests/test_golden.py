"""The CPU checker against the committed golden vectors (outputs of the reference's own host code; see
tests/golden/make_golden.py). Runs without the reference tree."""
import ctypes as C
import os

import numpy as np

from oracle import oracle as orc
from tests.test_oracle_pin import plan_cases, router_case, emu_case, mc_case

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))


def test_formats():
    L = orc.lib()
    mine = np.array([L.orc_e4m3_decode(i) for i in range(256)], np.float32)
    assert np.array_equal(mine.view(np.uint32)[np.isfinite(mine)], G["e4m3_decode"].view(np.uint32)[np.isfinite(mine)])
    assert np.array_equal(np.isnan(mine), np.isnan(G["e4m3_decode"]))
    v = G["encode_in"]
    assert np.array_equal(np.array([L.orc_e4m3_encode(C.c_float(float(x))) for x in v], np.uint8), G["encode_out"])
    assert np.array_equal(orc.bf16_bits(v), G["bf16_out"])


def test_quantiser_and_gemv():
    w8, sc = orc.quantize_bf16(G["q_w"])
    assert np.array_equal(w8, G["q_w8"]) and np.array_equal(sc, G["q_scale"])
    y, m = orc.gemv(w8, sc, G["gemv_x"], mag=True)
    assert np.array_equal(y, G["gemv_y"]) and np.array_equal(m, G["gemv_mag"])


def test_plan_cases():
    blob = G["plan_blob"].astype(np.uint64); at = 0
    for (cfg, ids, name), rc, ln in zip(plan_cases(), G["plan_rc"], G["plan_len"]):
        work, seg, maps, meta = orc.plan_buffers()
        assert orc.moe_plan(cfg, ids, work, seg, maps, meta) == rc, name
        if rc == 0:
            nw, ns = int(meta[0]), int(meta[1])
            got = np.concatenate([work[: nw * 9], seg[: ns * 4], maps[: nw + 8], maps[1160: 1160 + nw + 8], meta])
            assert np.array_equal(got, blob[at: at + int(ln)]), name
            fill = np.uint64(0x5A5A5A5A5A5A5A5A)  # nothing past the written prefix is touched
            assert np.all(work[nw * 9:] == fill) and np.all(seg[ns * 4:] == fill) and np.all(maps[nw + 8: 1160] == fill)
        else:
            assert all(np.all(b == np.uint64(0x5A5A5A5A5A5A5A5A)) for b in (work, seg, maps, meta)), name
        at += int(ln)
    assert at == len(blob)


def test_incumbent_group():
    g = orc.plan_global(G["grp_ids"], 128, ystride=9)
    assert np.array_equal(g["xmap"][:512], G["grp_x"][:512]) and np.array_equal(g["ymap"][:512], G["grp_y"][:512])
    seg = G["grp_seg"].reshape(-1, 4)
    assert np.array_equal(g["seg3"], seg[:-1, :3]) and tuple(seg[-1]) == (256, 512, 64, 1)


def test_router_front_half():
    """the checker's router (RMSNorm, bf16 gate GEMV, top-8, weights) against the double oracle of the reference's own router test"""
    for i, (seed, xscale, norm) in enumerate(G["router_seeds"]):
        x, nw, gate = router_case(int(seed), float(xscale))
        xn, lg, ids, w, m = orc.router(x[None], nw, gate, 1e-6, 8, bool(norm))
        assert np.array_equal(ids[0], G["router_ids"][i])
        assert np.array_equal(lg[0], G["router_logits"][i]) and np.array_equal(xn[0][::16], G["router_xn16"][i])
        assert np.max(np.abs(w[0] - G["router_w"][i])) <= 1e-15 and abs(m[0] - G["router_margin"][i]) <= 1e-15


def test_gemv_emulation():
    """the kernels' f32 summation order against emu_row of the reference's grouped-GEMM test"""
    at = 0
    for seed, n, k in G["emu_seeds"]:
        w8, sc, x = emu_case(int(seed), int(n), int(k))
        assert np.array_equal(orc.gemv_emu(w8, sc, x).view(np.uint32), G["emu_y"][at: at + int(n)].view(np.uint32))
        at += int(n)


def test_act_quant():
    """activation quantiser against pq_ref of the reference's FP8 x FP8 GEMM test, on that test's own input stream"""
    q, s = orc.act_quant(G["pq_x"])
    assert np.array_equal(q, G["pq_q"]) and np.array_equal(s.view(np.uint32), G["pq_s"].view(np.uint32))


def test_combine_prefill_form():
    """slot-order multiply-then-add combine against mc_ref of the reference's prefill host-kernel test"""
    down, inv, wt = mc_case(31, 6, 256, 8)
    assert np.array_equal(orc.combine_mc(down, inv, wt).view(np.uint32), G["mc_out"].view(np.uint32))


def test_nvfp4_decode_table():
    """every NVFP4 element x scale pair against the table made from the reference's verification script"""
    mine = np.array([orc.nvfp4_bits(n, c) for n in range(16) for c in range(127)], np.uint32).reshape(16, 127)
    assert np.array_equal(mine, G["nvfp4_bits"])


def test_block_scaled_products():
    """C = A B^T of two block-scaled operands (NVFP4, MXFP4, MXFP8) against results of the reference's rational oracle, bit for bit"""
    pos = rpos = 0
    for fmt, m, n, k in G["mx_hdr"].tolist():
        bs = 16 if fmt == 0 else 32
        kb, eb = k // bs, (k // 2 if fmt < 2 else k)
        A = G["mx_blob"][pos:pos + eb * m]; pos += eb * m
        SA = G["mx_blob"][pos:pos + kb * m]; pos += kb * m
        B = G["mx_blob"][pos:pos + eb * n]; pos += eb * n
        SB = G["mx_blob"][pos:pos + kb * n]; pos += kb * n
        rc, got, _ = orc.mxmm(fmt, m, n, k, A, SA, B, SB)
        assert rc == 0 and np.array_equal(got.reshape(-1).view(np.uint64), G["mx_res"][rpos:rpos + m * n].view(np.uint64))
        rpos += m * n
    assert pos == len(G["mx_blob"]) and rpos == len(G["mx_res"])
