"""Regenerates tests/golden/*.npz from the reference's own host code (oracle/_ref/libref*.so, built by
`make -C oracle ref` from the reference sources). Run where the reference tree is present:

    python tests/golden/make_golden.py

Inputs are seeded; the outputs are what the reference functions returned. The vectors are small on purpose
(a few hundred KB) and travel with the repository, unlike the reference build itself.
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as orc  # noqa: E402
from tests.test_oracle_pin import plan_cases, router_case, emu_case, ref_emu, pq_case, mc_case  # noqa: E402

U8P, U16P, U32P, U64P, F32P, F64P = orc.U8P, orc.U16P, orc.U32P, orc.U64P, orc.F32P, orc.F64P
p = lambda a, t: a.ctypes.data_as(t)


def main():
    R = orc.ref_lib(); G = orc.ref_group_lib()
    if R is None or G is None:
        raise SystemExit("reference build not present: run `make -C oracle ref` first")
    rng = np.random.default_rng(2026)
    out = {}
    out["e4m3_decode"] = np.array([R.omega_fp8_e4m3_ref(i) for i in range(256)], np.float32)
    v = np.concatenate([rng.normal(0, 120, 3000), rng.normal(0, 0.02, 3000), rng.uniform(-460, 460, 2000)]).astype(np.float32)
    out["encode_in"] = v
    out["encode_out"] = np.array([R.omega_gpu_fp8_e4m3_rne(C.c_float(float(x))) for x in v], np.uint8)
    out["bf16_out"] = np.array([R.omega_fp32_to_bf16(C.c_float(float(x))) for x in v], np.uint16)
    # quantiser + double GEMV on a seeded 256 x 512 weight (N(0, 0.02) as the benchmark configurations)
    n, k = 256, 512
    w = orc.bf16_bits(rng.normal(0, 0.02, (n, k)).astype(np.float32)); w[128:, :128] = 0
    w8 = np.empty((n, k), np.uint8); sc = np.empty((n // 128, k // 128), np.uint16)
    assert R.omega_gpu_fp8_quantize_bf16(C.c_uint32(n), C.c_uint32(k), p(w, U16P), p(w8, U8P), p(sc, U16P)) == 0
    x = rng.normal(0, 1, k).astype(np.float32)
    y = np.empty(n, np.float64); m = np.empty(n, np.float64)
    R.omega_fp8_gemv_oracle(p(w8, U8P), p(sc, U16P), C.c_uint32(n), C.c_uint32(k), p(x, F32P), p(y, F64P), p(m, F64P))
    out.update(q_w=w, q_w8=w8, q_scale=sc, gemv_x=x, gemv_y=y, gemv_mag=m)
    # routing plan: every case of the reference's own plan test, outputs concatenated
    rcs, blobs = [], []
    for cfg, ids, _ in plan_cases():
        bufs = orc.plan_buffers()
        r = C.c_uint64(99)
        assert R.omega_moe_plan(C.byref(r), p(cfg, U64P), C.c_uint64(8), p(ids, U64P), C.c_uint64(1024), p(bufs[0], U64P), C.c_uint64(10368),
                                p(bufs[1], U64P), C.c_uint64(1028), p(bufs[2], U64P), C.c_uint64(2320), p(bufs[3], U64P), C.c_uint64(8)) == 0
        rcs.append(r.value)
        nw = int(bufs[3][0]) if r.value == 0 else 0
        ns = int(bufs[3][1]) if r.value == 0 else 0
        # keep the written prefix only (the rest is the 0x5a fill, checked separately)
        blobs.append(np.concatenate([bufs[0][: nw * 9], bufs[1][: ns * 4], bufs[2][: nw + 8], bufs[2][1160: 1160 + nw + 8], bufs[3]]) if r.value == 0 else np.zeros(0, np.uint64))
    out["plan_rc"] = np.array(rcs, np.uint64)
    out["plan_len"] = np.array([len(b) for b in blobs], np.uint64)
    out["plan_blob"] = np.concatenate(blobs).astype(np.uint32)  # every value fits 32 bits
    assert np.array_equal(out["plan_blob"].astype(np.uint64), np.concatenate(blobs))
    # the incumbent host GROUP on a 64-token, 8-of-128 routing table
    ids = np.stack([rng.choice(128, 8, replace=False) for _ in range(64)]).astype(np.uint32)
    ox = np.zeros(1168, np.uint32); oy = np.zeros(1168, np.uint32); os_ = np.zeros(1028, np.uint32)
    ns = G.moe_incumbent(C.c_uint32(64), p(ids, U32P), p(ox, U32P), p(oy, U32P), p(os_, U32P))
    out.update(grp_ids=ids, grp_x=ox[:576], grp_y=oy[:576], grp_seg=os_[: ns * 4])
    # router front half: the double oracle inside the reference's own router test, on seeded cases (inputs are regenerated from the seeds)
    RR = orc.ref_router_lib()
    if RR is None:
        raise SystemExit("reference router oracle not present: run `make -C oracle ref` first")
    seeds = [(11, 1.0, 1), (12, 1.0, 0), (13, 0.01, 1), (14, 50.0, 1), (15, 1.0, 1), (16, 3.0, 0)]
    r_ids, r_w, r_lg, r_xn, r_m = [], [], [], [], []
    for seed, xscale, norm in seeds:
        x, nw, gate = router_case(seed, xscale)
        xn = np.empty(2048, np.float64); lg = np.empty(128, np.float64); ids = np.empty(8, np.uint32); w = np.empty(8, np.float64); m = C.c_double(0)
        RR.ref_router_oracle(p(x, F32P), p(nw, F32P), p(gate, U16P), C.c_int(norm), p(xn, F64P), p(lg, F64P), p(ids, U32P), p(w, F64P), C.byref(m))
        r_ids.append(ids.copy()); r_w.append(w.copy()); r_lg.append(lg.copy()); r_xn.append(xn[::16].copy()); r_m.append(m.value)
    out.update(router_seeds=np.array(seeds, np.float64), router_ids=np.stack(r_ids), router_w=np.stack(r_w), router_logits=np.stack(r_lg),
               router_xn16=np.stack(r_xn), router_margin=np.array(r_m))
    # three static functions of the reference's own tests, compiled in place (oracle/ref_static_shims.c)
    EMU, PQ, MC = orc.ref_static_lib("emu"), orc.ref_static_lib("pq"), orc.ref_static_lib("mc")
    if EMU is None or PQ is None or MC is None:
        raise SystemExit("reference static-function shims not present: run `make -C oracle ref` first")
    emu_seeds = [(21, 128, 512), (22, 128, 768), (23, 128, 2048)]           # inputs are regenerated from the seeds
    out["emu_seeds"] = np.array(emu_seeds, np.uint32)
    out["emu_y"] = np.concatenate([ref_emu(*emu_case(*c)) for c in emu_seeds])
    x = pq_case(8, 512)                                                     # the reference generator's own stream: kept as data
    q = np.empty((8, 512), np.uint8); s_ = np.empty((8, 4), np.float32)
    for r in range(8):
        PQ.ref_pq(p(x[r], F32P), C.c_uint32(512), p(q[r], U8P), p(s_[r], F32P))
    out.update(pq_x=x, pq_q=q, pq_s=s_)
    down, inv, wt = mc_case(31, 6, 256, 8)
    ref = np.empty((6, 256), np.float32)
    MC.ref_mc(p(down, F32P), p(inv, U32P), p(wt, F32P), C.c_uint32(6), C.c_uint32(256), C.c_uint32(8), p(ref, F32P))
    out["mc_out"] = ref
    # NVFP4 element x scale: the exact rationals of the reference's verification script (tests/models/mxfmt-check.py: e2m1, ue4m3), as binary32 bits
    import importlib.util
    from tests.test_oracle_pin import MXFMT
    spec = importlib.util.spec_from_file_location("mxfmt_check", MXFMT); mx = importlib.util.module_from_spec(spec); spec.loader.exec_module(mx)
    tab = np.empty((16, 127), np.uint32)
    for n in range(16):
        for c in range(127):
            v = mx.e2m1(n) * mx.ue4m3(c)
            tab[n, c] = mx.frac_to_f32bits(abs(v)) | ((n & 8) << 28)        # the sign of a zero product is the element's
    out["nvfp4_bits"] = tab
    # block-scaled products: inputs from the reference script's generator, results from its rational oracle (left-to-right binary64 sums)
    from tests.test_oracle_pin import mx_cases
    hdr, blobs, res = [], [], []
    for (fmt, mm, nn, k, A, SA, B, SB) in mx_cases(mx, rounds=2, seed=2027):
        kb = k // mx.BS[fmt]; eb = k // 2 if fmt < 2 else k
        _, seq, babs, _ = mx.mx_reference(fmt, mm, nn, k, A, SA, B, SB)
        hdr.append((fmt, mm, nn, k))
        blobs.append(np.concatenate([A[:eb * mm], SA[:kb * mm], B[:eb * nn], SB[:kb * nn]]))
        res.append(np.array([float(v) for v in seq], np.float64))
    out.update(mx_hdr=np.array(hdr, np.uint32), mx_blob=np.concatenate(blobs), mx_res=np.concatenate(res))
    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_vectors.npz"), {k_: v_.shape for k_, v_ in out.items()})


if __name__ == "__main__":
    main()
