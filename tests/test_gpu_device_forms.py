"""The stream-ordered device forms (_async / _dev) of the C-ABI, each against the host-staged entry or the checker it must agree with.

These are the forms a serving process uses (device pointers in, nothing staged, nothing read back); the host-staged entries that the
other GPU tests call go through the same kernels but not through these argument paths. W4 is run at the full size of the benchmark's
W4 configuration (x bf16 [16, 4096], W int4 [4096, 4096], fp16 scale per 32) against the double self-oracle: the reference has no
integer-W4 arithmetic, so that parity is unpinned.
"""
import ctypes as C

import numpy as np
import pytest

from cudapp_b200 import api
from oracle import oracle as orc
from tests.test_gpu_ops import make_weights, rel_l2

pytestmark = pytest.mark.gpu


def dev(a):
    import torch
    a = np.ascontiguousarray(a)
    view = {np.dtype(np.uint32): np.int32, np.dtype(np.uint16): np.int16, np.dtype(np.uint64): np.int64}.get(a.dtype)
    return torch.from_numpy(a.view(view) if view else a).to("cuda:0")


def va(t):
    return C.c_uint64(t.data_ptr())


def group_table(t, ids):
    tab = np.empty((len(ids), 2), np.uint64)
    for i, e in enumerate(ids):
        w, s = C.c_uint64(), C.c_uint64()
        assert api.lib.omega_gpu_fp8_tensor_entry(t, C.c_uint32(int(e)), C.byref(w), C.byref(s)) == 0
        tab[i] = (w.value, s.value)
    return tab


def test_gemv_grouped_dev_and_async():
    """grouped GEMV, device forms: the _dev entry takes a row that carries the reference router's 2^64 fold and removes it exactly
    (src/omega_gpu_fp8_api.h:115-118); the _async entry takes plain rows, shared or one per group, f32 or bf16"""
    import torch
    rng = np.random.default_rng(31)
    E, n, k, groups = 12, 256, 1024, 8
    w8, sc = make_weights(rng, E, n, k)
    rc, t = api.fp8_tensor_upload(E, n, k, w8, sc); assert rc == 0, api.last_error()
    ids = rng.choice(E, groups, replace=False).astype(np.uint32)
    x1 = rng.normal(0, 1, (1, k)).astype(np.float32)
    rc, want = api.fp8_gemv_grouped_f32(t, ids, x1); assert rc == 0, api.last_error()
    d_tab = dev(group_table(t, ids))
    d_xf = dev((x1 * np.float32(2.0 ** 64)).astype(np.float32))           # exact: a power of two
    y = np.empty((groups, n), np.float32)
    info = api.Fp8Info()
    rc = api.lib.omega_gpu_fp8_gemv_grouped_dev(t, C.c_uint32(groups), va(d_tab), va(d_xf), y.ctypes.data_as(C.c_void_p), C.byref(info))
    assert rc == 0, api.last_error()
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32)) and info.groups == groups
    assert api.lib.omega_gpu_fp8_gemv_grouped_dev(t, C.c_uint32(groups), C.c_uint64(0), va(d_xf), y.ctypes.data_as(C.c_void_p), None) == api.BAD_ARGS
    # _async: shared f32 row, then one bf16 row per group
    s = torch.cuda.Stream()
    d_x1 = dev(x1); d_y = torch.full((groups, n), -999.0, dtype=torch.float32, device="cuda:0")
    torch.cuda.synchronize()
    rc = api.lib.omega_gpu_fp8_gemv_grouped_async(t, C.c_uint32(groups), va(d_tab), va(d_x1), C.c_uint32(1), C.c_int(0), va(d_y), C.c_void_p(s.cuda_stream))
    assert rc == 0, api.last_error()
    s.synchronize()
    assert np.array_equal(d_y.cpu().numpy().view(np.uint32), want.view(np.uint32))
    xg = orc.bf16_bits(rng.normal(0, 1, (groups, k)).astype(np.float32))
    rc, want_g = api.fp8_gemv_grouped_f32(t, ids, orc.bf16_to_f32(xg)); assert rc == 0, api.last_error()
    d_xg = dev(xg); d_y.fill_(-999.0); torch.cuda.synchronize()
    rc = api.lib.omega_gpu_fp8_gemv_grouped_async(t, C.c_uint32(groups), va(d_tab), va(d_xg), C.c_uint32(groups), C.c_int(1), va(d_y), C.c_void_p(s.cuda_stream))
    assert rc == 0, api.last_error()
    s.synchronize()
    assert np.array_equal(d_y.cpu().numpy().view(np.uint32), want_g.view(np.uint32))
    assert api.lib.omega_gpu_fp8_gemv_grouped_async(t, C.c_uint32(groups), va(d_tab), va(d_xg), C.c_uint32(3), C.c_int(1), va(d_y), C.c_void_p(s.cuda_stream)) == api.BAD_ARGS
    api.fp8_tensor_free(t)


def test_fp8gemm_async_with_and_without_maps():
    """row-table GEMM, device form (the reference's record entry, src/omega_gpu_fp8gemm_api.h:103): segment records from the device
    plan; without maps row p reads x row p and writes y row p, with maps it reads x[XMAP[p]] and writes y[YMAP[p]]"""
    import torch
    rng = np.random.default_rng(32)
    E, n, k, T, S = 10, 256, 512, 21, 3
    w8, sc = make_weights(rng, E, n, k)
    rc, t = api.fp8_tensor_upload(E, n, k, w8, sc); assert rc == 0, api.last_error()
    picks = np.stack([rng.choice(E, S, replace=False) for _ in range(T)]).astype(np.uint32)
    x = rng.uniform(-2, 2, (T, k)).astype(np.float32)
    g = orc.plan_global(picks, E, ystride=S)
    R = g["rows"]
    ids_sorted = np.repeat(np.arange(E, dtype=np.uint32), g["counts"])
    rc, want = api.fp8gemm(t, ids_sorted, g["xmap"][:R], x); assert rc == 0, api.last_error()    # sorted row p <- x[xmap[p]]
    # the device plan builds the segment records (directory = the tensor's own entries)
    d_dir = dev(group_table(t, np.arange(E)))
    d_ids = dev(picks)
    d_counts = torch.zeros(E, dtype=torch.int32, device="cuda:0"); d_starts = torch.zeros_like(d_counts)
    d_xmap = torch.zeros(R + 8, dtype=torch.int32, device="cuda:0"); d_ymap = torch.zeros_like(d_xmap)
    d_seg = torch.zeros(E * 8, dtype=torch.int32, device="cuda:0"); d_hdr = torch.zeros(8, dtype=torch.int32, device="cuda:0")
    o = api.MoePlanOut(d_counts.data_ptr(), d_starts.data_ptr(), d_xmap.data_ptr(), d_ymap.data_ptr(), d_seg.data_ptr(), d_dir.data_ptr(), 0, 0, 0, d_hdr.data_ptr())
    s = torch.cuda.Stream()
    torch.cuda.synchronize()
    rc = api.lib.omega_gpu_moe_plan_async(C.c_uint32(T), C.c_uint32(S), C.c_uint32(E), C.c_uint32(S), C.c_uint32(0), va(d_ids), C.byref(o), C.c_void_p(s.cuda_stream))
    assert rc == 0, api.last_error()
    s.synchronize()
    hdr = d_hdr.cpu().numpy().view(np.uint32)
    assert hdr[0] == R and hdr[3] == 0
    assert np.array_equal(d_counts.cpu().numpy().view(np.uint32), g["counts"]) and np.array_equal(d_starts.cpu().numpy().view(np.uint32), g["starts"])
    assert np.array_equal(d_xmap.cpu().numpy().view(np.uint32), g["xmap"]) and np.array_equal(d_ymap.cpu().numpy().view(np.uint32), g["ymap"])
    segs = int(hdr[1])
    d_x = dev(x)
    # with maps: y row ymap[p] = token * S + slot
    d_y = torch.full((T * S, n), -999.0, dtype=torch.float32, device="cuda:0"); torch.cuda.synchronize()
    rc = api.lib.omega_gpu_fp8gemm_async(t, C.c_uint32(R), C.c_uint32(segs), va(d_seg), va(d_x), C.c_int(0), va(d_y), va(d_xmap), va(d_ymap), C.c_void_p(s.cuda_stream))
    assert rc == 0, api.last_error()
    s.synchronize()
    got = d_y.cpu().numpy()
    assert np.array_equal(got[g["ymap"][:R]].view(np.uint32), want.view(np.uint32))
    # without maps: the caller gathers x into sorted order itself
    d_xs = dev(x[g["xmap"][:R]]); d_y2 = torch.full((R, n), -999.0, dtype=torch.float32, device="cuda:0"); torch.cuda.synchronize()
    rc = api.lib.omega_gpu_fp8gemm_async(t, C.c_uint32(R), C.c_uint32(segs), va(d_seg), va(d_xs), C.c_int(0), va(d_y2), C.c_uint64(0), C.c_uint64(0), C.c_void_p(s.cuda_stream))
    assert rc == 0, api.last_error()
    s.synchronize()
    assert np.array_equal(d_y2.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # one map without the other is refused
    assert api.lib.omega_gpu_fp8gemm_async(t, C.c_uint32(R), C.c_uint32(segs), va(d_seg), va(d_x), C.c_int(0), va(d_y), va(d_xmap), C.c_uint64(0), C.c_void_p(s.cuda_stream)) == api.BAD_ARGS
    api.fp8_tensor_free(t)


def test_topk_async_and_residual_norm_async():
    import torch
    rng = np.random.default_rng(33)
    T, E, K, H = 37, 128, 8, 1024
    logits = orc.bf16_bits(np.round(rng.normal(0, 1, (T, E)) * 4) / 4)       # coarse values: many ties, the lowest index must win
    d_lg = dev(logits); d_ids = torch.zeros((T, K), dtype=torch.int32, device="cuda:0"); d_w = torch.zeros((T, K), dtype=torch.float32, device="cuda:0")
    s = torch.cuda.Stream(); torch.cuda.synchronize()
    rc = api.lib.omega_gpu_moe_topk_async(C.c_uint32(T), C.c_uint32(E), C.c_uint32(K), C.c_int(1), va(d_lg), va(d_ids), va(d_w), C.c_void_p(s.cuda_stream))
    assert rc == 0, api.last_error()
    s.synchronize()
    rid, rw = orc.topk(orc.bf16_to_f32(logits), K, True)
    assert np.array_equal(d_ids.cpu().numpy().view(np.uint32), rid) and np.max(np.abs(d_w.cpu().numpy() - rw)) <= 1e-5
    # residual step: h = bf16->f32(x16), xn = bf16(RMSNorm(h)); then h += m, h16 = bf16(h)
    x16 = orc.bf16_bits(rng.normal(0, 1.5, (T, H)).astype(np.float32)); m = rng.normal(0, 0.3, (T, H)).astype(np.float32)
    d_x16 = dev(x16); d_m = dev(m)
    d_h = torch.zeros((T, H), dtype=torch.float32, device="cuda:0"); d_xn = torch.zeros((T, H), dtype=torch.int16, device="cuda:0"); d_h16 = torch.zeros_like(d_xn)
    torch.cuda.synchronize()
    rc = api.lib.omega_gpu_residual_norm_async(C.c_uint32(T), C.c_uint32(H), C.c_float(1e-6), va(d_x16), C.c_uint64(0), va(d_h), va(d_xn), C.c_uint64(0), C.c_void_p(s.cuda_stream))
    assert rc == 0, api.last_error()
    s.synchronize()
    h0 = orc.bf16_to_f32(x16)
    assert np.array_equal(d_h.cpu().numpy(), h0)
    assert np.array_equal(d_xn.cpu().numpy().view(np.uint16), orc.bf16_bits(orc.rmsnorm(h0, 1e-6)))
    rc = api.lib.omega_gpu_residual_norm_async(C.c_uint32(T), C.c_uint32(H), C.c_float(1e-6), C.c_uint64(0), va(d_m), va(d_h), va(d_xn), va(d_h16), C.c_void_p(s.cuda_stream))
    assert rc == 0, api.last_error()
    s.synchronize()
    h1 = h0 + m
    assert np.array_equal(d_h.cpu().numpy(), h1) and np.array_equal(d_h16.cpu().numpy().view(np.uint16), orc.bf16_bits(h1))
    assert np.array_equal(d_xn.cpu().numpy().view(np.uint16), orc.bf16_bits(orc.rmsnorm(h1, 1e-6)))
    assert api.lib.omega_gpu_residual_norm_async(C.c_uint32(0), C.c_uint32(H), C.c_float(1e-6), C.c_uint64(0), va(d_m), va(d_h), va(d_xn), va(d_h16), C.c_void_p(s.cuda_stream)) == api.BAD_ARGS


def test_w4_gemm_full_size():
    """the benchmark's W4 configuration at its own size: 16 x 4096 activations, 4096 x 4096 int4 weights; double self-oracle (parity unpinned:
    no reference W4), the benchmark's bars on the unrounded f32 result and on the bf16 output"""
    rng = np.random.default_rng(41)
    n, k, m = 4096, 4096, 16
    packed, sc = orc.w4_quantize(rng.normal(0, 0.02, (n, k)).astype(np.float32))
    xb = orc.bf16_bits(rng.normal(0, 1, (m, k)).astype(np.float32))
    rc, t, _ = api.w4_upload(packed, sc); assert rc == 0, api.last_error()
    rc, y16, y32 = api.w4_gemm_bf16(t, n, xb); assert rc == 0, api.last_error()
    ref = orc.w4_gemm(packed, sc, orc.bf16_to_f32(xb))
    assert np.max(np.abs(y32 - ref)) <= 1e-2 and rel_l2(y32, ref) <= 1e-3, (float(np.max(np.abs(y32 - ref))), rel_l2(y32, ref))
    assert np.array_equal(y16, orc.bf16_bits(y32))
    api.lib.omega_gpu_w4_free(t)


@pytest.mark.parametrize("n,k,m", [(256, 1024, 16), (128, 2048, 21), (4096, 4096, 16), (256, 768, 19)])
def test_mxfp4_gemm(n, k, m):
    """MXFP4 weights (E2M1 + E8M0 per 32: docs/models/MXFP4.md of the reference) times bf16 activations against the double checker, whose element
    decoder equals the reference's own verification oracle record for record (tests/test_oracle_pin.py). Every nibble value and a wide range of
    scales occur, among them scale 0 (2^-127) and large ones; the NaN scale is refused at upload."""
    rng = np.random.default_rng(n + k)
    packed = rng.integers(0, 256, (n, k // 2)).astype(np.uint8)
    scale = rng.integers(110, 135, (n, k // 32)).astype(np.uint8)
    scale[0, 0] = 0; scale[1, 1] = 1; scale[n - 1, k // 32 - 1] = 140
    xb = orc.bf16_bits(rng.normal(0, 1, (m, k)).astype(np.float32))
    t = C.c_void_p()
    bad = scale.copy(); bad[3, 2] = 255
    assert api.lib.omega_gpu_mxfp4_upload(C.c_uint32(n), C.c_uint32(k), packed.ctypes.data_as(C.c_void_p), bad.ctypes.data_as(C.c_void_p), C.byref(t)) == api.NAN_WEIGHT and not t.value
    assert api.lib.omega_gpu_mxfp4_upload(C.c_uint32(n), C.c_uint32(k + 32), packed.ctypes.data_as(C.c_void_p), scale.ctypes.data_as(C.c_void_p), C.byref(t)) == api.BAD_ARGS
    assert api.lib.omega_gpu_mxfp4_upload(C.c_uint32(n), C.c_uint32(k), packed.ctypes.data_as(C.c_void_p), scale.ctypes.data_as(C.c_void_p), C.byref(t)) == 0, api.last_error()
    rc, y16, y32 = api.w4_gemm_bf16(t, n, xb); assert rc == 0, api.last_error()
    ref = orc.mxfp4_gemm(packed, scale, orc.bf16_to_f32(xb))
    mag = orc.mxfp4_gemm(packed & 0x77, scale, np.abs(orc.bf16_to_f32(xb)))                 # sum of |terms|: the reference's own error measure for a dot product
    assert np.all(np.abs(y32 - ref) <= 1e-5 * mag + 1e-30), float(np.max(np.abs(y32 - ref) / (mag + 1e-30)))
    assert rel_l2(y32, ref) <= 1e-3 and np.array_equal(y16, orc.bf16_bits(y32))
    rc, _, yb = api.w4_gemm_bf16(t, n, xb); assert rc == 0 and np.array_equal(yb.view(np.uint32), y32.view(np.uint32))
    api.lib.omega_gpu_w4_free(t)


@pytest.mark.parametrize("n,k,m", [(256, 1024, 16), (128, 2048, 21), (4096, 4096, 16), (256, 768, 19)])
def test_nvfp4_gemm(n, k, m):
    """NVFP4 weights (E2M1 + one unsigned E4M3 scale per 16 columns: native/models/nvfp4.om of the reference) times bf16 activations against the
    double checker, whose element x scale decoder equals the reference's verification oracle for every pair (tests/test_oracle_pin.py). Every nibble
    and every valid scale code occur (zero and subnormal scales among them); NaN and sign-set scales are refused at upload."""
    rng = np.random.default_rng(n + k + 1)
    packed = rng.integers(0, 256, (n, k // 2)).astype(np.uint8)
    scale = rng.integers(0, 127, (n, k // 16)).astype(np.uint8)
    scale[0, 0] = 0; scale[1, 1] = 1; scale[n - 1, k // 16 - 1] = 126
    xb = orc.bf16_bits(rng.normal(0, 1, (m, k)).astype(np.float32))
    t = C.c_void_p()
    up = lambda kk, sc: api.lib.omega_gpu_nvfp4_upload(C.c_uint32(n), C.c_uint32(kk), packed.ctypes.data_as(C.c_void_p), sc.ctypes.data_as(C.c_void_p), C.byref(t))
    bad = scale.copy(); bad[3, 2] = 127
    assert up(k, bad) == api.NAN_WEIGHT and not t.value
    bad[3, 2] = 0x88
    assert up(k, bad) == api.BAD_ARGS and not t.value
    assert up(k + 32, scale) == api.BAD_ARGS
    assert up(k, scale) == 0, api.last_error()
    rc, y16, y32 = api.w4_gemm_bf16(t, n, xb); assert rc == 0, api.last_error()
    ref = orc.nvfp4_gemm(packed, scale, orc.bf16_to_f32(xb))
    mag = orc.nvfp4_gemm(packed & 0x77, scale, np.abs(orc.bf16_to_f32(xb)))                 # sum of |terms|
    assert np.all(np.abs(y32 - ref) <= 1e-5 * mag + 1e-30), float(np.max(np.abs(y32 - ref) / (mag + 1e-30)))
    assert rel_l2(y32, ref) <= 1e-3 and np.array_equal(y16, orc.bf16_bits(y32))
    rc, _, yb = api.w4_gemm_bf16(t, n, xb); assert rc == 0 and np.array_equal(yb.view(np.uint32), y32.view(np.uint32))
    api.lib.omega_gpu_w4_free(t)


def test_hbm_probe():
    """the in-process bandwidth probe bench.py reports beside the roofline: plausible figures for an HBM3e part, sizes outside its range refused"""
    cg, rg = C.c_float(0), C.c_float(0)
    assert api.lib.omega_gpu_hbm_peak(C.c_uint64(1 << 20), C.c_uint32(2), C.byref(cg), C.byref(rg)) == api.BAD_ARGS      # below 256 MiB: L2 would serve it
    assert api.lib.omega_gpu_hbm_peak(C.c_uint64(256 << 20), C.c_uint32(0), C.byref(cg), C.byref(rg)) == api.BAD_ARGS
    assert api.lib.omega_gpu_hbm_peak(C.c_uint64(256 << 20), C.c_uint32(3), C.byref(cg), C.byref(rg)) == 0, api.last_error()
    assert 1000.0 < cg.value < 10000.0 and 1000.0 < rg.value < 10000.0, (cg.value, rg.value)


@pytest.mark.parametrize("fmt", [0, 1])
def test_fp4_gemm_against_block_scaled_product(fmt):
    """Both operands quantised: the reference's own definition of a block-scaled GEMM (native/models/mxdot.om `mxmm`: exact block terms, added left to
    right in binary64; the checker's restatement is pinned to the reference's rational oracle in tests/test_oracle_pin.py). An FP4 element times its block
    scale is exact in bf16, so the quantised activations go to the 4-bit GEMM as bf16 rows without loss; every block term is then exact in the kernel too
    (sums of small integers times powers of two, or times a 4-bit significand) and only the f32 running sum over blocks rounds: the reference's rule for an
    f32-accumulating kernel, |delta| < 1e-5 x sum of |terms| (tests/gpu_fp8_api_test.c:51)."""
    rng = np.random.default_rng(40 + fmt)
    m, n, k = 16, 256, 1024
    bs = 16 if fmt == 0 else 32
    A = rng.integers(0, 256, (m, k // 2)).astype(np.uint8); B = rng.integers(0, 256, (n, k // 2)).astype(np.uint8)
    if fmt == 0:
        SA = rng.integers(20, 100, (m, k // bs)).astype(np.uint8); SB = rng.integers(0, 127, (n, k // bs)).astype(np.uint8)
        dec = orc.nvfp4_bits
    else:
        SA = rng.integers(117, 137, (m, k // bs)).astype(np.uint8); SB = rng.integers(100, 150, (n, k // bs)).astype(np.uint8)
        dec = orc.mxfp4_bits
    nib = np.stack([A & 15, A >> 4], -1).reshape(m, k)                                   # low nibble = even column
    x = np.array([[dec(int(nib[i, c]), int(SA[i, c // bs])) for c in range(k)] for i in range(m)], np.uint32).view(np.float32)
    xb = orc.bf16_bits(x)
    assert np.array_equal(orc.bf16_to_f32(xb).view(np.uint32), x.view(np.uint32))        # element x scale is exact in bf16
    t = C.c_void_p()
    up = api.lib.omega_gpu_nvfp4_upload if fmt == 0 else api.lib.omega_gpu_mxfp4_upload
    assert up(C.c_uint32(n), C.c_uint32(k), B.ctypes.data_as(C.c_void_p), SB.ctypes.data_as(C.c_void_p), C.byref(t)) == 0, api.last_error()
    rc, y16, y32 = api.w4_gemm_bf16(t, n, xb); assert rc == 0, api.last_error()
    rc, ref, mag = orc.mxmm(fmt, m, n, k, A, SA, B, SB)
    assert rc == 0
    assert np.all(np.abs(y32 - ref) <= 1e-5 * mag + 1e-30), float(np.max(np.abs(y32 - ref) / (mag + 1e-30)))
    assert np.array_equal(y16, orc.bf16_bits(y32))
    api.lib.omega_gpu_w4_free(t)


def test_nvfp4_quantiser_bit_exact():
    """the GPU block quantiser against the checker's restatement of the reference's encoder (pinned in tests/test_oracle_pin.py): magnitudes over forty binades,
    zero blocks, infinities (saturate), every block's scale and nibbles bit for bit; a NaN refuses the call"""
    rng = np.random.default_rng(7)
    rows, k = 128, 1024
    mag = rng.uniform(-30, 10, (rows, k))
    x = (rng.choice([-1.0, 1.0], (rows, k)) * np.exp2(mag) * rng.uniform(1, 2, (rows, k))).astype(np.float32)
    x[::7, :64] = 0.0; x[1::11, 3] = np.inf; x[2::13, 40] = -np.inf
    xb = orc.bf16_bits(x); xr = orc.bf16_to_f32(xb)
    packed = np.zeros((rows, k // 2), np.uint8); scales = np.zeros((rows, k // 16), np.uint8)
    q = lambda w: api.lib.omega_gpu_nvfp4_quantize_bf16(C.c_uint32(rows), C.c_uint32(k), w.ctypes.data_as(C.c_void_p), packed.ctypes.data_as(C.c_void_p), scales.ctypes.data_as(C.c_void_p))
    assert q(xb) == 0, api.last_error()
    wp, ws = orc.nvfp4_quantize(xr)
    assert np.array_equal(scales, ws) and np.array_equal(packed, wp)
    bad = xb.copy(); bad[5, 17] = 0x7fc0
    before = packed.copy()
    assert q(bad) == api.NAN_WEIGHT and np.array_equal(packed, before)
    assert api.lib.omega_gpu_nvfp4_quantize_bf16(C.c_uint32(rows), C.c_uint32(k + 8), xb.ctypes.data_as(C.c_void_p), packed.ctypes.data_as(C.c_void_p), scales.ctypes.data_as(C.c_void_p)) == api.BAD_ARGS
    # what was quantised is a valid tensor for the GEMM entries (no scale code above 126 comes out of the encoder)
    n = rows
    t = C.c_void_p()
    assert api.lib.omega_gpu_nvfp4_upload(C.c_uint32(n), C.c_uint32(k), packed[:n].ctypes.data_as(C.c_void_p), scales[:n].ctypes.data_as(C.c_void_p), C.byref(t)) == 0, api.last_error()
    api.lib.omega_gpu_w4_free(t)


@pytest.mark.parametrize("fmt", [0, 1, 2])
def test_w4_grouped_gemm_by_expert(fmt):
    """4-bit expert weights: the grouped form (one launch over a routing plan's 16-row tiles, rows gathered by xmap, results scattered by ymap) gives,
    for every routed pick, the bits the plain entry gives for that expert's own matrix on that token's row. Formats: int4 + fp16 scales, MXFP4, NVFP4."""
    import torch
    rng = np.random.default_rng(90 + fmt)
    E, n, k, T, S = 8, 256, 1024, 50, 4
    packed = rng.integers(0, 256, (E * n, k // 2)).astype(np.uint8)
    if fmt == 0:
        scale = rng.uniform(0.001, 0.01, (E * n, k // 32)).astype(np.float16).view(np.uint16); up = api.lib.omega_gpu_w4_upload
    elif fmt == 1:
        scale = rng.integers(118, 124, (E * n, k // 32)).astype(np.uint8); up = api.lib.omega_gpu_mxfp4_upload
    else:
        scale = rng.integers(30, 80, (E * n, k // 16)).astype(np.uint8); up = api.lib.omega_gpu_nvfp4_upload
    picks = np.stack([rng.choice(E, S, replace=False) for _ in range(T)]).astype(np.uint32)
    picks[3, 1] = 0xFFFFFFFF                                                         # an absent pick: no row
    xb = orc.bf16_bits(rng.normal(0, 1, (T, k)).astype(np.float32))
    # reference: every expert's own tensor through the plain entry, all token rows
    per = k // 32 if fmt < 2 else k // 16
    want = np.zeros((E, T, n), np.float32)
    for e in range(E):
        te = C.c_void_p()
        assert up(C.c_uint32(n), C.c_uint32(k), packed[e * n:(e + 1) * n].ctypes.data_as(C.c_void_p), np.ascontiguousarray(scale[e * n:(e + 1) * n]).ctypes.data_as(C.c_void_p), C.byref(te)) == 0, api.last_error()
        rc, _, y = api.w4_gemm_bf16(te, n, xb); assert rc == 0, api.last_error()
        want[e] = y
        api.lib.omega_gpu_w4_free(te)
    t = C.c_void_p()
    assert up(C.c_uint32(E * n), C.c_uint32(k), packed.ctypes.data_as(C.c_void_p), scale.ctypes.data_as(C.c_void_p), C.byref(t)) == 0, api.last_error()
    R = T * S
    max_tiles = R // 16 + E + 8
    assert api.lib.omega_gpu_w4_gemm_grouped_async(t, C.c_uint64(1), C.c_uint64(1), C.c_uint64(0), C.c_uint64(0), C.c_uint64(1), C.c_uint64(0), C.c_uint64(1), None) == api.BAD_ARGS   # not reserved
    assert api.lib.omega_gpu_w4_reserve_grouped(t, C.c_uint32(n + 1), C.c_uint32(max_tiles)) == api.BAD_ARGS
    assert api.lib.omega_gpu_w4_reserve_grouped(t, C.c_uint32(n), C.c_uint32(max_tiles)) == 0, api.last_error()
    d_ids = dev(picks)
    d_counts = torch.zeros(E, dtype=torch.int32, device="cuda:0"); d_starts = torch.zeros_like(d_counts)
    d_xmap = torch.zeros(R + 8, dtype=torch.int32, device="cuda:0"); d_ymap = torch.zeros_like(d_xmap)
    d_tiles = torch.zeros(max_tiles * 4, dtype=torch.int32, device="cuda:0"); d_hdr = torch.zeros(8, dtype=torch.int32, device="cuda:0")
    o = api.MoePlanOut(d_counts.data_ptr(), d_starts.data_ptr(), d_xmap.data_ptr(), d_ymap.data_ptr(), 0, 0, 0, 0, d_tiles.data_ptr(), d_hdr.data_ptr())
    s = torch.cuda.Stream(); torch.cuda.synchronize()
    assert api.lib.omega_gpu_moe_plan_async(C.c_uint32(T), C.c_uint32(S), C.c_uint32(E), C.c_uint32(S), C.c_uint32(16), va(d_ids), C.byref(o), C.c_void_p(s.cuda_stream)) == 0, api.last_error()
    d_x = dev(xb); d_y = torch.full((R, n), -999.0, dtype=torch.float32, device="cuda:0"); torch.cuda.synchronize()
    assert api.lib.omega_gpu_w4_gemm_grouped_async(t, va(d_tiles), va(d_hdr), va(d_xmap), va(d_ymap), va(d_x), C.c_uint64(0), va(d_y), C.c_void_p(s.cuda_stream)) == 0, api.last_error()
    s.synchronize()
    got = d_y.cpu().numpy().reshape(T, S, n)
    hdr = d_hdr.cpu().numpy().view(np.uint32)
    assert hdr[3] == 0 and hdr[0] == R - 1 and 0 < hdr[2] <= max_tiles
    for tk in range(T):
        for sl in range(S):
            e = picks[tk, sl]
            if e == 0xFFFFFFFF:
                assert np.all(got[tk, sl] == -999.0)                               # untouched
            else:
                assert np.array_equal(got[tk, sl].view(np.uint32), want[e, tk].view(np.uint32)), (tk, sl)
    api.lib.omega_gpu_w4_free(t)
