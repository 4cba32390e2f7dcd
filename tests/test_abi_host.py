"""Host-side contract of the C-ABI library, runnable without a GPU: every declared symbol is exported, record
layouts match the reference's, argument refusals and the NaN-weight refusal come back before any device work
(the reference's host-only tier, tests/gpu_fp8_api_test.c:4-31), and with no device a compute call fails loudly
with CHIP_FAIL instead of falling back to the CPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from cudapp_b200 import api
from oracle import oracle as orc
from tests.conftest import HAVE_GPU

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in ("b200moe_fp8.h", "b200moe_fp8gemm.h", "b200moe_plan.h", "b200moe_ext.h"):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(omega_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_every_declared_symbol_is_exported():
    syms = declared_symbols()
    assert len(syms) >= 45
    missing = [s for s in syms if not hasattr(api.lib, s)]
    assert not missing, missing


def test_rc_names_and_helpers():
    assert [api.rc_name(r) for r in (0, -1, -2, -3, -4, -5)] == ["OK", "BAD_ARGS", "TOO_LARGE", "CODEGEN_FAIL", "CHIP_FAIL", "NAN_WEIGHT"]
    L = orc.lib()
    for c in range(256):
        a, b = api.lib.omega_fp8_e4m3_ref(c), L.orc_e4m3_decode(c)
        assert (np.isnan(a) and np.isnan(b)) or a == b
        assert api.lib.omega_fp8_e4m3_is_nan(C.c_uint8(c)) == (1 if c & 0x7F == 0x7F else 0)
    rng = np.random.default_rng(2)
    for v in np.concatenate([rng.normal(0, 100, 3000), rng.normal(0, .01, 3000), [0.0, -0.0, 448, 1e9, -1e9, 2.0 ** -10, 3 * 2.0 ** -10]]).astype(np.float32):
        assert api.lib.omega_gpu_fp8_e4m3_rne(C.c_float(float(v))) == L.orc_e4m3_encode(C.c_float(float(v)))
    w = np.zeros(100, np.uint8); w[17] = 0x7F; w[60] = 0xFF
    first = C.c_size_t(0)
    assert api.lib.omega_fp8_pack_scan_nan(w.ctypes.data_as(C.c_void_p), C.c_size_t(100), C.byref(first)) == 2 and first.value == 17


def test_exported_double_oracle():
    """the exported host helper omega_fp8_gemv_oracle (src/omega_gpu_fp8_api.h:224-238; never called by a compute entry) against the checker"""
    rng = np.random.default_rng(5)
    n, k = 256, 512
    w8, sc = orc.quantize_bf16(orc.bf16_bits(rng.normal(0, 0.02, (n, k)).astype(np.float32)))
    x = rng.normal(0, 1, k).astype(np.float32)
    y = np.empty(n, np.float64); m = np.empty(n, np.float64)
    api.lib.omega_fp8_gemv_oracle.restype = None
    api.lib.omega_fp8_gemv_oracle(w8.ctypes.data_as(C.c_void_p), sc.ctypes.data_as(C.c_void_p), C.c_uint32(n), C.c_uint32(k), x.ctypes.data_as(C.c_void_p),
                                  y.ctypes.data_as(C.c_void_p), m.ctypes.data_as(C.c_void_p))
    ry, rm = orc.gemv(w8, sc, x, mag=True)
    assert np.max(np.abs(y - ry) / rm) < 1e-14 and np.max(np.abs(m - rm) / rm) < 1e-14     # same products, summation order may differ
    api.lib.omega_fp8_gemv_oracle(w8.ctypes.data_as(C.c_void_p), sc.ctypes.data_as(C.c_void_p), C.c_uint32(n), C.c_uint32(k), x.ctypes.data_as(C.c_void_p),
                                  y.ctypes.data_as(C.c_void_p), None)                         # the magnitude output is optional
    assert np.max(np.abs(y - ry) / rm) < 1e-14


def test_upload_refusals_before_device():
    w = np.zeros((1, 128, 128), np.uint8); s = np.full((1, 1, 1), 0x3F80, np.uint16)
    assert api.fp8_tensor_upload(1, 128, 100, w, s)[0] == api.BAD_ARGS          # k not a multiple of 128
    assert api.fp8_tensor_upload(0, 128, 128, w, s)[0] == api.BAD_ARGS
    assert api.fp8_tensor_upload(1, 128, 32768 + 128, w, s)[0] == api.TOO_LARGE
    h = C.c_void_p(123)
    assert api.lib.omega_gpu_fp8_tensor_upload(C.c_uint32(1), C.c_uint32(128), C.c_uint32(128), None, None, C.byref(h)) == api.BAD_ARGS and not h.value
    w[0, 5, 7] = 0xFF
    rc, t = api.fp8_tensor_upload(1, 128, 128, w, s)
    assert rc == api.NAN_WEIGHT and t is None and "NaN code at byte %d" % (5 * 128 + 7) in api.last_error()
    w[0, 5, 7] = 0
    s[0, 0, 0] = 0x7F80                                                              # inf scale
    assert api.fp8_tensor_upload(1, 128, 128, w, s)[0] == api.BAD_ARGS
    assert api.lib.omega_gpu_fp8_gemv_f32(None, C.c_uint32(0), None, None, None) == api.BAD_ARGS
    assert api.lib.omega_gpu_fp8gemm_f32(None, C.c_uint32(1), None, None, None, C.c_uint32(1), None, None) == api.BAD_ARGS
    assert api.lib.omega_gpu_fp8_prepare(C.c_uint32(100)) == api.BAD_ARGS and api.lib.omega_gpu_fp8_prepare(C.c_uint32(65536)) == api.TOO_LARGE


def test_plan_units_argument_refusals_and_host_serialisers():
    """ABI1 status 32 for wrong lengths / aliasing without touching outputs (tests/moe/caller.c:108-111), and the
    pure host serialisers against the checker."""
    cfg = np.array([1, 1, 8, 256, 256, 1152, 257, 1160], np.uint64); ids = np.zeros(1024, np.uint64)
    work, seg, maps, meta = orc.plan_buffers()
    r = C.c_uint64(77)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    assert api.lib.omega_moe_plan(C.byref(r), p(cfg), C.c_uint64(8), p(ids), C.c_uint64(1024), p(work), C.c_uint64(10368), p(work), C.c_uint64(1028),
                                  p(maps), C.c_uint64(2320), p(meta), C.c_uint64(8)) == 32
    assert api.lib.omega_moe_plan(C.byref(r), p(cfg), C.c_uint64(8), p(ids), C.c_uint64(1023), p(work), C.c_uint64(10368), p(seg), C.c_uint64(1028),
                                  p(maps), C.c_uint64(2320), p(meta), C.c_uint64(8)) == 32
    assert r.value == 77 and work[0] == np.uint64(0x5A5A5A5A5A5A5A5A)
    # serialisers on a checker-made plan
    L = orc.lib()
    cfg = np.array([1, 31, 8, 256, 256, 1152, 257, 1160], np.uint64); ids = (np.arange(1024) * 29 % 256).astype(np.uint64)
    assert orc.moe_plan(cfg, ids, work, seg, maps, meta) == 0
    dirs = np.zeros(514, np.uint64)
    for j in range(257):
        dirs[2 * j] = j * 256 + 4096; dirs[2 * j + 1] = dirs[2 * j] + 128
    for mut in ("ok", "map", "dir", "seg"):
        mp, sg, dr = maps.copy(), seg.copy(), dirs.copy()
        if mut == "map": mp[0] = 2 ** 64 - 1
        if mut == "dir": dr[0] = 0
        if mut == "seg": sg[2] = 2 ** 64 - 1
        a = np.full(9280, 90, np.uint8); b = a.copy()
        want = L.orc_moe_maps32(p(meta), p(mp), p(a))
        assert api.lib.omega_moe_maps32(C.byref(r), p(meta), C.c_uint64(8), p(mp), C.c_uint64(2320), p(b), C.c_uint64(9280)) == 0
        assert r.value == want and np.array_equal(a, b)
        a = np.full(8224, 90, np.uint8); b = a.copy()
        want = L.orc_moe_segs32(p(sg), p(meta), p(dr), p(a))
        assert api.lib.omega_moe_segs32(C.byref(r), p(sg), C.c_uint64(1028), p(meta), C.c_uint64(8), p(dr), C.c_uint64(514), p(b), C.c_uint64(8224)) == 0
        assert r.value == want and np.array_equal(a, b)
    wire = np.zeros(4096, np.uint8); wire.view(np.uint32)[:] = np.arange(1024) % 257
    for n in (0, 5, 1024, 1025):
        a = np.full(1024, 7, np.uint64); b = a.copy()
        want = L.orc_moe_ids32(p(wire), C.c_uint64(n), p(a))
        assert api.lib.omega_moe_ids32(C.byref(r), p(wire), C.c_uint64(4096), C.c_uint64(n), p(b), C.c_uint64(1024)) == 0 and r.value == want and np.array_equal(a, b)
    for n in (0, 1, 14, 15, 128, 129):
        c = np.array([1, n, 2048, 512, 9, 512, 128, 0], np.uint64)
        a = np.full(1024, 3, np.uint64); am = np.full(4, 3, np.uint64); b = a.copy(); bm = am.copy()
        want = L.orc_moe_windows(p(c), p(a), p(am))
        assert api.lib.omega_moe_windows(C.byref(r), p(c), C.c_uint64(8), p(b), C.c_uint64(1024), p(bm), C.c_uint64(4)) == 0
        assert r.value == want and np.array_equal(a, b) and np.array_equal(am, bm)
    q = [4096, 8192, 12288, 65536, 131072, 196608, 262144, 512, 14, 126, 134, 9, 1, 1, 1, 256]
    for f, v in [(None, None), (8, 15), (9, 125), (7, 513), (12, 0), (3, 4096), (0, 2 ** 64 - 8)]:
        req = np.array(q, np.uint64)
        if f is not None: req[f] = v
        a = np.full(64, 9, np.uint8); b = a.copy()
        want = L.orc_moe_group(p(req), p(a))
        assert api.lib.omega_moe_group(C.byref(r), p(req), C.c_uint64(16), p(b), C.c_uint64(64)) == 0 and r.value == want and np.array_equal(a, b)


@pytest.mark.skipif(HAVE_GPU, reason="checks the no-device behaviour")
def test_no_device_fails_loudly():
    w = np.zeros((1, 128, 128), np.uint8); s = np.full((1, 1, 1), 0x3F80, np.uint16)
    rc, t = api.fp8_tensor_upload(1, 128, 128, w, s)
    assert rc == api.CHIP_FAIL and t is None and "CUDA" in api.last_error()
    rc, _, _ = api.fp8_quantize_bf16(np.zeros((128, 128), np.uint16))
    assert rc == api.CHIP_FAIL
    rc, _, _ = api.moe_topk_bf16(np.zeros((2, 128), np.uint16))
    assert rc == api.CHIP_FAIL
    cfg = np.array([1, 1, 8, 256, 256, 1152, 257, 1160], np.uint64)
    work, seg, maps, meta = orc.plan_buffers()
    st, _ = api.omega_moe_plan(cfg, np.zeros(1024, np.uint64), work, seg, maps, meta)
    assert st == 14 and work[0] == np.uint64(0x5A5A5A5A5A5A5A5A)


def test_expert_parallel_create_refusals_before_device():
    """shapes that cannot be sharded are refused on the host before any device work: tokens or experts not divisible by the rank count, a rank
    outside the world, no layers"""
    dummy = (C.c_void_p * 2)(C.c_void_p(1), C.c_void_p(1))      # never dereferenced: the refusals come first
    out = C.c_void_p(123)
    cr = api.lib.omega_gpu_moe_epstack_create
    for world, rank, layers, experts, tokens in ((4, 0, 2, 128, 254), (3, 0, 2, 128, 255), (4, 4, 2, 128, 256), (4, 0, 0, 128, 256), (0, 0, 2, 128, 256), (65, 0, 2, 130, 260)):
        out.value = 123
        assert cr(C.c_uint32(world), C.c_uint32(rank), C.c_uint32(layers), dummy, C.c_uint32(experts), C.c_uint32(tokens), C.c_float(1e-6), C.byref(out)) == api.BAD_ARGS
        assert not out.value
    assert cr(C.c_uint32(2), C.c_uint32(0), C.c_uint32(2), None, C.c_uint32(128), C.c_uint32(256), C.c_float(1e-6), C.byref(out)) == api.BAD_ARGS
    ep = C.c_void_p(123)
    ce = api.lib.omega_gpu_moe_ep_create
    for world, rank, experts, topk, hidden, tl in ((4, 0, 130, 8, 2048, 64), (4, 5, 128, 8, 2048, 64), (4, 0, 128, 0, 2048, 64), (4, 0, 128, 8, 2052, 64), (4, 0, 128, 8, 2048, 0)):
        ep.value = 123
        assert ce(C.c_uint32(world), C.c_uint32(rank), C.c_uint32(experts), C.c_uint32(topk), C.c_uint32(hidden), C.c_uint32(tl), C.byref(ep)) == api.BAD_ARGS
        assert not ep.value


REFERENCE = os.environ.get("B200MOE_REFERENCE", os.path.normpath(os.path.join(ROOT, "..", "reference")))


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "src")), reason="the reference tree (for its headers) is not on this machine")
def test_c_caller_compiled_against_the_reference_headers(tmp_path):
    """tests/abi_against_reference_headers.c includes the reference's own omega_gpu_fp8_api.h / omega_gpu_fp8gemm_api.h / cudapp_native.h and is
    linked with libb200moe.so: the boundary as a C caller of the reference sees it"""
    import subprocess
    exe = str(tmp_path / "abi_ref")
    libdir = os.path.join(ROOT, "cudapp_b200", "lib")
    cc = subprocess.run(["gcc", "-std=gnu11", "-Wall", "-Werror", "-I", os.path.join(REFERENCE, "src"), os.path.join(ROOT, "tests", "abi_against_reference_headers.c"),
                         "-L", libdir, "-lb200moe", "-Wl,-rpath," + libdir, "-o", exe], capture_output=True, text=True)
    assert cc.returncode == 0, cc.stderr
    run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and "PASS" in run.stdout, run.stdout + run.stderr
