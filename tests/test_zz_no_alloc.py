"""The allocation-free row-table GEMM entry point against the ordinary one.

omega_gpu_fp8gemm_noalloc exists for hosts that cannot call cudaMalloc while they run (an embedder that owns all
device memory through its own arena, or code in a section where an allocation's device-wide synchronisation is not
acceptable). It must give exactly the bits of omega_gpu_fp8gemm_f32 on the same row table, and it must do so on a
second call too, because both calls reuse one fixed device array that still holds the first call's segment table.
Collected last on purpose: if it fails, every other test has already run.
"""
import ctypes as C

import numpy as np
import pytest

from cudapp_b200 import api
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def test_noalloc_matches_staged_entry_twice():
    import torch
    rng = np.random.default_rng(77)
    E, n, k = 24, 256, 1024
    w8 = np.empty((E, n, k), np.uint8); sc = np.empty((E, n // 128, k // 128), np.uint16)
    for e in range(E):
        w8[e], sc[e] = orc.quantize_bf16(orc.bf16_bits(rng.normal(0, 0.02, (n, k)).astype(np.float32)))
    rc, t = api.fp8_tensor_upload(E, n, k, w8, sc)
    assert rc == 0, api.last_error()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream()
    # Four tables in a row on the one shared array. The second has fewer segments than the first, so stale records must not
    # leak into it; the third has more than 1024 rows (the table builder then runs several passes and carries its segment
    # count across them) with only a third of the experts present, and bf16 activations; the fourth is small again.
    for tokens, topk, seed, x_bf16, experts_used in ((40, 6, 1, 0, E), (9, 2, 2, 0, E), (600, 6, 3, 1, 8), (5, 3, 4, 1, E)):
        r = np.random.default_rng(seed)
        pool = np.sort(r.choice(E, experts_used, replace=False))
        picks = np.stack([r.choice(pool, topk, replace=False) for _ in range(tokens)])
        order = np.lexsort((np.repeat(np.arange(tokens), topk), picks.reshape(-1)))
        ids = picks.reshape(-1)[order].astype(np.uint32); rows = np.repeat(np.arange(tokens), topk)[order].astype(np.uint32)
        x = r.uniform(-2, 2, (tokens, k)).astype(np.float32)
        if x_bf16:
            xb = orc.bf16_bits(x)
            rc, want = api.fp8gemm(t, ids, rows, xb)
            d_x = torch.from_numpy(xb.view(np.int16)).to(dev)
        else:
            rc, want = api.fp8gemm(t, ids, rows, x)
            d_x = torch.from_numpy(x).to(dev)
        assert rc == 0, api.last_error()
        d_ids = torch.from_numpy(ids.view(np.int32)).to(dev); d_rows = torch.from_numpy(rows.view(np.int32)).to(dev)
        d_y = torch.full((len(ids), n), -999.0, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        rc = api.lib.omega_gpu_fp8gemm_noalloc(t, C.c_uint32(len(ids)), C.c_uint64(d_ids.data_ptr()), C.c_uint64(d_rows.data_ptr()), C.c_uint64(d_x.data_ptr()),
                                               C.c_int(x_bf16), C.c_uint32(tokens), C.c_uint64(d_y.data_ptr()), C.c_void_p(stream.cuda_stream))
        assert rc == 0, api.last_error()
        stream.synchronize()
        got = d_y.cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (tokens, topk)
    # a row index at or past x_rows would make the GEMM read x out of bounds: refused like the staged entry refuses it
    bad_rows = rows.copy(); bad_rows[len(bad_rows) // 2] = tokens
    d_bad_rows = torch.from_numpy(bad_rows.view(np.int32)).to(dev)
    d_y.fill_(-999.0); torch.cuda.synchronize()
    rc = api.lib.omega_gpu_fp8gemm_noalloc(t, C.c_uint32(len(ids)), C.c_uint64(d_ids.data_ptr()), C.c_uint64(d_bad_rows.data_ptr()), C.c_uint64(d_x.data_ptr()),
                                           C.c_int(x_bf16), C.c_uint32(tokens), C.c_uint64(d_y.data_ptr()), C.c_void_p(stream.cuda_stream))
    assert rc == api.BAD_ARGS and "x_rows" in api.last_error()
    stream.synchronize()
    assert bool((d_y == -999.0).all()), "a refused call must not queue the GEMM"
    # refusals: unsorted ids are reported, an oversized request is refused with a message
    bad = ids.copy(); bad[0], bad[-1] = bad[-1], bad[0]
    d_bad = torch.from_numpy(bad.view(np.int32)).to(dev)
    rc = api.lib.omega_gpu_fp8gemm_noalloc(t, C.c_uint32(len(bad)), C.c_uint64(d_bad.data_ptr()), C.c_uint64(d_rows.data_ptr()), C.c_uint64(d_x.data_ptr()),
                                           C.c_int(x_bf16), C.c_uint32(tokens), C.c_uint64(d_y.data_ptr()), C.c_void_p(stream.cuda_stream))
    assert rc == api.BAD_ARGS and "non-decreasing" in api.last_error()
    rc = api.lib.omega_gpu_fp8gemm_noalloc(t, C.c_uint32(1048577), C.c_uint64(d_ids.data_ptr()), C.c_uint64(d_rows.data_ptr()), C.c_uint64(d_x.data_ptr()),
                                           C.c_int(0), C.c_uint32(tokens), C.c_uint64(d_y.data_ptr()), C.c_void_p(stream.cuda_stream))
    assert rc == api.TOO_LARGE and "maximum" in api.last_error()
    # on a stream that is being captured the call is refused before anything is queued; the capture stays valid and the
    # library does not latch (the next ordinary call still works)
    cap = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=cap, capture_error_mode="thread_local"):
        rc = api.lib.omega_gpu_fp8gemm_noalloc(t, C.c_uint32(len(ids)), C.c_uint64(d_ids.data_ptr()), C.c_uint64(d_rows.data_ptr()), C.c_uint64(d_x.data_ptr()),
                                               C.c_int(x_bf16), C.c_uint32(tokens), C.c_uint64(d_y.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        d_y.add_(0.0)   # the capture must still accept work
    assert rc == api.BAD_ARGS and "captured" in api.last_error()
    rc = api.lib.omega_gpu_fp8gemm_noalloc(t, C.c_uint32(len(ids)), C.c_uint64(d_ids.data_ptr()), C.c_uint64(d_rows.data_ptr()), C.c_uint64(d_x.data_ptr()),
                                           C.c_int(x_bf16), C.c_uint32(tokens), C.c_uint64(d_y.data_ptr()), C.c_void_p(stream.cuda_stream))
    assert rc == 0, api.last_error()
    stream.synchronize()
    assert np.array_equal(d_y.cpu().numpy().view(np.uint32), want.view(np.uint32))
    api.fp8_tensor_free(t)
