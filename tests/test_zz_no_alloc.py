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
    # two different tables: the second has fewer segments, so stale records of the first must not leak into it
    for tokens, topk, seed in ((40, 6, 1), (9, 2, 2)):
        r = np.random.default_rng(seed)
        picks = np.stack([r.choice(E, topk, replace=False) for _ in range(tokens)])
        order = np.lexsort((np.repeat(np.arange(tokens), topk), picks.reshape(-1)))
        ids = picks.reshape(-1)[order].astype(np.uint32); rows = np.repeat(np.arange(tokens), topk)[order].astype(np.uint32)
        x = r.uniform(-2, 2, (tokens, k)).astype(np.float32)
        rc, want = api.fp8gemm(t, ids, rows, x)
        assert rc == 0, api.last_error()
        d_ids = torch.from_numpy(ids.view(np.int32)).to(dev); d_rows = torch.from_numpy(rows.view(np.int32)).to(dev)
        d_x = torch.from_numpy(x).to(dev); d_y = torch.full((len(ids), n), -999.0, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        rc = api.lib.omega_gpu_fp8gemm_noalloc(t, C.c_uint32(len(ids)), C.c_uint64(d_ids.data_ptr()), C.c_uint64(d_rows.data_ptr()), C.c_uint64(d_x.data_ptr()),
                                               C.c_int(0), C.c_uint32(tokens), C.c_uint64(d_y.data_ptr()), C.c_void_p(stream.cuda_stream))
        assert rc == 0, api.last_error()
        stream.synchronize()
        got = d_y.cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # refusals: unsorted ids are reported, an oversized request is refused with a message
    bad = ids.copy(); bad[0], bad[-1] = bad[-1], bad[0]
    d_bad = torch.from_numpy(bad.view(np.int32)).to(dev)
    rc = api.lib.omega_gpu_fp8gemm_noalloc(t, C.c_uint32(len(bad)), C.c_uint64(d_bad.data_ptr()), C.c_uint64(d_rows.data_ptr()), C.c_uint64(d_x.data_ptr()),
                                           C.c_int(0), C.c_uint32(tokens), C.c_uint64(d_y.data_ptr()), C.c_void_p(stream.cuda_stream))
    assert rc == api.BAD_ARGS and "non-decreasing" in api.last_error()
    rc = api.lib.omega_gpu_fp8gemm_noalloc(t, C.c_uint32(1048577), C.c_uint64(d_ids.data_ptr()), C.c_uint64(d_rows.data_ptr()), C.c_uint64(d_x.data_ptr()),
                                           C.c_int(0), C.c_uint32(tokens), C.c_uint64(d_y.data_ptr()), C.c_void_p(stream.cuda_stream))
    assert rc == api.TOO_LARGE and "maximum" in api.last_error()
    api.fp8_tensor_free(t)
