"""Failure detection of the expert-parallel stack on a GPU, with no GPU fault: the failure is made on the host (a rank is told to
expect one more input row than anybody will ever deliver), the kernel's bounded wait runs out after about a millisecond and the
kernel returns by itself with an error code; the kernels queued behind it do nothing; the status call reports the code and
latches the process, after which every compute call is refused (the reference's contract for a completion of unknown outcome,
src/omega_gpu_session.h:27-29, src/omega_gpu_wait.h:20-24). The latch is for the life of the process, so the scenario runs in
a child process and this file only reads its report."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

CHILD = r'''
import ctypes as C, json, sys
import numpy as np
sys.path.insert(0, %r)
import torch
from cudapp_b200 import api
from oracle import oracle as orc
from tests.test_gpu_layer import build_layer
rng = np.random.default_rng(5)
E, H, I, topk, Ln, T = 16, 512, 256, 4, 2, 32
ms = [build_layer(rng, E, H, I, T, api.ENGINE_MMA, topk) for _ in range(Ln)]
arr = (C.c_void_p * Ln)(*[m["layer"] for m in ms])
eps = C.c_void_p()
assert api.lib.omega_gpu_moe_epstack_create(C.c_uint32(1), C.c_uint32(0), C.c_uint32(Ln), arr, C.c_uint32(E), C.c_uint32(T), C.c_float(1e-6), C.byref(eps)) == 0, api.last_error()
dev = torch.device("cuda", 0)
lg = torch.from_numpy(orc.bf16_bits(rng.normal(0, 1, (Ln, T, E)).astype(np.float32)).view(np.int16)).to(dev)
x = torch.from_numpy(orc.bf16_bits(rng.normal(0, 1, (T, H)).astype(np.float32)).view(np.int16)).to(dev)
out = torch.zeros((T, H), dtype=torch.int16, device=dev)
s = torch.cuda.Stream(); torch.cuda.synchronize()
step = lambda: api.lib.omega_gpu_moe_epstack_step_async(eps, C.c_uint64(lg.data_ptr()), C.c_uint64(x.data_ptr()), C.c_uint64(out.data_ptr()), C.c_void_p(s.cuda_stream))
rep = {}
rep["good_step_rc"] = step(); rep["good_status"] = api.lib.omega_gpu_moe_epstack_status(eps, C.c_void_p(s.cuda_stream))
good = out.cpu().numpy().copy()
api.lib.omega_gpu_moe_test_set_wait_limit(C.c_uint32(4000))            # about a millisecond instead of about a second
assert api.lib.omega_gpu_moe_epstack_test_expect_extra(eps, C.c_uint32(1)) == 0, api.last_error()
out.zero_(); torch.cuda.synchronize()
import time
t0 = time.perf_counter()
rep["bad_step_rc"] = step()
rep["bad_status"] = api.lib.omega_gpu_moe_epstack_status(eps, C.c_void_p(s.cuda_stream))
rep["bad_step_seconds"] = time.perf_counter() - t0
rep["error_text"] = api.last_error()
rep["output_untouched"] = bool((out == 0).all().item())                # the kernels behind the failed one did nothing
rep["next_step_rc"] = step()                                           # latched: refused before any launch
logits_h = orc.bf16_bits(rng.normal(0, 1, (T, E)).astype(np.float32)); x_h = orc.bf16_bits(rng.normal(0, 1, (T, H)).astype(np.float32))
rep["next_layer_rc"] = api.moe_layer_bf16(ms[0]["layer"], logits_h, x_h, topk)[0]
rep["good_output_nonzero"] = bool(np.any(good != 0))
rep["context_alive"] = bool(torch.ones(4, device=dev).sum().item() == 4.0)      # the CUDA context itself is still usable
print("REPORT " + json.dumps(rep)); sys.stdout.flush()
'''


def test_bounded_wait_runs_out_and_latches():
    r = subprocess.run([sys.executable, "-c", CHILD % ROOT], capture_output=True, text=True, timeout=300, cwd=ROOT)
    lines = [l for l in r.stdout.splitlines() if l.startswith("REPORT ")]
    assert r.returncode == 0 and lines, (r.returncode, r.stdout[-2000:], r.stderr[-2000:])
    rep = json.loads(lines[-1][7:])
    assert rep["good_step_rc"] == 0 and rep["good_status"] == 0 and rep["good_output_nonzero"]
    assert rep["bad_step_rc"] == 0                       # launches are queued; the failure shows in the status
    assert rep["bad_status"] in (13, 14), rep            # the expert kernel's wait for its input rows gave up (producer or scale-loader role first)
    assert rep["bad_step_seconds"] < 20.0, rep
    assert "latched" in rep["error_text"]
    assert rep["output_untouched"]
    from cudapp_b200 import api
    assert rep["next_step_rc"] == api.CHIP_FAIL and rep["next_layer_rc"] == api.CHIP_FAIL
    assert rep["context_alive"]


def test_step_before_connect_is_refused():
    """rank 0 of a two-rank stack that never exchanged handles with its peer: refused on the host, nothing is launched"""
    import ctypes as C
    import torch
    from cudapp_b200 import api
    from oracle import oracle as orc
    from tests.test_gpu_layer import build_layer, free_layer
    rng = np.random.default_rng(6)
    E, H, I, topk, Ln, T = 16, 512, 256, 4, 2, 32
    ms = [build_layer(rng, E // 2, H, I, T, api.ENGINE_MMA, topk) for _ in range(Ln)]      # this rank's half of the experts
    arr = (C.c_void_p * Ln)(*[m["layer"] for m in ms])
    eps = C.c_void_p()
    assert api.lib.omega_gpu_moe_epstack_create(C.c_uint32(2), C.c_uint32(0), C.c_uint32(Ln), arr, C.c_uint32(E), C.c_uint32(T), C.c_float(1e-6), C.byref(eps)) == 0, api.last_error()
    dev = torch.device("cuda", 0)
    lg = torch.zeros((Ln, T, E), dtype=torch.int16, device=dev); x = torch.zeros((T // 2, H), dtype=torch.int16, device=dev); out = torch.zeros_like(x)
    rc = api.lib.omega_gpu_moe_epstack_step_async(eps, C.c_uint64(lg.data_ptr()), C.c_uint64(x.data_ptr()), C.c_uint64(out.data_ptr()), C.c_void_p(0))
    assert rc == api.BAD_ARGS and "not connected" in api.last_error()
    api.lib.omega_gpu_moe_epstack_free(eps)
    for m in ms:
        free_layer(m)
