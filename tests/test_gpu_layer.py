"""GPU parity of the whole MoE layer and of the layer stack against the CPU checker, through the C-ABI.

The checker strings the reference's operators together exactly as its host glue does
(tests/gpu_decode_graph_test.c:129-147): top-k, per pick gate|up GEMV -> SiLU gate -> down GEMV, slot-order weighted
sum. Bars (the benchmark's): routing ids bit-exact, outputs max-abs <= 1e-2 and rel-L2 <= 1e-3 on the f32 result.
"""
import ctypes as C

import numpy as np
import pytest

from cudapp_b200 import api
from oracle import oracle as orc
from tests.test_gpu_ops import make_weights, rel_l2

pytestmark = pytest.mark.gpu


def build_layer(rng, E, H, I, max_tokens, engine, topk=8, **kw):
    wgu, sgu = make_weights(rng, E, 2 * I, H)
    wdn, sdn = make_weights(rng, E, H, I)
    rc, tgu = api.fp8_tensor_upload(E, 2 * I, H, wgu, sgu); assert rc == 0, api.last_error()
    rc, tdn = api.fp8_tensor_upload(E, H, I, wdn, sdn); assert rc == 0, api.last_error()
    rc, layer = api.moe_layer_create(tgu, tdn, topk=topk, max_tokens=max_tokens, engine=engine, **kw)
    assert rc == 0, api.last_error()
    return dict(wgu=wgu, sgu=sgu, wdn=wdn, sdn=sdn, tgu=tgu, tdn=tdn, layer=layer)


def free_layer(m):
    api.lib.omega_gpu_moe_layer_free(m["layer"]); api.fp8_tensor_free(m["tgu"]); api.fp8_tensor_free(m["tdn"])


def check_layer(m, logits, xb, topk, tol_abs=1e-2, tol_rel=1e-3):
    rc, o16, o32, ids, w = api.moe_layer_bf16(m["layer"], logits, xb, topk)
    assert rc == 0, api.last_error()
    ref, rid, rw = orc.moe_layer(logits, xb, m["wgu"], m["sgu"], m["wdn"], m["sdn"], topk)
    assert np.array_equal(ids, rid)
    assert np.max(np.abs(w - rw)) <= 1e-5
    err, rl2 = float(np.max(np.abs(o32 - ref))), rel_l2(o32, ref)
    assert err <= tol_abs and rl2 <= tol_rel, (err, rl2)
    assert np.array_equal(o16, orc.bf16_bits(o32))
    return err, rl2


@pytest.mark.parametrize("engine", [api.ENGINE_FMA, api.ENGINE_MMA])
@pytest.mark.parametrize("tokens", [1, 7, 64])
def test_layer_small(engine, tokens):
    rng = np.random.default_rng(100 + tokens)
    E, H, I, topk = 16, 512, 256, 4
    m = build_layer(rng, E, H, I, 64, engine, topk)
    logits = orc.bf16_bits(rng.normal(0, 1, (tokens, E)).astype(np.float32))
    xb = orc.bf16_bits(rng.normal(0, 1, (tokens, H)).astype(np.float32))
    check_layer(m, logits, xb, topk)
    assert api.lib.omega_gpu_moe_layer_launches(m["layer"]) >= 4
    free_layer(m)


@pytest.mark.parametrize("E,H,I,topk,T", [(8, 4096, 1536, 4, 40), (16, 1024, 640, 6, 100), (12, 256, 128, 2, 33)])
def test_layer_other_shapes(E, H, I, topk, T):
    """the one-launch expert kernel at the edges of its shape range: the longest rows (32 K blocks), an odd number of K blocks in the down
    projection (5), a single K block; with more and with fewer units than CTAs"""
    rng = np.random.default_rng(E + H + I)
    m = build_layer(rng, E, H, I, T, api.ENGINE_MMA, topk)
    logits = orc.bf16_bits(rng.normal(0, 1, (T, E)).astype(np.float32))
    xb = orc.bf16_bits(rng.normal(0, 1, (T, H)).astype(np.float32))
    check_layer(m, logits, xb, topk)
    rc, _, o32b, _, _ = api.moe_layer_bf16(m["layer"], logits, xb, topk)          # a second call: same bits (work-list words cleared between calls)
    rc2, _, o32c, _, _ = api.moe_layer_bf16(m["layer"], logits, xb, topk)
    assert rc == 0 and rc2 == 0 and np.array_equal(o32b.view(np.uint32), o32c.view(np.uint32))
    free_layer(m)


@pytest.mark.parametrize("engine", [api.ENGINE_FMA, api.ENGINE_MMA])
def test_layer_decode_shape(engine):
    """the decode configuration's architecture (hidden 2048, expert intermediate 768, top-8) on 32 experts, 64 tokens"""
    rng = np.random.default_rng(7)
    E, H, I = 32, 2048, 768
    m = build_layer(rng, E, H, I, 64, engine)
    logits = orc.bf16_bits(rng.normal(0, 1, (64, E)).astype(np.float32))
    xb = orc.bf16_bits(rng.normal(0, 1, (64, H)).astype(np.float32))
    check_layer(m, logits, xb, 8)
    free_layer(m)


@pytest.mark.parametrize("engine", [api.ENGINE_FMA, api.ENGINE_MMA])
def test_stack_small(engine):
    rng = np.random.default_rng(9)
    E, H, I, topk, T, Ln = 16, 512, 256, 4, 24, 3
    ms = [build_layer(rng, E, H, I, 32, engine, topk) for _ in range(Ln)]
    rc, stack = api.moe_stack_create([m["layer"] for m in ms], 1e-6); assert rc == 0, api.last_error()
    logits = orc.bf16_bits(rng.normal(0, 1, (Ln, T, E)).astype(np.float32))
    xb = orc.bf16_bits(rng.normal(0, 1, (T, H)).astype(np.float32))
    rc, o16, o32 = api.moe_stack_bf16(stack, logits, xb); assert rc == 0, api.last_error()
    h = orc.bf16_to_f32(xb)
    for l in range(Ln):
        xn = orc.bf16_bits(orc.rmsnorm(h, 1e-6))
        mo, _, _ = orc.moe_layer(logits[l], xn, ms[l]["wgu"], ms[l]["sgu"], ms[l]["wdn"], ms[l]["sdn"], topk)
        h = h + mo
    assert np.max(np.abs(o32 - h)) <= 1e-2 and rel_l2(o32, h) <= 1e-3
    assert np.array_equal(o16, orc.bf16_bits(o32))
    # each layer's own RMSNorm weight (the reference's RES COMBINE|NORM, src/omega_blackwell_codegen_dec.c:261-286): new weights
    # take effect at the next step of the same captured graph
    nws = [rng.uniform(0.5, 1.5, H).astype(np.float32) for _ in range(Ln)]
    for l in range(Ln):
        assert api.lib.omega_gpu_moe_stack_set_norm(stack, C.c_uint32(l), nws[l].ctypes.data_as(C.c_void_p)) == 0, api.last_error()
    assert api.lib.omega_gpu_moe_stack_set_norm(stack, C.c_uint32(Ln), nws[0].ctypes.data_as(C.c_void_p)) == api.BAD_ARGS
    rc, w16, w32 = api.moe_stack_bf16(stack, logits, xb); assert rc == 0, api.last_error()
    h = orc.bf16_to_f32(xb)
    for l in range(Ln):
        xn = orc.bf16_bits(orc.rmsnorm(h, 1e-6, nws[l]))
        mo, _, _ = orc.moe_layer(logits[l], xn, ms[l]["wgu"], ms[l]["sgu"], ms[l]["wdn"], ms[l]["sdn"], topk)
        h = h + mo
    assert np.max(np.abs(w32 - h)) <= 1e-2 and rel_l2(w32, h) <= 1e-3 and not np.array_equal(w32, o32)
    ones = np.ones(H, np.float32)
    for l in range(Ln):
        assert api.lib.omega_gpu_moe_stack_set_norm(stack, C.c_uint32(l), ones.ctypes.data_as(C.c_void_p)) == 0
    rc, o16b, o32b = api.moe_stack_bf16(stack, logits, xb)          # graph replay: identical bits
    assert rc == 0 and np.array_equal(o32, o32b)
    assert api.lib.omega_gpu_moe_stack_launches(stack) >= Ln * 3
    api.lib.omega_gpu_moe_stack_free(stack)
    for m in ms:
        free_layer(m)


def test_epstack_world1_equals_stack():
    """the fused expert-parallel stack with one rank (its own peer) against the ordinary stack: identical bits"""
    import ctypes as C
    import torch
    rng = np.random.default_rng(21)
    E, H, I, topk, Ln = 16, 512, 256, 4, 3
    ms = [build_layer(rng, E, H, I, 32, api.ENGINE_MMA, topk) for _ in range(Ln)]
    rc, stack = api.moe_stack_create([m["layer"] for m in ms], 1e-6); assert rc == 0, api.last_error()
    arr = (C.c_void_p * Ln)(*[m["layer"] for m in ms])
    eps = C.c_void_p()
    # the layers' workspace holds 32 tokens; the expert-parallel stack is created for those 32 and run with all of them
    T2 = 32
    logits2 = orc.bf16_bits(rng.normal(0, 1, (Ln, T2, E)).astype(np.float32)); x2 = orc.bf16_bits(rng.normal(0, 1, (T2, H)).astype(np.float32))
    nws = [rng.uniform(0.5, 1.5, H).astype(np.float32) for _ in range(Ln)]       # each layer's own RMSNorm weight, the same on both stacks
    for l in range(Ln):
        assert api.lib.omega_gpu_moe_stack_set_norm(stack, C.c_uint32(l), nws[l].ctypes.data_as(C.c_void_p)) == 0, api.last_error()
    rc, want16, want32 = api.moe_stack_bf16(stack, logits2, x2); assert rc == 0, api.last_error()
    assert api.lib.omega_gpu_moe_epstack_create(C.c_uint32(1), C.c_uint32(0), C.c_uint32(Ln), arr, C.c_uint32(E), C.c_uint32(T2), C.c_float(1e-6), C.byref(eps)) == 0, api.last_error()
    for l in range(Ln):
        assert api.lib.omega_gpu_moe_epstack_set_norm(eps, C.c_uint32(l), nws[l].ctypes.data_as(C.c_void_p)) == 0, api.last_error()
    dev = torch.device("cuda", 0)
    d_lg = torch.from_numpy(logits2.view(np.int16)).to(dev); d_x = torch.from_numpy(x2.view(np.int16)).to(dev); d_o = torch.empty((T2, H), dtype=torch.int16, device=dev)
    s = torch.cuda.Stream()
    torch.cuda.synchronize()
    for _ in range(2):   # twice: the counters must come back to their starting state
        assert api.lib.omega_gpu_moe_epstack_step_async(eps, C.c_uint64(d_lg.data_ptr()), C.c_uint64(d_x.data_ptr()), C.c_uint64(d_o.data_ptr()), C.c_void_p(s.cuda_stream)) == 0, api.last_error()
        assert api.lib.omega_gpu_moe_epstack_status(eps, C.c_void_p(s.cuda_stream)) == 0
        assert np.array_equal(d_o.cpu().numpy().view(np.uint16), want16)
    api.lib.omega_gpu_moe_epstack_free(eps)
    api.lib.omega_gpu_moe_stack_free(stack)
    for m in ms:
        free_layer(m)


@pytest.mark.parametrize("pieces", [(1, 1), (2, 3)])
def test_layer_prefill_shape_skewed(pieces):
    """prefill-shaped work on the tensor-core engine: many tokens, router logits skewed by a per-expert bias N(0, 0.5) so segment
    sizes range from a few rows to several row tiles. With one piece the activations are plain FP8: the checker then applies the
    same activation quantiser (as the reference tests its own FP8 x FP8 path) and the bars are the usual ones; the distance to the
    unquantised checker is reported as quantisation error, not asserted. With (2, 3) pieces the unquantised checker is the bar."""
    xp, ap = pieces
    rng = np.random.default_rng(31)
    E, H, I, topk, T = 32, 512, 256, 8, 768
    m = build_layer(rng, E, H, I, T, api.ENGINE_MMA, topk, x_pieces=xp, act_pieces=ap)
    bias = rng.normal(0, 0.5, E).astype(np.float32)
    logits = orc.bf16_bits((rng.normal(0, 1, (T, E)) + bias).astype(np.float32))
    xb = orc.bf16_bits(rng.normal(0, 1, (T, H)).astype(np.float32))
    rc, o16, o32, ids, w = api.moe_layer_bf16(m["layer"], logits, xb, topk)
    assert rc == 0, api.last_error()
    counts = np.bincount(ids.reshape(-1), minlength=E)
    assert counts.max() > 64 and counts.max() > 2 * counts.min()           # several tiles for the busiest expert, real skew
    if (xp, ap) == (1, 1):
        ref, rid, rw = orc.moe_layer(logits, xb, m["wgu"], m["sgu"], m["wdn"], m["sdn"], topk, x_pieces=1, act_pieces=1)
    else:
        ref, rid, rw = orc.moe_layer(logits, xb, m["wgu"], m["sgu"], m["wdn"], m["sdn"], topk)
    assert np.array_equal(ids, rid)
    assert np.max(np.abs(o32 - ref)) <= 1e-2 and rel_l2(o32, ref) <= 1e-3, (float(np.max(np.abs(o32 - ref))), rel_l2(o32, ref))
    free_layer(m)


def test_layer_prefill_wide_tiles_equal_narrow():
    """the 128-row-tile kernel against the 32-row-tile kernel on the same layer and inputs (plain FP8 activations): the same
    promotion order per K block, so the results agree to rounding noise; segments of every size from a few rows to several tiles,
    row counts that are not multiples of 32, experts with no rows at all"""
    rng = np.random.default_rng(57)
    E, H, I, topk, T = 32, 512, 256, 8, 700
    wgu, sgu = make_weights(rng, E, 2 * I, H)
    wdn, sdn = make_weights(rng, E, H, I)
    rc, tgu = api.fp8_tensor_upload(E, 2 * I, H, wgu, sgu); assert rc == 0, api.last_error()
    rc, tdn = api.fp8_tensor_upload(E, H, I, wdn, sdn); assert rc == 0, api.last_error()
    bias = rng.normal(0, 1.0, E).astype(np.float32); bias[:3] = -30.0        # three experts never picked
    logits = orc.bf16_bits((rng.normal(0, 1, (T, E)) + bias).astype(np.float32))
    xb = orc.bf16_bits(rng.normal(0, 1, (T, H)).astype(np.float32))
    outs = {}
    for rows in (32, 128):
        rc, layer = api.moe_layer_create(tgu, tdn, topk=topk, max_tokens=T, engine=api.ENGINE_MMA, x_pieces=1, act_pieces=1, tile_rows=rows)
        assert rc == 0, api.last_error()
        rc, o16, o32, ids, w = api.moe_layer_bf16(layer, logits, xb, topk)
        assert rc == 0, api.last_error()
        outs[rows] = (o32, ids)
        api.lib.omega_gpu_moe_layer_free(layer)
    counts = np.bincount(outs[32][1].reshape(-1), minlength=E)
    assert counts.min() == 0 and counts.max() > 128 and np.any(counts % 32 != 0)
    assert np.array_equal(outs[32][1], outs[128][1])
    assert rel_l2(outs[128][0], outs[32][0]) <= 1e-5, rel_l2(outs[128][0], outs[32][0])
    ref, rid, rw = orc.moe_layer(logits, xb, wgu, sgu, wdn, sdn, topk, x_pieces=1, act_pieces=1)
    assert np.max(np.abs(outs[128][0] - ref)) <= 1e-2 and rel_l2(outs[128][0], ref) <= 1e-3
    # a request the wide kernel cannot serve is refused, not silently served by another path
    rc, layer = api.moe_layer_create(tgu, tdn, topk=topk, max_tokens=T, engine=api.ENGINE_MMA, x_pieces=2, act_pieces=3, tile_rows=128)
    assert rc == api.BAD_ARGS and layer is None
    api.fp8_tensor_free(tgu); api.fp8_tensor_free(tdn)


def test_fp8_tensor_peak_probe():
    """the tcgen05 probe that gives the prefill roofline its denominator returns a plausible figure for a B200"""
    import ctypes as C
    tf, ms = C.c_float(0), C.c_float(0)
    rc = api.lib.omega_gpu_fp8_tensor_peak(C.c_uint32(4000), C.c_uint32(3), C.byref(tf), C.byref(ms))
    assert rc == 0, api.last_error()
    assert 500.0 < tf.value < 6000.0, (tf.value, ms.value)


def test_router_then_layer_routed():
    """residual rows -> router front half (RMSNorm, gate GEMV, top-k; bf16 normalised rows out) -> the layer with that routing, all on
    the device with no host round trip; the checker strings its router and its layer together the same way"""
    import ctypes as C
    import torch
    rng = np.random.default_rng(91)
    E, H, I, topk, T = 32, 512, 256, 4, 48
    m = build_layer(rng, E, H, I, T, api.ENGINE_MMA, topk)
    gate = orc.bf16_bits(rng.uniform(-0.05, 0.05, (E, H)).astype(np.float32))
    nw = rng.uniform(0.8, 1.2, H).astype(np.float32)
    x = rng.uniform(-2.0, 2.0, (T, H)).astype(np.float32)
    rc, r = api.moe_router_create(gate, nw); assert rc == 0, api.last_error()
    dev = torch.device("cuda", 0)
    xd = torch.from_numpy(x).to(dev)
    xn16 = torch.empty((T, H), dtype=torch.int16, device=dev); ids = torch.empty((T, topk), dtype=torch.int32, device=dev)
    wts = torch.empty((T, topk), dtype=torch.float32, device=dev); out32 = torch.empty((T, H), dtype=torch.float32, device=dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    u64 = lambda t: C.c_uint64(t.data_ptr())
    rc = api.lib.omega_gpu_moe_router_rows_async(r, C.c_uint32(T), u64(xd), C.c_uint32(0), C.c_float(1e-6), C.c_int(1), C.c_float(1.0), C.c_uint32(topk),
                                                 C.c_uint64(0), u64(xn16), C.c_uint64(0), u64(ids), u64(wts), stream)
    assert rc == 0, api.last_error()
    rc = api.lib.omega_gpu_moe_layer_routed_async(m["layer"], C.c_uint32(T), u64(ids), u64(wts), u64(xn16), u64(out32), C.c_uint64(0), stream)
    assert rc == 0, api.last_error()
    assert api.lib.omega_gpu_moe_layer_status(m["layer"], stream) == 0, api.last_error()   # plan accepted, no wait ran out
    ids_h = ids.cpu().numpy().view(np.uint32); wts_h = wts.cpu().numpy(); xn_h = xn16.cpu().numpy().view(np.uint16); o32 = out32.cpu().numpy()
    oxn, olg, oids, ow, margin = orc.router(x, nw, gate, 1e-6, topk, True)
    sure = margin >= 1e-4
    assert np.array_equal(ids_h[sure], oids[sure]) and np.max(np.abs(wts_h[sure] - ow[sure])) <= 1e-5
    # bf16 rows: the double oracle rounded the same way, at most one bf16 step apart where the f32 value sits on a rounding boundary
    want = orc.bf16_bits(oxn.astype(np.float32)).astype(np.int32)
    assert np.max(np.abs(xn_h.astype(np.int32) - want)) <= 1 and np.mean(xn_h.astype(np.int32) != want) < 1e-2
    ref, _, _ = orc.moe_layer(None, xn_h, m["wgu"], m["sgu"], m["wdn"], m["sdn"], topk, routing=(ids_h, wts_h))
    assert np.max(np.abs(o32 - ref)) <= 1e-2 and rel_l2(o32, ref) <= 1e-3, (float(np.max(np.abs(o32 - ref))), rel_l2(o32, ref))
    # an id outside the layer's experts: the plan refuses (no rows, so the kernels that follow do nothing) and the status entry says so;
    # the next good call clears it
    bad = ids.clone(); bad[0, 0] = 100000
    rc = api.lib.omega_gpu_moe_layer_routed_async(m["layer"], C.c_uint32(T), u64(bad), u64(wts), u64(xn16), u64(out32), C.c_uint64(0), stream)
    assert rc == 0 and api.lib.omega_gpu_moe_layer_status(m["layer"], stream) == 102
    rc = api.lib.omega_gpu_moe_layer_routed_async(m["layer"], C.c_uint32(T), u64(ids), u64(wts), u64(xn16), u64(out32), C.c_uint64(0), stream)
    assert rc == 0 and api.lib.omega_gpu_moe_layer_status(m["layer"], stream) == 0
    assert np.array_equal(out32.cpu().numpy(), o32)
    api.lib.omega_gpu_moe_router_free(r)
    free_layer(m)


def test_stack_with_router_inside():
    """The stack computes its own routing: per layer residual (+ combine of the layer before) -> router (RMSNorm with the layer's norm weight,
    bf16 gate GEMV, top-k) -> plan -> experts, the reference's order (src/omega_gpu_decode_graph.c:341-351); no logits input. The checker follows
    layer by layer with its double-precision router; where a token's margin between the last selected and the first unselected logit is
    below 1e-4 the selection may legitimately differ (the reference router test's own rule, tests/gpu_router_test.c:95-111), so such a token is
    left out of the comparison from that layer on."""
    rng = np.random.default_rng(77)
    E, H, I, topk, T, Ln = 16, 512, 256, 4, 24, 3
    ms = [build_layer(rng, E, H, I, 32, api.ENGINE_MMA, topk) for _ in range(Ln)]
    rc, stack = api.moe_stack_create([m["layer"] for m in ms], 1e-6); assert rc == 0, api.last_error()
    gates = [orc.bf16_bits(rng.uniform(-0.05, 0.05, (E, H)).astype(np.float32)) for _ in range(Ln)]
    nws = [rng.uniform(0.8, 1.2, H).astype(np.float32) for _ in range(Ln)]
    routers = []
    for l in range(Ln):
        rc, r = api.moe_router_create(gates[l], nws[l]); assert rc == 0, api.last_error()
        routers.append(r)
    xb = orc.bf16_bits(rng.normal(0, 1, (T, H)).astype(np.float32))
    o16 = np.empty((T, H), np.uint16); o32 = np.empty((T, H), np.float32)
    run = lambda: api.lib.omega_gpu_moe_stack_bf16(stack, C.c_uint32(T), None, xb.ctypes.data_as(C.c_void_p), o16.ctypes.data_as(C.c_void_p), o32.ctypes.data_as(C.c_void_p))
    assert run() == api.BAD_ARGS                                           # no routers yet: the stack wants logits
    for l in range(Ln - 1):
        assert api.lib.omega_gpu_moe_stack_set_router(stack, C.c_uint32(l), routers[l]) == 0, api.last_error()
    assert run() == api.BAD_ARGS                                           # one layer still without a router
    assert api.lib.omega_gpu_moe_stack_set_router(stack, C.c_uint32(Ln - 1), routers[Ln - 1]) == 0, api.last_error()
    assert api.lib.omega_gpu_moe_stack_set_router(stack, C.c_uint32(Ln), routers[0]) == api.BAD_ARGS
    assert run() == 0, api.last_error()
    h = orc.bf16_to_f32(xb)
    keep = np.ones(T, bool)
    for l in range(Ln):
        xn64, lg, ids, w, margin = orc.router(h, nws[l], gates[l], 1e-6, topk, True)
        keep &= margin >= 1e-4
        xn = orc.bf16_bits(orc.rmsnorm(h, 1e-6, nws[l]))
        mo, _, _ = orc.moe_layer(None, xn, ms[l]["wgu"], ms[l]["sgu"], ms[l]["wdn"], ms[l]["sdn"], topk, routing=(ids, w.astype(np.float32)))
        h = h + mo
    assert keep.sum() >= T - 3
    assert np.max(np.abs(o32[keep] - h[keep])) <= 1e-2 and rel_l2(o32[keep], h[keep]) <= 1e-3, (float(np.max(np.abs(o32[keep] - h[keep]))), rel_l2(o32[keep], h[keep]))
    assert np.array_equal(o16, orc.bf16_bits(o32))
    first = o32.copy()
    assert run() == 0 and np.array_equal(first.view(np.uint32), o32.view(np.uint32))       # graph replay: identical bits
    assert api.lib.omega_gpu_moe_stack_launches(stack) == 5 * Ln + 1
    # taking a router away puts the stack back on given logits
    assert api.lib.omega_gpu_moe_stack_set_router(stack, C.c_uint32(0), None) == 0
    assert run() == api.BAD_ARGS
    api.lib.omega_gpu_moe_stack_free(stack)
    for r in routers:
        api.lib.omega_gpu_moe_router_free(r)
    for m in ms:
        free_layer(m)


@pytest.mark.parametrize("engine", [api.ENGINE_FMA, api.ENGINE_MMA])
def test_layer_with_shared_expert(engine):
    """The reference's ninth group (src/omega_gpu_q36_graph.h:7-21, :53-55): tensors of experts + 1, the last one the shared expert that every
    token goes through in one more slot after its routed picks; the plan puts those rows in the last segment and the combine runs over
    topk + 1 slots in slot order. From logits the shared slot has weight 1."""
    rng = np.random.default_rng(91)
    Er, H, I, topk, T = 16, 512, 256, 4, 24
    wgu, sgu = make_weights(rng, Er + 1, 2 * I, H); wdn, sdn = make_weights(rng, Er + 1, H, I)
    rc, tgu = api.fp8_tensor_upload(Er + 1, 2 * I, H, wgu, sgu); assert rc == 0, api.last_error()
    rc, tdn = api.fp8_tensor_upload(Er + 1, H, I, wdn, sdn); assert rc == 0, api.last_error()
    rc, layer = api.moe_layer_create(tgu, tdn, topk=topk, max_tokens=32, engine=engine, shared_expert=True); assert rc == 0, api.last_error()
    logits = orc.bf16_bits(rng.normal(0, 1, (T, Er)).astype(np.float32)); xb = orc.bf16_bits(rng.normal(0, 1, (T, H)).astype(np.float32))
    rc, o16, o32, ids, w = api.moe_layer_bf16(layer, logits, xb, topk + 1); assert rc == 0, api.last_error()
    rid, rw = orc.topk(orc.bf16_to_f32(logits), topk, True)
    assert np.array_equal(ids[:, :topk], rid) and np.all(ids[:, topk] == Er) and np.all(w[:, topk] == 1.0) and np.max(np.abs(w[:, :topk] - rw)) <= 1e-5
    ids5 = np.concatenate([rid, np.full((T, 1), Er, np.uint32)], 1); w5 = np.concatenate([rw.astype(np.float32), np.ones((T, 1), np.float32)], 1)
    ref, _, _ = orc.moe_layer(None, xb, wgu, sgu, wdn, sdn, topk + 1, routing=(ids5, w5))
    assert np.max(np.abs(o32 - ref)) <= 1e-2 and rel_l2(o32, ref) <= 1e-3, (float(np.max(np.abs(o32 - ref))), rel_l2(o32, ref))
    # without the shared expert's contribution the result is far off: the slot is really computed
    ref_routed, _, _ = orc.moe_layer(None, xb, wgu, sgu, wdn, sdn, topk, routing=(rid, rw.astype(np.float32)))
    assert rel_l2(o32, ref_routed) > 0.1
    # a stack of two such layers with the router inside; the routers carry the shared expert's gate: slot weight = sigmoid(gate . xn)
    if engine == api.ENGINE_MMA:
        rc, layer2 = api.moe_layer_create(tgu, tdn, topk=topk, max_tokens=32, engine=engine, shared_expert=True); assert rc == 0, api.last_error()
        rc, stack = api.moe_stack_create([layer, layer2], 1e-6); assert rc == 0, api.last_error()
        gates = [orc.bf16_bits(rng.uniform(-0.05, 0.05, (Er, H)).astype(np.float32)) for _ in range(2)]
        sgate = [orc.bf16_bits(rng.uniform(-0.05, 0.05, H).astype(np.float32)) for _ in range(2)]
        nws = [rng.uniform(0.8, 1.2, H).astype(np.float32) for _ in range(2)]
        routers = []
        for l in range(2):
            rc, r = api.moe_router_create(gates[l], nws[l]); assert rc == 0, api.last_error()
            assert api.lib.omega_gpu_moe_router_set_shared_gate(r, sgate[l].ctypes.data_as(C.c_void_p)) == 0, api.last_error()
            assert api.lib.omega_gpu_moe_stack_set_router(stack, C.c_uint32(l), r) == 0, api.last_error()
            routers.append(r)
        s16 = np.empty((T, H), np.uint16); s32 = np.empty((T, H), np.float32)
        assert api.lib.omega_gpu_moe_stack_bf16(stack, C.c_uint32(T), None, xb.ctypes.data_as(C.c_void_p), s16.ctypes.data_as(C.c_void_p), s32.ctypes.data_as(C.c_void_p)) == 0, api.last_error()
        h = orc.bf16_to_f32(xb); keep = np.ones(T, bool)
        for l in range(2):
            xn64, lg, lids, lw, margin = orc.router(h, nws[l], gates[l], 1e-6, topk, True)
            keep &= margin >= 1e-4
            sw = 1.0 / (1.0 + np.exp(-(xn64 @ orc.bf16_to_f32(sgate[l]).astype(np.float64))))
            i5 = np.concatenate([lids, np.full((T, 1), Er, np.uint32)], 1); w5 = np.concatenate([lw, sw[:, None]], 1).astype(np.float32)
            mo, _, _ = orc.moe_layer(None, orc.bf16_bits(orc.rmsnorm(h, 1e-6, nws[l])), wgu, sgu, wdn, sdn, topk + 1, routing=(i5, w5))
            h = h + mo
        assert keep.sum() >= T - 3 and np.max(np.abs(s32[keep] - h[keep])) <= 1e-2 and rel_l2(s32[keep], h[keep]) <= 1e-3
        api.lib.omega_gpu_moe_stack_free(stack)
        for r in routers:
            api.lib.omega_gpu_moe_router_free(r)
        api.lib.omega_gpu_moe_layer_free(layer2)
    api.lib.omega_gpu_moe_layer_free(layer); api.fp8_tensor_free(tgu); api.fp8_tensor_free(tdn)


@pytest.mark.parametrize("fmt", [0, 1, 2])
def test_w4_layer(fmt):
    """One MoE layer with 4-bit expert weights (int4 + fp16 scales, MXFP4, NVFP4) against the checker: the reference's top-k rule, per expert the double
    GEMM over the decoded weights (the decoders are pinned to the reference's oracles), the SiLU gate rounded to bf16 as the layer rounds it, the
    slot-order combine. hidden 1024, expert intermediate 768 (the six-group K quarter of the down projection), 8 experts, top-2, 40 tokens."""
    rng = np.random.default_rng(300 + fmt)
    E, H, I, K, T = 8, 1024, 768, 2, 40
    pgu = rng.integers(0, 256, (E * 2 * I, H // 2)).astype(np.uint8); pdn = rng.integers(0, 256, (E * H, I // 2)).astype(np.uint8)
    if fmt == 0:
        sgu = rng.uniform(0.002, 0.006, (E * 2 * I, H // 32)).astype(np.float16).view(np.uint16); sdn = rng.uniform(0.002, 0.006, (E * H, I // 32)).astype(np.float16).view(np.uint16)
        up, gemm = api.lib.omega_gpu_w4_upload, lambda p, sc, x: orc.w4_gemm(p, sc.view(np.float16), x)
    elif fmt == 1:
        sgu = rng.integers(117, 121, (E * 2 * I, H // 32)).astype(np.uint8); sdn = rng.integers(117, 121, (E * H, I // 32)).astype(np.uint8)
        up, gemm = api.lib.omega_gpu_mxfp4_upload, orc.mxfp4_gemm
    else:
        sgu = rng.integers(24, 40, (E * 2 * I, H // 16)).astype(np.uint8); sdn = rng.integers(24, 40, (E * H, I // 16)).astype(np.uint8)
        up, gemm = api.lib.omega_gpu_nvfp4_upload, orc.nvfp4_gemm
    tg, td = C.c_void_p(), C.c_void_p()
    assert up(C.c_uint32(E * 2 * I), C.c_uint32(H), pgu.ctypes.data_as(C.c_void_p), sgu.ctypes.data_as(C.c_void_p), C.byref(tg)) == 0, api.last_error()
    assert up(C.c_uint32(E * H), C.c_uint32(I), pdn.ctypes.data_as(C.c_void_p), sdn.ctypes.data_as(C.c_void_p), C.byref(td)) == 0, api.last_error()
    layer = C.c_void_p()
    assert api.lib.omega_gpu_moe_w4_layer_create(tg, td, C.c_uint32(E + 1), C.c_uint32(K), C.c_uint32(64), C.c_int(1), C.byref(layer)) == api.BAD_ARGS
    assert api.lib.omega_gpu_moe_w4_layer_create(tg, td, C.c_uint32(E), C.c_uint32(K), C.c_uint32(64), C.c_int(1), C.byref(layer)) == 0, api.last_error()
    logits = orc.bf16_bits(rng.normal(0, 1, (T, E)).astype(np.float32)); xb = orc.bf16_bits(rng.normal(0, 1, (T, H)).astype(np.float32))
    o16 = np.zeros((T, H), np.uint16); o32 = np.zeros((T, H), np.float32); ids = np.zeros((T, K), np.uint32); wts = np.zeros((T, K), np.float32)
    P = lambda a: a.ctypes.data_as(C.c_void_p)
    assert api.lib.omega_gpu_moe_w4_layer_bf16(layer, C.c_uint32(T), P(logits), P(xb), P(o16), P(o32), P(ids), P(wts)) == 0, api.last_error()
    rid, rw = orc.topk(orc.bf16_to_f32(logits), K, True)
    assert np.array_equal(ids, rid) and np.max(np.abs(wts - rw)) <= 1e-5
    x = orc.bf16_to_f32(xb)
    dn = np.zeros((T, K, H), np.float32)
    for e in range(E):
        tk, sl = np.nonzero(ids == e)
        if len(tk) == 0:
            continue
        gu = gemm(pgu[e * 2 * I:(e + 1) * 2 * I], np.ascontiguousarray(sgu[e * 2 * I:(e + 1) * 2 * I]), x[tk]).astype(np.float32)
        act = orc.bf16_to_f32(orc.bf16_bits(orc.swiglu(gu)))
        dn[tk, sl] = gemm(pdn[e * H:(e + 1) * H], np.ascontiguousarray(sdn[e * H:(e + 1) * H]), act).astype(np.float32)
    ref = orc.combine(wts, dn)
    err, rl2 = float(np.max(np.abs(o32 - ref))), rel_l2(o32, ref)
    assert err <= 1e-2 * max(1.0, float(np.max(np.abs(ref)))) and rl2 <= 1e-3, (err, rl2, float(np.max(np.abs(ref))))
    assert np.array_equal(o16, orc.bf16_bits(o32))
    o32b = np.zeros_like(o32)
    assert api.lib.omega_gpu_moe_w4_layer_bf16(layer, C.c_uint32(T), P(logits), P(xb), None, P(o32b), None, None) == 0 and np.array_equal(o32b.view(np.uint32), o32.view(np.uint32))
    assert api.lib.omega_gpu_moe_w4_layer_launches(layer) == 6
    api.lib.omega_gpu_moe_w4_layer_free(layer); api.lib.omega_gpu_w4_free(tg); api.lib.omega_gpu_w4_free(td)
