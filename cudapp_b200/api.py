"""ctypes binding of libb200moe.so: the same entry points a C caller links against, with numpy buffers.

Function names and argument meaning are the C ones (include/*.h); each wrapper returns the C return code
first so tests read like the reference's own C tests. There is no fallback: if the shared library is missing
the import raises, and with no CUDA device every compute call returns CHIP_FAIL (-4).
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libb200moe.so")

OK, BAD_ARGS, TOO_LARGE, CODEGEN_FAIL, CHIP_FAIL, NAN_WEIGHT = 0, -1, -2, -3, -4, -5
ENGINE_AUTO, ENGINE_FMA, ENGINE_MMA = 0, 1, 2

if not os.path.exists(LIB_PATH):
    raise ImportError("libb200moe.so is not built: run `python -m cudapp_b200.build` (needs nvcc); no CPU fallback exists")
lib = C.CDLL(LIB_PATH)


class Fp8Info(C.Structure):
    _fields_ = [("experts", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32), ("groups", C.c_uint32), ("lane_bytes", C.c_uint32),
                ("rows_per_warp", C.c_uint32), ("warps_per_cta", C.c_uint32), ("depth", C.c_uint32), ("grid_x", C.c_uint32),
                ("grid_y", C.c_uint32), ("steps", C.c_uint32), ("weight_bytes", C.c_uint64), ("scale_bytes", C.c_uint64),
                ("elapsed_ns", C.c_uint64), ("call_ns", C.c_uint64), ("completion_marker", C.c_uint32), ("kernel_cache_hit", C.c_bool),
                ("target_chip", C.c_char * 64), ("sm_architecture", C.c_uint32), ("general", C.c_uint32)]


class Fp8GemmInfo(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("segments", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32), ("mt", C.c_uint32),
                ("warps_per_cta", C.c_uint32), ("lane_bytes", C.c_uint32), ("grid_x", C.c_uint32), ("grid_y", C.c_uint32),
                ("passes_max", C.c_uint32), ("weight_bytes", C.c_uint64), ("streamed_bytes", C.c_uint64), ("elapsed_ns", C.c_uint64),
                ("call_ns", C.c_uint64), ("completion_marker", C.c_uint32), ("kernel_cache_hit", C.c_bool), ("general", C.c_uint32)]


class MoeConfig(C.Structure):
    _fields_ = [("topk", C.c_uint32), ("max_tokens", C.c_uint32), ("engine", C.c_uint32), ("x_pieces", C.c_uint32), ("act_pieces", C.c_uint32),
                ("norm_topk", C.c_uint32), ("first_expert", C.c_uint32), ("local_experts", C.c_uint32), ("tile_rows", C.c_uint32), ("shared_expert", C.c_uint32)]


class MoePlanOut(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("counts_va", "starts_va", "xmap_va", "ymap_va", "seg_a_va", "dir_a_va", "seg_b_va", "dir_b_va", "tiles_va", "header_va")]


assert C.sizeof(Fp8Info) == 160 and C.sizeof(Fp8GemmInfo) == 88

VP = C.c_void_p
lib.omega_gpu_fp8_rc_name.restype = C.c_char_p
lib.omega_gpu_fp8_last_error.restype = C.c_char_p
lib.omega_gpu_fp8gemm_rc_name.restype = C.c_char_p
lib.omega_gpu_fp8gemm_last_error.restype = C.c_char_p
lib.omega_gpu_fp8_e4m3_rne.restype = C.c_uint8
lib.omega_gpu_fp8_e4m3_rne.argtypes = [C.c_float]
lib.omega_fp8_e4m3_ref.restype = C.c_float
lib.omega_fp8_e4m3_ref.argtypes = [C.c_uint8]
lib.omega_fp8_pack_scan_nan.restype = C.c_size_t
lib.omega_gpu_fp8_tensor_free.argtypes = [VP]
lib.omega_gpu_w4_free.argtypes = [VP]
lib.omega_gpu_moe_layer_free.argtypes = [VP]
lib.omega_gpu_moe_stack_free.argtypes = [VP]
lib.omega_gpu_moe_layer_launches.argtypes = [VP]
lib.omega_gpu_moe_layer_launches.restype = C.c_uint32
lib.omega_gpu_moe_stack_launches.argtypes = [VP]
lib.omega_gpu_moe_stack_launches.restype = C.c_uint32
for _n in ("omega_moe_plan", "omega_moe_group", "omega_moe_ids32", "omega_moe_maps32", "omega_moe_segs32", "omega_moe_windows"):
    getattr(lib, _n).restype = C.c_uint32


def _p(a):
    return None if a is None else a.ctypes.data_as(VP)


def last_error():
    return lib.omega_gpu_fp8_last_error().decode()


def rc_name(rc):
    return lib.omega_gpu_fp8_rc_name(C.c_int(rc)).decode()


# ---------------------------------------------------------------- tensors and quantiser
def fp8_tensor_upload(experts, n, k, w, scale_bf16):
    """-> (rc, handle). w uint8 [experts][n][k], scale_bf16 uint16 [experts][n/128][k/128]."""
    h = VP()
    rc = lib.omega_gpu_fp8_tensor_upload(C.c_uint32(experts), C.c_uint32(n), C.c_uint32(k), _p(w), _p(scale_bf16), C.byref(h))
    return rc, (h if rc == 0 else None)


def fp8_tensor_free(t):
    lib.omega_gpu_fp8_tensor_free(t)


def fp8_tensor_shape(t):
    e, n, k = C.c_uint32(), C.c_uint32(), C.c_uint32()
    lib.omega_gpu_fp8_tensor_shape(t, C.byref(e), C.byref(n), C.byref(k))
    return e.value, n.value, k.value


def fp8_tensor_entry(t, expert):
    w, s = C.c_uint64(), C.c_uint64()
    rc = lib.omega_gpu_fp8_tensor_entry(t, C.c_uint32(expert), C.byref(w), C.byref(s))
    return rc, w.value, s.value


def fp8_quantize_bf16(w_bf16):
    n, k = w_bf16.shape
    w = np.ascontiguousarray(w_bf16, dtype=np.uint16)
    w8 = np.empty((n, k), np.uint8); sc = np.empty((max(n // 128, 1), max(k // 128, 1)), np.uint16)
    rc = lib.omega_gpu_fp8_quantize_bf16(C.c_uint32(n), C.c_uint32(k), _p(w), _p(w8), _p(sc))
    return rc, w8, sc


# ---------------------------------------------------------------- GEMV / grouped GEMM
def fp8_gemv_f32(t, expert, x, info=None):
    _, n, _ = fp8_tensor_shape(t)
    x = np.ascontiguousarray(x, dtype=np.float32); y = np.empty(n, np.float32)
    rc = lib.omega_gpu_fp8_gemv_f32(t, C.c_uint32(expert), _p(x), _p(y), C.byref(info) if info is not None else None)
    return rc, y


def fp8_gemv_bf16(t, expert, x_bf16, info=None):
    _, n, _ = fp8_tensor_shape(t)
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16); y = np.empty(n, np.float32)
    rc = lib.omega_gpu_fp8_gemv_bf16(t, C.c_uint32(expert), _p(x), _p(y), C.byref(info) if info is not None else None)
    return rc, y


def fp8_gemv_grouped_f32(t, expert_ids, x, info=None):
    _, n, k = fp8_tensor_shape(t)
    ids = np.ascontiguousarray(expert_ids, dtype=np.uint32); x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    y = np.empty((len(ids), n), np.float32)
    rc = lib.omega_gpu_fp8_gemv_grouped_f32(t, C.c_uint32(len(ids)), _p(ids), _p(x), C.c_uint32(x.shape[0]), _p(y), C.byref(info) if info is not None else None)
    return rc, y


def fp8gemm(t, expert_ids, token_rows, x, info=None):
    """x float32 -> omega_gpu_fp8gemm_f32, uint16 -> omega_gpu_fp8gemm_bf16."""
    _, n, k = fp8_tensor_shape(t)
    ids = np.ascontiguousarray(expert_ids, dtype=np.uint32); rows = np.ascontiguousarray(token_rows, dtype=np.uint32)
    x = np.ascontiguousarray(x).reshape(-1, k)
    y = np.empty((len(ids), n), np.float32)
    fn = lib.omega_gpu_fp8gemm_bf16 if x.dtype == np.uint16 else lib.omega_gpu_fp8gemm_f32
    if x.dtype != np.uint16:
        x = x.astype(np.float32, copy=False)
    rc = fn(t, C.c_uint32(len(ids)), _p(ids), _p(rows), _p(x), C.c_uint32(x.shape[0]), _p(y), C.byref(info) if info is not None else None)
    return rc, y


# ---------------------------------------------------------------- router, plan, glue
def moe_topk_bf16(logits_bf16, topk=8, norm_topk=True):
    lg = np.ascontiguousarray(logits_bf16, dtype=np.uint16)
    T, E = lg.shape
    ids = np.empty((T, topk), np.uint32); w = np.empty((T, topk), np.float32)
    rc = lib.omega_gpu_moe_topk_bf16(C.c_uint32(T), C.c_uint32(E), C.c_uint32(topk), C.c_int(1 if norm_topk else 0), _p(lg), _p(ids), _p(w))
    return rc, ids, w


def moe_plan_u32(ids, experts, ystride=None):
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    T, S = ids.shape
    ystride = S if ystride is None else ystride
    counts = np.zeros(experts, np.uint32); starts = np.zeros(experts, np.uint32)
    xmap = np.zeros(T * S + 8, np.uint32); ymap = np.zeros(T * S + 8, np.uint32); seg3 = np.zeros((experts, 3), np.uint32)
    rows, segs = C.c_uint32(), C.c_uint32()
    rc = lib.omega_gpu_moe_plan_u32(C.c_uint32(T), C.c_uint32(S), C.c_uint32(experts), C.c_uint32(ystride), _p(ids), _p(counts), _p(starts),
                                    _p(xmap), _p(ymap), _p(seg3), C.byref(rows), C.byref(segs))
    return rc, dict(counts=counts, starts=starts, xmap=xmap[: rows.value + 8], ymap=ymap[: rows.value + 8], seg3=seg3[: segs.value], rows=rows.value)


def omega_moe_plan(cfg, ids, work, seg, maps, meta):
    """ABI1 call: -> (status, result)."""
    r = C.c_uint64(99)
    st = lib.omega_moe_plan(C.byref(r), _p(cfg), C.c_uint64(len(cfg)), _p(ids), C.c_uint64(len(ids)), _p(work), C.c_uint64(len(work)),
                            _p(seg), C.c_uint64(len(seg)), _p(maps), C.c_uint64(len(maps)), _p(meta), C.c_uint64(len(meta)))
    return st, r.value


def swiglu_f32(gu):
    gu = np.ascontiguousarray(gu, dtype=np.float32)
    rows, two_i = gu.shape
    act = np.empty((rows, two_i // 2), np.float32)
    return lib.omega_gpu_swiglu_f32(C.c_uint32(rows), C.c_uint32(two_i // 2), _p(gu), _p(act)), act


def moe_combine_f32(w, d):
    w = np.ascontiguousarray(w, dtype=np.float32); d = np.ascontiguousarray(d, dtype=np.float32)
    T, S, H = d.shape
    out = np.empty((T, H), np.float32)
    return lib.omega_gpu_moe_combine_f32(C.c_uint32(T), C.c_uint32(S), C.c_uint32(H), _p(w), _p(d), _p(out)), out


def act_quant_f32(x, pieces=1):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = x.shape
    q = np.empty((pieces, rows, k), np.uint8); s = np.empty((rows, k // 128), np.float32)   # the library's layout is piece-major
    rc = lib.omega_gpu_act_quant_f32(C.c_uint32(rows), C.c_uint32(k), C.c_uint32(pieces), _p(x), _p(q), _p(s))
    return rc, np.ascontiguousarray(q.transpose(1, 0, 2)), s


# ---------------------------------------------------------------- W4
def w4_upload(packed, scale_f16):
    packed = np.ascontiguousarray(packed, dtype=np.uint8); sc = np.ascontiguousarray(scale_f16, dtype=np.uint16)
    n, k = packed.shape[0], packed.shape[1] * 2
    h = VP()
    rc = lib.omega_gpu_w4_upload(C.c_uint32(n), C.c_uint32(k), _p(packed), _p(sc), C.byref(h))
    return rc, (h if rc == 0 else None), (n, k)


def w4_gemm_bf16(t, n, x_bf16):
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    m = x.shape[0]
    y16 = np.empty((m, n), np.uint16); y32 = np.empty((m, n), np.float32)
    return lib.omega_gpu_w4_gemm_bf16(t, C.c_uint32(m), _p(x), _p(y16), _p(y32)), y16, y32


# ---------------------------------------------------------------- layer and stack
def moe_layer_create(gate_up, down, topk=8, max_tokens=256, engine=ENGINE_AUTO, x_pieces=0, act_pieces=0, norm_topk=True, tile_rows=0, shared_expert=False):
    cfg = MoeConfig(topk, max_tokens, engine, x_pieces, act_pieces, 1 if norm_topk else 0, 0, 0, tile_rows, 1 if shared_expert else 0)
    h = VP()
    rc = lib.omega_gpu_moe_layer_create(gate_up, down, C.byref(cfg), C.byref(h))
    return rc, (h if rc == 0 else None)


def moe_layer_bf16(layer, logits_bf16, x_bf16, topk=8):
    lg = np.ascontiguousarray(logits_bf16, dtype=np.uint16); x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    T, H = x.shape
    o16 = np.empty((T, H), np.uint16); o32 = np.empty((T, H), np.float32)
    ids = np.empty((T, topk), np.uint32); w = np.empty((T, topk), np.float32)
    rc = lib.omega_gpu_moe_layer_bf16(layer, C.c_uint32(T), _p(lg), _p(x), _p(o16), _p(o32), _p(ids), _p(w))
    return rc, o16, o32, ids, w


def moe_stack_create(layers, eps=1e-6):
    arr = (VP * len(layers))(*layers)
    h = VP()
    rc = lib.omega_gpu_moe_stack_create(C.c_uint32(len(layers)), arr, C.c_float(eps), C.byref(h))
    return rc, (h if rc == 0 else None)


def moe_stack_bf16(stack, logits_bf16, x_bf16, want_f32=True):
    lg = np.ascontiguousarray(logits_bf16, dtype=np.uint16); x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    T, H = x.shape
    o16 = np.empty((T, H), np.uint16); o32 = np.empty((T, H), np.float32) if want_f32 else None
    rc = lib.omega_gpu_moe_stack_bf16(stack, C.c_uint32(T), _p(lg), _p(x), _p(o16), _p(o32))
    return rc, o16, o32


def bf16_bits(x):
    """f32 array -> bf16 bit patterns (uint16), round to nearest even, NaN kept quiet"""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (b & 0x7FFFFFFF) > 0x7F800000
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(nan, ((b >> 16) | 0x40).astype(np.uint16), r)


def bf16_to_f32(bits):
    """bf16 bit patterns (uint16) -> f32"""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def moe_router_create(gate_bf16, norm_w):
    g = np.ascontiguousarray(gate_bf16, dtype=np.uint16); nw = np.ascontiguousarray(norm_w, dtype=np.float32)
    E, H = g.shape
    h = VP()
    rc = lib.omega_gpu_moe_router_create(C.c_uint32(E), C.c_uint32(H), _p(g), _p(nw), C.byref(h))
    return rc, (h if rc == 0 else None)


def moe_router_f32(router, x, experts, eps=1e-6, norm_topk=True, out_scale=1.0, topk=8):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, H = x.shape
    xn = np.empty((rows, H), np.float32); lg = np.empty((rows, experts), np.float32)
    ids = np.empty((rows, topk), np.uint32); w = np.empty((rows, topk), np.float32)
    rc = lib.omega_gpu_moe_router_f32(router, C.c_uint32(rows), _p(x), C.c_float(eps), C.c_int(1 if norm_topk else 0), C.c_float(out_scale), C.c_uint32(topk),
                                      _p(xn), _p(lg), _p(ids), _p(w))
    return rc, xn, lg, ids, w
