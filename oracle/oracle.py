"""ctypes access to the CPU checker (liboracle.so) and, where it was built, to the reference's own host
code (_ref/libref.so, _ref/libref_group.so).

Test infrastructure only: imported by tests/, by the smoke check and by the benchmark's CPU-baseline and
reference legs. The product package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
U8P, U16P, U32P, U64P = (C.POINTER(t) for t in (C.c_uint8, C.c_uint16, C.c_uint32, C.c_uint64))
F32P, F64P = C.POINTER(C.c_float), C.POINTER(C.c_double)


def _ptr(a, typ):
    return None if a is None else a.ctypes.data_as(typ)


def build(ref=False):
    """Compile the checker (and, with ref=True and the reference tree present, the reference build)."""
    subprocess.run(["make", "-s", "-C", HERE, "all"], check=True)
    where = os.environ.get("B200MOE_REFERENCE", os.path.normpath(os.path.join(HERE, "..", "..", "reference")))   # beside this repository's folder
    if ref and os.path.isdir(where):
        subprocess.run(["make", "-s", "-C", HERE, "ref", "REF=" + where], check=True)


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.orc_bf16_to_f32.restype = C.c_float; L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_bf16.restype = C.c_uint16; L.orc_f32_to_bf16.argtypes = [C.c_float]
        L.orc_e4m3_decode.restype = C.c_float; L.orc_e4m3_decode.argtypes = [C.c_uint8]
        L.orc_e4m3_encode.restype = C.c_uint8; L.orc_e4m3_encode.argtypes = [C.c_float]
        L.orc_f32_to_f16.restype = C.c_uint16; L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_f16_to_f32.restype = C.c_float; L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_gemv_emu_row.restype = C.c_float
        for n in ("orc_moe_plan", "orc_moe_ids32", "orc_moe_maps32", "orc_moe_segs32", "orc_moe_windows", "orc_moe_group"):
            getattr(L, n).restype = C.c_uint64
        L.orc_plan_global.restype = C.c_int64
        _lib = L
    return _lib


def ref_lib():
    """The reference's own host functions, or None when that build is not present."""
    path = os.path.join(HERE, "_ref", "libref.so")
    if not os.path.exists(path):
        return None
    L = C.CDLL(path)
    L.omega_fp8_e4m3_ref.restype = C.c_float; L.omega_fp8_e4m3_ref.argtypes = [C.c_uint8]
    L.omega_gpu_fp8_e4m3_rne.restype = C.c_uint8; L.omega_gpu_fp8_e4m3_rne.argtypes = [C.c_float]
    L.omega_bf16_to_fp32.restype = C.c_float; L.omega_bf16_to_fp32.argtypes = [C.c_uint16]
    L.omega_fp32_to_bf16.restype = C.c_uint16; L.omega_fp32_to_bf16.argtypes = [C.c_float]
    return L


def ref_group_lib():
    path = os.path.join(HERE, "_ref", "libref_group.so")
    return C.CDLL(path) if os.path.exists(path) else None


# ---------------------------------------------------------------- numpy front ends

def bf16_bits(x):
    """f32 array -> bf16 bit patterns (uint16), round to nearest even (vectorised orc_f32_to_bf16)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (b & 0x7FFFFFFF) > 0x7F800000
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(nan, ((b >> 16) | 0x40).astype(np.uint16), r)


def bf16_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def e4m3_table():
    L = lib()
    return np.array([L.orc_e4m3_decode(i) for i in range(256)], dtype=np.float32)


def quantize_bf16(w_bf16):
    """bf16 bits [n][k] -> (e4m3 codes [n][k], bf16 scales [n/128][k/128])."""
    n, k = w_bf16.shape
    w = np.ascontiguousarray(w_bf16, dtype=np.uint16)
    w8 = np.empty((n, k), np.uint8); sc = np.empty((n // 128, k // 128), np.uint16)
    rc = lib().orc_quantize_bf16(C.c_uint32(n), C.c_uint32(k), _ptr(w, U16P), _ptr(w8, U8P), _ptr(sc, U16P))
    if rc != 0:
        raise ValueError("orc_quantize_bf16 refused the input")
    return w8, sc


def gemv(w8, sc, x, mag=False):
    n, k = w8.shape
    w8 = np.ascontiguousarray(w8); sc = np.ascontiguousarray(sc); x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(n, np.float64); m = np.empty(n, np.float64) if mag else None
    lib().orc_gemv(_ptr(w8, U8P), _ptr(sc, U16P), C.c_uint32(n), C.c_uint32(k), _ptr(x, F32P), _ptr(y, F64P), _ptr(m, F64P))
    return (y, m) if mag else y


def gemv_emu(w8, sc, x):
    n, k = w8.shape
    w8 = np.ascontiguousarray(w8); sc = np.ascontiguousarray(sc); x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(n, np.float32)
    lib().orc_gemv_emu(_ptr(w8, U8P), _ptr(sc, U16P), C.c_uint32(n), C.c_uint32(k), _ptr(x, F32P), _ptr(y, F32P))
    return y


def topk(logits, k=8, norm=True):
    """logits f32 [T][E] -> (ids u32 [T][k], weights f64 [T][k])."""
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    T, E = lg.shape
    ids = np.empty((T, k), np.uint32); w = np.empty((T, k), np.float64)
    L = lib()
    for t in range(T):
        L.orc_topk(_ptr(lg[t], F32P), C.c_uint32(E), C.c_uint32(k), C.c_int(1 if norm else 0), _ptr(ids[t], U32P), _ptr(w[t], F64P))
    return ids, w


def router(x, norm_w, gate_bf16, eps=1e-6, k=8, norm=True):
    """x f32 [rows][H], norm_w f32 [H], gate bf16 bits [E][H] -> (xn f64 [rows][H], logits f64 [rows][E], ids u32 [rows][k],
    weights f64 [rows][k], margin f64 [rows])."""
    x = np.ascontiguousarray(x, dtype=np.float32); nw = np.ascontiguousarray(norm_w, dtype=np.float32)
    g = np.ascontiguousarray(gate_bf16, dtype=np.uint16)
    rows, H = x.shape; E = g.shape[0]
    xn = np.empty((rows, H), np.float64); lg = np.empty((rows, E), np.float64)
    ids = np.empty((rows, k), np.uint32); w = np.empty((rows, k), np.float64); margin = np.empty(rows, np.float64)
    L = lib()
    for r in range(rows):
        m = C.c_double(0)
        L.orc_router(_ptr(x[r], F32P), _ptr(nw, F32P), _ptr(g, U16P), C.c_uint32(H), C.c_uint32(E), C.c_uint32(k), C.c_float(eps), C.c_int(1 if norm else 0),
                     _ptr(xn[r], F64P), _ptr(lg[r], F64P), _ptr(ids[r], U32P), _ptr(w[r], F64P), C.byref(m))
        margin[r] = m.value
    return xn, lg, ids, w, margin


def ref_router_lib():
    path = os.path.join(HERE, "_ref", "libref_router.so")
    return C.CDLL(path) if os.path.exists(path) else None


def ref_static_lib(which):
    """One of the reference test files' static functions, compiled in place (oracle/ref_static_shims.c): which = "emu", "pq" or "mc"."""
    path = os.path.join(HERE, "_ref", "libref_%s.so" % which)
    if not os.path.exists(path):
        return None
    L = C.CDLL(path)
    if which == "emu":
        L.ref_emu_row.restype = C.c_float
    return L


def combine_mc(down, inv, wt):
    """prefill form of the combine: down f32 [R][H], inv u32 [T][K], wt f32 [T][K] -> out f32 [T][H] (accumulator starts at +0)."""
    down = np.ascontiguousarray(down, dtype=np.float32); inv = np.ascontiguousarray(inv, dtype=np.uint32); wt = np.ascontiguousarray(wt, dtype=np.float32)
    T, K = inv.shape
    H = down.shape[1]
    out = np.empty((T, H), np.float32)
    lib().orc_combine_mc(_ptr(down, F32P), _ptr(inv, U32P), _ptr(wt, F32P), C.c_uint32(T), C.c_uint32(H), C.c_uint32(K), _ptr(out, F32P))
    return out


def swiglu(gu):
    gu = np.ascontiguousarray(gu, dtype=np.float32)
    rows, two_i = gu.shape
    act = np.empty((rows, two_i // 2), np.float32)
    L = lib()
    for r in range(rows):
        L.orc_swiglu(_ptr(gu[r], F32P), C.c_uint32(two_i // 2), _ptr(act[r], F32P))
    return act


def combine(w, d):
    """w f32 [T][S], d f32 [T][S][H] -> out f32 [T][H] (multiply then add, slot order)."""
    w = np.ascontiguousarray(w, dtype=np.float32); d = np.ascontiguousarray(d, dtype=np.float32)
    T, S, H = d.shape
    out = np.empty((T, H), np.float32)
    L = lib()
    for t in range(T):
        L.orc_combine(_ptr(w[t], F32P), _ptr(d[t], F32P), C.c_uint32(S), C.c_uint32(H), _ptr(out[t], F32P))
    return out


def rmsnorm(x, eps=1e-6, w=None):
    """x f32 [T][H] -> x * rsqrt(mean(x^2) + eps) * w (w f32 [H], None = ones)"""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = None if w is None else np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty_like(x)
    L = lib()
    for t in range(x.shape[0]):
        L.orc_rmsnorm(_ptr(x[t], F32P), _ptr(w, F32P), C.c_uint32(x.shape[1]), C.c_float(eps), _ptr(out[t], F32P))
    return out


def plan_buffers(fill=0x5A):
    mk = lambda n: np.full(n, fill * 0x0101010101010101, np.uint64)
    return mk(10368), mk(1028), mk(2320), mk(8)


def moe_plan(cfg, ids, work, seg, maps, meta):
    cfg = np.ascontiguousarray(cfg, dtype=np.uint64); ids = np.ascontiguousarray(ids, dtype=np.uint64)
    return int(lib().orc_moe_plan(_ptr(cfg, U64P), _ptr(ids, U64P), _ptr(work, U64P), _ptr(seg, U64P), _ptr(maps, U64P), _ptr(meta, U64P)))


def plan_global(ids, experts, ystride=None):
    """ids u32 [T][S] -> dict(counts, starts, xmap, ymap, seg3 [segs][3], rows). Any T."""
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    T, S = ids.shape
    ystride = S if ystride is None else ystride
    counts = np.empty(experts, np.uint32); starts = np.empty(experts, np.uint32)
    xmap = np.zeros(T * S + 8, np.uint32); ymap = np.zeros(T * S + 8, np.uint32)
    seg3 = np.zeros((experts, 3), np.uint32); rows = C.c_uint32(0)
    n = lib().orc_plan_global(C.c_uint32(T), C.c_uint32(S), C.c_uint32(experts), C.c_uint32(ystride), _ptr(ids, U32P),
                              _ptr(counts, U32P), _ptr(starts, U32P), _ptr(xmap, U32P), _ptr(ymap, U32P), _ptr(seg3, U32P), C.byref(rows))
    if n < 0:
        raise ValueError("expert id out of range")
    return dict(counts=counts, starts=starts, xmap=xmap[: rows.value + 8], ymap=ymap[: rows.value + 8], seg3=seg3[:n], rows=rows.value)


def act_quant(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = x.shape
    q = np.empty((rows, k), np.uint8); s = np.empty((rows, k // 128), np.float32)
    L = lib()
    for r in range(rows):
        L.orc_act_quant(_ptr(x[r], F32P), C.c_uint32(k), _ptr(q[r], U8P), _ptr(s[r], F32P))
    return q, s


def act_pieces(x, pieces):
    """x f32 [rows][k] -> (q u8 [rows][pieces][k], s f32 [rows][k/128])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = x.shape
    q = np.empty((rows, pieces, k), np.uint8); s = np.empty((rows, k // 128), np.float32)
    L = lib()
    for r in range(rows):
        L.orc_act_pieces(_ptr(x[r], F32P), C.c_uint32(k), C.c_uint32(pieces), _ptr(q[r], U8P), _ptr(s[r], F32P))
    return q, s


def act_pieces_decode(q, s):
    rows, pieces, k = q.shape
    out = np.empty((rows, k), np.float64)
    L = lib()
    for r in range(rows):
        L.orc_act_pieces_decode(_ptr(np.ascontiguousarray(q[r]), U8P), _ptr(np.ascontiguousarray(s[r]), F32P), C.c_uint32(k), C.c_uint32(pieces), _ptr(out[r], F64P))
    return out


def w4_quantize(w):
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    packed = np.empty((n, k // 2), np.uint8); sc = np.empty((n, k // 32), np.uint16)
    lib().orc_w4_quantize(C.c_uint32(n), C.c_uint32(k), _ptr(w, F32P), _ptr(packed, U8P), _ptr(sc, U16P))
    return packed, sc


def w4_gemm(packed, sc, x, threads=None):
    import concurrent.futures as cf
    packed = np.ascontiguousarray(packed); sc = np.ascontiguousarray(sc); x = np.ascontiguousarray(x, dtype=np.float32)
    n, k = packed.shape[0], packed.shape[1] * 2
    m = x.shape[0]
    y = np.empty((m, n), np.float64)
    L = lib()
    threads = threads or min(os.cpu_count() or 1, 32)
    step = max(1, (n + threads - 1) // threads)

    def run(r0):
        L.orc_w4_gemm_rows(_ptr(packed, U8P), _ptr(sc, U16P), C.c_uint32(k), C.c_uint32(r0), C.c_uint32(min(n, r0 + step)),
                           C.c_uint32(n), _ptr(x, F32P), C.c_uint32(m), _ptr(y, F64P))
    with cf.ThreadPoolExecutor(threads) as ex:
        list(ex.map(run, range(0, n, step)))
    return y


def mxfp4_bits(nib, scale):
    L = lib(); L.orc_mxfp4_bits.restype = C.c_uint32
    return int(L.orc_mxfp4_bits(C.c_uint32(int(nib)), C.c_uint32(int(scale))))


def mxfp4_gemm(packed, scale_e8m0, x, threads=None):
    """packed u8 [n][k/2] (low nibble = even column), scale u8 [n][k/32], x f32 [m][k] -> y f64 [m][n]"""
    import concurrent.futures as cf
    packed = np.ascontiguousarray(packed, dtype=np.uint8); sc = np.ascontiguousarray(scale_e8m0, dtype=np.uint8); x = np.ascontiguousarray(x, dtype=np.float32)
    n, k = packed.shape[0], packed.shape[1] * 2
    m = x.shape[0]
    y = np.empty((m, n), np.float64)
    L = lib()
    threads = threads or min(os.cpu_count() or 1, 32)
    step = max(1, (n + threads - 1) // threads)

    def run(r0):
        L.orc_mxfp4_gemm_rows(_ptr(packed, U8P), _ptr(sc, U8P), C.c_uint32(k), C.c_uint32(r0), C.c_uint32(min(n, r0 + step)), C.c_uint32(n), _ptr(x, F32P), C.c_uint32(m), _ptr(y, F64P))
    with cf.ThreadPoolExecutor(threads) as ex:
        list(ex.map(run, range(0, n, step)))
    return y


def nvfp4_bits(nib, scale):
    L = lib(); L.orc_nvfp4_bits.restype = C.c_uint32
    return int(L.orc_nvfp4_bits(C.c_uint32(int(nib)), C.c_uint32(int(scale))))


def nvfp4_gemm(packed, scale_ue4m3, x, threads=None):
    """packed u8 [n][k/2] (low nibble = even column), scale u8 [n][k/16] (E4M3 codes 0..126), x f32 [m][k] -> y f64 [m][n]"""
    import concurrent.futures as cf
    packed = np.ascontiguousarray(packed, dtype=np.uint8); sc = np.ascontiguousarray(scale_ue4m3, dtype=np.uint8); x = np.ascontiguousarray(x, dtype=np.float32)
    n, k = packed.shape[0], packed.shape[1] * 2
    m = x.shape[0]
    y = np.empty((m, n), np.float64)
    L = lib()
    threads = threads or min(os.cpu_count() or 1, 32)
    step = max(1, (n + threads - 1) // threads)

    def run(r0):
        L.orc_nvfp4_gemm_rows(_ptr(packed, U8P), _ptr(sc, U8P), C.c_uint32(k), C.c_uint32(r0), C.c_uint32(min(n, r0 + step)), C.c_uint32(n), _ptr(x, F32P), C.c_uint32(m), _ptr(y, F64P))
    with cf.ThreadPoolExecutor(threads) as ex:
        list(ex.map(run, range(0, n, step)))
    return y


def nvfp4_enc(bits, scale):
    """E2M1 nibbles of binary32 bit patterns `bits` (u32 array) under one scale code; 0xff where the reference's unit traps"""
    bits = np.ascontiguousarray(bits, dtype=np.uint32); out = np.empty(bits.size, np.uint8)
    lib().orc_nvfp4_enc_many(_ptr(bits, U32P), C.c_size_t(bits.size), C.c_uint32(int(scale)), _ptr(out, U8P))
    return out


def nvfp4_scale(amax_bits):
    amax_bits = np.ascontiguousarray(amax_bits, dtype=np.uint32); out = np.empty(amax_bits.size, np.uint8)
    lib().orc_nvfp4_scale_many(_ptr(amax_bits, U32P), C.c_size_t(amax_bits.size), _ptr(out, U8P))
    return out


def nvfp4_quantize(x):
    """x f32 [rows][k] -> (packed u8 [rows][k/2], scales u8 [rows][k/16]) by the reference's block rule; raises on a NaN value"""
    x = np.ascontiguousarray(x, dtype=np.float32); rows, k = x.shape
    packed = np.empty((rows, k // 2), np.uint8); scales = np.empty((rows, k // 16), np.uint8)
    L = lib(); L.orc_nvfp4_quantize.restype = C.c_size_t
    bad = L.orc_nvfp4_quantize(_ptr(x.view(np.uint32), U32P), C.c_size_t(rows), C.c_size_t(k), _ptr(packed, U8P), _ptr(scales, U8P))
    if bad:
        raise ValueError("nvfp4_quantize: %d blocks hold a NaN" % bad)
    return packed, scales


def mxmm(fmt, m, n, k, A, SA, B, SB):
    """block-scaled C = A B^T of the reference's mxdot unit (fmt 0 NVFP4, 1 MXFP4, 2 MXFP8): returns (rc, C f64 [m][n], sum of |terms| [m][n])"""
    A = np.ascontiguousarray(A, dtype=np.uint8); B = np.ascontiguousarray(B, dtype=np.uint8)
    SA = np.ascontiguousarray(SA, dtype=np.uint8); SB = np.ascontiguousarray(SB, dtype=np.uint8)
    Cm = np.zeros((m, n), np.float64); mag = np.zeros((m, n), np.float64)
    L = lib(); L.orc_mxmm.restype = C.c_int
    rc = L.orc_mxmm(C.c_uint32(fmt), C.c_uint32(m), C.c_uint32(n), C.c_uint32(k), _ptr(A, U8P), _ptr(SA, U8P), _ptr(B, U8P), _ptr(SB, U8P), _ptr(Cm, F64P), _ptr(mag, F64P))
    return int(rc), Cm, mag


def expert_rows(wgu, sgu, wdn, sdn, x, row_expert, row_token, row_dest, n_dest, threads=None, x_pieces=0, act_pieces=0):
    """Gate|up GEMV, SwiGLU and down GEMV for every sorted row (the reference host glue); ctypes releases
    the GIL, so rows are spread over `threads` host threads. Returns dn f32 [n_dest][hidden]."""
    import concurrent.futures as cf
    E, n2, hidden = wgu.shape
    inter = n2 // 2
    wgu = np.ascontiguousarray(wgu); sgu = np.ascontiguousarray(sgu); wdn = np.ascontiguousarray(wdn); sdn = np.ascontiguousarray(sdn)
    x = np.ascontiguousarray(x, dtype=np.float32)
    re_ = np.ascontiguousarray(row_expert, dtype=np.uint32); rt = np.ascontiguousarray(row_token, dtype=np.uint32)
    rd = np.ascontiguousarray(row_dest, dtype=np.uint32)
    rows = len(re_)
    dn = np.zeros((n_dest, hidden), np.float32)
    L = lib()
    threads = threads or min(os.cpu_count() or 1, 64)
    step = max(1, (rows + threads * 4 - 1) // (threads * 4))

    def run(p0):
        L.orc_expert_rows_q(_ptr(wgu, U8P), _ptr(sgu, U16P), _ptr(wdn, U8P), _ptr(sdn, U16P), C.c_uint32(hidden), C.c_uint32(inter),
                            _ptr(x, F32P), _ptr(re_, U32P), _ptr(rt, U32P), _ptr(rd, U32P), C.c_uint32(p0), C.c_uint32(min(rows, p0 + step)), _ptr(dn, F32P),
                            C.c_uint32(x_pieces), C.c_uint32(act_pieces))
    with cf.ThreadPoolExecutor(threads) as ex:
        list(ex.map(run, range(0, rows, step)))
    return dn


def moe_layer(logits_bf16, x_bf16, wgu, sgu, wdn, sdn, topk_k=8, threads=None, x_pieces=0, act_pieces=0, routing=None):
    """One MoE layer exactly as the reference host glue strings the operators together: top-k (lowest
    index on ties, renormalised softmax), per pick gate|up GEMV -> SwiGLU -> down GEMV, slot-order weighted
    sum. Inputs bf16 bit patterns; returns (out f32 [T][H], ids, wts f32). x_pieces / act_pieces > 0 pass the layer input /
    the gated activations through the e4m3 piece quantiser first (the tensor-core engine's arithmetic model)."""
    x = bf16_to_f32(x_bf16)
    T, H = x.shape
    if routing is not None:   # (ids u32 [T][k], weights f32 [T][k]) computed elsewhere (the router front half); logits_bf16 is ignored
        ids, wts = np.ascontiguousarray(routing[0], dtype=np.uint32), np.ascontiguousarray(routing[1], dtype=np.float32)
    else:
        ids, w64 = topk(bf16_to_f32(logits_bf16), topk_k, True)
        wts = w64.astype(np.float32)
    re_ = ids.reshape(-1); rt = np.repeat(np.arange(T, dtype=np.uint32), topk_k); rd = np.arange(T * topk_k, dtype=np.uint32)
    dn = expert_rows(wgu, sgu, wdn, sdn, x, re_, rt, rd, T * topk_k, threads, x_pieces, act_pieces)
    out = combine(wts, dn.reshape(T, topk_k, H))
    return out, ids, wts
