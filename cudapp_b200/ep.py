"""Expert-parallel driver for the MoE layer stack: one process per GPU, torch.distributed for the plumbing.

Rank r of G holds experts [r*E/G, (r+1)*E/G) of every layer and tokens [r*T/G, (r+1)*T/G). Per layer each rank runs
the library's dispatch / experts / combine entry points (csrc/moe_ep.cu); rows travel either by NCCL all-to-all of
fixed-capacity regions ("nccl") or by direct peer stores over NVLink inside the kernels ("p2p", CUDA IPC mappings
exchanged once at start-up). The whole step is captured in a CUDA graph. The reference has no multi-GPU path; the
contract here is "same numbers as one GPU".
"""
import ctypes as C
import os

import numpy as np

E, H, I, TOPK = 128, 2048, 768, 8


def expert_range(rank, world, experts):
    per = experts // world
    return rank * per, (rank + 1) * per


def token_range(rank, world, tokens):
    per = tokens // world
    return rank * per, (rank + 1) * per


def region_layout(tokens_local, topk, hidden):
    """(rows per region incl. its header row, bytes per activation row) -- must match csrc/moe_ep.cu"""
    return tokens_local * topk + 1, hidden * 2 + 16


def pack_regions(ids, x_bf16, world, experts, rank_unused=None):
    """numpy restatement of the dispatch packing for protocol tests: ids u32 [T][K], x uint16 [T][H] ->
    (send uint8 [world][rows][row_bytes], slot_pos u32 [T*K]). Region d holds this rank's picks for rank d in
    (token, slot) order; row 0 of a region is its header {count}."""
    T, K = ids.shape
    Hh = x_bf16.shape[1]
    rows, rb = region_layout(T, K, Hh)
    per = experts // world
    send = np.zeros((world, rows, rb), np.uint8)
    slot_pos = np.zeros(T * K, np.uint32)
    fill = [0] * world
    for t in range(T):
        for s in range(K):
            d = int(ids[t, s]) // per
            j = fill[d]; fill[d] += 1
            send[d, 1 + j, : Hh * 2] = x_bf16[t].view(np.uint8)
            send[d, 1 + j, Hh * 2:].view(np.uint32)[:2] = (int(ids[t, s]) - d * per, t * K + s)
            slot_pos[t * K + s] = d * rows + 1 + j
    for d in range(world):
        send[d, 0, :4].view(np.uint32)[0] = fill[d]
    return send, slot_pos


class EpStack:
    """48-layer (or fewer) expert-parallel stack on this rank's GPU."""

    def __init__(self, api, torch, dist, rank, world, layers, tokens, mode="p2p", engine=0, seed_base=0):
        self.mode = mode
        self._build_local(api, torch, dist, rank, world, layers, tokens, engine, seed_base, max_tokens=tokens + 1)
        self._build_exchange()

    def _build_local(self, api, torch, dist, rank, world, layers, tokens, engine, seed_base, max_tokens):
        self.api, self.torch, self.dist, self.rank, self.world = api, torch, dist, rank, world
        self.T, self.Tl, self.Ln = tokens, tokens // world, layers
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        e0, e1 = expert_range(rank, world, E)
        El = e1 - e0
        self.layers, self.tensors = [], []
        w8 = torch.empty((E, 2 * I, H), dtype=torch.uint8, device=dev); sc = torch.empty((E, 2 * I // 128, H // 128), dtype=torch.int16, device=dev)
        d8 = torch.empty((E, H, I), dtype=torch.uint8, device=dev); dsc = torch.empty((E, H // 128, I // 128), dtype=torch.int16, device=dev)
        lib = api.lib
        for l in range(layers):
            g = torch.Generator(device=dev); g.manual_seed(seed_base + l)     # same stream of numbers as the 1-GPU benchmark
            wgu = (torch.randn((E * 2 * I, H), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
            wdn = (torch.randn((E * H, I), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
            torch.cuda.synchronize()
            assert lib.omega_gpu_fp8_quantize_bf16_dev(C.c_uint32(E * 2 * I), C.c_uint32(H), C.c_uint64(wgu.data_ptr()), C.c_uint64(w8.data_ptr()), C.c_uint64(sc.data_ptr())) == 0, api.last_error()
            assert lib.omega_gpu_fp8_quantize_bf16_dev(C.c_uint32(E * H), C.c_uint32(I), C.c_uint64(wdn.data_ptr()), C.c_uint64(d8.data_ptr()), C.c_uint64(dsc.data_ptr())) == 0, api.last_error()
            tg, td = C.c_void_p(), C.c_void_p()
            assert lib.omega_gpu_fp8_tensor_upload_dev(C.c_uint32(El), C.c_uint32(2 * I), C.c_uint32(H), C.c_uint64(w8[e0:e1].data_ptr()), C.c_uint64(sc[e0:e1].data_ptr()), C.byref(tg)) == 0, api.last_error()
            assert lib.omega_gpu_fp8_tensor_upload_dev(C.c_uint32(El), C.c_uint32(H), C.c_uint32(I), C.c_uint64(d8[e0:e1].data_ptr()), C.c_uint64(dsc[e0:e1].data_ptr()), C.byref(td)) == 0, api.last_error()
            rc, layer = api.moe_layer_create(tg, td, topk=TOPK, max_tokens=max_tokens, engine=engine)
            assert rc == 0, api.last_error()
            self.layers.append(layer); self.tensors += [tg, td]
            del wgu, wdn
        del w8, sc, d8, dsc
        torch.cuda.empty_cache()

    def _build_exchange(self):
        api, torch, dist, rank, world, layers, tokens, dev, lib, mode = self.api, self.torch, self.dist, self.rank, self.world, self.Ln, self.T, self.dev, self.api.lib, self.mode
        rc, self.share = api.moe_stack_create(self.layers, 1e-6)       # one scratch workspace for all local layers
        assert rc == 0, api.last_error()
        ep = C.c_void_p()
        assert lib.omega_gpu_moe_ep_create(C.c_uint32(world), C.c_uint32(rank), C.c_uint32(E), C.c_uint32(TOPK), C.c_uint32(H), C.c_uint32(self.Tl), C.byref(ep)) == 0, api.last_error()
        self.ep = ep
        buf = (C.c_uint64 * 8)()
        assert lib.omega_gpu_moe_ep_buffers(ep, buf) == 0
        self.buf = list(buf)
        if mode == "p2p":
            h = (C.c_uint8 * 64)()
            assert lib.omega_gpu_moe_ep_export(ep, h) == 0, api.last_error()
            mine = torch.tensor(list(h), dtype=torch.uint8, device=dev)
            allh = torch.empty(world * 64, dtype=torch.uint8, device=dev)
            dist.all_gather_into_tensor(allh, mine)
            hb = (C.c_uint8 * (world * 64))(*allh.cpu().tolist())
            assert lib.omega_gpu_moe_ep_connect(ep, hb) == 0, api.last_error()
            dist.barrier()
        else:
            self._send = self._wrap(self.buf[0], world * self.buf[4]); self._recv = self._wrap(self.buf[1], world * self.buf[4])
            self._dn = self._wrap(self.buf[2], world * self.buf[5]); self._back = self._wrap(self.buf[3], world * self.buf[5])
        Tl = self.Tl
        self.h = torch.empty((Tl, H), dtype=torch.float32, device=dev); self.xn = torch.empty((Tl, H), dtype=torch.int16, device=dev)
        self.m = torch.empty((Tl, H), dtype=torch.float32, device=dev); self.out16 = torch.empty((Tl, H), dtype=torch.int16, device=dev)
        self.logits = torch.empty((layers, Tl, E), dtype=torch.int16, device=dev); self.x = torch.empty((Tl, H), dtype=torch.int16, device=dev)
        self.graph = None
        self.launches = 0

    def _wrap(self, va, nbytes):
        """a torch uint8 view over library-owned device memory (for the NCCL collectives)"""
        torch = self.torch

        class _Iface:
            pass
        o = _Iface()
        o.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(va), False), "version": 2}
        return torch.as_tensor(o, device=self.dev)

    def record(self, stream):
        """enqueue one whole step (all layers) on `stream`"""
        lib, api, Tl = self.api.lib, self.api, self.Tl
        sp = C.c_void_p(stream)
        n = 0
        ok = lib.omega_gpu_residual_norm_async(C.c_uint32(Tl), C.c_uint32(H), C.c_float(1e-6), C.c_uint64(self.x.data_ptr()), C.c_uint64(0), C.c_uint64(self.h.data_ptr()),
                                               C.c_uint64(self.xn.data_ptr()), C.c_uint64(0), sp); n += 1
        assert ok == 0, api.last_error()
        for l in range(self.Ln):
            assert lib.omega_gpu_moe_ep_dispatch_async(self.ep, C.c_uint32(Tl), C.c_uint64(self.logits[l].data_ptr()), C.c_uint64(self.xn.data_ptr()), sp) == 0, api.last_error()
            n += 4 + (1 if self.mode == "p2p" else 0)
            if self.mode == "nccl":
                self.dist.all_to_all_single(self._recv, self._send)
            assert lib.omega_gpu_moe_ep_experts_async(self.ep, self.layers[l], sp) == 0, api.last_error()
            n += 1 + int(lib.omega_gpu_moe_layer_launches(self.layers[l])) + (3 if self.mode == "p2p" else 0)
            if self.mode == "nccl":
                self.dist.all_to_all_single(self._back, self._dn)
            assert lib.omega_gpu_moe_ep_combine_async(self.ep, C.c_uint32(Tl), C.c_uint64(self.m.data_ptr()), C.c_uint64(0), sp) == 0, api.last_error()
            n += 1 + (1 if self.mode == "p2p" else 0)
            last = l + 1 == self.Ln
            assert lib.omega_gpu_residual_norm_async(C.c_uint32(Tl), C.c_uint32(H), C.c_float(1e-6), C.c_uint64(0), C.c_uint64(self.m.data_ptr()), C.c_uint64(self.h.data_ptr()),
                                                     C.c_uint64(0 if last else self.xn.data_ptr()), C.c_uint64(self.out16.data_ptr() if last else 0), sp) == 0, api.last_error()
            n += 1
        self.launches = n

    def capture(self):
        torch = self.torch
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.record(s.cuda_stream)          # one eager step first (lazy initialisation, NCCL warm-up)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        code = self.status()
        if code != 0:   # fail at once rather than replaying a step whose cross-GPU waits run out
            raise RuntimeError("expert-parallel step failed on rank %d: a bounded wait ran out (code %d)" % (self.rank, code))
        self.dist.barrier()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.record(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize(); self.dist.barrier()

    def step(self):
        self.graph.replay()

    def status(self):
        return int(self.api.lib.omega_gpu_moe_ep_status(self.ep, C.c_void_p(self.torch.cuda.current_stream().cuda_stream)))


class FusedEpStack(EpStack):
    """Two launches per layer and rank, three with the two-launch expert path (csrc/moe_ep.cu, "fused expert-parallel stack"): routing of all layers from the
    gathered logits up front, activation pieces and result rows travel by peer stores, waits are atomic counters."""

    def __init__(self, api, torch, dist, rank, world, layers, tokens, engine=0, seed_base=0):
        self.mode = "fused"
        self._build_local(api, torch, dist, rank, world, layers, tokens, engine, seed_base, max_tokens=tokens)
        lib, dev = api.lib, self.dev
        arr = (C.c_void_p * layers)(*self.layers)
        eps = C.c_void_p()
        assert lib.omega_gpu_moe_epstack_create(C.c_uint32(world), C.c_uint32(rank), C.c_uint32(layers), arr, C.c_uint32(E), C.c_uint32(tokens), C.c_float(1e-6), C.byref(eps)) == 0, api.last_error()
        self.eps = eps
        if world > 1:
            h = (C.c_uint8 * 64)()
            assert lib.omega_gpu_moe_epstack_export(eps, h) == 0, api.last_error()
            mine = torch.tensor(list(h), dtype=torch.uint8, device=dev)
            allh = torch.empty(world * 64, dtype=torch.uint8, device=dev)
            dist.all_gather_into_tensor(allh, mine)
            hb = (C.c_uint8 * (world * 64))(*allh.cpu().tolist())
            assert lib.omega_gpu_moe_epstack_connect(eps, hb) == 0, api.last_error()
            dist.barrier()
        Tl = self.Tl
        self.logits = torch.empty((layers, Tl, E), dtype=torch.int16, device=dev); self.x = torch.empty((Tl, H), dtype=torch.int16, device=dev)
        self.gathered = torch.empty((world, layers, Tl, E), dtype=torch.int16, device=dev)
        self.logits_all = torch.empty((layers, world * Tl, E), dtype=torch.int16, device=dev)
        self.out16 = torch.empty((Tl, H), dtype=torch.int16, device=dev)
        lib.omega_gpu_moe_epstack_h.restype = C.c_uint64
        self.h = self._wrap_f32(int(lib.omega_gpu_moe_epstack_h(eps)), Tl * H).view(Tl, H)
        self.graph = None
        self.launches = 0

    def _wrap_f32(self, va, n):
        torch = self.torch

        class _Iface:
            pass
        o = _Iface()
        o.__cuda_array_interface__ = {"shape": (int(n),), "typestr": "<f4", "data": (int(va), False), "version": 2}
        return torch.as_tensor(o, device=self.dev)

    def record(self, stream):
        lib, api = self.api.lib, self.api
        if self.world > 1:   # every rank needs the router logits of all tokens: they are small (tokens x experts x 2 bytes per layer)
            self.dist.all_gather_into_tensor(self.gathered.view(-1).view(self.torch.uint8), self.logits.view(-1).view(self.torch.uint8))
            self.logits_all.view(self.Ln, self.world, self.Tl, E).copy_(self.gathered.permute(1, 0, 2, 3))
        else:
            self.logits_all.copy_(self.logits)
        assert lib.omega_gpu_moe_epstack_step_async(self.eps, C.c_uint64(self.logits_all.data_ptr()), C.c_uint64(self.x.data_ptr()), C.c_uint64(self.out16.data_ptr()),
                                                    C.c_void_p(stream)) == 0, api.last_error()
        lib.omega_gpu_moe_epstack_launches.restype = C.c_uint32
        self.launches = int(lib.omega_gpu_moe_epstack_launches(self.eps)) + 2

    def status(self):
        return int(self.api.lib.omega_gpu_moe_epstack_status(self.eps, C.c_void_p(self.torch.cuda.current_stream().cuda_stream)))

    def step_checked(self, step_index, timeout_s=5.0):
        """step() behind the host-side hand-shake: raises before anything is launched when a peer left, is silent or disagrees"""
        why = agree(default_store(self.dist), self.rank, self.world, step_index, {"tokens": self.T, "layers": self.Ln, "world": self.world}, timeout_s)
        if why is not None:
            raise RuntimeError("expert-parallel step %d not launched: %s" % (step_index, why))
        self.step()

    def close(self):
        """free this rank's exchange object, layers and tensors (every rank must have finished its steps: peers map this memory)"""
        self.torch.cuda.synchronize(); self.dist.barrier()
        self.graph = None
        self.api.lib.omega_gpu_moe_epstack_free(self.eps)
        for layer in self.layers:
            self.api.lib.omega_gpu_moe_layer_free(layer)
        for t in self.tensors:
            self.api.fp8_tensor_free(t)
        self.layers, self.tensors = [], []
        self.torch.cuda.empty_cache(); self.dist.barrier()


def default_store(dist):
    """the rendezvous key-value store of the default process group (host side, independent of the GPU collectives)"""
    return dist.distributed_c10d._get_default_store()


def leave(store, rank):
    """A rank that stops between two steps (none of its kernels in flight) says so on the host; its peers see it in their next agree()."""
    store.set("b200moe/left/%d" % rank, "1")


def agree(store, rank, world, step, payload, timeout_s=5.0):
    """Host-side hand-shake before step `step` is enqueued. Every rank posts `payload` (what it is about to launch: token count, layer
    count, ...) and reads its peers'. Returns None when every rank answered with the same payload; otherwise a sentence saying which rank
    left, did not answer in time, or posted something else. Nothing is launched on a disagreement: the kernels of a step wait for rows
    from every rank, so a step with a missing or mismatched peer could only end in their bounded waits running out."""
    import datetime
    import json
    key = lambda r: "b200moe/agree/%d/%d" % (step, r)
    gone = lambda: [r for r in range(world) if store.check(["b200moe/left/%d" % r])]
    if gone():
        return "rank(s) %s left before step %d" % (gone(), step)
    store.set(key(rank), json.dumps(payload, sort_keys=True))
    try:
        store.wait([key(r) for r in range(world)], datetime.timedelta(seconds=timeout_s))
    except Exception:
        if gone():
            return "rank(s) %s left before step %d" % (gone(), step)
        missing = [r for r in range(world) if not store.check([key(r)])]
        return "rank(s) %s did not answer for step %d within %.1f s" % (missing, step, timeout_s)
    mine = json.dumps(payload, sort_keys=True)
    for r in range(world):
        other = store.get(key(r)).decode()
        if other != mine:
            return "rank %d posted %s for step %d, this rank %s" % (r, other, step, mine)
    return None


def parity_check(api, torch, dist, rank, world, tokens, engine, layers=2, seed_base=0):
    """Outside any timed region: a `layers`-deep instance of the fused expert-parallel stack (same seeds as the first layers of the
    benchmark) against the single-GPU stack that rank 0 builds over all experts from the same seeds. Every rank's residual rows
    must equal the single-GPU rows bit for bit. Returns the verdict agreed by all ranks."""
    st = FusedEpStack(api, torch, dist, rank, world, layers, tokens, engine=engine, seed_base=seed_base)
    logits, x = make_inputs(layers, tokens, seed=77)
    t0, t1 = token_range(rank, world, tokens)
    st.logits.copy_(torch.from_numpy(np.ascontiguousarray(logits[:, t0:t1]).view(np.int16))); st.x.copy_(torch.from_numpy(np.ascontiguousarray(x[t0:t1]).view(np.int16)))
    st.capture()            # one eager step, then the captured graph
    st.step()               # the replayed graph must give the same rows
    torch.cuda.synchronize()
    code = st.status()
    mine = torch.cat([st.h.reshape(-1).view(torch.int32), st.out16.reshape(-1).to(torch.int32)])      # f32 bits and bf16 bits of this rank's rows
    gathered = torch.empty((world, mine.numel()), dtype=torch.int32, device=st.dev)
    dist.all_gather_into_tensor(gathered.view(-1), mine)
    ok = torch.tensor([1 if code == 0 else 0], dtype=torch.int32, device=st.dev)
    if rank == 0 and code == 0:
        dev = st.dev
        full = []
        w8 = torch.empty((E, 2 * I, H), dtype=torch.uint8, device=dev); sc = torch.empty((E, 2 * I // 128, H // 128), dtype=torch.int16, device=dev)
        d8 = torch.empty((E, H, I), dtype=torch.uint8, device=dev); dsc = torch.empty((E, H // 128, I // 128), dtype=torch.int16, device=dev)
        lib = api.lib
        tensors = []
        for l in range(layers):
            g = torch.Generator(device=dev); g.manual_seed(seed_base + l)
            wgu = (torch.randn((E * 2 * I, H), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
            wdn = (torch.randn((E * H, I), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
            torch.cuda.synchronize()
            assert lib.omega_gpu_fp8_quantize_bf16_dev(C.c_uint32(E * 2 * I), C.c_uint32(H), C.c_uint64(wgu.data_ptr()), C.c_uint64(w8.data_ptr()), C.c_uint64(sc.data_ptr())) == 0, api.last_error()
            assert lib.omega_gpu_fp8_quantize_bf16_dev(C.c_uint32(E * H), C.c_uint32(I), C.c_uint64(wdn.data_ptr()), C.c_uint64(d8.data_ptr()), C.c_uint64(dsc.data_ptr())) == 0, api.last_error()
            tg, td = C.c_void_p(), C.c_void_p()
            assert lib.omega_gpu_fp8_tensor_upload_dev(C.c_uint32(E), C.c_uint32(2 * I), C.c_uint32(H), C.c_uint64(w8.data_ptr()), C.c_uint64(sc.data_ptr()), C.byref(tg)) == 0, api.last_error()
            assert lib.omega_gpu_fp8_tensor_upload_dev(C.c_uint32(E), C.c_uint32(H), C.c_uint32(I), C.c_uint64(d8.data_ptr()), C.c_uint64(dsc.data_ptr()), C.byref(td)) == 0, api.last_error()
            rc, layer = api.moe_layer_create(tg, td, topk=TOPK, max_tokens=tokens, engine=engine)
            assert rc == 0, api.last_error()
            full.append(layer); tensors += [tg, td]
            del wgu, wdn
        del w8, sc, d8, dsc
        rc, stack = api.moe_stack_create(full, 1e-6); assert rc == 0, api.last_error()
        rc, o16, o32 = api.moe_stack_bf16(stack, logits, x); assert rc == 0, api.last_error()
        got = gathered.cpu().numpy()
        Tl = tokens // world
        h_bits = np.concatenate([got[r, : Tl * H] for r in range(world)]).view(np.uint32).reshape(tokens, H)
        o_bits = np.concatenate([got[r, Tl * H:] for r in range(world)]).astype(np.uint16).reshape(tokens, H)
        same = bool(np.array_equal(h_bits, o32.view(np.uint32)) and np.array_equal(o_bits, o16))
        ok[0] = 1 if same else 0
        lib.omega_gpu_moe_stack_free(stack)
        for layer in full:
            lib.omega_gpu_moe_layer_free(layer)
        for t in tensors:
            api.fp8_tensor_free(t)
        torch.cuda.empty_cache()
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    st.close()
    return bool(ok.item() == 1), code


def make_inputs(layers, tokens, seed=0):
    from cudapp_b200.api import bf16_bits
    rng = np.random.default_rng(seed)
    logits = bf16_bits(rng.normal(0, 1, (layers, tokens, E)).astype(np.float32))
    x = bf16_bits(rng.normal(0, 1, (tokens, H)).astype(np.float32))
    return logits, x


def bench(args, rank, world):
    import json
    import time
    import torch
    import torch.distributed as dist
    from cudapp_b200 import api
    import datetime
    import sys
    import threading
    local = int(os.environ.get("LOCAL_RANK", rank))
    limit = float(os.environ.get("B200MOE_BENCH_LIMIT_S", "420"))

    def give_up():
        # every device wait is bounded, so a rank stuck here is waiting on the host for a peer that already left
        sys.stderr.write("rank %d: benchmark exceeded %.0f s; leaving\n" % (rank, limit)); sys.stderr.flush()
        os._exit(3)
    watchdog = threading.Timer(limit, give_up); watchdog.daemon = True; watchdog.start()
    torch.cuda.set_device(local)
    os.environ.setdefault("B200MOE_DEVICE", str(local))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")   # NCCL only carries a barrier, small gathers and reductions here; no rank's buffers get bound to a multicast object
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=180))
    mode = os.environ.get("B200MOE_EP_MODE", "fused")
    Ln, T = args.layers, args.tokens
    parity = None
    if mode == "fused":
        same, code = parity_check(api, torch, dist, rank, world, T, args.engine)
        parity = {"bit_equal": same, "layers": 2, "ranks": world, "against": "single-GPU stack on rank 0, same seeds", "status": code}
        if not same:
            if rank == 0:
                print(json.dumps({"metric": "moe_layer_tokens_per_s", "n_gpus": world, "parity": parity, "error": "expert-parallel rows differ from the single-GPU stack"}))
            sys.stdout.flush(); torch.cuda.synchronize(); dist.barrier()
            os._exit(4)
    st = FusedEpStack(api, torch, dist, rank, world, Ln, T, engine=args.engine) if mode == "fused" else EpStack(api, torch, dist, rank, world, Ln, T, mode=mode, engine=args.engine)
    logits, x = make_inputs(Ln, T)
    t0, t1 = token_range(rank, world, T)
    lg_h = torch.from_numpy(np.ascontiguousarray(logits[:, t0:t1]).view(np.int16)).pin_memory(); x_h = torch.from_numpy(np.ascontiguousarray(x[t0:t1]).view(np.int16)).pin_memory()
    out_h = torch.empty((t1 - t0, H), dtype=torch.int16).pin_memory()
    st.logits.copy_(lg_h); st.x.copy_(x_h)
    st.capture()
    from bench import ClockSampler
    for _ in range(max(args.warmup, 3)):
        st.step()
    torch.cuda.synchronize(); dist.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        ev0.record()
        for _ in range(args.steps):
            st.step()
        ev1.record()
        torch.cuda.synchronize()
    dist.barrier()
    ms = torch.tensor([ev0.elapsed_time(ev1)], device="cuda"); dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    status = st.status()
    assert status == 0, "a bounded cross-GPU wait ran out (code %d)" % status
    assert torch.isfinite(st.h).all()
    # end to end: this rank's slice from pinned host memory in, its output slice back, every step
    def e2e_step():
        st.logits.copy_(lg_h, non_blocking=True); st.x.copy_(x_h, non_blocking=True)
        st.step()
        out_h.copy_(st.out16, non_blocking=True)
        torch.cuda.synchronize()
    e2e_step(); dist.barrier()
    t_0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    e2e = torch.tensor([(time.perf_counter() - t_0) / args.steps], device="cuda"); dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
    if rank == 0:
        total_s = float(ms.item()) * 1e-3
        from bench import GU_BYTES, DN_BYTES, measured_peak
        peak, kind = measured_peak()
        per_gpu_bytes = Ln * (E // world) * (GU_BYTES + DN_BYTES)
        achieved = per_gpu_bytes / (total_s / args.steps) / 1e9
        print(json.dumps({
            "metric": "moe_layer_tokens_per_s", "value": T * args.steps / total_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": float(ms.item()) / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 weights, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": "48-layer MoE expert stack, 256 decode tokens/step, 128 experts top-8, hidden 2048, inter 768", "layers": Ln, "tokens_per_step": T,
                       "parallelism": "ep%d (experts and tokens sharded; %s)" % (world, {"fused": "rows and results by peer stores over NVLink inside the layer kernels, 2 launches per layer", "p2p": "direct peer stores over NVLink", "nccl": "NCCL all-to-all"}[mode]),
                       "l2": "%.1f GB of weights per GPU per step: larger than L2" % (per_gpu_bytes / 1e9)},
            "e2e": {"value": T / float(e2e.item()), "unit": "tokens/s", "h2d_bytes_per_step": int((lg_h.numel() + x_h.numel()) * 2 * world), "d2h_bytes_per_step": int(out_h.numel() * 2 * world)},
            "gpu_launches": int(st.launches) * args.steps, "parity": parity,
            "roofline": {"bound": "hbm", "kernel": "whole step per GPU (weights streamed once)", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": kind + " copy bandwidth", "traffic": None},
            "clocks": clocks.summary()}))
    torch.cuda.synchronize(); dist.barrier()
    sys.stdout.flush(); sys.stderr.flush()
    os._exit(0)   # a process group whose collectives sit in a captured graph does not tear down reliably; leave at once
