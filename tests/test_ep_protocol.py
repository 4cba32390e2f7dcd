"""Expert-parallel exchange protocol on CPU: two gloo ranks pack their picks into fixed-capacity regions exactly as
the dispatch kernel does (cudapp_b200.ep.pack_regions restates its layout), exchange them with all-to-all, run their
local experts through the CPU checker, return the rows and combine in slot order. The result must equal the
single-process checker bit for bit (same per-row arithmetic, same combine order)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from cudapp_b200 import ep
    from oracle import oracle as orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    E, H, I, K, T = 8, 128, 128, 2, 12
    rng = np.random.default_rng(5)
    wgu = np.empty((E, 2 * I, H), np.uint8); sgu = np.empty((E, 2, 1), np.uint16); wdn = np.empty((E, H, I), np.uint8); sdn = np.empty((E, 1, 1), np.uint16)
    for e in range(E):
        wgu[e], sgu[e] = orc.quantize_bf16(orc.bf16_bits(rng.normal(0, 0.02, (2 * I, H)).astype(np.float32)))
        wdn[e], sdn[e] = orc.quantize_bf16(orc.bf16_bits(rng.normal(0, 0.02, (H, I)).astype(np.float32)))
    logits = orc.bf16_bits(rng.normal(0, 1, (T, E)).astype(np.float32)); xb = orc.bf16_bits(rng.normal(0, 1, (T, H)).astype(np.float32))
    want, _, _ = orc.moe_layer(logits, xb, wgu, sgu, wdn, sdn, K, threads=1)
    t0, t1 = ep.token_range(rank, world, T); e0, e1 = ep.expert_range(rank, world, E)
    Tl = t1 - t0
    ids, w64 = orc.topk(orc.bf16_to_f32(logits[t0:t1]), K, True)
    send, slot_pos = ep.pack_regions(ids, xb[t0:t1], world, E)
    rows, rb = ep.region_layout(Tl, K, H)
    recv = torch.zeros(world * rows * rb, dtype=torch.uint8)
    dist.all_to_all_single(recv, torch.from_numpy(send.reshape(-1)))
    recv = recv.numpy().reshape(world, rows, rb)
    dn = np.zeros((world, rows, H), np.float32)
    for r in range(world):
        cnt = int(recv[r, 0, :4].view(np.uint32)[0])
        for j in range(cnt):
            row = recv[r, 1 + j]
            eid = int(row[H * 2:].view(np.uint32)[0]) + e0
            x = orc.bf16_to_f32(row[: H * 2].view(np.uint16))[None]
            dn[r, 1 + j] = orc.expert_rows(wgu, sgu, wdn, sdn, x, [eid], [0], [0], 1, threads=1)[0]
    back = torch.zeros(world * rows * H, dtype=torch.float32)
    dist.all_to_all_single(back, torch.from_numpy(dn.reshape(-1)))
    back = back.numpy().reshape(world * rows, H)
    got = orc.combine(w64.astype(np.float32), back[slot_pos].reshape(Tl, K, H))
    ok = bool(np.array_equal(got, want[t0:t1]))
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    if rank == 0:
        ret.put(all(flags))
    dist.destroy_process_group()


def test_ep_protocol_two_gloo_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True


def test_ranges():
    from cudapp_b200 import ep
    assert [ep.expert_range(r, 4, 128) for r in range(4)] == [(0, 32), (32, 64), (64, 96), (96, 128)]
    assert ep.token_range(7, 8, 256) == (224, 256) and ep.region_layout(32, 8, 2048) == (257, 4112)


def test_fused_transport_row_addressing():
    """The fused expert-parallel transport lets a sender compute where a pick's row lives on the rank that owns the expert: the pick's
    sorted row in the plan over all experts minus the start of that rank's first expert. That must be the row the owner's own plan
    (over its experts only, ids of other ranks absent) gives the same pick, for every rank count, so that senders and owners agree
    without exchanging anything but the router logits."""
    from oracle import oracle as orc
    rng = np.random.default_rng(9)
    E, K, T = 128, 8, 96
    bias = rng.normal(0, 0.7, E)
    ids, _ = orc.topk((rng.normal(0, 1, (T, E)) + bias).astype(np.float32), K, True)
    g = orc.plan_global(ids, E)
    pos = np.empty(T * K, np.int64); pos[g["ymap"][: g["rows"]]] = np.arange(g["rows"])          # pick (t * K + s) -> sorted row over all experts
    for world in (1, 2, 4, 8):
        El = E // world
        for rank in range(world):
            local = np.where((ids >= rank * El) & (ids < (rank + 1) * El), ids - rank * El, 0xFFFFFFFF).astype(np.uint32)
            l = orc.plan_global(local, El)
            mine = np.flatnonzero(local.reshape(-1) != 0xFFFFFFFF)
            assert l["rows"] == len(mine) == int(g["counts"][rank * El:(rank + 1) * El].sum())
            lpos = np.empty(T * K, np.int64); lpos[l["ymap"][: l["rows"]]] = np.arange(l["rows"])
            assert np.array_equal(pos[mine] - int(g["starts"][rank * El]), lpos[mine])
            # the owner's plan lists the same source tokens in the same order as the slice of the global plan
            assert np.array_equal(l["xmap"][: l["rows"]], g["xmap"][int(g["starts"][rank * El]): int(g["starts"][rank * El]) + l["rows"]])


# ---------------------------------------------------------------- buffer discipline of the fused transport (a model, no GPU)
def _simulate_fused(routes, world, layers, credits, order):
    """Event model of the fused expert-parallel stack's hand-offs (csrc/moe_ep.cu). Per rank and layer two kernels run in stream order:
    EXPERT(l) starts when the delivered-row counter of parity l & 1 has reached everything the rank's plan expects up to layer l;
    COMBINE(l) starts when every rank that holds an expert of this rank's tokens has finished EXPERT(l), and then stores the rows of
    layer l + 1 into their owners' buffers of parity (l + 1) & 1. routes[l][src][dst] = rows src's tokens send to dst's experts for
    layer l. With credits, a sender first waits until the destination has finished the expert kernel of the last layer that used the
    same buffers (layer l - 1 when sending for l + 1). `order` = rank priority of an adversarial scheduler: the first rank that can
    move always moves. Returns (finished, violations): a violation = rows stored into a buffer whose previous rows were not consumed
    yet, or an expert kernel released before its own layer's rows were all in."""
    stage = [0] * world                    # kernels completed per rank: 0 = initial scatter pending, then 1 + 2 * l (+1) ...
    delivered = [[[0] * layers for _ in range(world)] for _ in range(2)]    # [parity][dst][layer] rows stored (kept per layer to audit)
    expert_done = [-1] * world
    violations = []

    def rows_expected(dst, upto_layer, parity):
        return sum(routes[l][s][dst] for l in range(upto_layer + 1) if l & 1 == parity for s in range(world))

    def send(src, layer):                  # rows of `layer` leave src
        for dst in range(world):
            n = routes[layer][src][dst]
            if not n:
                continue
            if layer >= 2 and expert_done[dst] < layer - 2:
                violations.append(("overwrite", src, dst, layer))
            delivered[layer & 1][dst][layer] += n

    def can_send(src, layer):
        if not credits or layer < 2:
            return True
        return all(expert_done[dst] >= layer - 2 for dst in range(world) if routes[layer][src][dst])

    progress = True
    while progress:
        progress = False
        for r in order:
            k = stage[r]
            if k == 0:                      # initial scatter: rows of layer 0
                send(r, 0); stage[r] = 1; progress = True; break
            l, phase = (k - 1) // 2, (k - 1) % 2
            if l >= layers:
                continue
            if phase == 0:                  # EXPERT(l): the counter of its parity only grows and is compared with a running total
                got = sum(delivered[l & 1][r])
                if got >= rows_expected(r, l, l & 1):
                    if sum(delivered[l & 1][r][: l + 1]) < rows_expected(r, l, l & 1):
                        violations.append(("early release", r, l))
                    expert_done[r] = l; stage[r] = k + 1; progress = True; break
            else:                           # COMBINE(l): needs the results of every rank its tokens were routed to
                need = [d for d in range(world) if routes[l][r][d]]
                if all(expert_done[d] >= l for d in need) and (l + 1 >= layers or can_send(r, l + 1)):
                    if l + 1 < layers:
                        send(r, l + 1)
                    stage[r] = k + 1; progress = True; break
    return all(s == 1 + 2 * layers for s in stage), violations


def test_fused_transport_buffer_credits():
    """Routing in which rank 0 sends nothing to rank 1 for two layers and then does: without the buffer credit rank 0 may store rows of
    layer 2 into rank 1's buffers while rank 1 has not consumed layer 0 (the model catches it: rows overwritten and the counter gate
    released early); with the credit every schedule finishes without a violation."""
    world, layers = 2, 5
    z = lambda: [[0] * world for _ in range(world)]
    routes = [z() for _ in range(layers)]
    for l in range(layers):
        routes[l][1][1] = 16                              # rank 1's tokens stay on rank 1's experts
        routes[l][0][0] = 16
    routes[0][1][0] = 0
    routes[2][0][1] = 8; routes[2][0][0] = 8              # from layer 2 on rank 0's tokens also use rank 1's experts
    routes[3][0][1] = 8; routes[3][0][0] = 8
    routes[4][0][1] = 4; routes[4][0][0] = 12
    done, bad = _simulate_fused(routes, world, layers, credits=False, order=[0, 1])     # rank 0 runs ahead whenever it can
    assert any(v[0] == "overwrite" for v in bad), "the model must catch the missing credit"
    for order in ([0, 1], [1, 0]):
        done, bad = _simulate_fused(routes, world, layers, credits=True, order=order)
        assert done and not bad, (order, bad)
    # dense routing (every rank sends to every rank in every layer), four ranks, every rank in turn favoured by the scheduler
    world, layers = 4, 6
    routes = [[[3 + ((l + s + d) % 4) for d in range(world)] for s in range(world)] for l in range(layers)]
    for first in range(world):
        order = [first] + [r for r in range(world) if r != first]
        done, bad = _simulate_fused(routes, world, layers, credits=True, order=order)
        assert done and not bad, (order, bad)


# ---------------------------------------------------------------- failures made on the host: a peer that disagrees, a peer that left
def _agree_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import datetime
    import torch.distributed as dist
    from cudapp_b200 import ep
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    store = ep.default_store(dist)
    out = {}
    launched = []                                             # stands for "kernels were enqueued"
    def step(i, payload, timeout=3.0):
        why = ep.agree(store, rank, world, i, payload, timeout)
        if why is None:
            launched.append(i)
        return why
    out["ok"] = step(0, {"tokens": 256, "layers": 48})                                       # everybody agrees
    out["mismatch"] = step(1, {"tokens": 256 if rank == 0 else 128, "layers": 48})           # rank 1 is about to launch another shape
    out["silent"] = ep.agree(store, rank, 3, 2, {"tokens": 256}, 1.0)                        # a third rank that never joined: it does not answer
    if rank == 1:
        ep.leave(store, rank)                                                                # rank 1 stops between steps ...
        out["left"] = "n/a"
    else:
        out["left"] = step(3, {"tokens": 256, "layers": 48})                                 # ... rank 0 learns of it before its next launch
    out["launched"] = launched
    ret.put((rank, out))
    if rank == 0:
        import time
        time.sleep(0.5)
    dist.destroy_process_group()


def test_host_side_failures_stop_a_step_before_launch():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_agree_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for r in (0, 1):
        assert got[r]["ok"] is None and got[r]["launched"] == [0]                            # only the agreed step was launched, on both ranks
        assert "posted" in got[r]["mismatch"]
    assert "left" in got[0]["left"] and "[1]" in got[0]["left"]
    for r in (0, 1):
        assert "did not answer" in got[r]["silent"] and "[2]" in got[r]["silent"]
