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
