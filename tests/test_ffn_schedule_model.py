"""Event model of the one-launch expert kernel's unit hand-over inside a CTA (cudapp_b200/csrc/fp8_ffn_sm100.cu): the producer streams its own
gate|up units and then the down units a scheduler warp publishes into a ring; the scheduler takes the next ticket only when the producer is within
FFN_AHEAD K blocks of needing it. The model runs the two roles as interleaved state machines under every fair and unfair order the seed picks and
checks what the kernel relies on: no order deadlocks, every published unit is consumed exactly once and in order, the scheduler is never more than
one whole unit plus the look-ahead in front of the producer (so the 64-entry ring cannot wrap onto an unread entry), and the end marker arrives."""
import random

import pytest


def run(my_gu, kbx, kba, ahead, tickets_left, seed, ring=64):
    rng = random.Random(seed)
    gu_kbs = my_gu * kbx
    prog = 0                       # K blocks the producer has issued (s_prog)
    published = 0                  # ring entries published (s_published)
    entries = []                   # what the scheduler published: ticket or None (end marker)
    sched_i, sched_done = 0, False
    prod_n, prod_kb, prod_unit, prod_done = 0, 0, None, False
    consumed = []
    pool = list(range(tickets_left))   # the layer's work list as this CTA sees it: other CTAs may take tickets in between
    steps = 0
    while not (sched_done and prod_done):
        steps += 1
        assert steps < 100000, "no progress: deadlock"
        who = rng.choice(("sched", "prod")) if not sched_done and not prod_done else ("prod" if sched_done else "sched")
        if who == "sched":
            need = gu_kbs + sched_i * kba
            if prog + ahead < need:
                continue           # waits for the producer to come closer
            # another CTA may have taken some tickets meanwhile
            for _ in range(rng.randint(0, 2)):
                if pool:
                    pool.pop(0)
            t = pool.pop(0) if pool else None
            entries.append(t); published += 1; sched_i += 1
            assert published - len(consumed) <= 2 + (ahead + kba - 1) // kba, "scheduler too far ahead of the producer"
            assert published - len(consumed) < ring
            if t is None:
                sched_done = True
        else:
            if prod_unit is None:
                if prod_n < my_gu:
                    prod_unit = ("gu", prod_n); prod_kb = 0
                else:
                    i = prod_n - my_gu
                    if published <= i:
                        continue   # waits for the ring entry
                    t = entries[i]
                    consumed.append(t)
                    if t is None:
                        prod_done = True
                        continue
                    prod_unit = ("dn", t); prod_kb = 0
            kb_total = kbx if prod_unit[0] == "gu" else kba
            prod_kb += 1; prog += 1
            if prod_kb == kb_total:
                prod_unit = None; prod_n += 1
    assert consumed == entries and consumed[-1] is None and consumed.count(None) == 1
    assert prog == gu_kbs + (len(consumed) - 1) * kba
    return steps


@pytest.mark.parametrize("ahead", [0, 1, 4, 6, 9])
def test_unit_hand_over_never_deadlocks(ahead):
    seeds = 0
    for my_gu in (0, 1, 3):
        for kbx in (1, 4, 16):
            for kba in (1, 2, 5, 6):
                for tickets in (0, 1, 7):
                    for seed in range(6):
                        run(my_gu, kbx, kba, ahead, tickets, seed * 7919 + my_gu + kbx + kba + tickets)
                        seeds += 1
    assert seeds == 3 * 3 * 4 * 3 * 6
