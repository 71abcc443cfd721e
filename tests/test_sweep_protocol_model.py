"""Host-side model of the sweep kernel's row_done / row_free hand-offs
(dihydrogen_b200/csrc/conv_tc_sweep.cuh) under random schedules.

mbarrier parity waits only tell a barrier's current phase from the previous
one.  The model runs the issuers and the two epilogue halves as coroutines
over barriers with exactly that semantics and checks that no wait passes on
the wrong completion and that nobody waits for ever:

* with the rule the kernel uses (an issuer waits only for output rows its own
  input row adds into) for every filter height, issuer count and column
  height the planner can produce;
* and that the rule it replaced (always the last two rows of the column for
  the rows below it) does lock up, so the model can see the failure at all.
"""
import random

import pytest


def simulate(groups, th, fh, steps, seed, virtual, wait_rows, cg=1):
    """Returns ("ok" | "deadlock", wrong_passes).  cg > 1: the multi-group
    kernel, where row i is cg sub-rows dealt to the issuers in sequence and
    row_done[i] needs all of them."""
    rnd = random.Random(seed)
    rows = th + fh - 1
    completions, arrivals = {}, {}

    def barrier(name):
        completions[name], arrivals[name] = 0, 0

    for i in range(rows):
        barrier(("done", i))
    for j in range(th):
        barrier(("free", j))

    def arrive(name):
        arrivals[name] += 1
        if arrivals[name] == (cg if name[0] == "done" else 1):
            arrivals[name] = 0
            completions[name] += 1

    def passes(name, parity):
        return (completions[name] & 1) != parity

    wrong = []
    for j in range(th):
        arrive(("free", j))  # the epilogue's initial zeroing hands every row out once

    def issuer(mq):
        base = 0
        for step in range(steps):
            parity, real = step & 1, step not in virtual
            q = (mq + groups - base % groups) % groups if real else mq
            while q < rows * cg:
                i = q // cg
                for j in wait_rows(i, th, fh):
                    while not passes(("free", j), parity):
                        yield "wait"
                    if completions[("free", j)] != step + 1:
                        wrong.append(("issuer", mq, step, i, j))
                yield "work"
                arrive(("done", i))
                q += groups
            if real:
                base = (base + rows * cg) % groups

    def epilogue(half):
        for step in range(steps):
            parity = step & 1
            for j in range(half, th, 2):
                for i in range(j, j + fh):
                    while not passes(("done", i), parity):
                        yield "wait"
                    if completions[("done", i)] != step + 1:
                        wrong.append(("epilogue", half, step, j, i))
                yield "work"
                arrive(("free", j))

    threads = [issuer(m) for m in range(groups)] + [epilogue(0), epilogue(1)]
    alive = [True] * len(threads)
    idle = 0
    while any(alive):
        k = rnd.randrange(len(threads))
        if not alive[k]:
            continue
        try:
            idle = idle + 1 if next(threads[k]) == "wait" else 0
        except StopIteration:
            alive[k], idle = False, 0
        if idle > 20000:
            return "deadlock", wrong
    return "ok", wrong


def touched_rows(i, th, fh):
    """What the kernel waits for: the top two of the output rows that input
    row i adds into (each epilogue half retires in ascending order)."""
    hi, lo = min(i, th - 1), max(0, i - fh + 1)
    return [hi, hi - 1] if hi - 1 >= lo else [hi]


def last_two_rows(i, th, fh):
    ja = min(i, th - 1)
    return [ja, ja - 1] if ja >= 1 else [ja]


@pytest.mark.parametrize("fh", [1, 2, 3, 5])
def test_protocol_never_locks_or_passes_early(fh):
    for groups in range(1, min(fh, 3) + 1):
        for th in range(2, 14):
            for seed in range(8):
                virtual = (0, 1, 8, 9) if seed % 2 else (0, 5, 9)
                state, wrong = simulate(groups, th, fh, 10, seed, virtual, touched_rows)
                assert state == "ok" and not wrong, (fh, groups, th, seed, state, wrong[:2])


def test_waiting_for_a_row_one_does_not_touch_locks_up():
    states = {simulate(3, 7, 3, 12, seed, (0, 1, 10, 11), last_two_rows)[0] for seed in range(20)}
    assert "deadlock" in states


@pytest.mark.parametrize("cg", [3, 4, 8])
def test_multi_group_protocol(cg):
    for th in (2, 3, 7, 12, 24):
        for seed in range(6):
            state, wrong = simulate(3, th, 3, 8, seed, (0, 1, 6, 7), touched_rows, cg=cg)
            assert state == "ok" and not wrong, (cg, th, seed, state, wrong[:2])
