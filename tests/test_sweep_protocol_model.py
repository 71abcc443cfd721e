"""Host-side model of the sweep kernel's row_done / row_free hand-offs
(dihydrogen_b200/csrc/conv_tc_sweep.cuh) under random schedules.

mbarrier parity waits only tell a barrier's current phase from the previous
one.  The model runs the issuers and the two epilogue halves as coroutines
over barriers with exactly that semantics and checks that no wait passes on
the wrong completion, that no issuer adds into a row that has not been retired
and that nobody waits for ever:

* with the rule the kernel uses (an issuer waits only for output rows its own
  input row adds into) for every filter height, issuer count and column
  height the planner can produce;
* and that the rule it replaced (always the last two rows of the column for
  the rows below it) does lock up, so the model can see the failure at all.
"""
import random

import pytest


def simulate(groups, th, fh, steps, seed, virtual, wait_rows, cg=1, nhalf=2, blocked=False, ipg=1, sync=True):
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

    def issuer_blocked(mq):
        # the sweep kernel: issuer mq owns a contiguous block of rows in every step
        rpg = -(-rows // groups)
        for step in range(steps):
            parity = step & 1
            for i in range(mq * rpg, min(rows, (mq + 1) * rpg)):
                for j in wait_rows(i, th, fh):
                    while not passes(("free", j), parity):
                        yield "wait"
                    if completions[("free", j)] != step + 1:
                        wrong.append(("issuer", mq, step, i, j))
                for j in range(max(0, i - fh + 1), min(i, th - 1) + 1):
                    if completions[("free", j)] < step + 1:
                        wrong.append(("issuer adds into an unretired row", mq, step, i, j))
                yield "work"
                arrive(("done", i))

    iss_done = [[0] * ipg for _ in range(groups)]  # steps finished by issuer (mq, mh)

    def issuer_blocked_pair(mq, mh):
        # the sweep kernel with two A slots per group: issuer (mq, mh) owns the group's real
        # rows whose slot is mh (a running count), the first issuer all virtual ones; the
        # issuers of a group start a step only when all of them have finished the one before
        rpg = -(-rows // groups)
        lap = 0
        for step in range(steps):
            if sync and step > 0:
                while min(iss_done[mq]) < step:
                    yield "wait"
            parity, real = step & 1, step not in virtual
            for i in range(mq * rpg, min(rows, (mq + 1) * rpg)):
                mine = (lap == mh) if real else (mh == 0)
                if real:
                    lap = (lap + 1) % ipg
                if not mine:
                    continue
                for j in wait_rows(i, th, fh):
                    while not passes(("free", j), parity):
                        yield "wait"
                    if completions[("free", j)] != step + 1:
                        wrong.append(("issuer", mq, mh, step, i, j))
                for j in range(max(0, i - fh + 1), min(i, th - 1) + 1):
                    if completions[("free", j)] < step + 1:
                        wrong.append(("issuer adds into an unretired row", mq, mh, step, i, j))
                yield "work"
                arrive(("done", i))
            iss_done[mq][mh] = step + 1

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
                # data hazard: every output row this input row adds into must have been
                # retired (zeroed) for this step, whether or not it was waited for
                for j in range(max(0, i - fh + 1), min(i, th - 1) + 1):
                    if completions[("free", j)] < step + 1:
                        wrong.append(("issuer adds into an unretired row", mq, step, i, j))
                yield "work"
                arrive(("done", i))
                q += groups
            if real:
                base = (base + rows * cg) % groups

    def epilogue(half):
        for step in range(steps):
            parity = step & 1
            for j in range(half, th, nhalf):
                for i in range(j, j + fh):
                    while not passes(("done", i), parity):
                        yield "wait"
                    if completions[("done", i)] != step + 1:
                        wrong.append(("epilogue", half, step, j, i))
                yield "work"
                arrive(("free", j))

    if ipg > 1:
        threads = [issuer_blocked_pair(m, h) for m in range(groups) for h in range(ipg)]
    else:
        threads = [(issuer_blocked if blocked else issuer)(m) for m in range(groups)]
    threads += [epilogue(h) for h in range(nhalf)]
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


def touched_rows(i, th, fh, n=2):
    """What the kernel waits for: the top n (= epilogue warps per quadrant) of
    the output rows that input row i adds into; each of those warps retires its
    rows in ascending order, so they stand for all rows below."""
    hi, lo = min(i, th - 1), max(0, i - fh + 1)
    return list(range(hi, max(lo, hi - n + 1) - 1, -1))


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


@pytest.mark.parametrize("nhalf", [2, 3, 4])
def test_protocol_with_rows_dealt_in_blocks(nhalf):
    """The sweep kernel deals a step's rows to its issuers in contiguous blocks
    (so that concurrent MMAs touch disjoint accumulator columns)."""
    for fh in (1, 2, 3, 5):
        for groups in range(1, min(fh, 3) + 1):
            for th in range(2, 14):
                for seed in range(6):
                    state, wrong = simulate(groups, th, fh, 10, seed, (), lambda i, t, f: touched_rows(i, t, f, nhalf),
                                            nhalf=nhalf, blocked=True)
                    assert state == "ok" and not wrong, (nhalf, fh, groups, th, seed, state, wrong[:2])


@pytest.mark.parametrize("nhalf", [2, 3])
def test_protocol_with_two_issuers_per_group(nhalf):
    """Two A slots and two issuer warps per converter group: the second issuer
    skips the rows it does not own, virtual steps entirely, so the issuers of a
    group wait for each other once per step; without that wait a parity wait
    can look at a barrier two completions early (the model must see that too)."""
    for fh in (1, 2, 3, 5):
        for groups in range(1, min(fh, 3) + 1):
            for th in range(2, 12):
                for seed in range(6):
                    virtual = (0, 1, 8, 9) if seed % 2 else (0, 5, 6, 11)
                    state, wrong = simulate(groups, th, fh, 12, seed, virtual,
                                            lambda i, t, f: touched_rows(i, t, f, nhalf), nhalf=nhalf, ipg=2)
                    assert state == "ok" and not wrong, (nhalf, fh, groups, th, seed, state, wrong[:2])
    bad = [simulate(3, 7, 3, 12, seed, (0, 1, 5, 6, 7, 8), lambda i, t, f: touched_rows(i, t, f, 3), nhalf=3, ipg=2,
                    sync=False) for seed in range(30)]
    assert any(state != "ok" or wrong for state, wrong in bad)


@pytest.mark.parametrize("nhalf", [3, 4])
def test_protocol_with_more_epilogue_warps_per_quadrant(nhalf):
    """12 or 16 epilogue warps: every (nhalf)-th row per warp, the issuers wait
    for the top nhalf rows they add into."""
    for fh in (1, 2, 3, 5):
        for groups in range(1, min(fh, 3) + 1):
            for th in range(2, 14):
                for seed in range(6):
                    virtual = (0, 1, 8, 9) if seed % 2 else (0, 5, 9)
                    state, wrong = simulate(groups, th, fh, 10, seed, virtual,
                                            lambda i, t, f: touched_rows(i, t, f, nhalf), nhalf=nhalf)
                    assert state == "ok" and not wrong, (nhalf, fh, groups, th, seed, state, wrong[:2])
    # waiting for two rows only would let an issuer add into a row the third warp has not retired
    bad = [simulate(3, 7, 3, 10, seed, (0, 1, 8, 9), touched_rows, nhalf=nhalf)[1] for seed in range(10)]
    assert any(bad)


def test_waiting_for_a_row_one_does_not_touch_locks_up():
    states = {simulate(3, 7, 3, 12, seed, (0, 1, 10, 11), last_two_rows)[0] for seed in range(20)}
    assert "deadlock" in states


@pytest.mark.parametrize("cg", [3, 4, 8])
def test_multi_group_protocol(cg):
    for th in (2, 3, 7, 12, 24):
        for seed in range(6):
            state, wrong = simulate(3, th, 3, 8, seed, (0, 1, 6, 7), touched_rows, cg=cg)
            assert state == "ok" and not wrong, (cg, th, seed, state, wrong[:2])
