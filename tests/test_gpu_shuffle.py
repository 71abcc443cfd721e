"""Re-distribution between two block decompositions on emulated ranks: every
cell ends up with its owner in the other distribution (bit-exact), halo cells
of the destination are left alone, and the way back restores the source."""
import numpy as np
import pytest
import torch

import dihydrogen_b200 as dc
from dihydrogen_b200 import _abi

import emu

pytestmark = pytest.mark.gpu

# global shape (W, H, [D,] C, N), source grid, destination grid, destination overlap
CASES = [
    ([12, 10, 8, 3, 4], [1, 1, 1, 1, 4], [1, 1, 4, 1, 1], [0, 0, 1, 0, 0]),   # sample-parallel -> D-partitioned with halo
    ([12, 10, 8, 3, 4], [2, 2, 1, 1, 1], [1, 1, 2, 1, 2], [0, 0, 1, 0, 0]),   # 2x2 in W, H -> D x N
    ([20, 9, 2, 6], [1, 3, 1, 2], [2, 1, 1, 3], [1, 0, 0, 0]),                # 4-D, ragged splits, 6 ranks
    ([16, 8, 8, 2, 1], [1, 1, 1, 1, 1], [1, 1, 1, 1, 1], [0, 0, 0, 0, 0]),    # one rank: a local copy
    ([7, 5, 3, 2, 2], [1, 1, 3, 1, 1], [1, 1, 3, 1, 1], [0, 0, 1, 0, 0]),     # same split, only the halo differs
]


def _tensor(shape, grid, overlap, loc):
    return dc.Tensor(shape, loc, dc.Distribution.make_overlapped_distribution(grid, overlap))


@pytest.mark.parametrize("shape,sgrid,dgrid,dov", CASES)
def test_forward_and_backward(shape, sgrid, dgrid, dov):
    n = int(np.prod(sgrid))
    assert n == int(np.prod(dgrid))
    rng = np.random.default_rng(1)
    g = rng.normal(size=tuple(reversed(shape))).astype(np.float32)
    srcs, dsts, backs, shufflers = [], [], [], []
    for loc in emu.locales(n):
        s = _tensor(shape, sgrid, [0] * len(shape), loc)
        d = _tensor(shape, dgrid, dov, loc)
        b = _tensor(shape, sgrid, [0] * len(shape), loc)
        emu.scatter_owned(s, g)
        d.allocate()
        d.buffer.fill_(-7.0)
        b.allocate()
        srcs.append(s), dsts.append(d), backs.append(b)
        shufflers.append(dc.TensorShuffler(s, d, connect=False))
    for which in ("fwd", "bwd"):
        blobs = [sh.export(which) for sh in shufflers]
        for sh in shufflers:
            sh.connect(which, blobs)
    for rep in range(3):  # the receive windows alternate: run through both halves
        for sh, s in zip(shufflers, srcs):
            sh.put("fwd", s.get_buffer())
        for sh, d in zip(shufflers, dsts):
            sh.wait_unpack("fwd", d.get_buffer())
    torch.cuda.synchronize()
    assert np.array_equal(emu.gather_owned(dsts, g.shape), g)
    for d in dsts:  # halo cells untouched
        own = torch.zeros_like(d.buffer, dtype=torch.bool)
        own[tuple(slice(o, o + l) for o, l in reversed(list(zip(d.dist.overlap, d.local_shape))))] = True
        assert bool((d.buffer[~own] == -7.0).all())
    for sh, d in zip(shufflers, dsts):
        sh.put("bwd", d.get_buffer())
    for sh, b in zip(shufflers, backs):
        sh.wait_unpack("bwd", b.get_buffer())
    torch.cuda.synchronize()
    assert np.array_equal(emu.gather_owned(backs, g.shape), g)
    assert all(sh.status("fwd") == _abi.OK and sh.status("bwd") == _abi.OK for sh in shufflers)


def test_wait_expires_with_status_when_a_sender_never_comes():
    """A rank whose peer never puts gets DCB_PEER_TIMEOUT from the bounded wait,
    not a hang, and the destination stays as it was."""
    shape, n = [8, 6, 4, 2, 2], 2
    srcs, dsts, shufflers = [], [], []
    for loc in emu.locales(n):
        s = _tensor(shape, [1, 1, 1, 1, 2], [0] * 5, loc)
        d = _tensor(shape, [1, 1, 2, 1, 1], [0] * 5, loc)
        s.allocate(), d.allocate()
        srcs.append(s), dsts.append(d)
        shufflers.append(dc.TensorShuffler(s, d, connect=False))
    blobs = [sh.export("fwd") for sh in shufflers]
    for sh in shufflers:
        sh.connect("fwd", blobs)
    assert _abi.lib().dcb_set_wait_budget_ns(20_000_000) == _abi.OK
    try:
        shufflers[0].put("fwd", srcs[0].get_buffer())  # rank 1 never puts
        dsts[0].buffer.fill_(3.0)
        shufflers[0].wait_unpack("fwd", dsts[0].get_buffer())
        assert shufflers[0].status("fwd") == _abi.PEER_TIMEOUT
        assert bool((dsts[0].buffer == 3.0).all())
    finally:
        _abi.lib().dcb_set_wait_budget_ns(2_000_000_000)
