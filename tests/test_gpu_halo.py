"""Halo kernels and the peer-store transport against the oracle, bit-exact.
Ranks are emulated on one device (tests/emu.py); every call goes through the
C ABI."""
import ctypes

import numpy as np
import pytest
import torch

import dihydrogen_b200 as dc
from dihydrogen_b200 import _abi
from oracle import oracle as O

import emu

pytestmark = pytest.mark.gpu

CASES = [
    ([8, 9, 3, 2], [1, 2, 1, 1], [0, 1, 0, 0]),
    ([8, 9, 3, 2], [2, 2, 1, 1], [1, 1, 0, 0]),
    ([11, 9, 2, 2], [3, 2, 1, 1], [2, 2, 0, 0]),
    ([16, 12, 4, 2], [2, 2, 1, 1], [4, 2, 0, 0]),
    ([7, 8, 9, 2, 1], [1, 1, 2, 1, 1], [0, 0, 1, 0, 0]),
    ([9, 8, 7, 2, 1], [2, 2, 2, 1, 1], [1, 2, 1, 0, 0]),
    ([9, 8, 13, 2, 2], [1, 2, 4, 1, 1], [0, 1, 3, 0, 0]),
    ([64, 32, 16, 3, 1], [2, 2, 2, 1, 1], [2, 2, 2, 0, 0]),   # 16-byte aligned rows
    ([256, 64, 8, 4, 1], [1, 1, 4, 1, 1], [0, 0, 1, 0, 0]),   # long runs, float4 path
    ([130, 36, 12, 2, 1], [1, 2, 2, 1, 1], [0, 3, 1, 0, 0]),  # float2 path
    ([12, 10, 5, 2, 1], [3, 1, 1, 1, 1], [1, 0, 0, 0, 0]),    # 5-D W faces (unimplemented upstream)
]


def make_ranks(shape, locale, overlap):
    n = int(np.prod(locale))
    ts = [dc.Tensor(shape, l, dc.Distribution.make_overlapped_distribution(locale, overlap)) for l in emu.locales(n)]
    return ts


@pytest.mark.parametrize("shape,locale,overlap", CASES)
def test_exchange_known_answer(shape, locale, overlap):
    g = np.arange(int(np.prod(shape)), dtype=np.float32).reshape(tuple(reversed(shape)))
    ts = make_ranks(shape, locale, overlap)
    for t in ts:
        t.allocate()
        t.buffer.fill_(-7.0)  # stale halo contents must not survive
        src = tuple(slice(o, o + l) for o, l in reversed(list(zip(t.offset, t.local_shape))))
        t.owned().copy_(torch.from_numpy(np.ascontiguousarray(g[src])))
        for d in range(t.nd - 2):
            t.clear_halo(d)
    hxs = [dc.HaloExchange(t) for t in ts]
    emu.connect_halo(hxs)
    emu.exchange_all(hxs)
    torch.cuda.synchronize()
    shards = O.make_shards(shape, locale, overlap)
    for t, sh, hx in zip(ts, shards, hxs):
        assert hx.status() == _abi.OK
        assert t.get_local_real_shape() == sh.real
        assert np.array_equal(t.buffer.cpu().numpy(), O.fill_by_definition(sh, g)), f"rank {sh.rank}"


@pytest.mark.parametrize("shape,locale,overlap", CASES)
def test_exchange_that_clears_the_boundary_slabs_itself(shape, locale, overlap):
    """DCB_HALO_CLEAR_BOUNDARY: no clear_halo pass before the exchange; the launch
    that packs a dimension zeroes that dimension's halo slabs at the boundary of
    the global tensor.  Same known answer, from buffers full of stale values,
    three exchanges in a row (the double-buffered slabs come round)."""
    ts = make_ranks(shape, locale, overlap)
    hxs = None
    shards = O.make_shards(shape, locale, overlap)
    for rep in range(3):
        g = (np.arange(int(np.prod(shape)), dtype=np.float32) * (rep + 1)).reshape(tuple(reversed(shape)))
        for t in ts:
            if t.buffer is None:
                t.allocate()
            t.buffer.fill_(float("nan"))
            src = tuple(slice(o, o + l) for o, l in reversed(list(zip(t.offset, t.local_shape))))
            t.owned().copy_(torch.from_numpy(np.ascontiguousarray(g[src])))
        if hxs is None:
            hxs = [dc.HaloExchange(t) for t in ts]
            emu.connect_halo(hxs)
        for dim in range(len(shape) - 2):
            for h in hxs:
                h.pack_put(dim, clear_boundary=True)
            for h in hxs:
                h.wait_unpack(dim)
        torch.cuda.synchronize()
        for t, sh, hx in zip(ts, shards, hxs):
            assert hx.status() == _abi.OK
            assert np.array_equal(t.buffer.cpu().numpy(), O.fill_by_definition(sh, g)), f"rank {sh.rank} rep {rep}"


@pytest.mark.parametrize("shape,locale,overlap", CASES[:8])
@pytest.mark.parametrize("op", ["SUM", "MAX", "MIN", "ID"])
def test_reverse_exchange_matches_oracle(shape, locale, overlap, op):
    rng = np.random.default_rng(1)
    ts = make_ranks(shape, locale, overlap)
    shards = O.make_shards(shape, locale, overlap)
    bufs = []
    for t, sh in zip(ts, shards):
        b = rng.integers(-50, 50, sh.np_real_shape()).astype(np.float32)
        bufs.append(b)
        emu.upload(t, b)
    hxs = [dc.HaloExchange(t) for t in ts]
    emu.connect_halo(hxs)
    emu.exchange_all(hxs, is_reverse=True, op=op)
    torch.cuda.synchronize()
    O.exchange(shards, bufs, reverse=True, op=op)
    for t, b in zip(ts, bufs):
        assert np.array_equal(t.buffer.cpu().numpy(), b)


def test_repeated_exchanges_alternate_buffers():
    """Three exchanges in a row on one plan (double-buffered slabs, epoch flags)."""
    shape, locale, overlap = [16, 12, 4, 2], [2, 2, 1, 1], [1, 1, 0, 0]
    ts = make_ranks(shape, locale, overlap)
    shards = O.make_shards(shape, locale, overlap)
    hxs = None
    for it in range(3):
        g = (np.arange(int(np.prod(shape)), dtype=np.float32) * (it + 1)).reshape(tuple(reversed(shape)))
        for t in ts:
            if t.buffer is None:
                t.allocate()
            t.buffer.zero_()
            src = tuple(slice(o, o + l) for o, l in reversed(list(zip(t.offset, t.local_shape))))
            t.owned().copy_(torch.from_numpy(np.ascontiguousarray(g[src])))
        if hxs is None:
            hxs = [dc.HaloExchange(t) for t in ts]
            emu.connect_halo(hxs)
        emu.exchange_all(hxs)
        torch.cuda.synchronize()
        for t, sh in zip(ts, shards):
            assert np.array_equal(t.buffer.cpu().numpy(), O.fill_by_definition(sh, g))


@pytest.mark.parametrize("shape,overlap", [([8, 9, 3, 2], [1, 2, 0, 0]), ([16, 8, 6, 2, 1], [4, 1, 2, 0, 0])])
def test_clear_halo(shape, overlap):
    """legacy/tests/tensor/test_tensor_mpi_cuda.cu:163-262: fill with 1, clear
    dim i, outer cells of dim i are 0 and everything else is still 1."""
    locale = [2 if o else 1 for o in overlap]
    t = make_ranks(shape, locale, overlap)[0]
    sh = O.make_shards(shape, locale, overlap)[0]
    for dim in range(len(shape) - 2):
        t.allocate()
        t.buffer.fill_(1.0)
        t.clear_halo(dim)
        ref = np.ones(sh.np_real_shape(), np.float32)
        O.clear_halo(sh, ref, dim)
        assert np.array_equal(t.buffer.cpu().numpy(), ref)
    t.buffer.fill_(1.0)
    d = t.desc()
    _abi.call("dcb_clear_halo", ctypes.byref(d), ctypes.c_void_p(t.get_buffer()), -1, None)
    ref = np.ones(sh.np_real_shape(), np.float32)
    for dim in range(len(shape) - 2):
        O.clear_halo(sh, ref, dim)
    assert np.array_equal(t.buffer.cpu().numpy(), ref)


@pytest.mark.parametrize("pitched", [False, True])
@pytest.mark.parametrize("width", [1, 2, 3])
@pytest.mark.parametrize("dim", [0, 1, 2])
def test_pack_unpack_slab(dim, width, pitched):
    """TraverseHalo + PackFunctor (halo_packing_cuda.hpp:85-167) for every
    side, inner/outer, widths up to the overlap.  Dense rows: the packed
    buffer is the slab in memory order.  Padded rows (the default layout of a
    shard with a W halo: 12 cells one float into a pitch of 16): H and D slabs
    carry the padding between their rows, so the packed buffer is checked by
    unpacking it into a second shard."""
    shape, locale, overlap = [12, 10, 14, 2, 1], [2, 2, 2, 1, 1], [3, 3, 3, 0, 0]
    dist = dc.Distribution.make_overlapped_distribution(locale, overlap)
    t, t2 = (dc.Tensor(shape, emu.locales(8)[0], dist, pitch_align=None if pitched else 1) for _ in range(2))
    assert (t.get_pitch(), t.lead) == ((16, 1) if pitched else (12, 0))
    real = t.get_local_real_shape()
    rng = np.random.default_rng(dim * 10 + width)
    src = rng.normal(size=tuple(reversed(real))).astype(np.float32)
    emu.upload(t, src)
    t2.allocate()
    d = t.desc()
    nd, ov, n = 5, 3, real[dim]
    for side in (0, 1):
        for inner in (0, 1):
            if side == 1:
                start = n - ov - width if inner else n - ov
            else:
                start = ov if inner else ov - width
            sl = [slice(None)] * nd
            sl[nd - 1 - dim] = slice(start, start + width)
            sl = tuple(sl)
            packed = torch.zeros(t._storage[sl].numel(), dtype=torch.float32, device="cuda")
            _abi.call("dcb_halo_pack", ctypes.byref(d), ctypes.c_void_p(t.get_buffer()), dim, side, width, inner,
                      ctypes.c_void_p(packed.data_ptr()), None)
            if not pitched:
                assert np.array_equal(packed.cpu().numpy(), src[sl].ravel())
            t2._storage.zero_()
            _abi.call("dcb_halo_unpack_slab", ctypes.byref(d), ctypes.c_void_p(t2.get_buffer()), dim, side, width,
                      inner, ctypes.c_void_p(packed.data_ptr()), _abi.HALO_OPS["ID"], None)
            ref = np.zeros_like(src)
            ref[sl] = src[sl]
            assert np.array_equal(t2.buffer.cpu().numpy(), ref)
            # unpack with SUM doubles the slab
            _abi.call("dcb_halo_unpack_slab", ctypes.byref(d), ctypes.c_void_p(t.get_buffer()), dim, side, width,
                      inner, ctypes.c_void_p(packed.data_ptr()), _abi.HALO_OPS["SUM"], None)
            ref = src.copy()
            ref[sl] *= 2
            assert np.array_equal(t.buffer.cpu().numpy(), ref)
            emu.upload(t, src)


def test_wait_budget_expires_with_status_not_hang():
    """A flag nobody sets: the unpack kernel gives up after its budget, records
    DCB_PEER_TIMEOUT and the context stays usable."""
    shape, locale, overlap = [8, 8, 2, 1], [1, 2, 1, 1], [0, 1, 0, 0]
    ts = make_ranks(shape, locale, overlap)
    for t in ts:
        t.allocate()
    hxs = [dc.HaloExchange(t) for t in ts]
    emu.connect_halo(hxs)
    assert _abi.lib().dcb_set_wait_budget_ns(5_000_000) == _abi.OK
    try:
        hxs[0].pack_put(1)      # rank 0 sends; rank 1 never does
        hxs[0].wait_unpack(1)   # waits for rank 1's slab: must time out
        assert hxs[0].status() == _abi.PEER_TIMEOUT
        assert hxs[0].status() == _abi.OK  # record cleared
        x = torch.ones(4, device="cuda")
        assert float(x.sum()) == 4.0       # context still alive
    finally:
        _abi.lib().dcb_set_wait_budget_ns(2_000_000_000)


def test_unconnected_plan_is_refused():
    shape, locale, overlap = [8, 8, 2, 1], [1, 2, 1, 1], [0, 1, 0, 0]
    t = make_ranks(shape, locale, overlap)[0]
    t.allocate()
    hx = dc.HaloExchange(t)
    with pytest.raises(_abi.DcbError) as e:
        hx.exchange()
    assert e.value.status == _abi.NOT_CONNECTED


def test_peer_allreduce_emulated():
    """tensor::Allreduce known answer (legacy/tests/tensor/test_allreduce_cuda.cu):
    buf[i] = i + rank; every rank ends with n*i + n(n-1)/2, identical bits."""
    n, count = 4, 1000
    bes = emu.make_backends(n, max_count=1024)
    for rep in range(3):
        ts = [torch.arange(count, dtype=torch.float32, device="cuda") + r + rep for r in range(n)]
        emu.allreduce_all(bes, ts)
        torch.cuda.synchronize()
        expect = n * (np.arange(count, dtype=np.float32) + rep) + n * (n - 1) / 2
        for b, t in zip(bes, ts):
            assert b.allreducer.status() == _abi.OK
            assert np.array_equal(t.cpu().numpy(), expect)


def test_peer_allreduce_takes_vectors_longer_than_its_slots():
    """A filter gradient (K*C*taps floats) can exceed the communicator's
    max_count; dcb_allreduce_sum then goes through in max_count-sized pieces,
    one epoch each.  One rank here (kernels of several ranks that wait for one
    another must not share a GPU); tests/mp_worker.py runs it across processes."""
    be = emu.make_backends(1, max_count=256)[0]
    count = 3 * 256 + 5
    for rep in range(3):
        t = torch.arange(count, dtype=torch.float32, device="cuda") * (rep + 1)
        be.allreducer.allreduce(t.data_ptr(), t.numel())
        torch.cuda.synchronize()
        assert be.allreducer.status() == _abi.OK
        assert np.array_equal(t.cpu().numpy(), np.arange(count, dtype=np.float32) * (rep + 1))
    with pytest.raises(_abi.DcbError):  # the emulation halves keep the limit
        be.allreducer.push(t.data_ptr(), count)
