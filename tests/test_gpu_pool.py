"""Pooling kernels against the oracle, through the C ABI and through the
Pooling operator on emulated ranks (halo exchange forward, reverse exchange
with SUM backward)."""
import ctypes

import numpy as np
import pytest
import torch

import dihydrogen_b200 as dc
from dihydrogen_b200 import _abi
from oracle import oracle as O

import emu
from test_gpu_conv import _nd

pytestmark = pytest.mark.gpu

MODES = list(_abi.POOL_MODES)

# N, C, spatial extents, window, pads, strides
CASES = [
    (2, 3, (7, 9, 11), (3, 3, 3), (1, 1, 1), (2, 2, 2)),
    (1, 2, (8, 10), (2, 2), (0, 0), (2, 2)),
    (2, 2, (6, 7, 8), (3, 3, 3), (1, 1, 1), (1, 1, 1)),
    (1, 2, (9, 300), (3, 3), (0, 0), (1, 1)),
    (1, 1, (4, 6, 520), (2, 2, 2), (0, 0, 0), (2, 2, 2)),
    (1, 2, (11, 13), (5, 5), (2, 2), (3, 3)),
    # long rows of window 3 / stride 2 / pad 1: the four-cells-per-thread backward pass over several warps
    (1, 2, (5, 6, 260), (3, 3, 3), (1, 1, 1), (2, 2, 2)),
    (1, 2, (9, 64), (3, 3), (1, 1), (2, 2)),
    (1, 1, (4, 5, 131), (3, 3, 3), (0, 1, 1), (2, 2, 2)),
    # even extents everywhere: every thread of the 2 x 2-rows backward pass owns a whole block
    (1, 2, (6, 8, 72), (3, 3, 3), (1, 1, 1), (2, 2, 2)),
]


def _pd(window, pads, strides, mode):
    nsd = len(window)
    pd = _abi.PoolDesc()
    pd.nsd, pd.mode = nsd, _abi.POOL_MODES[mode]
    for i in range(3):
        pd.window[i], pd.pads[i], pd.strides[i] = 1, 0, 1
    for i in range(nsd):
        pd.window[3 - nsd + i], pd.pads[3 - nsd + i], pd.strides[3 - nsd + i] = window[i], pads[i], strides[i]
    return pd


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("case", CASES)
def test_kernels_against_oracle(case, mode):
    N, C, sp, window, pads, strides = case
    rng = np.random.default_rng(3)
    # small integers: ties inside windows, so that "first maximum" matters
    x = rng.integers(-4, 5, size=(N, C, *sp)).astype(np.float32)
    y_ref = O.pool_fwd(x, window, pads, strides, mode)
    dy = rng.normal(size=y_ref.shape).astype(np.float32)
    dx_ref = O.pool_bwd(x, dy, window, pads, strides, mode)
    xs, dys = torch.from_numpy(x).cuda(), torch.from_numpy(dy).cuda()
    y0 = rng.normal(size=y_ref.shape).astype(np.float32)
    dx0 = rng.normal(size=x.shape).astype(np.float32)
    y, dx = torch.zeros_like(dys), torch.zeros_like(xs)
    pd, xd, yd = _pd(window, pads, strides, mode), _nd(xs), _nd(y)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    _abi.call("dcb_pool_fwd", ctypes.byref(pd), ctypes.byref(xd), ctypes.byref(yd), 1.0, P(xs), 0.0, P(y), None)
    _abi.call("dcb_pool_bwd", ctypes.byref(pd), ctypes.byref(xd), ctypes.byref(yd), 1.0, P(y), P(dys), P(xs), 0.0,
              P(dx), None, 0, None)
    torch.cuda.synchronize()
    emu.assert_close(y.cpu().numpy(), y_ref, 1e-6, "y")
    emu.assert_close(dx.cpu().numpy(), dx_ref, 2e-6, "dx")
    # with the index workspace: the same gradient, bit for bit
    need = _abi.lib().dcb_pool_bwd_workspace_bytes(ctypes.byref(pd), ctypes.byref(xd), ctypes.byref(yd))
    assert need == (y.numel() if mode == "MAX" else 0)
    if need:
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        dx2 = torch.full_like(xs, 9.0)
        _abi.call("dcb_pool_bwd", ctypes.byref(pd), ctypes.byref(xd), ctypes.byref(yd), 1.0, P(y), P(dys), P(xs), 0.0,
                  P(dx2), P(ws), need, None)
        torch.cuda.synchronize()
        assert torch.equal(dx2, dx)
    # alpha / beta
    yb, dxb = torch.from_numpy(y0).cuda(), torch.from_numpy(dx0).cuda()
    _abi.call("dcb_pool_fwd", ctypes.byref(pd), ctypes.byref(xd), ctypes.byref(yd), 0.5, P(xs), 2.0, P(yb), None)
    _abi.call("dcb_pool_bwd", ctypes.byref(pd), ctypes.byref(xd), ctypes.byref(yd), 0.5, P(y), P(dys), P(xs), -1.0,
              P(dxb), None, 0, None)
    torch.cuda.synchronize()
    emu.assert_close(yb.cpu().numpy(), 0.5 * y_ref + 2.0 * y0, 2e-6, "y blend")
    emu.assert_close(dxb.cpu().numpy(), 0.5 * dx_ref - dx0, 4e-6, "dx blend")


def test_rejects_mismatched_output_extent():
    x = torch.zeros(1, 1, 8, 8, device="cuda")
    y = torch.zeros(1, 1, 5, 4, device="cuda")
    pd, xd, yd = _pd((2, 2), (0, 0), (2, 2), "MAX"), _nd(x), _nd(y)
    st = _abi.lib().dcb_pool_fwd(ctypes.byref(pd), ctypes.byref(xd), ctypes.byref(yd), 1.0,
                                 ctypes.c_void_p(x.data_ptr()), 0.0, ctypes.c_void_p(y.data_ptr()), None)
    assert st == _abi.BAD_ARG


# global shape (W, H, [D,] C, N), locale, window, pad, stride
PARTITIONED = [
    ([20, 16, 12, 3, 2], [1, 1, 4, 1, 1], 3, 1, 1),
    ([16, 16, 16, 2, 1], [2, 2, 2, 1, 1], 3, 1, 2),
    ([24, 20, 3, 2], [2, 2, 1, 1], 3, 1, 1),
    ([16, 12, 8, 2, 1], [1, 2, 2, 1, 1], 2, 0, 2),
    ([18, 14, 10, 2, 1], [1, 2, 2, 1, 1], 3, 0, 1),
]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("shape,locale,window,pad,stride", PARTITIONED)
def test_partitioned_pooling_matches_single_domain(shape, locale, window, pad, stride, mode):
    nd = len(shape)
    nsd = nd - 2
    n = int(np.prod(locale))
    bes = emu.make_backends(n)
    win, pads, strides = [window] * nsd, [pad] * nsd, [stride] * nsd
    rng = np.random.default_rng(5)
    gx = rng.integers(-4, 5, size=tuple(reversed(shape))).astype(np.float32)
    y_ref = O.pool_fwd(gx, win, pads, strides, mode)
    gdy = rng.normal(size=y_ref.shape).astype(np.float32)
    dx_ref = O.pool_bwd(gx, gdy, win, pads, strides, mode)
    xs, ys, dxs, dys, pools = [], [], [], [], []
    for be in bes:
        x = dc.create_input_tensor(shape, locale, win, strides, [1] * nsd, be.locale)
        y = dc.create_pooling_output_tensor(x, win, strides, pads)
        dx = dc.create_d_input_tensor(x)
        dy = dc.create_pooling_d_output_tensor(y)
        for t in (x, y, dx, dy):
            t.allocate()
        emu.scatter_owned(x, gx)
        own = x.owned().clone()
        x.buffer.fill_(float("nan"))  # halos must be produced by the exchange
        x.owned().copy_(own)
        dx.buffer.fill_(float("nan"))  # and every cell of dx by the backward pass
        emu.scatter_owned(dy, gdy)
        pool = dc.Pooling(be, nd)
        pool.setup(x, y, dx, dy, win, pads, strides, mode, connect=False)
        xs.append(x), ys.append(y), dxs.append(dx), dys.append(dy), pools.append(pool)
    assert list(ys[0].shape) == list(reversed(y_ref.shape))
    emu.connect_halo([p.halo_xch_input for p in pools])
    emu.connect_halo([p.halo_xch_d_input for p in pools])
    for x in xs:
        for d in range(nsd):
            x.clear_halo(d)
    emu.exchange_all([p.halo_xch_input for p in pools])
    for p, x, y in zip(pools, xs, ys):
        p.forward(1.0, x, 0.0, y, skip_halo_exchange=True)
    for p, x, y, dx, dy in zip(pools, xs, ys, dxs, dys):
        p.backward(1.0, y, dy, x, 0.0, dx, skip_halo_exchange=True)
    emu.exchange_all([p.halo_xch_d_input for p in pools], is_reverse=True, op="SUM")
    torch.cuda.synchronize()
    emu.assert_close(emu.gather_owned(ys, y_ref.shape), y_ref, 1e-6, "y")
    emu.assert_close(emu.gather_owned(dxs, gx.shape), dx_ref, 4e-6, "dx")
