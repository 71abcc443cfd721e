"""dcb_bn_stats_noalloc: the allocation-free variant of the batch-norm
statistics kernel, for hosts that cannot let the library call cudaMalloc (a
framework allocator that owns the device, code inside a stream capture, a
latency-bound loop).  Checked through the C ABI against dcb_bn_stats on the
same input, twice in a row because both calls reuse the one fixed scratch
array.  Collected last so that a failure here cannot hide other tests."""
import ctypes

import numpy as np
import pytest
import torch

import dihydrogen_b200 as dc
from dihydrogen_b200 import _abi
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _stats_with_plan(t):
    be = dc.BackendDNNLib(dc.Locale(0, 1))
    bn = dc.BatchNormalization(be, t.nd, 0.9, 1e-5, False)
    C = t.local_shape[-2]
    st = torch.zeros(2 * C, device="cuda")
    bn.forward_stage1(t, st[:C], st[C:], True)
    torch.cuda.synchronize()
    return st.cpu().numpy()


def _stats_noalloc(t):
    C = t.local_shape[-2]
    st = torch.full((2 * C,), float("nan"), device="cuda")
    xd = t.nd_desc()
    _abi.call("dcb_bn_stats_noalloc", ctypes.byref(xd), ctypes.c_void_p(t.get_base_ptr()),
              ctypes.c_void_p(st[:C].data_ptr()), ctypes.c_void_p(st[C:].data_ptr()), None)
    torch.cuda.synchronize()
    return st.cpu().numpy()


@pytest.mark.parametrize("shape,locale,overlap", [
    ([64, 48, 40, 16, 1], [1, 1, 1, 1, 1], [0, 0, 0, 0, 0]),   # dense, float4 path
    ([33, 9, 6, 3, 2], [1, 1, 2, 1, 1], [0, 0, 1, 0, 0]),       # halo in D, scalar path
])
def test_noalloc_matches_planned_stats_twice(shape, locale, overlap):
    rng = np.random.default_rng(0)
    n = int(np.prod(locale))
    t = dc.Tensor(shape, dc.Locale(0, n), dc.Distribution.make_overlapped_distribution(locale, overlap))
    for rep in range(2):  # second call finds the scratch as the first left it
        t.allocate()
        t.buffer.copy_(torch.from_numpy(rng.normal(0.2 * rep, 1.5, t.np_real_shape()).astype(np.float32)))
        ref = _stats_with_plan(t)
        got = _stats_noalloc(t)
        # same kernel, same fixed-order reduction: tolerance of the other BN tests
        assert np.allclose(got, ref, rtol=1e-5, atol=1e-5 * np.abs(ref).max()), (rep, got, ref)
        # and against the CPU restatement of channel_sums_and_sqsums on the owned cells
        s, q = O.bn_sums(np.ascontiguousarray(t.owned().cpu().numpy()))
        want = np.concatenate([s, q])
        assert np.allclose(got, want, rtol=1e-5, atol=1e-5 * np.abs(want).max()), (rep, got, want)


def test_noalloc_rejects_too_many_channels():
    xd = _abi.NdDesc()
    xd.nsd, xd.n, xd.c = 2, 1, 2000
    xd.dims[0], xd.dims[1], xd.dims[2] = 1, 2, 4
    xd.sn, xd.sc = 2000 * 8, 8
    xd.strides[0], xd.strides[1], xd.strides[2] = 8, 4, 1
    buf = torch.zeros(2000 * 8, device="cuda")
    out = torch.zeros(4000, device="cuda")
    st = _abi.lib().dcb_bn_stats_noalloc(ctypes.byref(xd), ctypes.c_void_p(buf.data_ptr()),
                                         ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(out[2000:].data_ptr()), None)
    assert st == _abi.UNSUPPORTED
    assert b"1024" in _abi.lib().dcb_last_error()
