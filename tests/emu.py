"""Several DistConv ranks emulated inside one process on one GPU.

Kernels that wait on a peer must never be launched before the kernel they wait
for when both run on the same device, so the emulation is phase-ordered: all
ranks pack+put a dimension, then all ranks wait+unpack it; all ranks push
their all-reduce contribution, then all pull.  With this order every wait is
already satisfied when its kernel starts.
"""
import numpy as np
import torch

import dihydrogen_b200 as dc


def locales(n):
    return [dc.Locale(r, n) for r in range(n)]


def connect_halo(hxs):
    blobs = [h.export() for h in hxs]
    for h in hxs:
        h.connect(blobs)


def exchange_all(hxs, is_reverse=False, op="ID"):
    nsd = hxs[0].tensor.nd - 2
    for dim in range(nsd):
        for h in hxs:
            h.pack_put(dim, is_reverse=is_reverse, op=op)
        for h in hxs:
            h.wait_unpack(dim, is_reverse=is_reverse, op=op)


def make_backends(n, max_count=32768, options=None):
    bes = [dc.BackendDNNLib(l, options=options, allreduce="peer", allreduce_max_count=max_count, connect=False)
           for l in locales(n)]
    blobs = [b.allreducer.export() for b in bes]
    for b in bes:
        b.allreducer.connect(blobs)
    return bes


def allreduce_all(bes, tensors):
    for b, t in zip(bes, tensors):
        b.allreducer.push(t.data_ptr(), t.numel())
    for b, t in zip(bes, tensors):
        b.allreducer.pull(t.data_ptr(), t.numel())


def upload(t: dc.Tensor, arr: np.ndarray):
    t.allocate()
    t.buffer.copy_(torch.from_numpy(np.ascontiguousarray(arr)))


def scatter_owned(t: dc.Tensor, g: np.ndarray):
    """Allocate t and fill its owned cells from the global array g."""
    t.allocate()
    src = tuple(slice(o, o + l) for o, l in reversed(list(zip(t.offset, t.local_shape))))
    t.owned().copy_(torch.from_numpy(np.ascontiguousarray(g[src])))


def gather_owned(ts, shape_np):
    g = np.zeros(shape_np, np.float32)
    for t in ts:
        dst = tuple(slice(o, o + l) for o, l in reversed(list(zip(t.offset, t.local_shape))))
        g[dst] = t.owned().cpu().numpy()
    return g


def assert_close(got, ref, tol=1e-5, what=""):
    """Element-wise |got-ref| <= tol * (|ref| + rms(ref)): relative error with
    the tensor's RMS as the floor for cancelling sums."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    rms = np.sqrt(np.mean(ref * ref)) if ref.size else 0.0
    err = np.abs(got - ref)
    bound = tol * (np.abs(ref) + rms) + 1e-30
    worst = (err / bound).max() if ref.size else 0.0
    assert worst <= 1.0, f"{what}: worst error {worst:.3g}x the {tol:g} bound (max abs err {err.max():.3g}, rms {rms:.3g})"
