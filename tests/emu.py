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


def scatter_owned_into(t: dc.Tensor, g: np.ndarray):
    """Fill the owned cells of an allocated t from the global array g."""
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


def check_stages(K, gx, w, scale, bias, pads, strides, y, mean, var, z, bwd=None, tol=1e-5, what=""):
    """Every stage of a conv + batch-norm layer against the oracle FED WITH THE
    GPU'S OWN PREVIOUS STAGE, each at the 1e-5 contract (the reference's own
    criterion is 1.5e-5, legacy/tests/dnn_backend/test_cudnn_util.sh.in:50-86):
    rounding does not compound from stage to stage, so no bound needs widening.
    Arguments are global numpy arrays gathered from the ranks; ``bwd`` holds
    gdz, dscale, dbias, dmean, dvar, dy, dw, dx of the backward pass."""
    from oracle import oracle as O

    assert_close(y, O.conv_fwd(gx, w, pads, strides), tol, what + "conv output")
    s, q = O.bn_sums(y)
    nps = y.size // K
    m, v, _, _ = O.bn_sums_to_statistics(s, q, nps, 0.9, np.zeros(K), np.ones(K))
    assert_close(mean, m, tol, what + "mean")
    assert_close(var, v, tol, what + "var")
    assert_close(z, O.bn_normalize(y, mean, var, scale, bias, 1e-5), tol, what + "bn output")
    if bwd is None:
        return
    gdz = bwd["gdz"]
    dsc, dbi, dme, dva = O.bn_backprop1(y, gdz, mean, var, scale, 1e-5)
    assert_close(bwd["dscale"], dsc, tol, what + "dscale")
    assert_close(bwd["dbias"], dbi, tol, what + "dbias")
    assert_close(bwd["dmean"], dme, tol, what + "dmean")
    assert_close(bwd["dvar"], dva, tol, what + "dvar")
    dy = bwd["dy"]
    assert_close(dy, O.bn_backprop2(y, gdz, mean, var, scale, bwd["dmean"], bwd["dvar"], 1e-5, nps), tol,
                 what + "bn dx")
    assert_close(bwd["dw"], O.conv_bwd_filter(gx, dy, w.shape[2:], pads, strides), tol, what + "filter gradient")
    dx = np.zeros_like(gx)
    O.conv_bwd_data(w, dy, dx, pads, strides)
    assert_close(bwd["dx"], dx, tol, what + "input gradient")
