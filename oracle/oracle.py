"""TEST INFRASTRUCTURE ONLY -- the checker, never the product.

CPU oracle for DistConv's spatially-parallel conv + batch-norm path.  Only
``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may
import this module; nothing under ``dihydrogen_b200/`` does.

Arrays are numpy, framework order ``(N, C, [D,] H, W)`` with W fastest, which is
the memory order of the reference's tensors (its dimension 0 is W:
legacy/include/distconv/distconv.hpp:103-109).  ``ref dim i`` therefore maps to
numpy axis ``nd-1-i``.

What is restated, and from where:

* geometry -- block decomposition with the remainder going to the leading
  ranks (legacy/include/distconv/tensor/tensor_mpi.hpp:458-488), rank -> grid
  index with dimension 0 fastest (tensor_mpi.hpp:47-56), per-side halo widths
  (legacy/include/distconv/distconv.hpp:21-99) and the convolution output
  shape (distconv.hpp:135-200, 365-413).  Pinned by ``tests/golden/geom_*.txt``,
  which the reference's own headers printed (``oracle/ref_driver.cpp``).
* halo exchange -- ordered per-dimension exchange, dimension 0 first, each
  slab spanning the halo-extended extent of every other dimension
  (legacy/include/distconv/tensor/halo_exchange_cuda.hpp:56-126, 267-271,
  322-357); which cells a slab covers (halo_cuda.hpp:34-88); pack/unpack and
  the accumulate ops (halo_packing_cuda.hpp:60-167).  Pinned by the known
  answer of legacy/tests/tensor/test_halo_exchange_cuda.cu:52-233 (every halo
  cell inside the global domain equals its global linear offset).
* convolution / batch-norm arithmetic -- ``conv_oracle.c`` (see its header).
* pooling -- the arithmetic lives in cuDNN (cudnnPoolingForward / Backward,
  reached from legacy/include/distconv/dnn_backend/pooling.hpp:212-283; no
  version pinned), restated below from its documented semantics: modes as
  pooling.hpp:27-48 maps them, padding ignored by MAX and counted (or not) by
  the averages, the gradient of a maximum sent to one cell per window.  The
  reference pins the forward pass against another framework
  (legacy/tests/dnn_backend/chainer_pooling.py); ``tests/test_oracle_cpu.py``
  does the same against torch's CPU pooling.
"""
from __future__ import annotations

import ctypes
import itertools
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    """Compile conv_oracle.c into oracle/liboracle.so (gcc, OpenMP)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "conv_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O3", "-march=native", "-fopenmp", "-fPIC", "-shared", "-o", so, src, "-lm"]
        )
    return so


class _TDesc(ctypes.Structure):
    _fields_ = [(k, ctypes.c_int64) for k in ("n", "c", "d", "h", "w", "sn", "sc", "sd", "sh", "sw")]


class _CDesc(ctypes.Structure):
    _fields_ = [
        (k, ctypes.c_int)
        for k in ("fd", "fh", "fw", "pd", "ph", "pw", "sd", "sh", "sw", "dd", "dh", "dw")
    ]


def _lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.oracle_num_threads.restype = ctypes.c_int
    return _LIB


def num_threads() -> int:
    return int(_lib().oracle_num_threads())


def set_num_threads(n: int) -> int:
    """OpenMP thread count of the C loops (a launcher may have exported
    OMP_NUM_THREADS=1); returns the count now in force."""
    _lib().oracle_set_num_threads(ctypes.c_int(int(n)))
    return num_threads()


def host_cores() -> int:
    """Cores this process may run on."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def _as5(a: np.ndarray) -> np.ndarray:
    """View a 4-D (N,C,H,W) array as 5-D (N,C,1,H,W)."""
    assert a.dtype == np.float32
    if a.ndim == 4:
        return a[:, :, None, :, :]
    assert a.ndim == 5
    return a


def _tdesc(a5: np.ndarray) -> _TDesc:
    it = a5.itemsize
    for s in a5.strides:
        assert s % it == 0
    return _TDesc(*[int(v) for v in a5.shape], *[int(s // it) for s in a5.strides])


def _ptr(a: np.ndarray):
    return ctypes.c_void_p(a.__array_interface__["data"][0])


def _cdesc(fshape, pads, strides, dilations) -> _CDesc:
    def t3(v, fill):
        v = list(v)
        return [fill] * (3 - len(v)) + v

    return _CDesc(*t3(fshape, 1), *t3(pads, 0), *t3(strides, 1), *t3(dilations, 1))


def conv_out_extent(i, f, p, s, d=1):
    df = f + (f - 1) * (d - 1)
    return (i + 2 * p - df) // s + 1


def conv_fwd(x, w, pads, strides, dilations=None, alpha=1.0, beta=0.0, y=None):
    """cuDNN-style forward cross-correlation; x may be a strided view."""
    nsd = x.ndim - 2
    dilations = dilations or [1] * nsd
    oshape = [conv_out_extent(x.shape[2 + i], w.shape[2 + i], pads[i], strides[i], dilations[i]) for i in range(nsd)]
    if y is None:
        y = np.zeros((x.shape[0], w.shape[0], *oshape), dtype=np.float32)
    assert list(y.shape[2:]) == oshape, (y.shape, oshape)
    w = np.ascontiguousarray(w, dtype=np.float32)
    x5, y5 = _as5(x), _as5(y)
    xd, yd, cd = _tdesc(x5), _tdesc(y5), _cdesc(w.shape[2:], pads, strides, dilations)
    _lib().oracle_conv_fwd(_ptr(x5), ctypes.byref(xd), _ptr(w), _ptr(y5), ctypes.byref(yd), ctypes.byref(cd),
                           ctypes.c_double(alpha), ctypes.c_double(beta))
    return y


def conv_bwd_data(w, dy, dx, pads, strides, dilations=None, alpha=1.0, beta=0.0):
    """dx (given, possibly a strided view) receives the adjoint w.r.t. x."""
    nsd = dy.ndim - 2
    dilations = dilations or [1] * nsd
    w = np.ascontiguousarray(w, dtype=np.float32)
    x5, y5 = _as5(dx), _as5(dy)
    xd, yd, cd = _tdesc(x5), _tdesc(y5), _cdesc(w.shape[2:], pads, strides, dilations)
    _lib().oracle_conv_bwd_data(_ptr(w), _ptr(y5), ctypes.byref(yd), _ptr(x5), ctypes.byref(xd), ctypes.byref(cd),
                                ctypes.c_double(alpha), ctypes.c_double(beta))
    return dx


def conv_bwd_filter(x, dy, fshape, pads, strides, dilations=None, alpha=1.0, beta=0.0, dw=None):
    nsd = dy.ndim - 2
    dilations = dilations or [1] * nsd
    if dw is None:
        dw = np.zeros((dy.shape[1], x.shape[1], *fshape), dtype=np.float32)
    assert dw.flags["C_CONTIGUOUS"]
    x5, y5 = _as5(x), _as5(dy)
    xd, yd, cd = _tdesc(x5), _tdesc(y5), _cdesc(fshape, pads, strides, dilations)
    _lib().oracle_conv_bwd_filter(_ptr(x5), ctypes.byref(xd), _ptr(y5), ctypes.byref(yd), _ptr(dw), ctypes.byref(cd),
                                  ctypes.c_double(alpha), ctypes.c_double(beta))
    return dw


# --------------------------------------------------------------------------
# pooling
# --------------------------------------------------------------------------

POOL_MODES = ("MAX", "AVERAGE", "AVERAGE_NO_PAD")


def _pool_windows(x5, window, pads, strides):
    """(taps, N, C, oD, oH, oW) stack of the window cells of every output, NaN
    where a cell is padding, and the flat input index of each (-1 = padding)."""
    n, c = x5.shape[:2]
    ext = x5.shape[2:]
    out = [conv_out_extent(e, w, p, s) for e, w, p, s in zip(ext, window, pads, strides)]
    idx = np.arange(int(np.prod(ext))).reshape(ext)
    vals, where = [], []
    grids = np.meshgrid(*[np.arange(o) for o in out], indexing="ij")
    for tap in itertools.product(*[range(w) for w in window]):
        coord = [g * s - p + t for g, s, p, t in zip(grids, strides, pads, tap)]
        ok = np.ones(out, bool)
        for cd, e in zip(coord, ext):
            ok &= (cd >= 0) & (cd < e)
        cl = [np.clip(cd, 0, e - 1) for cd, e in zip(coord, ext)]
        flat = np.where(ok, idx[tuple(cl)], -1)
        v = x5.reshape(n, c, -1)[:, :, np.maximum(flat, 0).ravel()].reshape(n, c, *out).astype(np.float64)
        v[:, :, ~ok] = np.nan
        vals.append(v)
        where.append(flat)
    return np.stack(vals), np.stack(where), out


def _pool_count(where, window, mode):
    if mode == "AVERAGE":
        return float(np.prod(window))
    return np.maximum((where >= 0).sum(axis=0), 1).astype(np.float64)


def pool_fwd(x, window, pads, strides, mode="MAX"):
    """y = pool(x); window / pads / strides per spatial axis, outermost first."""
    assert mode in POOL_MODES
    x5 = _as5(x)
    nsd = x.ndim - 2
    w3, p3, s3 = ([a] * (3 - nsd) + list(v) for a, v in ((1, window), (0, pads), (1, strides)))
    vals, where, out = _pool_windows(x5, w3, p3, s3)
    if mode == "MAX":
        y = np.nanmax(vals, axis=0)
    else:
        y = np.nansum(vals, axis=0) / _pool_count(where, w3, mode)
    return y.astype(np.float32).reshape(x.shape[:2] + tuple(out[3 - nsd:]))


def pool_bwd(x, dy, window, pads, strides, mode="MAX"):
    """dx of pool_fwd, padding cells dropped.  MAX: the whole of dy[o] goes to
    the first cell of o's window (scan order outermost axis first) that holds
    the maximum."""
    assert mode in POOL_MODES
    x5, dy5 = _as5(x), _as5(dy)
    nsd = x.ndim - 2
    w3, p3, s3 = ([a] * (3 - nsd) + list(v) for a, v in ((1, window), (0, pads), (1, strides)))
    vals, where, out = _pool_windows(x5, w3, p3, s3)
    n, c = x5.shape[:2]
    dx = np.zeros((n, c, int(np.prod(x5.shape[2:]))), np.float64)
    g = dy5.astype(np.float64)
    if mode == "MAX":
        first = np.argmax(np.where(np.isnan(vals), -np.inf, vals), axis=0)  # ties: lowest tap index
        for i in range(n):
            for j in range(c):
                tgt = np.take_along_axis(where, first[i, j][None], axis=0)[0]
                np.add.at(dx[i, j], tgt.ravel(), g[i, j].ravel())
    else:
        share = g / _pool_count(where, w3, mode)
        for t in range(where.shape[0]):
            ok = where[t] >= 0
            for i in range(n):
                for j in range(c):
                    np.add.at(dx[i, j], where[t][ok], share[i, j][ok])
    return dx.astype(np.float32).reshape(x.shape)


# --------------------------------------------------------------------------
# batch-norm
# --------------------------------------------------------------------------

def bn_sums(x):
    x5 = _as5(x)
    C = x5.shape[1]
    s = np.zeros(C, np.float64)
    q = np.zeros(C, np.float64)
    xd = _tdesc(x5)
    _lib().oracle_bn_sums(_ptr(x5), ctypes.byref(xd), _ptr(s), _ptr(q))
    return s, q


def bn_sums_to_statistics(sums, sqsums, num_per_sum, decay, running_mean, running_var):
    """Returns (mean, var, running_mean, running_var) as fp32 (batchnorm.cu:297-312)."""
    C = len(sums)
    mean = np.asarray(sums, np.float32).copy()
    var = np.asarray(sqsums, np.float32).copy()
    rm = np.asarray(running_mean, np.float32).copy()
    rv = np.asarray(running_var, np.float32).copy()
    _lib().oracle_bn_sums_to_statistics(ctypes.c_int64(num_per_sum), ctypes.c_float(decay), ctypes.c_int64(C),
                                        _ptr(mean), _ptr(var), _ptr(rm), _ptr(rv))
    return mean, var, rm, rv


def bn_normalize(x, mean, var, scale, bias, eps, y=None):
    if y is None:
        y = np.zeros(x.shape, np.float32)
    x5, y5 = _as5(x), _as5(y)
    xd, yd = _tdesc(x5), _tdesc(y5)
    f = lambda a: np.ascontiguousarray(a, np.float32)
    mean, var, scale, bias = f(mean), f(var), f(scale), f(bias)
    _lib().oracle_bn_normalize(_ptr(x5), ctypes.byref(xd), _ptr(mean), _ptr(var), _ptr(scale), _ptr(bias),
                               ctypes.c_float(eps), _ptr(y5), ctypes.byref(yd))
    return y


def bn_backprop1(x, dy, mean, var, scale, eps):
    x5, y5 = _as5(x), _as5(dy)
    C = x5.shape[1]
    xd, yd = _tdesc(x5), _tdesc(y5)
    f = lambda a: np.ascontiguousarray(a, np.float32)
    mean, var, scale = f(mean), f(var), f(scale)
    out = [np.zeros(C, np.float64) for _ in range(4)]
    _lib().oracle_bn_backprop1(_ptr(x5), ctypes.byref(xd), _ptr(y5), ctypes.byref(yd), _ptr(mean), _ptr(var),
                               _ptr(scale), ctypes.c_float(eps), *[_ptr(o) for o in out])
    return out  # dscale, dbias, dmean, dvar


def bn_backprop2(x, dy, mean, var, scale, dmean, dvar, eps, num_per_sum, dx=None):
    if dx is None:
        dx = np.zeros(x.shape, np.float32)
    x5, y5, d5 = _as5(x), _as5(dy), _as5(dx)
    xd, yd, dd = _tdesc(x5), _tdesc(y5), _tdesc(d5)
    f = lambda a: np.ascontiguousarray(a, np.float32)
    mean, var, scale, dmean, dvar = f(mean), f(var), f(scale), f(dmean), f(dvar)
    _lib().oracle_bn_backprop2(_ptr(x5), ctypes.byref(xd), _ptr(y5), ctypes.byref(yd), _ptr(mean), _ptr(var),
                               _ptr(scale), _ptr(dmean), _ptr(dvar), ctypes.c_float(eps),
                               ctypes.c_int64(num_per_sum), _ptr(d5), ctypes.byref(dd))
    return dx


# --------------------------------------------------------------------------
# geometry (reference dimension order: index 0 = W ... -2 = C, -1 = N)
# --------------------------------------------------------------------------

def rank_to_index(rank, locale_shape):
    """tensor_mpi.hpp:47-56: dimension 0 varies fastest."""
    idx = []
    for n in locale_shape:
        idx.append(rank % n)
        rank //= n
    return idx


def index_to_rank(idx, locale_shape):
    r, m = 0, 1
    for i, n in zip(idx, locale_shape):
        r += i * m
        m *= n
    return r


def split_extent(total, parts, index):
    """tensor_mpi.hpp:458-488 with block size 1: remainder to the leading ranks."""
    base, rem = divmod(total, parts)
    return base + (1 if index < rem else 0)


def split_offset(total, parts, index):
    return sum(split_extent(total, parts, j) for j in range(index))


@dataclass
class Shard:
    """One rank's piece of a block-distributed tensor (reference order W..N)."""
    shape: list          # global shape
    locale: list         # process grid
    overlap: list        # halo width per dim (both sides)
    rank: int
    idx: list = None
    local: list = None
    offset: list = None

    def __post_init__(self):
        self.idx = rank_to_index(self.rank, self.locale)
        if self.local is None:
            self.local = [split_extent(s, p, i) for s, p, i in zip(self.shape, self.locale, self.idx)]
        if self.offset is None:
            self.offset = [split_offset(s, p, i) for s, p, i in zip(self.shape, self.locale, self.idx)]
        self.overlap = [o if p > 1 else 0 for o, p in zip(self.overlap, self.locale)]

    @property
    def nd(self):
        return len(self.shape)

    @property
    def real(self):
        return [l + 2 * o for l, o in zip(self.local, self.overlap)]

    def np_real_shape(self):
        return tuple(reversed(self.real))

    def owned_slices(self):
        """numpy slices selecting the owned cells inside the real buffer."""
        return tuple(slice(o, o + l) for o, l in reversed(list(zip(self.overlap, self.local))))

    def peer(self, dim, side):
        """halo_exchange_cuda.hpp:322-357: +-1 along dim, None at the edge or
        when the neighbour's shard is empty."""
        if self.locale[dim] == 1 or self.overlap[dim] == 0 or min(self.local) == 0:
            return None
        j = self.idx[dim] + (1 if side == 1 else -1)
        if j < 0 or j >= self.locale[dim]:
            return None
        if split_extent(self.shape[dim], self.locale[dim], j) == 0:
            return None
        idx = list(self.idx)
        idx[dim] = j
        return index_to_rank(idx, self.locale)


def get_halo_sizes(shard: Shard, filter_dims, strides, dilations, with_padding):
    """distconv.hpp:21-99.  Returns fwd_send, bwd_send, fwd_recv, bwd_recv."""
    nd = shard.nd
    fs, bs, fr, br = ([0] * nd for _ in range(4))
    for i in range(nd - 2):
        if shard.locale[i] == 1:
            continue
        df = filter_dims[i] + (filter_dims[i] - 1) * (dilations[i] - 1)
        if df % 2 == 0:
            assert strides[i] == df
            continue
        radius = (df - 1) // 2
        s = strides[i]
        off = shard.offset[i]
        if shard.idx[i] == 0:
            if with_padding:
                br[i] = radius
        else:
            x = off - (0 if with_padding else radius)
            br[i] = radius - (s - (x % s)) % s
            bs[i] = radius - (x - 1) % s
        if shard.idx[i] == shard.locale[i] - 1 and not with_padding:
            pass
        else:
            y = off + shard.local[i] - 1 - (0 if with_padding else radius)
            fr[i] = radius - y % s
            fs[i] = radius - (s - ((y + 1) % s)) % s
        fs[i], fr[i], bs[i], br[i] = (max(v, 0) for v in (fs[i], fr[i], bs[i], br[i]))
    return fs, bs, fr, br


def conv_output_local_shape(shard: Shard, filter_dims, strides, dilations, with_padding, K):
    """distconv.hpp:135-200."""
    fs, bs, fr, br = get_halo_sizes(shard, filter_dims, strides, dilations, with_padding)
    out = list(shard.local)
    for i in range(shard.nd - 2):
        df = filter_dims[i] + (filter_dims[i] - 1) * (dilations[i] - 1)
        ext = shard.local[i] + br[i] + fr[i]
        if with_padding and shard.locale[i] == 1:
            ext += df - 1
        out[i] = 0 if ext < df else -(-(ext - df + 1) // strides[i])
    out[-2] = K
    return out


# --------------------------------------------------------------------------
# halo exchange
# --------------------------------------------------------------------------

LHS, RHS = 0, 1


def halo_slab(real_shape, dim, side, width, inner):
    """numpy slices of one slab of a halo-extended buffer whose halo on ``dim``
    is ``width`` cells wide (halo_cuda.hpp:34-88).  real_shape is in reference
    order; the returned slices are in numpy order."""
    nd = len(real_shape)
    n = real_shape[dim]
    if side == RHS:
        start = n - 2 * width if inner else n - width
    else:
        start = width if inner else 0
    sl = [slice(None)] * nd
    sl[nd - 1 - dim] = slice(start, start + width)
    return tuple(sl)


def _accum(dst, src, op):
    if op == "ID":
        dst[...] = src
    elif op == "SUM":
        dst += src
    elif op == "MAX":
        np.maximum(dst, src, out=dst)
    elif op == "MIN":
        np.minimum(dst, src, out=dst)
    else:
        raise ValueError(op)


def clear_halo(shard: Shard, buf: np.ndarray, dim: int):
    """legacy/src/tensor/tensor_mpi_cuda.cu:14-82: zero both outer slabs of dim."""
    w = shard.overlap[dim]
    if w == 0:
        return
    for side in (LHS, RHS):
        buf[halo_slab(shard.real, dim, side, w, inner=False)] = 0


def exchange(shards, bufs, reverse=False, op="ID", dims=None):
    """Ordered halo exchange among all ranks (halo_exchange_cuda.hpp:56-126).

    Forward: pack the inner slab, the neighbour unpacks it into its outer slab.
    Reverse: pack the outer slab, the neighbour accumulates it into its inner
    slab with ``op`` (halo_packing_cuda.hpp:100).
    """
    nd = shards[0].nd
    for dim in (range(nd) if dims is None else dims):
        packed = {}
        for sh, b in zip(shards, bufs):
            w = sh.overlap[dim]
            for side in (LHS, RHS):
                peer = sh.peer(dim, side)
                if peer is None or w == 0:
                    continue
                packed[(peer, 1 - side)] = b[halo_slab(sh.real, dim, side, w, inner=not reverse)].copy()
        for r, (sh, b) in enumerate(zip(shards, bufs)):
            w = sh.overlap[dim]
            for side in (LHS, RHS):
                if (r, side) not in packed:
                    continue
                dst = b[halo_slab(sh.real, dim, side, w, inner=reverse)]
                _accum(dst, packed[(r, side)], "ID" if not reverse else op)


def fill_by_definition(shard: Shard, g: np.ndarray) -> np.ndarray:
    """The halo-extended shard whose every cell (owned or halo) holds the
    global tensor's value at that global index, zero outside the domain: what
    clear_halo + exchange must produce
    (legacy/tests/tensor/test_halo_exchange_cuda.cu:114-170)."""
    nd = shard.nd
    out = np.zeros(shard.np_real_shape(), g.dtype)
    src, dst = [], []
    for ax in range(nd):
        d = nd - 1 - ax
        lo = shard.offset[d] - shard.overlap[d]
        hi = shard.offset[d] + shard.local[d] + shard.overlap[d]
        clo, chi = max(lo, 0), min(hi, shard.shape[d])
        src.append(slice(clo, chi))
        dst.append(slice(clo - lo, chi - lo))
    out[tuple(dst)] = g[tuple(src)]
    return out


def make_shards(shape, locale, overlap):
    n = int(np.prod(locale))
    return [Shard(list(shape), list(locale), list(overlap), r) for r in range(n)]


def scatter(shards, g):
    """Owned cells from the global array, halos zero."""
    bufs = []
    for sh in shards:
        b = np.zeros(sh.np_real_shape(), g.dtype)
        src = tuple(slice(o, o + l) for o, l in reversed(list(zip(sh.offset, sh.local))))
        b[sh.owned_slices()] = g[src]
        bufs.append(b)
    return bufs


def gather(shards, bufs, shape_np):
    g = np.zeros(shape_np, bufs[0].dtype)
    for sh, b in zip(shards, bufs):
        dst = tuple(slice(o, o + l) for o, l in reversed(list(zip(sh.offset, sh.local))))
        g[dst] = b[sh.owned_slices()]
    return g
