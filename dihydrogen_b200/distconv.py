"""Host-side mirror of DistConv's operator interface for the spatially-parallel
conv + batch-norm path, driving libdistconv_b200 through its C ABI.

Names, argument meaning and return conventions follow the reference:

* ``Distribution``      legacy/include/distconv/tensor/distribution.hpp:14-270
* ``Locale``            tensor::LocaleMPI, tensor_mpi.hpp:18-93 (rank -> grid
                        index with dimension 0 fastest)
* ``Tensor``            tensor::Tensor<T, LocaleMPI, CUDAAllocator>, tensor.hpp:38-653
                        and TensorImpl, tensor_mpi.hpp:98-574
* ``get_halo_sizes`` / ``create_*_tensor``   distconv.hpp:21-99, 253-515
* ``HaloExchange``      halo_exchange_cuda.hpp:18-423
* ``BackendDNNLib``     dnn_backend.hpp:635-980 (stream + communicators)
* ``Convolution``       convolution.hpp:19-3003
* ``BatchNormalization`` batchnorm.hpp:100-581
* ``LeakyReLU``         leaky_relu.hpp

Dimension order is the reference's everywhere in this module: index 0 is W,
then H, [D], C, N; ``-2`` is C and ``-1`` is N.  Device buffers are torch CUDA
tensors in NC[D]HW order; torch is used for memory and streams only, every
kernel on the path is launched by the library.
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from . import _abi
from ._abi import ConvDesc, NdDesc, TensorDesc, call

LHS, RHS = 0, 1
SIDES = (LHS, RHS)


def _stream_ptr(stream=None) -> ctypes.c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def _ptr(v) -> ctypes.c_void_p:
    return ctypes.c_void_p(int(v))


def _zero_on(stream, *tensors):
    """Zero fills that stand in for a kernel (an empty shard's contribution),
    ordered on the stream that kernel would have run on."""
    if stream is None or not tensors or not tensors[0].is_cuda:
        for t in tensors:
            t.zero_()
        return
    with torch.cuda.stream(stream):
        for t in tensors:
            t.zero_()


def get_dilated_filter_size(f: int, d: int) -> int:
    return f + (f - 1) * (d - 1)


# ---------------------------------------------------------------------------
# Distribution / Locale
# ---------------------------------------------------------------------------
class Distribution:
    def __init__(self, locale_shape, split_shape=None, overlap=None):
        self.locale_shape = list(locale_shape)
        self.split_shape = list(split_shape) if split_shape is not None else list(locale_shape)
        self.overlap = list(overlap) if overlap is not None else [0] * len(self.locale_shape)
        for l, s in zip(self.locale_shape, self.split_shape):
            if l % s:
                raise ValueError("locale_shape must be divisible by split_shape")
        self.fixup_overlap()

    @staticmethod
    def make_localized_distribution(nd):
        return Distribution([1] * nd)

    @staticmethod
    def make_distribution(locale_shape):
        return Distribution(locale_shape)

    @staticmethod
    def make_shared_distribution(locale_shape, split_shape=None):
        return Distribution(locale_shape, split_shape or [1] * len(locale_shape))

    @staticmethod
    def make_overlapped_distribution(locale_shape, overlap):
        return Distribution(locale_shape, locale_shape, overlap)

    def num_dims(self):
        return len(self.locale_shape)

    def get_locale_shape(self):
        return self.locale_shape

    def get_split_shape(self):
        return self.split_shape

    def get_overlap(self, dim=None):
        return self.overlap if dim is None else self.overlap[dim]

    def get_num_ranks_per_split(self, dim):
        return self.locale_shape[dim] // self.split_shape[dim]

    def is_distributed(self, dim=None):
        if dim is None:
            return any(s > 1 for s in self.split_shape)
        return self.split_shape[dim] > 1

    def is_shared(self):
        return any(self.get_num_ranks_per_split(i) > 1 for i in range(self.num_dims()))

    def set_overlap(self, overlap):
        self.overlap = list(overlap)

    def clear_overlap(self):
        self.overlap = [0] * self.num_dims()

    def fixup_overlap(self):
        for i in range(self.num_dims()):
            if not self.is_distributed(i):
                self.overlap[i] = 0

    def copy(self):
        return Distribution(self.locale_shape, self.split_shape, self.overlap)

    def __eq__(self, o):
        return (self.locale_shape, self.split_shape, self.overlap) == (o.locale_shape, o.split_shape, o.overlap)


class Locale:
    """A rank of a group.  ``allgather(bytes) -> list[bytes]`` is the only
    host collective the set-up needs (handles of peer-mapped slabs); compute
    collectives go through ``Allreduce``."""

    def __init__(self, rank: int, size: int, allgather: Optional[Callable[[bytes], List[bytes]]] = None):
        self.rank, self.size, self._allgather = rank, size, allgather

    def get_rank(self):
        return self.rank

    def get_size(self):
        return self.size

    def get_rank_idx(self, dist: Distribution):
        idx, r = [], self.rank
        for n in dist.locale_shape:
            idx.append(r % n)
            r //= n
        return idx

    def allgather(self, blob: bytes) -> List[bytes]:
        if self.size == 1:
            return [blob]
        if self._allgather is None:
            raise RuntimeError("this Locale has no host allgather")
        return self._allgather(blob)

    @staticmethod
    def from_torch_distributed(group=None):
        """Locale over an initialised torch.distributed process group."""
        import torch.distributed as dist

        rank, size = dist.get_rank(group), dist.get_world_size(group)

        def ag(blob: bytes):
            out = [None] * size
            dist.all_gather_object(out, blob, group=group)
            return out

        return Locale(rank, size, ag)


def _rank_of(idx, locale_shape):
    r, m = 0, 1
    for i, n in zip(idx, locale_shape):
        r += i * m
        m *= n
    return r


# ---------------------------------------------------------------------------
# Tensor
# ---------------------------------------------------------------------------
def _split_extent(total, parts, index):
    base, rem = divmod(total, parts)
    return base + (1 if index < rem else 0)


class Tensor:
    """Block-distributed tensor shard with halo cells on both sides of every
    partitioned dimension that has an overlap.

    ``local_shape_of`` optionally maps a grid index to that rank's local shape
    (the reference's *requested local shape*, used for convolution outputs
    whose split follows the input's); offsets are the running sums over the
    lower-indexed ranks, which the reference obtains with an Allgather
    (tensor_mpi.hpp:509-563).
    """

    def __init__(self, shape, locale: Locale, dist: Distribution,
                 local_shape_of: Optional[Callable[[Sequence[int]], Sequence[int]]] = None,
                 pitch_align: Optional[int] = None):
        self.shape = list(shape)
        self.locale = locale
        self.dist = dist.copy()
        self.nd = len(self.shape)
        self._local_shape_of = local_shape_of
        self.proc_idx = locale.get_rank_idx(self.dist)
        self.split_idx = [p // self.dist.get_num_ranks_per_split(i) for i, p in enumerate(self.proc_idx)]
        self.local_shape = self._local_of(self.proc_idx)
        self.offset = []
        for d in range(self.nd):
            off = 0
            if self.dist.is_distributed(d):
                per = self.dist.get_num_ranks_per_split(d)
                for j in range(0, self.split_idx[d]):
                    idx = list(self.proc_idx)
                    idx[d] = j * per
                    off += self._local_of(idx)[d]
            self.offset.append(off)
        # Row pitch (tensor.hpp:184-192 get_pitch; the reference pads rows with
        # CUDAPitchedAllocator, memory_cuda.hpp:68-104).  A shard with halo
        # cells along W has rows of local + 2 * overlap cells, rarely a multiple
        # of 16 bytes; such rows are padded to PITCH_ALIGN floats so that the
        # bulk-copy fed tensor-core kernels can address them.  Shards without a
        # W halo stay dense.  pitch_align=1 forces dense rows.
        # Inside a padded row the halo-extended cells start `lead` floats in, so
        # that the OWNED cells start on a 16-byte boundary: bulk stores and
        # vector accesses of the kernels that write a shard's interior need
        # that, while the kernels that read the window with its halo fetch from
        # the boundary below it.  Row: [lead pad][halo][owned][halo][tail pad].
        if pitch_align is None:
            pitch_align = self.PITCH_ALIGN if self.dist.overlap[0] > 0 else 1
        self.pitch_align = max(1, int(pitch_align))
        real_w = self.local_shape[0] + 2 * self.dist.overlap[0]
        self.lead = (-self.dist.overlap[0]) % self.pitch_align
        self.pitch = -(-(self.lead + real_w) // self.pitch_align) * self.pitch_align
        self.buffer: Optional[torch.Tensor] = None
        self._storage: Optional[torch.Tensor] = None

    PITCH_ALIGN = 4  # floats: 16 bytes

    def _local_of(self, proc_idx):
        if self._local_shape_of is not None:
            return list(self._local_shape_of(proc_idx))
        out = []
        for d in range(self.nd):
            if self.dist.is_distributed(d):
                sidx = proc_idx[d] // self.dist.get_num_ranks_per_split(d)
                out.append(_split_extent(self.shape[d], self.dist.split_shape[d], sidx))
            else:
                out.append(self.shape[d])
        return out

    # -- shape queries (reference names) --
    def get_num_dims(self):
        return self.nd

    def get_num_spatial_dims(self):
        return self.nd - 2

    def get_shape(self):
        return self.shape

    def get_local_shape(self):
        return self.local_shape

    def get_overlap(self):
        return self.dist.overlap

    def get_halo_width(self, dim=None):
        return self.dist.overlap if dim is None else self.dist.overlap[dim]

    def get_local_real_shape(self):
        return [l + 2 * o for l, o in zip(self.local_shape, self.dist.overlap)]

    def get_local_size(self):
        n = 1
        for v in self.local_shape:
            n *= v
        return n

    def get_size(self):
        n = 1
        for v in self.shape:
            n *= v
        return n

    def get_global_index(self):
        return self.offset

    def get_distribution(self):
        return self.dist

    def get_locale(self):
        return self.locale

    def get_split_index(self):
        return self.split_idx

    def get_proc_index(self):
        return self.proc_idx

    def is_split_root(self):
        return all(p % self.dist.get_num_ranks_per_split(i) == 0 for i, p in enumerate(self.proc_idx))

    def get_dimension_rank_offset(self, dim, rank_idx):
        off = 0
        per = self.dist.get_num_ranks_per_split(dim)
        for j in range(0, rank_idx // per):
            idx = list(self.proc_idx)
            idx[dim] = j * per
            off += self._local_of(idx)[dim]
        return off

    # -- memory --
    def np_real_shape(self):
        return tuple(reversed(self.get_local_real_shape()))

    def get_pitch(self):
        """Elements between consecutive rows of the buffer (tensor.hpp:184-192)."""
        return self.pitch

    def get_local_pitched_shape(self):
        """The halo-extended shape with the row padded to the pitch
        (tensor.hpp:483-485)."""
        r = self.get_local_real_shape()
        r[0] = self.pitch
        return r

    def new_storage(self, device="cuda", zero=True) -> torch.Tensor:
        """A device array laid out like this shard's buffer (rows padded to the
        pitch); pass it to set_view."""
        shp = tuple(reversed(self.get_local_pitched_shape()))
        return (torch.zeros if zero else torch.empty)(shp, dtype=torch.float32, device=device)

    def allocate(self, device="cuda"):
        self.set_view(self.new_storage(device))
        return 0

    def set_view(self, buf: torch.Tensor):
        """Use ``buf`` as the shard's memory (tensor.hpp:604-623 View): either
        a contiguous array of the pitched shape (new_storage) or, for a dense
        shard, of the halo-extended shape.  ``buffer`` is the halo-extended
        shard without the row padding, a strided view when rows are padded
        (it starts ``lead`` floats into the array)."""
        real_w = self.local_shape[0] + 2 * self.dist.overlap[0]
        if tuple(buf.shape) == self.np_real_shape() and buf.stride(-1) == 1 and (
                buf.dim() < 2 or buf.stride(-2) == self.pitch):
            # already the un-padded view of a pitched array (or dense)
            self._storage = buf
            self.buffer = buf
            return
        assert tuple(buf.shape) == tuple(reversed(self.get_local_pitched_shape())) and buf.is_contiguous(), \
            "set_view wants an array of the pitched shape"
        self._storage = buf
        self.buffer = buf[..., self.lead:self.lead + real_w] if self.pitch != real_w else buf

    def get_buffer(self) -> int:
        return self.buffer.data_ptr()

    def get_strides(self):
        """Element strides of the halo-extended buffer, reference order."""
        st, acc = [], 1
        for i, r in enumerate(self.get_local_real_shape()):
            st.append(acc)
            acc *= self.pitch if i == 0 else r
        return st

    def get_local_offset(self, idx, idx_include_halo=False):
        st = self.get_strides()
        ov = self.dist.overlap
        return sum((i + (0 if idx_include_halo else o)) * s for i, o, s in zip(idx, ov, st))

    def get_base_ptr(self) -> int:
        return self.get_buffer() + 4 * self.get_local_offset([0] * self.nd)

    def owned(self) -> torch.Tensor:
        sl = tuple(slice(o, o + l) for o, l in reversed(list(zip(self.dist.overlap, self.local_shape))))
        return self.buffer[sl]

    def zero(self, stream=None):
        _zero_on(stream, self._storage)

    def desc(self) -> TensorDesc:
        d = TensorDesc()
        d.ndims, d.dtype = self.nd, 0
        real = self.get_local_real_shape()
        for i in range(self.nd):
            d.local_shape[i] = self.local_shape[i]
            d.real_shape[i] = real[i]
            d.overlap[i] = self.dist.overlap[i]
        d.pitch = self.pitch
        return d

    def clear_halo(self, dim, stream=None):
        """Tensor::clear_halo (legacy/src/tensor/tensor_mpi_cuda.cu:66-82)."""
        if self.get_local_size() == 0:
            return
        d = self.desc()
        call("dcb_clear_halo", ctypes.byref(d), _ptr(self.get_buffer()), dim, _stream_ptr(stream))

    def nd_desc(self, widths_lo=None, widths_hi=None) -> NdDesc:
        """cuDNN-style descriptor of the owned cells extended by widths_lo /
        widths_hi halo cells per spatial dimension
        (setup_tensor_descriptor, dnn_backend_impl.hpp:31-70)."""
        nsd = self.nd - 2
        lo = widths_lo or [0] * nsd
        hi = widths_hi or [0] * nsd
        st = self.get_strides()
        d = NdDesc()
        d.nsd = nsd
        d.n, d.c = self.local_shape[-1], self.local_shape[-2]
        d.sn, d.sc = st[-1], st[-2]
        for i in range(3):
            d.dims[i], d.strides[i] = 1, 0
        for i in range(nsd):  # ref dim i -> slot 2 - i
            d.dims[2 - i] = self.local_shape[i] + lo[i] + hi[i]
            d.strides[2 - i] = st[i]
        if nsd == 2:
            d.strides[0] = st[1] * (self.local_shape[1] + lo[1] + hi[1])
        return d

    def nd_ptr(self, widths_lo=None) -> int:
        nsd = self.nd - 2
        lo = list(widths_lo or [0] * nsd) + [0, 0]
        idx = [self.dist.overlap[i] - lo[i] for i in range(self.nd)]
        return self.get_buffer() + 4 * self.get_local_offset(idx, True)

    def full_nd_desc(self) -> NdDesc:
        ov = self.dist.overlap[: self.nd - 2]
        return self.nd_desc(ov, ov)


# ---------------------------------------------------------------------------
# geometry helpers (distconv.hpp)
# ---------------------------------------------------------------------------
def _halo_sizes_for(shape, dist: Distribution, split_idx, offset, local_shape, filter_dims, strides, dilations,
                    with_padding):
    nd = len(shape)
    fs, bs, fr, br = ([0] * nd for _ in range(4))
    for i in range(nd - 2):
        if dist.split_shape[i] == 1:
            continue
        df = get_dilated_filter_size(filter_dims[i], dilations[i])
        if df % 2 == 0:
            assert strides[i] == df
            continue
        radius, s, off = (df - 1) // 2, strides[i], offset[i]
        if split_idx[i] == 0:
            if with_padding:
                br[i] = radius
        else:
            x = off - (0 if with_padding else radius)
            br[i] = radius - (s - (x % s)) % s
            bs[i] = radius - (x - 1) % s
        if not (split_idx[i] == dist.split_shape[i] - 1 and not with_padding):
            y = off + local_shape[i] - 1 - (0 if with_padding else radius)
            fr[i] = radius - y % s
            fs[i] = radius - (s - ((y + 1) % s)) % s
        fs[i], fr[i], bs[i], br[i] = (max(v, 0) for v in (fs[i], fr[i], bs[i], br[i]))
    return fs, bs, fr, br


def get_halo_sizes(input: Tensor, filter_dims, strides, dilations, with_padding):
    """internal::get_halo_sizes (distconv.hpp:21-99): fwd_send, bwd_send,
    fwd_recv, bwd_recv per dimension."""
    return _halo_sizes_for(input.shape, input.dist, input.split_idx, input.offset, input.local_shape, filter_dims,
                           strides, dilations, with_padding)


def _conv_out_local(input: Tensor, proc_idx, filter_dims, strides, dilations, with_padding, K):
    """get_convolution_output_local_tensor_shape (distconv.hpp:135-200) for
    the rank at grid index proc_idx."""
    d = input.dist
    split_idx = [p // d.get_num_ranks_per_split(i) for i, p in enumerate(proc_idx)]
    local = input._local_of(proc_idx)
    offset = []
    for dim in range(input.nd):
        off = 0
        if d.is_distributed(dim):
            per = d.get_num_ranks_per_split(dim)
            for j in range(split_idx[dim]):
                idx = list(proc_idx)
                idx[dim] = j * per
                off += input._local_of(idx)[dim]
        offset.append(off)
    fs, bs, fr, br = _halo_sizes_for(input.shape, d, split_idx, offset, local, filter_dims, strides, dilations,
                                     with_padding)
    out = list(local)
    for i in range(input.nd - 2):
        df = get_dilated_filter_size(filter_dims[i], dilations[i])
        ext = local[i] + br[i] + fr[i]
        if with_padding and d.split_shape[i] == 1:
            ext += df - 1
        out[i] = 0 if ext < df else -(-(ext - df + 1) // strides[i])
    out[-2] = K
    return out


def create_input_tensor(shape, locale_shape, filter_dims, strides, dilations, locale: Locale) -> Tensor:
    """distconv.hpp:253-288: overlap = (dilated filter - 1)/2 in every
    partitioned spatial dimension."""
    nd = len(shape)
    overlap = [0] * nd
    for i in range(nd - 2):
        if locale_shape[i] == 1:
            continue
        df = get_dilated_filter_size(filter_dims[i], dilations[i])
        if df % 2:
            overlap[i] = (df - 1) // 2
        else:
            assert df == strides[i]
    return Tensor(shape, locale, Distribution.make_overlapped_distribution(locale_shape, overlap))


def create_d_input_tensor(input: Tensor) -> Tensor:
    return Tensor(input.shape, input.locale, input.dist, input._local_shape_of)


def create_convolution_output_tensor(input: Tensor, filter_shape, strides, pads, dilations) -> Tensor:
    """distconv.hpp:365-413.  filter_shape is (fw, fh, [fd,] C, K)."""
    nd, nsd = input.nd, input.nd - 2
    use_padding = pads[0] != 0
    out_shape = [0] * nd
    for i in range(nsd):
        df = get_dilated_filter_size(filter_shape[i], dilations[i])
        assert (df - 1) % 2 == 0 and (pads[i] * 2 + 1 == df or pads[i] == 0)
        if input.shape[i] + 2 * pads[i] >= df:
            out_shape[i] = -(-(input.shape[i] - df + 1 + 2 * pads[i]) // strides[i])
    out_shape[-2], out_shape[-1] = filter_shape[-1], input.shape[-1]
    dist = input.dist.copy()
    dist.clear_overlap()
    fdims = list(filter_shape[:nsd])
    K = filter_shape[-1]
    return Tensor(out_shape, input.locale, dist,
                  lambda pidx: _conv_out_local(input, pidx, fdims, strides, dilations, use_padding, K))


def create_convolution_d_output_tensor(output: Tensor, filter_shape, dilations) -> Tensor:
    """distconv.hpp:455-481: same split as the output, overlap = stencil."""
    nd = output.nd
    dist = output.dist.copy()
    overlap = [0] * nd
    for i in range(nd - 2):
        f = get_dilated_filter_size(filter_shape[i], dilations[i])
        assert (f - 1) % 2 == 0
        if dist.locale_shape[i] > 1:
            overlap[i] = (f - 1) // 2
    dist.set_overlap(overlap)
    return Tensor(output.shape, output.locale, dist, output._local_of)


def create_pooling_output_tensor(input: Tensor, window, strides, pads) -> Tensor:
    """distconv.hpp:518-565: odd windows with pad 0 or (window-1)/2, even
    windows with stride == window and no padding; window / strides / pads in
    reference order (W first)."""
    nd, nsd = input.nd, input.nd - 2
    use_padding = pads[0] != 0
    out_shape = list(input.shape)
    for i in range(nsd):
        if input.shape[i] + 2 * pads[i] < window[i]:
            out_shape[i] = 0
        elif window[i] % 2:
            assert pads[i] == 0 or pads[i] * 2 + 1 == window[i]
            assert (pads[i] != 0) == use_padding
            out_shape[i] = -(-(input.shape[i] - window[i] + 1 + 2 * pads[i]) // strides[i])
        else:
            assert pads[i] == 0 and strides[i] == window[i]
            out_shape[i] = input.shape[i] // strides[i]
    dist = input.dist.copy()
    dist.clear_overlap()
    wdims, C = list(window[:nsd]), input.shape[-2]
    return Tensor(out_shape, input.locale, dist,
                  lambda pidx: _conv_out_local(input, pidx, wdims, strides, [1] * nsd, use_padding, C))


def create_pooling_d_output_tensor(output: Tensor) -> Tensor:
    """distconv.hpp:567-581."""
    return Tensor(output.shape, output.locale, output.dist.copy(), output._local_of)


# ---------------------------------------------------------------------------
# HaloExchange
# ---------------------------------------------------------------------------
class HaloExchange:
    """tensor::HaloExchange (halo_exchange_cuda.hpp:18-423) over the
    peer-store transport.  Two-phase set-up: construct on every rank, gather
    ``export()`` blobs, ``connect(blobs)``; ``setup()`` does both through the
    tensor's Locale."""

    def __init__(self, tensor: Tensor):
        self.tensor = tensor
        self.peers = [[self.find_peer_rank(d, s) for s in SIDES] for d in range(_abi.DCB_MAX_DIMS)]
        flat = (ctypes.c_int32 * (2 * _abi.DCB_MAX_DIMS))(*[p for ds in self.peers for p in ds])
        self._plan = ctypes.c_void_p()
        d = tensor.desc()
        call("dcb_halo_plan_create", ctypes.byref(d), flat, tensor.locale.rank, ctypes.byref(self._plan))

    def __del__(self):
        try:
            if getattr(self, "_plan", None):
                _abi.lib().dcb_halo_plan_destroy(self._plan)
        except Exception:
            pass

    def is_exchange_required(self, dim):
        t = self.tensor
        if dim >= t.nd:
            return False
        return (t.dist.is_distributed(dim) and t.dist.split_shape[dim] > 1 and t.get_halo_width(dim) > 0
                and t.get_local_size() > 0)

    def find_peer_rank(self, dim, side):
        """halo_exchange_cuda.hpp:322-357; -1 stands for MPI_PROC_NULL."""
        t = self.tensor
        if not self.is_exchange_required(dim):
            return -1
        ls = t.dist.locale_shape
        j = t.proc_idx[dim] + (1 if side == RHS else -1)
        if j < 0 or j >= ls[dim]:
            return -1
        if t.get_dimension_rank_offset(dim, j) == t.shape[dim]:
            return -1
        idx = list(t.proc_idx)
        idx[dim] = j
        if 0 in t._local_of(idx):
            return -1
        return _rank_of(idx, ls)

    def export(self) -> bytes:
        buf = ctypes.create_string_buffer(_abi.HALO_BLOB_BYTES)
        call("dcb_halo_plan_export", self._plan, buf)
        return buf.raw

    def connect(self, blobs: Sequence[bytes]):
        joined = ctypes.create_string_buffer(b"".join(blobs), _abi.HALO_BLOB_BYTES * len(blobs))
        call("dcb_halo_plan_connect", self._plan, joined, len(blobs))

    def setup(self):
        self.connect(self.tensor.locale.allgather(self.export()))
        return self

    @staticmethod
    def _flags(is_reverse=False, skip_unpack=False, op="ID", clear_boundary=False):
        return (_abi.HALO_REVERSE if is_reverse else 0) | (_abi.HALO_SKIP_UNPACK if skip_unpack else 0) | \
            (_abi.HALO_CLEAR_BOUNDARY if clear_boundary else 0) | _abi.HALO_OPS[op]

    def exchange(self, stream=None, is_reverse=False, skip_unpack=False, op="ID", clear_boundary=False):
        """All dimensions in order.  ``clear_boundary``: the launch that packs a
        dimension also zeroes that dimension's halo slabs that have no neighbour
        (what Tensor::clear_halo before the exchange leaves behind), saving one
        launch per partitioned dimension."""
        call("dcb_halo_exchange", self._plan, _ptr(self.tensor.get_buffer()),
             self._flags(is_reverse, skip_unpack, op, clear_boundary), _stream_ptr(stream))

    def pack_put(self, dim, stream=None, is_reverse=False, op="ID", clear_boundary=False):
        call("dcb_halo_pack_put", self._plan, _ptr(self.tensor.get_buffer()), dim,
             self._flags(is_reverse, False, op, clear_boundary), _stream_ptr(stream))

    def wait_unpack(self, dim, stream=None, is_reverse=False, op="ID"):
        call("dcb_halo_wait_unpack", self._plan, _ptr(self.tensor.get_buffer()), dim,
             self._flags(is_reverse, False, op), _stream_ptr(stream))

    def unpack(self, stream=None, is_reverse=False, op="ID"):
        call("dcb_halo_unpack", self._plan, _ptr(self.tensor.get_buffer()),
             self._flags(is_reverse, False, op), _stream_ptr(stream))

    def status(self, stream=None) -> int:
        return _abi.lib().dcb_halo_plan_status(self._plan, _stream_ptr(stream))


# ---------------------------------------------------------------------------
# Re-distribution and dump
# ---------------------------------------------------------------------------
def owned_box(t: Tensor, rank: int):
    """(offset, extent) in global coordinates of what ``rank`` owns of ``t``;
    extent all zero for a rank that is not the root of a replicated dimension
    (only roots hold the authoritative copy, tensor_mpi.hpp is_split_root)."""
    ls = t.dist.locale_shape
    pidx, r = [], rank
    for n in ls:
        pidx.append(r % n)
        r //= n
    per = [t.dist.get_num_ranks_per_split(i) for i in range(t.nd)]
    if any(p % q for p, q in zip(pidx, per)):
        return [0] * t.nd, [0] * t.nd
    ext = t._local_of(pidx)
    off = []
    for d in range(t.nd):
        o = 0
        if t.dist.is_distributed(d):
            for j in range(pidx[d] // per[d]):
                idx = list(pidx)
                idx[d] = j * per[d]
                o += t._local_of(idx)[d]
        off.append(o)
    if 0 in ext:
        ext = [0] * t.nd
    return off, list(ext)


class TensorShuffler:
    """tensor::TensorMPICUDAShuffler (shuffle_mpi_cuda.hpp:14-512): moves a
    tensor between two distributions of the same global shape.  Cells travel
    as peer stores into the owner's receive window; see csrc/shuffle.cu."""

    def __init__(self, src: Tensor, dst: Tensor, connect=True):
        assert list(src.shape) == list(dst.shape) and src.locale.size == dst.locale.size
        self.src, self.dst = src, dst
        self.locale = src.locale
        self._plans = {}
        for key, (a, b) in (("fwd", (src, dst)), ("bwd", (dst, src))):
            n = self.locale.size
            sb, db = (_abi.Box * n)(), (_abi.Box * n)()
            for r in range(n):
                for boxes, t in ((sb, a), (db, b)):
                    off, ext = owned_box(t, r)
                    for i in range(t.nd):
                        boxes[r].off[i], boxes[r].ext[i] = off[i], ext[i]
            plan = ctypes.c_void_p()
            ad, bd = a.desc(), b.desc()
            call("dcb_shuffle_plan_create", ctypes.byref(ad), ctypes.byref(bd), sb, db, self.locale.rank, n,
                 ctypes.byref(plan))
            self._plans[key] = plan
        if connect:
            self.setup()

    def __del__(self):
        try:
            for p in getattr(self, "_plans", {}).values():
                _abi.lib().dcb_shuffle_plan_destroy(p)
        except Exception:
            pass

    def export(self, which: str) -> bytes:
        buf = ctypes.create_string_buffer(_abi.SHUFFLE_BLOB_BYTES)
        call("dcb_shuffle_plan_export", self._plans[which], buf)
        return buf.raw

    def connect(self, which: str, blobs: Sequence[bytes]):
        joined = ctypes.create_string_buffer(b"".join(blobs), _abi.SHUFFLE_BLOB_BYTES * len(blobs))
        call("dcb_shuffle_plan_connect", self._plans[which], joined, len(blobs))

    def setup(self):
        for which in ("fwd", "bwd"):
            self.connect(which, self.locale.allgather(self.export(which)))
        return self

    # src / dst are buffer addresses (Tensor.get_buffer()), as in the reference
    def shuffle_forward(self, src: int, dst: int, stream=None):
        call("dcb_shuffle", self._plans["fwd"], _ptr(src), _ptr(dst), _stream_ptr(stream))

    def shuffle_backward(self, src: int, dst: int, stream=None):
        call("dcb_shuffle", self._plans["bwd"], _ptr(src), _ptr(dst), _stream_ptr(stream))

    # halves, for ranks that share a device (every put before any wait)
    def put(self, which: str, src: int, stream=None):
        call("dcb_shuffle_put", self._plans[which], _ptr(src), _stream_ptr(stream))

    def wait_unpack(self, which: str, dst: int, stream=None):
        call("dcb_shuffle_wait_unpack", self._plans[which], _ptr(dst), _stream_ptr(stream))

    def status(self, which: str, stream=None) -> int:
        return _abi.lib().dcb_shuffle_plan_status(self._plans[which], _stream_ptr(stream))


def dump_tensor(t: Tensor, file_path: str, binary: bool = False) -> int:
    """distconv.hpp:581-631: rank 0 writes the whole tensor in memory order
    (dimension 0 fastest, no halos) to ``file_path + ".out"`` as raw float32, or
    ``+ ".txt"`` one value per line.  Collective: every rank contributes what it
    owns through the locale's allgather."""
    off, ext = owned_box(t, t.locale.rank)
    own = t.owned().detach().cpu().numpy().astype(np.float32) if 0 not in ext else np.zeros(0, np.float32)
    blobs = t.locale.allgather(own.tobytes())
    if t.locale.rank != 0:
        return 0
    g = np.zeros(tuple(reversed(t.shape)), np.float32)
    for r, blob in enumerate(blobs):
        o, e = owned_box(t, r)
        if 0 in e:
            continue
        sl = tuple(slice(a, a + b) for a, b in reversed(list(zip(o, e))))
        g[sl] = np.frombuffer(blob, np.float32).reshape(tuple(reversed(e)))
    if binary:
        g.tofile(file_path + ".out")
    else:
        with open(file_path + ".txt", "w") as f:
            for v in g.ravel():
                f.write(f"{v:g}\n")
    return 0


def dump_local_tensor(t: Tensor, file_path: str, binary: bool = False) -> int:
    """distconv.hpp:633-671: every rank writes its own shard (halo cells
    included, as the reference copies out the whole local buffer) to
    ``file_path_<rank>``."""
    a = t.buffer.detach().cpu().numpy().astype(np.float32)
    path = f"{file_path}_{t.locale.rank}"
    if binary:
        a.tofile(path + ".out")
    else:
        with open(path + ".txt", "w") as f:
            for v in a.ravel():
                f.write(f"{v:g}\n")
    return 0


# ---------------------------------------------------------------------------
# All-reduce and backend
# ---------------------------------------------------------------------------
class Allreduce:
    """tensor::Allreduce<float> (allreduce.hpp:8-19).  ``kind`` "peer" uses the
    in-kernel peer-memory reduction (short vectors), "nccl" an NCCL
    communicator created by the library."""

    def __init__(self, locale: Locale, kind="peer", max_count=4096, connect=True):
        self.locale, self.kind = locale, kind
        self._comm = ctypes.c_void_p()
        if kind == "peer":
            call("dcb_comm_create_peer", locale.rank, locale.size, max_count, ctypes.byref(self._comm))
            if connect:
                self.connect(locale.allgather(self.export()))
        elif kind == "nccl":
            idbuf = ctypes.create_string_buffer(_abi.NCCL_ID_BYTES)
            if locale.rank == 0:
                call("dcb_nccl_unique_id", idbuf)
            uid = locale.allgather(idbuf.raw)[0]
            call("dcb_comm_create_nccl", ctypes.create_string_buffer(uid, _abi.NCCL_ID_BYTES), locale.rank,
                 locale.size, ctypes.byref(self._comm))
        else:
            raise ValueError(kind)

    def __del__(self):
        try:
            if getattr(self, "_comm", None):
                _abi.lib().dcb_comm_destroy(self._comm)
        except Exception:
            pass

    def export(self) -> bytes:
        buf = ctypes.create_string_buffer(_abi.COMM_BLOB_BYTES)
        call("dcb_comm_export", self._comm, buf)
        return buf.raw

    def connect(self, blobs):
        joined = ctypes.create_string_buffer(b"".join(blobs), _abi.COMM_BLOB_BYTES * len(blobs))
        call("dcb_comm_connect", self._comm, joined, len(blobs))

    def allreduce(self, ptr: int, count: int, stream=None):
        call("dcb_allreduce_sum", self._comm, _ptr(ptr), count, _stream_ptr(stream))

    def push(self, ptr: int, count: int, stream=None):
        call("dcb_allreduce_push", self._comm, _ptr(ptr), count, _stream_ptr(stream))

    def pull(self, ptr: int, count: int, stream=None):
        call("dcb_allreduce_pull", self._comm, _ptr(ptr), count, _stream_ptr(stream))

    def status(self, stream=None) -> int:
        return _abi.lib().dcb_comm_status(self._comm, _stream_ptr(stream))


class Options:
    """backend::Options (dnn_backend.hpp:46-63) with the environment overrides
    of legacy/src/dnn_backend/options.cpp:13-71: a variable that is SET (to
    anything, as in the reference) turns its option on.  ``math_mode`` has no
    counterpart there: ``MATH_FP32`` (3xTF32 on tensor cores, fp32 quality),
    ``MATH_TF32`` (one TF32 pass), ``MATH_BF16`` (bf16 operands, fp32
    accumulation) or ``MATH_FP32_SIMT`` (CUDA cores)."""

    def __init__(self, overlap_halo_exchange=False, deterministic=True, enable_profiling=False,
                 math_mode=_abi.MATH_FP32, ws_capacity_factor=1.0):
        env = os.environ
        self.overlap_halo_exchange = overlap_halo_exchange or "DISTCONV_OVERLAP_HALO_EXCHANGE" in env
        self.deterministic = deterministic or "DISTCONV_DETERMINISTIC" in env
        self.enable_profiling = enable_profiling or any(
            k in env for k in ("DISTCONV_ENABLE_PROFILING", "DISTCONV_PROFILING", "DISTCONV_NVTX"))
        self.ws_capacity_factor = float(env.get("DISTCONV_WS_CAPACITY_FACTOR", ws_capacity_factor))
        self.math_mode = math_mode


class BackendDNNLib:
    """DNNBackend<GPUDNNBackend> (dnn_backend.hpp:635-980): owns the main
    stream and a working all-reduce communicator (the reference never
    constructs its own, communicator_manager.cpp:26-57)."""

    def __init__(self, locale: Locale, stream=None, options: Optional[Options] = None, allreduce: str = "peer",
                 allreduce_max_count: int = 32768, connect=True):
        self.locale = locale
        self.stream = stream
        self.options = options or Options()
        self.allreducer = Allreduce(locale, allreduce, allreduce_max_count, connect=connect)

    def get_name(self):
        return "B200"

    def get_stream(self):
        return self.stream

    def get_comm(self):
        return self.locale

    def wait(self):
        (self.stream or torch.cuda.current_stream()).synchronize()


# ---------------------------------------------------------------------------
# Convolution
# ---------------------------------------------------------------------------
class Convolution:
    """Convolution<BackendDNNLib, float> (convolution.hpp:19-3003), spatial
    parallelism only (no channel/filter parallelism)."""

    def __init__(self, backend: BackendDNNLib, num_dims: int, halo_exchange_method="AL", chanfilt_algo="NONE"):
        self.be = backend
        self.num_dims = num_dims
        self.nsd = num_dims - 2
        self._plan_fwd = ctypes.c_void_p()
        self._plan_bwd = ctypes.c_void_p()
        self._plan_wgrad = ctypes.c_void_p()
        self.halo_xch_input = None
        self.halo_xch_d_output = None
        self._ready = False

    def __del__(self):
        try:
            for p in [getattr(self, "_plan_fwd", None), getattr(self, "_plan_bwd", None),
                      getattr(self, "_plan_wgrad", None)] + list(
                    getattr(self, "_ov_plans", [])):
                if p:
                    _abi.lib().dcb_conv_plan_destroy(p)
        except Exception:
            pass

    def setup(self, input: Tensor, filter: torch.Tensor, output: Tensor, d_input: Optional[Tensor],
              d_filter: Optional[torch.Tensor], d_output: Optional[Tensor], pads, strides, dilations, num_groups=1,
              fwd_algo="DEFAULT", bwd_data_algo="DEFAULT", bwd_filter_algo="DEFAULT", ws_size=0,
              skip_bp_data=False, deconv=False, connect=True):
        """convolution.hpp:119-290.  ``filter`` is a dense torch tensor
        (K, C, [fd,] fh, fw); pads/strides/dilations are in reference order
        (W first).  Algorithm names are accepted and ignored: there is one
        kernel family."""
        assert num_groups == 1 and not deconv
        nsd = self.nsd
        self.input, self.output, self.d_input, self.d_output = input, output, d_input, d_output
        self.pads, self.strides, self.dilations = list(pads), list(strides), list(dilations)
        self.filter_dims = [filter.shape[-1 - i] for i in range(nsd)]  # W first
        self.K, self.C = filter.shape[0], filter.shape[1]
        # setup_halo_xch (convolution.hpp:2672-2686).  The d_output exchanger is
        # built on d_output, which is what backward data needs.
        self.halo_xch_input = HaloExchange(input)
        self.halo_xch_d_output = HaloExchange(d_output) if d_output is not None else None
        if connect:
            self.halo_xch_input.setup()
            if self.halo_xch_d_output is not None:
                self.halo_xch_d_output.setup()
        if input.get_local_size() == 0 or output.get_local_size() == 0:
            self._ready = False
            self.empty = True
            return
        self.empty = False
        stencil = []
        for i in range(nsd):
            wd = get_dilated_filter_size(self.filter_dims[i], dilations[i])
            if wd % 2:
                stencil.append((wd - 1) // 2)
            else:
                assert strides[i] == wd
                stencil.append(0)
        for i in range(nsd):
            assert pads[i] == pads[0] and (pads[i] == stencil[i] or pads[i] == 0)
        use_padding = pads[0] != 0
        self.halo_fwd_send, self.halo_bwd_send, self.halo_fwd_recv, self.halo_bwd_recv = get_halo_sizes(
            input, self.filter_dims, strides, dilations, use_padding)
        ov = input.get_overlap()
        # setup_convolution_descriptor (convolution.hpp:2541-2670)
        pads_fp, pads_bp = list(pads), []
        for i in range(nsd):
            pads_bp.append(stencil[i] if pads[i] == 0 else stencil[i] * strides[i])
        for i in range(nsd):
            if ov[i] > 0:
                pads_fp[i] = 0
            else:
                pads_fp[i] = pads[i]
                pads_bp[i] = pads[i]
        lo, hi = self.halo_bwd_recv[:nsd], self.halo_fwd_recv[:nsd]
        self._x_lo = lo
        xd = input.nd_desc(lo, hi)
        yd = output.nd_desc()
        self._plan_fwd = self._make_plan(xd, yd, pads_fp)
        self._setup_overlap(input, xd, yd, pads_fp, lo, hi)
        if d_output is not None:
            # Backward data.  The reference hands cuDNN the halo-extended d_input
            # (convolution.hpp:2541-2670), whose halo cells then receive partial
            # sums nobody reads.  Where a partitioned dimension has unit stride
            # and dilation only the OWNED cells of d_input are computed here:
            # they start on a 16-byte boundary of a padded row (the halo cells do
            # not), which the bulk stores of the tensor-core kernels need, and
            # no work goes into cells that are thrown away.  In the descriptor's
            # terms the padding grows by d_output's halo width.
            dyd = d_output.full_nd_desc()
            dyov = d_output.get_overlap()
            dlo, dhi = list(lo), list(hi)
            for i in range(nsd):
                if ov[i] > 0 and strides[i] == 1 and dilations[i] == 1:
                    dlo[i] = dhi[i] = 0
                    pads_bp[i] = stencil[i] + dyov[i]
            self._dx_lo = dlo
            dxd = (d_input or input).nd_desc(dlo, dhi)
            self._plan_bwd = self._make_plan(dxd, dyd, pads_bp)
            # Backward filter: the forward geometry with d_output's owned cells in
            # the output's place.  (The reference passes the halo-extended
            # d_output with its halo cleared, convolution.hpp:878-1107; the owned
            # cells alone give the same sums, start on a 16-byte boundary and need
            # no clearing.)
            self._plan_wgrad = self._make_plan(xd, d_output.nd_desc(), pads_fp)
        self._ready = True

    def _setup_overlap(self, input: Tensor, xd: NdDesc, yd: NdDesc, pads_fp, lo, hi):
        """setup_tensors_overlap (convolution.hpp:1497-1584), forward pass: the
        output is cut into an interior that reads no halo cell and one boundary
        slab per side with a neighbour; the interior runs while the halo is in
        flight.  As in the reference only with one partitioned dimension
        (convolution.hpp:212-245 gives the reason: diagonal halo cells), and here
        only for unit stride and dilation in it."""
        self._ov = None
        self._ov_plans = []
        if not self.be.options.overlap_halo_exchange:
            return
        nsd = self.nsd
        ov = input.get_overlap()
        dims = [i for i in range(nsd) if ov[i] > 0 and input.dist.locale_shape[i] > 1]
        if len(dims) != 1 or self.strides[dims[0]] != 1 or self.dilations[dims[0]] != 1:
            return
        i = dims[0]
        slot = 2 - i
        f, out_ext = self.filter_dims[i], yd.dims[slot]
        b_lo = lo[i] if self.halo_xch_input.peers[i][0] >= 0 else 0
        b_hi = hi[i] if self.halo_xch_input.peers[i][1] >= 0 else 0
        if b_lo + b_hi == 0 or out_ext <= b_lo + b_hi:
            return  # nothing to wait for, or too thin to have an interior
        regions = []
        for a, b in ((b_lo, out_ext - b_hi), (0, b_lo), (out_ext - b_hi, out_ext)):
            if b <= a:
                continue
            xr, yr = NdDesc(), NdDesc()
            ctypes.memmove(ctypes.byref(xr), ctypes.byref(xd), ctypes.sizeof(NdDesc))
            ctypes.memmove(ctypes.byref(yr), ctypes.byref(yd), ctypes.sizeof(NdDesc))
            # no padding in a partitioned dimension: output plane o reads window planes [o, o + f)
            xr.dims[slot], yr.dims[slot] = (b - a) + f - 1, b - a
            plan = self._make_plan(xr, yr, pads_fp)
            self._ov_plans.append(plan)
            regions.append((plan, 4 * a * xd.strides[slot], 4 * a * yd.strides[slot]))
        self._ov = (i, regions)
        self._ov_stream = torch.cuda.Stream(priority=-1)
        self._ov_events = (torch.cuda.Event(), torch.cuda.Event())

    def _forward_overlapped(self, alpha, input: Tensor, filter: torch.Tensor, beta, output: Tensor):
        """convolution.hpp:520-600: put the halo, run the interior, then the
        boundary slabs once the neighbours' cells have been unpacked."""
        dim, regions = self._ov
        main = self.be.stream if isinstance(self.be.stream, torch.cuda.Stream) else torch.cuda.current_stream()
        self._clear_halos(input, main)
        self.halo_xch_input.pack_put(dim, main)
        self._ov_events[0].record(main)
        self._ov_stream.wait_event(self._ov_events[0])
        self.halo_xch_input.wait_unpack(dim, self._ov_stream)
        self._ov_events[1].record(self._ov_stream)
        self.forward_regions(alpha, input, filter, beta, output, main, self._ov_events[1])
        return 0

    def forward_regions(self, alpha, input: Tensor, filter: torch.Tensor, beta, output: Tensor, stream=None,
                        halo_ready: Optional[torch.cuda.Event] = None):
        """The interior and then the boundary slabs of the overlapped forward
        pass; the boundary slabs wait for ``halo_ready`` (None: the halo is
        already in place)."""
        _, regions = self._ov
        x0, y0 = input.nd_ptr(self._x_lo), output.get_base_ptr()
        for n, (plan, xoff, yoff) in enumerate(regions):  # the interior comes first
            if n == 1 and halo_ready is not None:
                stream.wait_event(halo_ready)  # the boundary slabs read the halo
            call("dcb_conv_fwd", plan, float(alpha), _ptr(x0 + xoff), _ptr(filter.data_ptr()), float(beta),
                 _ptr(y0 + yoff), _stream_ptr(stream))

    def _make_plan(self, xd: NdDesc, yd: NdDesc, pads):
        nsd = self.nsd
        cd = ConvDesc()
        cd.nsd, cd.k, cd.c, cd.groups = nsd, self.K, self.C, 1
        cd.math_mode = self.be.options.math_mode
        for s in range(3):
            cd.filter[s], cd.pads[s], cd.strides[s], cd.dilations[s] = 1, 0, 1, 1
        for i in range(nsd):
            cd.filter[2 - i] = self.filter_dims[i]
            cd.pads[2 - i] = pads[i]
            cd.strides[2 - i] = self.strides[i]
            cd.dilations[2 - i] = self.dilations[i]
        plan = ctypes.c_void_p()
        call("dcb_conv_plan_create", ctypes.byref(cd), ctypes.byref(xd), ctypes.byref(yd), ctypes.byref(plan))
        return plan

    def _plan_of(self, which: int):
        return (self._plan_fwd, self._plan_bwd, self._plan_wgrad)[which]

    def kernel_kind(self, which: int) -> int:
        plan = self._plan_of(which)
        return _abi.lib().dcb_conv_plan_kernel_kind(plan, which)

    def kernel_variant(self, which: int) -> int:
        """dcb_conv_plan_kernel_variant: 0 fp32 CUDA-core, 1 / 2 tcgen05 row
        kernel (bulk-copy fed / register fed), 3 sweep, 4 multi-group sweep,
        5 tcgen05 backward filter."""
        return _abi.lib().dcb_conv_plan_kernel_variant(self._plan_of(which), which)

    # -- halo --
    def _clear_halos(self, t: Tensor, stream):
        for dim in range(self.nsd):
            d = t.dist
            if d.is_distributed(dim) and d.locale_shape[dim] > 1 and d.get_overlap(dim) > 0:
                t.clear_halo(dim, stream)

    def forward_exchange_halo(self, input: Tensor, stream=None):
        self.halo_xch_input.exchange(stream or self.be.stream)

    def backward_data_exchange_halo(self, d_output: Tensor, stream=None, skip_unpack=False):
        # d_output's halo cells at the tensor's boundary stand in for the padding
        self.halo_xch_d_output.exchange(stream or self.be.stream, skip_unpack=skip_unpack, clear_boundary=True)

    # -- compute --
    def forward(self, alpha, input: Tensor, filter: torch.Tensor, beta, output: Tensor,
                skip_halo_exchange=False, skip_chanfilt_comm=False, dump_profile=False, inference=False,
                statistics=None):
        """convolution.hpp:342-639 (no-overlap branch).

        ``statistics=(sums, sqsums)`` (two K-float device tensors, beta must be
        0) asks the convolution's epilogue for the per-filter sum and sum of
        squares of the output, i.e. what ``BatchNormalization.forward_stage1``
        would compute from ``output``.  Returns 1 when they were produced
        (pass ``statistics_ready=True`` to the batch-norm), else 0: the caller
        then runs stage 1 as usual."""
        if input.get_local_size() == 0 or output.get_local_size() == 0:
            return 0
        s = self.be.stream
        prof = self.be.options.enable_profiling
        if not skip_halo_exchange and getattr(self, "_ov", None) is not None:
            return self._forward_overlapped(alpha, input, filter, beta, output)
        if prof:  # the reference's range names (convolution.hpp:361-364, 420-423, 2695-2708)
            torch.cuda.nvtx.range_push("conv/forward")
        try:
            return self._forward(alpha, input, filter, beta, output, skip_halo_exchange, statistics, s, prof)
        finally:
            if prof:
                torch.cuda.nvtx.range_pop()

    def _forward(self, alpha, input, filter, beta, output, skip_halo_exchange, statistics, s, prof):
        if not skip_halo_exchange:
            if prof:
                torch.cuda.nvtx.range_push("conv/forward/exchange_halo")
            # Tensor::clear_halo + exchange (convolution.hpp:405-414, 327-340) in one
            # launch per half: the pack launch zeroes the boundary slabs
            self.halo_xch_input.exchange(s, clear_boundary=True)
            if prof:
                torch.cuda.nvtx.range_pop()
        if statistics is not None and float(beta) == 0.0 and input.is_split_root():
            st = _abi.lib().dcb_conv_fwd_stats(self._plan_fwd, float(alpha), _ptr(input.nd_ptr(self._x_lo)),
                                               _ptr(filter.data_ptr()), _ptr(output.get_base_ptr()),
                                               _ptr(statistics[0].data_ptr()), _ptr(statistics[1].data_ptr()),
                                               _stream_ptr(s))
            if st == _abi.OK:
                return 1
            if st != _abi.UNSUPPORTED:
                _abi.check(st, "dcb_conv_fwd_stats")
        call("dcb_conv_fwd", self._plan_fwd, float(alpha), _ptr(input.nd_ptr(self._x_lo)), _ptr(filter.data_ptr()),
             float(beta), _ptr(output.get_base_ptr()), _stream_ptr(s))
        return 0

    def backward_data(self, alpha, filter: torch.Tensor, d_output: Tensor, beta, d_input: Tensor,
                      skip_halo_exchange=False, skip_chanfilt_comm=False, dump_profile=False):
        """convolution.hpp:682-876."""
        if filter.numel() == 0 or d_output.get_local_size() == 0 or d_input.get_local_size() == 0:
            return 0
        s = self.be.stream
        if not skip_halo_exchange:
            self.backward_data_exchange_halo(d_output, s)
        call("dcb_conv_bwd_data", self._plan_bwd, float(alpha), _ptr(filter.data_ptr()),
             _ptr(d_output.get_buffer()), float(beta), _ptr(d_input.nd_ptr(self._dx_lo)), _stream_ptr(s))
        return 0

    def backward_filter(self, alpha, input: Tensor, d_output: Tensor, beta, d_filter: torch.Tensor, reduce=True,
                        skip_chanfilt_comm=False, dump_profile=False):
        """convolution.hpp:878-1107, then the all-reduce of the filter gradient
        over all ranks.  Only d_output's owned cells are read, so its halo is
        not cleared first (the reference clears it because cuDNN is handed the
        halo-extended tensor)."""
        s = self.be.stream
        if (input.get_local_size() == 0 or d_output.get_local_size() == 0 or d_filter.numel() == 0
                or not input.is_split_root()):
            _zero_on(s, d_filter)
        else:
            call("dcb_conv_bwd_filter", self._plan_wgrad, float(alpha), _ptr(input.nd_ptr(self._x_lo)),
                 _ptr(d_output.get_base_ptr()), float(beta), _ptr(d_filter.data_ptr()), _stream_ptr(s))
        if reduce:
            self.allreduce_gradients(d_filter)
        return 0

    def allreduce_gradients(self, g: torch.Tensor):
        self.be.allreducer.allreduce(g.data_ptr(), g.numel(), self.be.stream)

    def apply_bias(self, alpha, bias: torch.Tensor, beta, output: Tensor):
        """convolution.hpp:641-659."""
        if output.get_local_size() == 0:
            return 0
        yd = output.nd_desc()
        call("dcb_bias_fwd", float(alpha), _ptr(bias.data_ptr()), float(beta), ctypes.byref(yd),
             _ptr(output.get_base_ptr()), _stream_ptr(self.be.stream))
        return 0

    def backward_bias(self, alpha, d_output: Tensor, beta, bias_gradient: torch.Tensor, reduce=True):
        """convolution.hpp:1109-1142."""
        if d_output.get_local_size() == 0:
            _zero_on(self.be.stream, bias_gradient)
        else:
            yd = d_output.nd_desc()
            call("dcb_bias_bwd", float(alpha), ctypes.byref(yd), _ptr(d_output.get_base_ptr()), float(beta),
                 _ptr(bias_gradient.data_ptr()), _stream_ptr(self.be.stream))
        if reduce:
            self.allreduce_gradients(bias_gradient)
        return 0

    def wait(self):
        self.be.wait()

    def is_overlap_fwd_halo_exchange_enabled(self):
        return getattr(self, "_ov", None) is not None

    def is_overlap_bwd_halo_exchange_enabled(self):
        return False


# ---------------------------------------------------------------------------
# BatchNormalization
# ---------------------------------------------------------------------------
class BatchNormalization:
    """BatchNormalization<BackendDNNLib, float> (batchnorm.hpp:100-581).
    Statistics vectors are contiguous torch tensors of C floats; ``mean`` and
    ``var`` should be the two halves of one 2C tensor so their all-reduce
    fuses (batchnorm.hpp:191-211)."""

    def __init__(self, backend: BackendDNNLib, num_dims: int, decay: float, epsilon: float, global_stats: bool,
                 impl="PEER"):
        self.be, self.num_dims = backend, num_dims
        self.decay, self.epsilon, self.global_stats = float(decay), float(epsilon), bool(global_stats)
        self._plans = {}

    def __del__(self):
        try:
            for p in getattr(self, "_plans", {}).values():
                _abi.lib().dcb_bn_plan_destroy(p)
        except Exception:
            pass

    def _plan(self, t: Tensor):
        key = (tuple(t.local_shape), tuple(t.dist.overlap))
        if key not in self._plans:
            xd = t.nd_desc()
            p = ctypes.c_void_p()
            call("dcb_bn_plan_create", ctypes.byref(xd), ctypes.byref(p))
            self._plans[key] = p
        return self._plans[key]

    # forward
    def forward_stage1(self, input: Tensor, mean, var, is_training=True):
        if not is_training:
            return 0
        s = self.be.stream
        if input.get_local_size() == 0 or not input.is_split_root():
            _zero_on(s, mean, var)
            return 0
        call("dcb_bn_stats", self._plan(input), _ptr(input.get_base_ptr()), _ptr(mean.data_ptr()),
             _ptr(var.data_ptr()), _stream_ptr(s))
        return 0

    def _allreduce_pair(self, a, b, fn):
        n = a.numel()
        if a.data_ptr() + 4 * n == b.data_ptr():
            fn(a.data_ptr(), 2 * n)
        elif b.data_ptr() + 4 * n == a.data_ptr():
            fn(b.data_ptr(), 2 * n)
        else:
            fn(a.data_ptr(), n)
            fn(b.data_ptr(), n)

    def forward_allreduce(self, mean, var, is_training=True):
        if not is_training or not self.global_stats:
            return 0
        ar = self.be.allreducer
        self._allreduce_pair(mean, var, lambda p, n: ar.allreduce(p, n, self.be.stream))
        return 0

    def forward_stage2(self, input: Tensor, mean, var, running_mean, running_var, scale, bias, output: Tensor,
                       is_training=True, leaky_relu_slope=None):
        """``leaky_relu_slope``: also apply the LeakyReLU that follows the
        batch-norm, in the same pass over the tensor."""
        s = self.be.stream
        C = input.local_shape[-2]
        if is_training:
            stat_shape = input.shape if self.global_stats else input.local_shape
            nps = 1
            for v in stat_shape:
                nps *= v
            nps //= stat_shape[-2]
            call("dcb_bn_finalize", C, nps, self.decay, _ptr(mean.data_ptr()), _ptr(var.data_ptr()),
                 _ptr(running_mean.data_ptr()), _ptr(running_var.data_ptr()), _stream_ptr(s))
            m, v = mean, var
        else:
            m, v = running_mean, running_var
        if input.get_local_size() == 0:
            return 0
        xd, yd = input.nd_desc(), output.nd_desc()
        if leaky_relu_slope is not None:
            call("dcb_bn_apply_leaky_relu", ctypes.byref(xd), _ptr(input.get_base_ptr()), _ptr(m.data_ptr()),
                 _ptr(v.data_ptr()), _ptr(scale.data_ptr()), _ptr(bias.data_ptr()), self.epsilon,
                 float(leaky_relu_slope), ctypes.byref(yd), _ptr(output.get_base_ptr()), _stream_ptr(s))
            return 0
        call("dcb_bn_apply", ctypes.byref(xd), _ptr(input.get_base_ptr()), _ptr(m.data_ptr()), _ptr(v.data_ptr()),
             _ptr(scale.data_ptr()), _ptr(bias.data_ptr()), self.epsilon, ctypes.byref(yd),
             _ptr(output.get_base_ptr()), _stream_ptr(s))
        return 0

    def forward(self, input, mean, var, running_mean, running_var, scale, bias, output, is_training=True,
                statistics_ready=False):
        """``statistics_ready``: mean / var already hold this rank's sums and
        sums of squares (from ``Convolution.forward(..., statistics=...)``)."""
        if not statistics_ready:
            self.forward_stage1(input, mean, var, is_training)
        self.forward_allreduce(mean, var, is_training)
        self.forward_stage2(input, mean, var, running_mean, running_var, scale, bias, output, is_training)
        return 0

    # backward
    def backward_stage1(self, input: Tensor, d_output: Tensor, mean, var, scale, scale_gradient, bias_gradient,
                        mean_gradient, var_gradient):
        s = self.be.stream
        if input.get_local_size() == 0 or not input.is_split_root():
            _zero_on(s, scale_gradient, bias_gradient, mean_gradient, var_gradient)
            return 0
        dyd = d_output.nd_desc()
        call("dcb_bn_bwd_reduce", self._plan(input), _ptr(input.get_base_ptr()), ctypes.byref(dyd),
             _ptr(d_output.get_base_ptr()), _ptr(mean.data_ptr()), _ptr(var.data_ptr()), _ptr(scale.data_ptr()),
             self.epsilon, _ptr(scale_gradient.data_ptr()), _ptr(bias_gradient.data_ptr()),
             _ptr(mean_gradient.data_ptr()), _ptr(var_gradient.data_ptr()), _stream_ptr(s))
        return 0

    def backward_allreduce(self, scale_gradient, bias_gradient, mean_gradient, var_gradient,
                           skip_weights=False):
        """batchnorm.hpp:360-400: dmean||dvar when global statistics are on,
        then dscale, dbias."""
        ar = self.be.allreducer
        f = lambda p, n: ar.allreduce(p, n, self.be.stream)
        if self.global_stats:
            self._allreduce_pair(mean_gradient, var_gradient, f)
        if not skip_weights:
            self._allreduce_pair(scale_gradient, bias_gradient, f)
        return 0

    def backward_stage2(self, input: Tensor, d_output: Tensor, mean, var, scale, mean_gradient, var_gradient,
                        d_input: Tensor):
        if input.get_local_size() == 0:
            return 0
        stat_shape = input.shape if self.global_stats else input.local_shape
        nps = 1
        for v in stat_shape:
            nps *= v
        nps //= stat_shape[-2]
        xd, dyd, dxd = input.nd_desc(), d_output.nd_desc(), d_input.nd_desc()
        call("dcb_bn_bwd_apply", ctypes.byref(xd), _ptr(input.get_base_ptr()), ctypes.byref(dyd),
             _ptr(d_output.get_base_ptr()), _ptr(mean.data_ptr()), _ptr(var.data_ptr()), _ptr(scale.data_ptr()),
             _ptr(mean_gradient.data_ptr()), _ptr(var_gradient.data_ptr()), self.epsilon, nps, ctypes.byref(dxd),
             _ptr(d_input.get_base_ptr()), _stream_ptr(self.be.stream))
        return 0

    def backward(self, input, d_output, mean, var, scale, scale_gradient, bias_gradient, mean_gradient,
                 var_gradient, d_input):
        self.backward_stage1(input, d_output, mean, var, scale, scale_gradient, bias_gradient, mean_gradient,
                             var_gradient)
        self.backward_allreduce(scale_gradient, bias_gradient, mean_gradient, var_gradient)
        self.backward_stage2(input, d_output, mean, var, scale, mean_gradient, var_gradient, d_input)
        return 0


class Pooling:
    """Pooling<BackendDNNLib, float> (pooling.hpp:70-482): halo exchange of the
    input, pooling over the halo-extended shard, and in the backward pass the
    reverse exchange that adds the gradients a rank computed for its
    neighbours' cells to their owners (HaloExchangeAccumOp::SUM)."""

    def __init__(self, backend: BackendDNNLib, num_dims: int, halo_exchange_method="AL"):
        self.be = backend
        self.num_dims = num_dims
        self.nsd = num_dims - 2
        self.halo_xch_input = None
        self.halo_xch_d_input = None

    def setup(self, input: Tensor, output: Tensor, d_input: Tensor, d_output: Tensor, windows, pads, strides,
              mode: str, connect=True):
        """pooling.hpp:101-209; windows / pads / strides in reference order (W
        first), all dimensions equal as the reference demands."""
        nsd = self.nsd
        assert len(windows) == nsd and len(pads) == nsd and len(strides) == nsd
        assert len(set(windows)) == 1 and len(set(pads)) == 1 and len(set(strides)) == 1
        for w, p, st in zip(windows, pads, strides):
            if w % 2:
                stencil = (w - 1) // 2
                assert p in (0, stencil) and st in (1, stencil + 1)
            else:
                assert w == st and p == 0
        assert input.dist == d_input.dist
        assert mode in _abi.POOL_MODES
        self.mode = mode
        self.input, self.output, self.d_input, self.d_output = input, output, d_input, d_output
        use_padding = pads[0] != 0
        self.halo_fwd_send, self.halo_bwd_send, self.halo_fwd_recv, self.halo_bwd_recv = get_halo_sizes(
            input, list(windows), list(strides), [1] * nsd, use_padding)
        # where a dimension is split the halo stands in for the padding (pooling.hpp:189-194)
        eff_pads = [0 if input.dist.split_shape[i] > 1 else pads[i] for i in range(nsd)]
        self._lo, self._hi = self.halo_bwd_recv[:nsd], self.halo_fwd_recv[:nsd]
        self._pd = _abi.PoolDesc()
        self._pd.nsd, self._pd.mode = nsd, _abi.POOL_MODES[mode]
        for s_ in range(3):
            self._pd.window[s_], self._pd.pads[s_], self._pd.strides[s_] = 1, 0, 1
        for i in range(nsd):
            self._pd.window[2 - i], self._pd.pads[2 - i], self._pd.strides[2 - i] = windows[i], eff_pads[i], strides[i]
            # The halo of a rank at the boundary of the global tensor stands for
            # padding.  The reference leaves it to cuDNN as zero data; here the
            # kernel is told, so that MAX and AVERAGE_NO_PAD agree with one rank.
            split = input.dist.split_shape[i] > 1
            first, last = input.split_idx[i] == 0, input.split_idx[i] == input.dist.split_shape[i] - 1
            self._pd.outside_lo[2 - i] = self._lo[i] if split and first else 0
            self._pd.outside_hi[2 - i] = self._hi[i] if split and last else 0
        self.halo_xch_input = HaloExchange(input)
        self.halo_xch_d_input = HaloExchange(d_input)
        if connect:
            self.halo_xch_input.setup()
            self.halo_xch_d_input.setup()
        # index workspace of the backward pass (one byte per output cell, MAX
        # only); allocated by the first backward call, when the tensors have memory
        self._ws = None

    def _halo_dims(self, t: Tensor):
        d = t.dist
        return [i for i in range(self.nsd) if d.is_distributed(i) and d.locale_shape[i] > 1 and d.get_overlap(i) > 0]

    def forward(self, alpha, input: Tensor, beta, output: Tensor, training=True, skip_halo_exchange=False):
        """pooling.hpp:212-244.  Ranks with an empty output still take part in
        the exchange."""
        s = self.be.stream
        if not skip_halo_exchange:
            for dim in self._halo_dims(input):
                input.clear_halo(dim, s)
            self.halo_xch_input.exchange(s)
        if output.get_local_size() == 0:
            return 0
        xd, yd = input.nd_desc(self._lo, self._hi), output.nd_desc()
        call("dcb_pool_fwd", ctypes.byref(self._pd), ctypes.byref(xd), ctypes.byref(yd), float(alpha),
             _ptr(input.nd_ptr(self._lo)), float(beta), _ptr(output.get_base_ptr()), _stream_ptr(s))
        return 0

    def backward(self, alpha, output: Tensor, d_output: Tensor, input: Tensor, beta, d_input: Tensor,
                 skip_halo_exchange=False):
        """pooling.hpp:246-283: gradients for the halo cells are computed here
        and travel back with SUM.  The exchange moves whole halos, so the cells
        of d_input's halo that no local window reaches are cleared first."""
        if d_input.get_local_size() == 0:
            return 0
        s = self.be.stream
        for dim in self._halo_dims(d_input):
            d_input.clear_halo(dim, s)
        if d_output.get_local_size() > 0:
            xd, yd = input.nd_desc(self._lo, self._hi), output.nd_desc()
            dxd, dyd = d_input.nd_desc(self._lo, self._hi), d_output.nd_desc()
            assert list(xd.strides) == list(dxd.strides) and list(yd.strides) == list(dyd.strides)
            if self._ws is None:
                need = _abi.lib().dcb_pool_bwd_workspace_bytes(ctypes.byref(self._pd), ctypes.byref(xd),
                                                               ctypes.byref(yd))
                self._ws = torch.empty(max(need, 0), dtype=torch.uint8, device=d_input.buffer.device)
            call("dcb_pool_bwd", ctypes.byref(self._pd), ctypes.byref(xd), ctypes.byref(yd), float(alpha),
                 _ptr(output.get_base_ptr()), _ptr(d_output.get_base_ptr()), _ptr(input.nd_ptr(self._lo)),
                 float(beta), _ptr(d_input.nd_ptr(self._lo)),
                 _ptr(self._ws.data_ptr() if self._ws.numel() else 0), self._ws.numel(), _stream_ptr(s))
        if not skip_halo_exchange:
            self.halo_xch_d_input.exchange(s, is_reverse=True, op="SUM")
        return 0

    def wait(self):
        self.be.wait()


class LeakyReLU:
    """LeakyReLU<BackendDNNLib> (leaky_relu.hpp, leaky_relu.cu:14-41)."""

    def __init__(self, backend: BackendDNNLib):
        self.be = backend

    def forward(self, input: Tensor, negative_slope: float, output: Tensor):
        if input.get_local_size() == 0:
            return 0
        xd, yd = input.nd_desc(), output.nd_desc()
        call("dcb_leaky_relu_fwd", ctypes.byref(xd), _ptr(input.get_base_ptr()), float(negative_slope),
             ctypes.byref(yd), _ptr(output.get_base_ptr()), _stream_ptr(self.be.stream))
        return 0

    def backward(self, input: Tensor, d_output: Tensor, negative_slope: float, d_input: Tensor):
        if input.get_local_size() == 0:
            return 0
        xd, dyd, dxd = input.nd_desc(), d_output.nd_desc(), d_input.nd_desc()
        call("dcb_leaky_relu_bwd", ctypes.byref(xd), _ptr(input.get_base_ptr()), ctypes.byref(dyd),
             _ptr(d_output.get_base_ptr()), float(negative_slope), ctypes.byref(dxd), _ptr(d_input.get_base_ptr()),
             _stream_ptr(self.be.stream))
        return 0
