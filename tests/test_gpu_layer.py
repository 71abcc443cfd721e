"""The whole path -- halo exchange, convolution forward / backward-data /
backward-filter on the halo-extended shard, distributed batch-norm -- on
emulated ranks, against the single-domain oracle and, for the 2-D case, against
outputs of the reference's own ref::Backend."""
import os

import numpy as np
import pytest
import torch

import dihydrogen_b200 as dc
from dihydrogen_b200 import _abi
from oracle import oracle as O

import emu
from conftest import GOLDEN

pytestmark = pytest.mark.gpu


class Layer:
    """conv -> BN on n emulated ranks, phase-ordered."""

    def __init__(self, shape, locale, K, f, strides, pad, mode=_abi.MATH_FP32):
        self.nd = len(shape)
        nsd = self.nd - 2
        self.n = int(np.prod(locale))
        self.bes = emu.make_backends(self.n, options=dc.Options(math_mode=mode))
        dil = [1] * nsd
        self.K, self.C = K, shape[-2]
        fshape = list(f) + [self.C, K]
        pads = [(ff - 1) // 2 if pad else 0 for ff in f]
        self.x, self.dx, self.y, self.dy, self.z, self.dz, self.convs, self.bns = ([] for _ in range(8))
        w0 = torch.zeros((K, self.C, *reversed(f)), device="cuda")
        for be in self.bes:
            x = dc.create_input_tensor(shape, locale, f, strides, dil, be.locale)
            y = dc.create_convolution_output_tensor(x, fshape, strides, pads, dil)
            dy = dc.create_convolution_d_output_tensor(y, fshape, dil)
            dx = dc.create_d_input_tensor(x)
            z = dc.Tensor(y.shape, be.locale, y.dist, y._local_of)
            dz = dc.Tensor(y.shape, be.locale, y.dist, y._local_of)
            for t in (x, y, dy, dx, z, dz):
                t.allocate()
            conv = dc.Convolution(be, self.nd)
            conv.setup(x, w0, y, dx, None, dy, pads, strides, dil, connect=False)
            self.x.append(x), self.dx.append(dx), self.y.append(y), self.dy.append(dy)
            self.z.append(z), self.dz.append(dz), self.convs.append(conv)
            self.bns.append(dc.BatchNormalization(be, self.nd, 0.9, 1e-5, True))
        emu.connect_halo([c.halo_xch_input for c in self.convs])
        emu.connect_halo([c.halo_xch_d_output for c in self.convs])
        self.out_shape = self.y[0].shape

    def forward(self, gx, w, scale, bias, fused_stats=False):
        K = self.K
        self.w = torch.from_numpy(w).cuda()
        for x in self.x:
            if gx is not None:  # None: the owned cells were written by the layer before
                x.buffer.fill_(float("nan"))  # halos must be produced by the exchange
                src = tuple(slice(o, o + l) for o, l in reversed(list(zip(x.offset, x.local_shape))))
                x.owned().copy_(torch.from_numpy(np.ascontiguousarray(gx[src])))
            for d in range(self.nd - 2):
                x.clear_halo(d)
        emu.exchange_all([c.halo_xch_input for c in self.convs])
        self.stats = [torch.zeros(2 * K, device="cuda") for _ in self.bes]
        self.fused = []
        for c, x, y, st in zip(self.convs, self.x, self.y, self.stats):
            self.fused.append(c.forward(1.0, x, self.w, 0.0, y, skip_halo_exchange=True,
                                        statistics=(st[:K], st[K:]) if fused_stats else None))
        self.rm = [torch.zeros(K, device="cuda") for _ in self.bes]
        self.rv = [torch.ones(K, device="cuda") for _ in self.bes]
        self.scale, self.bias = torch.from_numpy(scale).cuda(), torch.from_numpy(bias).cuda()
        for bn, y, st, got in zip(self.bns, self.y, self.stats, self.fused):
            if not got:  # the conv epilogue did not deliver them
                bn.forward_stage1(y, st[:K], st[K:], True)
        emu.allreduce_all(self.bes, self.stats)
        for bn, y, z, st, rm, rv in zip(self.bns, self.y, self.z, self.stats, self.rm, self.rv):
            bn.forward_stage2(y, st[:K], st[K:], rm, rv, self.scale, self.bias, z, True)
        torch.cuda.synchronize()

    def backward(self, gdz):
        K = self.K
        for dz in self.dz:
            if gdz is not None:  # None: filled by the layer after this one
                emu.scatter_owned(dz, gdz)
        ga = [torch.zeros(2 * K, device="cuda") for _ in self.bes]
        gb = [torch.zeros(2 * K, device="cuda") for _ in self.bes]
        for bn, y, dz, st, a, b in zip(self.bns, self.y, self.dz, self.stats, ga, gb):
            bn.backward_stage1(y, dz, st[:K], st[K:], self.scale, b[:K], b[K:], a[:K], a[K:])
        emu.allreduce_all(self.bes, ga)
        emu.allreduce_all(self.bes, gb)
        for bn, y, dz, dy, st, a in zip(self.bns, self.y, self.dz, self.dy, self.stats, ga):
            dy.buffer.fill_(float("nan"))
            bn.backward_stage2(y, dz, st[:K], st[K:], self.scale, a[:K], a[K:], dy)
        self.dscale, self.dbias = gb[0][:K], gb[0][K:]
        self.dmean, self.dvar = ga[0][:K], ga[0][K:]
        # backward filter first (it reads dy's owned cells only: the halo is still
        # poisoned here), then exchange, then backward data -- the driver's order
        # (distconv_benchmark.cpp:569-589)
        self.dw = [torch.zeros_like(self.w) for _ in self.bes]
        for c, x, dy, dw in zip(self.convs, self.x, self.dy, self.dw):
            c.backward_filter(1.0, x, dy, 0.0, dw, reduce=False)
        emu.allreduce_all(self.bes, self.dw)
        # the halo cells at the tensor's boundary stand in for the padding (the
        # exchange of Convolution.backward_data clears them in its pack launches)
        for dy in self.dy:
            for d in range(self.nd - 2):
                dy.clear_halo(d)
        emu.exchange_all([c.halo_xch_d_output for c in self.convs])
        for c, dy, dx in zip(self.convs, self.dy, self.dx):
            c.backward_data(1.0, self.w, dy, 0.0, dx, skip_halo_exchange=True)
        torch.cuda.synchronize()


def oracle_layer(gx, w, scale, bias, gdz, pads, strides):
    K = w.shape[0]
    y = O.conv_fwd(gx, w, pads, strides)
    s, q = O.bn_sums(y)
    nps = y.size // K
    m, v, rm, rv = O.bn_sums_to_statistics(s, q, nps, 0.9, np.zeros(K), np.ones(K))
    z = O.bn_normalize(y, m, v, scale, bias, 1e-5)
    dsc, dbi, dme, dva = O.bn_backprop1(y, gdz, m, v, scale, 1e-5)
    dy = O.bn_backprop2(y, gdz, m, v, scale, np.float32(dme), np.float32(dva), 1e-5, nps)
    dw = O.conv_bwd_filter(gx, dy, w.shape[2:], pads, strides)
    dx = np.zeros_like(gx)
    O.conv_bwd_data(w, dy, dx, pads, strides)
    return dict(y=y, z=z, mean=m, var=v, dscale=dsc, dbias=dbi, dy=dy, dw=dw, dx=dx)


def check_layer_stages(L, gx, w, scale, bias, gdz, pads, strides, tol=1e-5, what=""):
    """emu.check_stages on the tensors of an emulated-rank Layer: every stage
    against the oracle fed with the GPU's own previous stage, at 1e-5."""
    K = L.K
    osh = tuple(reversed(L.out_shape))
    for st in L.stats:
        assert torch.equal(st, L.stats[0])  # identical bits on every rank
    bwd = None
    if gdz is not None:
        for dw in L.dw:
            assert torch.equal(dw, L.dw[0])  # all ranks hold the same reduced gradient
        bwd = dict(gdz=gdz, dscale=L.dscale.cpu().numpy(), dbias=L.dbias.cpu().numpy(),
                   dmean=L.dmean.cpu().numpy(), dvar=L.dvar.cpu().numpy(), dy=emu.gather_owned(L.dy, osh),
                   dw=L.dw[0].cpu().numpy(), dx=emu.gather_owned(L.dx, gx.shape))
    emu.check_stages(K, gx, w, scale, bias, pads, strides, emu.gather_owned(L.y, osh),
                     L.stats[0][:K].cpu().numpy(), L.stats[0][K:].cpu().numpy(), emu.gather_owned(L.z, osh),
                     bwd, tol, what)


LAYERS = [
    # shape (W..N), locale, K, filter (W..), strides, name
    ([32, 32, 8, 2], [1, 2, 1, 1], 8, [3, 3], [1, 1]),                 # BASELINE config 1 geometry, reduced
    ([24, 20, 6, 2], [2, 2, 1, 1], 5, [5, 5], [1, 1]),                 # config 4 family: 5x5, H x W partition
    ([20, 16, 12, 4, 1], [1, 1, 4, 1, 1], 16, [3, 3, 3], [1, 1, 1]),   # config 2: D partition
    ([16, 16, 16, 4, 1], [2, 2, 2, 1, 1], 16, [3, 3, 3], [1, 1, 1]),   # config 3 layer 1: 2x2x2
    ([16, 16, 16, 8, 1], [2, 2, 2, 1, 1], 8, [3, 3, 3], [2, 2, 2]),    # config 3 layer 2: stride 2
    ([18, 14, 13, 3, 2], [1, 2, 3, 1, 1], 4, [3, 3, 3], [1, 1, 1]),    # uneven split
]


@pytest.mark.parametrize("mode", [_abi.MATH_FP32_SIMT, _abi.MATH_FP32])
@pytest.mark.parametrize("shape,locale,K,f,strides", LAYERS)
def test_layer_matches_single_domain_oracle(shape, locale, K, f, strides, mode):
    rng = np.random.default_rng(11)
    C = shape[-2]
    gx = rng.normal(0, 1, tuple(reversed(shape))).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / (C * np.prod(f))), (K, C, *reversed(f))).astype(np.float32)
    scale = rng.uniform(0.5, 1.5, K).astype(np.float32)
    bias = rng.normal(0, 0.5, K).astype(np.float32)
    L = Layer(shape, locale, K, f, strides, pad=1, mode=mode)
    gdz = rng.normal(0, 1, tuple(reversed(L.out_shape))).astype(np.float32)
    L.forward(gx, w, scale, bias)
    L.backward(gdz)
    pads = [(ff - 1) // 2 for ff in reversed(f)]
    check_layer_stages(L, gx, w, scale, bias, gdz, pads, list(reversed(strides)))


def test_w_partitioned_shards_of_the_2x2x2_grid_take_the_tensor_core_kernels():
    """BASELINE configs[2] layer 1 on its own 2 x 2 x 2 grid, reduced extents:
    every shard is partitioned along W, so its rows are local + 2 halo cells
    = 134 floats (2 mod 4) and only the padded row pitch lets the bulk-copy
    fed tcgen05 kernels take them.  All three passes must run on tensor cores
    (forward: sweep kernel, backward data: sweep / multi-group sweep, backward
    filter: the tcgen05 kernel) and meet the 1e-5 contract stage by stage."""
    shape, locale, K, f, strides = [264, 24, 12, 4, 1], [2, 2, 2, 1, 1], 16, [3, 3, 3], [1, 1, 1]
    rng = np.random.default_rng(17)
    gx = rng.uniform(0, 1, tuple(reversed(shape))).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / (4 * 27)), (K, 4, 3, 3, 3)).astype(np.float32)
    scale = rng.uniform(0.5, 1.5, K).astype(np.float32)
    bias = rng.normal(0, 0.5, K).astype(np.float32)
    L = Layer(shape, locale, K, f, strides, pad=1)
    for x, dy in zip(L.x, L.dy):
        assert x.get_local_real_shape()[0] == 134 and x.get_pitch() == 140
        assert dy.get_pitch() == 140 and x.owned().data_ptr() % 16 == 0
    for c in L.convs:
        assert [c.kernel_kind(i) for i in range(3)] == [1, 1, 1]
        assert c.kernel_variant(0) == 3 and c.kernel_variant(1) in (3, 4) and c.kernel_variant(2) == 5
    gdz = rng.normal(0, 1, tuple(reversed(L.out_shape))).astype(np.float32)
    L.forward(gx, w, scale, bias, fused_stats=True)
    assert all(L.fused), "the sweep kernel delivers the statistics on W-partitioned shards too"
    L.backward(gdz)
    for c in L.convs:
        assert _abi.lib().dcb_conv_plan_status(c._plan_fwd, None) == _abi.OK
        assert _abi.lib().dcb_conv_plan_status(c._plan_bwd, None) == _abi.OK
        assert _abi.lib().dcb_conv_plan_status(c._plan_wgrad, None) == _abi.OK
    check_layer_stages(L, gx, w, scale, bias, gdz, [1, 1, 1], [1, 1, 1])


def test_config1_against_reference_backend_outputs():
    """2-D layer split along H over 2 ranks: conv outputs and gradients equal
    what Convolution<ref::Backend> produced for the same seeded inputs."""
    z = np.load(os.path.join(GOLDEN, "conv_cfg1_lite_h2.npz"))
    x, w, dy = z["x"], z["w"], z["dy"]
    N, C, H, W = x.shape
    K = w.shape[0]
    L = Layer([W, H, C, N], [1, 2, 1, 1], K, [3, 3], [1, 1], pad=1)
    L.forward(x, w, np.ones(K, np.float32), np.zeros(K, np.float32))
    emu.assert_close(emu.gather_owned(L.y, z["y"].shape), z["y"], 2e-5, "y vs ref::Backend")
    # backward conv on the reference's dy (bypassing BN)
    for t in L.dy:
        t.buffer.zero_()
        src = tuple(slice(o, o + l) for o, l in reversed(list(zip(t.offset, t.local_shape))))
        t.owned().copy_(torch.from_numpy(np.ascontiguousarray(dy[src])))
    dws = [torch.zeros_like(L.w) for _ in L.bes]
    for c, xt, dyt, dw in zip(L.convs, L.x, L.dy, dws):
        c.backward_filter(1.0, xt, dyt, 0.0, dw, reduce=False)
    emu.allreduce_all(L.bes, dws)
    emu.exchange_all([c.halo_xch_d_output for c in L.convs])
    for c, dyt, dx in zip(L.convs, L.dy, L.dx):
        c.backward_data(1.0, L.w, dyt, 0.0, dx, skip_halo_exchange=True)
    torch.cuda.synchronize()
    emu.assert_close(dws[0].cpu().numpy(), z["dw"], 2e-5, "dw vs ref::Backend")
    emu.assert_close(emu.gather_owned(L.dx, x.shape), z["dx"], 2e-5, "dx vs ref::Backend")


@pytest.mark.parametrize("shape,locale", [([32, 16, 12, 4, 1], [1, 1, 2, 1, 1]), ([24, 20, 9, 4, 2], [1, 1, 3, 1, 1])])
def test_layer_with_statistics_from_the_conv_epilogue(shape, locale):
    """D-partitioned layers whose shards the sweep kernel takes: the BN
    statistics come out of the convolution's epilogue on every rank and the
    normalised output still matches the single-domain oracle."""
    K, f, strides = 16, [3, 3, 3], [1, 1, 1]
    rng = np.random.default_rng(5)
    C = shape[-2]
    gx = rng.normal(0.2, 1, tuple(reversed(shape))).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / (C * 27)), (K, C, 3, 3, 3)).astype(np.float32)
    scale = rng.uniform(0.5, 1.5, K).astype(np.float32)
    bias = rng.normal(0, 0.5, K).astype(np.float32)
    L = Layer(shape, locale, K, f, strides, pad=1)
    L.forward(gx, w, scale, bias, fused_stats=True)
    assert all(L.fused), "the sweep kernel should have produced the statistics"
    check_layer_stages(L, gx, w, scale, bias, None, [1] * 3, [1] * 3)


@pytest.mark.parametrize("shape,locale,K,f", [
    ([20, 16, 12, 4, 1], [1, 1, 4, 1, 1], 16, [3, 3, 3]),   # D split over 4: two inner ranks with two boundary slabs
    ([24, 20, 3, 2], [1, 2, 1, 1], 5, [5, 5]),              # 2-D, H split, halo of 2
    ([24, 16, 6, 3, 2], [2, 1, 1, 1, 1], 8, [3, 3, 3]),     # W split: the slabs are column ranges
])
def test_overlap_regions_equal_the_whole_convolution(shape, locale, K, f):
    """Options.overlap_halo_exchange: the interior and boundary slabs together
    give the convolution of the whole shard (the hand-offs between the halo
    exchange and the slabs are exercised across processes in mp_worker.py)."""
    nd, nsd = len(shape), len(shape) - 2
    n = int(np.prod(locale))
    C = shape[-2]
    rng = np.random.default_rng(21)
    gx = rng.normal(size=tuple(reversed(shape))).astype(np.float32)
    w = rng.normal(0, 0.1, (K, C, *reversed(f))).astype(np.float32)
    wt = torch.from_numpy(w).cuda()
    pads, ones = [(ff - 1) // 2 for ff in f], [1] * nsd
    bes = emu.make_backends(n, options=dc.Options(overlap_halo_exchange=True))
    xs, ys, convs = [], [], []
    for be in bes:
        x = dc.create_input_tensor(shape, locale, f, ones, ones, be.locale)
        y = dc.create_convolution_output_tensor(x, list(f) + [C, K], ones, pads, ones)
        emu.scatter_owned(x, gx)
        y.allocate()
        y.buffer.fill_(float("nan"))
        conv = dc.Convolution(be, nd)
        conv.setup(x, wt, y, None, None, None, pads, ones, ones, connect=False)
        xs.append(x), ys.append(y), convs.append(conv)
    emu.connect_halo([c.halo_xch_input for c in convs])
    assert all(c.is_overlap_fwd_halo_exchange_enabled() for c in convs)
    assert sorted(len(c._ov[1]) for c in convs)[-1] == (3 if n > 2 else 2)
    emu.exchange_all([c.halo_xch_input for c in convs])
    for c, x, y in zip(convs, xs, ys):
        c.forward_regions(1.0, x, wt, 0.0, y, torch.cuda.current_stream())
    torch.cuda.synchronize()
    ref = O.conv_fwd(gx, w, list(reversed(pads)), list(reversed(ones)))
    emu.assert_close(emu.gather_owned(ys, ref.shape), ref, 1e-5, "y")


def _leaky(a, slope):
    return np.where(a > 0, a, slope * a).astype(np.float32)


def test_config3_two_layer_chain_forward_and_backward():
    """BASELINE configs[2], reduced: conv(4->16, 3^3, s1) -> BN -> LeakyReLU(0.01)
    -> conv(16->32, 3^3, s2) -> BN on a 2 x 2 x 2 grid, forward and backward,
    against the same chain on the unpartitioned tensor."""
    locale, f, slope = [2, 2, 2, 1, 1], [3, 3, 3], 0.01
    rng = np.random.default_rng(33)
    gx = rng.uniform(0, 1, (1, 4, 16, 16, 16)).astype(np.float32)
    w1 = rng.normal(0, np.sqrt(2.0 / (4 * 27)), (16, 4, 3, 3, 3)).astype(np.float32)
    w2 = rng.normal(0, np.sqrt(2.0 / (16 * 27)), (32, 16, 3, 3, 3)).astype(np.float32)
    s1, b1 = rng.uniform(0.5, 1.5, 16).astype(np.float32), rng.normal(0, 0.5, 16).astype(np.float32)
    s2, b2 = rng.uniform(0.5, 1.5, 32).astype(np.float32), rng.normal(0, 0.5, 32).astype(np.float32)
    L1 = Layer([16, 16, 16, 4, 1], locale, 16, f, [1, 1, 1], pad=1)
    L2 = Layer([16, 16, 16, 16, 1], locale, 32, f, [2, 2, 2], pad=1)
    gdz = rng.normal(0, 1, tuple(reversed(L2.out_shape))).astype(np.float32)
    relus = [dc.LeakyReLU(be) for be in L1.bes]
    # forward
    L1.forward(gx, w1, s1, b1)
    for lr, z, x2 in zip(relus, L1.z, L2.x):
        x2.buffer.fill_(float("nan"))
        lr.forward(z, slope, x2)  # into the halo-extended input of layer 2
    L2.forward(None, w2, s2, b2)
    # backward
    L2.backward(gdz)
    for lr, z, dx2, dz1 in zip(relus, L1.z, L2.dx, L1.dz):
        dz1.allocate()
        lr.backward(z, dx2, slope, dz1)
    L1.backward(None)
    # the same chain on one domain, stage by stage: every stage is checked
    # against the oracle fed with what the GPU produced for the stage before
    p, one, two = [1, 1, 1], [1, 1, 1], [2, 2, 2]
    z1 = emu.gather_owned(L1.z, (1, 16, 16, 16, 16))
    a1 = emu.gather_owned(L2.x, (1, 16, 16, 16, 16))
    assert np.array_equal(a1, _leaky(z1, slope))  # the activation is exact
    check_layer_stages(L2, a1, w2, s2, b2, gdz, p, two, what="layer 2 ")
    dx2 = emu.gather_owned(L2.dx, a1.shape)
    dz1 = emu.gather_owned(L1.dz, a1.shape)
    assert np.array_equal(dz1, np.where(z1 > 0, dx2, np.float32(slope) * dx2).astype(np.float32))
    check_layer_stages(L1, gx, w1, s1, b1, dz1, p, one, what="layer 1 ")
