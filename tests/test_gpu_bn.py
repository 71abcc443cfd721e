"""Batch-norm kernels against the oracle (fp32, 1e-5 relative)."""
import numpy as np
import pytest
import torch

import dihydrogen_b200 as dc
from oracle import oracle as O

import emu

pytestmark = pytest.mark.gpu

TOL = 1e-5

# shape (W..N), locale, overlap: dense, D-halo (contiguous planes), H/W halos
# (strided rows), odd extents (scalar path)
CASES = [
    ([32, 16, 8, 4, 2], [1, 1, 1, 1, 1], [0, 0, 0, 0, 0]),
    ([32, 16, 8, 4, 2], [1, 1, 2, 1, 1], [0, 0, 1, 0, 0]),
    ([32, 16, 8, 4, 1], [2, 2, 2, 1, 1], [1, 1, 1, 0, 0]),
    ([33, 7, 5, 3, 2], [1, 1, 1, 1, 1], [0, 0, 0, 0, 0]),
    ([34, 9, 6, 2], [1, 2, 1, 1], [0, 2, 0, 0]),
    ([130, 129, 3, 1], [1, 1, 1, 1], [0, 0, 0, 0]),
    ([64, 64, 64, 16, 1], [1, 1, 1, 1, 1], [0, 0, 0, 0, 0]),
    # W halo: padded rows, a unit of the kernels packs several rows (16 + 16 + 5 of a plane's 37)
    ([512, 37, 3, 4, 1], [2, 1, 1, 1, 1], [1, 0, 0, 0, 0]),
    ([32, 50, 3, 2, 1], [2, 1, 1, 1, 1], [1, 0, 0, 0, 0]),
]


def _rank0(shape, locale, overlap):
    n = int(np.prod(locale))
    return dc.Tensor(shape, dc.Locale(0, n), dc.Distribution.make_overlapped_distribution(locale, overlap))


@pytest.mark.parametrize("shape,locale,overlap", CASES)
def test_bn_forward_backward_local(shape, locale, overlap):
    rng = np.random.default_rng(3)
    be = dc.BackendDNNLib(dc.Locale(0, 1))
    x_t, y_t, dy_t, dx_t = (_rank0(shape, locale, overlap) for _ in range(4))
    real = x_t.np_real_shape()
    C = shape[-2]
    xb = rng.normal(0.3, 1.5, real).astype(np.float32)
    dyb = rng.normal(0, 1, real).astype(np.float32)
    emu.upload(x_t, xb)
    emu.upload(dy_t, dyb)
    y_t.allocate()
    dx_t.allocate()
    own = O.Shard(shape, locale, overlap, 0).owned_slices()
    x, dy = xb[own], dyb[own]

    bn = dc.BatchNormalization(be, len(shape), decay=0.9, epsilon=1e-5, global_stats=False)
    stats = torch.zeros(2 * C, device="cuda")
    mean, var = stats[:C], stats[C:]
    rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    scale = torch.from_numpy(rng.uniform(0.5, 1.5, C).astype(np.float32)).cuda()
    bias = torch.from_numpy(rng.normal(0, 1, C).astype(np.float32)).cuda()

    bn.forward_stage1(x_t, mean, var, True)
    s, q = O.bn_sums(x)
    emu.assert_close(mean.cpu().numpy(), s, TOL, "sums")
    emu.assert_close(var.cpu().numpy(), q, TOL, "sqsums")
    bn.forward_stage2(x_t, mean, var, rm, rv, scale, bias, y_t, True)
    nps = x.size // C
    m_ref, v_ref, rm_ref, rv_ref = O.bn_sums_to_statistics(s, q, nps, 0.9, np.zeros(C), np.ones(C))
    emu.assert_close(mean.cpu().numpy(), m_ref, TOL, "mean")
    emu.assert_close(var.cpu().numpy(), v_ref, 2e-5, "var")
    emu.assert_close(rm.cpu().numpy(), rm_ref, TOL, "running_mean")
    emu.assert_close(rv.cpu().numpy(), rv_ref, TOL, "running_var")
    # apply is checked with the GPU's own statistics so only its arithmetic is compared
    m_g, v_g = mean.cpu().numpy(), var.cpu().numpy()
    y_ref = O.bn_normalize(x, m_g, v_g, scale.cpu().numpy(), bias.cpu().numpy(), 1e-5)
    emu.assert_close(y_t.owned().cpu().numpy(), y_ref, TOL, "y")
    # halo cells of the output are untouched
    mask = np.ones(real, bool)
    mask[own] = False
    assert not y_t.buffer.cpu().numpy()[mask].any()

    grads = [torch.zeros(C, device="cuda") for _ in range(4)]
    dscale, dbias, dmean, dvar = grads
    bn.backward_stage1(x_t, dy_t, mean, var, scale, dscale, dbias, dmean, dvar)
    ref = O.bn_backprop1(x, dy, m_g, v_g, scale.cpu().numpy(), 1e-5)
    for g, r, nme in zip(grads, ref, ("dscale", "dbias", "dmean", "dvar")):
        emu.assert_close(g.cpu().numpy(), r, 2e-5, nme)
    bn.backward_stage2(x_t, dy_t, mean, var, scale, dmean, dvar, dx_t)
    dx_ref = O.bn_backprop2(x, dy, m_g, v_g, scale.cpu().numpy(), dmean.cpu().numpy(), dvar.cpu().numpy(), 1e-5, nps)
    emu.assert_close(dx_t.owned().cpu().numpy(), dx_ref, TOL, "dx")


def test_bn_stats_are_reproducible():
    """Fixed-order two-stage reduction: identical bits run to run."""
    shape = [64, 64, 32, 8, 1]
    t = _rank0(shape, [1] * 5, [0] * 5)
    emu.upload(t, np.random.default_rng(0).normal(size=t.np_real_shape()).astype(np.float32))
    be = dc.BackendDNNLib(dc.Locale(0, 1))
    bn = dc.BatchNormalization(be, 5, 0.9, 1e-5, False)
    outs = []
    for _ in range(3):
        st = torch.zeros(16, device="cuda")
        bn.forward_stage1(t, st[:8], st[8:], True)
        outs.append(st.cpu().numpy().copy())
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])


@pytest.mark.parametrize("locale", [[1, 1, 2, 1, 1], [2, 2, 2, 1, 1]])
def test_bn_global_stats_emulated_ranks(locale):
    """Distributed BN == single-rank BN (the reference's own criterion,
    legacy/tests/dnn_backend/test_cudnn_util.sh.in:387-425): per-channel sums
    all-reduced across the spatial partition."""
    shape = [16, 12, 10, 4, 2]
    C = 4
    rng = np.random.default_rng(5)
    g = rng.normal(0.1, 2.0, tuple(reversed(shape))).astype(np.float32)
    gdy = rng.normal(0, 1, g.shape).astype(np.float32)
    n = int(np.prod(locale))
    bes = emu.make_backends(n)
    dist = dc.Distribution.make_distribution(locale)
    xs, ys, dys, dxs = ([dc.Tensor(shape, b.locale, dist) for b in bes] for _ in range(4))
    for x, dy, y, dx in zip(xs, dys, ys, dxs):
        emu.scatter_owned(x, g)
        emu.scatter_owned(dy, gdy)
        y.allocate()
        dx.allocate()
    bns = [dc.BatchNormalization(b, 5, 0.9, 1e-5, True) for b in bes]
    stats = [torch.zeros(2 * C, device="cuda") for _ in bes]
    rms = [torch.zeros(C, device="cuda") for _ in bes]
    rvs = [torch.ones(C, device="cuda") for _ in bes]
    scale = torch.from_numpy(rng.uniform(0.5, 1.5, C).astype(np.float32)).cuda()
    bias = torch.from_numpy(rng.normal(0, 1, C).astype(np.float32)).cuda()
    for bn, x, st in zip(bns, xs, stats):
        bn.forward_stage1(x, st[:C], st[C:], True)
    emu.allreduce_all(bes, stats)
    for bn, x, y, st, rm, rv in zip(bns, xs, ys, stats, rms, rvs):
        bn.forward_stage2(x, st[:C], st[C:], rm, rv, scale, bias, y, True)
    s, q = O.bn_sums(g)
    nps = g.size // C
    m_ref, v_ref, _, _ = O.bn_sums_to_statistics(s, q, nps, 0.9, np.zeros(C), np.ones(C))
    y_ref = O.bn_normalize(g, m_ref, v_ref, scale.cpu().numpy(), bias.cpu().numpy(), 1e-5)
    for st in stats:  # every rank holds identical statistics
        assert np.array_equal(st.cpu().numpy(), stats[0].cpu().numpy())
    emu.assert_close(stats[0][:C].cpu().numpy(), m_ref, 1e-5, "mean")
    emu.assert_close(stats[0][C:].cpu().numpy(), v_ref, 2e-5, "var")
    emu.assert_close(emu.gather_owned(ys, g.shape), y_ref, 2e-5, "y")
    # backward
    g4 = [[torch.zeros(2 * C, device="cuda") for _ in bes] for _ in range(2)]  # (dmean|dvar), (dscale|dbias)
    for bn, x, dy, st, a, b in zip(bns, xs, dys, stats, g4[0], g4[1]):
        bn.backward_stage1(x, dy, st[:C], st[C:], scale, b[:C], b[C:], a[:C], a[C:])
    emu.allreduce_all(bes, g4[0])
    emu.allreduce_all(bes, g4[1])
    for bn, x, dy, dx, st, a in zip(bns, xs, dys, dxs, stats, g4[0]):
        bn.backward_stage2(x, dy, st[:C], st[C:], scale, a[:C], a[C:], dx)
    m_g, v_g = stats[0][:C].cpu().numpy(), stats[0][C:].cpu().numpy()
    dsc, dbi, dme, dva = O.bn_backprop1(g, gdy, m_g, v_g, scale.cpu().numpy(), 1e-5)
    emu.assert_close(g4[1][0][:C].cpu().numpy(), dsc, 2e-5, "dscale")
    emu.assert_close(g4[1][0][C:].cpu().numpy(), dbi, 2e-5, "dbias")
    dx_ref = O.bn_backprop2(g, gdy, m_g, v_g, scale.cpu().numpy(), g4[0][0][:C].cpu().numpy(),
                            g4[0][0][C:].cpu().numpy(), 1e-5, nps)
    emu.assert_close(emu.gather_owned(dxs, g.shape), dx_ref, 1e-5, "dx")


def test_leaky_relu():
    shape = [33, 9, 4, 2]
    be = dc.BackendDNNLib(dc.Locale(0, 1))
    x_t, y_t, dy_t, dx_t = (_rank0(shape, [1] * 4, [0] * 4) for _ in range(4))
    rng = np.random.default_rng(0)
    x = rng.normal(size=x_t.np_real_shape()).astype(np.float32)
    dy = rng.normal(size=x.shape).astype(np.float32)
    emu.upload(x_t, x)
    emu.upload(dy_t, dy)
    y_t.allocate()
    dx_t.allocate()
    lr = dc.LeakyReLU(be)
    lr.forward(x_t, 0.01, y_t)
    lr.backward(x_t, dy_t, 0.01, dx_t)
    assert np.array_equal(y_t.buffer.cpu().numpy(), np.where(x > 0, x, np.float32(0.01) * x))
    assert np.array_equal(dx_t.buffer.cpu().numpy(), np.where(x > 0, dy, np.float32(0.01) * dy))


def test_bn_apply_fused_with_leaky_relu_matches_the_two_passes():
    rng = np.random.default_rng(3)
    x = torch.from_numpy(rng.normal(0.1, 1.5, (2, 5, 6, 7, 40)).astype(np.float32)).cuda()
    C = 5
    mean = torch.from_numpy(rng.normal(0, 0.3, C).astype(np.float32)).cuda()
    var = torch.from_numpy(rng.uniform(0.5, 2, C).astype(np.float32)).cuda()
    scale = torch.from_numpy(rng.uniform(0.5, 1.5, C).astype(np.float32)).cuda()
    bias = torch.from_numpy(rng.normal(0, 0.5, C).astype(np.float32)).cuda()
    loc = dc.Locale(0, 1)
    be = dc.BackendDNNLib(loc, allreduce="peer", allreduce_max_count=64)
    shape = [40, 7, 6, C, 2]
    dist = dc.Distribution.make_localized_distribution(5)
    tx, ty, tz, tf = (dc.Tensor(shape, loc, dist) for _ in range(4))
    for t in (tx, ty, tz, tf):
        t.allocate()
    tx.buffer.copy_(x)
    bn = dc.BatchNormalization(be, 5, 0.9, 1e-5, True)
    rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    bn.forward_stage2(tx, mean, var, rm, rv, scale, bias, ty, is_training=False)
    dc.LeakyReLU(be).forward(ty, 0.01, tz)
    bn.forward_stage2(tx, mean, var, rm, rv, scale, bias, tf, is_training=False, leaky_relu_slope=0.01)
    torch.cuda.synchronize()
    assert torch.equal(tf.buffer, tz.buffer)


def test_empty_shard_zero_fills_run_on_the_backend_stream():
    """A rank without cells contributes zeros to the all-reduces; those fills
    must be ordered on the backend's stream like the kernels they replace.
    The stream is kept busy, then writes 5s: a fill on another stream would
    run first and the 5s would survive."""
    side = torch.cuda.Stream()
    locale = dc.Locale(1, 2)
    be = dc.BackendDNNLib(locale, stream=side, connect=False)
    # D extent 1 over two ranks: the second one owns nothing
    t = dc.Tensor([8, 8, 1, 4, 1], locale, dc.Distribution.make_overlapped_distribution([1, 1, 2, 1, 1], [0] * 5))
    assert t.get_local_size() == 0
    t.allocate()
    bn = dc.BatchNormalization(be, 5, 0.9, 1e-5, True)
    vals = [torch.ones(4, device="cuda") for _ in range(6)]
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        torch.cuda._sleep(20_000_000)
        for v in vals:
            v.fill_(5.0)
    bn.forward_stage1(t, vals[0], vals[1], True)
    bn.backward_stage1(t, t, vals[0], vals[1], vals[0], vals[2], vals[3], vals[4], vals[5])
    torch.cuda.synchronize()
    for v in vals:
        assert float(v.abs().max()) == 0.0
