"""The oracle against the reference's own outputs (golden fixtures) and the
reference tests' known answers.  No GPU."""
import os

import numpy as np
import pytest

from conftest import GOLDEN, conv_fixtures, geom_fixtures, parse_geom
from oracle import oracle as O


@pytest.mark.parametrize("fname", geom_fixtures())
def test_geometry_matches_reference(fname):
    (shape, locale, filt, strides, pad, K), ranks = parse_geom(os.path.join(GOLDEN, fname))
    nd, nsd = len(shape), len(shape) - 2
    overlap = [(f - 1) // 2 if l > 1 else 0 for f, l in zip(filt, locale)] + [0, 0]
    shards = O.make_shards(shape, locale, overlap)
    assert len(shards) == len(ranks)
    for sh, ref in zip(shards, ranks):
        assert sh.local == ref["local"]
        assert sh.real == ref["real"]
        assert sh.offset == ref["offset"]
        fs, bs, fr, br = O.get_halo_sizes(sh, filt, strides, [1] * nsd, bool(pad))
        assert fs[:nsd] == ref["fwd_send"] and bs[:nsd] == ref["bwd_send"]
        assert fr[:nsd] == ref["fwd_recv"] and br[:nsd] == ref["bwd_recv"]
        out = O.conv_output_local_shape(sh, filt, strides, [1] * nsd, bool(pad), K)
        assert out == ref["out_local"]


@pytest.mark.parametrize("fname", conv_fixtures())
def test_conv_oracle_matches_ref_backend(fname):
    """conv_oracle.c vs Convolution<ref::Backend> run on the same inputs."""
    z = np.load(os.path.join(GOLDEN, fname))
    x, w, dy = z["x"], z["w"], z["dy"]
    f = w.shape[-1]
    p = (f - 1) // 2
    y = O.conv_fwd(x, w, [p, p], [1, 1])
    dx = np.zeros_like(x)
    O.conv_bwd_data(w, dy, dx, [p, p], [1, 1])
    dw = O.conv_bwd_filter(x, dy, (f, f), [p, p], [1, 1])
    # ref::Backend accumulates in fp32 element by element; the oracle in fp64.
    for got, ref in ((y, z["y"]), (dx, z["dx"]), (dw, z["dw"])):
        scale = np.abs(ref).max()
        assert np.abs(got - ref).max() <= 2e-6 * scale


@pytest.mark.parametrize("fname", conv_fixtures())
def test_conv_oracle_on_shards_matches_global(fname):
    """Distributed == single rank: running the oracle per shard on the
    halo-extended buffers, with the reference's descriptor rules, reproduces
    the global result (the self-consistency contract of
    legacy/tests/dnn_backend/test_cudnn_util.sh.in:387-425)."""
    z = np.load(os.path.join(GOLDEN, fname))
    x, w = z["x"], z["w"]
    locale = [int(v) for v in z["locale"]]
    f = w.shape[-1]
    p = (f - 1) // 2
    N, C, H, W = x.shape
    shape = [W, H, C, N]
    overlap = [p if l > 1 else 0 for l in locale[:2]] + [0, 0]
    shards = O.make_shards(shape, locale, overlap)
    y_glob = O.conv_fwd(x, w, [p, p], [1, 1])
    for sh in shards:
        buf = O.fill_by_definition(sh, x)
        pads = [0 if sh.overlap[1] else p, 0 if sh.overlap[0] else p]  # (H, W)
        y = O.conv_fwd(buf, w, pads, [1, 1])
        ysl = tuple(slice(o, o + l) for o, l in ((0, N), (0, w.shape[0]), (sh.offset[1], sh.local[1]),
                                                 (sh.offset[0], sh.local[0])))
        assert np.array_equal(y, y_glob[ysl])


HALO_CASES = [
    # shape (W..N), locale, overlap
    ([8, 9, 3, 2], [1, 2, 1, 1], [0, 1, 0, 0]),
    ([8, 9, 3, 2], [2, 2, 1, 1], [1, 1, 0, 0]),
    ([11, 9, 2, 2], [3, 2, 1, 1], [2, 2, 0, 0]),
    ([7, 8, 9, 2, 1], [1, 1, 2, 1, 1], [0, 0, 1, 0, 0]),
    ([9, 8, 7, 2, 1], [2, 2, 2, 1, 1], [1, 2, 1, 0, 0]),
    ([9, 8, 13, 2, 2], [1, 2, 4, 1, 1], [0, 1, 3, 0, 0]),
]


@pytest.mark.parametrize("shape,locale,overlap", HALO_CASES)
def test_halo_exchange_known_answer(shape, locale, overlap):
    """legacy/tests/tensor/test_halo_exchange_cuda.cu:52-233: owned cells hold
    their global linear offset; after the exchange every halo cell inside the
    global domain holds its own global offset, edges and corners included."""
    g = np.arange(int(np.prod(shape)), dtype=np.float32).reshape(tuple(reversed(shape)))
    shards = O.make_shards(shape, locale, overlap)
    bufs = O.scatter(shards, g)
    O.exchange(shards, bufs)
    for sh, b in zip(shards, bufs):
        assert np.array_equal(b, O.fill_by_definition(sh, g))


@pytest.mark.parametrize("shape,locale,overlap", HALO_CASES[:5])
def test_halo_reverse_sum_multiplicity(shape, locale, overlap):
    """test_halo_exchange_cuda.cu:245-334: all-ones tensor, forward exchange,
    then reverse exchange with SUM: an owned cell ends at 1 + (number of
    neighbour halo cells that alias it)."""
    g = np.ones(tuple(reversed(shape)), np.float32)
    shards = O.make_shards(shape, locale, overlap)
    bufs = O.scatter(shards, g)
    O.exchange(shards, bufs)
    O.exchange(shards, bufs, reverse=True, op="SUM")
    total = O.gather(shards, bufs, g.shape)
    # Along one partitioned dimension an interior boundary cell is counted once
    # more per neighbour whose halo covers it; the ordered exchange compounds
    # the factors of the dimensions, so the result is a product of per-dim
    # multiplicities.
    expect = np.ones_like(g)
    nd = len(shape)
    for d in range(nd):
        if locale[d] == 1 or overlap[d] == 0:
            continue
        mult = np.ones(shape[d], np.float32)
        edges = np.cumsum([O.split_extent(shape[d], locale[d], j) for j in range(locale[d])])[:-1]
        for e in edges:
            mult[e - overlap[d]: e + overlap[d]] += 1
        sh = [1] * nd
        sh[nd - 1 - d] = shape[d]
        expect = expect * mult.reshape(sh)
    assert np.array_equal(total, expect)


def test_bn_oracle_known_answer():
    """Closed form on x[n,c,h,w] = c + (w even ? +1 : -1): mean c, biased
    variance 1, unbiased n/(n-1) (batchnorm.cu:302-308)."""
    N, C, H, W = 2, 3, 4, 6
    x = np.zeros((N, C, H, W), np.float32)
    for c in range(C):
        x[:, c] = c + np.where(np.arange(W) % 2 == 0, 1.0, -1.0)
    s, q = O.bn_sums(x)
    n = N * H * W
    mean, var, rm, rv = O.bn_sums_to_statistics(s, q, n, 0.9, np.zeros(C), np.ones(C))
    assert np.allclose(mean, np.arange(C))
    assert np.allclose(var, n / (n - 1.0), rtol=1e-6)
    assert np.allclose(rm, 0.1 * np.arange(C)) and np.allclose(rv, 0.9 + 0.1 * n / (n - 1.0))
    y = O.bn_normalize(x, mean, var, np.full(C, 2.0), np.full(C, 0.5), 0.0)
    inv = 1 / np.sqrt(n / (n - 1.0))
    assert np.allclose(y[:, 1, :, 0], 2 * inv + 0.5, rtol=1e-6)


def test_bn_oracle_backward_matches_autograd_formula():
    """backprop1/backprop2 (batchnorm.cu:920-956, 1327-1362) agree with the
    analytic gradient of y = scale*(x-mean)/sqrt(var_unbiased+eps)+bias when
    the variance's own n/(n-1) convention is used throughout."""
    rng = np.random.default_rng(0)
    N, C, H, W = 2, 3, 5, 4
    x = rng.normal(0, 1, (N, C, H, W)).astype(np.float32)
    dy = rng.normal(0, 1, (N, C, H, W)).astype(np.float32)
    scale = rng.uniform(0.5, 1.5, C).astype(np.float32)
    eps = 1e-5
    n = N * H * W
    s, q = O.bn_sums(x)
    mean, var, _, _ = O.bn_sums_to_statistics(s, q, n, 0.9, np.zeros(C), np.ones(C))
    dscale, dbias, dmean, dvar = O.bn_backprop1(x, dy, mean, var, scale, eps)
    dx = O.bn_backprop2(x, dy, mean, var, scale, dmean, dvar, eps, n)
    xd, dyd = x.astype(np.float64), dy.astype(np.float64)
    m = xd.mean(axis=(0, 2, 3), keepdims=True)
    v = xd.var(axis=(0, 2, 3), keepdims=True, ddof=1)
    inv = 1 / np.sqrt(v + eps)
    sc = scale.reshape(1, C, 1, 1).astype(np.float64)
    dxhat = dyd * sc
    dvar_ref = (-dxhat * (xd - m) * inv**3 / 2).sum(axis=(0, 2, 3), keepdims=True)
    dmean_ref = (-dxhat * inv).sum(axis=(0, 2, 3), keepdims=True)
    dx_ref = dxhat * inv + dmean_ref / n + dvar_ref * 2 / (n - 1) * (xd - m)
    assert np.allclose(dx, dx_ref, rtol=1e-4, atol=1e-5)
    assert np.allclose(dbias, dyd.sum(axis=(0, 2, 3)), rtol=1e-6)
    assert np.allclose(dscale, (dyd * (xd - m) * inv).sum(axis=(0, 2, 3)), rtol=1e-4, atol=1e-5)


# --------------------------------------------------------------------------
# pooling: the restatement against torch's CPU pooling (an independent
# implementation, as the reference's own test uses another framework:
# legacy/tests/dnn_backend/chainer_pooling.py)
# --------------------------------------------------------------------------
@pytest.mark.parametrize("mode", O.POOL_MODES)
@pytest.mark.parametrize("shape,window,pads,strides", [
    ((2, 3, 7, 9, 11), (3, 3, 3), (1, 1, 1), (2, 2, 2)),
    ((1, 2, 8, 10), (2, 2), (0, 0), (2, 2)),
    ((2, 2, 6, 7, 8), (3, 3, 3), (1, 1, 1), (1, 1, 1)),
    ((1, 2, 9, 12), (3, 3), (0, 0), (1, 1)),
    ((1, 1, 11, 13), (5, 5), (2, 2), (3, 3)),
])
def test_pooling_oracle_against_torch(shape, window, pads, strides, mode):
    import torch
    import torch.nn.functional as F

    rng = np.random.default_rng(0)
    x = rng.integers(-3, 4, size=shape).astype(np.float32)  # ties on purpose
    xt = torch.tensor(x, requires_grad=True)
    three = len(window) == 3
    if mode == "MAX":
        y = (F.max_pool3d if three else F.max_pool2d)(xt, window, strides, pads)
    else:
        y = (F.avg_pool3d if three else F.avg_pool2d)(xt, window, strides, pads,
                                                      count_include_pad=(mode == "AVERAGE"))
    dy = torch.tensor(rng.normal(size=y.shape).astype(np.float32))
    y.backward(dy)
    np.testing.assert_allclose(O.pool_fwd(x, window, pads, strides, mode), y.detach().numpy(), rtol=0, atol=1e-6)
    np.testing.assert_allclose(O.pool_bwd(x, dy.numpy(), window, pads, strides, mode), xt.grad.numpy(), rtol=0,
                               atol=2e-6)


# --------------------------------------------------------------------------
# convolution and batch-norm: the restatement against an independent
# implementation (torch on the CPU, in fp64, gradients by autograd) for the
# branches the reference's own CPU backend cannot pin: 5-D tensors, strides,
# dilations, no padding.  What cuDNN computes for the reference at these
# shapes is the published cross-correlation torch implements too.
# --------------------------------------------------------------------------
@pytest.mark.parametrize("shape,K,f,pads,strides,dil", [
    ((2, 3, 7, 8, 9), 4, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1)),   # 5-D
    ((1, 4, 9, 10, 12), 5, (3, 3, 3), (1, 1, 1), (2, 2, 2), (1, 1, 1)), # 5-D, stride 2 (configs[2] layer 2)
    ((1, 2, 11, 9, 13), 3, (3, 3, 3), (2, 2, 2), (1, 1, 1), (2, 2, 2)), # 5-D, dilation 2
    ((2, 3, 8, 7, 9), 4, (3, 3, 3), (0, 0, 0), (1, 1, 1), (1, 1, 1)),   # 5-D, no padding
    ((1, 2, 9, 8, 10), 3, (3, 3, 3), (0, 0, 0), (2, 2, 2), (1, 1, 1)),  # 5-D, no padding, stride 2
    ((2, 3, 12, 14), 4, (5, 5), (2, 2), (1, 1), (1, 1)),                # 4-D, 5 x 5 (configs[3])
    ((1, 3, 13, 11), 2, (3, 3), (1, 1), (2, 2), (1, 1)),                # 4-D, stride 2
    ((1, 2, 7, 9, 8), 3, (1, 3, 3), (0, 1, 1), (1, 2, 1), (1, 1, 2)),   # mixed per-dimension settings
])
def test_conv_oracle_against_torch_fp64(shape, K, f, pads, strides, dil):
    import torch
    import torch.nn.functional as F

    rng = np.random.default_rng(3)
    C = shape[1]
    x = rng.normal(size=shape).astype(np.float32)
    w = rng.normal(0, 0.3, (K, C) + tuple(f)).astype(np.float32)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    wt = torch.tensor(w, dtype=torch.float64, requires_grad=True)
    conv = F.conv3d if len(f) == 3 else F.conv2d
    yt = conv(xt, wt, None, strides, pads, dil)
    dy = rng.normal(size=tuple(yt.shape)).astype(np.float32)
    yt.backward(torch.tensor(dy, dtype=torch.float64))
    y = O.conv_fwd(x, w, list(pads), list(strides), list(dil))
    assert y.shape == tuple(yt.shape)
    dx = np.zeros_like(x)
    O.conv_bwd_data(w, dy, dx, list(pads), list(strides), list(dil))
    dw = O.conv_bwd_filter(x, dy, tuple(f), list(pads), list(strides), list(dil))
    # the oracle accumulates in fp64 and rounds once to fp32
    for got, ref, what in ((y, yt.detach().numpy(), "y"), (dx, xt.grad.numpy(), "dx"), (dw, wt.grad.numpy(), "dw")):
        assert np.abs(got - ref).max() <= 1.5e-7 * np.abs(ref).max() + 1e-30, what
    # alpha / beta blend (y = alpha * conv + beta * y)
    y0 = rng.normal(size=y.shape).astype(np.float32)
    yb = O.conv_fwd(x, w, list(pads), list(strides), list(dil), alpha=0.5, beta=2.0, y=y0.copy())
    np.testing.assert_allclose(yb, 0.5 * yt.detach().numpy() + 2.0 * y0, rtol=0, atol=3e-6)


@pytest.mark.parametrize("shape", [(2, 3, 5, 6, 7), (3, 4, 9, 8)])
def test_bn_oracle_against_torch_fp64(shape):
    """Statistics, normalisation and the backward pass against torch's fp64
    batch-norm.  The reference normalises with the UNBIASED variance
    (batchnorm.cu:302-308: var * n / (n - 1)); torch normalises with the biased
    one, so torch runs with eps' = eps * (n-1)/n on inputs and a scale
    multiplied by sqrt((n-1)/n), which makes the two forward functions (and
    hence all gradients) identical."""
    import torch
    import torch.nn.functional as F

    rng = np.random.default_rng(4)
    C = shape[1]
    n = int(np.prod(shape)) // C
    eps, decay = 1e-5, 0.9
    x = rng.normal(0.3, 1.2, shape).astype(np.float32)
    dy = rng.normal(size=shape).astype(np.float32)
    scale = rng.uniform(0.5, 1.5, C).astype(np.float32)
    bias = rng.normal(0, 0.5, C).astype(np.float32)
    rm0, rv0 = rng.normal(size=C).astype(np.float32), rng.uniform(0.5, 2, C).astype(np.float32)
    s, q = O.bn_sums(x)
    mean, var, rm, rv = O.bn_sums_to_statistics(s, q, n, decay, rm0, rv0)
    y = O.bn_normalize(x, mean, var, scale, bias, eps)
    dscale, dbias, dmean, dvar = O.bn_backprop1(x, dy, mean, var, scale, eps)
    dx = O.bn_backprop2(x, dy, mean, var, scale, dmean, dvar, eps, n)

    r = (n - 1.0) / n
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    st = torch.tensor(scale, dtype=torch.float64, requires_grad=True)
    bt = torch.tensor(bias, dtype=torch.float64, requires_grad=True)
    rmt, rvt = torch.tensor(rm0, dtype=torch.float64), torch.tensor(rv0, dtype=torch.float64)
    # (x - m) / sqrt(v_b * n/(n-1) + eps) = sqrt(r) * (x - m) / sqrt(v_b + eps * r)
    yt = F.batch_norm(xt, rmt, rvt, st * np.sqrt(r), bt, training=True, momentum=1 - decay, eps=eps * r)
    yt.backward(torch.tensor(dy, dtype=torch.float64))
    xd = x.astype(np.float64)
    red = (0,) + tuple(range(2, len(shape)))
    assert np.allclose(mean, xd.mean(axis=red), rtol=1e-6, atol=1e-7)
    assert np.allclose(var, xd.var(axis=red, ddof=1), rtol=2e-6)
    # running statistics: decay * old + (1 - decay) * new, with the unbiased variance (torch does the same)
    assert np.allclose(rm, rmt.numpy(), rtol=1e-6, atol=1e-7) and np.allclose(rv, rvt.numpy(), rtol=2e-6)
    # fp32 arithmetic in the reference's operation order against fp64: a few ulp
    np.testing.assert_allclose(y, yt.detach().numpy(), rtol=0, atol=4e-6)
    np.testing.assert_allclose(dbias, bt.grad.numpy(), rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(dscale, st.grad.numpy(), rtol=1e-5, atol=1e-5)  # d/d(scale) of scale * sqrt(r) * xhat
    np.testing.assert_allclose(dx, xt.grad.numpy(), rtol=0, atol=1e-5)
