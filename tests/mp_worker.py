"""Worker run by torchrun (one process per GPU): real peer-store halo exchange,
peer-memory and NCCL all-reduce, the conv + BN layer, pooling with its reverse
SUM exchange and the tensor re-distribution across processes, each checked
against the single-domain oracle.  Launched by
tests/test_gpu_multiproc.py."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import dihydrogen_b200 as dc  # noqa: E402
from dihydrogen_b200 import _abi  # noqa: E402
from oracle import oracle as O  # noqa: E402
import emu  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    loc = dc.Locale.from_torch_distributed()
    n, r = loc.size, loc.rank

    # ---- halo exchange, known answer, several exchanges in a row ----
    for shape, locale, overlap in (([16, 12, 8 * n, 3, 1], [1, 1, n, 1, 1], [0, 0, 2, 0, 0]),
                                   ([18, 8 * n, 6, 2, 2], [1, n, 1, 1, 1], [0, 1, 0, 0, 0]),
                                   ([8 * n, 10, 6, 2, 1], [n, 1, 1, 1, 1], [3, 0, 0, 0, 0])):
        t = dc.Tensor(shape, loc, dc.Distribution.make_overlapped_distribution(locale, overlap))
        hx = dc.HaloExchange(t).setup()
        sh = O.Shard(shape, locale, overlap, r)
        for rep in range(3):
            g = (np.arange(int(np.prod(shape)), dtype=np.float32) * (rep + 1)).reshape(tuple(reversed(shape)))
            emu.scatter_owned(t, g)
            for d in range(t.nd - 2):
                t.clear_halo(d)
            hx.exchange()
            torch.cuda.synchronize()
            assert hx.status() == _abi.OK
            assert np.array_equal(t.buffer.cpu().numpy(), O.fill_by_definition(sh, g)), (shape, rep, r)
        dist.barrier()

    # ---- all-reduce: peer-memory and NCCL flavours ----
    for kind in ("peer", "nccl"):
        ar = dc.Allreduce(loc, kind, 2048)
        for rep in range(3):
            v = torch.arange(1000, dtype=torch.float32, device="cuda") + r + rep
            ar.allreduce(v.data_ptr(), v.numel())
            torch.cuda.synchronize()
            expect = n * (np.arange(1000, dtype=np.float32) + rep) + n * (n - 1) / 2
            assert np.array_equal(v.cpu().numpy(), expect), (kind, rep)
        assert ar.status() == _abi.OK
        dist.barrier()

    # ---- conv + BN layer split along D, forward and backward ----
    rng = np.random.default_rng(7)
    shape, locale, K, f = [32, 24, 8 * n, 4, 1], [1, 1, n, 1, 1], 16, [3, 3, 3]
    C = shape[-2]
    gx = rng.normal(0, 1, tuple(reversed(shape))).astype(np.float32)
    w = rng.normal(0, np.sqrt(2.0 / (C * 27)), (K, C, 3, 3, 3)).astype(np.float32)
    gdz = rng.normal(0, 1, (1, K, 8 * n, 24, 32)).astype(np.float32)
    scale = rng.uniform(0.5, 1.5, K).astype(np.float32)
    bias = rng.normal(0, 0.5, K).astype(np.float32)
    be = dc.BackendDNNLib(loc)
    ones3 = [1, 1, 1]
    x = dc.create_input_tensor(shape, locale, f, ones3, ones3, loc)
    y = dc.create_convolution_output_tensor(x, f + [C, K], ones3, ones3, ones3)
    dy = dc.create_convolution_d_output_tensor(y, f + [C, K], ones3)
    dx = dc.create_d_input_tensor(x)
    z = dc.Tensor(y.shape, loc, y.dist, y._local_of)
    dz = dc.Tensor(y.shape, loc, y.dist, y._local_of)
    emu.scatter_owned(x, gx)
    emu.scatter_owned(dz, gdz)
    for t in (y, dy, dx, z):
        t.allocate()
    wt = torch.from_numpy(w).cuda()
    conv = dc.Convolution(be, 5)
    conv.setup(x, wt, y, dx, None, dy, ones3, ones3, ones3)
    bn = dc.BatchNormalization(be, 5, 0.9, 1e-5, True)
    st = torch.zeros(2 * K, device="cuda")
    rm, rv = torch.zeros(K, device="cuda"), torch.ones(K, device="cuda")
    sc, bi = torch.from_numpy(scale).cuda(), torch.from_numpy(bias).cuda()
    conv.forward(1.0, x, wt, 0.0, y)
    bn.forward(y, st[:K], st[K:], rm, rv, sc, bi, z, True)
    ga, gb = torch.zeros(2 * K, device="cuda"), torch.zeros(2 * K, device="cuda")
    bn.backward(y, dz, st[:K], st[K:], sc, gb[:K], gb[K:], ga[:K], ga[K:], dy)
    dw = torch.zeros_like(wt)
    conv.backward_filter(1.0, x, dy, 0.0, dw)
    conv.backward_data(1.0, wt, dy, 0.0, dx)
    torch.cuda.synchronize()
    assert conv.halo_xch_input.status() == _abi.OK and conv.halo_xch_d_output.status() == _abi.OK

    y_ref = O.conv_fwd(gx, w, ones3, ones3)
    s, q = O.bn_sums(y_ref)
    nps = y_ref.size // K
    m, v, _, _ = O.bn_sums_to_statistics(s, q, nps, 0.9, np.zeros(K), np.ones(K))
    z_ref = O.bn_normalize(y_ref, m, v, scale, bias, 1e-5)
    dsc, dbi, dme, dva = O.bn_backprop1(y_ref, gdz, m, v, scale, 1e-5)
    dy_ref = O.bn_backprop2(y_ref, gdz, m, v, scale, np.float32(dme), np.float32(dva), 1e-5, nps)
    dw_ref = O.conv_bwd_filter(gx, dy_ref, (3, 3, 3), ones3, ones3)
    dx_ref = np.zeros_like(gx)
    O.conv_bwd_data(w, dy_ref, dx_ref, ones3, ones3)

    def own(t, g):
        sl = tuple(slice(o, o + l) for o, l in reversed(list(zip(t.offset, t.local_shape))))
        return g[sl]

    emu.assert_close(y.owned().cpu().numpy(), own(y, y_ref), 1e-5, "y")
    emu.assert_close(z.owned().cpu().numpy(), own(z, z_ref), 3e-5, "z")
    emu.assert_close(dy.owned().cpu().numpy(), own(dy, dy_ref), 5e-5, "bn dx")
    emu.assert_close(dw.cpu().numpy(), dw_ref, 5e-5, "dw")
    emu.assert_close(dx.owned().cpu().numpy(), own(dx, dx_ref), 5e-5, "dx")
    dist.barrier()

    # ---- the same forward pass with the interior running while the halo is in flight ----
    be_ov = dc.BackendDNNLib(loc, options=dc.Options(overlap_halo_exchange=True))
    conv_ov = dc.Convolution(be_ov, 5)
    y_ov = dc.create_convolution_output_tensor(x, f + [C, K], ones3, ones3, ones3)
    y_ov.allocate()
    conv_ov.setup(x, wt, y_ov, None, None, None, ones3, ones3, ones3)
    assert conv_ov.is_overlap_fwd_halo_exchange_enabled() == (n > 1)
    for rep in range(3):
        y_ov.buffer.fill_(float("nan"))
        conv_ov.forward(1.0, x, wt, 0.0, y_ov)
    torch.cuda.synchronize()
    assert conv_ov.halo_xch_input.status() == _abi.OK
    emu.assert_close(y_ov.owned().cpu().numpy(), own(y_ov, y_ref), 1e-5, "y, overlapped")
    dist.barrier()

    # ---- pooling across processes: halo exchange forward, reverse SUM backward ----
    for mode in ("MAX", "AVERAGE_NO_PAD"):
        pshape, plocale = [20, 12, 6 * n, 3, 2], [1, 1, n, 1, 1]
        gpx = rng.integers(-4, 5, size=tuple(reversed(pshape))).astype(np.float32)
        py_ref = O.pool_fwd(gpx, ones3_w := [3, 3, 3], ones3, ones3, mode)
        gpdy = rng.normal(size=py_ref.shape).astype(np.float32)
        pdx_ref = O.pool_bwd(gpx, gpdy, ones3_w, ones3, ones3, mode)
        px = dc.create_input_tensor(pshape, plocale, ones3_w, ones3, ones3, loc)
        py = dc.create_pooling_output_tensor(px, ones3_w, ones3, ones3)
        pdx, pdy = dc.create_d_input_tensor(px), dc.create_pooling_d_output_tensor(py)
        emu.scatter_owned(px, gpx)
        emu.scatter_owned(pdy, gpdy)
        py.allocate(), pdx.allocate()
        pool = dc.Pooling(be, 5)
        pool.setup(px, py, pdx, pdy, ones3_w, ones3, ones3, mode)
        pool.forward(1.0, px, 0.0, py)
        pool.backward(1.0, py, pdy, px, 0.0, pdx)
        torch.cuda.synchronize()
        assert pool.halo_xch_input.status() == _abi.OK and pool.halo_xch_d_input.status() == _abi.OK
        emu.assert_close(py.owned().cpu().numpy(), own(py, py_ref), 1e-6, "pool y " + mode)
        emu.assert_close(pdx.owned().cpu().numpy(), own(pdx, pdx_ref), 4e-6, "pool dx " + mode)
        dist.barrier()

    # ---- re-distribution: sample-parallel <-> D-partitioned, there and back ----
    sshape = [16, 12, 4 * n, 3, 2 * n]
    gs = rng.normal(size=tuple(reversed(sshape))).astype(np.float32)
    ts = dc.Tensor(sshape, loc, dc.Distribution.make_overlapped_distribution([1, 1, 1, 1, n], [0] * 5))
    td = dc.Tensor(sshape, loc, dc.Distribution.make_overlapped_distribution([1, 1, n, 1, 1], [0, 0, 1, 0, 0]))
    tb = dc.Tensor(sshape, loc, dc.Distribution.make_overlapped_distribution([1, 1, 1, 1, n], [0] * 5))
    emu.scatter_owned(ts, gs)
    td.allocate(), tb.allocate()
    shf = dc.TensorShuffler(ts, td)
    for rep in range(3):
        shf.shuffle_forward(ts.get_buffer(), td.get_buffer())
        shf.shuffle_backward(td.get_buffer(), tb.get_buffer())
    torch.cuda.synchronize()
    assert shf.status("fwd") == _abi.OK and shf.status("bwd") == _abi.OK
    assert np.array_equal(td.owned().cpu().numpy(), own(td, gs))
    assert np.array_equal(tb.owned().cpu().numpy(), own(tb, gs))
    dist.barrier()
    print(f"mp ok rank {r} of {n}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
