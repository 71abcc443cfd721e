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

    # ---- all-reduce of a vector longer than the slots: max_count-sized pieces ----
    ar = dc.Allreduce(loc, "peer", 256)
    cnt = 3 * 256 + 5
    for rep in range(3):
        v = torch.arange(cnt, dtype=torch.float32, device="cuda") + r + rep
        ar.allreduce(v.data_ptr(), v.numel())
        torch.cuda.synchronize()
        expect = n * (np.arange(cnt, dtype=np.float32) + rep) + n * (n - 1) / 2
        assert np.array_equal(v.cpu().numpy(), expect), ("chunked", rep)
    assert ar.status() == _abi.OK
    dist.barrier()

    # ---- conv + BN layer, forward and backward, on several grids ----
    rng = np.random.default_rng(7)
    be = dc.BackendDNNLib(loc)

    def gather_global(t, shape_np):
        """The global tensor from every rank's owned cells (host side)."""
        parts = [None] * n
        dist.all_gather_object(parts, (list(t.offset), list(t.local_shape), t.owned().cpu().numpy()))
        g = np.zeros(shape_np, np.float32)
        for off, loc_shape, a in parts:
            g[tuple(slice(o, o + l) for o, l in reversed(list(zip(off, loc_shape))))] = a
        return g

    def layer_case(shape, locale, K, f, what):
        """Halo exchange + conv + BN forward and backward with this process
        grid; every stage against the single-domain oracle fed with the GPUs'
        own previous stage, at 1e-5 (P ranks == 1 rank,
        legacy/tests/dnn_backend/test_cudnn_util.sh.in:387-425)."""
        nd, nsd = len(shape), len(shape) - 2
        C = shape[-2]
        ones, pads = [1] * nsd, [(ff - 1) // 2 for ff in f]
        gx = rng.normal(0, 1, tuple(reversed(shape))).astype(np.float32)
        w = rng.normal(0, np.sqrt(2.0 / (C * np.prod(f))), (K, C, *reversed(f))).astype(np.float32)
        scale = rng.uniform(0.5, 1.5, K).astype(np.float32)
        bias = rng.normal(0, 0.5, K).astype(np.float32)
        x = dc.create_input_tensor(shape, locale, f, ones, ones, loc)
        y = dc.create_convolution_output_tensor(x, list(f) + [C, K], ones, pads, ones)
        dy = dc.create_convolution_d_output_tensor(y, list(f) + [C, K], ones)
        dx = dc.create_d_input_tensor(x)
        z = dc.Tensor(y.shape, loc, y.dist, y._local_of)
        dz = dc.Tensor(y.shape, loc, y.dist, y._local_of)
        osh = tuple(reversed(y.shape))
        gdz = rng.normal(0, 1, osh).astype(np.float32)
        emu.scatter_owned(x, gx)
        emu.scatter_owned(dz, gdz)
        for t in (y, dy, dx, z):
            t.allocate()
        x.buffer.fill_(float("nan"))  # the halo must come from the exchange
        emu.scatter_owned_into(x, gx)
        dy.buffer.fill_(float("nan"))
        wt = torch.from_numpy(w).cuda()
        conv = dc.Convolution(be, nd)
        conv.setup(x, wt, y, dx, None, dy, pads, ones, ones)
        bn = dc.BatchNormalization(be, nd, 0.9, 1e-5, True)
        st = torch.zeros(2 * K, device="cuda")
        rm, rv = torch.zeros(K, device="cuda"), torch.ones(K, device="cuda")
        sc, bi = torch.from_numpy(scale).cuda(), torch.from_numpy(bias).cuda()
        ga, gb = torch.zeros(2 * K, device="cuda"), torch.zeros(2 * K, device="cuda")
        dw = torch.zeros_like(wt)
        for rep in range(2):  # twice: the exchange's double buffers and epochs come round
            conv.forward(1.0, x, wt, 0.0, y)
            bn.forward(y, st[:K], st[K:], rm, rv, sc, bi, z, True)
            bn.backward(y, dz, st[:K], st[K:], sc, gb[:K], gb[K:], ga[:K], ga[K:], dy)
            conv.backward_filter(1.0, x, dy, 0.0, dw)
            conv.backward_data(1.0, wt, dy, 0.0, dx)
        torch.cuda.synchronize()
        assert conv.halo_xch_input.status() == _abi.OK and conv.halo_xch_d_output.status() == _abi.OK
        assert be.allreducer.status() == _abi.OK
        assert _abi.lib().dcb_conv_plan_status(conv._plan_fwd, None) == _abi.OK
        assert _abi.lib().dcb_conv_plan_status(conv._plan_bwd, None) == _abi.OK
        assert _abi.lib().dcb_conv_plan_status(conv._plan_wgrad, None) == _abi.OK
        # the halo-extended input shard, bit for bit (edges and corners included)
        sh = O.Shard(shape, locale, list(x.dist.overlap), r)
        assert np.array_equal(x.buffer.cpu().numpy(), O.fill_by_definition(sh, gx)), what + ": halo contents"
        bwd = dict(gdz=gdz, dscale=gb[:K].cpu().numpy(), dbias=gb[K:].cpu().numpy(), dmean=ga[:K].cpu().numpy(),
                   dvar=ga[K:].cpu().numpy(), dy=gather_global(dy, osh), dw=dw.cpu().numpy(),
                   dx=gather_global(dx, gx.shape))
        emu.check_stages(K, gx, w, scale, bias, list(reversed(pads)), ones, gather_global(y, osh),
                         st[:K].cpu().numpy(), st[K:].cpu().numpy(), gather_global(z, osh), bwd, 1e-5, what + ": ")
        dist.barrier()
        return x, y, wt, conv, gx, w

    # a D split; a W split (rows padded to the pitch); the grid the benchmark's weak-scaling
    # ladder uses at this rank count (4 -> D x H, 8 -> 2 x 2 x 2); with 8 ranks also the
    # 2 x 4 grid of the 2-D large-image layer
    grid = {1: [1, 1, 1], 2: [1, 1, 2], 4: [1, 2, 2], 8: [2, 2, 2]}.get(n, [1, 1, n])
    ext = [24 * g if i == 0 else (10 * g if i == 1 else 6 * g) for i, g in enumerate(grid)]
    x, y, wt, conv, gx, w = layer_case([32, 24, 8 * n, 4, 1], [1, 1, n, 1, 1], 16, [3, 3, 3], "D split")
    if n > 1:
        layer_case([20 * n, 12, 10, 4, 1], [n, 1, 1, 1, 1], 16, [3, 3, 3], "W split")
    if n in (4, 8):
        layer_case(ext + [4, 1], grid + [1, 1], 16, [3, 3, 3], "grid " + "x".join(map(str, grid)))
    if n == 8:
        layer_case([32 * 4, 24 * 2, 8, 2], [4, 2, 1, 1], 8, [5, 5], "2-D layer, 2 x 4 grid")
    ones3, f, C, K = [1, 1, 1], [3, 3, 3], 4, 16
    y_ref = O.conv_fwd(gx, w, ones3, ones3)

    def own(t, g):
        sl = tuple(slice(o, o + l) for o, l in reversed(list(zip(t.offset, t.local_shape))))
        return g[sl]

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
