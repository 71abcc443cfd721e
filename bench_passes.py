#!/usr/bin/env python
"""Per-pass timing of the layer's operators on one GPU, on the per-GPU shard
of a BASELINE configuration (fp32):

    python bench_passes.py [--shape cfg2|cfg3l2|cfg4] [--local-d D] [--reps R]

    cfg2    N=1, C=4 -> K=16, 3x3x3, stride 1, pad 1, D x 256 x 256 (default; also
            layer 1 of configs[2] at 8 GPUs)
    cfg3l2  layer 2 of configs[2] at 8 GPUs: N=1, C=16 -> K=32, 3x3x3, stride 2,
            pad 1, 256^3 -> 128^3
    cfg4    configs[3] at 8 GPUs: N=2, C=32 -> K=32, 5x5, pad 2, 2048 x 1024

Times, with CUDA events on the launching stream and inputs resident in HBM:
convolution forward (with and without the BN statistics in its epilogue),
backward data, backward filter, BN statistics, BN apply, BN backward reduce and
BN backward apply; and, on the convolution's output, a max-pooling (3^n window,
stride 2, forward and backward) and a one-rank re-distribution.  Prints one JSON line with ms per pass and, for each, the
kernel family the plan resolved to.  `--local-d 64` is the small case used for
profiler captures.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


# name: (N, C, K, spatial input extents slowest first, filter, stride, pad)
SHAPES = {
    "cfg2": (1, 4, 16, [256, 256, 256], [3, 3, 3], 1, 1),
    "cfg3l2": (1, 16, 32, [256, 256, 256], [3, 3, 3], 2, 1),
    "cfg4": (2, 32, 32, [2048, 1024], [5, 5], 1, 2),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", choices=sorted(SHAPES), default="cfg2")
    ap.add_argument("--local-d", type=int, default=None, help="cfg2 / cfg3l2: D extent of the input shard")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--grid", default=None,
                    help="process grid w,h[,d]: time rank 0's shard of a tensor partitioned this way (the spatial "
                         "extents above are the SHARD's; halo cells are allocated, rows padded to the pitch, no "
                         "exchange runs) instead of an unpartitioned tensor")
    args = ap.parse_args()
    import torch

    import dihydrogen_b200 as dc
    from dihydrogen_b200 import _abi
    from bench import DECAY, EPS

    if not torch.cuda.is_available():
        raise SystemExit("bench_passes.py needs a CUDA device")
    torch.manual_seed(0)
    N, C_IN, K_OUT, sp, f, stride, pad = SHAPES[args.shape]
    sp = list(sp)
    if args.local_d and len(sp) == 3:
        sp[0] = args.local_d
    nsd = len(sp)
    grid = [int(v) for v in args.grid.split(",")] if args.grid else [1] * nsd  # W first
    assert len(grid) == nsd
    nranks = int(np.prod(grid))
    locale = dc.Locale(0, nranks)
    strides, dil, pads = [stride] * nsd, [1] * nsd, [pad] * nsd
    fshape = list(reversed(f)) + [C_IN, K_OUT]
    gshape = [e * g for e, g in zip(reversed(sp), grid)]  # the global tensor: the shard times the grid
    x = dc.create_input_tensor(gshape + [C_IN, N], grid + [1, 1], list(reversed(f)), strides, dil, locale)
    y = dc.create_convolution_output_tensor(x, fshape, strides, pads, dil)
    z = dc.Tensor(y.shape, locale, y.dist, y._local_of)
    dx = dc.create_d_input_tensor(x)
    dy = dc.create_convolution_d_output_tensor(y, fshape, dil)
    dz = dc.Tensor(y.shape, locale, y.dist, y._local_of)
    for t in (x, y, z, dx, dy, dz):
        t.allocate()
    x.buffer.normal_()
    dz.buffer.normal_()
    w = torch.randn(K_OUT, C_IN, *f, device="cuda") * (2.0 / (C_IN * int(np.prod(f)))) ** 0.5
    dw = torch.zeros_like(w)
    be = dc.BackendDNNLib(locale, options=dc.Options(), allreduce="peer", allreduce_max_count=4096,
                          connect=nranks == 1)
    conv = dc.Convolution(be, nsd + 2)
    conv.setup(x, w, y, dx, None, dy, pads, strides, dil, connect=nranks == 1)
    bn = dc.BatchNormalization(be, nsd + 2, DECAY, EPS, True)
    K = K_OUT
    stats = torch.zeros(2 * K, device="cuda")
    mean, var = stats[:K], stats[K:]
    rm, rv = torch.zeros(K, device="cuda"), torch.ones(K, device="cuda")
    scale, bias = torch.ones(K, device="cuda"), torch.zeros(K, device="cuda")
    g = [torch.zeros(K, device="cuda") for _ in range(4)]
    stream = torch.cuda.current_stream()

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.reps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.reps

    ms = {}
    ms["conv_fwd"] = timed(lambda: conv.forward(1.0, x, w, 0.0, y, skip_halo_exchange=True))
    fused = conv.forward(1.0, x, w, 0.0, y, skip_halo_exchange=True, statistics=(mean, var)) == 1
    if fused:
        ms["conv_fwd_with_bn_statistics"] = timed(
            lambda: conv.forward(1.0, x, w, 0.0, y, skip_halo_exchange=True, statistics=(mean, var)))
    ms["bn_stats"] = timed(lambda: bn.forward_stage1(y, mean, var, True))
    if nranks == 1:
        bn.forward(y, mean, var, rm, rv, scale, bias, z, True)
    else:  # no peers here: this shard's own sums stand in for the all-reduced ones
        bn.forward_stage1(y, mean, var, True)
    ms["bn_finalize_apply"] = timed(lambda: bn.forward_stage2(y, mean, var, rm, rv, scale, bias, z, True))
    ms["bn_bwd_reduce"] = timed(lambda: bn.backward_stage1(y, dz, mean, var, scale, g[0], g[1], g[2], g[3]))
    ms["bn_bwd_apply"] = timed(lambda: bn.backward_stage2(y, dz, mean, var, scale, g[2], g[3], dy))
    ms["conv_bwd_filter"] = timed(lambda: conv.backward_filter(1.0, x, dy, 0.0, dw, reduce=False))
    ms["conv_bwd_data"] = timed(lambda: conv.backward_data(1.0, w, dy, 0.0, dx, skip_halo_exchange=True))
    gbs = {}
    if nranks == 1:
        # pooling of the conv output (3^n window, stride 2, pad 1, MAX) and a local
        # re-distribution of it (one rank: the shuffle's put and wait_unpack kernels)
        win, pp, ps = [3] * nsd, [1] * nsd, [2] * nsd
        px = dc.create_input_tensor(list(y.shape), [1] * (nsd + 2), win, ps, [1] * nsd, locale)
        py = dc.create_pooling_output_tensor(px, win, ps, pp)
        pdx, pdy = dc.create_d_input_tensor(px), dc.create_pooling_d_output_tensor(py)
        px.set_view(y.buffer)
        for t in (py, pdx, pdy):
            t.allocate()
        pdy.buffer.normal_()
        pool = dc.Pooling(be, nsd + 2)
        pool.setup(px, py, pdx, pdy, win, pp, ps, "MAX")
        ms["pool_max_fwd"] = timed(lambda: pool.forward(1.0, px, 0.0, py, skip_halo_exchange=True))
        ms["pool_max_bwd"] = timed(lambda: pool.backward(1.0, py, pdy, px, 0.0, pdx, skip_halo_exchange=True))
        shf = dc.TensorShuffler(px, pdx)
        ms["shuffle_local"] = timed(lambda: shf.shuffle_forward(px.get_buffer(), pdx.get_buffer()))
        ybytes = 4.0 * y.buffer.numel()
        gbs = {"pool_max_fwd": (ybytes + 4.0 * py.buffer.numel()) / (ms["pool_max_fwd"] * 1e-3) / 1e9,
               "pool_max_bwd": (2 * ybytes + 8.0 * py.buffer.numel()) / (ms["pool_max_bwd"] * 1e-3) / 1e9,
               "shuffle_local": 4 * ybytes / (ms["shuffle_local"] * 1e-3) / 1e9}
    vox = N * int(np.prod(sp))
    out_vox = N * int(np.prod([(e + 2 * pad - fe) // stride + 1 for e, fe in zip(sp, f)]))
    flop = 2.0 * out_vox * K_OUT * C_IN * int(np.prod(f))
    fwd = (ms["conv_fwd_with_bn_statistics"] if fused else ms["conv_fwd"] + ms["bn_stats"]) + ms["bn_finalize_apply"]
    bwd = ms["bn_bwd_reduce"] + ms["bn_bwd_apply"] + ms["conv_bwd_filter"] + ms["conv_bwd_data"]
    kinds = {n: ("tcgen05" if conv.kernel_kind(i) == 1 else "fp32-simt")
             for i, n in enumerate(("conv_fwd", "conv_bwd_data", "conv_bwd_filter"))}
    print(json.dumps({"workload": f"{args.shape} shard, N={N}, {' x '.join(map(str, sp))}, C={C_IN} -> K={K_OUT}, "
                                  f"{'x'.join(map(str, f))}, stride {stride}",
                      "ms": {k: round(v, 4) for k, v in ms.items()}, "kernels": kinds,
                      "conv_tflops": {k: round(flop / (ms[k] * 1e-3) / 1e12, 2)
                                      for k in ("conv_fwd", "conv_bwd_data", "conv_bwd_filter")},
                      "algorithmic_gb_per_s": {k: round(v, 1) for k, v in gbs.items()},
                      "forward_ms": round(fwd, 4), "backward_ms": round(bwd, 4),
                      "forward_backward_voxels_per_s": vox / ((fwd + bwd) * 1e-3),
                      "status": [conv.halo_xch_input.status(), int(_abi.lib().dcb_conv_plan_status(conv._plan_fwd, None)),
                                 int(_abi.lib().dcb_conv_plan_status(conv._plan_bwd, None)),
                                 int(_abi.lib().dcb_conv_plan_status(conv._plan_wgrad, None))]}))


if __name__ == "__main__":
    main()
