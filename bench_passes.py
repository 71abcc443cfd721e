#!/usr/bin/env python
"""Per-pass timing of the layer's operators on one GPU, BASELINE configs[1]
shard (N=1, C=4 -> K=16, 3x3x3, stride 1, pad 1, fp32, D x 256 x 256):

    python bench_passes.py [--local-d D] [--reps R]

Times, with CUDA events on the launching stream and inputs resident in HBM:
convolution forward (with and without the BN statistics in its epilogue),
backward data, backward filter, BN statistics, BN apply, BN backward reduce and
BN backward apply.  Prints one JSON line with ms per pass and, for each, the
kernel family the plan resolved to.  `--local-d 64` is the small case used for
profiler captures.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--local-d", type=int, default=256)
    ap.add_argument("--reps", type=int, default=5)
    args = ap.parse_args()
    import torch

    import dihydrogen_b200 as dc
    from dihydrogen_b200 import _abi
    from bench import C_IN, K_OUT, DECAY, EPS, layer_geometry

    if not torch.cuda.is_available():
        raise SystemExit("bench_passes.py needs a CUDA device")
    torch.manual_seed(0)
    locale = dc.Locale(0, 1)
    geo = layer_geometry(1, locale, local_d=args.local_d)
    x, y, z = geo["input"], geo["conv_out"], geo["bn_out"]
    dx = dc.create_d_input_tensor(x)
    dy = dc.create_convolution_d_output_tensor(y, geo["filter_shape"], geo["dilations"])
    dz = dc.Tensor(y.shape, locale, y.dist, y._local_of)
    for t in (x, y, z, dx, dy, dz):
        t.allocate()
    x.buffer.normal_()
    dz.buffer.normal_()
    w = torch.randn(K_OUT, C_IN, 3, 3, 3, device="cuda") * 0.14
    dw = torch.zeros_like(w)
    be = dc.BackendDNNLib(locale, options=dc.Options(), allreduce="peer", allreduce_max_count=4096)
    conv = dc.Convolution(be, 5)
    conv.setup(x, w, y, dx, None, dy, geo["pads"], geo["strides"], geo["dilations"])
    bn = dc.BatchNormalization(be, 5, DECAY, EPS, True)
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
    ms["conv_fwd_with_bn_statistics"] = timed(
        lambda: conv.forward(1.0, x, w, 0.0, y, skip_halo_exchange=True, statistics=(mean, var)))
    ms["bn_stats"] = timed(lambda: bn.forward_stage1(y, mean, var, True))
    bn.forward(y, mean, var, rm, rv, scale, bias, z, True)
    ms["bn_finalize_apply"] = timed(lambda: bn.forward_stage2(y, mean, var, rm, rv, scale, bias, z, True))
    ms["bn_bwd_reduce"] = timed(lambda: bn.backward_stage1(y, dz, mean, var, scale, g[0], g[1], g[2], g[3]))
    ms["bn_bwd_apply"] = timed(lambda: bn.backward_stage2(y, dz, mean, var, scale, g[2], g[3], dy))
    ms["conv_bwd_filter"] = timed(lambda: conv.backward_filter(1.0, x, dy, 0.0, dw, reduce=False))
    ms["conv_bwd_data"] = timed(lambda: conv.backward_data(1.0, w, dy, 0.0, dx, skip_halo_exchange=True))
    vox = args.local_d * 256 * 256
    fwd = ms["conv_fwd_with_bn_statistics"] + ms["bn_finalize_apply"]
    bwd = ms["bn_bwd_reduce"] + ms["bn_bwd_apply"] + ms["conv_bwd_filter"] + ms["conv_bwd_data"]
    kinds = {n: ("tcgen05" if conv.kernel_kind(i) == 1 else "fp32-simt")
             for i, n in enumerate(("conv_fwd", "conv_bwd_data", "conv_bwd_filter"))}
    print(json.dumps({"workload": f"configs[1] shard, {args.local_d} x 256 x 256, C=4 -> K=16, 3x3x3",
                      "ms": {k: round(v, 4) for k, v in ms.items()}, "kernels": kinds,
                      "forward_ms": round(fwd, 4), "backward_ms": round(bwd, 4),
                      "forward_backward_voxels_per_s": vox / ((fwd + bwd) * 1e-3),
                      "status": [conv.halo_xch_input.status(), int(_abi.lib().dcb_conv_plan_status(conv._plan_fwd, None)),
                                 int(_abi.lib().dcb_conv_plan_status(conv._plan_bwd, None))]}))


if __name__ == "__main__":
    main()
