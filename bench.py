#!/usr/bin/env python
"""Benchmark of the DistConv hot path on B200: one {halo exchange + 3-D
convolution forward + distributed batch-norm forward} layer pass.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[1]): input N=1, C=4, 256^3 fp32 ~N(0,1),
3x3x3 filters K=16 stride 1 pad 1 He-init, BN over the channel dimension with
per-channel statistics all-reduced over the spatial partition.  Weak scaling:
every GPU owns a 256^3 shard, the global volume is 256 x 256 x (256*N) split
along D.  Inputs are seeded, synthetic and independent of the partitioning.

Prints ONE JSON line (rank 0).  `value` is voxels/s with inputs resident in
HBM; `e2e` is the same pass driven from pinned host buffers (H2D of the input
shard and D2H of the BN output inside the timed region).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

EXTENT = 256
C_IN, K_OUT = 4, 16
FILTER = [3, 3, 3]
EPS, DECAY = 1e-5, 0.9


def layer_geometry(n_gpus, locale, extent=EXTENT, local_d=None):
    """Tensors (unallocated) of the benchmark layer for this rank: the global
    volume grows with the GPU count along D (weak scaling).  local_d shrinks
    the per-GPU D extent (profiling captures only)."""
    import dihydrogen_b200 as dc

    shape = [extent, extent, (local_d or extent) * n_gpus, C_IN, 1]  # W, H, D, C, N
    locale_shape = [1, 1, n_gpus, 1, 1]
    strides, dil = [1, 1, 1], [1, 1, 1]
    x = dc.create_input_tensor(shape, locale_shape, FILTER, strides, dil, locale)
    fshape = FILTER + [C_IN, K_OUT]
    y = dc.create_convolution_output_tensor(x, fshape, strides, [1, 1, 1], dil)
    z = dc.Tensor(y.shape, locale, y.dist, y._local_of)
    return dict(shape=shape, locale_shape=locale_shape, input=x, conv_out=y, bn_out=z, strides=strides,
                dilations=dil, pads=[1, 1, 1], filter_shape=fshape)


def synth_input_shard(seed, offset_d, local_d, extent):
    """x ~ N(0,1), keyed on (seed, channel, global D index): the same global
    tensor whatever the partitioning."""
    out = np.empty((1, C_IN, local_d, extent, extent), np.float32)
    for c in range(C_IN):
        for d in range(local_d):
            rng = np.random.default_rng([seed, c, offset_d + d])
            out[0, c, d] = rng.standard_normal((extent, extent), dtype=np.float32)
    return out


def synth_filter(seed):
    rng = np.random.default_rng([seed, 12345])
    fan_in = C_IN * 27
    return (rng.standard_normal((K_OUT, C_IN, 3, 3, 3)) * np.sqrt(2.0 / fan_in)).astype(np.float32)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for l in self.proc.stdout:
            self.lines.append(l)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            f = [v.strip() for v in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# --------------------------------------------------------------------------
# CPU arm: the oracle port on host cores, on a bounded D-slab of the workload
# --------------------------------------------------------------------------
def cpu_layer_pass(sample_d, extent, seed=0, repeats=1):
    """One halo-free conv forward + BN forward on a (sample_d x extent x
    extent) slab with the restated CPU arithmetic; returns (seconds, threads)."""
    from oracle import oracle as O

    x = synth_input_shard(seed, 0, sample_d, extent)
    w = synth_filter(seed)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        y = O.conv_fwd(x, w, [1, 1, 1], [1, 1, 1])
        s, q = O.bn_sums(y)
        nps = y.size // K_OUT
        m, v, _, _ = O.bn_sums_to_statistics(s, q, nps, DECAY, np.zeros(K_OUT), np.ones(K_OUT))
        O.bn_normalize(y, m, v, np.ones(K_OUT, np.float32), np.zeros(K_OUT, np.float32), EPS)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best, O.num_threads()


def pick_cpu_sample(extent, target_s=4.0):
    """Calibrate on a thin slab, then size the sample for about target_s."""
    t, _ = cpu_layer_pass(2, extent)
    per_plane = t / 2
    d = int(max(2, min(extent, target_s / max(per_plane, 1e-6))))
    return d


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    extent = EXTENT
    sample_d = pick_cpu_sample(extent, target_s=3.0)
    times = []
    threads = 1
    for i in range(args.warmup + args.steps):
        t, threads = cpu_layer_pass(sample_d, extent)
        if i >= args.warmup:
            times.append(t)
    mean_t = sum(times) / len(times)
    vox = sample_d * extent * extent
    value = vox / mean_t
    sample = f"conv3d fwd + BN fwd on a {sample_d}x{extent}x{extent} D-slab of the 256^3 shard (C=4->K=16), fp64-accumulate port, OpenMP"
    line = {
        "impl": "reference", "metric": "voxels/s per halo+conv3d+BN layer", "value": value, "unit": "voxels/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean_t * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "BASELINE configs[1]: 3-D conv+BN layer, N=1 C=4 256^3 -> K=16 3x3x3 s1 p1, fwd",
                   "partition": "D", "note": "the reference's own CPU backend (ref::Backend) is 4-D/stride-1 only "
                   "and has no BN, so the 5-D workload is timed with the CPU restatement (oracle/)"},
        "cpu_baseline": {"value": value, "unit": "voxels/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "voxels/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    import dihydrogen_b200 as dc
    from dihydrogen_b200 import _abi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("NCCL_DEBUG", "WARN")  # keep NCCL's version banner off stdout
    if world > 1:
        # NCCL writes its version banner to stdout when the first communicator
        # comes up; stdout carries the one JSON line, so point fd 1 at stderr
        # until that has happened
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            warm = torch.zeros(1, device="cuda")
            dist.all_reduce(warm)
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
        locale = dc.Locale.from_torch_distributed()
    else:
        locale = dc.Locale(0, 1)
    _abi.lib()
    # nvidia-smi needs a few hundred ms to start: sample from here on, the
    # timed regions below are what runs while it samples
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    geo = layer_geometry(world, locale, local_d=args.local_d)
    x, y, z = geo["input"], geo["conv_out"], geo["bn_out"]
    for t in (x, y, z):
        t.allocate()
    extent = EXTENT
    local_d = x.local_shape[2]
    host_x = torch.from_numpy(synth_input_shard(0, x.offset[2], local_d, extent)).pin_memory()
    host_z = torch.empty(tuple(reversed(z.local_shape)), dtype=torch.float32).pin_memory()
    w = torch.from_numpy(synth_filter(0)).cuda()
    x.owned().copy_(host_x)

    be = dc.BackendDNNLib(locale, options=dc.Options(overlap_halo_exchange=args.overlap), allreduce="peer",
                          allreduce_max_count=4096)
    conv = dc.Convolution(be, 5)
    conv.setup(x, w, y, None, None, None, geo["pads"], geo["strides"], geo["dilations"])
    bn = dc.BatchNormalization(be, 5, DECAY, EPS, True)
    stats = torch.zeros(2 * K_OUT, device="cuda")
    mean, var = stats[:K_OUT], stats[K_OUT:]
    rm, rv = torch.zeros(K_OUT, device="cuda"), torch.ones(K_OUT, device="cuda")
    scale, bias = torch.ones(K_OUT, device="cuda"), torch.zeros(K_OUT, device="cuda")
    stream = torch.cuda.current_stream()

    launches = {"n": 0}
    partitioned = world > 1

    fuse = not args.no_fused_stats
    overlapped = conv.is_overlap_fwd_halo_exchange_enabled()
    extra_launches = 2 * (len(conv._ov[1]) - 1) if overlapped else 0

    def step():
        # the conv epilogue also delivers the BN statistics of its output
        # (falls back to the separate statistics pass if the plan cannot)
        got = conv.forward(1.0, x, w, 0.0, y, statistics=(mean, var) if fuse else None)
        bn.forward(y, mean, var, rm, rv, scale, bias, z, True, statistics_ready=bool(got))
        # clear_halo (1 per partitioned dim), pack+put and wait+unpack (1 each per
        # partitioned dim), filter image, conv, statistics (fold of the epilogue's
        # partials, or the separate pass), all-reduce, finalize, apply
        # (--overlap: interior + boundary slabs, each with its filter image, and
        # the statistics as their own pass)
        launches["n"] += (3 if partitioned else 0) + 6 + extra_launches
        return got

    def e2e_step():
        x.owned().copy_(host_x, non_blocking=True)
        step()
        host_z.copy_(z.owned(), non_blocking=True)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        launches["n"] = 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            tt = torch.tensor([ms], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        return ms / steps

    ms_step = timed(step, args.steps, max(args.warmup, 3))
    n_launch = launches["n"]
    ms_e2e_serial = timed(e2e_step, max(2, min(args.steps, 5)), 2)

    def e2e_pipelined(steps):
        """The same end-to-end pass the way a host would drive it: the input
        copy of step i+1 and the result copy of step i-1 run on copy streams
        beside the compute of step i (two device buffers each for the input
        shard and the BN output, two pinned result buffers).  Every step still
        copies its own input in and its own result out inside the timed
        region, pipeline fill and drain included."""
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        xb = [x.buffer, torch.zeros_like(x.buffer)]
        zb = [z.buffer, torch.empty_like(z.buffer)]
        hz = [host_z, torch.empty_like(host_z).pin_memory()]
        comp_done, d2h_done = [None, None], [None, None]
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        s_in.wait_stream(stream)
        for i in range(steps):
            b = i & 1
            x.set_view(xb[b])
            z.set_view(zb[b])
            with torch.cuda.stream(s_in):
                if comp_done[b] is not None:
                    s_in.wait_event(comp_done[b])  # the pass that last read this input buffer
                x.owned().copy_(host_x, non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            stream.wait_event(ev_in)
            if d2h_done[b] is not None:
                stream.wait_event(d2h_done[b])  # the copy that last read this output buffer
            step()
            comp_done[b] = torch.cuda.Event()
            comp_done[b].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[b])
                hz[b].copy_(z.owned(), non_blocking=True)
                d2h_done[b] = torch.cuda.Event()
                d2h_done[b].record(s_out)
        for ev in d2h_done:
            if ev is not None:
                stream.wait_event(ev)
        e1.record(stream)
        barrier()
        x.set_view(xb[0])
        z.set_view(zb[0])
        ms = e0.elapsed_time(e1)
        if world > 1:
            tt = torch.tensor([ms], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        return ms / steps

    ms_e2e = e2e_pipelined(max(4, min(args.steps, 8)))

    # per-kernel timing of the forward pass on this rank (rank 0 reports)
    import ctypes

    def time_call(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    fused_ok = bool(step()) if fuse else False
    t_conv = time_call(lambda: conv.forward(1.0, x, w, 0.0, y, skip_halo_exchange=True,
                                            statistics=(mean, var) if fused_ok else None))
    t_stats = time_call(lambda: bn.forward_stage1(y, mean, var, True))
    t_apply = time_call(lambda: bn.forward_stage2(y, mean, var, rm, rv, scale, bias, z, True))
    clocks = sampler.stop() if rank == 0 else None
    st = conv.halo_xch_input.status()
    if st != _abi.OK:
        raise SystemExit("halo exchange reported " + str(st))

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    vox_local = local_d * extent * extent
    vox_total = vox_local * world
    in_el = C_IN * (local_d + (2 if partitioned else 0)) * extent * extent
    out_el = K_OUT * vox_local
    conv_bytes = 4 * (in_el + K_OUT * C_IN * 27 + out_el)
    kernels = {
        "conv_fwd": {"ms": t_conv, "bytes": conv_bytes, "flops": 2 * K_OUT * C_IN * 27 * vox_local},
        "bn_finalize_apply": {"ms": t_apply, "bytes": 8 * out_el},
    }
    if not fused_ok:
        kernels["bn_stats"] = {"ms": t_stats, "bytes": 4 * out_el}
    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the
    # ncu capture of a 64 x 256 x 256 shard, which scales with the D extent:
    # bytes per shard voxel times this launch's voxels.
    ncu_vox = 64 * 256 * 256
    traffic_per_voxel = {"conv_fwd": (69.34e6 + 208.91e6) / ncu_vox, "bn_stats": (268.46e6 + 4.00e6) / ncu_vox,
                         "bn_finalize_apply": (268.45e6 + 222.17e6) / ncu_vox}
    dom = max(kernels, key=lambda k: kernels[k]["ms"])
    ach = kernels[dom]["bytes"] / (kernels[dom]["ms"] * 1e-3) / 1e9
    roofline = {"kernel": dom, "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": ach / peaks["hbm_gbs"], "peak_source": peak_kind, "traffic": traffic_per_voxel[dom] * vox_local,
                "traffic_source": "ncu capture of a 64x256x256 shard scaled by voxels (profiles/)",
                "kernels_ms": {k: round(v["ms"], 4) for k, v in kernels.items()},
                "kernels_gbs": {k: round(v["bytes"] / (v["ms"] * 1e-3) / 1e9, 1) for k, v in kernels.items()},
                "conv_tflops": kernels["conv_fwd"]["flops"] / (t_conv * 1e-3) / 1e12,
                "conv_kernel": "tcgen05" if conv.kernel_kind(0) == 1 else "fp32-simt",
                "bn_statistics": "from the conv epilogue" if fused_ok else "separate pass",
                "bn_stats_separate_pass_ms": round(t_stats, 4)}

    cpu = None
    if world == 1 and not args.skip_cpu:
        sample_d = pick_cpu_sample(extent, target_s=8.0)
        t_cpu, threads = cpu_layer_pass(sample_d, extent)
        cpu = {"value": sample_d * extent * extent / t_cpu, "unit": "voxels/s", "cores": threads, "kind": "port",
               "sample": f"conv3d fwd + BN fwd on a {sample_d}x{extent}x{extent} D-slab of the shard, "
                         f"{t_cpu:.2f} s, fp64-accumulate CPU restatement (the reference's ref::Backend is "
                         "4-D only and has no BN)"}

    line = {
        "metric": "voxels/s per halo+conv3d+BN layer", "value": vox_total / (ms_step * 1e-3), "unit": "voxels/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "BASELINE configs[1]: 3-D conv+BN layer, N=1 C=4 256^3 per GPU -> K=16 3x3x3 s1 p1, "
                               "halo exchange + conv fwd + BN fwd (global stats)"
                               + ("" if args.local_d is None else f" [REDUCED local D={args.local_d}: profiling only]"),
                   "partition": f"D over {world} GPU(s), halo width 1", "global_volume": geo["shape"][:3],
                   "overlap_halo_exchange": bool(overlapped),
                   "l2": "inputs larger than L2 (268 MB in, 1 GiB conv out per GPU)",
                   "allreduce": "peer-memory kernel, 2C floats"},
        "e2e": {"value": vox_total / (ms_e2e * 1e-3), "unit": "voxels/s", "ms_per_step": ms_e2e,
                "ms_per_step_unpipelined": ms_e2e_serial,
                "note": "pinned host -> device input copy, layer pass, device -> pinned host result copy every step; "
                        "copies of neighbouring steps overlap on two copy streams (double-buffered)",
                "h2d_bytes_per_step": int(host_x.numel() * 4), "d2h_bytes_per_step": int(host_z.numel() * 4)},
        "gpu_launches": n_launch,
        "roofline": roofline,
        "clocks": clocks,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-fused-stats", action="store_true",
                    help="run the BN statistics as their own pass instead of taking them from the conv epilogue")
    ap.add_argument("--overlap", action="store_true",
                    help="Options.overlap_halo_exchange: interior convolution while the halo is in flight, then "
                         "the boundary slabs (off by default, as in the reference)")
    ap.add_argument("--local-d", type=int, default=None,
                    help="per-GPU D extent instead of 256 (small case for profiler captures; not a bench value)")
    ap.add_argument("--skip-cpu", action="store_true", help="skip the CPU baseline leg (profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
