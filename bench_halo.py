#!/usr/bin/env python
"""Halo-exchange sweep (BASELINE.json configs[4]): fp32 5-D tensors, N=1,
C in {4,16,64}, S in {128,256,512}, halo width in {1,2,3}.

    python bench_halo.py [--max-gb G] [--reps R]                 # one GPU
    python -m torch.distributed.run --nproc-per-node P ... bench_halo.py

One GPU: two ranks are emulated in the process (their receive slabs live on the
same device), partitioned along W, H or D in turn, so every face orientation
is measured.  The two halves of an exchange are timed apart: "pack+put" reads
the strided face and stores it into the neighbour's slab, "wait+unpack" copies
the slab into the halo cells.  Each moves 4E bytes in and 4E out per face
(E = width x product of the other real extents), so GB/s = 8E x faces / time is
the HBM figure.  All ranks put before any rank waits, so no kernel ever waits
for a kernel that has not been launched.

P GPUs (torchrun): real ranks, S^3 split along D; the whole exchange is timed
(max over ranks) and the bytes of one face (4E) over that time is the NVLink
figure per direction of one neighbour pair; with more than two ranks an interior
rank sends and receives two faces, which `nvlink_GBs_egress_busiest_gpu` counts.
With `--grid w,h,d` the S^3 volume is partitioned in two or three dimensions and the
ordered W, H, D exchange is timed as a whole; the figure is the bytes one GPU sends
over that time.

The payload is the global-offset fill of the reference's halo test, and every
configuration is checked for exact halo contents after the timed runs.
Prints one JSON line per configuration and a last summary line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def global_offset_fill(t, torch):
    """Owned cell <- its global linear offset modulo 2^24 (exact in fp32)."""
    ls = t.local_shape  # W,H,D,C,N
    idx = [torch.arange(ls[i], device="cuda", dtype=torch.int64) + t.offset[i] for i in range(5)]
    sh = t.shape
    lin = idx[4].view(-1, 1, 1, 1, 1)
    for i in (3, 2, 1, 0):
        v = [1, 1, 1, 1, 1]
        v[4 - i] = -1
        lin = lin * sh[i] + idx[i].view(*v)
    t.owned().copy_((lin % (1 << 24)).to(torch.float32))


def check_halo(t, dim, torch):
    """The halo cells along `dim` must hold the neighbour's global offsets."""
    ls, ov, sh = t.local_shape, t.dist.overlap, t.shape
    w = ov[dim]
    full = t.buffer.view(tuple(reversed(t.get_local_real_shape())))
    ok = True
    for side in (0, 1):
        lo = t.offset[dim] - w if side == 0 else t.offset[dim] + ls[dim]
        if lo < 0 or lo + w > sh[dim]:
            continue
        rng = [torch.arange(ls[i], device="cuda", dtype=torch.int64) + t.offset[i] for i in range(5)]
        rng[dim] = torch.arange(w, device="cuda", dtype=torch.int64) + lo
        lin = rng[4].view(-1, 1, 1, 1, 1)
        for i in (3, 2, 1, 0):
            v = [1, 1, 1, 1, 1]
            v[4 - i] = -1
            lin = lin * sh[i] + rng[i].view(*v)
        sl = []
        for i in (4, 3, 2, 1, 0):
            if i == dim:
                start = 0 if side == 0 else ov[i] + ls[i]
                sl.append(slice(start, start + w))
            else:
                sl.append(slice(ov[i], ov[i] + ls[i]))
        ok = ok and bool(torch.equal(full[tuple(sl)], (lin % (1 << 24)).to(torch.float32)))
    return ok


def make_tensor(dc, shape, locale_shape, width, locale):
    ov = [width if locale_shape[i] > 1 else 0 for i in range(5)]
    t = dc.Tensor(shape, locale, dc.Distribution.make_overlapped_distribution(locale_shape, ov))
    t.allocate()
    return t


def run_emulated(args, torch, dc):
    from dihydrogen_b200 import _abi

    results = []
    locs = [dc.Locale(r, 2) for r in range(2)]
    for C in args.channels:
        for S in args.sizes:
            if 2 * C * S ** 3 * 4 / 1e9 > args.max_gb:
                continue
            for width in args.widths:
                for dim in (0, 1, 2):
                    shape = [S, S, S, C, 1]
                    ls = [1, 1, 1, 1, 1]
                    ls[dim] = 2
                    ts = [make_tensor(dc, shape, ls, width, l) for l in locs]
                    for t in ts:
                        global_offset_fill(t, torch)
                    hx = [dc.HaloExchange(t) for t in ts]
                    blobs = [h.export() for h in hx]
                    for h in hx:
                        h.connect(blobs)
                    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                    t_put = t_unpack = 0.0
                    for it in range(args.reps + 3):
                        ev[0].record()
                        for h in hx:
                            h.pack_put(dim)
                        ev[1].record()
                        for h in hx:
                            h.wait_unpack(dim)
                        ev[2].record()
                        torch.cuda.synchronize()
                        if it >= 3:
                            t_put += ev[0].elapsed_time(ev[1])
                            t_unpack += ev[1].elapsed_time(ev[2])
                    exact = all(check_halo(t, dim, torch) for t in ts)
                    status = max(h.status() for h in hx)
                    real = ts[0].get_local_real_shape()
                    E = width * C
                    for i in range(3):
                        if i != dim:
                            E *= real[i]
                    faces = 2  # rank 0 sends its RHS face, rank 1 its LHS face
                    r = {"mode": "1gpu-emulated-2-ranks", "C": C, "S": S, "width": width, "dim": "WHD"[dim],
                         "face_MB": 4 * E / 1e6,
                         "pack_put_us": 1e3 * t_put / args.reps, "wait_unpack_us": 1e3 * t_unpack / args.reps,
                         "pack_put_GBs": 8 * E * faces / (t_put / args.reps * 1e-3) / 1e9,
                         "wait_unpack_GBs": 8 * E * faces / (t_unpack / args.reps * 1e-3) / 1e9,
                         "exact": exact, "status": status}
                    print(json.dumps(r), flush=True)
                    results.append(r)
                    del hx, ts
                    torch.cuda.empty_cache()
                    if not exact or status != _abi.OK:
                        raise SystemExit("halo contents differ from the global-offset fill")
    return results


def run_ranks(args, torch, dc, dist, world, rank):
    from dihydrogen_b200 import _abi

    locale = dc.Locale.from_torch_distributed()
    results = []
    for C in args.channels:
        for S in args.sizes:
            if C * S ** 3 * 4 / world / 1e9 > args.max_gb:
                continue
            for width in args.widths:
                shape, ls = [S, S, S, C, 1], [1, 1, world, 1, 1]
                if args.grid:
                    ls = list(args.grid) + [1, 1]
                t = make_tensor(dc, shape, ls, width, locale)
                global_offset_fill(t, torch)
                hx = dc.HaloExchange(t).setup()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                total = 0.0
                for it in range(args.reps + 3):
                    torch.cuda.synchronize()
                    dist.barrier()
                    torch.cuda.synchronize()
                    e0.record()
                    hx.exchange()
                    e1.record()
                    torch.cuda.synchronize()
                    if it >= 3:
                        total += e0.elapsed_time(e1)
                ms = torch.tensor([total / args.reps], device="cuda")
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                parts = [d for d in range(3) if ls[d] > 1]
                good = torch.tensor([1 if (all(check_halo(t, d, torch) for d in parts)
                                           and hx.status() == _abi.OK) else 0], device="cuda")
                dist.all_reduce(good, op=dist.ReduceOp.MIN)
                if args.grid:
                    # cells a rank with neighbours on every side sends: the face of dimension d spans the
                    # owned cells of the later dimensions and the halo-extended ones of the earlier (the
                    # exchanges run in the order W, H, D, so that edges and corners travel on)
                    sent = 0
                    for d in parts:
                        e = width * C
                        for o in range(3):
                            if o != d:
                                e *= S // ls[o] + (2 * width if (o < d and ls[o] > 1) else 0)
                        sent += e * (2 if ls[d] > 2 else 1)
                    r = {"mode": f"{world}gpu-grid-" + "x".join(str(v) for v in ls[:3]), "C": C, "S": S,
                         "width": width, "dim": "".join("WHD"[d] for d in parts), "sent_MB_per_gpu": 4 * sent / 1e6,
                         "exchange_us": 1e3 * float(ms.item()),
                         "nvlink_GBs_per_direction": 4 * sent / (float(ms.item()) * 1e-3) / 1e9,
                         "exact": bool(good.item())}
                    if rank == 0:
                        print(json.dumps(r), flush=True)
                    results.append(r)
                    dist.barrier()
                    del hx, t
                    torch.cuda.empty_cache()
                    if not r["exact"]:
                        raise SystemExit("halo contents differ from the global-offset fill")
                    continue
                E = width * C * S * S
                r = {"mode": f"{world}gpu-D-partition", "C": C, "S": S, "width": width, "dim": "D",
                     "face_MB": 4 * E / 1e6, "exchange_us": 1e3 * float(ms.item()),
                     "nvlink_GBs_per_direction": 4 * E / (float(ms.item()) * 1e-3) / 1e9,
                     # a rank with a neighbour on both sides sends (and receives) two faces per exchange
                     "nvlink_GBs_egress_busiest_gpu": (2 if world > 2 else 1) * 4 * E / (float(ms.item()) * 1e-3) / 1e9,
                     "exact": bool(good.item())}
                if rank == 0:
                    print(json.dumps(r), flush=True)
                results.append(r)
                dist.barrier()
                del hx, t
                torch.cuda.empty_cache()
                if not r["exact"]:
                    raise SystemExit("halo contents differ from the global-offset fill")
    if not args.grid:
        results += run_shuffle(args, torch, dc, dist, world, rank, locale)
    return results


def run_shuffle(args, torch, dc, dist, world, rank, locale):
    """Re-distribution sample-parallel -> D-partitioned and back (C=16, N=world
    samples of 128^3 / 256^3): every rank sends (world-1)/world of its shard over
    NVLink.  Checked bit-exact against the round trip."""
    from dihydrogen_b200 import _abi

    out = []
    for S in (128, 256):
        shape = [S, S, S, 16, world]
        if 4.0 * S ** 3 * 16 / 1e9 > args.max_gb:
            continue
        ts = dc.Tensor(shape, locale, dc.Distribution.make_overlapped_distribution([1, 1, 1, 1, world], [0] * 5))
        td = dc.Tensor(shape, locale, dc.Distribution.make_overlapped_distribution([1, 1, world, 1, 1], [0, 0, 1, 0, 0]))
        tb = dc.Tensor(shape, locale, dc.Distribution.make_overlapped_distribution([1, 1, 1, 1, world], [0] * 5))
        for t in (ts, td, tb):
            t.allocate()
        ts.buffer.normal_()
        shf = dc.TensorShuffler(ts, td)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        total = 0.0
        for it in range(args.reps + 3):
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            e0.record()
            shf.shuffle_forward(ts.get_buffer(), td.get_buffer())
            e1.record()
            torch.cuda.synchronize()
            if it >= 3:
                total += e0.elapsed_time(e1)
            shf.shuffle_backward(td.get_buffer(), tb.get_buffer())
        torch.cuda.synchronize()
        ms = torch.tensor([total / args.reps], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        good = torch.tensor([1 if (torch.equal(tb.buffer, ts.buffer) and shf.status("fwd") == _abi.OK
                                   and shf.status("bwd") == _abi.OK) else 0], device="cuda")
        dist.all_reduce(good, op=dist.ReduceOp.MIN)
        sent = 4.0 * ts.buffer.numel() * (world - 1) / world
        r = {"mode": f"{world}gpu-shuffle sample->D", "C": 16, "S": S, "width": 0, "dim": "N->D",
             "shard_MB": 4.0 * ts.buffer.numel() / 1e6, "shuffle_us": 1e3 * float(ms.item()),
             "nvlink_GBs_per_direction": sent / (float(ms.item()) * 1e-3) / 1e9, "exact": bool(good.item())}
        if rank == 0:
            print(json.dumps(r), flush=True)
        out.append(r)
        dist.barrier()
        del shf, ts, td, tb
        torch.cuda.empty_cache()
        if not r["exact"]:
            raise SystemExit("the re-distribution round trip changed the tensor")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--channels", type=int, nargs="+", default=[4, 16, 64])
    ap.add_argument("--sizes", type=int, nargs="+", default=[128, 256, 512])
    ap.add_argument("--widths", type=int, nargs="+", default=[1, 2, 3])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--grid", type=lambda v: [int(x) for x in v.split(",")], default=None,
                    help="ranks along W,H,D (torchrun only; their product is the world size): the whole "
                         "ordered exchange of a 2-D / 3-D partition instead of the split along D")
    ap.add_argument("--max-gb", type=float, default=20.0,
                    help="skip configurations whose tensors exceed this many GB on one device")
    args = ap.parse_args()
    import torch

    import dihydrogen_b200 as dc

    if not torch.cuda.is_available():
        raise SystemExit("bench_halo.py needs a CUDA device")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        if args.grid and (len(args.grid) != 3 or args.grid[0] * args.grid[1] * args.grid[2] != world):
            raise SystemExit("--grid w,h,d must multiply to the world size")
        res = run_ranks(args, torch, dc, dist, world, rank)
        key = "nvlink_GBs_per_direction"
    else:
        res = run_emulated(args, torch, dc)
        key = "pack_put_GBs"
    if rank == 0 and res:
        best = max(res, key=lambda r: r[key])
        print(json.dumps({"summary": True, "configs": len(res), "best_" + key: best[key],
                          "best_config": {k: best[k] for k in ("C", "S", "width", "dim")}}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
