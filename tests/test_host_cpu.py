"""Host-side logic of the product (no GPU): geometry of the Python mirror
against fixtures printed by the reference's own headers, the C ABI's symbol
table, and the 2-rank set-up path over gloo."""
import ctypes
import os
import re
import subprocess
import sys

import pytest

from conftest import GOLDEN, ROOT, geom_fixtures, parse_geom

import dihydrogen_b200 as dc
from dihydrogen_b200 import _abi


def _tensors_for(case, rank):
    shape, locale, filt, strides, pad, K = case
    nsd = len(shape) - 2
    nranks = 1
    for l in locale:
        nranks *= l
    loc = dc.Locale(rank, nranks)
    dil = [1] * nsd
    inp = dc.create_input_tensor(shape, locale, filt, strides, dil, loc)
    fshape = list(filt) + [shape[-2], K]
    pads = [(f - 1) // 2 if pad else 0 for f in filt]
    out = dc.create_convolution_output_tensor(inp, fshape, strides, pads, dil)
    dout = dc.create_convolution_d_output_tensor(out, fshape, dil)
    return inp, out, dout, dil


@pytest.mark.parametrize("fname", geom_fixtures())
def test_tensor_geometry_matches_reference(fname):
    case, ranks = parse_geom(os.path.join(GOLDEN, fname))
    shape, locale, filt, strides, pad, K = case
    nsd = len(shape) - 2
    for ref in ranks:
        inp, out, dout, dil = _tensors_for(case, ref["rank"])
        assert inp.get_local_shape() == ref["local"]
        assert inp.get_local_real_shape() == ref["real"]
        assert inp.get_global_index() == ref["offset"]
        fs, bs, fr, br = dc.get_halo_sizes(inp, filt, strides, dil, bool(pad))
        assert fs[:nsd] == ref["fwd_send"] and bs[:nsd] == ref["bwd_send"]
        assert fr[:nsd] == ref["fwd_recv"] and br[:nsd] == ref["bwd_recv"]
        assert out.get_shape() == ref["out_shape"]
        assert out.get_local_shape() == ref["out_local"]
        assert out.get_global_index() == ref["out_offset"]
        assert dout.get_local_real_shape() == ref["dout_real"]
        assert int(inp.is_split_root()) == ref["split_root"]


def test_rank_grid_order_dim0_fastest():
    """tensor_mpi.hpp:47-56."""
    d = dc.Distribution.make_distribution([2, 3, 1, 1])
    assert dc.Locale(0, 6).get_rank_idx(d) == [0, 0, 0, 0]
    assert dc.Locale(1, 6).get_rank_idx(d) == [1, 0, 0, 0]
    assert dc.Locale(2, 6).get_rank_idx(d) == [0, 1, 0, 0]
    assert dc.Locale(5, 6).get_rank_idx(d) == [1, 2, 0, 0]


def test_distribution_fixup_overlap():
    """distribution.hpp:236-243: overlap only survives on distributed dims."""
    d = dc.Distribution.make_overlapped_distribution([1, 2, 1, 1], [1, 1, 0, 0])
    assert d.get_overlap() == [0, 1, 0, 0]
    assert d.is_distributed(1) and not d.is_distributed(0)


def test_abi_library_exports_every_declared_symbol():
    lib = _abi.lib()
    hdr = open(os.path.join(ROOT, "include", "dcb.h")).read()
    declared = set(re.findall(r"^(?:int32_t|int64_t|const char\*)\s+(dcb_[a-z0-9_]+)\s*\(", hdr, re.M))
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in dcb.h but not exported"
    assert declared == set(_abi.EXPORTED_SYMBOLS)
    assert lib.dcb_version() >= 100
    assert lib.dcb_status_string(_abi.PEER_TIMEOUT) == b"DCB_PEER_TIMEOUT"


def test_abi_rejects_bad_arguments_without_a_gpu():
    lib = _abi.lib()
    assert lib.dcb_set_wait_budget_ns(0) == _abi.BAD_ARG
    d = _abi.TensorDesc()
    d.ndims = 3
    assert lib.dcb_clear_halo(ctypes.byref(d), ctypes.c_void_p(16), 0, None) == _abi.BAD_ARG
    assert b"ndims" in lib.dcb_last_error()


_GLOO_SCRIPT = r"""
import os, sys
sys.path.insert(0, {root!r})
import torch.distributed as dist
import dihydrogen_b200 as dc
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
loc = dc.Locale.from_torch_distributed()
blobs = loc.allgather(bytes([loc.rank]) * 4)
assert blobs == [b"\x00" * 4, b"\x01" * 4], blobs
shape, locale = [64, 64, 16, 4], [1, 2, 1, 1]
t = dc.create_input_tensor(shape, locale, [3, 3], [1, 1], [1, 1], loc)
assert t.get_local_shape() == [64, 32, 16, 4] and t.get_local_real_shape() == [64, 34, 16, 4]
assert t.get_global_index() == [0, 32 * loc.rank, 0, 0]
# peers as HaloExchange::find_peer_rank computes them, without touching a device
hx = dc.HaloExchange.__new__(dc.HaloExchange)
hx.tensor = t
peers = [hx.find_peer_rank(1, s) for s in (0, 1)]
assert peers == ([-1, 1] if loc.rank == 0 else [0, -1]), peers
# weak-scaling shard layout used by bench.py
import bench
assert bench.grid_for(2, "auto") == [1, 1, 2] and bench.grid_for(4, "auto") == [1, 2, 2]
assert bench.grid_for(8, "auto") == [2, 2, 2] and bench.grid_for(8, "d") == [1, 1, 8]
g = bench.layer_geometry(bench.grid_for(2, "auto"), loc, extent=16)
assert g["shape"][2] == 32 and g["input"].get_local_shape()[2] == 16
# a W-partitioned shard pads its rows to 16 bytes (the pitch), others stay dense
tw = dc.create_input_tensor([36, 8, 4, 2], [2, 1, 1, 1], [3, 3], [1, 1], [1, 1], loc)
# the owned cells start on a 16-byte boundary: 3 floats of lead, then the halo cell
assert tw.get_local_real_shape()[0] == 20 and tw.lead == 3 and tw.get_pitch() == 24
tw = dc.create_input_tensor([34, 8, 4, 2], [2, 1, 1, 1], [3, 3], [1, 1], [1, 1], loc)
assert tw.get_local_real_shape()[0] == 19 and tw.get_pitch() == 24 and tw.get_strides() == [1, 24, 192, 768]
assert tw.get_local_pitched_shape() == [24, 8, 4, 2] and tw.desc().pitch == 24
tw.allocate(device="cpu")
assert tuple(tw.buffer.shape) == (2, 4, 8, 19) and tw.buffer.stride() == (768, 192, 24, 1)
assert tw.owned().data_ptr() % 16 == 0 and tw.get_buffer() % 16 == 12
assert t.get_pitch() == 64 and g["input"].get_pitch() == 16
# dump_tensor: rank 0 writes the global tensor, no halos, dimension 0 fastest
import numpy as np
g5 = np.arange(6 * 8 * 4 * 2, dtype=np.float32).reshape(2, 4, 8, 6)  # N, C, H, W
td = dc.create_input_tensor([6, 8, 4, 2], [1, 2, 1, 1], [3, 3], [1, 1], [1, 1], loc)
td.allocate(device="cpu")
td.buffer.fill_(-1.0)
import torch
td.owned().copy_(torch.from_numpy(g5[:, :, 4 * loc.rank:4 * loc.rank + 4, :].copy()))
assert dc.distconv.owned_box(td, 1) == ([0, 4, 0, 0], [6, 4, 4, 2])
dc.dump_tensor(td, {dump!r}, binary=True)
dc.dump_tensor(td, {dump!r}, binary=False)
dist.barrier()
if loc.rank == 0:
    assert np.array_equal(np.fromfile({dump!r} + ".out", np.float32), g5.ravel())
    assert np.array_equal(np.loadtxt({dump!r} + ".txt", dtype=np.float32), g5.ravel())
dist.barrier()
print("ok", loc.rank)
"""


def test_two_rank_setup_over_gloo(tmp_path):
    port = 29500 + os.getpid() % 2000
    script = tmp_path / "gloo2.py"
    script.write_text(_GLOO_SCRIPT.format(root=ROOT, port=port, dump=str(tmp_path / "dump")))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, cwd=ROOT) for r in range(2)]
    outs = [p.communicate(timeout=240)[0].decode() for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o
        assert f"ok {r}" in o


def test_options_environment_overrides(monkeypatch):
    """legacy/src/dnn_backend/options.cpp:13-71: a DISTCONV_* variable that is
    set, whatever its value, switches its option on."""
    import dihydrogen_b200 as dc

    for k in ("DISTCONV_OVERLAP_HALO_EXCHANGE", "DISTCONV_DETERMINISTIC", "DISTCONV_ENABLE_PROFILING",
              "DISTCONV_PROFILING", "DISTCONV_NVTX", "DISTCONV_WS_CAPACITY_FACTOR"):
        monkeypatch.delenv(k, raising=False)
    o = dc.Options(deterministic=False)
    assert not (o.overlap_halo_exchange or o.deterministic or o.enable_profiling) and o.ws_capacity_factor == 1.0
    monkeypatch.setenv("DISTCONV_OVERLAP_HALO_EXCHANGE", "0")
    monkeypatch.setenv("DISTCONV_DETERMINISTIC", "1")
    monkeypatch.setenv("DISTCONV_NVTX", "")
    monkeypatch.setenv("DISTCONV_WS_CAPACITY_FACTOR", "2.5")
    o = dc.Options(deterministic=False)
    assert o.overlap_halo_exchange and o.deterministic and o.enable_profiling and o.ws_capacity_factor == 2.5
