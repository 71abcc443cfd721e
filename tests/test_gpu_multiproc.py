"""One process per GPU: the peer-store halo transport over CUDA IPC / NVLink,
both all-reduce flavours and the whole layer, against the oracle.  Needs two
GPUs; skipped on a single-GPU box (the emulated-rank tests cover the logic
there)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_layer_across_processes(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    port = 29600 + os.getpid() % 300 + nproc
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "mp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-4000:]
    for k in range(nproc):
        assert f"mp ok rank {k} of {nproc}" in out, out[-4000:]
