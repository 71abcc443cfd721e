"""The C++ host side (include/distconv_b200.hpp): it must compile and link
against the C ABI on a machine without a GPU, and on a GPU the compiled check
program runs one conv + batch-norm layer through DistConv's class names with
the ranks as host threads."""
import os
import shutil
import subprocess

import pytest

import dihydrogen_b200.build as build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "dihydrogen_b200")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _compile(out, source="shim_layer_check.cpp", extra=()):
    build.build()
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), *extra,
           "-I", os.path.join(CUDA, "include"), os.path.join(ROOT, "tests", "cpp", source),
           "-o", str(out), "-L", PKG, "-ldistconv_b200", "-L", os.path.join(CUDA, "lib64"), "-lcudart", "-pthread",
           "-Wl,-rpath," + PKG]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return str(out)


MPI_SHIM = ("-I", os.path.join(ROOT, "oracle", "mpi_shim"))


@pytest.mark.skipif(shutil.which("g++") is None, reason="no g++")
def test_shim_compiles_and_links(tmp_path):
    exe = _compile(tmp_path / "shim_layer_check")
    assert os.path.exists(exe)


@pytest.mark.gpu
@pytest.mark.parametrize("ranks", [1, 2, 4])
def test_shim_layer(tmp_path, ranks):
    exe = _compile(tmp_path / "shim_layer_check")
    r = subprocess.run([exe, str(ranks)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "shim_layer_check OK" in r.stdout, r.stdout + r.stderr


@pytest.mark.skipif(shutil.which("g++") is None, reason="no g++")
def test_shim_with_mpi_constructors_compiles_and_links(tmp_path):
    """LocaleMPI(MPI_Comm) and DNNBackend(MPI_Comm, Handle_t, Stream_t, Options)
    exist behind DISTCONV_B200_HAS_MPI; compiled here against the thread-rank
    mpi.h stand-in that the oracle's reference driver uses."""
    exe = _compile(tmp_path / "shim_mpi_check", "shim_mpi_check.cpp", MPI_SHIM)
    assert os.path.exists(exe)


@pytest.mark.gpu
def test_shim_with_mpi_constructors(tmp_path):
    exe = _compile(tmp_path / "shim_mpi_check", "shim_mpi_check.cpp", MPI_SHIM)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "shim_mpi_check OK" in r.stdout, r.stdout + r.stderr
