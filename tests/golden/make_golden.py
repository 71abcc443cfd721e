"""Generates the golden fixtures in this folder from the reference itself.

Run where the DiHydrogen tree is available (the REFERENCE variable of oracle/Makefile):

    make -C oracle ref REFERENCE=<DiHydrogen tree> && python tests/golden/make_golden.py

It drives ``oracle/_ref/ref_driver`` -- the reference's own header-only CPU
code compiled where it lies (tensor model, get_halo_sizes, output-shape
helpers, Convolution<ref::Backend>) -- and stores

* ``geom_<name>.txt``: per-rank local shape, halo-extended shape, global
  offset, halo widths and conv-output geometry printed by the reference;
* ``conv_<name>.npz``: seeded inputs and the reference's forward /
  backward-data / backward-filter outputs for small 4-D stride-1 problems
  (all ref::Backend supports).

The fixtures are small (a few hundred KB in total) and travel with the repo;
nothing at test time reads the reference tree.
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
DRIVER = os.path.join(ROOT, "oracle", "_ref", "ref_driver")

# name: (shape W..N, locale W..N, filter W.., strides W.., pad flag, K)
GEOM_CASES = {
    "cfg1_2d_h2": ([64, 64, 16, 4], [1, 2, 1, 1], [3, 3], [1, 1], 1, 16),
    "cfg2_3d_d8": ([256, 256, 256, 4, 1], [1, 1, 8, 1, 1], [3, 3, 3], [1, 1, 1], 1, 16),
    "cfg2_3d_d4": ([256, 256, 256, 4, 1], [1, 1, 4, 1, 1], [3, 3, 3], [1, 1, 1], 1, 16),
    "cfg2_3d_d2": ([256, 256, 256, 4, 1], [1, 1, 2, 1, 1], [3, 3, 3], [1, 1, 1], 1, 16),
    "cfg3_l1_222": ([512, 512, 512, 4, 1], [2, 2, 2, 1, 1], [3, 3, 3], [1, 1, 1], 1, 16),
    "cfg3_l2_222_s2": ([512, 512, 512, 16, 1], [2, 2, 2, 1, 1], [3, 3, 3], [2, 2, 2], 1, 32),
    "cfg4_2d_w4h2_f5": ([4096, 4096, 32, 2], [4, 2, 1, 1], [5, 5], [1, 1], 1, 32),
    "uneven_3d_223_s2": ([16, 16, 17, 4, 1], [2, 2, 3, 1, 1], [3, 3, 3], [2, 2, 2], 1, 8),
    "uneven_2d_h3": ([10, 13, 3, 2], [1, 3, 1, 1], [3, 3], [1, 1], 1, 4),
    "uneven_2d_w3h2_f5": ([23, 19, 2, 2], [3, 2, 1, 1], [5, 5], [1, 1], 1, 3),
    "nopad_2d_h2": ([12, 12, 2, 1], [1, 2, 1, 1], [3, 3], [1, 1], 0, 3),
    "s2_2d_h4": ([32, 30, 2, 1], [1, 4, 1, 1], [3, 3], [2, 2], 1, 3),
    "s2_2d_h4_f5": ([32, 31, 2, 1], [1, 4, 1, 1], [5, 5], [2, 2], 1, 3),
    "single_3d": ([8, 8, 8, 2, 1], [1, 1, 1, 1, 1], [3, 3, 3], [1, 1, 1], 1, 4),
}

# name: (N, C, H, W, K, f, locale(W,H,C,N), seed)
CONV_CASES = {
    "tiny_h2": (2, 3, 12, 10, 4, 3, [1, 2, 1, 1], 0),
    "tiny_w2h2_f5": (1, 2, 14, 16, 3, 5, [2, 2, 1, 1], 1),
    "tiny_h3_uneven": (2, 2, 13, 9, 5, 3, [1, 3, 1, 1], 2),
    "cfg1_lite_h2": (2, 8, 32, 32, 8, 3, [1, 2, 1, 1], 3),
    "single": (1, 3, 9, 11, 2, 3, [1, 1, 1, 1], 4),
}


def run_geom(shape, locale, filt, strides, pad, K):
    nd = len(shape)
    args = [DRIVER, "geom", str(nd), *map(str, shape), *map(str, locale), *map(str, filt), *map(str, strides),
            str(pad), str(K)]
    return subprocess.check_output(args).decode()


def make_conv_inputs(N, C, H, W, K, f, seed):
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = rng.normal(0, 0.1, (K, C, f, f)).astype(np.float32)
    dy = rng.normal(0, 1, (N, K, H, W)).astype(np.float32)
    return x, w, dy


def run_conv(N, C, H, W, K, f, locale, seed):
    x, w, dy = make_conv_inputs(N, C, H, W, K, f, seed)
    with tempfile.TemporaryDirectory() as d:
        x.tofile(d + "/x.bin")
        w.tofile(d + "/w.bin")
        dy.tofile(d + "/dy.bin")
        with open(d + "/spec.txt", "w") as fh:
            fh.write(f"4 {W} {H} {C} {N} {' '.join(map(str, locale))} {f} {f} 1 1 1 {K}\n")
        subprocess.check_call([DRIVER, "conv", d], stdout=subprocess.DEVNULL)
        y = np.fromfile(d + "/y.bin", np.float32).reshape(N, K, H, W)
        dx = np.fromfile(d + "/dx.bin", np.float32).reshape(N, C, H, W)
        dw = np.fromfile(d + "/dw.bin", np.float32).reshape(K, C, f, f)
    return dict(x=x, w=w, dy=dy, y=y, dx=dx, dw=dw, locale=np.array(locale), seed=np.array(seed))


def main():
    if not os.path.exists(DRIVER):
        sys.exit("build oracle/_ref/ref_driver first: make -C oracle ref REFERENCE=<DiHydrogen tree>")
    for name, case in GEOM_CASES.items():
        txt = "# " + " ".join(map(str, case)) + "\n" + run_geom(*case)
        with open(os.path.join(HERE, f"geom_{name}.txt"), "w") as f:
            f.write(txt)
    for name, case in CONV_CASES.items():
        np.savez_compressed(os.path.join(HERE, f"conv_{name}.npz"), **run_conv(*case))
    print("wrote", len(GEOM_CASES), "geometry and", len(CONV_CASES), "conv fixtures")


if __name__ == "__main__":
    main()
