import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def parse_geom(path):
    """Parses a geom_*.txt fixture written by the reference's own headers
    (oracle/ref_driver.cpp `geom`).  Returns (case tuple, list of per-rank dicts)."""
    import ast

    with open(path) as f:
        lines = [l.strip() for l in f if l.strip()]
    hdr = lines[0][1:].strip()
    # "[shape] [locale] [filter] [strides] pad K"
    parts = hdr.replace("] [", "]|[").replace("] ", "]|", 1)
    lists = []
    rest = hdr
    while rest.startswith("["):
        end = rest.index("]") + 1
        lists.append(ast.literal_eval(rest[:end]))
        rest = rest[end:].strip()
    pad, K = (int(v) for v in rest.split())
    case = (*lists, pad, K)
    ranks = []
    for l in lines[1:]:
        toks = l.split()
        d = {}
        for k, v in zip(toks[0::2], toks[1::2]):
            d[k] = [int(x) for x in v.split(",")] if k not in ("rank", "split_root") else int(v)
        ranks.append(d)
    return case, ranks


def geom_fixtures():
    return sorted(f for f in os.listdir(GOLDEN) if f.startswith("geom_"))


def conv_fixtures():
    return sorted(f for f in os.listdir(GOLDEN) if f.startswith("conv_"))
