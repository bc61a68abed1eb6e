import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def golden_cases():
    return sorted(f[:-4] for f in os.listdir(GOLDEN) if f.endswith(".npz") and f.startswith("w"))


def load_golden(name):
    d = dict(np.load(os.path.join(GOLDEN, name + ".npz")))
    q, n, k, g = int(d["q"]), int(d["n"]), int(d["k"]), int(d["g"])
    d["quantized_w"] = np.unpackbits(d["quantized_w"])[: n * k * q].reshape(n, k, q)
    d["requant_out"] = np.unpackbits(d["requant_out"])[: n * k * q].reshape(n * (k // g), g, q)
    d["export_w_quant"] = d["export_w_quant"].reshape(q, n, k // 8)
    d["export_w_scale"] = d["export_w_scale"].view(np.float16).reshape(q, n, k // g)
    d["export_w_zero"] = d["export_w_zero"].view(np.float16).reshape(n, k // g)
    d.update(q=q, n=n, k=k, g=g, m=int(d["m"]))
    d.setdefault("bias_f16", None)
    return d


@pytest.fixture(scope="session")
def built_lib():
    """The in-tree shared library; built on demand (nvcc cross-compiles without a GPU)."""
    from elutq_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.lib()


@pytest.fixture(scope="session")
def cpu_oracle_lib():
    from oracle import build as obuild
    obuild.build()
    from oracle import cpu_baseline
    return cpu_baseline
