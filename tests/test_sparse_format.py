"""The runtime's optional extra bit-plane ("sparse" weights) on the host: directory format as
the reference's loader reads it (C++/ops/src/arm/parameters.cpp:44-64: weight_mask.bin, the
tails of w_quant.bin and w_scale.bin, sparse_mask_len) and the oracle's statement of what the
reference's kernel adds for a listed block (C++/ops/src/arm/arm_t_mac_kernal.cpp:678-788).
No exporter of the reference writes this format (HLQ.py:180), so there is no reference-made
fixture: the oracle is checked against a bit-by-bit statement of the same sum."""
import json
import os

import numpy as np
import pytest

from elutq_b200 import format as F
from oracle import hlq_oracle as O


def make_sparse(n, k, g, fraction, seed=0):
    rng = np.random.default_rng(seed)
    pairs = [(x, y) for x in range(0, n, 32) for y in range(0, k, g) if rng.random() < fraction]
    mask = np.array(pairs, dtype=np.uint32).reshape(-1, 2)
    p = mask.shape[0]
    return F.SparsePlane(mask, rng.integers(0, 256, (p, 32, g // 8), dtype=np.uint8),
                         (rng.standard_normal((p, 32)) * 0.01).astype(np.float16))


def test_sparse_directory_round_trip_and_layout(tmp_path):
    d = O.synth_linear(96, 512, 2, 128, seed=1)
    sp = make_sparse(96, 512, 128, 0.5, seed=2)
    assert sp.pairs > 0
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], None, 128, sp)
    F.write_export_dir(str(tmp_path), lin)
    cfg = json.load(open(tmp_path / "weight_config.json"))
    dense = 96 * 512 * 2 // 8
    # the sizes the reference's loader computes (parameters.cpp:37-64)
    assert cfg["use_sparse"] is True and cfg["sparse_mask_len"] == 2 * sp.pairs and cfg["base_bit"] == 2
    assert cfg["weight_data_len"] == dense + sp.pairs * 4 * 128 == os.path.getsize(tmp_path / "w_quant.bin")
    assert os.path.getsize(tmp_path / "w_scale.bin") == 2 * (2 * 96 * 512 // 128 + sp.pairs * 32)
    assert os.path.getsize(tmp_path / "weight_mask.bin") == 4 * 2 * sp.pairs
    r = F.read_export_dir(str(tmp_path))
    assert np.array_equal(r.w_quant, lin.w_quant) and r.groupsize == 128
    assert np.array_equal(r.sparse.mask, sp.mask) and np.array_equal(r.sparse.blocks, sp.blocks)
    assert np.array_equal(r.sparse.scales.view(np.uint16), sp.scales.view(np.uint16))
    # a block off the 32-row grid is refused
    bad = np.fromfile(tmp_path / "weight_mask.bin", dtype=np.uint32)
    bad[0] = 8
    bad.tofile(tmp_path / "weight_mask.bin")
    with pytest.raises(ValueError):
        F.read_export_dir(str(tmp_path))


def test_oracle_adds_what_the_kernel_adds():
    n, k, g = 64, 256, 64
    d = O.synth_linear(n, k, 3, g, m=2, seed=3)
    sp = make_sparse(n, k, g, 0.6, seed=4)
    y = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, sparse=(sp.mask, sp.blocks, sp.scales))
    y0 = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g)
    # bit by bit: out[x + r] += scale[r] * sum over the group of bit * activation
    extra = np.zeros_like(y0)
    xf = d["x"].astype(np.float64)
    for p in range(sp.pairs):
        x0, c0 = int(sp.mask[p, 0]), int(sp.mask[p, 1])
        for r in range(32):
            for c in range(g):
                if (int(sp.blocks[p, r, c // 8]) >> (c % 8)) & 1:
                    extra[:, x0 + r] += float(sp.scales[p, r]) * xf[:, c0 + c]
    assert np.abs((y - y0) - extra).max() <= 1e-12
