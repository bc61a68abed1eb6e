"""The C ABI on the host: symbols, packing, the streaming re-layout, the export format and
argument checking.  No CUDA call is made here."""
import os
import re

import numpy as np
import pytest

from conftest import GOLDEN, ROOT, golden_cases, load_golden
from elutq_b200 import _lib, format as F
from oracle import hlq_oracle as O


def test_library_exports_every_declared_symbol(built_lib):
    header = open(os.path.join(ROOT, "include", "hlq_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(hlq_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(built_lib, name), f"{name} is declared but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes table and header disagree"
    assert built_lib.hlq_abi_version() == 1


def test_status_strings(built_lib):
    assert built_lib.hlq_last_error_string(0) == b"ok"
    for code in range(1, 9):
        assert len(built_lib.hlq_last_error_string(code)) > 4
    assert b"unknown" in built_lib.hlq_last_error_string(99)


def test_kernel_selectors_check_their_argument(built_lib):
    """The process-wide kernel selectors (for tests and measurements) take 0 .. their last kernel
    and refuse anything else without changing the selection."""
    for fn, last in ((built_lib.hlq_select_batch_kernel, 3), (built_lib.hlq_select_prefill_kernel, 2)):
        for which in range(last + 1):
            assert fn(which) == 0
        assert fn(0) == 0
        for bad in (-1, last + 1, 99):
            assert fn(bad) == 1          # HLQ_ERR_INVALID_ARGUMENT


def test_workspace_size_grows_with_the_rows(built_lib):
    """A workspace sized for m rows serves every call with at most m rows: the size never shrinks
    as m grows (also across the row counts at which another kernel takes over)."""
    for (k, n, q, g) in [(2048, 640, 2, 64), (4096, 4096, 3, 128), (8192, 28672, 2, 128), (512, 128, 4, 32)]:
        prev = 0
        for m in range(1, 600):
            b = built_lib.hlq_workspace_bytes(m, k, n, q, g)
            assert b >= prev, (m, k, n, q, g)
            prev = b


def test_pack_matches_reference_bytes(built_lib):
    d = np.load(f"{GOLDEN}/pack_q4_n16_k64.npz")
    assert np.array_equal(F.pack_bits(d["planes"]), d["packed"])
    assert np.array_equal(F.unpack_bits(d["packed"]), d["planes"])


@pytest.mark.parametrize("name", golden_cases())
def test_export_from_tensors_matches_reference_bytes(built_lib, name):
    d = load_golden(name)
    lin = F.export_from_tensors(d["quantized_w"], d["w_scale_f32"], d["w_zero_f32"], d["bias_f16"])
    assert np.array_equal(lin.w_quant, d["export_w_quant"])
    assert np.array_equal(lin.w_scale.view(np.uint16), d["export_w_scale"].view(np.uint16))
    assert np.array_equal(lin.w_zero.view(np.uint16), d["export_w_zero"].view(np.uint16))
    assert lin.groupsize == d["g"]


def test_pack_edge_cases(built_lib):
    assert F.pack_bits(np.zeros((2, 0, 16), np.uint8)).shape == (2, 0, 2)
    assert F.pack_bits(np.zeros((0, 4, 8), np.uint8)).shape == (0, 4, 1)
    with pytest.raises(ValueError):
        F.pack_bits(np.zeros((1, 2, 12), np.uint8))
    with pytest.raises(_lib.HlqError):
        F.pack_bits(np.full((1, 1, 8), 2, np.uint8))          # not a bit
    rng = np.random.default_rng(0)
    bits = rng.integers(0, 2, size=(3, 5, 40), dtype=np.uint8)
    assert np.array_equal(F.unpack_bits(F.pack_bits(bits)), bits)
    assert np.array_equal(F.pack_bits(bits), O.pack_bits(bits))


SHAPES = [(2, 64, 512, 128), (2, 40, 1024, 128), (3, 33, 640, 64), (4, 8, 96, 32), (1, 100, 128, 128),
          (2, 32, 1152, 128), (3, 72, 576, 32)]


@pytest.mark.parametrize("q,n,k,g", SHAPES)
def test_stream_repack_roundtrip(built_lib, q, n, k, g):
    d = O.synth_linear(n, k, q, g, seed=q * 1000 + n)
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], None, g)
    planes, meta = F.repack_host(lin)
    np_, kp = -(-n // 32) * 32, -(-k // 512) * 512
    assert planes.size == q * np_ * kp // 8
    assert meta.size == (q + 1) * np_ * kp // g
    back = F.unrepack_host(planes, meta, n, k, g, q)
    assert np.array_equal(back.w_quant, lin.w_quant)
    assert np.array_equal(back.w_scale.view(np.uint16), lin.w_scale.view(np.uint16))
    assert np.array_equal(back.w_zero.view(np.uint16), lin.w_zero.view(np.uint16))
    # a permutation plus zero padding: the multiset of bytes is preserved
    assert np.array_equal(np.bincount(planes, minlength=256)[1:], np.bincount(lin.w_quant.ravel(), minlength=256)[1:])


def emulate_stream_gemv(planes, meta, x, n, k, g, q):
    """NumPy walk of the streaming buffers with the index arithmetic of lut8_gemv_kernel:
    per slice a 64 KB table block (entry e of chunk c at byte 256*e + offset(c)), per lane
    and byte position i the lookup address (e << 8) | 4*(8*j + ((i >> 1) ^ r)) | 128*(i & 1)."""
    np_, kp = -(-n // 32) * 32, -(-k // 512) * 512
    slices, octs, gpw = kp // 512, np_ // 8, 128 // g
    gshift = {128: 3, 64: 2, 32: 1}[g]
    xp = np.zeros(kp, np.float64)
    xp[:k] = x.astype(np.float64)
    cells = planes.reshape(slices, octs, q, 32, 16)
    # scales/zeros are stored two octs (a duo) at a time: [slice][duo][pp][lane][oct & 1][u]
    mt = meta.view(np.float16).astype(np.float64).reshape(slices, octs // 2, q + 1, 32, 2, gpw)
    mt = mt.transpose(0, 1, 4, 2, 3, 5).reshape(slices, octs, q + 1, 32, gpw)
    y = np.zeros(np_, np.float64)
    e = np.arange(256)
    bitsel = ((e[:, None] >> np.arange(8)[None, :]) & 1).astype(np.float64)     # [256, 8]
    for s in range(slices):
        xs = xp[512 * s:512 * (s + 1)]
        table = np.zeros(65536 // 4, np.float64)                                # fp32 words
        banks_seen = {}
        for c in range(64):
            j, b = c >> 4, c & 15
            off = 4 * (8 * j + (b >> 1)) + 128 * (b & 1)
            table[(e * 256 + off) // 4] = bitsel @ xs[8 * c:8 * c + 8]
        xsum = xs.reshape(-1, g).sum(axis=1)
        for oct_ in range(octs):
            for lane in range(32):
                r, j = lane >> 2, lane & 3
                tot = 0.0
                sums = np.zeros((q, gpw))
                for i in range(16):
                    addr_low = 4 * (8 * j + ((i >> 1) ^ r)) + 128 * (i & 1)
                    banks_seen.setdefault(i, set()).add((lane, (addr_low // 4) % 32))
                    u = i // (16 // gpw)
                    for p in range(q):
                        byte = int(cells[s, oct_, p, lane, i])
                        sums[p, u] += table[((byte << 8) | addr_low) // 4]
                for u in range(gpw):
                    tot += mt[s, oct_, q, lane, u] * xsum[gpw * j + (u ^ (r >> gshift))]
                    for p in range(q):
                        tot += mt[s, oct_, p, lane, u] * sums[p, u]
                y[8 * oct_ + r] += tot
        for i, seen in banks_seen.items():
            assert len({bank for _, bank in seen}) == 32, "lanes of one lookup must hit 32 banks"
    return y[:n]


@pytest.mark.parametrize("q,n,k,g", [(2, 40, 1024, 128), (3, 16, 640, 64), (2, 8, 544, 32), (1, 33, 128, 128)])
def test_stream_layout_computes_the_product(built_lib, q, n, k, g):
    d = O.synth_linear(n, k, q, g, seed=7, signed_alpha=True)
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], None, g)
    planes, meta = F.repack_host(lin)
    y = emulate_stream_gemv(planes, meta, d["x"][0], n, k, g, q)
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g)[0]
    np.testing.assert_allclose(y, ref, rtol=1e-9, atol=1e-9)


def test_repack_argument_checks(built_lib):
    L = built_lib
    pb, mb = _lib.c_int64(), _lib.c_int64()
    assert L.hlq_stream_sizes(64, 512, 128, 2, pb, mb) == 0
    assert pb.value == 2 * 64 * 512 // 8 and mb.value == 3 * 64 * 4 * 2
    assert L.hlq_stream_sizes(64, 512, 256, 2, pb, mb) == 2     # g not a streaming size
    assert L.hlq_stream_sizes(64, 500, 128, 2, pb, mb) == 2     # k % g
    assert L.hlq_stream_sizes(64, 512, 128, 5, pb, mb) == 2     # bits
    assert L.hlq_stream_sizes(0, 512, 128, 2, pb, mb) == 1
    assert L.hlq_repack_host(None, None, None, 64, 512, 128, 2, None, None) == 1
    assert L.hlq_workspace_bytes(1, 4096, 4096, 2, 128) == 256 + 512 + 4096 * 4
    assert L.hlq_workspace_bytes(0, 4096, 4096, 2, 128) == 0


def test_export_dir_roundtrip_and_loader_errors(built_lib, tmp_path):
    d = O.synth_linear(64, 256, 2, 128, seed=2, bias=True)
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], d["bias"], 128)
    p = str(tmp_path / "0" / "self_attn.q_proj")
    F.write_export_dir(p, lin)
    # byte-identical to what the oracle's restatement of the exporter writes
    p2 = str(tmp_path / "ref")
    O.write_export_dir(p2, d["w_quant"], d["w_scale"], d["w_zero"], d["bias"])
    for f in ("w_quant.bin", "w_scale.bin", "w_zero.bin", "bias.bin", "weight_config.json"):
        assert open(os.path.join(p, f), "rb").read() == open(os.path.join(p2, f), "rb").read()
    back = F.read_export_dir(p)                       # group size derived from w_zero.bin
    assert back.groupsize == 128 and back.bits == 2
    assert np.array_equal(back.w_quant, lin.w_quant) and np.array_equal(back.bias, lin.bias)
    F.write_export_dir(p, lin, write_groupsize=True)  # the key the C++ loader reads
    assert F.read_export_dir(p).groupsize == 128
    with pytest.raises(RuntimeError):
        F.read_export_dir(str(tmp_path / "missing"))
    open(os.path.join(p, "weight_config.json"), "w").write("{not json")
    with pytest.raises(RuntimeError):
        F.read_export_dir(p)
    F.write_export_dir(p, lin)
    with open(os.path.join(p, "w_quant.bin"), "ab") as f:
        f.truncate(100)
    with pytest.raises(ValueError):
        F.read_export_dir(p)
