"""The oracle against fixtures produced by the reference's own Python code
(tests/golden/make_golden.py), and the two restatements of the reference's fp16 kernel
against each other.  CPU only."""
import numpy as np
import pytest

from conftest import GOLDEN, golden_cases, load_golden
from oracle import hlq_oracle as O


@pytest.mark.parametrize("name", golden_cases())
def test_export_bytes_match_reference(name):
    d = load_golden(name)
    wq, ws, wz = O.export_arrays(d["quantized_w"], d["w_scale_f32"], d["w_zero_f32"])
    assert np.array_equal(wq, d["export_w_quant"])
    assert np.array_equal(ws.view(np.uint16), d["export_w_scale"].view(np.uint16))
    assert np.array_equal(wz.view(np.uint16), d["export_w_zero"].view(np.uint16))


def test_pack_matches_reference_packer():
    d = np.load(f"{GOLDEN}/pack_q4_n16_k64.npz")
    assert np.array_equal(O.pack_bits(d["planes"]), d["packed"])
    assert np.array_equal(O.unpack_bits(d["packed"]), d["planes"])


@pytest.mark.parametrize("name", golden_cases())
def test_dequant_and_product_match_reference(name):
    d = load_golden(name)
    g = d["g"]
    w32 = O.dequantize_export(d["export_w_quant"], d["export_w_scale"], d["export_w_zero"], g, np.float32)
    # the reference sums the planes in fp32 in plane order; allow one ulp of reassociation
    np.testing.assert_allclose(w32, d["w_hat_f32"], rtol=0, atol=2e-7)
    y = O.hlq_linear(d["x_f16"], d["export_w_quant"], d["export_w_scale"], d["export_w_zero"], g,
                     d["bias_f16"])
    np.testing.assert_allclose(y, d["y_f64"], rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("name", golden_cases())
def test_quantizer_matches_reference(name):
    d = load_golden(name)
    n, k, g, q = d["n"], d["k"], d["g"], d["q"]
    s16 = d["w_scale_f32"].astype(np.float16).astype(np.float32).reshape(n * (k // g), q)
    z16 = d["w_zero_f32"].astype(np.float16).astype(np.float32).reshape(n * (k // g))
    got = O.quantize_with_scales(d["requant_in"], s16, z16, q)
    same = (got == d["requant_out"]).all(axis=2)
    # ties between combinations can fall either way under different summation orders
    assert same.mean() > 0.999
    back = O.dequantize_with_scales(got, s16, z16)
    ref = O.dequantize_with_scales(d["requant_out"], s16, z16)
    np.testing.assert_allclose(back, ref, atol=1e-6)


def test_weight_config_keys():
    cfg = O.weight_config(64, 256, 2, False)
    assert cfg == {"weight_data_len": 64 * 256 * 2 // 8, "base_bit": 2, "use_sparse": False,
                   "in_channel": 256, "out_channel": 64, "has_bias": False}


@pytest.mark.parametrize("shape", [(2, 64, 256, 128, 1), (3, 64, 256, 64, 2), (4, 64, 128, 32, 1),
                                   (1, 128, 128, 128, 1)])
@pytest.mark.parametrize("threads", [1, 2])
def test_c_restatement_equals_numpy_chain(cpu_oracle_lib, shape, threads):
    q, n, k, g, m = shape
    d = O.synth_linear(n, k, q, g, m=m, seed=11, bias=True, signed_alpha=True)
    lin = cpu_oracle_lib.CpuLinear(d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"], threads=threads)
    y = lin.forward(d["x"])
    for row in range(m):
        ref = O.fp16_chain_gemv(d["x"][row], d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"])
        assert np.array_equal(y[row].view(np.uint16), ref.view(np.uint16))


def test_c_restatement_relayout_matches_numpy(cpu_oracle_lib):
    d = O.synth_linear(128, 256, 2, 128, seed=5)
    for threads in (1, 2, 4):
        lin = cpu_oracle_lib.CpuLinear(d["w_quant"], d["w_scale"], d["w_zero"], 128, threads=threads)
        bq, bs, bz = O.runtime_relayout(d["w_quant"], d["w_scale"], d["w_zero"], threads)
        assert np.array_equal(lin.quant, bq)
        assert np.array_equal(lin.scale.view(np.uint16), bs.view(np.uint16))
        assert np.array_equal(lin.zero.view(np.uint16), bz.view(np.uint16))


def test_c_restatement_rejects_ragged_chunks(cpu_oracle_lib):
    d = O.synth_linear(96, 128, 2, 128, seed=1)
    with pytest.raises(ValueError):
        cpu_oracle_lib.CpuLinear(d["w_quant"], d["w_scale"], d["w_zero"], 128, threads=2)  # 48 rows/chunk


def test_fp16_kernel_stays_in_its_error_envelope(cpu_oracle_lib):
    """The reference's all-fp16 kernel lands within a few 1e-3 (normwise) of the exact
    product; the 1e-3 gate of the CUDA path is taken against the exact product instead."""
    d = O.synth_linear(512, 1024, 2, 128, m=1, seed=0)
    lin = cpu_oracle_lib.CpuLinear(d["w_quant"], d["w_scale"], d["w_zero"], 128, threads=2)
    y64 = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], 128)
    err = O.normwise_error(lin.forward(d["x"]), y64)
    assert err < 8e-3
