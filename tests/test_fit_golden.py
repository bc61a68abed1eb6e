"""The alternating fit of plane scales and offsets (GPTQ/quant.py:104-153): the NumPy oracle
against the reference's own results (tests/golden/fit_cases.npz, made by make_golden_fit.py from
the reference's pseudo_quantize_tensor), and - on a GPU - the device kernel against both.

The fit alternates a discrete assignment with a least-squares solve, so two float
implementations can part ways at a weight that sits exactly between two values; such a weight
costs the same error either way, which is why the mean squared error is the quantity compared
(1e-5 relative on a whole case: the parted weights move it by a few 1e-6), with the scales compared where the assignments agree."""
import os

import numpy as np
import pytest

from oracle import hlq_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fit_cases.npz")
CASES = [(2, 64), (2, 128), (3, 64), (3, 128), (4, 128)]


def case(d, q, g):
    key = f"w{q}g{g}"
    w = d[key + "_w"]
    n, k = w.shape
    bits = np.unpackbits(d[key + "_bits"])[: n * k * q].reshape(n * (k // g), g, q)
    return (w.reshape(-1, g), d[key + "_scales"].reshape(-1, q), d[key + "_zeros"].reshape(-1), bits,
            float(d[key + "_mse"]), d[key + "_block_mse"])


def recon_mse(w, scales, zeros):
    """Reconstruction error with the reference's own assignment rule (quant.py:154-183)."""
    bits = O.quantize_with_scales(w, scales, zeros, scales.shape[1])
    rec = O.dequantize_with_scales(bits, scales, zeros)
    return ((w.astype(np.float64) - rec.astype(np.float64)) ** 2).mean(axis=1), bits


@pytest.mark.parametrize("q,g", CASES)
def test_oracle_fit_matches_the_reference(q, g):
    w, s_ref, z_ref, bits_ref, mse_ref, blk_ref = case(np.load(GOLDEN), q, g)
    s, z = O.fit_alternating(w, q)
    blk, bits = recon_mse(w, s, z)
    assert abs(blk.mean() - mse_ref) <= 1e-5 * mse_ref
    same = (bits == bits_ref).all(axis=(1, 2))
    assert same.mean() >= 0.9                              # blocks whose assignments agree entirely
    assert np.allclose(s[same], s_ref[same], rtol=2e-4, atol=1e-7)
    assert np.allclose(z[same], z_ref[same], rtol=2e-4, atol=1e-7)
    # the degenerate blocks: a constant block (singular system) reconstructs exactly
    const_block = 5 * (w.shape[0] // 24)
    assert blk[const_block] <= 1e-12 and blk_ref[const_block] <= 1e-12


@pytest.mark.gpu
@pytest.mark.parametrize("q,g", CASES)
def test_device_fit_matches_the_reference(q, g):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    from elutq_b200 import format as F
    w, s_ref, z_ref, bits_ref, mse_ref, blk_ref = case(np.load(GOLDEN), q, g)
    s, z = F.fit_alternating_device(torch.from_numpy(w).cuda(), q)
    s, z = s.cpu().numpy(), z.cpu().numpy()
    blk, bits = recon_mse(w, s, z)
    assert abs(blk.mean() - mse_ref) <= 1e-5 * mse_ref
    same = (bits == bits_ref).all(axis=(1, 2))
    assert same.mean() >= 0.9
    assert np.allclose(s[same], s_ref[same], rtol=2e-4, atol=1e-7)
    assert np.allclose(z[same], z_ref[same], rtol=2e-4, atol=1e-7)
    # the whole device pipeline: fit -> assignment -> exported arrays that the loader takes
    n, k = 24, 4 * g
    rec, quantized, w_scale, w_zero = F.pseudo_quantize_device(torch.from_numpy(w.reshape(n, k)).cuda(), q, g)
    mse_dev = float(((torch.from_numpy(w.reshape(n, k)).cuda().double() - rec.double()) ** 2).mean())
    assert abs(mse_dev - mse_ref) <= 1e-5 * mse_ref
    lin = F.export_from_tensors(quantized.cpu().numpy(), w_scale.cpu().numpy(), w_zero.cpu().numpy(), None, g)
    assert lin.bits == q and lin.out_channel == n and lin.in_channel == k and lin.groupsize == g
    from elutq_b200.linear import HLQLinear
    mod = HLQLinear.from_exported(lin, device=0)
    x = torch.randn(1, k, device="cuda").half()
    y = mod(x).float().cpu().numpy().astype(np.float64)
    want = x.float().cpu().numpy().astype(np.float64) @ O.dequantize_export(lin.w_quant, lin.w_scale, lin.w_zero, g,
                                                                            np.float64).T
    assert O.normwise_error(y, want) <= 1e-3
