"""The quantizer's assignment step on the device (hlq_quantize_with_scales_device) against the
reference's own outputs (golden fixtures made with GPTQ/quant.py) and the oracle."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from conftest import golden_cases, load_golden  # noqa: E402
from elutq_b200 import _lib, format as F  # noqa: E402
from oracle import hlq_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", golden_cases())
def test_device_quantizer_matches_the_reference_fixture(name):
    d = load_golden(name)
    n, k, g, q = d["n"], d["k"], d["g"], d["q"]
    s16 = d["w_scale_f32"].astype(np.float16).astype(np.float32).reshape(n * (k // g), q)
    z16 = d["w_zero_f32"].astype(np.float16).astype(np.float32).reshape(n * (k // g))
    got = F.quantize_with_scales_device(torch.from_numpy(d["requant_in"]).cuda(), torch.from_numpy(s16).cuda(),
                                        torch.from_numpy(z16).cuda()).cpu().numpy()
    # the restatement: same fp32 arithmetic up to the order in which a combination's scales are
    # added, so the same choice everywhere but at exact near-ties
    assert (got == O.quantize_with_scales(d["requant_in"], s16, z16, q)).all(axis=2).mean() > 0.9999
    # the reference itself (torch.matmul may sum the scales in another order: ties can differ)
    same = (got == d["requant_out"]).all(axis=2)
    assert same.mean() > 0.999
    np.testing.assert_allclose(O.dequantize_with_scales(got, s16, z16),
                               O.dequantize_with_scales(d["requant_out"], s16, z16), atol=1e-6)


@pytest.mark.parametrize("q,g,blocks", [(1, 128, 7), (2, 64, 1000), (3, 128, 333), (4, 32, 4096)])
def test_device_quantizer_equals_oracle_and_feeds_the_export(q, g, blocks):
    rng = np.random.default_rng(q * 100 + g)
    w = (0.03 * rng.standard_normal((blocks, g))).astype(np.float32)
    s = (0.02 * rng.standard_normal((blocks, q))).astype(np.float32)        # alternating mode: signs are free
    z = (0.01 * rng.standard_normal(blocks)).astype(np.float32)
    got = F.quantize_with_scales_device(torch.from_numpy(w).cuda(), torch.from_numpy(s).cuda(),
                                        torch.from_numpy(z).cuda())
    ref = O.quantize_with_scales(w, s, z, q)
    got = got.cpu().numpy()
    assert (got == ref).all(axis=2).mean() > 0.9999
    # nearest: no other combination is closer than the chosen one
    back = O.dequantize_with_scales(got, s, z)
    combos = O.bit_combinations(q)
    allv = (s @ combos.T)[:, None, :] + z[:, None, None]
    assert (np.abs(back - w)[..., None] <= np.abs(allv - w[..., None]) + 1e-6).all()


def test_device_quantizer_argument_errors():
    w = torch.zeros((2, 8), device="cuda")
    with pytest.raises(ValueError):
        F.quantize_with_scales_device(w, torch.zeros((3, 2), device="cuda"), torch.zeros(2, device="cuda"))
    with pytest.raises(_lib.HlqError):
        F.quantize_with_scales_device(w, torch.zeros((2, 5), device="cuda"), torch.zeros(2, device="cuda"))
    with pytest.raises(RuntimeError):
        F.quantize_with_scales_device(torch.zeros((2, 8)), torch.zeros((2, 2)), torch.zeros(2))
