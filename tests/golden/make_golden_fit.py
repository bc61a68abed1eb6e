"""Generates tests/golden/fit_cases.npz: inputs and results of the REFERENCE's alternating fit.

    python tests/golden/make_golden_fit.py <path of the ELUTQ checkout>       (CPU only)

Runs the reference's own pseudo_quantize_tensor(..., use_alternating_optimization=True)
(GPTQ/quant.py:185-213 -> find_optimal_params_alternating :118-153 -> quantize_with_scales
:154-174) on seeded weight matrices for q in {2, 3} x g in {64, 128} (plus one q = 4 case) and
stores, per case: the input weights, the fitted scales and offsets, the assigned bits, the
reconstruction and its mean squared error.  Each matrix has ordinary rows ~ N(0, 0.02), a few
heavy-tailed rows and two degenerate blocks (a constant block, whose normal equations are
singular, and a two-valued block)."""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = [(2, 64), (2, 128), (3, 64), (3, 128), (4, 128)]


def main(reference_root):
    sys.path.insert(0, os.path.join(reference_root, "GPTQ"))
    import quant
    out = {}
    for ci, (q, g) in enumerate(CASES):
        gen = torch.Generator().manual_seed(500 + ci)
        n, k = 24, 4 * g
        w = torch.randn(n, k, generator=gen) * 0.02
        w[3] = w[3] * (1 + 8 * (torch.rand(k, generator=gen) < 0.05).float())        # outliers
        w[5, :g] = 0.0123                                                          # constant block
        w[6, g:2 * g] = torch.where(torch.rand(g, generator=gen) < 0.5, torch.tensor(-0.01), torch.tensor(0.02))
        recon, quantized, scales, zeros = quant.pseudo_quantize_tensor(
            w.clone(), n_bit=q, zero_point=True, q_group_size=g, get_scale_zp=True, use_alternating_optimization=True)
        key = f"w{q}g{g}"
        out[key + "_w"] = w.numpy().astype(np.float32)
        out[key + "_scales"] = scales.numpy().astype(np.float32)          # [N, G, q]
        out[key + "_zeros"] = zeros.numpy().astype(np.float32)            # [N, G, 1]
        out[key + "_bits"] = np.packbits(quantized.numpy().astype(np.uint8), axis=None)
        out[key + "_mse"] = np.float64(torch.mean((w.double() - recon.double()) ** 2).item())
        blk = ((w.double() - recon.double()) ** 2).reshape(n * 4, g).mean(dim=1)
        out[key + "_block_mse"] = blk.numpy()
        print(key, "mse", out[key + "_mse"])
    np.savez_compressed(os.path.join(HERE, "fit_cases.npz"), **out)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
