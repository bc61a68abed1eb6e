"""Generate the golden fixtures in this directory by running the reference.

Run once, where a checkout of the ELUTQ reference is available:

    python tests/golden/make_golden.py /path/to/ELUTQ

It imports the reference's own Python modules (``GPTQ/quant.py`` and
``GPTQ/HLQ.py``) and records, for small seeded cases,

* the bytes ``HLQ.export`` writes (``w_quant.bin``, ``w_scale.bin``,
  ``w_zero.bin``) for given ``quantized_w / w_scale / w_zero`` tensors
  (GPTQ/HLQ.py:207-251),
* ``dequantize_with_scales`` and ``quantize_with_scales`` outputs
  (GPTQ/quant.py:154-183),
* the dense product ``x @ W_hat.T`` with ``W_hat`` produced by the reference's
  dequantizer from the fp16-rounded parameters, in float64,
* one case whose parameters come from the reference's alternating fit
  (``pseudo_quantize_tensor(..., use_alternating_optimization=True)``,
  GPTQ/quant.py:185-213), so that unordered and negative scales are covered.

The fixtures are committed; the tests never need the reference checkout.
"""
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, q, N, K, g, M, bias, mode)
CASES = [
    ("w2g128_n64_k256", 2, 64, 256, 128, 1, False, "random"),
    ("w3g64_n32_k256", 3, 32, 256, 64, 4, False, "random"),
    ("w4g32_n32_k128", 4, 32, 128, 32, 2, True, "random"),
    ("w1g128_n32_k128", 1, 32, 128, 128, 1, False, "random"),
    ("w2g128_n96_k512_signed", 2, 96, 512, 128, 3, True, "signed"),
    ("w2g128_n40_k1024", 2, 40, 1024, 128, 1, False, "random"),
    ("w3g128_n32_k256_fit", 3, 32, 256, 128, 2, False, "fit"),
    ("w2g64_n32_k128_fit", 2, 32, 128, 64, 1, False, "fit"),
]


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "GPTQ"))
    import quant  # noqa: E402  (reference module)
    import HLQ    # noqa: E402  (reference module)

    exporter = HLQ.HLQ(torch.nn.Linear(8, 8, bias=False))

    for idx, (name, q, n, k, g, m, has_bias, mode) in enumerate(CASES):
        gen = torch.Generator().manual_seed(1000 + idx)
        ng = k // g
        if mode == "fit":
            w = torch.randn(n, k, generator=gen) * 0.02
            _, quantized, scales, zeros = quant.pseudo_quantize_tensor(
                w, n_bit=q, zero_point=True, q_group_size=g, get_scale_zp=True,
                use_alternating_optimization=True)
            quantized_w = quantized.to(torch.uint8)            # [N, K, q]
            w_scale = scales.float()                           # [N, G, q]
            w_zero = zeros.float()                             # [N, G, 1]
        else:
            quantized_w = (torch.rand(n, k, q, generator=gen) < 0.5).to(torch.uint8)
            w_scale = torch.randn(n, ng, q, generator=gen) * 0.02
            if mode != "signed":
                w_scale = w_scale.abs()
            w_zero = torch.randn(n, ng, 1, generator=gen) * 0.01
        x = torch.randn(m, k, generator=gen).half()
        bias = (torch.randn(n, generator=gen) * 0.1).half() if has_bias else None

        with tempfile.TemporaryDirectory() as tmp:
            exporter.export(quantized_w, w_scale, w_zero, groupsize=g, output_dir=tmp, bit=q)
            raw_quant = np.fromfile(os.path.join(tmp, "w_quant.bin"), dtype=np.uint8)
            raw_scale = np.fromfile(os.path.join(tmp, "w_scale.bin"), dtype=np.uint8)
            raw_zero = np.fromfile(os.path.join(tmp, "w_zero.bin"), dtype=np.uint8)

        # the runtime sees the fp16-rounded parameters
        s16 = w_scale.half().float().reshape(n * ng, q)
        z16 = w_zero.half().float().reshape(n * ng)
        blocks = quantized_w.reshape(n * ng, g, q)
        w_hat32 = quant.dequantize_with_scales(blocks, s16, z16).reshape(n, k)
        w_hat64 = quant.dequantize_with_scales(
            blocks.double(), s16.double(), z16.double()).reshape(n, k)
        # dequantize_with_scales casts with .float(); redo the sum in float64
        w_hat64 = (blocks.double() * s16.double().unsqueeze(1)).sum(2) + z16.double().unsqueeze(1)
        w_hat64 = w_hat64.reshape(n, k)
        y64 = x.double() @ w_hat64.t()
        if bias is not None:
            y64 = y64 + bias.double()[None, :]

        # the reference quantizer on a fresh tensor with these scales
        t = torch.randn(n * ng, g, generator=gen) * 0.03
        requant = quant.quantize_with_scales(t, s16, z16, bits=q)

        out = {
            "q": q, "n": n, "k": k, "g": g, "m": m,
            "quantized_w": np.packbits(quantized_w.numpy(), axis=None),
            "w_scale_f32": w_scale.numpy(),
            "w_zero_f32": w_zero.numpy(),
            "x_f16": x.numpy(),
            "export_w_quant": raw_quant,
            "export_w_scale": raw_scale,
            "export_w_zero": raw_zero,
            "w_hat_f32": w_hat32.numpy(),
            "y_f64": y64.numpy(),
            "requant_in": t.numpy(),
            "requant_out": np.packbits(requant.numpy(), axis=None),
        }
        if bias is not None:
            out["bias_f16"] = bias.numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, "ok", y64.shape)

    # Pack_T_MAC_Weight alone, including the 4-plane case of the lm_head export
    gen = torch.Generator().manual_seed(77)
    planes = (torch.rand(4, 16, 64, generator=gen) < 0.5).to(torch.uint8)
    packed = exporter.Pack_T_MAC_Weight(planes, 4)
    np.savez_compressed(os.path.join(HERE, "pack_q4_n16_k64.npz"),
                        planes=planes.numpy(), packed=packed.numpy())
    print("pack ok")


if __name__ == "__main__":
    main(sys.argv[1])
