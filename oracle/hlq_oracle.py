"""CPU oracle for the HLQ (Hierarchical Linear Quantization) linear operator.

TEST INFRASTRUCTURE ONLY.  This module is the checker that the CUDA path is
compared against; nothing in the shipped package may import it.  Only tests,
the smoke check and the CPU-baseline leg of the benchmark use it.

It restates, in NumPy, the reference's definitions for the quantized-linear
path.  Every function names the reference lines it follows (paths are relative
to the ELUTQ project root).

Parity pin: the functions here are checked against fixtures that were produced
by importing the reference's own Python modules (``GPTQ/quant.py``,
``GPTQ/HLQ.py``); see ``tests/golden/make_golden.py``.  The reference ships no
tests or known-answer vectors of its own, so those generated fixtures are the
pin.

Notation: N = out_channel, K = in_channel, q = number of bit-planes,
g = group size, G = K // g.
"""
from __future__ import annotations

import itertools
import json
import os

import numpy as np

# --------------------------------------------------------------------------
# Bit-plane packing (GPTQ/HLQ.py:239-251, Pack_T_MAC_Weight)
# --------------------------------------------------------------------------


def pack_bits(bits: np.ndarray) -> np.ndarray:
    """``uint8 [q, N, K]`` of {0,1} -> ``uint8 [q, N, K/8]``.

    Byte ``i`` of a row holds input channels ``8i .. 8i+7``; channel ``8i+j``
    sits at bit ``j`` (LSB = lowest channel), as in GPTQ/HLQ.py:246-249.
    """
    bits = np.asarray(bits, dtype=np.uint8)
    if bits.ndim != 3:
        raise ValueError("bits must be [q, N, K]")
    if bits.shape[2] % 8:
        raise ValueError("K must be a multiple of 8")
    if bits.size and bits.max() > 1:
        raise ValueError("bit-plane entries must be 0 or 1")
    q, n, k = bits.shape
    weights = (1 << np.arange(8, dtype=np.uint16)).astype(np.uint16)
    grouped = bits.reshape(q, n, k // 8, 8).astype(np.uint16)
    return (grouped * weights).sum(axis=3).astype(np.uint8)


def unpack_bits(packed: np.ndarray) -> np.ndarray:
    """Inverse of :func:`pack_bits`: ``uint8 [q, N, K/8]`` -> ``uint8 [q, N, K]``."""
    packed = np.asarray(packed, dtype=np.uint8)
    q, n, kb = packed.shape
    shifts = np.arange(8, dtype=np.uint8)
    out = (packed[..., None] >> shifts) & 1
    return out.reshape(q, n, kb * 8).astype(np.uint8)


# --------------------------------------------------------------------------
# Export format (GPTQ/HLQ.py:177-236)
# --------------------------------------------------------------------------


def export_arrays(quantized_w: np.ndarray, w_scale: np.ndarray, w_zero: np.ndarray):
    """Tensors as handed to ``HLQ.export`` -> the three exported byte arrays.

    quantized_w ``[N, K, q]`` {0,1}; w_scale ``[N, G, q]``; w_zero ``[N, G, 1]``.
    Returns ``(w_quant uint8 [q,N,K/8], w_scale fp16 [q,N,G], w_zero fp16 [N,G])``:
    zeros are cast to fp16 unchanged in order (HLQ.py:218-221), scales are cast
    then permuted plane-major (HLQ.py:223-228), planes are permuted plane-major
    and packed (HLQ.py:230-236).
    """
    qw = np.asarray(quantized_w)
    if qw.ndim != 3 or np.asarray(w_scale).ndim != 3 or np.asarray(w_zero).ndim != 3:
        raise ValueError("quantized_w, w_scale and w_zero must all be 3-D")
    zero16 = np.asarray(w_zero, dtype=np.float32).astype(np.float16)[:, :, 0]
    scale16 = np.ascontiguousarray(
        np.asarray(w_scale, dtype=np.float32).astype(np.float16).transpose(2, 0, 1))
    planes = np.ascontiguousarray(qw.astype(np.uint8).transpose(2, 0, 1))
    return pack_bits(planes), scale16, np.ascontiguousarray(zero16)


def weight_config(n: int, k: int, q: int, has_bias: bool) -> dict:
    """The ``weight_config.json`` dictionary of GPTQ/HLQ.py:177-193.

    The exporter does not record the group size; readers derive it from the
    size of ``w_zero.bin``.
    """
    return {
        "weight_data_len": int(k * n * q / 8),
        "base_bit": int(q),
        "use_sparse": False,
        "in_channel": int(k),
        "out_channel": int(n),
        "has_bias": bool(has_bias),
    }


def write_export_dir(path, w_quant, w_scale16, w_zero16, bias16=None):
    """Write one linear's directory in the layout HLQ.fasterquant produces."""
    os.makedirs(path, exist_ok=True)
    q, n, kb = w_quant.shape
    np.asarray(w_zero16, dtype=np.float16).tofile(os.path.join(path, "w_zero.bin"))
    np.asarray(w_scale16, dtype=np.float16).tofile(os.path.join(path, "w_scale.bin"))
    np.asarray(w_quant, dtype=np.uint8).tofile(os.path.join(path, "w_quant.bin"))
    if bias16 is not None:
        np.asarray(bias16, dtype=np.float16).tofile(os.path.join(path, "bias.bin"))
    with open(os.path.join(path, "weight_config.json"), "w") as f:
        json.dump(weight_config(n, kb * 8, q, bias16 is not None), f, indent=4)


# --------------------------------------------------------------------------
# HLQ definition (GPTQ/quant.py:154-183)
# --------------------------------------------------------------------------


def bit_combinations(q: int) -> np.ndarray:
    """All 2^q rows of {0,1}^q in the order of quant.py:12-16 (first column is
    the slowest-varying one)."""
    return np.array(list(itertools.product([0, 1], repeat=int(q))), dtype=np.float32)


def quantize_with_scales(tensor, scales, zero_points, q: int) -> np.ndarray:
    """Nearest-combination quantizer (quant.py:154-174), fp32 like the reference.

    tensor ``[B, g]``, scales ``[B, q]``, zero_points ``[B]`` -> ``uint8 [B, g, q]``.
    Ties resolve to the lowest combination index (argmin).
    """
    t = np.asarray(tensor, dtype=np.float32)
    s = np.asarray(scales, dtype=np.float32)
    z = np.asarray(zero_points, dtype=np.float32)
    combos = bit_combinations(q)
    adjusted = t - z[:, None]
    values = s @ combos.T                                   # [B, 2^q]
    dist = np.abs(values[:, None, :] - adjusted[:, :, None])
    idx = dist.argmin(axis=2)
    return combos[idx].astype(np.uint8)


def dequantize_with_scales(quantized, scales, zero_points, dtype=np.float32) -> np.ndarray:
    """``sum_j b_j * alpha_j + z`` per element (quant.py:176-183).

    quantized ``[B, g, q]``, scales ``[B, q]``, zero_points ``[B]`` -> ``[B, g]``.
    """
    qv = np.asarray(quantized).astype(dtype)
    s = np.asarray(scales).astype(dtype)
    z = np.asarray(zero_points).astype(dtype)
    return (qv * s[:, None, :]).sum(axis=2) + z[:, None]


def dequantize_export(w_quant, w_scale16, w_zero16, g: int, dtype=np.float64) -> np.ndarray:
    """Exported arrays -> dense ``W_hat [N, K]`` in ``dtype``.

    Same arithmetic as :func:`dequantize_with_scales`, driven from the exported
    fp16 scales/zeros (HLQ.py:218,223), i.e. the values a runtime actually sees.
    """
    bits = unpack_bits(w_quant).astype(dtype)               # [q, N, K]
    q, n, k = bits.shape
    alpha = np.asarray(w_scale16).astype(dtype)             # [q, N, G]
    z = np.asarray(w_zero16).astype(dtype)                  # [N, G]
    alpha_full = np.repeat(alpha, g, axis=2)                # [q, N, K]
    return (bits * alpha_full).sum(axis=0) + np.repeat(z, g, axis=1)


def fit_alternating(t, bits: int, iters: int = 10):
    """The reference's alternating fit of plane scales and offset per block, restated in NumPy
    float32 (GPTQ/quant.py:118-153 with :95-102 and :104-116): start from range / (2^q - 1) * 2^j
    and the minimum; `iters` times assign every weight to the nearest of the 2^q values (first
    minimum; value i has bit j = (i >> j) & 1, then the constant) and solve the (q+1) x (q+1)
    normal equations with a pseudo-inverse.  Returns (scales [blocks, q], zeros [blocks])."""
    t = np.asarray(t, dtype=np.float32)
    nb, g = t.shape
    lo, hi = t.min(axis=1), t.max(axis=1)
    step = (hi - lo) / np.float32(2 ** bits - 1)
    scales = np.concatenate([step[:, None] * (2.0 ** np.arange(bits, dtype=np.float32))[None, :], lo[:, None]],
                            axis=1).astype(np.float32)
    combos = np.array([[(i >> j) & 1 for j in range(bits)] + [1] for i in range(2 ** bits)], dtype=np.float32)
    rtol = (bits + 1) * np.finfo(np.float32).eps          # torch.linalg.pinv's default for float32
    for _ in range(iters):
        comb_vals = scales @ combos.T                                              # [nb, 2^q]
        idx = np.argmin(np.abs(t[:, :, None] - comb_vals[:, None, :]), axis=2)     # [nb, g]
        B = combos[idx]                                                            # [nb, g, q+1]
        BtB = np.einsum("bgi,bgj->bij", B, B)
        BtY = np.einsum("bgi,bg->bi", B, t)
        inv = np.stack([np.linalg.pinv(m, rcond=rtol) for m in BtB]).astype(np.float32)
        scales = np.einsum("bij,bj->bi", inv, BtY).astype(np.float32)
    return scales[:, :bits], scales[:, bits]


def add_sparse_plane(w, mask, blocks, scales16, g: int):
    """The runtime's optional extra bit-plane added to a dequantized weight ``w`` [N, K]:
    for every listed block (x = first row, y = first channel of a group)
    ``w[x + r, y + c] += scale[r] * bit[r][c]``, which is what the reference's kernel adds to
    its output through its tables (C++/ops/src/arm/arm_t_mac_kernal.cpp:678-788; block and
    scale order as re-laid-out at :577-588 and read at :761-764; loader
    C++/ops/src/arm/parameters.cpp:44-64).  Bits are LSB-first along the channels, as in
    the dense planes."""
    mask = np.asarray(mask).reshape(-1, 2)
    for p in range(mask.shape[0]):
        x0, y0 = int(mask[p, 0]), int(mask[p, 1])
        bits = np.unpackbits(np.asarray(blocks[p], dtype=np.uint8), axis=1, bitorder="little")[:, :g]
        w[x0:x0 + 32, y0:y0 + g] += np.asarray(scales16[p]).astype(w.dtype)[:, None] * bits.astype(w.dtype)
    return w


def hlq_linear(x, w_quant, w_scale16, w_zero16, g: int, bias16=None, dtype=np.float64, sparse=None):
    """Value oracle: ``y = x . W_hat^T (+ bias)`` in ``dtype`` (default fp64).

    This is the reference's HLQ matmul in the form its evaluation uses: the
    dequantized weight written into an ``nn.Linear`` (HLQ.py:173).  ``sparse``: optional
    (mask, blocks, scales) of the runtime's extra bit-plane (see add_sparse_plane).
    """
    w = dequantize_export(w_quant, w_scale16, w_zero16, g, dtype)
    if sparse is not None:
        add_sparse_plane(w, sparse[0], sparse[1], sparse[2], g)
    y = np.asarray(x).astype(dtype) @ w.T
    if bias16 is not None:
        y = y + np.asarray(bias16).astype(dtype)[None, :]
    return y


def normwise_error(y, y_ref) -> float:
    """``max|y - y_ref| / max|y_ref|``: the error measure of the 1e-3 gate."""
    y = np.asarray(y, dtype=np.float64)
    y_ref = np.asarray(y_ref, dtype=np.float64)
    denom = np.abs(y_ref).max()
    if denom == 0:
        return float(np.abs(y).max())
    return float(np.abs(y - y_ref).max() / denom)


# --------------------------------------------------------------------------
# Reference runtime re-layout (C++/ops/src/arm/arm_t_mac_kernal.cpp:472-552)
# --------------------------------------------------------------------------


def runtime_relayout(w_quant, w_scale16, w_zero16, n_thread: int):
    """Export arrays -> the flat buffers the reference's kernel walks.

    bits   ``[thread][plane][rowblock of 32][byte j][row r<32]``  (:478-491)
    scales ``[thread][plane][rowblock of 32][group][row r<32]``   (:504-521)
    zeros  ``[rowblock of 32][group][row r<32]``                  (:530-541)
    with ``ceil(N / n_thread)`` rows per thread chunk (:477).
    """
    q, n, kb = w_quant.shape
    ng = w_zero16.shape[1]
    chunk = -(-n // n_thread)
    if chunk % 32 or n % 32:
        raise ValueError("rows per thread chunk must be a multiple of 32")
    bits_out, scale_out = [], []
    for t in range(n_thread):
        lo, hi = t * chunk, min((t + 1) * chunk, n)
        for p in range(q):
            blk = w_quant[p, lo:hi].reshape(-1, 32, kb)      # [rb, r, j]
            bits_out.append(blk.transpose(0, 2, 1).reshape(-1))
            sblk = w_scale16[p, lo:hi].reshape(-1, 32, ng)
            scale_out.append(sblk.transpose(0, 2, 1).reshape(-1))
    zeros = w_zero16.reshape(-1, 32, ng).transpose(0, 2, 1).reshape(-1)
    return (np.concatenate(bits_out) if bits_out else np.zeros(0, np.uint8),
            np.concatenate(scale_out) if scale_out else np.zeros(0, np.float16),
            np.ascontiguousarray(zeros))


# --------------------------------------------------------------------------
# Reference kernel in its own fp16 operation order (small cases only)
# --------------------------------------------------------------------------


def fp16_chain_gemv(x16, w_quant, w_scale16, w_zero16, g: int, bias16=None) -> np.ndarray:
    """One GEMV with every intermediate rounded to fp16 in the reference's order.

    Follows C++/ops/src/arm/arm_gemm.cpp:248-308 (group sums, zero term, planes,
    bias), the LUT build of arm_t_mac_kernal.cpp:95-138 and the per-plane update
    of arm_t_mac_kernal.cpp:364-469 (per 8 input channels: low-nibble entry then
    high-nibble entry; per group: multiply by alpha, then add across groups; per
    plane: one read-modify-write of the output).  Multiplies and adds are rounded
    separately (no fused multiply-add).  Pure Python loops over groups: use on
    small shapes; the C restatement in this directory covers the large ones.
    """
    f16 = np.float16
    x16 = np.asarray(x16, dtype=f16).reshape(-1)
    q, n, kb = w_quant.shape
    k = kb * 8
    ng = k // g
    # group sums, sequential fp16 adds (arm_gemm.cpp:250-255)
    xsum = np.zeros(ng, dtype=f16)
    for gi in range(ng):
        acc = f16(0)
        for v in x16[gi * g:(gi + 1) * g]:
            acc = f16(acc + v)
        xsum[gi] = acc
    # zero term (arm_gemm.cpp:259-286): out = sum_G xsum[G] * z[:, G]
    out = np.zeros(n, dtype=f16)
    z = np.asarray(w_zero16, dtype=f16)
    for gi in range(ng):
        out = (out + (xsum[gi] * z[:, gi]).astype(f16)).astype(f16)
    # 16-entry LUT per 4 activations, adds in order b = 0..3 (kernal.cpp:107-123)
    lut = np.zeros((k // 4, 16), dtype=f16)
    for e in range(16):
        acc = np.zeros(k // 4, dtype=f16)
        for b in range(4):
            if e >> b & 1:
                acc = (acc + x16[b::4]).astype(f16)
        lut[:, e] = acc
    chunks = np.arange(kb) * 2
    for p in range(q):
        plane = w_quant[p]                                    # [n, kb]
        lo = lut[chunks[None, :], (plane & 15)]               # [n, kb]
        hi = lut[chunks[None, :] + 1, (plane >> 4)]
        plane_acc = None
        for gi in range(ng):
            acc = np.zeros(n, dtype=f16)
            for j in range(gi * g // 8, (gi + 1) * g // 8):
                acc = (acc + lo[:, j]).astype(f16)
                acc = (acc + hi[:, j]).astype(f16)
            term = (acc * np.asarray(w_scale16[p][:, gi], dtype=f16)).astype(f16)
            plane_acc = term if plane_acc is None else (plane_acc + term).astype(f16)
        out = (out + plane_acc).astype(f16)
    if bias16 is not None:
        out = (out + np.asarray(bias16, dtype=f16)).astype(f16)
    return out


# --------------------------------------------------------------------------
# Seeded synthetic inputs with the shapes and distributions of the benchmark
# configurations (bit-planes Bernoulli(0.5), alpha = |N(0, 0.02)|, z ~ N(0, 0.01),
# activations ~ N(0, 1)); the second parameter is a standard deviation.
# --------------------------------------------------------------------------


def synth_linear(n: int, k: int, q: int, g: int, m: int = 1, seed: int = 0,
                 bias: bool = False, signed_alpha: bool = False):
    """Returns a dict of exported arrays plus activations for one linear."""
    rng = np.random.default_rng(seed)
    w_quant = rng.integers(0, 256, size=(q, n, k // 8), dtype=np.uint8)
    alpha = rng.standard_normal((q, n, k // g), dtype=np.float32) * 0.02
    if not signed_alpha:
        alpha = np.abs(alpha)
    z = rng.standard_normal((n, k // g), dtype=np.float32) * 0.01
    x = rng.standard_normal((m, k), dtype=np.float32)
    out = {
        "w_quant": w_quant,
        "w_scale": alpha.astype(np.float16),
        "w_zero": z.astype(np.float16),
        "x": x.astype(np.float16),
        "bias": None,
        "g": g,
    }
    if bias:
        out["bias"] = (rng.standard_normal(n, dtype=np.float32) * 0.1).astype(np.float16)
    return out
