"""The exported on-disk format of one quantized linear, and bit-plane packing.

Layout written by the reference's exporter (GPTQ/HLQ.py:177-236) and read by its
loader (C++/ops/src/arm/parameters.cpp:5-70), per linear directory:

    w_quant.bin          uint8 [q][N][K/8]   bit j of byte i = plane bit of channel 8i+j
    w_scale.bin          fp16  [q][N][K/g]
    w_zero.bin           fp16  [N][K/g]
    bias.bin (optional)  fp16  [N]
    weight_config.json   weight_data_len, base_bit, use_sparse, in_channel, out_channel,
                         has_bias (+ groupsize, which the reference's loader reads but its
                         exporter does not write; + sparse_mask_len with use_sparse)

With ``use_sparse`` the runtime's loader (parameters.cpp:44-64) expects one EXTRA bit-plane
for a list of 32-row x g-channel blocks: ``weight_mask.bin`` holds uint32 pairs (first output
row of the block, first input channel of its group), ``sparse_mask_len`` counts the uint32s;
``w_quant.bin`` continues, after the q dense planes, with one [32][g/8] byte block per pair
(arm_t_mac_kernal.cpp:577-588) and ``w_scale.bin`` with 32 fp16 scales per pair
(parameters.cpp:45, arm_t_mac_kernal.cpp:761-764):
    w[x + r, y + c] += scale[pair][r] * bit[pair][r][c]      (arm_t_mac_kernal.cpp:678-788).
No exporter in the reference writes this (HLQ.py:180 hard-codes use_sparse = False).

Packing goes through the C ABI (hlq_pack_bits / hlq_unpack_bits); there is no NumPy
re-implementation here.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import _lib


@dataclass
class SparsePlane:
    """The optional extra bit-plane of an exported linear: P blocks of 32 rows x g channels."""
    mask: np.ndarray               # uint32 [P, 2]: (first output row, first input channel), sorted by row
    blocks: np.ndarray             # uint8  [P, 32, g/8]: bit j of byte i = channel 8i+j of the group
    scales: np.ndarray             # fp16   [P, 32]: one scale per row of the block

    @property
    def pairs(self) -> int:
        return int(self.mask.shape[0])


@dataclass
class ExportedLinear:
    """The arrays of one exported linear, as NumPy views of the files' bytes."""
    w_quant: np.ndarray            # uint8 [q, N, K/8]
    w_scale: np.ndarray            # fp16  [q, N, K/g]
    w_zero: np.ndarray             # fp16  [N, K/g]
    bias: Optional[np.ndarray]     # fp16  [N] or None
    groupsize: int
    sparse: Optional[SparsePlane] = None

    @property
    def bits(self) -> int:
        return self.w_quant.shape[0]

    @property
    def out_channel(self) -> int:
        return self.w_quant.shape[1]

    @property
    def in_channel(self) -> int:
        return self.w_quant.shape[2] * 8

    def algorithmic_bytes(self) -> int:
        return self.w_quant.nbytes + self.w_scale.nbytes + self.w_zero.nbytes


def _ptr(a: np.ndarray):
    return a.ctypes.data


def pack_bits(bits: np.ndarray) -> np.ndarray:
    """uint8 [q, N, K] of {0,1} -> uint8 [q, N, K/8] (GPTQ/HLQ.py:239-251)."""
    bits = np.ascontiguousarray(bits, dtype=np.uint8)
    if bits.ndim != 3:
        raise ValueError("bits must be [q, N, K]")
    q, n, k = bits.shape
    if k % 8:
        raise ValueError("K must be a multiple of 8")
    out = np.empty((q, n, k // 8), np.uint8)
    _lib.check(_lib.lib().hlq_pack_bits(_ptr(bits), _ptr(out), q, n, k), "hlq_pack_bits")
    return out


def unpack_bits(packed: np.ndarray) -> np.ndarray:
    """uint8 [q, N, K/8] -> uint8 [q, N, K] of {0,1}."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    if packed.ndim != 3:
        raise ValueError("packed must be [q, N, K/8]")
    q, n, kb = packed.shape
    out = np.empty((q, n, kb * 8), np.uint8)
    _lib.check(_lib.lib().hlq_unpack_bits(_ptr(packed), _ptr(out), q, n, kb * 8), "hlq_unpack_bits")
    return out


def export_from_tensors(quantized_w, w_scale, w_zero, bias=None, groupsize: Optional[int] = None
                        ) -> ExportedLinear:
    """The tensors ``HLQ.export`` receives -> exported arrays (GPTQ/HLQ.py:207-236).

    quantized_w [N, K, q] of {0,1}; w_scale [N, G, q]; w_zero [N, G, 1]; bias [N] or None.
    Scales and zeros are rounded to fp16, scales and planes become plane-major.
    """
    qw = np.asarray(quantized_w)
    ws = np.asarray(w_scale, dtype=np.float32)
    wz = np.asarray(w_zero, dtype=np.float32)
    if qw.ndim != 3 or ws.ndim != 3 or wz.ndim != 3:
        raise ValueError("quantized_w, w_scale and w_zero must be 3-D")
    n, k, q = qw.shape
    g = groupsize or k // ws.shape[1]
    if ws.shape != (n, k // g, q) or wz.shape != (n, k // g, 1):
        raise ValueError("scale/zero shapes do not match [N, K/g, q] / [N, K/g, 1]")
    planes = np.ascontiguousarray(qw.astype(np.uint8).transpose(2, 0, 1))
    return ExportedLinear(
        w_quant=pack_bits(planes),
        w_scale=np.ascontiguousarray(ws.astype(np.float16).transpose(2, 0, 1)),
        w_zero=np.ascontiguousarray(wz.astype(np.float16)[:, :, 0]),
        bias=None if bias is None else np.ascontiguousarray(np.asarray(bias, dtype=np.float32).astype(np.float16)),
        groupsize=g,
    )


def write_export_dir(path: str, lin: ExportedLinear, write_groupsize: bool = False) -> None:
    """Write one linear directory exactly as the reference's exporter does.

    ``write_groupsize`` adds the ``groupsize`` key the reference's C++ loader looks for
    (parameters.cpp:17) but its exporter omits.
    """
    os.makedirs(path, exist_ok=True)
    lin.w_zero.astype(np.float16).tofile(os.path.join(path, "w_zero.bin"))
    sp = lin.sparse
    with open(os.path.join(path, "w_scale.bin"), "wb") as f:
        f.write(np.ascontiguousarray(lin.w_scale, dtype=np.float16).tobytes())
        if sp is not None:
            f.write(np.ascontiguousarray(sp.scales, dtype=np.float16).tobytes())
    with open(os.path.join(path, "w_quant.bin"), "wb") as f:
        f.write(np.ascontiguousarray(lin.w_quant, dtype=np.uint8).tobytes())
        if sp is not None:
            f.write(np.ascontiguousarray(sp.blocks, dtype=np.uint8).tobytes())
    dense_len = int(lin.in_channel * lin.out_channel * lin.bits / 8)
    cfg = {
        "weight_data_len": dense_len + (0 if sp is None else int(sp.blocks.size)),
        "base_bit": int(lin.bits),
        "use_sparse": sp is not None,
        "in_channel": int(lin.in_channel),
        "out_channel": int(lin.out_channel),
        "has_bias": lin.bias is not None,
    }
    if lin.bias is not None:
        lin.bias.astype(np.float16).tofile(os.path.join(path, "bias.bin"))
    if sp is not None:
        cfg["sparse_mask_len"] = int(sp.mask.size)
        cfg["groupsize"] = int(lin.groupsize)        # the block size cannot be derived without it
        np.ascontiguousarray(sp.mask, dtype=np.uint32).tofile(os.path.join(path, "weight_mask.bin"))
    if write_groupsize:
        cfg["groupsize"] = int(lin.groupsize)
    with open(os.path.join(path, "weight_config.json"), "w") as f:
        json.dump(cfg, f, indent=4)


def read_export_dir(path: str) -> ExportedLinear:
    """Read one linear directory (parameters.cpp:11-57).

    Errors follow the reference's loader where it has any: a missing or invalid
    ``weight_config.json`` raises (fileutils.cpp:32-43).  Unlike the reference, short
    reads raise too instead of being ignored (parameters.cpp:38).  The group size is taken
    from the config when present, else derived from the size of ``w_zero.bin``.  With
    ``use_sparse`` the extra plane's blocks, scales and mask are read as the loader does
    (parameters.cpp:44-64).
    """
    cfg_path = os.path.join(path, "weight_config.json")
    if not os.path.exists(cfg_path):
        raise RuntimeError(f"File is not exists: {cfg_path}")
    with open(cfg_path) as f:
        try:
            cfg = json.load(f)
        except json.JSONDecodeError as e:
            raise RuntimeError(f"Invalid json file: {cfg_path}") from e
    use_sparse = bool(cfg.get("use_sparse", False))
    q = int(cfg["base_bit"])
    k = int(cfg["in_channel"])
    n = int(cfg["out_channel"])
    if q < 1 or q > 4 or k % 8 or n <= 0:
        raise ValueError(f"unsupported weight_config: bits={q} in={k} out={n}")
    dense = n * k * q // 8
    want = int(cfg.get("weight_data_len", dense))
    if not use_sparse and want != dense:
        raise ValueError("weight_data_len does not match in_channel*out_channel*base_bit/8")
    w_quant = np.fromfile(os.path.join(path, "w_quant.bin"), dtype=np.uint8)
    if w_quant.size != want:
        raise ValueError(f"w_quant.bin holds {w_quant.size} bytes, expected {want}")
    w_zero = np.fromfile(os.path.join(path, "w_zero.bin"), dtype=np.float16)
    g = int(cfg.get("groupsize", 0) or 0)
    if g <= 0:
        if w_zero.size == 0 or (n * k) % w_zero.size:
            raise ValueError("cannot derive the group size from w_zero.bin")
        g = n * k // w_zero.size
    if k % g or g % 8 or w_zero.size != n * k // g:
        raise ValueError(f"w_zero.bin holds {w_zero.size} values, expected {n * k // g} at g={g}")
    w_scale = np.fromfile(os.path.join(path, "w_scale.bin"), dtype=np.float16)
    sparse = None
    if use_sparse:
        mlen = int(cfg.get("sparse_mask_len", -1))
        if mlen < 0 or mlen % 2:
            raise ValueError("use_sparse needs an even sparse_mask_len")
        pairs = mlen // 2
        mask = np.fromfile(os.path.join(path, "weight_mask.bin"), dtype=np.uint32)
        if mask.size != mlen:
            raise ValueError(f"weight_mask.bin holds {mask.size} values, expected {mlen}")
        if w_quant.size != dense + pairs * 4 * g:
            raise ValueError(f"w_quant.bin holds {w_quant.size} bytes, expected {dense + pairs * 4 * g} with {pairs} blocks")
        if w_scale.size != q * n * k // g + pairs * 32:
            raise ValueError(f"w_scale.bin holds {w_scale.size} values, expected {q * n * k // g + pairs * 32}")
        mask = mask.reshape(pairs, 2)
        if pairs and (np.any(mask[:, 0] % 32) or np.any(mask[:, 1] % g) or mask[:, 0].max() + 32 > n
                      or mask[:, 1].max() + g > k):
            raise ValueError("weight_mask.bin names a block outside the weight or off the 32-row / group grid")
        sparse = SparsePlane(mask, w_quant[dense:].reshape(pairs, 32, g // 8),
                             w_scale[q * n * k // g:].reshape(pairs, 32))
        w_quant, w_scale = w_quant[:dense], w_scale[:q * n * k // g]
    elif w_scale.size != q * n * k // g:
        raise ValueError(f"w_scale.bin holds {w_scale.size} values, expected {q * n * k // g}")
    bias = None
    if cfg.get("has_bias", False):
        bias = np.fromfile(os.path.join(path, "bias.bin"), dtype=np.float16)
        if bias.size != n:
            raise ValueError(f"bias.bin holds {bias.size} values, expected {n}")
    return ExportedLinear(w_quant.reshape(q, n, k // 8), w_scale.reshape(q, n, k // g),
                          w_zero.reshape(n, k // g), bias, g, sparse)


def repack_host(lin: ExportedLinear):
    """Exported arrays -> (planes, meta) of the streaming layout, on the CPU."""
    L = _lib.lib()
    pb, mb = _lib.c_int64(), _lib.c_int64()
    n, k, g, q = lin.out_channel, lin.in_channel, lin.groupsize, lin.bits
    _lib.check(L.hlq_stream_sizes(n, k, g, q, pb, mb), "hlq_stream_sizes")
    planes = np.empty(pb.value, np.uint8)
    meta = np.empty(mb.value // 2, np.uint16)
    wq = np.ascontiguousarray(lin.w_quant)
    ws = np.ascontiguousarray(lin.w_scale).view(np.uint16)
    wz = np.ascontiguousarray(lin.w_zero).view(np.uint16)
    _lib.check(L.hlq_repack_host(_ptr(wq), _ptr(ws), _ptr(wz), n, k, g, q, _ptr(planes), _ptr(meta)),
               "hlq_repack_host")
    return planes, meta


def unrepack_host(planes: np.ndarray, meta: np.ndarray, n: int, k: int, g: int, q: int) -> ExportedLinear:
    """Inverse of :func:`repack_host`."""
    L = _lib.lib()
    wq = np.empty((q, n, k // 8), np.uint8)
    ws = np.empty((q, n, k // g), np.uint16)
    wz = np.empty((n, k // g), np.uint16)
    planes = np.ascontiguousarray(planes, dtype=np.uint8)
    meta = np.ascontiguousarray(meta, dtype=np.uint16)
    _lib.check(L.hlq_unrepack_host(_ptr(planes), _ptr(meta), n, k, g, q, _ptr(wq), _ptr(ws), _ptr(wz)),
               "hlq_unrepack_host")
    return ExportedLinear(wq, ws.view(np.float16), wz.view(np.float16), None, g)


def quantize_with_scales_device(w, scales, zeros):
    """Assignment step of the reference's quantizer (quant.py:154-174) on the GPU.

    ``w`` fp32 CUDA ``[blocks, g]``, ``scales`` fp32 ``[blocks, q]``, ``zeros`` fp32 ``[blocks]``
    -> uint8 CUDA ``[blocks, g, q]`` of 0/1 (what ``HLQ.export`` receives as ``quantized_w``
    after its reshape, HLQ.py:207-208)."""
    import torch
    from . import _lib
    if not (w.is_cuda and scales.is_cuda and zeros.is_cuda):
        raise RuntimeError("quantize_with_scales_device runs on CUDA tensors only")
    w = w.contiguous().float()
    scales = scales.contiguous().float()
    zeros = zeros.contiguous().float().reshape(-1)
    blocks, g = w.shape
    q = scales.shape[1]
    if scales.shape[0] != blocks or zeros.numel() != blocks:
        raise ValueError("one row of scales and one zero per block")
    out = torch.empty((blocks, g, q), dtype=torch.uint8, device=w.device)
    with torch.cuda.device(w.device):
        st = _lib.lib().hlq_quantize_with_scales_device(w.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                                        out.data_ptr(), blocks, g, q,
                                                        torch.cuda.current_stream(w.device).cuda_stream)
    _lib.check(st, "hlq_quantize_with_scales_device")
    return out


def fit_alternating_device(w, bits: int, iters: int = 10):
    """Scales and offset of every block of weights by the reference's alternating fit
    (find_optimal_params_alternating, quant.py:118-153) on the GPU.

    ``w`` fp32 CUDA ``[blocks, g]`` -> (scales fp32 ``[blocks, bits]``, zeros fp32 ``[blocks]``)."""
    import torch
    from . import _lib
    if not w.is_cuda:
        raise RuntimeError("fit_alternating_device runs on CUDA tensors only")
    w = w.contiguous().float()
    blocks, g = w.shape
    scales = torch.empty((blocks, bits), dtype=torch.float32, device=w.device)
    zeros = torch.empty((blocks,), dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        st = _lib.lib().hlq_fit_alternating_device(w.data_ptr(), scales.data_ptr(), zeros.data_ptr(), blocks, g, bits,
                                                   iters, torch.cuda.current_stream(w.device).cuda_stream)
    _lib.check(st, "hlq_fit_alternating_device")
    return scales, zeros


def pseudo_quantize_device(w, bits: int, groupsize: int, iters: int = 10):
    """What the reference's ``pseudo_quantize_tensor(w, n_bit, True, g, False, get_scale_zp=True,
    use_alternating_optimization=True)`` returns (quant.py:185-213), computed on the GPU:
    (reconstruction fp32 ``[N, K]``, quantized_w uint8 ``[N, K, q]``, w_scale fp32 ``[N, K/g, q]``,
    w_zero fp32 ``[N, K/g, 1]``) - the tensors ``HLQ.export`` takes (HLQ.py:207-208) and
    ``export_from_tensors`` turns into the exported arrays."""
    n, k = w.shape
    if k % groupsize:
        raise ValueError("in_channel must be a multiple of the group size")
    blocks = w.contiguous().float().reshape(-1, groupsize)
    scales, zeros = fit_alternating_device(blocks, bits, iters)
    quantized = quantize_with_scales_device(blocks, scales, zeros)
    recon = (quantized.float() * scales.unsqueeze(1)).sum(dim=2) + zeros.unsqueeze(1)
    return (recon.reshape(n, k), quantized.reshape(n, k, bits), scales.reshape(n, k // groupsize, bits),
            zeros.reshape(n, k // groupsize, 1))
