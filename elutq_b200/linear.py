"""Quantized linear operator over HLQ weights: Python mirror of the reference's
``weight_tensor`` + ``load_Parameter`` + ``arm_gemm`` (C++/ops/include/arm/arm_gemm.h:4-14,
C++/ops/include/arm/parameters.h:17, C++/ops/include/arm/arm_nnstructures.h:11-37).

PyTorch supplies device memory and streams; all arithmetic is in the CUDA kernels behind
the C ABI.  There is no CPU path: using these classes without a GPU raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch

from . import _lib
from .format import ExportedLinear, SparsePlane, export_from_tensors, read_export_dir

_DTYPES = {torch.float16: _lib.HLQ_F16, torch.bfloat16: _lib.HLQ_BF16, torch.float32: _lib.HLQ_F32}


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _src_ptr(a):
    """Host NumPy array or CUDA tensor -> raw pointer (the library detects which)."""
    if a is None:
        return None
    if isinstance(a, torch.Tensor):
        if not a.is_contiguous():
            raise ValueError("tensor arguments must be contiguous")
        return a.data_ptr()
    return np.ascontiguousarray(a).ctypes.data


class HLQWeight:
    """Owns one device-resident quantized weight (the reference's ``weight_tensor``)."""

    def __init__(self, handle: int):
        self._h = ctypes.c_void_p(handle)
        info = _lib.WeightInfo()
        _lib.check(_lib.lib().hlq_weight_get_info(self._h, ctypes.byref(info)), "hlq_weight_get_info")
        self.info = info

    # -- construction ------------------------------------------------------------------
    @classmethod
    def from_export(cls, lin: ExportedLinear, device=0, tp_rank=0, tp_size=1,
                    shard_mode=_lib.HLQ_SHARD_NONE, flags=0) -> "HLQWeight":
        """Upload exported arrays (host NumPy arrays or CUDA tensors); mirrors
        ``load_Parameter(path, PARAM_TYPE_LINEAR, ...)`` (parameters.cpp:5-70)."""
        dev = torch.device("cuda", device if isinstance(device, int) else device.index or 0)
        keep = [np.ascontiguousarray(a) if isinstance(a, np.ndarray) else a
                for a in (lin.w_quant, lin.w_scale, lin.w_zero, lin.bias)]
        out = ctypes.c_void_p()
        with torch.cuda.device(dev):
            st = _lib.lib().hlq_weight_from_export(
                ctypes.byref(out), _src_ptr(keep[0]), _src_ptr(keep[1]), _src_ptr(keep[2]),
                _src_ptr(keep[3]), lin.in_channel, lin.out_channel, lin.groupsize, lin.bits,
                dev.index, tp_rank, tp_size, shard_mode, flags, _stream_ptr(dev))
        _lib.check(st, "hlq_weight_from_export")
        self = cls(out.value)
        if lin.sparse is not None and lin.sparse.pairs:
            sp = lin.sparse
            mask = np.ascontiguousarray(sp.mask, dtype=np.uint32)
            blocks = np.ascontiguousarray(sp.blocks, dtype=np.uint8)
            scales = np.ascontiguousarray(sp.scales, dtype=np.float16)
            with torch.cuda.device(dev):
                _lib.check(_lib.lib().hlq_weight_set_sparse(self._h, mask.ctypes.data, sp.pairs, blocks.ctypes.data,
                                                            scales.ctypes.data, _stream_ptr(dev)),
                           "hlq_weight_set_sparse")
        return self

    def build_batch_codes(self):
        """Adds the second copy of the planes as 4-bit code words (2- and 3-bit weights in the streaming
        layout; half a byte per weight of device memory): calls with 3..16 rows of activations read
        them instead of the planes.  Call before the weight goes into an HLQGroup."""
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().hlq_weight_build_batch_codes(self.handle, _stream_ptr(self.device)),
                       "hlq_weight_build_batch_codes")
            torch.cuda.current_stream(self.device).synchronize()
        info = _lib.WeightInfo()
        _lib.check(_lib.lib().hlq_weight_get_info(self._h, ctypes.byref(info)), "hlq_weight_get_info")
        self.info = info
        return self

    def sparse_pairs(self) -> int:
        v = ctypes.c_int(0)
        _lib.check(_lib.lib().hlq_weight_sparse_pairs(self.handle, ctypes.byref(v)), "hlq_weight_sparse_pairs")
        return v.value

    @classmethod
    def alloc(cls, in_channel, out_channel, groupsize, bits, has_bias=False, device=0, flags=0):
        """Uninitialised weight of the given shape (benchmarks fill it on the device)."""
        out = ctypes.c_void_p()
        _lib.check(_lib.lib().hlq_weight_alloc(ctypes.byref(out), in_channel, out_channel, groupsize,
                                               bits, int(has_bias), device, flags), "hlq_weight_alloc")
        return cls(out.value)

    # -- access ------------------------------------------------------------------------
    @property
    def handle(self):
        if self._h is None:
            raise RuntimeError("weight was freed")
        return self._h

    @property
    def device(self) -> torch.device:
        return torch.device("cuda", self.info.device)

    def buffers(self):
        """(planes_ptr, planes_bytes, meta_ptr, meta_bytes, bias_ptr) device addresses."""
        p, m, b = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        pb, mb = ctypes.c_int64(), ctypes.c_int64()
        _lib.check(_lib.lib().hlq_weight_buffers(self.handle, ctypes.byref(p), ctypes.byref(pb),
                                                 ctypes.byref(m), ctypes.byref(mb), ctypes.byref(b)),
                   "hlq_weight_buffers")
        return p.value, pb.value, m.value, mb.value, b.value

    def to_export(self) -> ExportedLinear:
        """Download this shard as exported arrays (bit-exact inverse of from_export)."""
        i = self.info
        q, n, k, g = i.bits, i.out_channel, i.in_channel, i.groupsize
        wq = np.empty((q, n, k // 8), np.uint8)
        ws = np.empty((q, n, k // g), np.float16)
        wz = np.empty((n, k // g), np.float16)
        bias = np.empty(n, np.float16) if i.has_bias else None
        with torch.cuda.device(self.device):
            st = _lib.lib().hlq_weight_to_export(
                self.handle, wq.ctypes.data, ws.ctypes.data, wz.ctypes.data,
                None if bias is None else bias.ctypes.data, _stream_ptr(self.device))
        _lib.check(st, "hlq_weight_to_export")
        sparse = None
        pairs = self.sparse_pairs()
        if pairs:
            mask = np.empty((pairs, 2), np.uint32)
            blocks = np.empty((pairs, 32, g // 8), np.uint8)
            scales = np.empty((pairs, 32), np.float16)
            with torch.cuda.device(self.device):
                _lib.check(_lib.lib().hlq_weight_get_sparse(self.handle, mask.ctypes.data, blocks.ctypes.data,
                                                            scales.ctypes.data, _stream_ptr(self.device)),
                           "hlq_weight_get_sparse")
            sparse = SparsePlane(mask, blocks, scales)
        return ExportedLinear(wq, ws, wz, bias, g, sparse)

    def free(self):
        if self._h is not None:
            _lib.lib().hlq_weight_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Workspace:
    """Device scratch of the forward kernels (the reference's ``temp_workplace``,
    arm_gemm.cpp:333-348).  One workspace serves one stream at a time."""

    def __init__(self, nbytes: int, device):
        self.device = torch.device(device)
        self.buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().hlq_workspace_init(self.buf.data_ptr(), self.buf.numel(),
                                                     _stream_ptr(self.device)), "hlq_workspace_init")

    @property
    def ptr(self):
        return self.buf.data_ptr()

    @property
    def nbytes(self):
        return self.buf.numel()

    def kernel_status(self) -> int:
        """Status word left by the kernels (0 = fine); synchronizes the current stream."""
        v = ctypes.c_int(0)
        with torch.cuda.device(self.device):
            _lib.lib().hlq_workspace_status(self.ptr, _stream_ptr(self.device), ctypes.byref(v))
        return v.value


def workspace_bytes(m: int, k: int, n: int, bits: int, groupsize: int) -> int:
    return int(_lib.lib().hlq_workspace_bytes(m, k, n, bits, groupsize))


def input_op(kind: int = 0, second: Optional[torch.Tensor] = None, gamma: Optional[torch.Tensor] = None,
             res_out: Optional[torch.Tensor] = None, eps: float = 0.0) -> "_lib.InputOp":
    """An hlq_input_op: HLQ_INPUT_GATED_SILU (x = gate, second = up) or HLQ_INPUT_ADD_RMSNORM
    (second = residual to add or None, gamma, optional res_out).  The caller keeps the tensors
    alive for as long as the op is used."""
    for t in (second, gamma, res_out):
        if t is not None and (not t.is_cuda or t.dtype != torch.float16 or not t.is_contiguous()):
            raise ValueError("input-transform tensors must be contiguous CUDA fp16")
    ptr = lambda t: t.data_ptr() if t is not None else None  # noqa: E731
    return _lib.InputOp(kind, float(eps), ptr(second), ptr(gamma), ptr(res_out))


def linear_forward_op(x: torch.Tensor, weight: HLQWeight, workspace: Workspace, out: torch.Tensor,
                      op: "_lib.InputOp") -> torch.Tensor:
    """LUT GEMV (m <= 16) with an input transform applied while its tables are built
    (hlq_linear_forward_op)."""
    i = weight.info
    m = x.numel() // i.in_channel
    with torch.cuda.device(x.device):
        st = _lib.lib().hlq_linear_forward_op(m, i.in_channel, i.out_channel, x.data_ptr(), _DTYPES[x.dtype],
                                              out.data_ptr(), _DTYPES[out.dtype], workspace.ptr, workspace.nbytes,
                                              weight.handle, ctypes.byref(op), _stream_ptr(x.device))
    _lib.check(st, "hlq_linear_forward_op")
    return out


def linear_forward(x: torch.Tensor, weight: HLQWeight, workspace: Workspace,
                   out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                   impl: int = _lib.IMPL_AUTO) -> torch.Tensor:
    """``y = x . W_hat^T + bias`` on the current CUDA stream; mirrors ``arm_gemm``
    (arm_gemm.cpp:871-924): x is ``[m, k]`` (or ``[..., k]``), y ``[m, n]``, y is overwritten."""
    if not x.is_cuda:
        raise RuntimeError("HLQ linear runs on CUDA tensors only (no CPU path)")
    i = weight.info
    k, n = i.in_channel, i.out_channel
    if x.shape[-1] != k:
        raise ValueError(f"x has {x.shape[-1]} input channels, the weight expects {k}")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, k)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    if x2.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("activations must be float16 or bfloat16")
    m = x2.shape[0]
    odt = out_dtype or (out.dtype if out is not None else x2.dtype)
    if out is None:
        out = torch.empty((m, n), dtype=odt, device=x.device)
    elif out.shape[-1] != n or out.numel() != m * n or not out.is_contiguous() or out.dtype != odt:
        raise ValueError("out must be a contiguous [m, n] tensor of the output dtype")
    need = workspace_bytes(m, k, n, i.bits, i.groupsize)
    if workspace.nbytes < need:
        raise ValueError(f"workspace holds {workspace.nbytes} bytes, {need} needed")
    with torch.cuda.device(x.device):
        st = _lib.lib().hlq_linear_forward_impl(
            impl, m, k, n, x2.data_ptr(), _DTYPES[x2.dtype], out.data_ptr(), _DTYPES[odt],
            workspace.ptr, workspace.nbytes, weight.handle, _stream_ptr(x.device))
    _lib.check(st, "hlq_linear_forward")
    return out.reshape(*lead, n)


class HLQGroup:
    """Several independent quantized linears run as one persistent kernel launch
    (hlq_group_*): e.g. the q/k/v projections of a layer, or gate and up."""

    def __init__(self, weights, max_m: int = 1):
        self.weights = list(weights)          # keeps the handles alive
        arr = (ctypes.c_void_p * len(self.weights))(*[w.handle.value for w in self.weights])
        out = ctypes.c_void_p()
        self.device = self.weights[0].device
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().hlq_group_create(ctypes.byref(out), len(self.weights), arr, max_m),
                       "hlq_group_create")
        self._h = out
        self.max_m = max_m
        self._bound = None

    def bind(self, xs, ys, ops=None):
        """xs[i]: [m, k_i] fp16/bf16 CUDA tensors; ys[i]: [m, n_i] outputs (one dtype each);
        ops[i]: optional input transform of member i (see input_op)."""
        if len(xs) != len(self.weights) or len(ys) != len(self.weights):
            raise ValueError("one x and one y per member")
        for x, y, w in zip(xs, ys, self.weights):
            if x.shape[-1] != w.info.in_channel or y.shape[-1] != w.info.out_channel:
                raise ValueError("x/y do not match the member's shape")
            if not (x.is_contiguous() and y.is_contiguous()):
                raise ValueError("x and y must be contiguous")
        xa = (ctypes.c_void_p * len(xs))(*[x.data_ptr() for x in xs])
        ya = (ctypes.c_void_p * len(ys))(*[y.data_ptr() for y in ys])
        oa = None
        if ops is not None:
            if len(ops) != len(self.weights):
                raise ValueError("one op per member")
            oa = (_lib.InputOp * len(ops))(*ops)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().hlq_group_bind_op(self._h, xa, ya, _DTYPES[xs[0].dtype], _DTYPES[ys[0].dtype],
                                                    oa, _stream_ptr(self.device)), "hlq_group_bind_op")
        self._bound = (list(xs), list(ys))    # keeps the tensors alive

    def forward(self, m: int = 1):
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().hlq_group_forward(self._h, m, _stream_ptr(self.device)), "hlq_group_forward")
        return self._bound[1]

    def kernel_status(self) -> int:
        v = ctypes.c_int(0)
        with torch.cuda.device(self.device):
            _lib.lib().hlq_group_status(self._h, _stream_ptr(self.device), ctypes.byref(v))
        return v.value

    def info(self):
        c, sb, ab = ctypes.c_int(), ctypes.c_int64(), ctypes.c_int64()
        _lib.check(_lib.lib().hlq_group_info(self._h, ctypes.byref(c), ctypes.byref(sb), ctypes.byref(ab)),
                   "hlq_group_info")
        return {"count": c.value, "scratch_bytes": sb.value, "algorithmic_bytes": ab.value}

    @property
    def handle(self):
        return self._h

    def free(self):
        if self._h is not None:
            _lib.lib().hlq_group_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class HLQLinear(torch.nn.Module):
    """Drop-in quantized ``Linear`` over an exported HLQ weight.

    ``from_export_dir`` reads what the reference's exporter writes; ``from_tensors`` takes
    the tensors the exporter is called with (GPTQ/HLQ.py:207-208).
    """

    def __init__(self, weight: HLQWeight, max_batch: int = 16, impl: int = _lib.IMPL_AUTO):
        super().__init__()
        self.weight = weight
        self.impl = impl
        i = weight.info
        self.in_features, self.out_features = i.in_channel, i.out_channel
        self.bits, self.groupsize = i.bits, i.groupsize
        self.workspace = Workspace(workspace_bytes(max_batch, i.in_channel, i.out_channel, i.bits,
                                                   i.groupsize), weight.device)

    @classmethod
    def from_exported(cls, lin: ExportedLinear, device=0, tp_rank=0, tp_size=1,
                      shard_mode=_lib.HLQ_SHARD_NONE, flags=0, **kw) -> "HLQLinear":
        return cls(HLQWeight.from_export(lin, device, tp_rank, tp_size, shard_mode, flags), **kw)

    @classmethod
    def from_export_dir(cls, path: str, device=0, **kw) -> "HLQLinear":
        return cls.from_exported(read_export_dir(path), device=device, **kw)

    @classmethod
    def from_tensors(cls, quantized_w, w_scale, w_zero, bias=None, groupsize=None, device=0, **kw):
        def host(t):
            return t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else t
        lin = export_from_tensors(host(quantized_w), host(w_scale), host(w_zero),
                                  None if bias is None else host(bias), groupsize)
        return cls.from_exported(lin, device=device, **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # a batch larger than the one the workspace was sized for: make a larger workspace
        # (an allocation: not allowed while a CUDA graph is being captured)
        m = x.numel() // self.in_features
        need = workspace_bytes(m, self.in_features, self.out_features, self.bits, self.groupsize)
        if need > self.workspace.nbytes:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError(f"a batch of {m} rows needs a {need}-byte workspace; construct the module "
                                   "with max_batch >= the batch before capturing a graph")
            torch.cuda.current_stream(x.device).synchronize()
            self.workspace = Workspace(need, self.weight.device)
        return linear_forward(x, self.weight, self.workspace, impl=self.impl)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"bits={self.bits}, groupsize={self.groupsize}")
