"""Python face of the decoder glue kernels (RMSNorm, RoPE + KV append + attention, gated SiLU,
argmax): thin wrappers over the C ABI on torch CUDA tensors, for the ops the reference's model
runs between two quantized linears (C++/examples/models/llama.cpp:193-215, 396-476, 554, 646,
717, 763).  fp16 only; nothing here falls back to PyTorch ops.
"""
from __future__ import annotations

import torch

from . import _lib


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _f16(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda or t.dtype != torch.float16 or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous CUDA fp16 tensor")
    return t


def rmsnorm(x, gamma, eps, out=None, residual=None, res_out=None):
    """out = norm(x) * gamma, or with `residual`: res_out = x + residual, out = norm(res_out) * gamma
    (launch_rms_norm / launch_pre_rms_norm).  `out` may be `x`, `res_out` may be `residual`."""
    _f16(x, "x"), _f16(gamma, "gamma")
    n = x.shape[-1]
    rows = x.numel() // n
    out = torch.empty_like(x) if out is None else _f16(out, "out")
    if residual is not None:
        _f16(residual, "residual")
        res_out = torch.empty_like(x) if res_out is None else _f16(res_out, "res_out")
    st = _lib.lib().hlq_rmsnorm(rows, n, x.data_ptr(), residual.data_ptr() if residual is not None else None,
                                res_out.data_ptr() if residual is not None else None, gamma.data_ptr(), float(eps),
                                out.data_ptr(), _stream(x))
    _lib.check(st, "hlq_rmsnorm")
    return (out, res_out) if residual is not None else out


def gated_silu(gate, up, out=None):
    """silu(gate) * up (gated_silu)."""
    _f16(gate, "gate"), _f16(up, "up")
    out = torch.empty_like(gate) if out is None else _f16(out, "out")
    n = gate.shape[-1]
    st = _lib.lib().hlq_gated_silu(gate.numel() // n, n, gate.data_ptr(), up.data_ptr(), out.data_ptr(), _stream(gate))
    _lib.check(st, "hlq_gated_silu")
    return out


def argmax(values, index_out=None, value_out=None):
    """First index of the largest element of a 1-d fp16/fp32 CUDA tensor (arm_argmax_last);
    returns (index int32[1], value float32[1]) device tensors."""
    if not values.is_cuda or not values.is_contiguous() or values.dtype not in (torch.float16, torch.float32):
        raise ValueError("values must be a contiguous CUDA fp16 or fp32 tensor")
    dt = _lib.HLQ_F16 if values.dtype == torch.float16 else _lib.HLQ_F32
    if index_out is None:
        index_out = torch.empty(1, dtype=torch.int32, device=values.device)
    if value_out is None:
        value_out = torch.empty(1, dtype=torch.float32, device=values.device)
    st = _lib.lib().hlq_argmax(values.numel(), values.data_ptr(), dt, index_out.data_ptr(), value_out.data_ptr(),
                               _stream(values))
    _lib.check(st, "hlq_argmax")
    return index_out, value_out


class DecodeAttention:
    """RoPE, KV-cache append and single-token attention as one kernel
    (launch_llama_qkv_apply_rotary + arm_cache + arm_attention for one token).

    Caches are [max_ctx][head_kv][dhead] fp16 as in the reference, or with `head_major`
    [head_kv][max_ctx][dhead] (faster: a head's positions are contiguous); `position` is an
    int32 device tensor of one element (the index the new token is written at)."""

    def __init__(self, head_q: int, head_kv: int, dhead: int, max_ctx: int, rotary_base: float, device,
                 scale: float | None = None, head_major: bool = False):
        self.head_q, self.head_kv, self.dhead, self.max_ctx = head_q, head_kv, dhead, max_ctx
        self.head_major = bool(head_major)     # caches [head_kv][max_ctx][dhead] instead of the reference's
        self.base = float(rotary_base)
        self.scale = float(scale) if scale is not None else float(dhead) ** -0.5
        need = _lib.lib().hlq_attention_workspace_bytes(head_q, head_kv, dhead, max_ctx)
        if need == 0:
            raise ValueError("unsupported attention shape")
        self.ws = torch.zeros(need, dtype=torch.uint8, device=device)
        self.nbytes = need

    def forward(self, q, k, v, kcache, vcache, position, out=None):
        for t, name in ((q, "q"), (k, "k"), (v, "v"), (kcache, "kcache"), (vcache, "vcache")):
            _f16(t, name)
        if position.dtype != torch.int32 or not position.is_cuda:
            raise ValueError("position must be an int32 CUDA tensor")
        want = (self.head_kv, self.max_ctx, self.dhead) if self.head_major else (self.max_ctx, self.head_kv, self.dhead)
        if tuple(kcache.shape) != want or kcache.shape != vcache.shape:
            raise ValueError(f"caches must have shape {want}")
        if out is None:
            out = torch.empty((self.head_q, self.dhead), dtype=torch.float16, device=q.device)
        st = _lib.lib().hlq_rope_cache_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), kcache.data_ptr(),
                                                 vcache.data_ptr(), position.data_ptr(), self.head_q, self.head_kv,
                                                 self.dhead, self.max_ctx, int(self.head_major), self.base, self.scale,
                                                 out.data_ptr(),
                                                 self.ws.data_ptr(), self.nbytes, _stream(q))
        _lib.check(st, "hlq_rope_cache_attention")
        return out

    def status(self) -> int:
        import ctypes
        ks = ctypes.c_int(0)
        _lib.lib().hlq_workspace_status(self.ws.data_ptr(), torch.cuda.current_stream(self.ws.device).cuda_stream,
                                        ctypes.byref(ks))
        return ks.value
