"""Decode chain: the ops of one token over all layers recorded once and run as ONE persistent
kernel (hlq_chain_* of the C ABI).  It stands where the reference's model loop makes one call
per op (C++/examples/models/llama.cpp:185-700): stages of linears whose inputs are ready
together, and the attention of one token, each stage reading what the one before wrote.
RMSNorm, the residual adds and the gated SiLU run inside the linears (see include/hlq_b200.h).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def interleave_rows(gate, up, axis: int):
    """Rows of a fused gate/up array as HLQ_CHAIN_OUT_GATED_SILU wants them: chunks of 16 gate
    rows, each followed by the 16 up rows of the same ffn channels.  `axis` is the row axis of
    the two arrays (NumPy arrays or torch tensors of equal shape)."""
    n = gate.shape[axis]
    if n % 16 or tuple(gate.shape) != tuple(up.shape):
        raise ValueError("gate and up must have the same shape and a multiple of 16 rows")
    split = list(gate.shape)
    split[axis:axis + 1] = [n // 16, 16]
    fused = list(gate.shape)
    fused[axis] = 2 * n
    if isinstance(gate, torch.Tensor):
        return torch.cat((gate.reshape(split), up.reshape(split)), dim=axis + 1).reshape(fused).contiguous()
    import numpy as np
    return np.ascontiguousarray(np.concatenate((gate.reshape(split), up.reshape(split)), axis=axis + 1).reshape(fused))


class DecodeChain:
    def __init__(self, device, ss_cells: int):
        self.device = torch.device(device)
        h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().hlq_chain_create(ctypes.byref(h), self.device.index, ss_cells), "hlq_chain_create")
        self._h = h
        self._keep = []          # tensors, weights and communicators the chain points into

    @staticmethod
    def linear(weight, x, y, in_kind=_lib.HLQ_CHAIN_IN_PLAIN, out_kind=_lib.HLQ_CHAIN_OUT_STORE, gamma=None,
               eps=0.0, ss_in=-1, ss_out=-1, norm_channels=0):
        for t in (x, y, gamma):
            if t is not None and (not t.is_cuda or t.dtype != torch.float16 or not t.is_contiguous()):
                raise ValueError("chain tensors must be contiguous CUDA fp16")
        m = _lib.ChainLinear(weight.handle.value, x.data_ptr(), y.data_ptr(), in_kind, out_kind,
                             gamma.data_ptr() if gamma is not None else None, float(eps), int(norm_channels),
                             int(ss_in), int(ss_out))
        m._keep = (weight, x, y, gamma)
        return m

    def add_linears(self, members, comm=None):
        arr = (_lib.ChainLinear * len(members))(*members)
        st = _lib.lib().hlq_chain_add_linears(self._h, len(members), arr, comm.handle if comm is not None else None)
        _lib.check(st, "hlq_chain_add_linears")
        self._keep += [m._keep for m in members] + [comm]

    def add_attention(self, attn, q, k, v, kcache, vcache, position, out):
        """`attn`: a glue.DecodeAttention (geometry and workspace)."""
        st = _lib.lib().hlq_chain_add_attention(
            self._h, q.data_ptr(), k.data_ptr(), v.data_ptr(), kcache.data_ptr(), vcache.data_ptr(),
            position.data_ptr(), attn.head_q, attn.head_kv, attn.dhead, attn.max_ctx, int(attn.head_major), attn.base,
            attn.scale, out.data_ptr(), attn.ws.data_ptr(), attn.nbytes)
        _lib.check(st, "hlq_chain_add_attention")
        self._keep.append((attn, q, k, v, kcache, vcache, position, out))

    def finish(self):
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().hlq_chain_finish(self._h, torch.cuda.current_stream(self.device).cuda_stream),
                       "hlq_chain_finish")

    def forward(self):
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().hlq_chain_forward(self._h, torch.cuda.current_stream(self.device).cuda_stream),
                       "hlq_chain_forward")

    def status(self) -> int:
        v = ctypes.c_int(0)
        with torch.cuda.device(self.device):
            _lib.lib().hlq_chain_status(self._h, torch.cuda.current_stream(self.device).cuda_stream, ctypes.byref(v))
        return v.value

    def info(self):
        a, b, c, d = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int64()
        _lib.check(_lib.lib().hlq_chain_info(self._h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), ctypes.byref(d)),
                   "hlq_chain_info")
        return {"stages": a.value, "linears": b.value, "rank_sums": c.value, "scratch_bytes": d.value}

    def free(self):
        if self._h is not None:
            _lib.lib().hlq_chain_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
