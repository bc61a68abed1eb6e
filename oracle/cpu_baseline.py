"""ctypes front end of the C restatement of the reference's CPU LUT kernel.

TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline); see cpu_lut_gemv.c.
"""
from __future__ import annotations

import ctypes
import os
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(HERE, "libhlq_cpu_oracle.so")
        if not os.path.exists(path):
            from . import build as _b
            _b.build()
        L = ctypes.CDLL(path)
        L.hlq_cpu_workspace_bytes.restype = ctypes.c_size_t
        L.hlq_cpu_workspace_bytes.argtypes = [ctypes.c_int] * 3
        L.hlq_cpu_gemm.restype = ctypes.c_int
        L.hlq_cpu_gemm.argtypes = ([ctypes.c_int] * 3 + [ctypes.c_void_p] * 6
                                   + [ctypes.c_int] * 3 + [ctypes.c_void_p])
        L.hlq_cpu_relayout.restype = ctypes.c_int
        L.hlq_cpu_relayout.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p] * 6
        L.hlq_cpu_max_threads.restype = ctypes.c_int
        _LIB = L
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


class CpuLinear:
    """A linear loaded the way the reference's ``load_Parameter`` does: exported
    arrays re-laid-out for a fixed thread count (parameters.cpp:5-70)."""

    def __init__(self, w_quant, w_scale16, w_zero16, g, bias16=None, threads=4):
        q, n, kb = w_quant.shape
        self.q, self.n, self.k, self.g, self.threads = q, n, kb * 8, g, threads
        self.quant = np.empty(w_quant.size, np.uint8)
        self.scale = np.empty(w_scale16.size, np.float16)
        self.zero = np.empty(w_zero16.size, np.float16)
        wq = np.ascontiguousarray(w_quant, dtype=np.uint8)
        ws = np.ascontiguousarray(w_scale16, dtype=np.float16)
        wz = np.ascontiguousarray(w_zero16, dtype=np.float16)
        rc = lib().hlq_cpu_relayout(n, self.k, g, q, threads, _p(wq), _p(ws), _p(wz),
                                    _p(self.quant), _p(self.scale), _p(self.zero))
        if rc:
            raise ValueError(f"re-layout rejected the shape (code {rc}): rows per thread "
                             "chunk must be a multiple of 32")
        self.bias = None if bias16 is None else np.ascontiguousarray(bias16, dtype=np.float16)
        self.ws = np.zeros(lib().hlq_cpu_workspace_bytes(self.k, g, threads), np.uint8)

    def forward(self, x16):
        x = np.ascontiguousarray(x16, dtype=np.float16).reshape(-1, self.k)
        y = np.empty((x.shape[0], self.n), np.float16)
        rc = lib().hlq_cpu_gemm(x.shape[0], self.k, self.n, _p(x), _p(y), _p(self.quant),
                                _p(self.scale), _p(self.zero), _p(self.bias), self.g, self.q,
                                self.threads, _p(self.ws))
        if rc:
            raise ValueError(f"hlq_cpu_gemm failed with code {rc}")
        return y

    def time_forward(self, x16, iters=20, warmup=3):
        for _ in range(warmup):
            self.forward(x16)
        t0 = time.perf_counter()
        for _ in range(iters):
            self.forward(x16)
        return (time.perf_counter() - t0) / iters


def max_threads() -> int:
    return lib().hlq_cpu_max_threads()
