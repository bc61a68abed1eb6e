"""CPU restatement (numpy, float64 inside) of the reference runtime's per-token glue ops.

TEST INFRASTRUCTURE ONLY: imported by tests/, never by the product path.

Each function follows the reference's C++ op named in its docstring; where the reference
rounds an intermediate to fp16 the restatement rounds there too, otherwise it computes in
float64 (the reference's fp16 dot products in attention are NOT imitated: parity of the CUDA
kernels is taken against the exact softmax(q.K)V with a tolerance, and is therefore unpinned
with respect to the NEON kernel's own rounding).
"""
from __future__ import annotations

import numpy as np


def rmsnorm(x, gamma, eps, residual=None):
    """C++/ops/src/arm/arm_rmsnorm.cpp:25-41 (plain) and :68-85 (with residual): the sum of
    squares is taken over t = x + residual before rounding, t is stored as fp16, and the
    rounded value is normalized: out = fp16(t16 * gamma / sqrt(mean(t^2) + eps)).
    Returns (out fp16, res_out fp16 or None)."""
    x = np.asarray(x, dtype=np.float16)
    t = x.astype(np.float64)
    res_out = None
    if residual is not None:
        t = t + np.asarray(residual, dtype=np.float16).astype(np.float64)
        res_out = t.astype(np.float16)
    rms = np.sqrt((t * t).sum(axis=-1, keepdims=True) / x.shape[-1] + eps)
    src = (res_out if residual is not None else x).astype(np.float64)
    out = (src * np.asarray(gamma, dtype=np.float16).astype(np.float64) / rms).astype(np.float16)
    return out, res_out


def rope(vec, position, base):
    """C++/ops/src/arm/arm_rotary.cpp:28-49: heads x dhead, pairs (j, j + dhead/2), angle
    position * base^(-2j/dhead) evaluated in fp32 by the reference; result stored as fp16."""
    v = np.asarray(vec, dtype=np.float16).astype(np.float64)
    d = v.shape[-1]
    j = np.arange(d // 2, dtype=np.float64)
    ang = np.float64(position) * np.power(np.float64(base), -(2.0 * j) / d)
    c, s = np.cos(ang), np.sin(ang)
    a, b = v[..., : d // 2], v[..., d // 2:]
    return np.concatenate((a * c - b * s, a * s + b * c), axis=-1).astype(np.float16)


def cache_append(kcache, vcache, k, v, position):
    """C++/ops/src/arm/arm_cache.cpp:17-21: caches are [position][head_kv][dhead]."""
    kcache[position] = k
    vcache[position] = v


def attention_single(q, kcache, vcache, nkv, scale):
    """C++/ops/src/arm/arm_attention.cpp:196-270: for query head h the kv head is
    h * head_kv / head_q; softmax over the first nkv cached positions of scale * q.k, then the
    weighted sum of v.  float64 throughout, result rounded to fp16."""
    q = np.asarray(q, dtype=np.float16).astype(np.float64)
    hq, d = q.shape
    hkv = kcache.shape[1]
    out = np.zeros((hq, d), dtype=np.float64)
    for h in range(hq):
        hk = h * hkv // hq
        K = kcache[:nkv, hk].astype(np.float64)
        V = vcache[:nkv, hk].astype(np.float64)
        s = (K @ q[h]) * scale
        p = np.exp(s - s.max())
        p /= p.sum()
        out[h] = p @ V
    return out.astype(np.float16)


def gated_silu(gate, up):
    """C++/ops/src/arm/arm_activation.cpp:36-49: up * gate / (1 + exp(-gate)), fp16 result."""
    g = np.asarray(gate, dtype=np.float16).astype(np.float64)
    u = np.asarray(up, dtype=np.float16).astype(np.float64)
    return (u * (g / (1.0 + np.exp(-g)))).astype(np.float16)


def argmax_first(values):
    """C++/ops/src/arm/arm_argmax.cpp:18-26: the first index of the largest value (strict >)."""
    return int(np.argmax(np.asarray(values)))
