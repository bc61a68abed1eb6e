"""CPU restatement (numpy) of one decoded token of the reference's model loop.

TEST INFRASTRUCTURE ONLY: imported by tests/, never by the product path.

Follows C++/examples/models/llama.cpp:150-774 op by op, with the ops of glue_oracle.py and the
value oracle of hlq_oracle.py: embedding row, per layer [residual add +] RMSNorm, q/k/v, RoPE,
cache append, single-token attention, o, residual add + RMSNorm, gate/up, gated SiLU, down;
final norm, lm_head.  Pinned by tests/golden/model_tiny_llama.npz: a directory written by the
reference's own quantizer driver together with the logits of the model that driver evaluates
(tests/test_model_golden.py).
"""
from __future__ import annotations

import numpy as np

from . import glue_oracle as GO
from . import hlq_oracle as O


class OracleDecoder:
    def __init__(self, export, n_heads, n_kv, rope_theta, eps, ctx=64):
        self.e, self.hq, self.hkv, self.theta, self.eps = export, int(n_heads), int(n_kv), float(rope_theta), float(eps)
        q = export.layers[0].linears["q"]
        self.dh = q.out_channel // self.hq
        self.w = [{k: O.dequantize_export(l.w_quant, l.w_scale, l.w_zero, l.groupsize, np.float64)
                   for k, l in layer.linears.items()} for layer in export.layers]
        h = export.lm_head
        self.head = (O.dequantize_export(h.w_quant, h.w_scale, h.w_zero, h.groupsize, np.float64)
                     if hasattr(h, "w_quant") else np.asarray(h, dtype=np.float64))
        self.kc = [np.zeros((ctx, self.hkv, self.dh), np.float16) for _ in export.layers]
        self.vc = [np.zeros((ctx, self.hkv, self.dh), np.float16) for _ in export.layers]

    @staticmethod
    def _lin(w, x16):
        return (np.asarray(x16, np.float16).astype(np.float64) @ w.T).astype(np.float16)

    def step(self, token, position):
        """Returns (logits float64 [vocab], final normed hidden fp16 [hidden])."""
        e = self.e
        x = np.asarray(e.embed[int(token)], np.float16)[None, :]
        delta = None
        for li, layer in enumerate(e.layers):
            w = self.w[li]
            if delta is None:
                xn, _ = GO.rmsnorm(x, layer.ln1, self.eps)
            else:
                xn, x = GO.rmsnorm(delta, layer.ln1, self.eps, residual=x)
            q = GO.rope(self._lin(w["q"], xn).reshape(self.hq, self.dh), position, self.theta)
            k = GO.rope(self._lin(w["k"], xn).reshape(self.hkv, self.dh), position, self.theta)
            v = self._lin(w["v"], xn).reshape(self.hkv, self.dh)
            GO.cache_append(self.kc[li], self.vc[li], k, v, position)
            att = GO.attention_single(q, self.kc[li], self.vc[li], position + 1, self.dh ** -0.5)
            o = self._lin(w["o"], att.reshape(1, -1))
            xn2, x = GO.rmsnorm(o, layer.ln2, self.eps, residual=x)
            act = GO.gated_silu(self._lin(w["gate"], xn2), self._lin(w["up"], xn2))
            delta = self._lin(w["down"], act)
        xf, _ = GO.rmsnorm(delta, e.final_norm, self.eps, residual=x)
        return xf.astype(np.float64)[0] @ self.head.T, xf[0]
