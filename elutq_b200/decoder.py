"""Random-init Llama-shaped decoder over HLQ linears, tensor-parallel over the GPUs of one
node.  It is the caller of the hot path that the reference's `llama::forward` is
(C++/examples/models/llama.cpp:150-774): per layer RMSNorm, q/k/v, RoPE, KV-cache append,
single-token attention, o, RMSNorm, gate/up, SiLU*up, down; then the final norm, lm_head and
argmax.  The quantized linears and the glue between them (`glue.py`: residual + RMSNorm,
RoPE + KV append + attention as one kernel, gated SiLU, argmax) are this package's kernels;
the embedding row copy is a library call; lm_head is a w4g128 HLQ linear as in the reference
(HLQ.py:76-78), or with `quantized_lm_head=False` an fp16 library product.  `fused_glue=False`
runs the same glue as PyTorch ops instead (the parity reference of the tests).  The whole
step is replayed as one CUDA graph; the position lives in device memory.

Tensor parallelism: q/k/v/gate/up are column-parallel (each rank holds whole heads / a slice
of the ffn), o/down are row-parallel followed by an all-reduce (NCCL), lm_head is
column-parallel with a local argmax and an all-gather of (value, index).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _lib
from .format import ExportedLinear
from .linear import HLQGroup, HLQWeight, Workspace, workspace_bytes


@dataclass
class DecoderConfig:
    hidden: int
    ffn: int
    layers: int
    n_heads: int
    n_kv: int
    head_dim: int
    vocab: int
    bits: int = 2
    groupsize: int = 128
    ctx: int = 2048
    rope_theta: float = 500000.0


PRESETS = {
    "llama3-8b": DecoderConfig(4096, 14336, 32, 32, 8, 128, 128256),
    "llama3-70b": DecoderConfig(8192, 28672, 80, 64, 8, 128, 128256),
    "tiny": DecoderConfig(1024, 2048, 2, 8, 2, 128, 4096, ctx=256),
}


def _random_export(n, k, q, g, gen, device):
    wq = torch.randint(0, 256, (q, n, k // 8), dtype=torch.uint8, device=device, generator=gen)
    ws = (torch.randn((q, n, k // g), device=device, generator=gen) * 0.02).abs().half()
    wz = (torch.randn((n, k // g), device=device, generator=gen) * 0.01).half()
    return ExportedLinear(wq, ws, wz, None, g)


class TPDecoder:
    """One decode step (batch 1) at position ctx-1 over a random, already filled KV cache."""

    def __init__(self, cfg: DecoderConfig, device: torch.device, rank: int = 0, world: int = 1,
                 group=None, seed: int = 0, grouped: bool = True, fused_allreduce: bool = False,
                 fused_glue: bool = True, quantized_lm_head: bool = True, fused_inputs: bool = False,
                 kv_head_major: bool = True, export=None, chain: bool = False):
        if cfg.n_heads % world or cfg.n_kv % world or cfg.ffn % world or cfg.vocab % world:
            raise ValueError("heads, kv heads, ffn and vocab must split evenly over the ranks")
        self.cfg, self.dev, self.rank, self.world, self.group = cfg, device, rank, world, group
        c = cfg
        self.hq, self.hkv = c.n_heads // world, c.n_kv // world
        q_dim, kv_dim = c.n_heads * c.head_dim, c.n_kv * c.head_dim
        gen = torch.Generator(device=device)
        rows, cols = _lib.HLQ_SHARD_ROWS, _lib.HLQ_SHARD_COLS
        self.layers = []
        self.linear_bytes = 0
        # one persistent kernel for all layers (chain.py): needs the package's glue and 128-wide heads
        self.use_chain = bool(chain and fused_glue and c.head_dim == 128 and (c.ffn // world) % 16 == 0)

        def source(n, k, lseed, bits=c.bits, groupsize=c.groupsize, given=None):
            if given is not None:           # a linear of an exported model (host arrays)
                if given.out_channel != n or given.in_channel != k:
                    raise ValueError(f"exported linear is {given.out_channel}x{given.in_channel}, expected {n}x{k}")
                return given
            gen.manual_seed(lseed)          # every rank draws the full tensor and keeps its shard
            return _random_export(n, k, bits, groupsize, gen, device)

        def load(n, k, mode, lseed, bits=c.bits, groupsize=c.groupsize, given=None):
            lin = source(n, k, lseed, bits, groupsize, given)
            w = HLQWeight.from_export(lin, device=device.index, tp_rank=rank, tp_size=world, shard_mode=mode)
            self.linear_bytes += w.info.algorithmic_bytes
            return w

        def load_gate_up(lseed_gate, lseed_up, given_gate, given_up):
            """This rank's gate and up rows as ONE weight whose rows alternate in chunks of 16
            (16 gate rows, the 16 up rows of the same ffn channels): the chain applies the gated
            SiLU where it completes such a block."""
            from .chain import interleave_rows
            fl = c.ffn // world
            lo, hi = rank * fl, (rank + 1) * fl
            g_lin = source(c.ffn, c.hidden, lseed_gate, given=given_gate)
            parts = [g_lin.w_quant[:, lo:hi], g_lin.w_scale[:, lo:hi], g_lin.w_zero[lo:hi]]
            del g_lin
            u_lin = source(c.ffn, c.hidden, lseed_up, given=given_up)
            fused = ExportedLinear(interleave_rows(parts[0], u_lin.w_quant[:, lo:hi], 1),
                                   interleave_rows(parts[1], u_lin.w_scale[:, lo:hi], 1),
                                   interleave_rows(parts[2], u_lin.w_zero[lo:hi], 0), None, u_lin.groupsize)
            del u_lin, parts
            w = HLQWeight.from_export(fused, device=device.index)
            self.linear_bytes += w.info.algorithmic_bytes
            return w

        def load_qkv(lseeds, givens):
            """This rank's q, k and v rows as ONE weight (rows q | k | v): one linear, one stage."""
            parts = []
            for (n, lseed, given) in zip((q_dim, kv_dim, kv_dim), lseeds, givens):
                lin = source(n, c.hidden, lseed, given=given)
                lo, hi = rank * (n // world), (rank + 1) * (n // world)
                parts.append((lin.w_quant[:, lo:hi], lin.w_scale[:, lo:hi], lin.w_zero[lo:hi], lin.groupsize))
                del lin
            cat = (lambda ts, ax: torch.cat(ts, dim=ax).contiguous()) if isinstance(parts[0][0], torch.Tensor) else \
                (lambda ts, ax: __import__("numpy").ascontiguousarray(__import__("numpy").concatenate(ts, axis=ax)))
            fused = ExportedLinear(cat([p[0] for p in parts], 1), cat([p[1] for p in parts], 1),
                                   cat([p[2] for p in parts], 0), None, parts[0][3])
            w = HLQWeight.from_export(fused, device=device.index)
            self.linear_bytes += w.info.algorithmic_bytes
            return w

        dt = torch.float16
        for li in range(c.layers):
            s0 = seed + li * 16
            ex = export.layers[li] if export is not None else None
            giv = (lambda name: ex.linears[name]) if ex is not None else (lambda name: None)
            L = {}
            if self.use_chain:
                L["qkv_w"] = load_qkv((s0 + 0, s0 + 1, s0 + 2), (giv("q"), giv("k"), giv("v")))
            else:
                L["q"] = load(q_dim, c.hidden, rows, s0 + 0, given=giv("q"))
                L["k"] = load(kv_dim, c.hidden, rows, s0 + 1, given=giv("k"))
                L["v"] = load(kv_dim, c.hidden, rows, s0 + 2, given=giv("v"))
            L["o"] = load(c.hidden, q_dim, cols, s0 + 3, given=giv("o"))
            L["down"] = load(c.hidden, c.ffn, cols, s0 + 6, given=giv("down"))
            if self.use_chain:
                L["gate_up"] = load_gate_up(s0 + 4, s0 + 5, giv("gate"), giv("up"))
            else:
                L["gate"] = load(c.ffn, c.hidden, rows, s0 + 4, given=giv("gate"))
                L["up"] = load(c.ffn, c.hidden, rows, s0 + 5, given=giv("up"))
            gen.manual_seed(s0 + 7)
            if ex is not None:
                L["ln1"] = torch.from_numpy(ex.ln1.astype("float16")).to(device)
                L["ln2"] = torch.from_numpy(ex.ln2.astype("float16")).to(device)
            else:
                L["ln1"] = (1 + 0.1 * torch.randn(c.hidden, device=device, generator=gen)).to(dt)
                L["ln2"] = (1 + 0.1 * torch.randn(c.hidden, device=device, generator=gen)).to(dt)
            # this rank's KV heads of a random cache filled up to ctx-1, [position][head][dhead]
            # as the reference keeps it (arm_cache.cpp:17-21)
            kfull = torch.randn((c.ctx, c.n_kv, c.head_dim), device=device, generator=gen).to(dt)
            vfull = torch.randn((c.ctx, c.n_kv, c.head_dim), device=device, generator=gen).to(dt)
            L["kc"] = kfull[:, rank * self.hkv:(rank + 1) * self.hkv].contiguous()
            L["vc"] = vfull[:, rank * self.hkv:(rank + 1) * self.hkv].contiguous()
            if export is not None:          # a real model starts with an empty cache
                L["kc"].zero_()
                L["vc"].zero_()
            if kv_head_major:
                # [head][position][dhead]: a head's positions are contiguous (a CTA of the attention
                # kernel reads 32 KB runs instead of 256 bytes out of every 2 KB)
                L["kc"] = L["kc"].permute(1, 0, 2).contiguous()
                L["vc"] = L["vc"].permute(1, 0, 2).contiguous()
            del kfull, vfull
            # buffers
            L["xn"] = torch.empty((1, c.hidden), dtype=dt, device=device)
            nq, nkv = self.hq * c.head_dim, self.hkv * c.head_dim
            L["qkv_o"] = torch.empty((1, nq + 2 * nkv), dtype=dt, device=device)       # q | k | v of this rank
            L["q_o"], L["k_o"], L["v_o"] = L["qkv_o"][:, :nq], L["qkv_o"][:, nq:nq + nkv], L["qkv_o"][:, nq + nkv:]
            L["att"] = torch.empty((1, self.hq * c.head_dim), dtype=dt, device=device)
            L["o_o"] = torch.empty((1, c.hidden), dtype=dt, device=device)
            L["xn2"] = torch.empty((1, c.hidden), dtype=dt, device=device)
            L["g_o"] = torch.empty((1, c.ffn // world), dtype=dt, device=device)
            L["u_o"] = torch.empty((1, c.ffn // world), dtype=dt, device=device)
            L["act"] = torch.empty((1, c.ffn // world), dtype=dt, device=device)
            L["d_o"] = torch.empty((1, c.hidden), dtype=dt, device=device)
            L["r1"] = torch.empty((1, c.hidden), dtype=dt, device=device)   # residual stream after attention's add
            L["r2"] = torch.empty((1, c.hidden), dtype=dt, device=device)   # ... after the MLP's add
            if grouped and not self.use_chain:
                L["qkv"] = HLQGroup([L["q"], L["k"], L["v"]], max_m=1)
                L["gu"] = HLQGroup([L["gate"], L["up"]], max_m=1)
            self.layers.append(L)
        gen.manual_seed(seed + 100003)
        vs = c.vocab // world
        self.lm_head = self.lm_w = None
        if export is not None:
            from .format import ExportedLinear as _EL
            self.embed = torch.from_numpy(export.embed.astype("float16")).to(device)
            self.norm = torch.from_numpy(export.final_norm.astype("float16")).to(device)
            quantized_lm_head = isinstance(export.lm_head, _EL)
            if quantized_lm_head:
                self.lm_w = load(c.vocab, c.hidden, rows, 0, given=export.lm_head)
                self.logits = torch.empty((1, vs), dtype=dt, device=device)
            else:
                self.lm_head = torch.from_numpy(
                    export.lm_head[rank * vs:(rank + 1) * vs].astype("float16")).to(device).contiguous()
        else:
            self.embed = (torch.randn((c.vocab, c.hidden), device=device, generator=gen) * 0.5).to(dt)
            self.norm = (1 + 0.1 * torch.randn(c.hidden, device=device, generator=gen)).to(dt)
        if export is not None:
            pass                            # loaded above
        elif quantized_lm_head:
            # the reference quantizes lm_head to w4g128 whatever the body uses (HLQ.py:76-78)
            self.lm_w = load(c.vocab, c.hidden, rows, seed + 100007, bits=4, groupsize=128)
            self.logits = torch.empty((1, vs), dtype=dt, device=device)
        else:
            self.lm_head = torch.empty((vs, c.hidden), dtype=dt, device=device)
            for r0 in range(0, c.vocab, 8192):      # every rank draws all rows, keeps its slice
                blk = (torch.randn((min(8192, c.vocab - r0), c.hidden), device=device, generator=gen) * 0.02).to(dt)
                lo, hi = max(r0, rank * vs), min(r0 + blk.shape[0], (rank + 1) * vs)
                if lo < hi:
                    self.lm_head[lo - rank * vs:hi - rank * vs] = blk[lo - r0:hi - r0]
        # scratch grows with the output rows
        n_max = max(c.hidden, c.ffn // world, q_dim // world, vs if quantized_lm_head else 0)
        need = workspace_bytes(1, c.hidden, n_max, c.bits, c.groupsize)
        self.ws = Workspace(need, device)
        pos = c.ctx - 1
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=device).float() / c.head_dim))
        ang = pos * inv
        self.cos, self.sin = torch.cos(ang), torch.sin(ang)
        self.pos = pos
        self.position = torch.tensor([pos], dtype=torch.int32, device=device)
        self.token = torch.zeros(1, dtype=torch.int64, device=device)    # input token id (a graph input)
        self.fused_glue = fused_glue
        self.kv_head_major = kv_head_major
        self.next_index = torch.zeros(1, dtype=torch.int32, device=device)
        self.next_value = torch.zeros(1, dtype=torch.float32, device=device)
        if fused_glue:
            from .glue import DecodeAttention
            self.attn = DecodeAttention(self.hq, self.hkv, c.head_dim, c.ctx, c.rope_theta, device,
                                        head_major=kv_head_major)
        self.x = torch.empty((1, c.hidden), dtype=dt, device=device)
        self.xfinal = torch.empty((1, c.hidden), dtype=dt, device=device)
        # norms and SiLU folded into the table build of the linear that follows them
        self.fused_inputs = bool(fused_inputs and fused_glue and grouped and quantized_lm_head and not self.use_chain)
        self._ops = []                       # keeps the op structs (and through them nothing else) alive
        prev_delta, prev_res = None, self.x
        for L in self.layers:
            if not grouped or self.use_chain:
                break
            if self.fused_inputs:
                from .linear import input_op
                n1 = input_op(_lib.HLQ_INPUT_ADD_RMSNORM, second=prev_res if prev_delta is not None else None,
                              gamma=L["ln1"], res_out=L["r1"] if prev_delta is not None else None, eps=1e-5)
                n1b = input_op(_lib.HLQ_INPUT_ADD_RMSNORM, second=prev_res if prev_delta is not None else None,
                               gamma=L["ln1"], eps=1e-5)
                src = prev_delta if prev_delta is not None else self.x
                L["qkv"].bind([src] * 3, [L["q_o"], L["k_o"], L["v_o"]], ops=[n1, n1b, n1b])
                res1 = L["r1"] if prev_delta is not None else self.x
                n2 = input_op(_lib.HLQ_INPUT_ADD_RMSNORM, second=res1, gamma=L["ln2"], res_out=L["r2"], eps=1e-5)
                n2b = input_op(_lib.HLQ_INPUT_ADD_RMSNORM, second=res1, gamma=L["ln2"], eps=1e-5)
                L["gu"].bind([L["o_o"]] * 2, [L["g_o"], L["u_o"]], ops=[n2, n2b])
                L["silu_op"] = input_op(_lib.HLQ_INPUT_GATED_SILU, second=L["u_o"])
                self._ops += [n1, n1b, n2, n2b]
                prev_delta, prev_res = L["d_o"], L["r2"]
            else:
                L["qkv"].bind([L["xn"]] * 3, [L["q_o"], L["k_o"], L["v_o"]])
                L["gu"].bind([L["xn2"]] * 2, [L["g_o"], L["u_o"]])
        if self.fused_inputs:
            from .linear import input_op
            self.final_op = input_op(_lib.HLQ_INPUT_ADD_RMSNORM, second=prev_res, gamma=self.norm,
                                     res_out=self.xfinal, eps=1e-5)
            self.final_src = prev_delta
        self.logit_max = torch.empty(2 * world, dtype=torch.float32, device=device)
        self.grouped = grouped
        self.graph = None
        # all-reduce of o / down inside the GEMV kernel instead of a separate NCCL launch
        self.comm = None
        if (fused_allreduce or self.use_chain) and world > 1:      # the chain sums the ranks inside its kernel
            from .tp import FusedAllReduceComm
            self.comm = FusedAllReduceComm(max_n=c.hidden, max_m=1, device=device.index, group=group)
        self.chain = None
        if self.use_chain:
            self._record_chain()

    def _record_chain(self):
        """All layers of one token as one persistent kernel: per layer the stages q/k/v ->
        attention -> o (+ residual add) -> gate/up (+ gated SiLU) -> down (+ residual add); the
        norms run in the table build of q/k/v and gate/up (the first layer's first norm, which has
        no producer inside the chain, stays a kernel of its own)."""
        from .chain import DecodeChain
        c, I = self.cfg, _lib
        ch = DecodeChain(self.dev, ss_cells=2 * len(self.layers))
        x = self.x
        for li, L in enumerate(self.layers):
            if li == 0:
                qkv_in = dict(x=L["xn"])
            else:
                qkv_in = dict(x=x, in_kind=I.HLQ_CHAIN_IN_NORM, gamma=L["ln1"], eps=1e-5, ss_in=2 * li - 1)
            ch.add_linears([ch.linear(L["qkv_w"], y=L["qkv_o"], **qkv_in)])
            ch.add_attention(self.attn, L["q_o"], L["k_o"], L["v_o"], L["kc"], L["vc"], self.position, L["att"])
            ch.add_linears([ch.linear(L["o"], L["att"], x, in_kind=I.HLQ_CHAIN_IN_ATTENTION,
                                      out_kind=I.HLQ_CHAIN_OUT_RESIDUAL, ss_out=2 * li)], comm=self.comm)
            ch.add_linears([ch.linear(L["gate_up"], x, L["act"], in_kind=I.HLQ_CHAIN_IN_NORM, gamma=L["ln2"],
                                      eps=1e-5, ss_in=2 * li, out_kind=I.HLQ_CHAIN_OUT_GATED_SILU)])
            ch.add_linears([ch.linear(L["down"], L["act"], x, out_kind=I.HLQ_CHAIN_OUT_RESIDUAL, ss_out=2 * li + 1)],
                           comm=self.comm)
        ch.finish()
        self.chain = ch

    @classmethod
    def from_export(cls, export, n_heads: int, n_kv: int, device, head_dim: int = None, ctx: int = 2048,
                    rope_theta: float = 500000.0, rank: int = 0, world: int = 1, group=None, **kw):
        """A decoder over an exported model (`model_io.read_model_export(dir)` or the path of
        the directory): what `llama::load_model` does (llama.cpp:59-115), with the linears
        sharded over the tensor-parallel ranks.  Head counts are not part of the export."""
        if isinstance(export, (str, bytes)):
            from .model_io import read_model_export
            export = read_model_export(export)
        q_lin = export.layers[0].linears["q"]
        if head_dim is None:
            head_dim = q_lin.out_channel // n_heads
        if q_lin.out_channel != n_heads * head_dim or export.layers[0].linears["k"].out_channel != n_kv * head_dim:
            raise ValueError("head counts do not match the exported q/k projections")
        cfg = DecoderConfig(export.hidden, export.ffn, len(export.layers), n_heads, n_kv, head_dim, export.vocab,
                            bits=q_lin.bits, groupsize=q_lin.groupsize, ctx=ctx, rope_theta=rope_theta)
        return cls(cfg, device, rank, world, group=group, export=export, **kw)

    # ------------------------------------------------------------------------------------
    def _linear(self, w, x, out):
        i = w.info
        st = _lib.lib().hlq_linear_forward(1, i.in_channel, i.out_channel, x.data_ptr(), _lib.HLQ_F16,
                                           out.data_ptr(), _lib.HLQ_F16, self.ws.ptr, self.ws.nbytes, w.handle,
                                           torch.cuda.current_stream(self.dev).cuda_stream)
        _lib.check(st, "hlq_linear_forward")

    def _logits(self, xn):
        if self.lm_w is None:
            return torch.matmul(xn, self.lm_head.t())
        self._linear(self.lm_w, xn, self.logits)
        return self.logits

    def _rope(self, t, heads):
        """Pairs (j, j + dhead/2) as in the reference (arm_rotary.cpp:28-49); fp32 math."""
        c = self.cfg
        t = t.view(heads, c.head_dim).float()
        a, b = t[:, :c.head_dim // 2], t[:, c.head_dim // 2:]
        return torch.cat((a * self.cos - b * self.sin, a * self.sin + b * self.cos), dim=-1).half()

    def _row_parallel(self, w, x, out, op=None):
        """o / down: this rank's partial product, summed over the ranks (`op`: input transform)."""
        if self.comm is not None:
            self.comm.forward(x, w, self.ws, out, op=op)
            return
        if op is not None:
            from .linear import linear_forward_op
            linear_forward_op(x, w, self.ws, out, op)
        else:
            self._linear(w, x, out)
        if self.world > 1:
            torch.distributed.all_reduce(out, group=self.group)

    def step_eager(self, token=None):
        """One decode step on `token` (None: the id already in self.token); returns the next
        token id (greedy) as a device tensor."""
        if self.use_chain:
            return self._step_chain(token)
        if self.fused_inputs:
            return self._step_fused_inputs(token)
        return self._step_fused(token) if self.fused_glue else self._step_torch(token)

    def _step_chain(self, token):
        """5 launches per token: the first layer's first norm, the chain kernel (all layers), the
        final norm, lm_head, argmax."""
        from . import glue
        if token is not None:
            self.token.fill_(int(token))
        torch.index_select(self.embed, 0, self.token, out=self.x)
        xn = self.layers[0]["xn"]
        glue.rmsnorm(self.x, self.layers[0]["ln1"], 1e-5, out=xn)
        self.chain.forward()
        glue.rmsnorm(self.x, self.norm, 1e-5, out=xn)
        logits = self._logits(xn)
        glue.argmax(logits.view(-1), self.next_index, self.next_value)
        self.last_logits = logits
        return self._pick(self.next_value, self.next_index)

    def _step_fused_inputs(self, token):
        """5 launches per layer: both norms (with their residual adds) and the gated SiLU run
        inside the table build of the linear they feed (hlq_input_op)."""
        from . import glue
        from .linear import linear_forward_op
        c = self.cfg
        if token is not None:
            self.token.fill_(int(token))
        torch.index_select(self.embed, 0, self.token, out=self.x)
        stream = torch.cuda.current_stream(self.dev).cuda_stream
        for L in self.layers:
            _lib.check(_lib.lib().hlq_group_forward(L["qkv"].handle, 1, stream), "hlq_group_forward")
            self.attn.forward(L["q_o"].view(self.hq, c.head_dim), L["k_o"].view(self.hkv, c.head_dim),
                              L["v_o"].view(self.hkv, c.head_dim), L["kc"], L["vc"], self.position,
                              out=L["att"].view(self.hq, c.head_dim))
            self._row_parallel(L["o"], L["att"], L["o_o"])
            _lib.check(_lib.lib().hlq_group_forward(L["gu"].handle, 1, stream), "hlq_group_forward")
            self._row_parallel(L["down"], L["g_o"], L["d_o"], op=L["silu_op"])
        linear_forward_op(self.final_src, self.lm_w, self.ws, self.logits, self.final_op)
        glue.argmax(self.logits.view(-1), self.next_index, self.next_value)
        self.last_logits = self.logits
        return self._pick(self.next_value, self.next_index)

    def _groups_or_linears(self, L, which, stream):
        if self.grouped:
            _lib.check(_lib.lib().hlq_group_forward(L[which].handle, 1, stream), "hlq_group_forward")
        elif which == "qkv":
            self._linear(L["q"], L["xn"], L["q_o"])
            self._linear(L["k"], L["xn"], L["k_o"])
            self._linear(L["v"], L["xn"], L["v_o"])
        else:
            self._linear(L["gate"], L["xn2"], L["g_o"])
            self._linear(L["up"], L["xn2"], L["u_o"])

    def _step_fused(self, token):
        """The glue as this package's kernels: 8 launches per layer.  The residual stream is
        carried the way the reference's model does (llama.cpp:193-215, 554, 717): each norm
        first adds the previous linear's output to it."""
        from . import glue
        c = self.cfg
        x = self.x
        if token is not None:
            self.token.fill_(int(token))
        torch.index_select(self.embed, 0, self.token, out=x)
        stream = torch.cuda.current_stream(self.dev).cuda_stream
        delta = None
        for L in self.layers:
            if delta is None:
                glue.rmsnorm(x, L["ln1"], 1e-5, out=L["xn"])
            else:
                glue.rmsnorm(delta, L["ln1"], 1e-5, out=L["xn"], residual=x, res_out=x)
            self._groups_or_linears(L, "qkv", stream)
            self.attn.forward(L["q_o"].view(self.hq, c.head_dim), L["k_o"].view(self.hkv, c.head_dim),
                              L["v_o"].view(self.hkv, c.head_dim), L["kc"], L["vc"], self.position,
                              out=L["att"].view(self.hq, c.head_dim))
            self._row_parallel(L["o"], L["att"], L["o_o"])
            glue.rmsnorm(L["o_o"], L["ln2"], 1e-5, out=L["xn2"], residual=x, res_out=x)
            self._groups_or_linears(L, "gu", stream)
            glue.gated_silu(L["g_o"], L["u_o"], out=L["act"])
            self._row_parallel(L["down"], L["act"], L["d_o"])
            delta = L["d_o"]
        xn = self.layers[0]["xn"]
        glue.rmsnorm(delta, self.norm, 1e-5, out=xn, residual=x, res_out=x)
        logits = self._logits(xn)                                     # this rank's slice of the vocabulary (fp16)
        glue.argmax(logits.view(-1), self.next_index, self.next_value)
        self.last_logits = logits
        return self._pick(self.next_value, self.next_index)

    def _pick(self, val, idx):
        """Greedy token over the ranks' slices: all-gather of (value, global index)."""
        c = self.cfg
        if self.world == 1:
            self.next_token = idx.long()
            return self.next_token
        mine = torch.stack((val[0].float(), (idx[0] + self.rank * (c.vocab // self.world)).float()))
        parts = self.logit_max.view(self.world, 2)
        torch.distributed.all_gather_into_tensor(self.logit_max, mine, group=self.group)
        best = parts[:, 0].argmax().view(1)
        self.next_token = parts[:, 1].gather(0, best).long()      # no host round trip: capturable
        return self.next_token

    def _step_torch(self, token):
        """The same step with the glue as PyTorch ops (fp32 math, fp16 storage)."""
        c = self.cfg
        x = self.x
        if token is not None:
            self.token.fill_(int(token))
        torch.index_select(self.embed, 0, self.token, out=x)
        stream = torch.cuda.current_stream(self.dev).cuda_stream

        def norm(t, w):
            tf = t.float()
            return (tf * w.float() / torch.sqrt((tf * tf).mean(dim=-1, keepdim=True) + 1e-5)).half()

        for L in self.layers:
            L["xn"].copy_(norm(x, L["ln1"]))
            self._groups_or_linears(L, "qkv", stream)
            q = self._rope(L["q_o"], self.hq)
            self.kv_rows(L, "kc", self.pos, self.pos + 1)[0] = self._rope(L["k_o"], self.hkv)
            self.kv_rows(L, "vc", self.pos, self.pos + 1)[0] = L["v_o"].view(self.hkv, c.head_dim)
            att = F.scaled_dot_product_attention(
                q.view(1, self.hq, 1, c.head_dim).float(),
                self.kv_rows(L, "kc", 0, self.pos + 1).permute(1, 0, 2).unsqueeze(0).float(),
                self.kv_rows(L, "vc", 0, self.pos + 1).permute(1, 0, 2).unsqueeze(0).float(), enable_gqa=True)
            L["att"].copy_(att.reshape(1, -1))
            self._row_parallel(L["o"], L["att"], L["o_o"])
            x.add_(L["o_o"])
            L["xn2"].copy_(norm(x, L["ln2"]))
            self._groups_or_linears(L, "gu", stream)
            g = L["g_o"].float()
            L["act"].copy_(L["u_o"].float() * (g / (1 + torch.exp(-g))))
            self._row_parallel(L["down"], L["act"], L["d_o"])
            x.add_(L["d_o"])
        xn = norm(x, self.norm)
        logits = self._logits(xn)
        val, idx = logits.float().max(dim=1)
        self.last_logits = logits
        return self._pick(val, idx.int())

    def capture(self, token: int = 1):
        """Warm up, then capture one step as a CUDA graph."""
        s = torch.cuda.Stream(device=self.dev)
        s.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(s):
            for _ in range(2):
                self.step_eager(token)
        torch.cuda.current_stream(self.dev).wait_stream(s)
        torch.cuda.synchronize(self.dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.step_eager(None)          # the graph reads the token id from self.token
        return self.graph

    def generate(self, first_token: int, n_tokens: int, start_position: int, use_graph: bool = True):
        """Greedy decoding of `n_tokens` tokens from `start_position` on (own glue kernels only:
        the position and the token id live in device memory, so ONE captured graph serves every
        step; between two replays the position is incremented and the chosen token fed back,
        both on the device).  Returns the token ids as a list."""
        if not self.fused_glue:
            raise RuntimeError("generate() needs the package's glue kernels (fused_glue=True)")
        if start_position < 0 or start_position + n_tokens > self.cfg.ctx:
            raise ValueError("positions leave the KV cache")
        self.position.fill_(start_position)
        self.token.fill_(int(first_token))
        if use_graph and self.graph is None:
            keep = self.position.clone()
            self.capture(first_token)
            self.position.copy_(keep)
            self.token.fill_(int(first_token))
        out = []
        for _ in range(n_tokens):
            if use_graph:
                self.graph.replay()
            else:
                self.step_eager(None)
            self.token.copy_(self.next_token.view(1))
            self.position.add_(1)
            out.append(self.next_token.view(1).clone())
        return [int(t) for t in torch.cat(out).tolist()]

    def launches_per_step(self) -> int:
        """Kernels of this package in one step (the embedding copy, the lm_head product and the
        collectives are library calls and not counted)."""
        if self.use_chain:
            return 4 + (1 if self.lm_w is not None else 0)
        per_layer = (2 if self.grouped else 5) + 2          # qkv, gate/up (+ o, down below)
        if self.fused_inputs:
            per_layer += 1                                  # attention
        elif self.fused_glue:
            per_layer += 4                                  # two norms, attention, gated silu
        tail = 1 if self.fused_inputs else (2 if self.fused_glue else 0)      # (final norm,) argmax
        return len(self.layers) * per_layer + tail + (1 if self.lm_w is not None else 0)

    def kv_rows(self, L, name, lo, hi):
        """Positions lo..hi-1 of a layer's K or V cache as a [position][head][dhead] view."""
        return L[name][:, lo:hi].permute(1, 0, 2) if self.kv_head_major else L[name][lo:hi]

    def hidden_after_step(self):
        return self.xfinal if self.fused_inputs else self.x
