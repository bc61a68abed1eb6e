"""Tensor-parallel sharding of HLQ linears over the GPUs of one node.

The reference splits a GEMV's output rows over CPU threads (C++/ops/src/arm/arm_gemm.cpp:
329-349); across GPUs the same split is column parallelism.  Splitting the input channels
(row parallelism) needs one sum over ranks.

    q, k, v, gate, up   column-parallel: rows of every plane, scale and zero  -> no collective
    o, down             row-parallel: whole groups of input channels          -> all-reduce(sum)

Sharding happens on the host so that each rank uploads only its part.
"""
from __future__ import annotations

import numpy as np

from . import _lib
from .format import ExportedLinear


def shard_unit(groupsize: int) -> int:
    """Granularity of a row-parallel split: whole groups and whole 128-channel words."""
    if groupsize > 128 and groupsize % 128 == 0:
        return groupsize
    return 128 if 128 % groupsize == 0 else groupsize


def shard_exported(lin: ExportedLinear, rank: int, size: int, mode: int) -> ExportedLinear:
    """The part of an exported linear that ``rank`` of ``size`` holds."""
    if size < 1 or not 0 <= rank < size:
        raise ValueError("rank/size out of range")
    if size == 1 or mode == _lib.HLQ_SHARD_NONE:
        return lin
    n, k, g = lin.out_channel, lin.in_channel, lin.groupsize
    if mode == _lib.HLQ_SHARD_ROWS:
        if n % size:
            raise ValueError(f"out_channel {n} does not split over {size} ranks")
        lo, hi = rank * (n // size), (rank + 1) * (n // size)
        return ExportedLinear(
            np.ascontiguousarray(lin.w_quant[:, lo:hi]), np.ascontiguousarray(lin.w_scale[:, lo:hi]),
            np.ascontiguousarray(lin.w_zero[lo:hi]),
            None if lin.bias is None else np.ascontiguousarray(lin.bias[lo:hi]), g)
    if mode == _lib.HLQ_SHARD_COLS:
        if k % size or (k // size) % shard_unit(g):
            raise ValueError(f"in_channel {k} does not split over {size} ranks in units of {shard_unit(g)}")
        ks = k // size
        lo, hi = rank * ks, (rank + 1) * ks
        return ExportedLinear(
            np.ascontiguousarray(lin.w_quant[:, :, lo // 8:hi // 8]),
            np.ascontiguousarray(lin.w_scale[:, :, lo // g:hi // g]),
            np.ascontiguousarray(lin.w_zero[:, lo // g:hi // g]),
            lin.bias if rank == 0 else None, g)   # the bias is added once, by rank 0
    raise ValueError("unknown shard mode")


def shard_activation(x, rank: int, size: int, mode: int):
    """Row-parallel linears consume the matching slice of the input channels."""
    if size == 1 or mode != _lib.HLQ_SHARD_COLS:
        return x
    ks = x.shape[-1] // size
    return x[..., rank * ks:(rank + 1) * ks]


class ColumnParallelLinear:
    """y_local = x . W_hat[rows of this rank]^T; gather=True all-gathers the rows."""

    def __init__(self, lin: ExportedLinear, group=None, device=0, gather=False, **kw):
        import torch.distributed as dist
        from .linear import HLQLinear
        self.group, self.gather = group, gather
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        self.linear = HLQLinear.from_exported(shard_exported(lin, self.rank, self.size, _lib.HLQ_SHARD_ROWS),
                                              device=device, **kw)

    def __call__(self, x):
        import torch
        import torch.distributed as dist
        y = self.linear(x)
        if not self.gather or self.size == 1:
            return y
        parts = [torch.empty_like(y) for _ in range(self.size)]
        dist.all_gather(parts, y.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


class RowParallelLinear:
    """y = sum over ranks of x[channels of this rank] . W_hat[:, channels]^T (all-reduce)."""

    def __init__(self, lin: ExportedLinear, group=None, device=0, reduce=True, **kw):
        import torch.distributed as dist
        from .linear import HLQLinear
        self.group, self.reduce = group, reduce
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        self.linear = HLQLinear.from_exported(shard_exported(lin, self.rank, self.size, _lib.HLQ_SHARD_COLS),
                                              device=device, **kw)

    def __call__(self, x_local):
        import torch.distributed as dist
        y = self.linear(x_local)
        if self.reduce and self.size > 1:
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y


class FusedAllReduceComm:
    """Peer-mapped receive buffers for `hlq_linear_forward_allreduce` (all-reduce fused into the
    GEMV).  The 64-byte handles travel through ``torch.distributed.all_gather_object``."""

    def __init__(self, max_n: int, max_m: int = 1, device=0, group=None):
        import ctypes
        import torch.distributed as dist
        self.group = group
        if dist.is_available() and dist.is_initialized():
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        L = _lib.lib()
        h = ctypes.c_void_p()
        _lib.check(L.hlq_tp_comm_create(ctypes.byref(h), self.rank, self.world, max_n, max_m, device),
                   "hlq_tp_comm_create")
        self._h = h
        mine = ctypes.create_string_buffer(64)
        _lib.check(L.hlq_tp_comm_handle(h, mine), "hlq_tp_comm_handle")
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, mine.raw, group=group)
        else:
            handles[0] = mine.raw
        blob = ctypes.create_string_buffer(b"".join(handles), 64 * self.world)
        _lib.check(L.hlq_tp_comm_connect(h, blob), "hlq_tp_comm_connect")
        if self.world > 1:
            dist.barrier(group=group)          # nobody launches before every mapping exists

    @property
    def handle(self):
        return self._h

    def forward(self, x, weight, workspace, out, op=None):
        """out <- sum over ranks of x_eff . W_hat[:, this rank's channels]^T (+ bias of rank 0);
        `op`: optional input transform (linear.input_op)."""
        import ctypes
        from .linear import _DTYPES, _stream_ptr
        i = weight.info
        m = x.shape[0]
        st = _lib.lib().hlq_linear_forward_allreduce_op(
            m, i.in_channel, i.out_channel, x.data_ptr(), _DTYPES[x.dtype], out.data_ptr(), _DTYPES[out.dtype],
            workspace.ptr, workspace.nbytes, weight.handle, self._h, ctypes.byref(op) if op is not None else None,
            _stream_ptr(x.device))
        _lib.check(st, "hlq_linear_forward_allreduce")
        return out

    def free(self):
        if self._h is not None:
            _lib.lib().hlq_tp_comm_free(self._h)
            self._h = None
