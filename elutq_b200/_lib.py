"""ctypes binding of libhlq_b200.so (the C ABI declared in include/hlq_b200.h).

There is no fallback: if the shared library has not been built the import of this
module's ``lib()`` raises, and every operator of the package fails with it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int64, c_size_t, c_uint, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "csrc", "libhlq_b200.so")

HLQ_OK = 0
HLQ_F16, HLQ_BF16, HLQ_F32 = 0, 1, 2
HLQ_SHARD_NONE, HLQ_SHARD_ROWS, HLQ_SHARD_COLS = 0, 1, 2
HLQ_LAYOUT_STREAM, HLQ_LAYOUT_EXPORT = 0, 1
HLQ_FLAG_FORCE_EXPORT_LAYOUT = 1
IMPL_AUTO, IMPL_LUT8, IMPL_LUT4, IMPL_GEMM = 0, 1, 2, 3


class HlqError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        text = lib().hlq_last_error_string(status).decode()
        extra = ""
        if status == 4:
            extra = f" [cudaError {lib().hlq_last_cuda_error()}]"
        super().__init__(f"{where}: {text}{extra} (hlq_status {status})")


class WeightInfo(ctypes.Structure):
    _fields_ = [
        ("in_channel", c_int), ("out_channel", c_int), ("groupsize", c_int), ("bits", c_int),
        ("has_bias", c_int), ("layout", c_int), ("device", c_int),
        ("tp_rank", c_int), ("tp_size", c_int), ("shard_mode", c_int),
        ("full_in_channel", c_int), ("full_out_channel", c_int),
        ("device_bytes", c_int64), ("algorithmic_bytes", c_int64),
    ]


# name -> (restype, argtypes); every symbol include/hlq_b200.h declares
SIGNATURES = {
    "hlq_quantize_with_scales_device": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_int, c_void_p]),
    "hlq_fit_alternating_device": (c_int, [c_void_p] * 3 + [c_int64, c_int, c_int, c_int, c_void_p]),
    "hlq_pack_bits": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64]),
    "hlq_unpack_bits": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64]),
    "hlq_pack_bits_device": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p]),
    "hlq_unpack_bits_device": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p]),
    "hlq_stream_sizes": (c_int, [c_int, c_int, c_int, c_int, POINTER(c_int64), POINTER(c_int64)]),
    "hlq_repack_host": (c_int, [c_void_p] * 3 + [c_int] * 4 + [c_void_p] * 2),
    "hlq_unrepack_host": (c_int, [c_void_p] * 2 + [c_int] * 4 + [c_void_p] * 3),
    "hlq_repack_device": (c_int, [c_void_p] * 3 + [c_int] * 4 + [c_void_p] * 3),
    "hlq_unrepack_device": (c_int, [c_void_p] * 2 + [c_int] * 4 + [c_void_p] * 4),
    "hlq_weight_from_export": (c_int, [POINTER(c_void_p)] + [c_void_p] * 4 + [c_int] * 8
                               + [c_uint, c_void_p]),
    "hlq_weight_to_export": (c_int, [c_void_p] * 6),
    "hlq_weight_free": (c_int, [c_void_p]),
    "hlq_weight_get_info": (c_int, [c_void_p, POINTER(WeightInfo)]),
    "hlq_weight_buffers": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_int64),
                                   POINTER(c_void_p), POINTER(c_int64), POINTER(c_void_p)]),
    "hlq_weight_alloc": (c_int, [POINTER(c_void_p)] + [c_int] * 6 + [c_uint]),
    "hlq_weight_set_sparse": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "hlq_weight_sparse_pairs": (c_int, [c_void_p, POINTER(c_int)]),
    "hlq_weight_build_batch_codes": (c_int, [c_void_p, c_void_p]),
    "hlq_select_batch_kernel": (c_int, [c_int]),
    "hlq_select_prefill_kernel": (c_int, [c_int]),
    "hlq_weight_get_sparse": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "hlq_workspace_bytes": (c_size_t, [c_int] * 5),
    "hlq_workspace_init": (c_int, [c_void_p, c_size_t, c_void_p]),
    "hlq_workspace_status": (c_int, [c_void_p, c_void_p, POINTER(c_int)]),
    "hlq_linear_forward": (c_int, [c_int] * 3 + [c_void_p, c_int, c_void_p, c_int, c_void_p,
                                                 c_size_t, c_void_p, c_void_p]),
    "hlq_linear_forward_impl": (c_int, [c_int] * 4 + [c_void_p, c_int, c_void_p, c_int, c_void_p,
                                                      c_size_t, c_void_p, c_void_p]),
    "hlq_linear_forward_static": (c_int, [c_int] * 3 + [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "hlq_tp_comm_create": (c_int, [POINTER(c_void_p)] + [c_int] * 5),
    "hlq_tp_comm_handle": (c_int, [c_void_p, c_void_p]),
    "hlq_tp_comm_connect": (c_int, [c_void_p, c_void_p]),
    "hlq_tp_comm_free": (c_int, [c_void_p]),
    "hlq_tp_comm_buffer_bytes": (c_int, [c_void_p, POINTER(c_size_t)]),
    "hlq_tp_comm_local_buffer": (c_int, [c_void_p, POINTER(c_void_p)]),
    "hlq_tp_comm_connect_pointers": (c_int, [c_void_p, POINTER(c_void_p)]),
    "hlq_tp_comm_set_spin_limit": (c_int, [c_void_p, c_int]),
    "hlq_static_scratch_status": (c_int, [c_int, c_void_p, POINTER(c_int)]),
    "hlq_linear_forward_allreduce": (c_int, [c_int] * 3 + [c_void_p, c_int, c_void_p, c_int, c_void_p, c_size_t,
                                             c_void_p, c_void_p, c_void_p]),
    "hlq_group_create": (c_int, [POINTER(c_void_p), c_int, POINTER(c_void_p), c_int]),
    "hlq_group_bind": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_void_p), c_int, c_int, c_void_p]),
    "hlq_group_forward": (c_int, [c_void_p, c_int, c_void_p]),
    "hlq_group_status": (c_int, [c_void_p, c_void_p, POINTER(c_int)]),
    "hlq_group_info": (c_int, [c_void_p, POINTER(c_int), POINTER(c_int64), POINTER(c_int64)]),
    "hlq_group_free": (c_int, [c_void_p]),
    "hlq_linear_forward_op": (c_int, [c_int] * 3 + [c_void_p, c_int, c_void_p, c_int, c_void_p, c_size_t, c_void_p,
                                                    c_void_p, c_void_p]),
    "hlq_linear_forward_allreduce_op": (c_int, [c_int] * 3 + [c_void_p, c_int, c_void_p, c_int, c_void_p, c_size_t,
                                                c_void_p, c_void_p, c_void_p, c_void_p]),
    "hlq_group_bind_op": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_void_p), c_int, c_int, c_void_p, c_void_p]),
    "hlq_chain_create": (c_int, [POINTER(c_void_p), c_int, c_int]),
    "hlq_chain_add_linears": (c_int, [c_void_p, c_int, c_void_p, c_void_p]),
    "hlq_chain_add_attention": (c_int, [c_void_p] * 7 + [c_int] * 5 + [c_float, c_float, c_void_p, c_void_p, c_size_t]),
    "hlq_chain_finish": (c_int, [c_void_p, c_void_p]),
    "hlq_chain_forward": (c_int, [c_void_p, c_void_p]),
    "hlq_chain_status": (c_int, [c_void_p, c_void_p, POINTER(c_int)]),
    "hlq_chain_trace": (c_int, [c_void_p, c_void_p, c_int, POINTER(c_int)]),
    "hlq_chain_info": (c_int, [c_void_p, POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int64)]),
    "hlq_chain_free": (c_int, [c_void_p]),
    "hlq_rmsnorm": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p]),
    "hlq_gated_silu": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "hlq_argmax": (c_int, [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "hlq_attention_workspace_bytes": (c_size_t, [c_int] * 4),
    "hlq_rope_cache_attention": (c_int, [c_void_p] * 6 + [c_int] * 5 + [c_float, c_float, c_void_p, c_void_p,
                                                                       c_size_t, c_void_p]),
    "hlq_last_error_string": (c_char_p, [c_int]),
    "hlq_last_cuda_error": (c_int, []),
    "hlq_kernel_launch_count": (c_int64, []),
    "hlq_abi_version": (c_int, []),
}

class InputOp(ctypes.Structure):
    """hlq_input_op: a transform of the activations fused into the LUT GEMV's table build."""
    _fields_ = [("kind", c_int), ("eps", c_float), ("d_second", c_void_p), ("d_gamma", c_void_p),
                ("d_res_out", c_void_p)]


class ChainLinear(ctypes.Structure):
    """hlq_chain_linear: one linear of a decode-chain stage."""
    _fields_ = [("w", c_void_p), ("d_x", c_void_p), ("d_y", c_void_p), ("in_kind", c_int), ("out_kind", c_int),
                ("d_gamma", c_void_p), ("eps", c_float), ("norm_channels", c_int), ("ss_in", c_int), ("ss_out", c_int)]


HLQ_CHAIN_IN_PLAIN, HLQ_CHAIN_IN_NORM, HLQ_CHAIN_IN_ATTENTION = 0, 1, 2
HLQ_CHAIN_OUT_STORE, HLQ_CHAIN_OUT_RESIDUAL, HLQ_CHAIN_OUT_GATED_SILU = 0, 1, 2
HLQ_INPUT_PLAIN, HLQ_INPUT_GATED_SILU, HLQ_INPUT_ADD_RMSNORM = 0, 1, 2
HLQ_KV_POSITION_MAJOR, HLQ_KV_HEAD_MAJOR = 0, 1

_LIB = None


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m elutq_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
    return _LIB


def check(status: int, where: str) -> None:
    if status != HLQ_OK:
        raise HlqError(status, where)
