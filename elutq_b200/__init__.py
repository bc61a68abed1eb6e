"""elutq_b200: B200 (sm_100a) implementation of ELUTQ's HLQ quantized-linear path.

Everything that computes lives in ``csrc/libhlq_b200.so`` behind the C ABI of
``include/hlq_b200.h``; this package is the thin host side.
"""
from ._lib import (HLQ_BF16, HLQ_F16, HLQ_F32, HLQ_FLAG_FORCE_EXPORT_LAYOUT, HLQ_LAYOUT_EXPORT,
                   HLQ_LAYOUT_STREAM, HLQ_SHARD_COLS, HLQ_SHARD_NONE, HLQ_SHARD_ROWS, IMPL_AUTO,
                   IMPL_GEMM, IMPL_LUT4, IMPL_LUT8, HlqError)
from .format import (ExportedLinear, export_from_tensors, pack_bits, read_export_dir, unpack_bits,
                     write_export_dir)

__all__ = [
    "ExportedLinear", "export_from_tensors", "pack_bits", "unpack_bits", "read_export_dir",
    "write_export_dir", "HlqError", "HLQ_F16", "HLQ_BF16", "HLQ_F32", "HLQ_SHARD_NONE",
    "HLQ_SHARD_ROWS", "HLQ_SHARD_COLS", "HLQ_LAYOUT_STREAM", "HLQ_LAYOUT_EXPORT",
    "HLQ_FLAG_FORCE_EXPORT_LAYOUT", "IMPL_AUTO", "IMPL_LUT8", "IMPL_LUT4", "IMPL_GEMM",
]


def __getattr__(name):
    # torch-dependent parts are imported on first use
    if name in ("HLQLinear", "HLQWeight", "HLQGroup", "Workspace", "linear_forward", "workspace_bytes"):
        from . import linear
        return getattr(linear, name)
    raise AttributeError(name)
