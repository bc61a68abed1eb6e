"""The allocation-free forward (hlq_linear_forward_static) against the ordinary one.

Some callers cannot allocate device memory when they run a linear (their own memory
manager owns all of HBM, or they sit in a section where cudaMalloc's device-wide
synchronization is not acceptable); for them the library keeps the kernel's scratch in a
fixed 1 MiB device array.  This file is collected last on purpose: if it fails under
`pytest -x`, every other test has already run.  It passes on its own and after the others,
because each call clears the part of the shared array it uses.
"""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from elutq_b200 import _lib, format as F  # noqa: E402
from oracle import hlq_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


def _static_status(L):
    ks = ctypes.c_int(-1)
    rc = L.hlq_static_scratch_status(torch.cuda.current_device(), torch.cuda.current_stream().cuda_stream,
                                     ctypes.byref(ks))
    return rc, ks.value


def _forward_pair(L, lin_mod, x, out_dtype):
    from elutq_b200 import linear as lm
    y_ref = lm.linear_forward(x, lin_mod.weight, lin_mod.workspace, out_dtype=out_dtype, impl=_lib.IMPL_LUT8)
    i = lin_mod.weight.info
    m = x.shape[0]
    y = torch.full((m, i.out_channel), float("nan"), dtype=out_dtype, device="cuda")
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]          # cudaMemGetInfo: the driver's view, not torch's cache
    st = L.hlq_linear_forward_static(m, i.in_channel, i.out_channel, x.data_ptr(), lm._DTYPES[x.dtype],
                                     y.data_ptr(), lm._DTYPES[out_dtype], lin_mod.weight.handle,
                                     torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "hlq_linear_forward_static")
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free call changed the device's free memory"
    assert _static_status(L) == (0, 0)
    return y, y_ref


@pytest.mark.parametrize("q,n,k,g,m", [(2, 4096, 4096, 128, 1), (3, 1000, 1536, 64, 5), (2, 96, 640, 32, 16),
                                       (2, 256, 1024, 128, 21)])
def test_static_scratch_forward_matches_workspace_forward(built_lib, q, n, k, g, m):
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from elutq_b200 import linear as lm
    L = built_lib
    # the first call on a device looks up the array's address; make it outside the measured calls
    L.hlq_static_scratch_status(0, torch.cuda.current_stream().cuda_stream, ctypes.byref(ctypes.c_int()))
    d = O.synth_linear(n, k, q, g, m=m, seed=31 + n, bias=True, signed_alpha=True)
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], d["bias"], g)
    mod = lm.HLQLinear.from_exported(lin, device=0, max_batch=m)
    x = torch.from_numpy(d["x"]).cuda()
    ref64 = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"])
    # two calls in a row (the second finds the array as the first left it), then another
    # shape's worth of leftovers in between is covered by the parametrization order
    for _ in range(2):
        y32, y32_ref = _forward_pair(L, mod, x, torch.float32)
        assert O.normwise_error(y32.cpu().numpy(), y32_ref.cpu().numpy()) <= 1e-6
        assert O.normwise_error(y32.cpu().numpy(), ref64) <= 1e-5
        y16, y16_ref = _forward_pair(L, mod, x, torch.float16)
        assert O.normwise_error(y16.float().cpu().numpy(), y16_ref.float().cpu().numpy()) <= 1e-3
        assert O.normwise_error(y16.float().cpu().numpy(), ref64) <= 1e-3


def test_static_scratch_limits(built_lib):
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from elutq_b200 import linear as lm
    L = built_lib
    st = torch.cuda.current_stream().cuda_stream
    # 16 rows of x against 28672 output rows need 1.9 MB of scratch: over the 1 MiB maximum
    d = O.synth_linear(28672, 512, 2, 128, m=16, seed=2)
    big = lm.HLQLinear.from_exported(F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], None, 128),
                                     device=0, max_batch=16)
    x = torch.from_numpy(d["x"]).cuda()
    y = torch.empty((16, 28672), dtype=torch.float16, device="cuda")
    assert lm.workspace_bytes(16, 512, 28672, 2, 128) > (1 << 20)
    assert L.hlq_linear_forward_static(16, 512, 28672, x.data_ptr(), 0, y.data_ptr(), 0, big.weight.handle, st) == 3
    assert L.hlq_linear_forward_static(1, 512, 28672, x.data_ptr(), 0, y.data_ptr(), 0, big.weight.handle, st) == 0
    torch.cuda.synchronize()
    ref = O.hlq_linear(d["x"][:1], d["w_quant"], d["w_scale"], d["w_zero"], 128)
    assert O.normwise_error(y[:1].float().cpu().numpy(), ref) <= 1e-3
    # shape and layout checks
    assert L.hlq_linear_forward_static(1, 256, 28672, x.data_ptr(), 0, y.data_ptr(), 0, big.weight.handle, st) == 2
    e = O.synth_linear(64, 512, 2, 128, seed=3)
    gen = lm.HLQLinear.from_exported(F.ExportedLinear(e["w_quant"], e["w_scale"], e["w_zero"], None, 128),
                                     device=0, flags=_lib.HLQ_FLAG_FORCE_EXPORT_LAYOUT)
    assert L.hlq_linear_forward_static(1, 512, 64, x.data_ptr(), 0, y.data_ptr(), 0, gen.weight.handle, st) == 6
    # 40 rows of x run as launches of 16 rows: the limit is that of 16 rows, not of 40
    f = O.synth_linear(4096, 512, 2, 128, m=40, seed=4)
    mid = lm.HLQLinear.from_exported(F.ExportedLinear(f["w_quant"], f["w_scale"], f["w_zero"], None, 128),
                                     device=0, max_batch=40)
    x40 = torch.from_numpy(f["x"]).cuda()
    y40 = torch.empty((40, 4096), dtype=torch.float16, device="cuda")
    assert L.hlq_linear_forward_static(40, 512, 4096, x40.data_ptr(), 0, y40.data_ptr(), 0, mid.weight.handle, st) == 0
    torch.cuda.synchronize()
    ref40 = O.hlq_linear(f["x"], f["w_quant"], f["w_scale"], f["w_zero"], 128)
    assert O.normwise_error(y40.float().cpu().numpy(), ref40) <= 1e-3
    assert _static_status(L) == (0, 0)
