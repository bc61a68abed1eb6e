"""Bounded device waits that run out, made on the host: nothing here faults, traps or hangs a
GPU.  A world-2 communicator of the fused all-reduce gets, as its peer's receive buffer, a
local allocation that nobody ever writes (the peer is withheld on the host side).  The kernel
then pushes its own sums, waits for the peer's with a short limit, gives up, reports status 1
through the workspace and returns; the context stays usable and an ordinary call afterwards is
correct."""
import ctypes
import time

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from elutq_b200 import _lib, format as F  # noqa: E402
from oracle import hlq_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.mark.timeout(120)
def test_fused_allreduce_gives_up_on_an_absent_peer(built_lib):
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from elutq_b200 import linear as lm
    L = built_lib
    n, k, q, g = 4096, 2048, 2, 128
    d = O.synth_linear(n, k, q, g, m=1, seed=5)
    mod = lm.HLQLinear.from_exported(F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], None, g), device=0)
    x = torch.from_numpy(d["x"]).cuda()
    comm = ctypes.c_void_p()
    _lib.check(L.hlq_tp_comm_create(ctypes.byref(comm), 0, 2, n, 1, 0), "hlq_tp_comm_create")
    nbytes = ctypes.c_size_t()
    _lib.check(L.hlq_tp_comm_buffer_bytes(comm, ctypes.byref(nbytes)), "hlq_tp_comm_buffer_bytes")
    absent = torch.zeros(nbytes.value + 256, dtype=torch.uint8, device="cuda")     # rank 1's buffer: never written by a rank 1
    base = (absent.data_ptr() + 255) // 256 * 256
    peers = (ctypes.c_void_p * 2)(None, base)
    _lib.check(L.hlq_tp_comm_connect_pointers(comm, peers), "hlq_tp_comm_connect_pointers")
    _lib.check(L.hlq_tp_comm_set_spin_limit(comm, 1 << 14), "hlq_tp_comm_set_spin_limit")
    ws = lm.Workspace(lm.workspace_bytes(1, k, n, q, g), "cuda:0")
    y = torch.zeros((1, n), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    st = L.hlq_linear_forward_allreduce(1, k, n, x.data_ptr(), _lib.HLQ_F16, y.data_ptr(), _lib.HLQ_F32, ws.ptr,
                                        ws.nbytes, mod.weight.handle, comm, stream)
    assert st == 0                                   # the launch itself is fine
    ks = ctypes.c_int(0)
    rc = L.hlq_workspace_status(ws.ptr, stream, ctypes.byref(ks))
    waited = time.perf_counter() - t0
    assert rc == 8 and ks.value == 1                 # HLQ_ERR_KERNEL, "a bounded wait ran out"
    assert waited < 20.0                             # one short limit, not one per wait
    _lib.check(L.hlq_tp_comm_free(comm), "hlq_tp_comm_free")
    # the context is intact: an ordinary forward on a fresh workspace is right
    ws2 = lm.Workspace(lm.workspace_bytes(1, k, n, q, g), "cuda:0")
    y2 = lm.linear_forward(x, mod.weight, ws2, out_dtype=torch.float32)
    torch.cuda.synchronize()
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g)
    assert O.normwise_error(y2.cpu().numpy(), ref) <= 1e-5 and ws2.kernel_status() == 0


def test_generic_kernel_reports_through_the_callers_workspace(built_lib):
    """The exported-layout kernel writes its status word into the caller's workspace header
    when there is one, so hlq_workspace_status covers every implementation."""
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from elutq_b200 import linear as lm
    d = O.synth_linear(64, 512, 2, 256, m=2, seed=8)
    mod = lm.HLQLinear.from_exported(F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], None, 256), device=0)
    assert mod.weight.info.layout == _lib.HLQ_LAYOUT_EXPORT
    y = mod(torch.from_numpy(d["x"]).cuda())
    torch.cuda.synchronize()
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], 256)
    assert O.normwise_error(y.float().cpu().numpy(), ref) <= 1e-3 and mod.workspace.kernel_status() == 0
