"""The extra bit-plane of "sparse" weights on the GPU, through the C ABI, against the oracle:
no block listed, a few, and every block; every kernel family; shards; bit-exact round trip."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from elutq_b200 import _lib, format as F  # noqa: E402
from oracle import hlq_oracle as O  # noqa: E402
from test_sparse_format import make_sparse  # noqa: E402

pytestmark = pytest.mark.gpu


def _lm():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from elutq_b200 import linear
    return linear


@pytest.mark.parametrize("fraction", [0.0, 0.05, 1.0])
@pytest.mark.parametrize("n,k,q,g,m", [(256, 1024, 2, 128, 1), (96, 640, 3, 64, 5), (4096, 4096, 2, 128, 2)])
def test_lut_gemv_with_the_extra_plane(fraction, n, k, q, g, m):
    lm = _lm()
    d = O.synth_linear(n, k, q, g, m=m, seed=11, bias=True)
    sp = make_sparse(n, k, g, fraction, seed=12)
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], d["bias"], g, sp if sp.pairs else None)
    mod = lm.HLQLinear.from_exported(lin, device=0, max_batch=m)
    assert mod.weight.sparse_pairs() == sp.pairs
    ref = O.hlq_linear(d["x"].astype(np.float32), d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"],
                       dtype=np.float64 if n < 1000 else np.float32, sparse=(sp.mask, sp.blocks, sp.scales))
    x = torch.from_numpy(d["x"]).cuda()
    y32 = lm.linear_forward(x, mod.weight, mod.workspace, out_dtype=torch.float32)
    y16 = mod(x)
    torch.cuda.synchronize()
    assert mod.workspace.kernel_status() == 0
    assert O.normwise_error(y32.cpu().numpy(), ref) <= 2e-5
    assert O.normwise_error(y16.float().cpu().numpy(), ref) <= 1e-3
    # twice in a row: the accumulators the plane is added into are clean again
    y32b = lm.linear_forward(x, mod.weight, mod.workspace, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert O.normwise_error(y32b.cpu().numpy(), ref) <= 2e-5
    back = mod.weight.to_export()
    assert np.array_equal(back.w_quant, lin.w_quant)
    if sp.pairs:
        assert np.array_equal(back.sparse.mask, sp.mask) and np.array_equal(back.sparse.blocks, sp.blocks)
        assert np.array_equal(back.sparse.scales.view(np.uint16), sp.scales.view(np.uint16))
    else:
        assert back.sparse is None


def test_other_kernels_add_the_plane_to_their_output():
    lm = _lm()
    # exported layout (g = 256: generic kernel) and the tensor-core path (64 rows)
    d = O.synth_linear(64, 512, 2, 256, m=3, seed=21)
    sp = make_sparse(64, 512, 256, 1.0, seed=22)
    mod = lm.HLQLinear.from_exported(F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], None, 256, sp), device=0)
    assert mod.weight.info.layout == _lib.HLQ_LAYOUT_EXPORT
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], 256, sparse=(sp.mask, sp.blocks, sp.scales))
    y = lm.linear_forward(torch.from_numpy(d["x"]).cuda(), mod.weight, mod.workspace, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert O.normwise_error(y.cpu().numpy(), ref) <= 1e-5
    e = O.synth_linear(256, 1024, 2, 64, m=64, seed=23)
    sp2 = make_sparse(256, 1024, 64, 0.3, seed=24)
    mod2 = lm.HLQLinear.from_exported(F.ExportedLinear(e["w_quant"], e["w_scale"], e["w_zero"], None, 64, sp2),
                                      device=0, max_batch=64)
    ref2 = O.hlq_linear(e["x"], e["w_quant"], e["w_scale"], e["w_zero"], 64, sparse=(sp2.mask, sp2.blocks, sp2.scales))
    y2 = lm.linear_forward(torch.from_numpy(e["x"]).cuda(), mod2.weight, mod2.workspace, out_dtype=torch.float32,
                           impl=_lib.IMPL_GEMM)
    torch.cuda.synchronize()
    assert O.normwise_error(y2.cpu().numpy(), ref2) <= 1e-3          # fp16 operands of the tensor-core path


@pytest.mark.parametrize("mode", [_lib.HLQ_SHARD_ROWS, _lib.HLQ_SHARD_COLS])
def test_shards_keep_their_blocks(mode):
    lm = _lm()
    from elutq_b200 import tp
    n, k, g = 128, 1024, 128
    d = O.synth_linear(n, k, 2, g, m=1, seed=31)
    sp = make_sparse(n, k, g, 0.5, seed=32)
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], None, g, sp)
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, sparse=(sp.mask, sp.blocks, sp.scales))
    parts, kept = [], 0
    for r in range(2):
        mod = lm.HLQLinear.from_exported(lin, device=0, tp_rank=r, tp_size=2, shard_mode=mode)
        kept += mod.weight.sparse_pairs()
        x = torch.from_numpy(np.ascontiguousarray(tp.shard_activation(d["x"], r, 2, mode))).cuda()
        parts.append(lm.linear_forward(x, mod.weight, mod.workspace, out_dtype=torch.float32).cpu().numpy())
    assert kept == sp.pairs
    y = np.concatenate(parts, axis=1) if mode == _lib.HLQ_SHARD_ROWS else parts[0] + parts[1]
    assert O.normwise_error(y, ref) <= 1e-5


def test_entry_points_without_the_plane_refuse_such_weights():
    lm = _lm()
    d = O.synth_linear(64, 512, 2, 128, seed=41)
    sp = make_sparse(64, 512, 128, 1.0, seed=42)
    mod = lm.HLQLinear.from_exported(F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], None, 128, sp), device=0)
    with pytest.raises(_lib.HlqError):
        lm.HLQGroup([mod.weight], max_m=1)
    x = torch.from_numpy(d["x"]).cuda()
    y = torch.empty((1, 64), dtype=torch.float16, device="cuda")
    st = _lib.lib().hlq_linear_forward_static(1, 512, 64, x.data_ptr(), 0, y.data_ptr(), 0, mod.weight.handle,
                                              torch.cuda.current_stream().cuda_stream)
    assert st == 6
