"""The small-batch kernel (3..16 rows of activations, one pass over the weights) against the oracle.

Tolerance: 1e-3 normwise for 16-bit outputs, as for the other kernels (the kernel rounds the
dequantized weights to fp16 and accumulates in fp32).
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from elutq_b200 import _lib, format as F  # noqa: E402
from oracle import hlq_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu

TOL_F16 = 1e-3
TOL_BF16 = 6e-3


@pytest.fixture(scope="module")
def L(built_lib):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    return built_lib


def make(d, g, **kw):
    from elutq_b200 import linear
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], d.get("bias"), g)
    return linear.HLQLinear.from_exported(lin, device=0, **kw)


def forward(mod, x, out_dtype=torch.float16):
    from elutq_b200 import linear
    y = linear.linear_forward(x, mod.weight, mod.workspace, out_dtype=out_dtype, impl=_lib.IMPL_LUT8)
    torch.cuda.synchronize()
    assert mod.workspace.kernel_status() == 0
    return y.float().cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("q", [2, 3])
@pytest.mark.parametrize("g", [128, 64, 32])
def test_every_row_count(L, q, g):
    """2..16 rows of x (two rows: the LUT kernel's paired pass), every group size of the streaming layout, ragged n and k, bias, signed scales."""
    d = O.synth_linear(200, 1152, q, g, m=16, seed=3 * q + g, bias=True, signed_alpha=True)
    mod = make(d, g, max_batch=16)
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"])
    x = torch.from_numpy(d["x"]).cuda()
    for m in range(2, 17):
        assert O.normwise_error(forward(mod, x[:m]), ref[:m]) <= TOL_F16, m


@pytest.mark.parametrize("q", [2, 3])
@pytest.mark.parametrize("n,k", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
def test_llama_shapes(L, n, k, q):
    d = O.synth_linear(n, k, q, 128, m=16, seed=170 + q)
    mod = make(d, 128, max_batch=16)
    ref = O.hlq_linear(d["x"].astype(np.float32), d["w_quant"], d["w_scale"], d["w_zero"], 128, dtype=np.float32)
    x = torch.from_numpy(d["x"]).cuda()
    for m in (2, 4, 8, 16):
        assert O.normwise_error(forward(mod, x[:m]), ref[:m]) <= TOL_F16, m


def test_repeated_calls_leave_clean_accumulators(L):
    """Calls with different row counts in a row: accumulators and counters return to zero each time, for
    this kernel's layout and the one-row kernel's alike."""
    d = O.synth_linear(512, 2048, 3, 128, m=16, seed=5)
    mod = make(d, 128, max_batch=16)
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], 128)
    x = torch.from_numpy(d["x"]).cuda()
    for m in (16, 1, 3, 8, 1, 16, 2):
        assert O.normwise_error(forward(mod, x[:m]), ref[:m]) <= TOL_F16, m


def test_bf16_activations(L):
    d = O.synth_linear(96, 1024, 3, 64, m=5, seed=19)
    mod = make(d, 64, max_batch=8)
    xb = torch.from_numpy(d["x"].astype(np.float32)).cuda().bfloat16()
    ref = O.hlq_linear(xb.float().cpu().numpy(), d["w_quant"], d["w_scale"], d["w_zero"], 64)
    assert O.normwise_error(forward(mod, xb, torch.bfloat16), ref) <= TOL_BF16


def test_group_launch_with_rows(L):
    """A group of unlike linears with 6 rows of x: one launch, every member against the oracle."""
    from elutq_b200 import linear
    shapes = [(256, 1024), (96, 2048), (640, 512)]
    ds = [O.synth_linear(n, k, 3, 128, m=6, seed=50 + i, bias=(i == 1)) for i, (n, k) in enumerate(shapes)]
    mods = [make(d, 128, max_batch=8) for d in ds]
    group = linear.HLQGroup([m.weight for m in mods], max_m=8)
    xs = [torch.from_numpy(d["x"]).cuda() for d in ds]
    ys = [torch.empty((6, n), dtype=torch.float16, device="cuda") for n, _ in shapes]
    group.bind(xs, ys)
    for _ in range(2):
        group.forward(6)
    torch.cuda.synchronize()
    assert group.kernel_status() == 0
    for d, y in zip(ds, ys):
        ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], 128, d["bias"])
        assert O.normwise_error(y.float().cpu().numpy(), ref) <= TOL_F16


@pytest.mark.parametrize("q", [2, 3])
@pytest.mark.parametrize("g", [128, 64, 32])
def test_code_words_give_the_same_numbers(L, q, g):
    """The optional copy of the planes as 4-bit code words: same tables, same selectors, so the same
    products up to the order of the fp32 additions; the handle reports the extra bytes."""
    d = O.synth_linear(200, 1152, q, g, m=16, seed=7 * q + g, bias=True, signed_alpha=True)
    plain = make(d, g, max_batch=16)
    coded = make(d, g, max_batch=16)
    before = coded.weight.info.device_bytes
    coded.weight.build_batch_codes()
    assert coded.weight.info.device_bytes - before == 224 * 1536 // 2      # n padded to 32, k to 512
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"])
    x = torch.from_numpy(d["x"]).cuda()
    for m in (1, 2, 3, 5, 8, 11, 16):
        ya, yb = forward(plain, x[:m]), forward(coded, x[:m])
        assert O.normwise_error(yb, ref[:m]) <= TOL_F16, m
        assert O.normwise_error(yb, ya) <= 2e-3, m      # one fp16 step of the output at most
    # the export is unaffected
    e0, e1 = plain.weight.to_export(), coded.weight.to_export()
    assert np.array_equal(e0.w_quant, e1.w_quant) and np.array_equal(e0.w_scale, e1.w_scale)


def test_code_words_in_a_group_at_llama_shapes(L):
    from elutq_b200 import linear
    shapes = [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)]
    ds = [O.synth_linear(n, k, 3, 128, m=8, seed=90 + i) for i, (n, k) in enumerate(shapes)]
    mods = [make(d, 128, max_batch=8) for d in ds]
    for mod in mods:
        mod.weight.build_batch_codes()
    group = linear.HLQGroup([m.weight for m in mods], max_m=8)
    xs = [torch.from_numpy(d["x"]).cuda() for d in ds]
    ys = [torch.empty((8, n), dtype=torch.float16, device="cuda") for n, _ in shapes]
    group.bind(xs, ys)
    for _ in range(2):
        group.forward(8)
    torch.cuda.synchronize()
    assert group.kernel_status() == 0
    for d, y in zip(ds, ys):
        ref = O.hlq_linear(d["x"].astype(np.float32), d["w_quant"], d["w_scale"], d["w_zero"], 128, dtype=np.float32)
        assert O.normwise_error(y.float().cpu().numpy(), ref) <= TOL_F16


@pytest.mark.parametrize("q,g", [(2, 128), (3, 128), (3, 64), (2, 32)])
def test_tcgen05_variant_gives_the_same_numbers(L, q, g):
    """The selectable tcgen05 kernel (weights dequantized into a shared-memory operand, accumulators
    in tensor memory) against the oracle and against the default kernel, with and without code words."""
    d = O.synth_linear(328, 1664, q, g, m=16, seed=11 * q + g, bias=True, signed_alpha=True)
    mod = make(d, g, max_batch=16)
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"])
    x = torch.from_numpy(d["x"]).cuda()
    base = {m: forward(mod, x[:m]) for m in (3, 8, 13, 16)}
    try:
        _lib.check(L.hlq_select_batch_kernel(2), "hlq_select_batch_kernel")
        for coded in (False, True):
            if coded:
                mod.weight.build_batch_codes()
            for m in (3, 8, 13, 16):
                y = forward(mod, x[:m])
                assert O.normwise_error(y, ref[:m]) <= TOL_F16, (m, coded)
                assert O.normwise_error(y, base[m]) <= 2e-3, (m, coded)
    finally:
        L.hlq_select_batch_kernel(0)


@pytest.mark.parametrize("q", [2, 3])
def test_tensor_memory_operand_variant_gives_the_same_numbers(L, q):
    """The selectable kernel whose weight operand lives in tensor memory (row codes, g = 128, rows a
    multiple of 128): against the oracle and the default kernel, one launch and a group of weights,
    with activations that change between calls so that a launch that wrote nothing cannot pass."""
    d = O.synth_linear(384, 1664, q, 128, m=16, seed=23 * q, bias=True, signed_alpha=True)
    mod = make(d, 128, max_batch=16)
    mod.weight.build_batch_codes()
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], 128, d["bias"])
    half = (d["x"] * np.float16(0.5)).astype(np.float16)
    ref_half = O.hlq_linear(half, d["w_quant"], d["w_scale"], d["w_zero"], 128, d["bias"])
    x, xh = torch.from_numpy(d["x"]).cuda(), torch.from_numpy(half).cuda()
    for m in (3, 8, 13, 16):
        assert O.normwise_error(forward(mod, x[:m]), ref[:m]) <= TOL_F16, m
    try:
        _lib.check(L.hlq_select_batch_kernel(3), "hlq_select_batch_kernel")
        for m in (3, 8, 13, 16):
            assert O.normwise_error(forward(mod, xh[:m]), ref_half[:m]) <= TOL_F16, m
        # a weight without row codes (rows not a multiple of 128) is served by the default kernel
        d2 = O.synth_linear(328, 1152, q, 128, m=8, seed=5, bias=False)
        mod2 = make(d2, 128, max_batch=16)
        mod2.weight.build_batch_codes()
        ref2 = O.hlq_linear(d2["x"], d2["w_quant"], d2["w_scale"], d2["w_zero"], 128, None)
        assert O.normwise_error(forward(mod2, torch.from_numpy(d2["x"]).cuda()), ref2) <= TOL_F16
    finally:
        L.hlq_select_batch_kernel(0)
