"""Parity of the CUDA path with the oracle, through the C ABI, on a B200.

Tolerances (normwise, max|y - y_ref| / max|y_ref| against the float64 product of the
dequantized weights): 1e-3 for fp16/bf16 outputs as the specification of the path states,
1e-5 for fp32 outputs (fp32 accumulation of fp16 inputs).  Packing and re-layout are
bit-exact.
"""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from conftest import golden_cases, load_golden  # noqa: E402
from elutq_b200 import _lib, format as F  # noqa: E402
from oracle import hlq_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu

TOL_F16 = 1e-3
TOL_BF16 = 6e-3   # bf16 has 8 significand bits: output rounding alone is 2^-9 = 2e-3
TOL_F32 = 1e-5


@pytest.fixture(scope="module")
def L(built_lib):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    return built_lib


def linear_mod():
    from elutq_b200 import linear
    return linear


def make(d, g, flags=0, **kw):
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], d.get("bias"), g)
    return lin, linear_mod().HLQLinear.from_exported(lin, device=0, flags=flags, **kw)


def run(mod, x16, out_dtype=torch.float16, impl=_lib.IMPL_AUTO):
    lm = linear_mod()
    x = torch.from_numpy(np.ascontiguousarray(x16)).cuda()
    y = lm.linear_forward(x, mod.weight, mod.workspace, out_dtype=out_dtype, impl=impl)
    torch.cuda.synchronize()
    assert mod.workspace.kernel_status() == 0
    return y.float().cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("name", golden_cases())
@pytest.mark.parametrize("layout", ["stream", "export"])
def test_golden_fixtures(L, name, layout):
    d = load_golden(name)
    lin = F.ExportedLinear(d["export_w_quant"], d["export_w_scale"], d["export_w_zero"], d["bias_f16"], d["g"])
    flags = _lib.HLQ_FLAG_FORCE_EXPORT_LAYOUT if layout == "export" else 0
    mod = linear_mod().HLQLinear.from_exported(lin, device=0, flags=flags)
    assert mod.weight.info.layout == (_lib.HLQ_LAYOUT_EXPORT if layout == "export" else _lib.HLQ_LAYOUT_STREAM)
    y16 = run(mod, d["x_f16"])
    y32 = run(mod, d["x_f16"], torch.float32)
    assert O.normwise_error(y16, d["y_f64"]) <= TOL_F16
    assert O.normwise_error(y32, d["y_f64"]) <= TOL_F32


SHAPES = [
    # q, n, k, g, m, bias, signed
    (2, 64, 512, 128, 1, False, False),
    (2, 40, 1024, 128, 1, True, True),      # n not a multiple of 32
    (3, 33, 640, 64, 3, False, True),       # ragged rows, partial last slice
    (4, 8, 96, 32, 2, True, False),         # k < one slice, k = 3 groups
    (1, 100, 128, 128, 1, False, False),    # k = g
    (2, 32, 1152, 128, 4, False, False),
    (3, 72, 576, 32, 8, True, True),
    (2, 256, 2048, 128, 16, False, False),
    (2, 96, 1024, 64, 17, False, False),    # more rows of x than one launch handles
    (3, 1024, 4096, 128, 1, False, False),
]


@pytest.mark.parametrize("q,n,k,g,m,bias,signed", SHAPES)
def test_stream_kernel_shapes(L, q, n, k, g, m, bias, signed):
    d = O.synth_linear(n, k, q, g, m=m, seed=100 + n + k, bias=bias, signed_alpha=signed)
    lin, mod = make(d, g, max_batch=m)
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"])
    # the LUT kernel by name: with more than 16 rows the dispatcher would pick the GEMM
    assert O.normwise_error(run(mod, d["x"], torch.float32, impl=_lib.IMPL_LUT8), ref) <= TOL_F32
    assert O.normwise_error(run(mod, d["x"], impl=_lib.IMPL_LUT8), ref) <= TOL_F16


@pytest.mark.parametrize("q,n,k,g,m,bias,signed", SHAPES + [
    (2, 64, 512, 256, 2, False, False),     # group sizes the streaming layout does not take
    (2, 48, 512, 512, 1, True, True),       # one group per row
    (3, 40, 240, 24, 2, False, True),       # groups that are not multiples of 32 channels
    (2, 16, 4104, 8, 1, False, False),      # more than one shared-memory tile, g = 8
])
def test_generic_kernel_shapes(L, q, n, k, g, m, bias, signed):
    d = O.synth_linear(n, k, q, g, m=m, seed=200 + n + k, bias=bias, signed_alpha=signed)
    lin, mod = make(d, g, flags=_lib.HLQ_FLAG_FORCE_EXPORT_LAYOUT, max_batch=m)
    assert mod.weight.info.layout == _lib.HLQ_LAYOUT_EXPORT
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"])
    assert O.normwise_error(run(mod, d["x"], torch.float32), ref) <= TOL_F32
    assert O.normwise_error(run(mod, d["x"]), ref) <= TOL_F16


def test_bf16_activations_and_outputs(L):
    d = O.synth_linear(64, 1024, 2, 128, m=2, seed=9)
    lin, mod = make(d, 128)
    xb = torch.from_numpy(d["x"].astype(np.float32)).cuda().bfloat16()
    xr = xb.float().cpu().numpy()
    ref = O.hlq_linear(xr, d["w_quant"], d["w_scale"], d["w_zero"], 128)
    lm = linear_mod()
    y32 = lm.linear_forward(xb, mod.weight, mod.workspace, out_dtype=torch.float32).cpu().numpy()
    yb = lm.linear_forward(xb, mod.weight, mod.workspace).float().cpu().numpy()
    assert O.normwise_error(y32, ref) <= TOL_F32
    assert O.normwise_error(yb, ref) <= TOL_BF16


def test_repeated_calls_agree(L):
    """The slices of a row are accumulated with fp32 atomics, so repeated calls agree to
    fp32 rounding (not bit for bit); accumulators and counters return to zero after every
    call, otherwise the second call would be off by a whole result."""
    d = O.synth_linear(4096, 4096, 2, 128, m=1, seed=0)
    lin, mod = make(d, 128)
    x = torch.from_numpy(d["x"]).cuda()
    lm = linear_mod()
    ys = [lm.linear_forward(x, mod.weight, mod.workspace, out_dtype=torch.float32).clone() for _ in range(5)]
    torch.cuda.synchronize()
    for y in ys[1:]:
        assert O.normwise_error(y.cpu().numpy(), ys[0].cpu().numpy()) <= 1e-6
    assert mod.workspace.kernel_status() == 0


@pytest.mark.parametrize("n,k,q,g", [(4096, 4096, 2, 128), (4096, 14336, 2, 128), (1024, 4096, 3, 128),
                                     (14336, 4096, 2, 128)])
def test_llama_shapes_against_oracle(L, n, k, q, g):
    """Full-size projections of the benchmark set against the float64 oracle."""
    d = O.synth_linear(n, k, q, g, m=1, seed=0)
    lin, mod = make(d, g)
    ref = O.hlq_linear(d["x"].astype(np.float32), d["w_quant"], d["w_scale"], d["w_zero"], g, dtype=np.float32)
    # float32 oracle at this size: its own rounding is ~1e-6 normwise
    assert O.normwise_error(run(mod, d["x"], torch.float32), ref) <= 2e-5
    assert O.normwise_error(run(mod, d["x"]), ref) <= TOL_F16


@pytest.mark.parametrize("m", [1, 4, 8, 16])
@pytest.mark.parametrize("n,k", [(4096, 4096), (1024, 4096)])
def test_w3g128_batches_at_llama_shapes(L, n, k, m):
    """Llama-3-8B projections at w3g128 with 1, 4, 8 and 16 rows of activations."""
    d = O.synth_linear(n, k, 3, 128, m=m, seed=40 + m)
    lin, mod = make(d, 128, max_batch=m)
    ref = O.hlq_linear(d["x"].astype(np.float32), d["w_quant"], d["w_scale"], d["w_zero"], 128, dtype=np.float32)
    assert O.normwise_error(run(mod, d["x"], torch.float32), ref) <= 2e-5
    assert O.normwise_error(run(mod, d["x"]), ref) <= TOL_F16


@pytest.mark.parametrize("q", [2, 3])
@pytest.mark.parametrize("n,k", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
def test_paired_rows_at_every_llama_shape(L, n, k, q):
    """2, 4, 8 and 16 rows of activations (passes of two rows with fp16 table entries) at all
    four projection shapes of the benchmark set, w2g128 and w3g128, the longest accumulation
    (k = 14336) included."""
    d = O.synth_linear(n, k, q, 128, m=16, seed=70 + q)
    lin, mod = make(d, 128, max_batch=16)
    ref = O.hlq_linear(d["x"].astype(np.float32), d["w_quant"], d["w_scale"], d["w_zero"], 128, dtype=np.float32)
    for m in (2, 4, 8, 16):
        assert O.normwise_error(run(mod, d["x"][:m]), ref[:m]) <= TOL_F16, m
    assert O.normwise_error(run(mod, d["x"][:3], torch.float32), ref[:3]) <= 2e-5


def test_linear_module_grows_its_workspace(L):
    """A module built with the default max_batch takes a prefill-sized batch: the workspace is
    re-made when a call needs more (fp16 and bf16 activations, tensor-core path)."""
    d = O.synth_linear(256, 1024, 2, 64, m=64, seed=12)
    lin, mod = make(d, 64)
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], 64)
    x = torch.from_numpy(d["x"]).cuda()
    y = mod(x)
    yb = mod(x.bfloat16())
    torch.cuda.synchronize()
    assert mod.workspace.kernel_status() == 0
    assert O.normwise_error(y.float().cpu().numpy(), ref) <= TOL_F16
    refb = O.hlq_linear(x.bfloat16().float().cpu().numpy(), d["w_quant"], d["w_scale"], d["w_zero"], 64)
    assert O.normwise_error(yb.float().cpu().numpy(), refb) <= TOL_BF16


def test_size_independent_properties(L):
    """Properties at full size: scaling x by two scales y by two, zero activations give
    exactly the bias, and the two independent kernels agree."""
    n, k, q, g = 4096, 4096, 2, 128
    d = O.synth_linear(n, k, q, g, m=1, seed=3, bias=False)
    lin, mod = make(d, g)
    _, gen = make(d, g, flags=_lib.HLQ_FLAG_FORCE_EXPORT_LAYOUT)
    y1 = run(mod, d["x"], torch.float32)
    y2 = run(mod, (d["x"].astype(np.float32) * 2).astype(np.float16), torch.float32)
    assert O.normwise_error(y2, 2 * y1) <= 1e-6          # exact up to the order of the slice sums
    yg = run(gen, d["x"], torch.float32)
    assert O.normwise_error(yg, y1) <= TOL_F32
    db = O.synth_linear(n, k, q, g, m=1, seed=3, bias=True)
    _, modb = make(db, g)
    y0 = run(modb, np.zeros_like(db["x"]))
    assert np.array_equal(y0, db["bias"].astype(np.float64)[None, :])


@pytest.mark.parametrize("q,n,k,g", [(2, 64, 512, 128), (3, 33, 640, 64), (4, 8, 96, 32), (2, 4096, 4096, 128)])
def test_weight_roundtrip_is_bit_exact(L, q, n, k, g):
    d = O.synth_linear(n, k, q, g, seed=n + q, bias=True)
    for flags in (0, _lib.HLQ_FLAG_FORCE_EXPORT_LAYOUT):
        lin, mod = make(d, g, flags=flags)
        back = mod.weight.to_export()
        assert np.array_equal(back.w_quant, lin.w_quant)
        assert np.array_equal(back.w_scale.view(np.uint16), lin.w_scale.view(np.uint16))
        assert np.array_equal(back.w_zero.view(np.uint16), lin.w_zero.view(np.uint16))
        assert np.array_equal(back.bias.view(np.uint16), lin.bias.view(np.uint16))


@pytest.mark.parametrize("q,n,k,g", [(2, 64, 512, 128), (3, 33, 640, 64), (4, 8, 96, 32)])
def test_device_repack_equals_host_repack(L, q, n, k, g):
    d = O.synth_linear(n, k, q, g, seed=1)
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], None, g)
    planes, meta = F.repack_host(lin)
    wq = torch.from_numpy(lin.w_quant).cuda()
    ws = torch.from_numpy(lin.w_scale.view(np.int16)).cuda()
    wz = torch.from_numpy(lin.w_zero.view(np.int16)).cuda()
    dp = torch.empty(planes.size, dtype=torch.uint8, device="cuda")
    dm = torch.empty(meta.size, dtype=torch.int16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.hlq_repack_device(wq.data_ptr(), ws.data_ptr(), wz.data_ptr(), n, k, g, q,
                                   dp.data_ptr(), dm.data_ptr(), st), "hlq_repack_device")
    assert np.array_equal(dp.cpu().numpy(), planes)
    assert np.array_equal(dm.cpu().numpy().view(np.uint16), meta)
    # and back
    bq, bs, bz = torch.empty_like(wq), torch.empty_like(ws), torch.empty_like(wz)
    _lib.check(L.hlq_unrepack_device(dp.data_ptr(), dm.data_ptr(), n, k, g, q, bq.data_ptr(),
                                     bs.data_ptr(), bz.data_ptr(), st), "hlq_unrepack_device")
    assert torch.equal(bq, wq) and torch.equal(bs, ws) and torch.equal(bz, wz)


def test_device_pack_unpack(L):
    rng = np.random.default_rng(4)
    bits = rng.integers(0, 2, size=(3, 50, 264), dtype=np.uint8)
    db = torch.from_numpy(bits).cuda()
    dp = torch.empty((3, 50, 33), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(L.hlq_pack_bits_device(db.data_ptr(), dp.data_ptr(), 3, 50, 264, st), "pack")
    assert np.array_equal(dp.cpu().numpy(), F.pack_bits(bits))
    du = torch.empty_like(db)
    _lib.check(L.hlq_unpack_bits_device(dp.data_ptr(), du.data_ptr(), 3, 50, 264, st), "unpack")
    assert torch.equal(du, db)
    assert L.hlq_pack_bits_device(None, None, 0, 0, 0, st) == 0      # empty input


def test_sharded_weights_reproduce_the_full_product(L):
    """Column-parallel shards concatenate, row-parallel shards add up (one GPU holding
    every shard in turn; the collective itself is covered by the CPU multi-process test)."""
    from elutq_b200 import tp
    n, k, q, g = 256, 2048, 2, 128
    d = O.synth_linear(n, k, q, g, m=2, seed=8, bias=True)
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], d["bias"], g)
    ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"])
    lm = linear_mod()
    for size in (2, 4):
        cols = [lm.HLQLinear.from_exported(lin, device=0, tp_rank=r, tp_size=size, shard_mode=_lib.HLQ_SHARD_ROWS)
                for r in range(size)]
        y = np.concatenate([run(mod, d["x"], torch.float32) for mod in cols], axis=1)
        assert O.normwise_error(y, ref) <= TOL_F32
        rows = [lm.HLQLinear.from_exported(lin, device=0, tp_rank=r, tp_size=size, shard_mode=_lib.HLQ_SHARD_COLS)
                for r in range(size)]
        y = sum(run(mod, tp.shard_activation(d["x"], r, size, _lib.HLQ_SHARD_COLS), torch.float32)
                for r, mod in enumerate(rows))
        assert O.normwise_error(y, ref) <= TOL_F32
        # the library's own split equals the host-side split
        for r, mod in enumerate(rows):
            want = tp.shard_exported(lin, r, size, _lib.HLQ_SHARD_COLS)
            got = mod.weight.to_export()
            assert np.array_equal(got.w_quant, want.w_quant)
            assert (got.bias is None) == (r != 0)


def test_group_launch_matches_oracle_and_single_launches(L):
    """Several projections in one persistent launch: same results as one launch each, to
    fp32 rounding."""
    lm = linear_mod()
    shapes = [(256, 1024), (64, 1024), (64, 1024), (1000, 1024), (512, 2560), (40, 512)]
    for q, g, m in [(2, 128, 1), (3, 64, 3)]:
        mods, xs, refs = [], [], []
        for i, (n, k) in enumerate(shapes):
            d = O.synth_linear(n, k, q, g, m=m, seed=50 + i, bias=(i % 2 == 0), signed_alpha=True)
            _, mod = make(d, g, max_batch=m)
            mods.append(mod)
            xs.append(torch.from_numpy(d["x"]).cuda())
            refs.append(O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"]))
        ys = [torch.empty((m, n), dtype=torch.float32, device="cuda") for n, _ in shapes]
        grp = lm.HLQGroup([mod.weight for mod in mods], max_m=m)
        grp.bind(xs, ys)
        for _ in range(3):                      # counters must return to zero between launches
            grp.forward(m)
        torch.cuda.synchronize()
        assert grp.kernel_status() == 0
        assert grp.info()["count"] == len(shapes)
        for mod, x, y, ref in zip(mods, xs, ys, refs):
            assert O.normwise_error(y.cpu().numpy(), ref) <= TOL_F32
            single = lm.linear_forward(x, mod.weight, mod.workspace, out_dtype=torch.float32)
            assert O.normwise_error(single.cpu().numpy(), y.cpu().numpy()) <= 1e-6
        y16 = [torch.empty((m, n), dtype=torch.float16, device="cuda") for n, _ in shapes]
        grp.bind(xs, y16)
        grp.forward(m)
        torch.cuda.synchronize()
        for y, ref in zip(y16, refs):
            assert O.normwise_error(y.float().cpu().numpy(), ref) <= TOL_F16
        with pytest.raises(_lib.HlqError):
            grp.forward(m + 1)                  # more rows than the group's scratch holds


def test_large_group_matches_single_launches(L):
    """A group of 78 linears (every CTA walks a dozen segments of several members): the same numbers as
    one launch per member (same tables, same sums; fp32 atomics in another order), three times in a row."""
    lm = linear_mod()
    gen = torch.Generator(device="cuda")
    shapes = [(4096, 4096), (2048, 8192), (1024, 4096)] * 26
    ws, xs, ys, refs = [], [], [], []
    for i, (n, k) in enumerate(shapes):
        gen.manual_seed(1000 + i)
        wq = torch.randint(0, 256, (2, n, k // 8), dtype=torch.uint8, device="cuda", generator=gen)
        sc = (torch.randn((2, n, k // 128), device="cuda", generator=gen) * 0.02).abs().half()
        zz = (torch.randn((n, k // 128), device="cuda", generator=gen) * 0.01).half()
        ws.append(lm.HLQWeight.from_export(F.ExportedLinear(wq, sc, zz, None, 128), device=0))
        xs.append(torch.randn((1, k), device="cuda", generator=gen).half())
        ys.append(torch.zeros((1, n), dtype=torch.float32, device="cuda"))
    wsp = lm.Workspace(lm.workspace_bytes(1, 8192, 4096, 2, 128), torch.device("cuda", 0))
    for w, x in zip(ws, xs):
        refs.append(lm.linear_forward(x, w, wsp, out_dtype=torch.float32).clone())
    group = lm.HLQGroup(ws, max_m=1)
    group.bind(xs, ys)
    for _ in range(3):
        for y in ys:
            y.zero_()
        group.forward(1)
        torch.cuda.synchronize()
        assert group.kernel_status() == 0
        for y, ref in zip(ys, refs):
            assert O.normwise_error(y.cpu().numpy(), ref.cpu().numpy()) <= 1e-6
    # one member against the oracle
    e = ws[1].to_export()
    ref = O.hlq_linear(xs[1].cpu().numpy().astype(np.float32), e.w_quant, e.w_scale, e.w_zero, 128, dtype=np.float32)
    assert O.normwise_error(ys[1].cpu().numpy(), ref) <= 2e-5


def test_group_rejects_mixed_members(L):
    lm = linear_mod()
    a = make(O.synth_linear(64, 512, 2, 128, seed=1), 128)[1]
    b = make(O.synth_linear(64, 512, 3, 128, seed=1), 128)[1]
    c = make(O.synth_linear(64, 512, 2, 128, seed=1), 128, flags=_lib.HLQ_FLAG_FORCE_EXPORT_LAYOUT)[1]
    with pytest.raises(_lib.HlqError):
        lm.HLQGroup([a.weight, b.weight])
    with pytest.raises(_lib.HlqError):
        lm.HLQGroup([a.weight, c.weight])
    grp = lm.HLQGroup([a.weight])
    with pytest.raises(_lib.HlqError):
        grp.forward(1)                          # not bound yet


def test_fused_allreduce_path_with_one_rank(L):
    """The GEMV with the all-reduce in its epilogue, world size 1 (push to itself, wait for
    its own flags, sum one term): same result as the plain GEMV, over several launches so
    that both halves of the double-buffered slots and the launch counter are exercised."""
    from elutq_b200 import tp
    lm = linear_mod()
    for (q, n, k, g, m) in [(2, 4096, 4096, 128, 1), (3, 200, 1536, 64, 3)]:
        d = O.synth_linear(n, k, q, g, m=m, seed=60 + n, bias=True, signed_alpha=True)
        lin, mod = make(d, g, max_batch=m)
        comm = tp.FusedAllReduceComm(max_n=n, max_m=m, device=0)
        x = torch.from_numpy(d["x"]).cuda()
        ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"])
        for _ in range(5):
            y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
            comm.forward(x, mod.weight, mod.workspace, y)
            torch.cuda.synchronize()
            assert mod.workspace.kernel_status() == 0
            assert O.normwise_error(y.cpu().numpy(), ref) <= TOL_F32
        with pytest.raises(_lib.HlqError):
            comm.forward(torch.cat([x, x, x, x, x, x])[: m + 1].contiguous(), mod.weight, mod.workspace,
                         torch.empty((m + 1, n), dtype=torch.float32, device="cuda"))   # more rows than max_m
        comm.free()


def test_argument_errors(L):
    d = O.synth_linear(64, 512, 2, 128, seed=1)
    lin, mod = make(d, 128)
    lm = linear_mod()
    x = torch.from_numpy(d["x"]).cuda()
    y = torch.empty((1, 64), dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    ws = mod.workspace
    h = mod.weight.handle
    assert L.hlq_linear_forward(1, 256, 64, x.data_ptr(), 0, y.data_ptr(), 0, ws.ptr, ws.nbytes, h, st) == 2
    assert L.hlq_linear_forward(1, 512, 64, x.data_ptr(), 0, y.data_ptr(), 0, ws.ptr, 16, h, st) == 3
    assert L.hlq_linear_forward(1, 512, 64, x.data_ptr() + 2, 0, y.data_ptr(), 0, ws.ptr, ws.nbytes, h, st) == 7
    assert L.hlq_linear_forward(1, 512, 64, x.data_ptr(), 2, y.data_ptr(), 0, ws.ptr, ws.nbytes, h, st) == 6
    assert L.hlq_linear_forward(1, 512, 64, None, 0, y.data_ptr(), 0, ws.ptr, ws.nbytes, h, st) == 1
    assert L.hlq_linear_forward(0, 512, 64, None, 0, None, 0, None, 0, h, st) == 0       # empty batch
    out = ctypes.c_void_p()
    bad = L.hlq_weight_from_export(ctypes.byref(out), lin.w_quant.ctypes.data, lin.w_scale.ctypes.data,
                                   lin.w_zero.ctypes.data, None, 512, 64, 100, 2, 0, 0, 1, 0, 0, st)
    assert bad == 2 and not out.value
    with pytest.raises(RuntimeError):
        lm.linear_forward(torch.from_numpy(d["x"]), mod.weight, mod.workspace)     # CPU tensor
    assert L.hlq_kernel_launch_count() > 0
