"""Parity of the decoder glue kernels (RMSNorm, RoPE + KV append + attention, gated SiLU,
argmax) with the numpy restatement of the reference's ops (oracle/glue_oracle.py).

Tolerances: fp16 outputs of fp32 arithmetic against float64 arithmetic rounded to fp16 may
differ by one fp16 ulp where the exact value sits near a rounding boundary, so element-wise
ops are compared with rtol 2e-3 (two ulps); the attention output (a softmax-weighted mean of
fp16 values, fp32 accumulation) with a normwise 1e-3 gate.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from elutq_b200 import _lib, glue  # noqa: E402
from oracle import glue_oracle as GO  # noqa: E402

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def t16(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def close16(got, ref, rtol=2e-3, atol=2e-4):
    g, r = got.astype(np.float64), ref.astype(np.float64)
    assert g.shape == r.shape
    bad = np.abs(g - r) > atol + rtol * np.abs(r)
    assert not bad.any(), f"{bad.sum()} of {bad.size} differ, worst {np.abs(g - r).max()}"


@pytest.mark.parametrize("rows,n", [(1, 4096), (1, 8192), (3, 1024), (1, 8), (2, 14336)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_rmsnorm_matches_reference_math(rows, n, with_residual):
    rng = np.random.default_rng(rows * 131 + n + with_residual)
    x = rng.standard_normal((rows, n)).astype(np.float16)
    gamma = (1 + 0.1 * rng.standard_normal(n)).astype(np.float16)
    res = rng.standard_normal((rows, n)).astype(np.float16) if with_residual else None
    ref_out, ref_res = GO.rmsnorm(x, gamma, 1e-5, res)
    if with_residual:
        out, res_out = glue.rmsnorm(t16(x), t16(gamma), 1e-5, residual=t16(res))
        # the sum of two fp16 values rounded once: exact in fp32, so bit-identical
        assert np.array_equal(res_out.cpu().numpy().view(np.uint16), ref_res.view(np.uint16))
    else:
        out = glue.rmsnorm(t16(x), t16(gamma), 1e-5)
    close16(out.cpu().numpy(), ref_out)


def test_rmsnorm_in_place_as_the_reference_calls_it():
    """llama.cpp:204-215 passes output == vals and res_output == residual."""
    rng = np.random.default_rng(5)
    n = 4096
    x = rng.standard_normal((1, n)).astype(np.float16)
    res = rng.standard_normal((1, n)).astype(np.float16)
    gamma = (1 + 0.1 * rng.standard_normal(n)).astype(np.float16)
    ref_out, ref_res = GO.rmsnorm(x, gamma, 1e-5, res)
    dx, dr = t16(x), t16(res)
    glue.rmsnorm(dx, t16(gamma), 1e-5, out=dx, residual=dr, res_out=dr)
    assert np.array_equal(dr.cpu().numpy().view(np.uint16), ref_res.view(np.uint16))
    close16(dx.cpu().numpy(), ref_out)


def test_rmsnorm_rejects_bad_shapes():
    x = torch.zeros((1, 12), dtype=torch.float16, device=DEV)
    g = torch.ones(12, dtype=torch.float16, device=DEV)
    with pytest.raises(_lib.HlqError):
        glue.rmsnorm(x, g, 1e-5)


@pytest.mark.parametrize("n", [8, 14336, 28672 // 8, 1000 * 8])
def test_gated_silu(n):
    rng = np.random.default_rng(n)
    g = (3 * rng.standard_normal((1, n))).astype(np.float16)
    u = rng.standard_normal((1, n)).astype(np.float16)
    out = glue.gated_silu(t16(g), t16(u))
    close16(out.cpu().numpy(), GO.gated_silu(g, u))


@pytest.mark.parametrize("n,dtype", [(128256, np.float32), (16032, np.float16), (5, np.float32), (1025, np.float16)])
def test_argmax_first_largest(n, dtype):
    rng = np.random.default_rng(n)
    v = rng.standard_normal(n).astype(dtype)
    v[n // 3] = v.max() + 1          # a clear winner ...
    idx, val = glue.argmax(t16(v))
    assert int(idx.item()) == GO.argmax_first(v) == n // 3
    assert float(val.item()) == float(v[n // 3])
    v[n // 3 + 1:] = np.minimum(v[n // 3 + 1:], v[n // 3])
    if n > 4:
        v[-1] = v[n // 3]            # ... and a tie later on: the first one wins
    idx, _ = glue.argmax(t16(v))
    assert int(idx.item()) == GO.argmax_first(v) == n // 3


ATT_CASES = [
    # head_q, head_kv, dhead, max_ctx, position
    (32, 8, 128, 2048, 2047),
    (32, 8, 128, 2048, 0),            # first token: attends to itself only
    (8, 1, 128, 2048, 1234),          # one kv head per rank, group of 8 (70B shapes over 8 ranks)
    (8, 8, 64, 300, 129),             # no grouping, 64-wide heads, ragged cache
    (6, 2, 128, 512, 127),            # group of 3, tile boundary
    (6, 2, 128, 512, 128),
    (4, 4, 128, 64, 5),               # cache shorter than one tile
]


@pytest.mark.parametrize("head_major", [False, True])
@pytest.mark.parametrize("hq,hkv,d,ctx,pos", ATT_CASES)
def test_rope_cache_attention(hq, hkv, d, ctx, pos, head_major):
    rng = np.random.default_rng(hq * 7 + hkv * 3 + d + pos)
    base = 500000.0
    q = rng.standard_normal((hq, d)).astype(np.float16)
    k = rng.standard_normal((hkv, d)).astype(np.float16)
    v = rng.standard_normal((hkv, d)).astype(np.float16)
    kc = rng.standard_normal((ctx, hkv, d)).astype(np.float16)
    vc = rng.standard_normal((ctx, hkv, d)).astype(np.float16)
    # oracle: rope, append, attend
    kc_ref, vc_ref = kc.copy(), vc.copy()
    GO.cache_append(kc_ref, vc_ref, GO.rope(k, pos, base), v, pos)
    ref = GO.attention_single(GO.rope(q, pos, base), kc_ref, vc_ref, pos + 1, d ** -0.5)

    att = glue.DecodeAttention(hq, hkv, d, ctx, base, DEV, head_major=head_major)
    # the reference's caches are [position][head][dhead]; head-major keeps a head's positions together
    lay = (lambda c: np.ascontiguousarray(c.transpose(1, 0, 2))) if head_major else (lambda c: c)
    unlay = (lambda c: c.transpose(1, 0, 2)) if head_major else (lambda c: c)
    dkc, dvc = t16(lay(kc)), t16(lay(vc))
    position = torch.tensor([pos], dtype=torch.int32, device=DEV)
    out = att.forward(t16(q), t16(k), t16(v), dkc, dvc, position)
    torch.cuda.synchronize()
    assert att.status() == 0
    got = out.cpu().numpy().astype(np.float64)
    err = np.abs(got - ref.astype(np.float64)).max() / np.abs(ref.astype(np.float64)).max()
    assert err <= 1e-3, err
    # the cache: v copied bit-exactly, roped k within an fp16 ulp (fp32 sin/cos of a large
    # angle against float64), everything else untouched
    gk, gv = unlay(dkc.cpu().numpy()), unlay(dvc.cpu().numpy())
    assert np.array_equal(gv.view(np.uint16), vc_ref.view(np.uint16))
    close16(gk[pos], kc_ref[pos], rtol=4e-3, atol=2e-3)
    mask = np.ones(ctx, dtype=bool)
    mask[pos] = False
    assert np.array_equal(gk[mask].view(np.uint16), kc[mask].view(np.uint16))
    # a second launch on the same workspace (counters re-zeroed by the kernel) agrees
    out2 = att.forward(t16(q), t16(k), t16(v), dkc, dvc, position)
    assert torch.equal(out, out2)


def test_attention_position_comes_from_device_memory_and_is_checked():
    hq, hkv, d, ctx = 4, 2, 128, 128
    att = glue.DecodeAttention(hq, hkv, d, ctx, 10000.0, DEV)
    z = lambda *s: torch.zeros(s, dtype=torch.float16, device=DEV)  # noqa: E731
    kc, vc = z(ctx, hkv, d), z(ctx, hkv, d)
    position = torch.tensor([ctx], dtype=torch.int32, device=DEV)      # one past the cache
    att.forward(z(hq, d), z(hkv, d), z(hkv, d), kc, vc, position)
    torch.cuda.synchronize()
    assert att.status() == 3
    att.ws.zero_()
    with pytest.raises(_lib.HlqError):                                   # group of 16 query heads
        glue.DecodeAttention(16, 1, 128, 64, 1e4, DEV).forward(z(16, d), z(1, d), z(1, d), z(64, 1, d), z(64, 1, d),
                                                                position)


# ---- input transforms fused into the LUT GEMV's table build ---------------------------------

def _linear_case(n, k, q=2, g=128, seed=0):
    from elutq_b200 import format as F, linear as lm
    from oracle import hlq_oracle as O
    d = O.synth_linear(n, k, q, g, m=1, seed=seed)
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], None, g)
    w = lm.HLQWeight.from_export(lin, device=0)
    ws = lm.Workspace(lm.workspace_bytes(1, k, n, q, g), torch.device(DEV))
    return d, w, ws, lm


@pytest.mark.parametrize("n,k", [(256, 1024), (96, 14336), (1024, 62 * 128)])
def test_gated_silu_inside_the_gemv_equals_the_two_kernels(n, k):
    d, w, ws, lm = _linear_case(n, k, seed=n + k)
    rng = np.random.default_rng(n)
    gate = t16((2 * rng.standard_normal((1, k))).astype(np.float16))
    up = t16(rng.standard_normal((1, k)).astype(np.float16))
    ref = lm.linear_forward(glue.gated_silu(gate, up), w, ws, out_dtype=torch.float32)
    out = torch.empty((1, n), dtype=torch.float32, device=DEV)
    lm.linear_forward_op(gate, w, ws, out, lm.input_op(_lib.HLQ_INPUT_GATED_SILU, second=up))
    torch.cuda.synchronize()
    assert ws.kernel_status() == 0
    # the tables see the same fp16 activations: equal up to the order of the slice sums
    err = (out - ref).abs().max() / ref.abs().max()
    assert err <= 1e-6, float(err)


@pytest.mark.parametrize("n,k,with_res", [(256, 4096, True), (1024, 8192, True), (320, 1024, False), (64, 640, True)])
def test_add_rmsnorm_inside_the_gemv_equals_the_two_kernels(n, k, with_res):
    d, w, ws, lm = _linear_case(n, k, seed=n + k + 1)
    rng = np.random.default_rng(k)
    x = t16(rng.standard_normal((1, k)).astype(np.float16))
    res = t16(rng.standard_normal((1, k)).astype(np.float16)) if with_res else None
    gamma = t16((1 + 0.1 * rng.standard_normal(k)).astype(np.float16))
    if with_res:
        xn, r_ref = glue.rmsnorm(x, gamma, 1e-5, residual=res)
    else:
        xn, r_ref = glue.rmsnorm(x, gamma, 1e-5), None
    ref = lm.linear_forward(xn, w, ws, out_dtype=torch.float32)
    out = torch.empty((1, n), dtype=torch.float32, device=DEV)
    r_out = torch.zeros((1, k), dtype=torch.float16, device=DEV) if with_res else None
    op = lm.input_op(_lib.HLQ_INPUT_ADD_RMSNORM, second=res, gamma=gamma, res_out=r_out, eps=1e-5)
    lm.linear_forward_op(x, w, ws, out, op)
    torch.cuda.synchronize()
    assert ws.kernel_status() == 0
    if with_res:
        assert torch.equal(r_out, r_ref)          # the residual stream: bit-exact
    # 1/rms is summed in another order than in the stand-alone kernel: a few normalized
    # activations may round to the neighbouring fp16 value
    err = (out - ref).abs().max() / ref.abs().max()
    assert err <= 5e-4, float(err)
    # and against the oracle of the whole chain
    from oracle import hlq_oracle as O
    xo, _ = GO.rmsnorm(x.cpu().numpy(), gamma.cpu().numpy(), 1e-5, res.cpu().numpy() if with_res else None)
    yo = O.hlq_linear(xo, d["w_quant"], d["w_scale"], d["w_zero"], 128, None)
    assert O.normwise_error(out.cpu().numpy(), yo) <= 1e-3


def test_group_members_with_input_transforms():
    from elutq_b200 import linear as lm
    k = 2048
    d1, w1, ws, _ = _linear_case(512, k, seed=5)
    d2, w2, _, _ = _linear_case(128, k, seed=6)
    rng = np.random.default_rng(3)
    x = t16(rng.standard_normal((1, k)).astype(np.float16))
    res = t16(rng.standard_normal((1, k)).astype(np.float16))
    gamma = t16((1 + 0.1 * rng.standard_normal(k)).astype(np.float16))
    xn, r_ref = glue.rmsnorm(x, gamma, 1e-5, residual=res)
    ws2 = lm.Workspace(lm.workspace_bytes(1, k, 512, 2, 128), torch.device(DEV))
    refs = [lm.linear_forward(xn, w, ws2) for w in (w1, w2)]
    ys = [torch.empty((1, 512), dtype=torch.float16, device=DEV), torch.empty((1, 128), dtype=torch.float16, device=DEV)]
    r_out = torch.zeros_like(x)
    grp = lm.HLQGroup([w1, w2], max_m=1)
    grp.bind([x, x], ys, ops=[lm.input_op(_lib.HLQ_INPUT_ADD_RMSNORM, second=res, gamma=gamma, res_out=r_out, eps=1e-5),
                              lm.input_op(_lib.HLQ_INPUT_ADD_RMSNORM, second=res, gamma=gamma, eps=1e-5)])
    grp.forward(1)
    torch.cuda.synchronize()
    assert grp.kernel_status() == 0
    assert torch.equal(r_out, r_ref)
    for y, r in zip(ys, refs):
        assert (y.float() - r.float()).abs().max() / r.float().abs().max() <= 2e-3


def test_input_transform_argument_errors():
    d, w, ws, lm = _linear_case(64, 512)
    x = torch.zeros((1, 512), dtype=torch.float16, device=DEV)
    out = torch.empty((1, 64), dtype=torch.float16, device=DEV)
    with pytest.raises(_lib.HlqError):          # gated SiLU without its second input
        lm.linear_forward_op(x, w, ws, out, lm.input_op(_lib.HLQ_INPUT_GATED_SILU))
    with pytest.raises(_lib.HlqError):          # norm without gamma
        lm.linear_forward_op(x, w, ws, out, lm.input_op(_lib.HLQ_INPUT_ADD_RMSNORM))
    with pytest.raises(_lib.HlqError):          # res_out may not alias the input
        lm.linear_forward_op(x, w, ws, out, lm.input_op(_lib.HLQ_INPUT_ADD_RMSNORM, gamma=x, res_out=x))
    with pytest.raises(_lib.HlqError):          # bf16 activations: not with a transform
        lm.linear_forward_op(x.bfloat16(), w, ws, out, lm.input_op(_lib.HLQ_INPUT_GATED_SILU, second=x))

