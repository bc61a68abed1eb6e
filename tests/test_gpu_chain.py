"""The decode chain (all layers of one token as one persistent kernel) against the same decoder
run as one launch per op.  Both use the same seeded weights; the chain fuses gate/up into one
weight with interleaved rows, applies norms, residual adds and the gated SiLU inside its
linears, and hands stages over through counters in device memory."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _decoders(seed, **kw):
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    from elutq_b200.decoder import PRESETS, TPDecoder
    dev = torch.device("cuda", 0)
    a = TPDecoder(PRESETS["tiny"], dev, 0, 1, seed=seed, chain=True, **kw)
    b = TPDecoder(PRESETS["tiny"], dev, 0, 1, seed=seed, chain=False, **kw)
    assert a.use_chain and a.chain is not None and not b.use_chain
    return a, b


@pytest.mark.timeout(120)
def test_chain_step_equals_the_step_of_separate_launches():
    a, b = _decoders(seed=17)
    info = a.chain.info()
    assert info["stages"] == 5 * len(a.layers) and info["linears"] == 4 * len(a.layers)
    assert a.launches_per_step() < b.launches_per_step()
    for step in range(3):                      # the chain's counters and cells are cleared every token
        ta, tb = a.step_eager(7 + step), b.step_eager(7 + step)
        torch.cuda.synchronize()
        assert a.chain.status() == 0 and a.attn.status() == 0
        xa, xb = a.hidden_after_step().float(), b.hidden_after_step().float()
        assert (xa - xb).abs().max() / xb.abs().max() <= 4e-3, step
        la, lb = a.last_logits.float(), b.last_logits.float()
        assert (la - lb).abs().max() / lb.abs().max() <= 1e-2
        top2 = torch.topk(lb.view(-1), 2).values
        if float(top2[0] - top2[1]) > 2e-2 * float(lb.abs().max()):
            assert int(ta.item()) == int(tb.item())
    # The cache rows the steps appended agree: bit-exactly in the first layer; further down an fp16
    # rounding that moved upstream shows (the random model's residual stream has channels of
    # magnitude 1e4, where one fp16 step is 8, and the norm in front of q/k/v divides by them)
    pos = a.pos
    for i, (La, Lb) in enumerate(zip(a.layers, b.layers)):
        va, vb = a.kv_rows(La, "vc", pos, pos + 1).float(), b.kv_rows(Lb, "vc", pos, pos + 1).float()
        if i == 0:
            assert torch.equal(va, vb)
        assert (va - vb).norm() / vb.norm() <= 3e-2


@pytest.mark.timeout(180)
@pytest.mark.parametrize("n_heads,n_kv,ctx,positions", [
    (8, 2, 256, (0, 1, 17, 100, 255)),        # groups of 4 heads, shares of a few positions
    (16, 2, 256, (3, 130, 255)),              # groups of 8 heads
    (16, 8, 4096, (5, 2000, 4095)),           # shares of more than one tile of 128 positions
])
def test_attention_stage_at_many_positions(n_heads, n_kv, ctx, positions):
    """One layer, a random cache, one token at several positions: the chain's attention stage (K rows
    into tensor-core fragments, fp16 weights, splits merged by the o projection) against the kernel
    of the separate launches.  One layer keeps the comparison well conditioned: 2e-3 in relative L2."""
    import dataclasses
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    from elutq_b200.decoder import PRESETS, TPDecoder
    dev = torch.device("cuda", 0)
    cfg = dataclasses.replace(PRESETS["tiny"], layers=1, n_heads=n_heads, n_kv=n_kv, ctx=ctx)
    a = TPDecoder(cfg, dev, 0, 1, seed=5, chain=True)
    b = TPDecoder(cfg, dev, 0, 1, seed=5, chain=False)
    assert a.use_chain and not b.use_chain
    for pos in positions:
        a.position.fill_(pos)
        b.position.fill_(pos)
        a.step_eager(11)
        b.step_eager(11)
        torch.cuda.synchronize()
        assert a.chain.status() == 0 and a.attn.status() == 0 and b.attn.status() == 0
        xa, xb = a.hidden_after_step().float(), b.hidden_after_step().float()
        assert (xa - xb).norm() / xb.norm() <= 2e-3, pos
        for name in ("kc", "vc"):
            assert torch.equal(a.kv_rows(a.layers[0], name, pos, pos + 1), b.kv_rows(b.layers[0], name, pos, pos + 1))


@pytest.mark.timeout(120)
def test_chain_in_a_graph_generates_the_same_tokens():
    a, b = _decoders(seed=23)
    ta = a.generate(3, 6, start_position=100, use_graph=True)
    tb = b.generate(3, 6, start_position=100, use_graph=False)
    assert a.chain.status() == 0
    assert ta == tb and len(ta) == 6
    for La, Lb in zip(a.layers, b.layers):
        ka, kb = a.kv_rows(La, "kc", 100, 106).float(), b.kv_rows(Lb, "kc", 100, 106).float()
        assert (ka - kb).norm() / kb.norm() <= 3e-2
        assert torch.equal(a.kv_rows(La, "kc", 106, 256), b.kv_rows(Lb, "kc", 106, 256))


@pytest.mark.timeout(120)
def test_chain_request_falls_back_where_the_kernel_does_not_apply(tmp_path):
    """The golden directory written by the reference's quantizer driver has heads of 64
    channels; the chain runs 128-channel heads only, so asking for it must quietly give the
    path of separate launches, with the reference model's logits."""
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    from elutq_b200.decoder import TPDecoder
    d = np.load(os.path.join(ROOT, "tests", "golden", "model_tiny_llama.npz"))
    for key in d.files:
        if key.startswith("file:"):
            p = tmp_path / key[5:]
            p.parent.mkdir(parents=True, exist_ok=True)
            p.write_bytes(d[key].tobytes())
    dec = TPDecoder.from_export(str(tmp_path), n_heads=int(d["n_heads"]), n_kv=int(d["n_kv"]),
                                device=torch.device("cuda", 0), ctx=64, rope_theta=float(d["rope_theta"]), chain=True)
    assert not dec.use_chain and dec.chain is None
    dec.position.fill_(0)
    dec.step_eager(int(d["tokens"][0]))
    torch.cuda.synchronize()
    ref = d["logits"][0].astype(np.float64)
    got = dec.last_logits.float().cpu().numpy()[0].astype(np.float64)
    assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-2


@pytest.mark.timeout(180)
def test_chain_against_the_decoder_oracle(tmp_path):
    """A small exported model (heads of 128 channels) through the decode chain, token by token, against
    the CPU decoder oracle (the reference model's op order over the float64 oracles): logits of six
    consecutive positions to 1e-2 normwise, the final hidden state to 2e-2 in relative L2."""
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from test_model_io import tiny_model
    from elutq_b200.decoder import TPDecoder
    from oracle.decoder_oracle import OracleDecoder
    m = tiny_model(layers=2, hidden=256, ffn=512, heads=4, kv=2, dhead=128, vocab=320, quant_head=True, seed=11)
    dec = TPDecoder.from_export(m, n_heads=4, n_kv=2, device=torch.device("cuda", 0), ctx=64, rope_theta=1e4, chain=True)
    assert dec.use_chain
    ora = OracleDecoder(m, 4, 2, 1e4, 1e-5, ctx=64)
    tokens = [5, 17, 300, 2, 41, 9]
    for pos, tok in enumerate(tokens):
        dec.position.fill_(pos)
        dec.step_eager(tok)
        torch.cuda.synchronize()
        assert dec.chain.status() == 0 and dec.attn.status() == 0
        want, hidden = ora.step(tok, pos)
        got = dec.last_logits.float().cpu().numpy()[0].astype(np.float64)
        assert np.abs(got - want).max() / np.abs(want).max() <= 1e-2, pos


@pytest.mark.timeout(120)
@pytest.mark.parametrize("q,g,hidden,ffn,n_out", [(2, 128, 1024, 640, 768), (3, 64, 512, 1536, 520)])
def test_down_takes_the_gate_up_sums_unfinished(q, g, hidden, ffn, n_out):
    """A chain of two linears, fused gate/up (with a bias, gated-SiLU output) and a down projection
    that takes exactly that output: the kernel skips gate/up's completion pass, down's consumers
    finish the sums themselves (ffn = 640: the second slice of down holds 128 channels) and
    down's completion pass clears them.  The intermediate output and the result against NumPy with
    the kernel's roundings, three tokens in a row (the sums are zero again each time)."""
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    from elutq_b200 import _lib, format as F
    from elutq_b200.chain import DecodeChain, interleave_rows
    from elutq_b200.linear import HLQWeight
    from oracle import hlq_oracle as O
    dev = torch.device("cuda", 0)
    dg = O.synth_linear(ffn, hidden, q, g, m=1, seed=51, bias=True, signed_alpha=True)
    du = O.synth_linear(ffn, hidden, q, g, m=1, seed=52, bias=True, signed_alpha=True)
    dd = O.synth_linear(n_out, ffn, q, g, m=1, seed=53, bias=True, signed_alpha=True)
    fused = F.ExportedLinear(interleave_rows(dg["w_quant"], du["w_quant"], 1), interleave_rows(dg["w_scale"], du["w_scale"], 1),
                             interleave_rows(dg["w_zero"], du["w_zero"], 0), interleave_rows(dg["bias"], du["bias"], 0), g)
    wgu = HLQWeight.from_export(fused, device=0)
    wd = HLQWeight.from_export(F.ExportedLinear(dd["w_quant"], dd["w_scale"], dd["w_zero"], dd["bias"], g), device=0)
    x = torch.zeros(hidden, dtype=torch.float16, device=dev)
    h = torch.zeros(ffn, dtype=torch.float16, device=dev)
    y = torch.zeros(n_out, dtype=torch.float16, device=dev)
    chain = DecodeChain(dev, 0)
    chain.add_linears([DecodeChain.linear(wgu, x, h, out_kind=_lib.HLQ_CHAIN_OUT_GATED_SILU)])
    chain.add_linears([DecodeChain.linear(wd, h, y)])
    chain.finish()
    rng = np.random.default_rng(5)
    for step in range(3):
        xs = rng.standard_normal(hidden).astype(np.float16)
        x.copy_(torch.from_numpy(xs))
        h.zero_()
        y.zero_()
        chain.forward()
        torch.cuda.synchronize()
        assert chain.status() == 0
        gate = O.hlq_linear(xs[None], dg["w_quant"], dg["w_scale"], dg["w_zero"], g, dg["bias"])[0].astype(np.float16).astype(np.float32)
        up = O.hlq_linear(xs[None], du["w_quant"], du["w_scale"], du["w_zero"], g, du["bias"])[0].astype(np.float16).astype(np.float32)
        href = (up * (gate / (1.0 + np.exp(-gate)))).astype(np.float16)
        hk = h.cpu().numpy()
        assert O.normwise_error(hk.astype(np.float64), href.astype(np.float64)) <= 2e-3, step
        yref = O.hlq_linear(hk[None], dd["w_quant"], dd["w_scale"], dd["w_zero"], g, dd["bias"])[0]
        assert O.normwise_error(y.float().cpu().numpy().astype(np.float64), yref) <= 1e-3, step
