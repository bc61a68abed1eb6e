"""Whole-model export directories (the reference's llama.py --export layout): write/read round
trips on the CPU, and on the GPU a decoder built from a directory against one built from the
same arrays in memory."""
import os

import numpy as np
import pytest

from elutq_b200 import format as F
from elutq_b200 import model_io as MIO
from oracle import hlq_oracle as O


def tiny_model(layers=2, hidden=256, ffn=512, heads=2, kv=1, dhead=128, vocab=320, quant_head=True, tied=False, seed=0):
    rng = np.random.default_rng(seed)

    def lin(n, k, q=2, g=128, s=0):
        d = O.synth_linear(n, k, q, g, m=1, seed=seed * 100 + s)
        return F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], None, g)

    ls = []
    for li in range(layers):
        linears = {"q": lin(heads * dhead, hidden, s=li * 8), "k": lin(kv * dhead, hidden, s=li * 8 + 1),
                   "v": lin(kv * dhead, hidden, s=li * 8 + 2), "o": lin(hidden, heads * dhead, s=li * 8 + 3),
                   "gate": lin(ffn, hidden, s=li * 8 + 4), "up": lin(ffn, hidden, s=li * 8 + 5),
                   "down": lin(hidden, ffn, s=li * 8 + 6)}
        ls.append(MIO.LayerExport(linears, (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float16),
                                  (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float16)))
    emb = (0.5 * rng.standard_normal((vocab, hidden))).astype(np.float16)
    if tied:
        head = emb
    elif quant_head:
        head = lin(vocab, hidden, q=4, s=999)
    else:
        head = (0.02 * rng.standard_normal((vocab, hidden))).astype(np.float16)
    return MIO.ModelExport(emb, (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float16), head, ls, tied)


def same_linear(a, b):
    return (np.array_equal(a.w_quant, b.w_quant) and np.array_equal(a.w_scale.view(np.uint16), b.w_scale.view(np.uint16))
            and np.array_equal(a.w_zero.view(np.uint16), b.w_zero.view(np.uint16)) and a.groupsize == b.groupsize)


@pytest.mark.parametrize("quant_head,tied", [(True, False), (False, False), (False, True)])
def test_model_directory_round_trip(tmp_path, quant_head, tied):
    m = tiny_model(quant_head=quant_head, tied=tied)
    MIO.write_model_export(str(tmp_path), m)
    # the reference exporter's names (llama.py:296-343, llama.cpp:66-111)
    assert os.path.exists(tmp_path / "final_rmsnorm_weight.bin")
    assert os.path.exists(tmp_path / "0" / "input_layernorm_weight.bin")
    assert os.path.exists(tmp_path / "1" / "mlp.down_proj" / "w_quant.bin")
    assert os.path.exists(tmp_path / ("shared_embed_lm_head.bin" if tied else "embed_tokens.bin"))
    assert os.path.isdir(tmp_path / "lm_head" / "lm_head") == quant_head
    r = MIO.read_model_export(str(tmp_path))
    assert len(r.layers) == 2 and r.hidden == 256 and r.vocab == 320 and r.ffn == 512 and r.tied == tied
    assert np.array_equal(r.embed.view(np.uint16), m.embed.view(np.uint16))
    assert np.array_equal(r.final_norm.view(np.uint16), m.final_norm.view(np.uint16))
    if quant_head:
        assert same_linear(r.lm_head, m.lm_head)
    else:
        assert np.array_equal(r.lm_head.view(np.uint16), (m.embed if tied else m.lm_head).view(np.uint16))
    for a, b in zip(r.layers, m.layers):
        assert np.array_equal(a.ln1.view(np.uint16), b.ln1.view(np.uint16))
        assert np.array_equal(a.ln2.view(np.uint16), b.ln2.view(np.uint16))
        for key in MIO.PROJ_DIRS:
            assert same_linear(a.linears[key], b.linears[key])


def test_model_directory_errors(tmp_path):
    with pytest.raises(RuntimeError):                       # nothing there
        MIO.read_model_export(str(tmp_path))
    m = tiny_model(layers=1)
    MIO.write_model_export(str(tmp_path), m)
    os.remove(tmp_path / "0" / "post_attention_layernorm_weight.bin")
    with pytest.raises(RuntimeError):
        MIO.read_model_export(str(tmp_path))
    MIO.write_model_export(str(tmp_path), m)
    (tmp_path / "0" / "input_layernorm_weight.bin").write_bytes(b"\0" * 10)     # wrong length
    with pytest.raises(ValueError):
        MIO.read_model_export(str(tmp_path))


@pytest.mark.gpu
def test_decoder_from_a_model_directory(tmp_path):
    torch = pytest.importorskip("torch")
    from elutq_b200.decoder import TPDecoder
    m = tiny_model(layers=2, quant_head=True, seed=3)
    MIO.write_model_export(str(tmp_path), m)
    dev = torch.device("cuda", 0)
    a = TPDecoder.from_export(str(tmp_path), n_heads=2, n_kv=1, device=dev, ctx=64, rope_theta=1e4)
    b = TPDecoder.from_export(m, n_heads=2, n_kv=1, device=dev, ctx=64, rope_theta=1e4)
    assert a.cfg.hidden == 256 and a.cfg.layers == 2 and a.cfg.vocab == 320 and a.cfg.head_dim == 128
    ta = a.generate(5, 4, start_position=0)
    tb = b.generate(5, 4, start_position=0, use_graph=False)
    assert ta == tb
    # first layer's q projection of the first token against the oracle, through the whole chain
    # embedding -> RMSNorm -> q_proj
    from oracle import glue_oracle as GO
    x0 = m.embed[5:6]
    xn, _ = GO.rmsnorm(x0, m.layers[0].ln1, 1e-5)
    lin = m.layers[0].linears["q"]
    want = O.hlq_linear(xn, lin.w_quant, lin.w_scale, lin.w_zero, lin.groupsize, None)
    c = TPDecoder.from_export(m, n_heads=2, n_kv=1, device=dev, ctx=64, rope_theta=1e4)
    c.position.fill_(0)
    c.step_eager(5)
    torch.cuda.synchronize()
    got = c.layers[0]["q_o"].float().cpu().numpy()
    assert O.normwise_error(got, want) <= 2e-3
    with pytest.raises(ValueError):
        TPDecoder.from_export(m, n_heads=3, n_kv=1, device=dev)
