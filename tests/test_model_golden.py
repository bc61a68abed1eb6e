"""A whole-model directory written by the reference's own quantizer driver
(tests/golden/make_golden_model.py runs GPTQ/llama.py's export_llama_weights and
llama_sequential with HLQ.fasterquant(output_dir=...) on a tiny random Llama) against this
package's reader/writer, the CPU decoder oracle, and - on a GPU - the decoder built from it.
The expected logits are those of the fake-quantized model the reference itself evaluates."""
import json
import os

import numpy as np
import pytest

from elutq_b200 import format as F
from elutq_b200 import model_io as MIO

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "model_tiny_llama.npz")


@pytest.fixture(scope="module")
def golden(tmp_path_factory):
    d = np.load(GOLDEN)
    root = tmp_path_factory.mktemp("ref_model")
    files = {}
    for key in d.files:
        if key.startswith("file:"):
            rel = key[5:]
            p = root / rel
            p.parent.mkdir(parents=True, exist_ok=True)
            p.write_bytes(d[key].tobytes())
            files[rel] = d[key].tobytes()
    meta = {k: d[k] for k in ("tokens", "logits", "hidden", "n_heads", "n_kv", "head_dim", "rope_theta", "eps")}
    return str(root), files, meta


def test_reader_takes_the_reference_written_directory(golden, tmp_path):
    root, files, meta = golden
    m = MIO.read_model_export(root)
    assert len(m.layers) == 2 and m.hidden == 128 and m.vocab == 256 and m.ffn == 256 and not m.tied
    # lm_head: the quantized directory wins over lm_head.bin, forced to w4g128 (HLQ.py:76-78)
    assert isinstance(m.lm_head, F.ExportedLinear) and m.lm_head.bits == 4 and m.lm_head.groupsize == 128
    for layer in m.layers:
        for key, lin in layer.linears.items():
            assert lin.bits == 2 and lin.groupsize == 128, key       # groupsize derived: the exporter omits it
    # writing it back gives the reference's bytes, file by file
    MIO.write_model_export(str(tmp_path), m)
    for rel, blob in files.items():
        if rel in ("config.json", "lm_head.bin"):                    # not ours to write (HF config; fp16 lm_head
            continue                                                 # shadowed by the quantized one)
        mine = (tmp_path / rel).read_bytes()
        if rel.endswith(".json"):
            a, b = json.loads(mine), json.loads(blob)
            a.pop("groupsize", None)
            assert a == b, rel
        else:
            assert mine == blob, rel


def test_cpu_decoder_oracle_matches_the_reference_models_logits(golden):
    """Pins the glue oracle (RMSNorm, RoPE pairing, attention scaling, SiLU, residual order) and
    the value oracle together against the logits of the reference's fake-quantized model."""
    from oracle.decoder_oracle import OracleDecoder
    root, _, meta = golden
    dec = OracleDecoder(MIO.read_model_export(root), meta["n_heads"], meta["n_kv"], meta["rope_theta"], meta["eps"])
    for pos, tok in enumerate(meta["tokens"]):
        logits, hidden = dec.step(int(tok), pos)
        ref_l, ref_h = meta["logits"][pos].astype(np.float64), meta["hidden"][pos].astype(np.float64)
        assert np.abs(hidden.astype(np.float64) - ref_h).max() / np.abs(ref_h).max() <= 6e-3, pos
        assert np.abs(logits - ref_l).max() / np.abs(ref_l).max() <= 6e-3, pos
        assert int(np.argmax(logits)) == int(np.argmax(ref_l)), pos


@pytest.mark.gpu
def test_gpu_decoder_on_the_reference_written_directory(golden):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    from elutq_b200.decoder import TPDecoder
    root, _, meta = golden
    dev = torch.device("cuda", 0)
    dec = TPDecoder.from_export(root, n_heads=int(meta["n_heads"]), n_kv=int(meta["n_kv"]), device=dev, ctx=64,
                                rope_theta=float(meta["rope_theta"]))
    for pos, tok in enumerate(meta["tokens"]):
        dec.position.fill_(pos)
        nxt = dec.step_eager(int(tok))
        torch.cuda.synchronize()
        logits = dec.last_logits.float().cpu().numpy()[0].astype(np.float64)
        ref_l = meta["logits"][pos].astype(np.float64)
        assert np.abs(logits - ref_l).max() / np.abs(ref_l).max() <= 1e-2, pos
        if np.sort(ref_l)[-1] - np.sort(ref_l)[-2] > 2e-2 * np.abs(ref_l).max():
            assert int(nxt.item()) == int(np.argmax(ref_l)), pos
    assert dec.ws.kernel_status() == 0 and dec.attn.status() == 0
