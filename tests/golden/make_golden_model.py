"""Generates tests/golden/model_tiny_llama.npz: a whole-model export directory written by the
REFERENCE's own quantizer driver, plus the logits of the model it evaluates.

    python tests/golden/make_golden_model.py <path of the ELUTQ checkout>      (needs transformers; CPU only)

What runs is the reference's code, unmodified, imported from the checkout's GPTQ directory:
  export_llama_weights      GPTQ/llama.py:286-343   embeddings, norms (fp16 .bin files)
  llama_sequential          GPTQ/llama.py:31-180    per layer: HLQ.add_batch (Hessian) and
                                                    HLQ.fasterquant(output_dir=...) for every linear,
                                                    then the lm_head, forced to w4g128 (HLQ.py:76-78)
on a 2-layer random-init LlamaForCausalLM (hidden 128, ffn 256, 2 heads / 1 kv head of 64,
vocabulary 256) with w2g128 and the alternating fit.  After the driver has run, the model's
linears hold the fake-quantized weights (HLQ.py:173) - the model whose perplexity the reference
reports - so its logits on a fixed token sequence are the reference's own answer for the
exported directory.  Stored: every file of the directory (relative path -> bytes), the token
ids, the logits [T, vocab] and the final normed hidden states [T, hidden] in float32.

Two shims adapt this container, neither touches the reference's arithmetic: `termcolor`
(imported by the reference's logger, not installed here) is replaced by a stub, and
torch.cuda.synchronize (called by fasterquant for its timing print) by a no-op, as there is
no CUDA device here.
"""
import argparse
import io
import logging
import os
import shutil
import sys
import tempfile
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main(reference_root):
    sys.modules.setdefault("termcolor", types.SimpleNamespace(colored=lambda s, *a, **k: s))
    sys.path.insert(0, os.path.join(reference_root, "GPTQ"))
    import torch
    torch.cuda.synchronize = lambda *a, **k: None
    import llama as ref_llama
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                      num_key_value_heads=1, head_dim=64, vocab_size=256, max_position_embeddings=256,
                      rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False, attention_bias=False)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).half().float()        # every parameter representable in fp16
    with torch.no_grad():                               # norm weights away from exactly 1
        for name, p in model.named_parameters():
            if "norm" in name:
                p.copy_((1 + 0.1 * torch.randn_like(p)).half().float())
    model.seqlen = 32
    out = tempfile.mkdtemp(prefix="hlq_golden_model_")
    args = argparse.Namespace(nsamples=4, true_sequential=False, wbits=2, groupsize=128, export=out, actorder=False,
                              percdamp=0.01, iters=10, lr=1e-3, alternating_optimization=True, skip_lmhead=False)
    ref_llama.args = args                               # the driver reads its flags from a module global
    g = torch.Generator().manual_seed(1)
    calib = [(torch.randint(0, cfg.vocab_size, (1, model.seqlen), generator=g), None) for _ in range(args.nsamples)]
    ref_llama.export_llama_weights(model, args, cfg)
    ref_llama.llama_sequential(model, calib, torch.device("cpu"), logging.getLogger("make_golden_model"))
    cfg.to_json_file(os.path.join(out, "config.json"))

    tokens = torch.randint(0, cfg.vocab_size, (1, 12), generator=g)
    model.eval()
    with torch.no_grad():
        logits = model(tokens).logits[0].float().numpy()
        hidden = model.model(tokens).last_hidden_state[0].float().numpy()      # after the final norm
    files = {}
    for root, _, names in os.walk(out):
        for n in names:
            p = os.path.join(root, n)
            files["file:" + os.path.relpath(p, out)] = np.frombuffer(open(p, "rb").read(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "model_tiny_llama.npz"), tokens=tokens[0].numpy().astype(np.int64),
                        logits=logits.astype(np.float32), hidden=hidden.astype(np.float32),
                        n_heads=np.int64(cfg.num_attention_heads), n_kv=np.int64(cfg.num_key_value_heads),
                        head_dim=np.int64(cfg.head_dim), rope_theta=np.float64(cfg.rope_parameters["rope_theta"]),
                        eps=np.float64(cfg.rms_norm_eps), **files)
    shutil.rmtree(out, ignore_errors=True)
    print("wrote model_tiny_llama.npz:", len(files), "files,", os.path.getsize(os.path.join(HERE, "model_tiny_llama.npz")), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
