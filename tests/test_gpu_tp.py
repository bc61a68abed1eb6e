"""Tensor-parallel decode on two GPUs against the same decoder on one GPU (NCCL).  Skipped
where fewer than two GPUs are visible; the sharding logic itself is covered on CPU ranks in
test_tp_gloo.py and on one GPU in test_gpu_gemv.py."""
import os
import sys
import tempfile

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp  # noqa: E402

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, init_file, out_dir, chain=False):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    from elutq_b200.decoder import PRESETS, TPDecoder
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world, device_id=dev)
    try:
        dec = TPDecoder(PRESETS["tiny"], dev, rank, world, seed=3, chain=chain)
        assert dec.use_chain == chain
        for tok in (5, 9, 2):               # several tokens: the rank sums' tags and slot sets alternate
            dec.step_eager(tok)
        torch.cuda.synchronize()
        if chain:
            assert dec.chain.status() == 0 and dec.chain.info()["rank_sums"] == 2 * len(dec.layers)
        if rank == 0:
            np.save(os.path.join(out_dir, "x_tp.npy"), dec.hidden_after_step().float().cpu().numpy())
            np.save(os.path.join(out_dir, "tok_tp.npy"), dec.next_token.cpu().numpy())
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(150)
def test_two_gpu_decode_matches_one_gpu():
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, ROOT)
    from elutq_b200.decoder import PRESETS, TPDecoder
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker, args=(2, os.path.join(tmp, "init"), tmp), nprocs=2, join=True)
        x_tp = np.load(os.path.join(tmp, "x_tp.npy"))
        tok_tp = np.load(os.path.join(tmp, "tok_tp.npy"))
    dev = torch.device("cuda", 0)
    one = TPDecoder(PRESETS["tiny"], dev, 0, 1, seed=3)
    for tok in (5, 9, 2):
        one.step_eager(tok)
    torch.cuda.synchronize()
    x1 = one.hidden_after_step().float().cpu().numpy()
    # fp16 activations between the layers: the two runs round at different places
    assert np.abs(x_tp - x1).max() / np.abs(x1).max() <= 1e-2
    assert int(tok_tp[0]) == int(one.next_token[0])


@pytest.mark.timeout(150)
def test_two_gpu_decode_chain_matches_one_gpu():
    """The decode chain (one persistent kernel per rank, rank sums of o and down inside it)
    on two GPUs against the decoder of separate launches on one GPU."""
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, ROOT)
    from elutq_b200.decoder import PRESETS, TPDecoder
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker, args=(2, os.path.join(tmp, "init"), tmp, True), nprocs=2, join=True)
        x_tp = np.load(os.path.join(tmp, "x_tp.npy"))
        tok_tp = np.load(os.path.join(tmp, "tok_tp.npy"))
    one = TPDecoder(PRESETS["tiny"], torch.device("cuda", 0), 0, 1, seed=3)
    for tok in (5, 9, 2):
        one.step_eager(tok)
    torch.cuda.synchronize()
    x1 = one.hidden_after_step().float().cpu().numpy()
    assert np.abs(x_tp - x1).max() / np.abs(x1).max() <= 1e-2
    assert int(tok_tp[0]) == int(one.next_token[0])


def _fused_worker(rank, world, init_file, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    from elutq_b200 import _lib, format as F, tp
    from elutq_b200.linear import HLQLinear, linear_forward
    from oracle import hlq_oracle as O
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world, device_id=dev)
    try:
        errs = []
        for (q, n, k, g, m) in [(2, 4096, 4096, 128, 1), (2, 1000, 2048, 64, 2)]:
            d = O.synth_linear(n, k, q, g, m=m, seed=21 + n, bias=True, signed_alpha=True)
            lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], d["bias"], g)
            mod = HLQLinear.from_exported(lin, device=rank, tp_rank=rank, tp_size=world,
                                          shard_mode=_lib.HLQ_SHARD_COLS, max_batch=m)
            comm = tp.FusedAllReduceComm(max_n=n, max_m=m, device=rank)
            x = torch.from_numpy(tp.shard_activation(d["x"], rank, world, _lib.HLQ_SHARD_COLS).copy()).to(dev)
            ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"])
            y_nccl = linear_forward(x, mod.weight, mod.workspace, out_dtype=torch.float32)
            dist.all_reduce(y_nccl)
            for it in range(6):            # both parities of the slots, several launch numbers
                y = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
                comm.forward(x, mod.weight, mod.workspace, y)
                torch.cuda.synchronize()
                assert mod.workspace.kernel_status() == 0
                errs.append(O.normwise_error(y.cpu().numpy(), ref))
                errs.append(O.normwise_error(y.cpu().numpy(), y_nccl.cpu().numpy()))
            dist.barrier()
            comm.free()
        np.save(os.path.join(out_dir, f"fused_{rank}.npy"), np.array(errs))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(150)
def test_fused_allreduce_matches_nccl_on_two_gpus():
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_fused_worker, args=(2, os.path.join(tmp, "init"), tmp), nprocs=2, join=True)
        for r in range(2):
            assert np.load(os.path.join(tmp, f"fused_{r}.npy")).max() <= 1e-5


def test_one_gpu_decoder_grouped_equals_ungrouped():
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    sys.path.insert(0, ROOT)
    from elutq_b200.decoder import PRESETS, TPDecoder
    dev = torch.device("cuda", 0)
    a = TPDecoder(PRESETS["tiny"], dev, 0, 1, seed=9, grouped=True)
    b = TPDecoder(PRESETS["tiny"], dev, 0, 1, seed=9, grouped=False)
    a.step_eager(7)
    b.step_eager(7)
    torch.cuda.synchronize()
    xa, xb = a.hidden_after_step().float(), b.hidden_after_step().float()
    assert (xa - xb).abs().max() / xb.abs().max() <= 2e-3
    g = a.capture(7)
    g.replay()
    torch.cuda.synchronize()
    assert torch.isfinite(a.hidden_after_step().float()).all()


def test_one_gpu_decoder_own_glue_equals_torch_glue():
    """The step with the package's glue kernels against the same step with PyTorch ops."""
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    sys.path.insert(0, ROOT)
    from elutq_b200.decoder import PRESETS, TPDecoder
    dev = torch.device("cuda", 0)
    a = TPDecoder(PRESETS["tiny"], dev, 0, 1, seed=11, fused_glue=True, fused_inputs=False)
    b = TPDecoder(PRESETS["tiny"], dev, 0, 1, seed=11, fused_glue=False)
    ta, tb = a.step_eager(7), b.step_eager(7)
    torch.cuda.synchronize()
    xa, xb = a.hidden_after_step().float(), b.hidden_after_step().float()
    assert (xa - xb).abs().max() / xb.abs().max() <= 4e-3
    la, lb = a.last_logits.float(), b.last_logits.float()
    assert (la - lb).abs().max() / lb.abs().max() <= 1e-2
    # the appended cache rows agree too (v bit-exactly)
    pos = a.pos
    for La, Lb in zip(a.layers, b.layers):
        va, vb = a.kv_rows(La, "vc", pos, pos + 1), b.kv_rows(Lb, "vc", pos, pos + 1)
        assert torch.equal(va, vb) or (va.float() - vb.float()).abs().max() <= 2e-2
    if int(lb.argmax()) == int(la.argmax()):
        assert int(ta.item()) == int(tb.item())
    g = a.capture(7)
    a.token.fill_(7)
    g.replay()
    torch.cuda.synchronize()
    assert a.attn.status() == 0
    assert (a.hidden_after_step().float() - xb).abs().max() / xb.abs().max() <= 4e-3


def test_one_gpu_decoder_norms_and_silu_inside_the_gemv():
    """5 launches per layer (input transforms) against 8 (separate glue kernels)."""
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    sys.path.insert(0, ROOT)
    from elutq_b200.decoder import PRESETS, TPDecoder
    dev = torch.device("cuda", 0)
    a = TPDecoder(PRESETS["tiny"], dev, 0, 1, seed=13, fused_inputs=True)
    b = TPDecoder(PRESETS["tiny"], dev, 0, 1, seed=13, fused_inputs=False)
    assert a.fused_inputs and not b.fused_inputs
    assert a.launches_per_step() < b.launches_per_step()
    ta, tb = a.step_eager(7), b.step_eager(7)
    torch.cuda.synchronize()
    xa, xb = a.hidden_after_step().float(), b.hidden_after_step().float()
    assert (xa - xb).abs().max() / xb.abs().max() <= 4e-3
    la, lb = a.last_logits.float(), b.last_logits.float()
    assert (la - lb).abs().max() / lb.abs().max() <= 1e-2
    g = a.capture(7)
    a.token.fill_(7)
    g.replay()
    torch.cuda.synchronize()
    assert (a.hidden_after_step().float() - xb).abs().max() / xb.abs().max() <= 4e-3


def test_generate_with_one_graph_equals_eager_steps():
    """Position and token id live in device memory: one captured graph decodes every step."""
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    sys.path.insert(0, ROOT)
    from elutq_b200.decoder import PRESETS, TPDecoder
    dev = torch.device("cuda", 0)
    a = TPDecoder(PRESETS["tiny"], dev, 0, 1, seed=21)
    b = TPDecoder(PRESETS["tiny"], dev, 0, 1, seed=21)
    ta = a.generate(3, 6, start_position=100, use_graph=True)
    tb = b.generate(3, 6, start_position=100, use_graph=False)
    assert ta == tb and len(ta) == 6
    assert int(a.position.item()) == 106 and a.attn.status() == 0
    # the cache rows 100..105 were written by the steps (equal up to the order of the GEMVs'
    # slice sums, which can move an fp16 rounding), nothing beyond them was touched
    for La, Lb in zip(a.layers, b.layers):
        assert (a.kv_rows(La, "kc", 100, 106).float() - b.kv_rows(Lb, "kc", 100, 106).float()).abs().max() <= 3e-2
        assert torch.equal(a.kv_rows(La, "kc", 106, 256), b.kv_rows(Lb, "kc", 106, 256))
        assert torch.equal(a.kv_rows(La, "vc", 106, 256), b.kv_rows(Lb, "vc", 106, 256))
    with pytest.raises(ValueError):
        a.generate(1, 10, start_position=250)

