"""Tensor-parallel sharding on CPU ranks (gloo, world size 2 and 4): the host-side split of
exported weights, the collectives' glue, and a rank that fails on the host.  Each rank
computes its shard's product with the oracle (no GPU here); the data path is the same one
`elutq_b200.tp` wires to NCCL on GPUs."""
import os
import sys
import tempfile

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, init_file, mode, out_dir):
    sys.path.insert(0, ROOT)
    from elutq_b200 import _lib, format as F, tp
    from oracle import hlq_oracle as O
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    try:
        n, k, q, g, m = 256, 2048, 2, 128, 3
        d = O.synth_linear(n, k, q, g, m=m, seed=4, bias=True, signed_alpha=True)
        lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], d["bias"], g)
        ref = O.hlq_linear(d["x"], d["w_quant"], d["w_scale"], d["w_zero"], g, d["bias"])
        if mode == "cols":      # row-parallel: shard the input channels, all-reduce the outputs
            sh = tp.shard_exported(lin, rank, world, _lib.HLQ_SHARD_COLS)
            xs = tp.shard_activation(d["x"], rank, world, _lib.HLQ_SHARD_COLS)
            assert (sh.bias is None) == (rank != 0)
            y = torch.from_numpy(O.hlq_linear(xs, sh.w_quant, sh.w_scale, sh.w_zero, g, sh.bias))
            dist.all_reduce(y, op=dist.ReduceOp.SUM)
            y = y.numpy()
        else:                   # column-parallel: shard the output rows, all-gather
            sh = tp.shard_exported(lin, rank, world, _lib.HLQ_SHARD_ROWS)
            part = torch.from_numpy(O.hlq_linear(d["x"], sh.w_quant, sh.w_scale, sh.w_zero, g, sh.bias))
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part)
            y = torch.cat(parts, dim=1).numpy()
        err = O.normwise_error(y, ref)
        np.save(os.path.join(out_dir, f"err_{mode}_{rank}.npy"), np.array([err]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("mode", ["rows", "cols"])
def test_sharded_product_over_gloo(world, mode):
    with tempfile.TemporaryDirectory() as tmp:
        init = os.path.join(tmp, "init")
        mp.spawn(_worker, args=(world, init, mode, tmp), nprocs=world, join=True)
        for r in range(world):
            assert np.load(os.path.join(tmp, f"err_{mode}_{r}.npy"))[0] <= 1e-12


def test_shard_shapes_and_errors():
    sys.path.insert(0, ROOT)
    from elutq_b200 import _lib, format as F, tp
    from oracle import hlq_oracle as O
    d = O.synth_linear(96, 1024, 3, 64, seed=1, bias=True)
    lin = F.ExportedLinear(d["w_quant"], d["w_scale"], d["w_zero"], d["bias"], 64)
    a = tp.shard_exported(lin, 1, 2, _lib.HLQ_SHARD_ROWS)
    assert a.w_quant.shape == (3, 48, 128) and a.w_scale.shape == (3, 48, 16) and a.bias.shape == (48,)
    b = tp.shard_exported(lin, 1, 2, _lib.HLQ_SHARD_COLS)
    assert b.w_quant.shape == (3, 96, 64) and b.w_zero.shape == (96, 8) and b.bias is None
    # the shards tile the original exactly
    assert np.array_equal(np.concatenate([tp.shard_exported(lin, r, 4, _lib.HLQ_SHARD_COLS).w_quant
                                          for r in range(4)], axis=2), lin.w_quant)
    assert tp.shard_unit(64) == 128 and tp.shard_unit(256) == 256 and tp.shard_unit(24) == 24
    with pytest.raises(ValueError):
        tp.shard_exported(lin, 0, 5, _lib.HLQ_SHARD_ROWS)       # 96 rows over 5 ranks
    with pytest.raises(ValueError):
        tp.shard_exported(lin, 0, 16, _lib.HLQ_SHARD_COLS)      # 64 channels per rank < 128
    with pytest.raises(ValueError):
        tp.shard_exported(lin, 2, 2, _lib.HLQ_SHARD_ROWS)
    assert tp.shard_exported(lin, 0, 1, _lib.HLQ_SHARD_COLS) is lin


def _failing_worker(rank, world, init_file, out_dir):
    """Rank 1 raises on the host before the collective; rank 0's all-reduce must end with an
    error within the group's timeout instead of hanging."""
    import datetime
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        os._exit(3)                       # leaves between steps, nothing in flight
    t = torch.ones(4)
    try:
        dist.all_reduce(t)
        outcome = "completed"
    except Exception:                     # noqa: BLE001
        outcome = "error"
    with open(os.path.join(out_dir, "outcome.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)


def test_lost_rank_ends_the_collective_with_an_error():
    with tempfile.TemporaryDirectory() as tmp:
        init = os.path.join(tmp, "init")
        ctx = mp.spawn(_failing_worker, args=(2, init, tmp), nprocs=2, join=False)
        for p in ctx.processes:
            p.join(60)
        assert open(os.path.join(tmp, "outcome.txt")).read() == "error"
