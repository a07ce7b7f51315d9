"""Data-parallel logic on CPU (gloo, world size 2): each rank runs the oracle's LSTM-LM step on
its shard of the batch columns; the summed gradients must equal the single-process gradients of
the whole batch, and after the same clipped SGD update every replica holds identical parameters."""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DIMS = dict(V=40, E=12, H=16, L=2, T=3, B=6)


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import oracle
    from dynet_b200 import dp, lm
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dp.init_process_group("gloo")
    V, E, H, L, T, B = (DIMS[k] for k in "VEHLTB")
    params = lm.init_params(V, E, H, L, seed=5)          # same seed on every rank: replicated parameters
    tokens, masks = lm.synthetic_batch(DIMS, seed=6, dropout=0.2)
    tok, msk = dp.shard_batch(tokens, masks, rank, world)
    grads = [np.zeros_like(p) for p in params]
    loss, _ = oracle.lstm_lm_fwdbwd((V, E, H, L, T, tok.shape[1]), params, grads, tok, msk[0], msk[1])
    flat = torch.from_numpy(np.concatenate(grads))
    dp.allreduce_sum_(flat)
    t_loss = torch.tensor([loss], dtype=torch.float64)
    dp.allreduce_sum_(t_loss)
    grads = [a.copy() for a in np.split(flat.numpy(), np.cumsum([p.size for p in params])[:-1])]
    oracle.sgd_update(params, grads, 0.1, 5.0)
    # replica consistency: max |theta_r - theta_0| must be exactly 0
    mine = torch.from_numpy(np.concatenate(params))
    ref = mine.clone()
    dist.broadcast(ref, src=0)
    dev = (mine - ref).abs().max()
    dist.all_reduce(dev, op=dist.ReduceOp.MAX)
    if rank == 0:
        np.save(out, np.concatenate([flat.numpy(), [t_loss.item(), dev.item()]]))
    dist.destroy_process_group()


def test_sharded_step_equals_full_batch(oracle, tmp_path):
    from dynet_b200 import dp, lm
    assert dp.shard_columns(7, 0, 2) == (0, 4) and dp.shard_columns(7, 1, 2) == (4, 7)
    out = str(tmp_path / "dp.npy")
    mp.spawn(_worker, args=(2, 29533 + os.getpid() % 200, out), nprocs=2, join=True)
    got = np.load(out)
    V, E, H, L, T, B = (DIMS[k] for k in "VEHLTB")
    params = lm.init_params(V, E, H, L, seed=5)
    tokens, masks = lm.synthetic_batch(DIMS, seed=6, dropout=0.2)
    grads = [np.zeros_like(p) for p in params]
    loss, _ = oracle.lstm_lm_fwdbwd((V, E, H, L, T, B), params, grads, tokens, masks[0], masks[1])
    want = np.concatenate(grads)
    assert abs(got[-2] - loss) <= 1e-5 * abs(loss)
    assert got[-1] == 0.0
    scale = np.abs(want).max()
    assert np.abs(got[:-2] - want).max() <= 1e-5 * scale
