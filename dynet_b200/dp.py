"""Data-parallel plumbing for the LSTM-LM step: one process per GPU, the global batch is split
by columns (sequences), parameters are replicated, and the flat gradient buffer is summed with
one all-reduce between backward and the trainer update.  The sum (not the mean) reproduces the
single-GPU gradient of the global batch because the loss is sum_batches(...).  The reference has
no GPU collective at all (its only data parallelism is CPU fork + shared memory, dynet/mp.h)."""
import os

import numpy as np


def shard_columns(n_cols, rank, world):
    """Contiguous block [lo, hi) of the batch columns owned by `rank` (sizes differ by at most 1)."""
    base, rem = divmod(n_cols, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_batch(tokens, masks, rank, world):
    """tokens [(T+1), B] and masks ((mask_x list, mask_h list) of [B, I]) -> this rank's columns."""
    lo, hi = shard_columns(tokens.shape[1], rank, world)
    tok = np.ascontiguousarray(tokens[:, lo:hi])
    if masks is None:
        return tok, None
    mx, mh = masks
    return tok, ([np.ascontiguousarray(m[lo:hi]) for m in mx], [np.ascontiguousarray(m[lo:hi]) for m in mh])


def init_process_group(backend):
    """Rendezvous from the torchrun environment (RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT)."""
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, world


def allreduce_sum_(tensor):
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM)
    return tensor
