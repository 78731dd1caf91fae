"""Batch sharding across the GPUs of one node.

Every node on the hot path is independent per sample (GEMM rows, convolution images, softmax /
layer-norm rows), so the batch is cut into contiguous shards, one per rank, with replicated
weights and no communication inside the forward pass. The only collective is the all-gather of
the final activations. One process per GPU; `torch.distributed` carries the collective (NCCL over
NVLink on GPUs, gloo in the CPU tests).
"""
import os

import torch
import torch.distributed as dist


def shard_bounds(total, world, rank):
    """[lo, hi) of rank's contiguous shard; the first `total % world` ranks hold one extra sample."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank %d of %d" % (rank, world))
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def init_from_env(backend):
    """Initialise the default process group from RANK / WORLD_SIZE / MASTER_* if they describe more
    than one process. Returns (rank, world, local_rank)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    return rank, world, local_rank


def all_gather_batch(local, total, out=None, group=None):
    """Concatenate every rank's shard (dim 0) in rank order on every rank.

    Shards follow shard_bounds(total, world, rank). With equal shards this is one
    all_gather_into_tensor straight into `out`; ragged shards are padded to the largest one.
    """
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        if out is None:
            return local
        out.copy_(local)
        return out
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    lo, hi = shard_bounds(total, world, rank)
    if local.shape[0] != hi - lo:
        raise ValueError("rank %d holds %d samples, expected %d" % (rank, local.shape[0], hi - lo))
    tail = tuple(local.shape[1:])
    if out is None:
        out = torch.empty((total,) + tail, dtype=local.dtype, device=local.device)
    if total % world == 0:
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    width = -(-total // world)
    padded = torch.zeros((width,) + tail, dtype=local.dtype, device=local.device)
    padded[:hi - lo] = local
    gathered = torch.empty((world * width,) + tail, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(gathered, padded, group=group)
    for r in range(world):
        rlo, rhi = shard_bounds(total, world, r)
        out[rlo:rhi] = gathered[r * width:r * width + (rhi - rlo)]
    return out


def sharded_forward(forward, x_local, total, out=None, group=None):
    """Run `forward` on this rank's shard and all-gather the result."""
    return all_gather_batch(forward(x_local), total, out=out, group=group)
