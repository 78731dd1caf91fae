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


class OverlappedGather:
    """All-gather of the outputs piece by piece, each piece on a side stream as soon as the forward pass has
    finished it, so that only the last piece's transfer is not hidden behind compute.

    Every rank cuts its shard into the same `chunks` = [(lo, n), ...] (local sample ranges in the order the
    forward pass completes them). Piece c of all ranks lands in one contiguous block of the gathered tensor, so
    each piece is a single all_gather_into_tensor straight into its place, without staging copies:

        gathered[world * lo_c + r * n_c + j] = rank r's local sample lo_c + j

    i.e. the batch is dealt to the ranks piece-cyclically instead of in one contiguous slab per rank
    (`global_rows` gives a rank's rows; with a single piece it is exactly shard_bounds). Samples are independent
    on this path, so which rank computes which sample does not change any result. Needs total % world == 0."""

    def __init__(self, total, chunks, group=None, timeline=None):
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if total % self.world:
            raise ValueError("OverlappedGather needs equal shards (total %d, world %d)" % (total, self.world))
        self.total, self.local, self.group = total, total // self.world, group
        pos = 0
        for lo, n in chunks:
            if lo != pos or n < 1:
                raise ValueError("chunks must tile [0, %d) in order, got %s" % (self.local, chunks))
            pos += n
        if pos != self.local:
            raise ValueError("chunks cover %d of %d local samples" % (pos, self.local))
        self.chunks = {lo: n for lo, n in chunks}
        self.timeline = timeline   # when a list: (start_event, end_event, bytes) per collective
        self._side = None

    def global_rows(self, rank=None):
        """Rows of the gathered tensor that `rank` computes, in the order of its local samples."""
        r = self.rank if rank is None else rank
        rows = []
        for lo, n in sorted(self.chunks.items()):
            rows.extend(range(self.world * lo + r * n, self.world * lo + (r + 1) * n))
        return rows

    def chunk_done(self, y_local, out, lo, n):
        """Call when local samples [lo, lo+n) of y_local are final (in stream order on the current stream)."""
        if self.chunks.get(lo) != n:
            raise ValueError("piece (%d, %d) is not in the plan" % (lo, n))
        dst = out[self.world * lo:self.world * (lo + n)]
        src = y_local[lo:lo + n]
        if self.world == 1:
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src)
            return
        if not y_local.is_cuda:
            dist.all_gather_into_tensor(dst, src.contiguous(), group=self.group)
            return
        main = torch.cuda.current_stream(y_local.device)
        if self._side is None:
            self._side = torch.cuda.Stream(y_local.device)
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            if self.timeline is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            dist.all_gather_into_tensor(dst, src, group=self.group)
            if self.timeline is not None:
                e1.record()
                self.timeline.append((e0, e1, dst.numel() * dst.element_size()))

    def finish(self, device=None):
        """Join the side stream into the current stream: afterwards `out` is complete in stream order."""
        if self._side is not None:
            torch.cuda.current_stream(device).wait_stream(self._side)


def sharded_forward(forward, x_local, total, out=None, group=None):
    """Run `forward` on this rank's shard and all-gather the result."""
    return all_gather_batch(forward(x_local), total, out=out, group=group)
