"""Batch sharding + output all-gather with two gloo ranks on the CPU."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

from dace_onnx_b200 import sharding


def test_shard_bounds_cover_the_batch():
    for total in [0, 1, 7, 8, 1024, 1025]:
        for world in [1, 2, 3, 4, 8]:
            spans = [sharding.shard_bounds(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_bounds(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, q):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                          MASTER_PORT=str(port))
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        r, w, _ = sharding.init_from_env("gloo")
        full = torch.arange(total * 6, dtype=torch.float32).reshape(total, 2, 3)
        lo, hi = sharding.shard_bounds(total, w, r)
        out = sharding.sharded_forward(lambda t: t * 2 + 1, full[lo:hi], total)
        ok = torch.equal(out, full * 2 + 1)
        # a shard of the wrong size is rejected
        try:
            sharding.all_gather_batch(full[:0] if hi - lo else full[:1], total)
            ok = False
        except ValueError:
            pass
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
        q.put((rank, ok))
    except Exception as exc:  # surfaced by the parent
        q.put((rank, repr(exc)))


@pytest.mark.parametrize("total", [8, 7])
def test_two_rank_gather_matches_single_process(total):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, total, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, True), (1, True)], results


def test_single_process_is_identity():
    x = torch.randn(5, 3)
    assert sharding.all_gather_batch(x, 5) is x
