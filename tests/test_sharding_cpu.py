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


def test_overlapped_gather_plan_single_process():
    g = sharding.OverlappedGather(12, [(0, 8), (8, 2), (10, 2)])
    assert g.global_rows() == list(range(12))
    y, out = torch.arange(12.0).reshape(12, 1), torch.zeros(12, 1)
    for lo, n in [(0, 8), (8, 2), (10, 2)]:
        g.chunk_done(y, out, lo, n)
    g.finish()
    assert torch.equal(out, y)
    with pytest.raises(ValueError):
        sharding.OverlappedGather(12, [(0, 8), (9, 3)])      # a hole
    with pytest.raises(ValueError):
        sharding.OverlappedGather(12, [(0, 8)])              # does not cover the shard
    with pytest.raises(ValueError):
        g.chunk_done(y, out, 8, 4)                           # not a planned piece


def _worker_overlapped(rank, world, port, q):
    try:
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                          MASTER_PORT=str(port))
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        sharding.init_from_env("gloo")
        total, chunks = 20, [(0, 6), (6, 2), (8, 2)]          # 10 local samples in three pieces
        g = sharding.OverlappedGather(total, chunks)
        rows = g.global_rows()
        # pieces of all ranks tile the batch exactly once
        every = sorted(sum((g.global_rows(r) for r in range(world)), []))
        ok = every == list(range(total)) and rows[:6] == list(range(6 * rank, 6 * rank + 6))
        full = torch.arange(total * 3, dtype=torch.float32).reshape(total, 3)
        y_local = full[rows] * 2 + 1                           # "forward" of this rank's rows
        out = torch.full((total, 3), -1.0)
        for lo, n in chunks:                                   # pieces complete one after the other
            g.chunk_done(y_local, out, lo, n)
        g.finish()
        ok = ok and torch.equal(out, full * 2 + 1)
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
        q.put((rank, ok))
    except Exception as exc:
        q.put((rank, repr(exc)))


def test_two_rank_overlapped_gather_places_every_piece():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_overlapped, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, True), (1, True)], results


def test_encoder_chunk_plans():
    from dace_onnx_b200.encoder import BertEncoderB200
    enc = BertEncoderB200.__new__(BertEncoderB200)
    enc.micro_batch = 256
    assert enc.device_chunks(128, 4) == [(0, 32), (32, 32), (64, 32), (96, 32)]
    assert enc.device_chunks(512, 4) == [(0, 256), (256, 64), (320, 64), (384, 64), (448, 64)]
    assert enc.device_chunks(512, 1) == [(0, 256), (256, 256)]
    assert enc.device_chunks(20, 4) == [(0, 20)]            # too small to cut
    assert enc.device_chunks(130, 4) == [(0, 33), (33, 33), (66, 33), (99, 31)]
    assert enc.host_chunks(128) == [(0, 64), (64, 64)]
    assert enc.host_chunks(1024) == [(0, 128), (128, 256), (384, 256), (640, 256), (896, 128)]
    for bsz in (1, 63, 64, 200, 511, 512, 1000):
        for plan in (enc.device_chunks(bsz, 4), enc.host_chunks(bsz)):
            assert plan[0][0] == 0 and sum(n for _, n in plan) == bsz
            assert all(a[0] + a[1] == b[0] for a, b in zip(plan, plan[1:]))
