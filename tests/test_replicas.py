"""Request sharding across replicas: host logic on the CPU, including a world-size-2 gloo run."""

import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402  (spawned ranks import this module without conftest)

entry.load_package()

from quic_cu_b200.config import EngineConfig
from quic_cu_b200.engine import Engine
from quic_cu_b200.replicas import (Request, StoreQueue, chunks_of, dispatch, group_store, merge, serve,
                                   serve_pulled, serve_sharded, shard)
from tests.fake_model import FakeModule, expected_generation


def _requests(n):
    return [Request(request_id=100 + i, prompt=tuple(range(1, 2 + i % 5)), max_tokens=3 + i % 4) for i in range(n)]


def _engine():
    return Engine(config=EngineConfig(max_context=128, decode_burst=2), max_batch_size=3, model_module=FakeModule())


def _expected(reqs):
    return [expected_generation(list(r.prompt), r.max_tokens, eos=None) for r in sorted(reqs, key=lambda r: r.request_id)]


def test_shard_is_a_partition_and_merge_restores_order():
    reqs = _requests(11)
    parts = [shard(reqs, r, 4) for r in range(4)]
    assert sorted(q.request_id for p in parts for q in p) == [q.request_id for q in reqs]
    assert [len(p) for p in parts] == [3, 3, 3, 2]
    outs = [serve(_engine(), p) for p in parts]
    assert merge(outs) == _expected(reqs)
    with pytest.raises(ValueError):
        merge([outs[0], outs[0]])
    with pytest.raises(ValueError):
        shard(reqs, 4, 4)


def test_single_process_serve_sharded():
    reqs = _requests(7)
    assert serve_sharded(_engine(), reqs) == _expected(reqs)


def test_dispatch_requeues_the_work_of_a_failed_replica():
    reqs = _requests(20)
    calls = {"bad": 0}

    def good(batch):
        return serve(_engine(), batch)

    def bad(batch):
        calls["bad"] += 1
        raise RuntimeError("replica lost")

    outputs, failed = dispatch(reqs, [good, bad, good], chunk=3)
    assert outputs == _expected(reqs)
    assert failed == [1] and calls["bad"] == 1
    with pytest.raises(RuntimeError):
        dispatch(reqs, [bad], chunk=3)


def _worker(rank, world, port, out_path):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    reqs = _requests(9)
    result = serve_sharded(_engine(), reqs, dist)
    if rank == 0:
        torch.save(result, out_path)
    else:
        assert result is None
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_gather(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out_path = str(tmp_path / "out.pt")
    mp.spawn(_worker, args=(2, port, out_path), nprocs=2, join=True)
    assert torch.load(out_path) == _expected(_requests(9))


def _pull_worker(rank, world, port, out_path, leave):
    """Rank 0 serves until the whole FIFO is done and collects; rank 1 either serves normally or
    leaves with its first chunk claimed and unfinished (between two iterations of its loop:
    no kernel, no collective in flight -- there are none on this path anyway)."""
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    reqs = _requests(23)
    chunk = 4
    queue = StoreQueue(group_store(dist), len(chunks_of(reqs, chunk)), rank, prefix="t", stale_s=0.4)
    dist.barrier()  # both queues exist (first heartbeat written) before anybody pulls
    if rank == 1 and leave:
        stats = serve_pulled(_engine(), reqs, queue, chunk=chunk, leave_after_chunks=1)
        assert stats["chunks"] == 1
        return  # gone: no goodbye, no destroy_process_group
    stats = serve_pulled(_engine(), reqs, queue, chunk=chunk)
    if rank == 0:
        assert queue.finished()
        merged = queue.collect()
        torch.save(([merged[k] for k in sorted(merged)], stats), out_path)
    if not leave:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("leave", [False, True])
def test_two_gloo_ranks_pull_chunks_and_a_leaver_is_replaced(tmp_path, leave):
    """World size 2 on the CPU: both replicas pull chunks from the queue in the group's store
    and every request is served exactly once; when rank 1 leaves with a claimed chunk, rank 0
    claims it again once the heartbeat is stale and the outputs are still complete."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out_path = str(tmp_path / "out.pt")
    mp.spawn(_pull_worker, args=(2, port, out_path, leave), nprocs=2, join=True)
    outputs, stats = torch.load(out_path)
    assert outputs == _expected(_requests(23))
    if leave:
        assert stats["chunks"] >= 5 and stats["requests"] >= 20  # rank 0 also served the orphan
