"""Request-sharded engine replicas: one independent engine per GPU, no collective.

The reference is a single-GPU engine (there is no distributed code in it).  A 0.5 B
parameter model fits every GPU many times over and requests are independent, so the
multi-GPU form of the path is N replicas that share nothing: the global FIFO of requests
is dealt out by request id, every replica serves its share with its own weights, KV slots
and scheduler, and the outputs are merged back in request-id order — exactly the order
``Engine.run`` returns (src/engine.py:168).

Two ways to run it:

* under ``torch.distributed`` (one process per GPU, e.g. ``torch.distributed.run``):
  ``serve_sharded`` takes this rank's share, serves it and gathers the outputs on rank 0;
  the process group is used only for that gather;
* in one host process with worker callables: ``dispatch`` is a pull-based dispatcher that
  re-queues the requests of a worker that fails (host-side failure handling; nothing here
  touches a GPU).
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Callable, Sequence


@dataclass(frozen=True)
class Request:
    request_id: int
    prompt: tuple          # token ids
    max_tokens: int


def shard(requests: Sequence[Request], rank: int, world: int) -> list[Request]:
    """Round-robin by position in the global FIFO: replica r gets requests r, r+world, ..."""
    if not 0 <= rank < world:
        raise ValueError("rank outside the world")
    return list(requests[rank::world])


def merge(parts: Sequence[dict]) -> list:
    """Outputs of all replicas ({request_id: tokens}) in request-id order."""
    merged: dict = {}
    for part in parts:
        overlap = merged.keys() & part.keys()
        if overlap:
            raise ValueError(f"request served twice: {sorted(overlap)[:3]}")
        merged.update(part)
    return [merged[k] for k in sorted(merged)]


def serve(engine, requests: Sequence[Request]) -> dict:
    """Runs one engine over its share and maps its outputs back to the global request ids."""
    local_ids = [engine.add_request_ids(list(r.prompt), max_tokens=r.max_tokens) for r in requests]
    outputs = engine.run()  # ordered by the engine's own request ids, which grow with submission
    order = sorted(range(len(requests)), key=lambda i: local_ids[i])
    return {requests[i].request_id: out for i, out in zip(order, outputs)}


def serve_sharded(engine, requests: Sequence[Request], dist=None):
    """This rank's share through ``engine``; rank 0 returns all outputs in request-id order,
    other ranks return None.  ``dist`` is ``torch.distributed`` (initialised) or None."""
    if dist is None or not dist.is_initialized():
        return merge([serve(engine, requests)])
    rank, world = dist.get_rank(), dist.get_world_size()
    mine = serve(engine, shard(requests, rank, world))
    gathered = [None] * world if rank == 0 else None
    dist.gather_object(mine, gathered, dst=0)
    return merge(gathered) if rank == 0 else None


def dispatch(requests: Sequence[Request], workers: Sequence[Callable[[list], dict]], chunk: int = 8):
    """Pull-based dispatch inside one process: workers take ``chunk`` requests at a time from
    the shared FIFO; a worker whose call raises is retired and its chunk goes back to the
    head of the queue.  Returns (outputs in request-id order, indices of failed workers)."""
    queue = deque(requests)
    alive = list(range(len(workers)))
    failed: list[int] = []
    parts: list[dict] = []
    while queue:
        if not alive:
            raise RuntimeError("every replica failed; requests left unserved")
        for w in list(alive):
            if not queue:
                break
            batch = [queue.popleft() for _ in range(min(chunk, len(queue)))]
            try:
                parts.append(workers[w](batch))
            except Exception:  # host-side failure of this replica: re-queue, retire it
                queue.extendleft(reversed(batch))
                alive.remove(w)
                failed.append(w)
    return merge(parts), failed
