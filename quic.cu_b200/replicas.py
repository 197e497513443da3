"""Request-sharded engine replicas: one independent engine per GPU, no collective.

The reference is a single-GPU engine (there is no distributed code in it).  A 0.5 B
parameter model fits every GPU many times over and requests are independent, so the
multi-GPU form of the path is N replicas that share nothing: the global FIFO of requests
is dealt out by request id, every replica serves its share with its own weights, KV slots
and scheduler, and the outputs are merged back in request-id order — exactly the order
``Engine.run`` returns (src/engine.py:168).

Three ways to run it:

* ``serve_pulled`` (the default under ``torch.distributed``, one process per GPU): the FIFO is
  cut into chunks and every replica PULLS the next unclaimed chunk from a shared queue kept in
  the process group's key-value store whenever its engine has room, so a replica that drew
  short requests simply takes more.  Claims, heartbeats and outputs go through the store, no
  collective is involved, and the chunk of a replica that stopped answering is claimed again
  by a survivor;
* ``serve_sharded``: a static round-robin deal by request id, outputs gathered on rank 0;
* ``dispatch``: the pull-based form inside one host process with worker callables (host-side
  failure handling for tests; nothing here touches a GPU).
"""

from __future__ import annotations

import pickle
import time
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


class StoreQueue:
    """Shared FIFO of request chunks over a ``torch.distributed`` key-value store.

    Keys (under ``prefix``): ``next`` = chunks handed out so far (atomic add), ``own/<i>`` =
    rank serving chunk i, ``out/<i>`` = pickled outputs of chunk i, ``done`` = chunks finished,
    ``hb/<rank>`` = last sign of life of a rank (host clock; all ranks share one host).  A
    chunk whose owner has shown no sign of life for ``stale_s`` seconds may be claimed again
    with a compare-and-set, so exactly one survivor re-serves it."""

    def __init__(self, store, n_chunks: int, rank: int, prefix: str = "quicq", stale_s: float = 5.0):
        self.store, self.n_chunks, self.rank, self.prefix, self.stale_s = store, n_chunks, rank, prefix, stale_s
        self.beat()

    def _k(self, name: str) -> str:
        return f"{self.prefix}/{name}"

    def beat(self) -> None:
        self.store.set(self._k(f"hb/{self.rank}"), repr(time.time()))

    def take(self) -> int | None:
        """Next unclaimed chunk, or None when every chunk has been handed out."""
        self.beat()
        if int(self.store.add(self._k("next"), 0)) >= self.n_chunks:
            return None
        idx = int(self.store.add(self._k("next"), 1)) - 1
        if idx >= self.n_chunks:
            return None
        self.store.set(self._k(f"own/{idx}"), str(self.rank))
        return idx

    def take_orphan(self) -> int | None:
        """A handed-out, unfinished chunk whose owner went silent; claimed for this rank."""
        self.beat()
        now = time.time()
        handed = min(int(self.store.add(self._k("next"), 0)), self.n_chunks)
        for idx in range(handed):
            if self.store.check([self._k(f"out/{idx}")]):
                continue
            own_key = self._k(f"own/{idx}")
            if not self.store.check([own_key]):
                continue  # claimed a moment ago, owner not written yet
            owner = self.store.get(own_key).decode()
            if int(owner) == self.rank:
                continue
            hb_key = self._k(f"hb/{owner}")
            last = float(self.store.get(hb_key).decode()) if self.store.check([hb_key]) else 0.0
            if now - last < self.stale_s:
                continue
            if self.store.compare_set(own_key, owner, str(self.rank)).decode() == str(self.rank):
                return idx
        return None

    def done(self, idx: int, outputs: dict) -> None:
        self.store.set(self._k(f"out/{idx}"), pickle.dumps(outputs))
        self.store.add(self._k("done"), 1)
        self.beat()

    def finished(self) -> bool:
        return int(self.store.add(self._k("done"), 0)) >= self.n_chunks

    def collect(self) -> dict:
        """All outputs {request_id: tokens}; call once ``finished()``."""
        merged: dict = {}
        for idx in range(self.n_chunks):
            merged.update(pickle.loads(self.store.get(self._k(f"out/{idx}"))))
        return merged


def group_store(dist):
    """The key-value store behind the default process group of ``torch.distributed``."""
    from torch.distributed import distributed_c10d

    return distributed_c10d._get_default_store()


def chunks_of(requests: Sequence[Request], chunk: int) -> list[list[Request]]:
    return [list(requests[i:i + chunk]) for i in range(0, len(requests), chunk)]


def serve_pulled(engine, requests: Sequence[Request], queue: StoreQueue, chunk: int = 16,
                 idle_sleep_s: float = 0.02, leave_after_chunks: int | None = None) -> dict:
    """Serves chunks pulled from ``queue`` until every chunk of the FIFO is finished (by this or
    by another replica); returns statistics of this replica.  ``requests`` is the whole FIFO,
    identical on every rank (only chunk indices travel).  The engine asks for more requests
    whenever fewer than a batch are waiting; a chunk is reported done when its last request is
    released.  ``leave_after_chunks``: after claiming that many chunks return at once, the last
    of them claimed but never served (tests of the re-queue path: a replica that leaves
    between two iterations of its loop)."""
    parts = chunks_of(requests, chunk)
    if len(parts) != queue.n_chunks:
        raise ValueError("queue was built for a different number of chunks")
    open_chunks: dict[int, dict] = {}  # chunk index -> {"left": n, "out": {request_id: tokens}}
    stats = {"chunks": 0, "requests": 0, "busy_s": 0.0}

    def claim(idx: int) -> list:
        stats["chunks"] += 1
        stats["requests"] += len(parts[idx])
        open_chunks[idx] = {"left": len(parts[idx]), "out": {}}
        return [(list(r.prompt), r.max_tokens, (idx, r.request_id)) for r in parts[idx]]

    def leaving() -> bool:
        return leave_after_chunks is not None and stats["chunks"] >= leave_after_chunks

    class _Leave(Exception):
        pass

    def source(room: int) -> list:
        out: list = []
        while room > 0:
            idx = queue.take()
            if idx is None:
                break
            out.extend(claim(idx))
            room -= len(parts[idx])
            if leaving():
                raise _Leave()  # the chunk just claimed is never handed to the engine
        return out

    def finish(tag, tokens) -> None:
        idx, request_id = tag
        entry = open_chunks[idx]
        entry["out"][request_id] = tokens
        entry["left"] -= 1
        if entry["left"] == 0:
            queue.done(idx, entry.pop("out"))
            del open_chunks[idx]

    engine.request_source, engine.on_finish = source, finish
    try:
        while True:
            t0 = time.perf_counter()
            try:
                engine.run()  # returns when nothing runs, nothing waits and the queue hands out nothing
            except _Leave:
                break
            finally:
                stats["busy_s"] += time.perf_counter() - t0
            if queue.finished():
                break
            idx = queue.take_orphan()
            if idx is not None:
                for ids, limit, tag in claim(idx):
                    engine.add_request_ids(ids, max_tokens=limit, tag=tag)
                continue
            time.sleep(idle_sleep_s)  # others still work on their chunks
    finally:
        engine.request_source = engine.on_finish = None
    return stats
