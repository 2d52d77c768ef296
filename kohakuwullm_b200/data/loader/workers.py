"""Worker-process pack loaders: rendering + tokenisation + packing run in ``workers`` child processes, the
trainer only takes finished packs off queues.

Each worker owns one shard of the record order (shard ``rank * workers + w`` of ``world * workers``, the same
cut the in-process ``ddp`` loader uses with ``worker=w``) and runs an ``IterativePackLoader`` (or, for pipeline
steps, a ``MicroBatchedLoader``) over it. The parent takes batches from the workers round-robin, so the stream
is deterministic for a given ``(world, workers)``; every batch arrives with the position to continue right
after it, and ``state_dict`` records, per worker shard, the position of the batch that was last CONSUMED
(batches a worker has produced ahead of the trainer are rendered again after a resume, never skipped) together
with which worker is next in the rotation. Resuming under another worker count or world size is refused: every
shard would move. Children are forked (the record source, renderer and tokenizer are inherited, nothing has to
be picklable) and touch no GPU. Reference: src/kohakuwullm/data/loader/fast_loader.py:24-225,
microbatch.py:20-261, resume.py:20-274.
"""

from __future__ import annotations

import io
import multiprocessing as mp
import queue
from typing import Callable

from kohakuwullm_b200.data.loader.iterative import IterativePackLoader, MicroBatchedLoader

_STOP = "__stop__"


def _worker_main(make_loader: Callable, state: dict | None, out: "mp.Queue", stop: "mp.Event") -> None:
    try:
        import torch

        # a forked child must not enter the parent's OpenMP thread pool (its worker threads do not exist here)
        torch.set_num_threads(1)
        loader = make_loader()
        if state is not None:
            loader.load_state_dict(state)
        for batch, pos in loader:
            # as BYTES: a tensor put on a multiprocessing queue travels as a shared-memory file descriptor that the
            # receiver has to fetch from a helper thread of the sender, which fails (EOFError) when the sender is a
            # forked child that is exiting or busy; a byte string goes through the pipe itself
            buf = io.BytesIO()
            torch.save(batch, buf)
            payload = buf.getvalue()
            while not stop.is_set():
                try:
                    out.put((payload, pos), timeout=0.2)
                    break
                except queue.Full:
                    continue
            if stop.is_set():
                break
    except BaseException as exc:  # noqa: BLE001  the parent re-raises it
        out.put((_STOP, f"{type(exc).__name__}: {exc}"))


class WorkerPackLoader:
    """Yields ``(batch, position)`` like the in-process loaders; wrap it in ``ResumableLoader`` for checkpoints.

    ``kind``: ``"iterative"`` (packs of at most ``k`` tokens) or ``"pipeline"`` (``MicroBatchedStep`` objects).
    For ``"pipeline"`` every rank must see the same steps, so ``rank`` / ``world`` are ignored (shard
    ``w`` of ``workers``)."""

    def __init__(self, records, renderer, encode, *, workers: int = 4, rank: int = 0, world: int = 1,
                 kind: str = "iterative", prefetch: int = 4, pin_memory: bool = False, **loader_kwargs):
        if workers < 1:
            raise ValueError("workers must be at least 1")
        if kind not in ("iterative", "pipeline"):
            raise ValueError(f"unknown worker loader kind {kind!r}")
        total_shards = workers if kind == "pipeline" else world * workers
        if len(records) < total_shards:
            # a worker whose shard is empty would exit without a batch; say what is wrong instead
            raise ValueError(f"{len(records)} records cannot feed {total_shards} loader shards "
                             f"({workers} workers x {1 if kind == 'pipeline' else world} ranks): use fewer workers")
        self.records, self.renderer, self.encode = records, renderer, encode
        self.workers, self.rank, self.world, self.kind = workers, rank, world, kind
        self.prefetch, self.pin_memory, self.kw = prefetch, pin_memory, loader_kwargs
        if kind == "pipeline":
            self.shards, self.first_shard = workers, 0
        else:
            self.shards, self.first_shard = world * workers, rank * workers
        self._positions: list[dict | None] = [None] * workers     # last consumed, per worker
        self._next = 0
        self._procs: list = []
        self._queues: list = []
        self._stop = None

    # ------------------------------------------------------------------ construction of one worker's loader
    def _factory(self, w: int) -> Callable:
        shard, shards = self.first_shard + w, self.shards
        cls = MicroBatchedLoader if self.kind == "pipeline" else IterativePackLoader

        def make():
            return cls(self.records, self.renderer, self.encode, shard=shard, shards=shards, **self.kw)

        return make

    # ------------------------------------------------------------------ resume
    def state_dict(self) -> dict:
        initial = [self._factory(w)().state_dict() for w in range(self.workers)] if any(
            p is None for p in self._positions) else None
        return {"workers": self.workers, "shards": self.shards, "first_shard": self.first_shard, "next": self._next,
                "positions": [p if p is not None else initial[w] for w, p in enumerate(self._positions)]}

    def load_state_dict(self, state: dict) -> None:
        if state["workers"] != self.workers:
            raise ValueError(f"loader state was saved with {state['workers']} worker processes and this loader has "
                             f"{self.workers}: shards are cut per worker, so every shard would move")
        if state["shards"] != self.shards or state["first_shard"] != self.first_shard:
            raise ValueError(f"loader state covers shards {state['first_shard']}..+{state['workers']} of "
                             f"{state['shards']}, this loader {self.first_shard}..+{self.workers} of {self.shards}")
        if self._procs:
            raise RuntimeError("load the loader state before iterating: a running worker reads its position at start")
        self._positions = list(state["positions"])
        self._next = int(state["next"])

    # ------------------------------------------------------------------ iteration
    def _start(self) -> None:
        ctx = mp.get_context("fork")
        self._stop = ctx.Event()
        for w in range(self.workers):
            q = ctx.Queue(maxsize=self.prefetch)
            p = ctx.Process(target=_worker_main, args=(self._factory(w), self._positions[w], q, self._stop), daemon=True)
            p.start()
            self._procs.append(p)
            self._queues.append(q)

    def close(self) -> None:
        if self._stop is not None:
            self._stop.set()
        for q in self._queues:
            try:
                while True:
                    q.get_nowait()
            except (queue.Empty, OSError, ValueError, EOFError):
                pass
        for p in self._procs:
            p.join(timeout=2.0)
            if p.is_alive():
                p.terminate()
        self._procs, self._queues, self._stop = [], [], None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass

    def __iter__(self):
        if not self._procs:
            self._start()
        try:
            while True:
                w = self._next
                proc = self._procs[w]
                while True:
                    try:
                        item = self._queues[w].get(timeout=1.0)
                        break
                    except queue.Empty:
                        if not proc.is_alive():
                            raise RuntimeError(f"loader worker {w} exited (code {proc.exitcode}) without a batch")
                batch, pos = item
                if isinstance(batch, str) and batch == _STOP:
                    raise RuntimeError(f"loader worker {w} failed: {pos}")
                import torch

                batch = torch.load(io.BytesIO(batch), weights_only=False)
                if self.pin_memory and hasattr(batch, "pin_memory"):
                    batch = batch.pin_memory()
                self._positions[w] = pos
                self._next = (w + 1) % self.workers
                yield batch, self.state_dict()
        finally:
            self.close()
