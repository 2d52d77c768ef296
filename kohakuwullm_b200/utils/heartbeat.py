"""Host-side liveness of the ranks of a job: who is still there, learnt BEFORE the next collective is launched.

A collective whose peer has died does not fail, it waits: NCCL until its watchdog fires minutes later, a kernel of
this library until its bounded wait runs out. Both are correct last resorts and both waste the time (and, on the GPU,
leave work in flight). The cheap first line is on the host: every rank writes a beat into the job's key-value store
from a daemon thread, and the step loop asks ``check()`` between steps, with none of its kernels or collectives in
flight. ``check`` raises ``PeerLost`` naming the rank when a peer's beat is older than ``timeout`` seconds or when a
peer announced that it is leaving (``leave()``: a rank that ends early on purpose, e.g. after an exception in its own
step, says so and the others stop at once instead of after the timeout).

    hb = RankHeartbeat.from_env(interval=1.0, timeout=15.0)     # one extra TCP store on MASTER_PORT + 1
    for batch in loader:
        hb.check()                                               # host only: no device work, no collective
        trainer.training_step(batch)
    hb.close()

The store is a ``torch.distributed.TCPStore`` of its own (rank 0 serves it), not the process group's: a store request
must never queue behind a collective. Nothing here touches a device. The reference has no counterpart (it relies on
the NCCL watchdog and ``elastic_launch(max_restarts=0)``); recovery is the same: end the run, resume from the last
checkpoint.
"""

from __future__ import annotations

import os
import threading
import time
from datetime import timedelta

from kohakuwullm_b200.pipe.hooks import Callback


class PeerLost(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} {reason}")
        self.rank, self.reason = rank, reason


class RankHeartbeat:
    """``store`` needs ``set(key, value)`` and ``get(key)`` (a ``TCPStore``, ``FileStore``, ``HashStore`` or a fake).
    Beats are wall-clock seconds of the WRITER; staleness is judged on the reader's own clock from the moment the
    value last CHANGED, so the ranks' clocks need not agree."""

    def __init__(self, store, rank: int, world: int, interval: float = 1.0, timeout: float = 15.0,
                 prefix: str = "kwu/hb", start: bool = True):
        if timeout <= 2 * interval:
            raise ValueError("timeout must be more than two beat intervals")
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.interval, self.timeout, self.prefix = float(interval), float(timeout), prefix
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._seen: dict[int, tuple[bytes, float]] = {}      # peer -> (last value, when it changed, on OUR clock)
        self._born = time.monotonic()
        self._last_check = 0.0
        self._count = 0
        self._beat()
        if start:
            self._thread = threading.Thread(target=self._run, name=f"kwu-heartbeat-{rank}", daemon=True)
            self._thread.start()

    # ------------------------------------------------------------------ construction from the launcher's environment
    @classmethod
    def from_env(cls, interval: float = 1.0, timeout: float = 15.0, port_offset: int = 1, **kw) -> "RankHeartbeat":
        from torch.distributed import TCPStore

        rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
        host = os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = int(os.environ.get("KWU_HEARTBEAT_PORT", int(os.environ.get("MASTER_PORT", 29500)) + port_offset))
        store = TCPStore(host, port, world_size=None, is_master=(rank == 0), timeout=timedelta(seconds=max(timeout, 30.0)),
                         wait_for_workers=False)
        return cls(store, rank, world, interval, timeout, **kw)

    # ------------------------------------------------------------------ writer side
    def _key(self, rank: int, what: str = "beat") -> str:
        return f"{self.prefix}/{what}/{rank}"

    def _beat(self) -> None:
        self._count += 1
        self.store.set(self._key(self.rank), f"{self._count}:{time.time():.3f}")

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self._beat()
            except Exception:  # noqa: BLE001  (the store's server went away with rank 0: the readers will notice)
                return

    def leave(self, reason: str = "left the job") -> None:
        """Announce an early exit; the other ranks' next ``check`` raises at once."""
        try:
            self.store.set(self._key(self.rank, "left"), reason)
        except Exception:  # noqa: BLE001
            pass
        self.close()

    def close(self) -> None:
        self._stop.set()
        if self._thread is not None and self._thread.is_alive() and threading.current_thread() is not self._thread:
            self._thread.join(timeout=2 * self.interval)
        self._thread = None

    # ------------------------------------------------------------------ reader side
    def _get(self, key: str) -> bytes | None:
        check = getattr(self.store, "check", None)
        try:
            if check is not None and not check([key]):
                return None
            return bytes(self.store.get(key))
        except Exception:  # noqa: BLE001  (a key that is not there yet, or a store whose server is gone)
            return None

    def check(self, force: bool = False) -> None:
        """Raise ``PeerLost`` if a peer said it left or has not beaten for ``timeout`` seconds. Looks at the store
        at most once per beat interval unless ``force``; in between it returns immediately."""
        now = time.monotonic()
        if not force and now - self._last_check < self.interval:
            return
        self._last_check = now
        for peer in range(self.world):
            if peer == self.rank:
                continue
            left = self._get(self._key(peer, "left"))
            if left is not None:
                raise PeerLost(peer, left.decode(errors="replace"))
            value = self._get(self._key(peer))
            if value is None:
                # never seen: allowed for ``timeout`` seconds after our own start (ranks do not start together)
                if now - self._born > self.timeout:
                    raise PeerLost(peer, f"never sent a heartbeat in {self.timeout:.0f} s")
                continue
            last = self._seen.get(peer)
            if last is None or last[0] != value:
                self._seen[peer] = (value, now)
            elif now - last[1] > self.timeout:
                raise PeerLost(peer, f"sent no heartbeat for {now - last[1]:.1f} s")

    def alive(self) -> list[int]:
        """Ranks whose beat changed within the timeout (this rank included), without raising."""
        now = time.monotonic()
        out = [self.rank]
        for peer in range(self.world):
            if peer == self.rank:
                continue
            value = self._get(self._key(peer))
            if value is None or self._get(self._key(peer, "left")) is not None:
                continue
            last = self._seen.get(peer)
            if last is None or last[0] != value:
                self._seen[peer] = (value, now)
                out.append(peer)
            elif now - last[1] <= self.timeout:
                out.append(peer)
        return sorted(out)


class HeartbeatCallback(Callback):
    """Trainer callback (both trainers): ``check`` before every step, ``leave`` when this rank's own step raised."""

    def __init__(self, heartbeat: RankHeartbeat):
        self.heartbeat = heartbeat

    def on_train_batch_start(self, *args, **kwargs) -> None:
        self.heartbeat.check()

    def on_exception(self, trainer, exc=None, *args, **kwargs) -> None:
        if not isinstance(exc, PeerLost):
            self.heartbeat.leave(f"raised {type(exc).__name__}: {exc}"[:200])

    def on_fit_end(self, *args, **kwargs) -> None:
        self.heartbeat.close()
