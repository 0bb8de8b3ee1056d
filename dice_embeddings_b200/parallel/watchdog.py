"""Heartbeats between ranks: a missing peer becomes a Python exception on the others.

Every rank publishes a monotonically increasing counter under ``hb/<rank>`` in a key-value store (a
``torch.distributed`` ``TCPStore`` / ``FileStore`` or any object with ``set(key, bytes)`` / ``get(key)``) and checks,
before launching its next step, that every peer's counter has moved within ``timeout`` seconds.  Failures are thus
learnt on the host, between steps, with no kernel or collective in flight; recovery is a restart from the last
checkpoint.  The reference has no failure detection (``dicee/trainer/torch_trainer_ddp.py:96-97`` raises
``NotImplementedError`` for snapshots)."""
from __future__ import annotations

import threading
import time
from typing import Dict, Optional


class RankFailure(RuntimeError):
    def __init__(self, rank: int, silent_for: float):
        super().__init__(f"no heartbeat from rank {rank} for {silent_for:.1f} s")
        self.rank, self.silent_for = rank, silent_for


class DictStore:
    """In-process stand-in for a distributed store (tests, single-node threads)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, key: str, value) -> None:
        with self._lock:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key: str) -> bytes:
        with self._lock:
            return self._d.get(key, b"")


class Heartbeat:
    def __init__(self, store, rank: int, world: int, timeout: float = 30.0, interval: float = 1.0,
                 clock=time.monotonic):
        self.store, self.rank, self.world = store, rank, world
        self.timeout, self.interval, self.clock = float(timeout), float(interval), clock
        self._count = 0
        self._seen: Dict[int, tuple] = {}          # peer -> (last counter, time it changed)
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self.failure: Optional[RankFailure] = None

    # ------------------------------------------------------------------ publishing
    def beat(self) -> None:
        self._count += 1
        self.store.set(f"hb/{self.rank}", str(self._count).encode())

    # ------------------------------------------------------------------ checking
    def _read(self, peer: int) -> int:
        try:
            key = f"hb/{peer}"
            check = getattr(self.store, "check", None)   # c10d stores block in get() until the key exists
            if check is not None and not check([key]):
                return 0
            raw = self.store.get(key)
            return int(raw.decode() or 0) if raw else 0
        except Exception:
            return 0

    def check(self) -> None:
        """Raise :class:`RankFailure` if a peer's counter has not advanced for ``timeout`` seconds."""
        now = self.clock()
        for peer in range(self.world):
            if peer == self.rank:
                continue
            c = self._read(peer)
            last = self._seen.get(peer)
            if last is None or c != last[0]:
                self._seen[peer] = (c, now)
            elif now - last[1] > self.timeout:
                self.failure = RankFailure(peer, now - last[1])
                raise self.failure
        if self.failure is not None:
            raise self.failure

    # ------------------------------------------------------------------ background mode
    def start(self) -> "Heartbeat":
        """Beat and check from a daemon thread; a detected failure is kept in ``self.failure`` and re-raised by the
        next ``check()`` / ``raise_if_failed()`` call of the training loop."""
        def loop():
            while not self._stop.wait(self.interval):
                self.beat()
                try:
                    self.check()
                except RankFailure:
                    return
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return self

    def raise_if_failed(self) -> None:
        if self.failure is not None:
            raise self.failure

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)
