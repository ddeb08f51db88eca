"""Rank health monitoring and failure detection on the host.

The reference has none (it tolerates half-written checkpoints and restarts from the last one).  Here
every rank publishes a heartbeat counter in the job's key-value store (`torch.distributed` TCPStore /
FileStore / a dict-like fake in tests) from a background thread; `check()` — called by the trainer between
steps, never while a kernel of this rank is in flight with peers — raises `PeerFailure` naming the ranks
whose heartbeat is older than `timeout_s`, so survivors stop before their next collective launch.  Device
kernels additionally bound every peer wait (`DeviceStatusError` / `PeerTimeoutError` from
`recml_b200.ops._lib.check_status`).  Recovery = restart from the last committed checkpoint, possibly with
a different world size (tables are stored as global arrays, see `recml_b200.ckpt`).
"""
from __future__ import annotations

import os
import threading
import time
from typing import Any, Callable


class PeerFailure(RuntimeError):
  def __init__(self, ranks, ages):
    super().__init__(f"ranks {ranks} missed heartbeats (seconds since last beat: {ages})")
    self.ranks, self.ages = ranks, ages


class FaultInjector:
  """Host-side fault injection for tests: `RECML_FAULT="stop_heartbeat:rank=1:step=3"` or
  `"raise:rank=0:step=5"`.  Nothing here touches a GPU."""

  def __init__(self, spec: str | None = None):
    spec = spec if spec is not None else os.environ.get("RECML_FAULT", "")
    self.kind, self.rank, self.step = None, None, None
    if spec:
      parts = spec.split(":")
      self.kind = parts[0]
      kv = dict(p.split("=") for p in parts[1:])
      self.rank, self.step = int(kv.get("rank", -1)), int(kv.get("step", -1))

  def fires(self, kind: str, rank: int, step: int) -> bool:
    return self.kind == kind and self.rank == rank and step >= self.step >= 0


class HealthMonitor:
  def __init__(self, store: Any, rank: int, world: int, *, interval_s: float = 0.5, timeout_s: float = 5.0,
               clock: Callable[[], float] = time.time, injector: FaultInjector | None = None):
    self.store, self.rank, self.world = store, rank, world
    self.interval_s, self.timeout_s, self.clock = interval_s, timeout_s, clock
    self.injector = injector or FaultInjector("")
    self._stop = threading.Event()
    self._thread: threading.Thread | None = None
    self._step = 0
    self._seen: dict[int, tuple[bytes, float]] = {}
    self._beats = 0

  @staticmethod
  def _key(rank: int) -> str:
    return f"recml/heartbeat/{rank}"

  def beat(self) -> None:
    self._beats += 1
    self.store.set(self._key(self.rank), str(self._beats).encode())

  def start(self) -> "HealthMonitor":
    self.beat()

    def loop():
      while not self._stop.wait(self.interval_s):
        if self.injector.fires("stop_heartbeat", self.rank, self._step):
          return
        try:
          self.beat()
        except Exception:  # the store went away with the job
          return

    self._thread = threading.Thread(target=loop, daemon=True, name="recml-heartbeat")
    self._thread.start()
    now = self.clock()
    self._seen = {r: (b"", now) for r in range(self.world)}
    return self

  def stop(self) -> None:
    self._stop.set()
    if self._thread is not None:
      self._thread.join(timeout=2 * self.interval_s + 1)

  @staticmethod
  def _left_key(rank: int) -> str:
    return f"recml/left/{rank}"

  def leave(self) -> None:
    """Announces that this rank leaves the job (between steps, with none of its kernels or collectives in
    flight) and stops its heartbeat; the peers' next `check()` raises `PeerFailure` naming it, before they
    launch anything that would wait for this rank."""
    try:
      self.store.set(self._left_key(self.rank), b"1")
    finally:
      self.stop()

  def _get(self, rank: int) -> bytes | None:
    try:
      if hasattr(self.store, "check") and not self.store.check([self._key(rank)]):
        return None
      return bytes(self.store.get(self._key(rank)))
    except Exception:  # pylint: disable=broad-except
      return None

  def check(self, step: int | None = None) -> None:
    """Raises PeerFailure when a peer's heartbeat value has not changed for `timeout_s`."""
    if step is not None:
      self._step = step
      if self.injector.fires("raise", self.rank, step):
        raise RuntimeError(f"injected failure on rank {self.rank} at step {step}")
    now = self.clock()
    late, ages = [], []
    for r in range(self.world):
      if r == self.rank:
        continue
      try:
        gone = bool(self.store.check([self._left_key(r)])) if hasattr(self.store, "check") else False
      except Exception:  # pylint: disable=broad-except
        gone = False
      if gone:
        late.append(r)
        ages.append(0.0)
        continue
      val = self._get(r)
      prev_val, prev_t = self._seen.get(r, (b"", now))
      if val is not None and val != prev_val:
        self._seen[r] = (val, now)
      elif now - prev_t > self.timeout_s:
        late.append(r)
        ages.append(round(now - prev_t, 2))
    if late:
      raise PeerFailure(late, ages)


class DictStore:
  """In-process stand-in for a distributed key-value store (tests)."""

  def __init__(self):
    self._d: dict[str, bytes] = {}
    self._mu = threading.Lock()

  def set(self, k, v):
    with self._mu:
      self._d[k] = bytes(v)

  def get(self, k):
    with self._mu:
      return self._d[k]

  def check(self, keys):
    with self._mu:
      return all(k in self._d for k in keys)
