"""Step annotations, device timers and progress reporting.

Stands in for the reference's profiler hooks: `jax.profiler.StepTraceAnnotation`
around every step (`recml/core/training/jax_trainer.py:570,623`), named scopes around
kernels, and CLU's `ReportProgress` with `.timed("checkpointing" | "eval")` shares
(`jax_trainer.py:496-501,526,769`).  On CUDA the annotations are NVTX ranges, phase
timers use CUDA events on the launching stream, and `trace()` exports a
`torch.profiler` Chrome trace.
"""
from __future__ import annotations

import collections
import contextlib
import logging as pylogging
import time

import torch

log = pylogging.getLogger("recml_b200.profiling")


@contextlib.contextmanager
def step_annotation(name: str, step_num: int):
  if torch.cuda.is_available():
    torch.cuda.nvtx.range_push(f"{name}:{step_num}")
    try:
      yield
    finally:
      torch.cuda.nvtx.range_pop()
  else:
    yield


@contextlib.contextmanager
def named_scope(name: str):
  if torch.cuda.is_available():
    torch.cuda.nvtx.range_push(name)
    try:
      yield
    finally:
      torch.cuda.nvtx.range_pop()
  else:
    yield


class DeviceStepTimer:
  """Elapsed device time between `start()` and `stop()` on the current stream."""

  def __init__(self, enabled: bool = True):
    self.enabled = enabled and torch.cuda.is_available()
    self._start = None

  def start(self):
    if self.enabled:
      self._start = torch.cuda.Event(enable_timing=True)
      self._start.record()

  def stop(self) -> float | None:
    if not self.enabled or self._start is None:
      return None
    end = torch.cuda.Event(enable_timing=True)
    end.record()
    end.synchronize()
    return self._start.elapsed_time(end)


class PhaseTimers:
  """Per-phase CUDA-event timers (id exchange / lookup / dense fwd / dense bwd /
  embedding bwd / all-reduce / optimizer).  `summary()` synchronises once."""

  def __init__(self, enabled: bool = True):
    self.enabled = enabled and torch.cuda.is_available()
    self._pairs: dict[str, list] = collections.defaultdict(list)

  @contextlib.contextmanager
  def phase(self, name: str):
    if not self.enabled:
      yield
      return
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    with named_scope(name):
      yield
    b.record()
    self._pairs[name].append((a, b))

  def summary(self) -> dict[str, float]:
    if not self.enabled:
      return {}
    torch.cuda.synchronize()
    out = {k: sum(a.elapsed_time(b) for a, b in v) / max(len(v), 1)
           for k, v in self._pairs.items()}
    self._pairs.clear()
    return out


class ReportProgress:
  """steps/sec every call window + wall-clock share of timed side activities.  With a summary `writer` the
  window also closes every `every_steps` steps and `steps_per_sec` / `uptime` go out as scalars, like the
  periodic action the reference's trainer runs after each step (`recml/core/training/jax_trainer.py:496-501,583`).
  """

  def __init__(self, every_secs: float = 60.0, *, writer=None, every_steps: int | None = None):
    self._every = every_secs
    self._every_steps = every_steps
    self._writer = writer
    self._t0 = self._last_t = time.time()
    self._last_step = None
    self._timed: dict[str, float] = collections.defaultdict(float)
    self.steps_per_sec: float | None = None

  def __call__(self, step: int) -> None:
    now = time.time()
    if self._last_step is None:
      self._last_step, self._last_t = step, now
      return
    due = now - self._last_t >= self._every
    if self._every_steps is not None and step - self._last_step >= self._every_steps:
      due = True
    if due and step > self._last_step:
      dt = max(now - self._last_t, 1e-9)
      self.steps_per_sec = (step - self._last_step) / dt
      shares = ", ".join(f"{k}: {100 * v / dt:.1f}%" for k, v in self._timed.items())
      log.info("step %d | %.2f steps/s | %s", step, self.steps_per_sec, shares)
      if self._writer is not None:
        self._writer.write_scalars(step, {"steps_per_sec": self.steps_per_sec, "uptime": now - self._t0})
      self._timed.clear()
      self._last_step, self._last_t = step, now

  @contextlib.contextmanager
  def timed(self, name: str):
    t = time.time()
    try:
      yield
    finally:
      self._timed[name] += time.time() - t


@contextlib.contextmanager
def trace(path: str, enabled: bool = True):
  """Chrome-trace export of everything inside the block."""
  if not enabled:
    yield
    return
  acts = [torch.profiler.ProfilerActivity.CPU]
  if torch.cuda.is_available():
    acts.append(torch.profiler.ProfilerActivity.CUDA)
  with torch.profiler.profile(activities=acts) as prof:
    yield
  prof.export_chrome_trace(path)


def kernel_timeline(step_fn, path: str, *, steps: int = 4, pick: int = 2, top: int = 40) -> dict:
  """Runs `step_fn` `steps` times under the profiler's CUDA activity records and writes, for step `pick`:
  the total duration and launch count per kernel name (the `top` largest), then every kernel in launch order
  with its start offset and duration in microseconds.  Returns {"kernels_per_step", "span_us", "busy_us"}.
  The steps must launch the same kernels each time (a steady-state training step does)."""
  import collections
  from torch.profiler import ProfilerActivity, profile
  with profile(activities=[ProfilerActivity.CUDA]) as prof:
    for _ in range(steps):
      step_fn()
    torch.cuda.synchronize()
  events = [e for e in prof.profiler.kineto_results.events() if str(e.device_type()).endswith("CUDA")]
  events.sort(key=lambda e: e.start_ns())
  per = len(events) // steps
  seg = events[pick * per:(pick + 1) * per]
  if not seg:
    raise RuntimeError("the profiler recorded no CUDA activity")
  t0 = seg[0].start_ns()
  span = (max(e.start_ns() + e.duration_ns() for e in seg) - t0) / 1e3
  busy = sum(e.duration_ns() for e in seg) / 1e3
  total, count = collections.Counter(), collections.Counter()
  for e in seg:
    total[e.name()[:90]] += e.duration_ns() / 1e3
    count[e.name()[:90]] += 1
  with open(path, "w") as f:
    f.write(f"kernels/step {per}; span {span:.0f} us; busy {busy:.0f} us\n")
    for name, us in total.most_common(top):
      f.write(f"{us:9.1f} us x{count[name]:4d}  {name}\n")
    f.write("----\n")
    for e in seg:
      f.write(f"{(e.start_ns() - t0) / 1e3:9.1f} +{e.duration_ns() / 1e3:8.1f} {e.name()[:110]}\n")
  return {"kernels_per_step": per, "span_us": span, "busy_us": busy}
