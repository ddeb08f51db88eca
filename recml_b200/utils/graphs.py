"""CUDA-graph capture of a whole training step.

The reference hands the step to a tracing compiler (`jax.jit` in `recml/core/training/
partitioning.py:128-145`).  Here the step is ordinary eager code whose kernels all take their
per-step varying values from device memory (sequence numbers of peer flags are ticked on the
device, optimizer hyper-parameters sit in a small device struct), so a step can be recorded
once into a CUDA graph and replayed with a single launch — which is what keeps an 8-GPU job with
a small per-GPU batch from being bound by Python and launch overhead.

Objects that keep per-step state on the host register here:
  graph_snapshot() / graph_restore(s)   capture runs the Python code without executing kernels, so
                                        host counters are rolled back afterwards
  graph_advance()                       what one executed step does to the host counters
  graph_pre_replay()                    refresh device-side hyper-parameters before a replay
Two graphs are recorded (for even and odd steps) because peer-visible buffers are
double-buffered by step parity and buffer addresses are baked into a graph.
"""
from __future__ import annotations

import weakref
from typing import Any, Callable

import torch

_REGISTRY: "weakref.WeakSet[Any]" = weakref.WeakSet()
_capturing = [False]


def register(obj: Any) -> None:
  _REGISTRY.add(obj)


def capturing() -> bool:
  return _capturing[0]


def _participants():
  return [o for o in list(_REGISTRY)]


def _tree_tensors(tree, out):
  if isinstance(tree, torch.Tensor):
    out.append(tree)
  elif isinstance(tree, dict):
    for v in tree.values():
      _tree_tensors(v, out)
  elif isinstance(tree, (list, tuple)):
    for v in tree:
      _tree_tensors(v, out)
  elif hasattr(tree, "values") and hasattr(tree, "offsets"):   # KeyedJagged
    out.append(tree.values)
    out.append(tree.offsets)
    if tree.weights is not None:
      out.append(tree.weights)
  return out


def _clone_tree(tree, fast: bool = False):
  """Deep copy of the tensors of a tree.  `fast` gathers all tensors of a dtype with ONE concatenation kernel
  and hands out views of the result instead of one memcpy each (a step returns ~16 tiny metric tensors, and 16
  launches between two graph replays are a visible share of a 3 ms step)."""
  if fast:
    src = _leaf_tensors(tree, [])
    if src:
      dst: list = [None] * len(src)
      groups: dict = {}
      for i, t in enumerate(src):
        groups.setdefault((t.dtype, t.device), []).append(i)
      for idxs in groups.values():
        if len(idxs) == 1:
          dst[idxs[0]] = src[idxs[0]].clone()
          continue
        flat = torch.cat([src[i].reshape(-1) for i in idxs])
        at = 0
        for i in idxs:
          n = src[i].numel()
          dst[i] = flat[at:at + n].view(src[i].shape)
          at += n
      it = iter(dst)
      return _rebuild(tree, it)
  return _clone_slow(tree)


def _leaf_tensors(tree, out):
  """Every tensor reachable through dicts, sequences, jagged batches and metric dataclasses."""
  if isinstance(tree, torch.Tensor):
    out.append(tree)
  elif isinstance(tree, dict):
    for v in tree.values():
      _leaf_tensors(v, out)
  elif isinstance(tree, (list, tuple)):
    for v in tree:
      _leaf_tensors(v, out)
  elif hasattr(tree, "values") and hasattr(tree, "offsets"):
    _tree_tensors(tree, out)
  elif hasattr(tree, "replace") and hasattr(tree, "__dataclass_fields__"):
    import dataclasses
    for f in dataclasses.fields(tree):
      _leaf_tensors(getattr(tree, f.name), out)
  return out


def _rebuild(tree, it):
  """Same structure as `tree` with its tensors replaced, in `_leaf_tensors` order, by those of `it`."""
  if isinstance(tree, torch.Tensor):
    return next(it)
  if isinstance(tree, dict):
    items = {k: _rebuild(v, it) for k, v in tree.items()}
    return items if type(tree) is dict else type(tree)(items)
  if isinstance(tree, (list, tuple)):
    return type(tree)(_rebuild(v, it) for v in tree)
  if hasattr(tree, "values") and hasattr(tree, "offsets"):
    import dataclasses
    vals, offs = next(it), next(it)
    return dataclasses.replace(tree, values=vals, offsets=offs, weights=None if tree.weights is None else next(it))
  if hasattr(tree, "replace") and hasattr(tree, "__dataclass_fields__"):
    import dataclasses
    return tree.replace(**{f.name: _rebuild(getattr(tree, f.name), it) for f in dataclasses.fields(tree)})
  return tree


def _clone_slow(tree):
  if isinstance(tree, torch.Tensor):
    return tree.clone()
  if isinstance(tree, dict):
    return type(tree)({k: _clone_slow(v) for k, v in tree.items()}) if type(tree) is not dict else \
        {k: _clone_slow(v) for k, v in tree.items()}
  if isinstance(tree, (list, tuple)):
    return type(tree)(_clone_slow(v) for v in tree)
  if hasattr(tree, "values") and hasattr(tree, "offsets"):
    import dataclasses
    return dataclasses.replace(tree, values=tree.values.clone(), offsets=tree.offsets.clone(),
                               weights=None if tree.weights is None else tree.weights.clone())
  if hasattr(tree, "replace") and hasattr(tree, "__dataclass_fields__"):   # metric states
    import dataclasses
    return tree.replace(**{f.name: _clone_slow(getattr(tree, f.name)) for f in dataclasses.fields(tree)})
  return tree


class GraphedStep:
  """Wraps `fn(inputs, state) -> (state, outputs)`.  The first `warmup` calls run eagerly; then two
  graphs are captured with the inputs of that moment as static buffers; later calls copy the new
  inputs into the static buffers and replay.  Inputs must keep their shapes."""

  def __init__(self, fn: Callable, warmup: int = 3):
    self.fn = fn
    self.warmup = warmup
    self.calls = 0
    self.graphs: list[torch.cuda.CUDAGraph] = []
    self.static_inputs: list[Any] = []
    self.static_outputs: list[Any] = []
    self.kernels_per_replay: list[int] = []
    self.phase = 0
    self.pool = None
    # Warm-up steps run on the stream that later records the graphs: autograd's gradient-accumulation
    # nodes remember the stream they were created on, and capture fails if that is the default one.
    self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None

  def _capture(self, inputs, state):
    parts = _participants()
    torch.cuda.synchronize()
    snaps = [(o, o.graph_snapshot()) for o in parts if hasattr(o, "graph_snapshot")]
    step0 = state.step
    import gc
    gc.collect()
    stream = self.stream
    stream.wait_stream(torch.cuda.current_stream())
    _capturing[0] = True
    try:
      from recml_b200.ops import _lib
      for _ in range(2):
        static_in = _clone_tree(inputs)
        g = torch.cuda.CUDAGraph()
        before = _lib.LAUNCHES["count"]
        with torch.cuda.graph(g, pool=self.pool, stream=stream):
          _, out = self.fn(static_in, state)
        # kernels of this library recorded into the graph: every replay launches them again
        self.kernels_per_replay.append(_lib.LAUNCHES["count"] - before)
        _lib.LAUNCHES["count"] = before
        self.pool = g.pool()
        self.graphs.append(g)
        self.static_inputs.append(static_in)
        self.static_outputs.append(out)
    finally:
      _capturing[0] = False
    # capture ran the Python of two steps without executing any kernel: roll the host state back
    for o, s in snaps:
      o.graph_restore(s)
    state.step = step0
    torch.cuda.current_stream().wait_stream(stream)

  def __call__(self, inputs, state):
    self.calls += 1
    if not torch.cuda.is_available():
      return self.fn(inputs, state)
    if self.calls <= self.warmup:
      cur = torch.cuda.current_stream()
      self.stream.wait_stream(cur)
      with torch.cuda.stream(self.stream):
        out = self.fn(inputs, state)
      cur.wait_stream(self.stream)
      return out
    if not self.graphs:
      self._capture(inputs, state)
    i = self.phase
    self.phase ^= 1
    dst, src = _tree_tensors(self.static_inputs[i], []), _tree_tensors(inputs, [])
    for d, s in zip(dst, src):
      if d.shape != s.shape:
        raise ValueError(f"graphed step needs fixed input shapes, got {tuple(s.shape)} vs {tuple(d.shape)}")
    if all(s.is_cuda for s in src):
      torch._foreach_copy_(dst, src)   # pylint: disable=protected-access
    else:
      for d, s in zip(dst, src):
        d.copy_(s, non_blocking=True)
    parts = _participants()
    for o in parts:
      if hasattr(o, "graph_pre_replay"):
        o.graph_pre_replay()
    self.graphs[i].replay()
    from recml_b200.ops import _lib
    _lib.LAUNCHES["count"] += self.kernels_per_replay[i]
    for o in parts:
      if hasattr(o, "graph_advance"):
        o.graph_advance()
    state.step += 1
    return state, _clone_tree(self.static_outputs[i], fast=True)
