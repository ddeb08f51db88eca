"""Partitioners: how a step is spread over the GPUs of the job.

Reference: `recml/core/training/partitioning.py:33-288` builds jit-ed functions with
input/output shardings over a device mesh and lets the compiler insert collectives.
Here each process owns one GPU, so a partitioner (1) moves this rank's batch slice to
the device through pinned memory, (2) lays out the initial state (broadcast replicated
parameters, slice sharded ones) and (3) installs the gradient synchronisation that
runs between backward and the optimizer step.
"""
from __future__ import annotations

import abc
import re
from typing import Any, Callable, Mapping, Sequence

import numpy as np
import torch
import torch.distributed as dist

from recml_b200.training import state as state_lib


def _tree_map(fn, tree):
  if isinstance(tree, dict):
    return {k: _tree_map(fn, v) for k, v in tree.items()}
  if isinstance(tree, (list, tuple)):
    out = [_tree_map(fn, v) for v in tree]
    return type(tree)(*out) if hasattr(tree, "_fields") else type(tree)(out)
  return fn(tree)


def default_device() -> torch.device:
  if torch.cuda.is_available():
    return torch.device("cuda", torch.cuda.current_device())
  return torch.device("cpu")


class _PinnedStager:
  """Reusable pinned host buffers so every H2D copy is asynchronous.

  A buffer is handed out again only after the copy that last read it has finished: `put` records
  an event behind the copy, and a buffer whose event is still pending is skipped (a new one is
  allocated, up to `max_per_key` per shape; beyond that the host waits for the oldest copy).
  Tensors of equal shape inside one batch therefore never share a buffer, however far the host
  runs ahead of the device.
  """

  def __init__(self, max_per_key: int = 16):
    self._bufs: dict[tuple, list[list]] = {}
    self.max_per_key = max_per_key

  def put(self, t: torch.Tensor, device: torch.device) -> torch.Tensor:
    """Pageable host tensor → device tensor through a pinned buffer (pinned inputs go directly)."""
    if t.is_pinned():
      return t.to(device, non_blocking=True)
    key = (tuple(t.shape), t.dtype)
    ring = self._bufs.setdefault(key, [])
    slot = next((s for s in ring if s[1] is None or s[1].query()), None)
    if slot is None:
      if len(ring) < self.max_per_key:
        slot = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True), None]
        ring.append(slot)
      else:
        slot = ring.pop(0)          # oldest copy: wait for it, then recycle its buffer
        slot[1].synchronize()
        ring.append(slot)
    slot[0].copy_(t)
    out = slot[0].to(device, non_blocking=True)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(device))
    slot[1] = ev
    return out


class Partitioner(abc.ABC):
  @abc.abstractmethod
  def shard_inputs(self, inputs: Any) -> Any:
    """Host batch → this rank's device-resident batch."""

  @abc.abstractmethod
  def partition_init(self, init_fn: Callable[[Any], state_lib.State], *,
                     abstract_batch: Any | None = None) -> Callable[[Any], state_lib.State]:
    """Wraps the state-creating function."""

  @abc.abstractmethod
  def partition_step(self, fn: Callable, *, training: bool = False) -> Callable:
    """Wraps the train / eval step."""


class NullPartitioner(Partitioner):
  """Single device, no communication."""

  def __init__(self, device: torch.device | str | None = None):
    self.device = torch.device(device) if device is not None else default_device()
    self._stager = _PinnedStager()

  def _put(self, x):
    if hasattr(x, "to_device") and not isinstance(x, (np.ndarray, torch.Tensor)):
      return x.to_device(self.device, self._stager if self.device.type == "cuda" else None)
    if isinstance(x, np.ndarray):
      x = torch.from_numpy(np.ascontiguousarray(x))
    if not isinstance(x, torch.Tensor):
      return x
    if self.device.type == "cuda" and not x.is_cuda:
      return self._stager.put(x, self.device)
    return x.to(self.device)

  def shard_inputs(self, inputs: Any) -> Any:
    return _tree_map(self._put, inputs)

  def partition_init(self, init_fn, *, abstract_batch=None):
    return init_fn

  def partition_step(self, fn, *, training: bool = False):
    return fn


class DataParallelPartitioner(NullPartitioner):
  """Batch split over all ranks; dense state replicated; gradients averaged.

  `inputs_are_global=False` (default) means every process already feeds its own slice
  (per-process batch = global / world, `recml/core/data/tf_dataset_factory.py:79-92`);
  with True the leading dim is sliced by rank.  Gradient averaging uses the fused
  cast+scale all-reduce kernel on NVLink when available, else `dist.all_reduce`.
  """

  def __init__(self, data_axis: str = "batch", *, group: Any = None,
               inputs_are_global: bool = False, device=None, grad_dtype: torch.dtype | None = None,
               use_cuda_graph: bool = False, graph_warmup_steps: int = 3,
               overlap_grad_reduce: bool = True):
    super().__init__(device)
    self.overlap_grad_reduce = overlap_grad_reduce
    self.use_cuda_graph = use_cuda_graph
    self.graph_warmup_steps = graph_warmup_steps
    self.data_axis = data_axis
    self.group = group
    self.inputs_are_global = inputs_are_global
    self.grad_dtype = grad_dtype
    self._reducer = None

  @property
  def world(self) -> int:
    return dist.get_world_size(self.group) if dist.is_initialized() else 1

  @property
  def rank(self) -> int:
    return dist.get_rank(self.group) if dist.is_initialized() else 0

  def shard_inputs(self, inputs: Any) -> Any:
    if self.inputs_are_global and self.world > 1:
      w, r = self.world, self.rank

      def cut(x):
        if hasattr(x, "slice_batch"):
          b = x.batch_size()
          return x.slice_batch(r * b // w, (r + 1) * b // w)
        if isinstance(x, (np.ndarray, torch.Tensor)) and x.ndim >= 1:
          b = x.shape[0]
          return x[r * b // w:(r + 1) * b // w]
        return x
      inputs = _tree_map(cut, inputs)
    return super().shard_inputs(inputs)

  def _get_reducer(self):
    if self._reducer is None:
      from recml_b200.comm import grad_reducer
      self._reducer = grad_reducer.make_reducer(self.group, self.device)
    return self._reducer

  def all_reduce_grads(self, params: Sequence[torch.Tensor]) -> None:
    if self.world == 1 or not params:
      return
    self._get_reducer().average_grads(params)

  def _attach_overlap(self, state: state_lib.State) -> None:
    """Lets the fused reducer start each gradient bucket from a hook inside backward, so the
    exchange runs under the rest of the backward pass (the embedding update above all)."""
    if self.world == 1 or not self.overlap_grad_reduce or state.optimizer is None:
      return
    reducer = self._get_reducer()
    params = [p for p in state.optimizer.params if p.requires_grad]
    if hasattr(reducer, "attach") and params:
      reducer.attach(params)

  def _replicate(self, state: state_lib.State) -> state_lib.State:
    if self.world > 1:
      with torch.no_grad():
        for t in list(state.params.values()) + list(state.mutable.values()):
          if not getattr(t, "_recml_partitioned", False):
            dist.broadcast(t, src=dist.get_global_rank(self.group, 0) if self.group else 0,
                           group=self.group)
    state.grad_sync = self.all_reduce_grads
    self._attach_overlap(state)
    return state

  def partition_init(self, init_fn, *, abstract_batch=None):
    def wrapped(batch):
      return self._replicate(init_fn(batch))
    return wrapped


  def partition_step(self, fn, *, training: bool = False):
    """With `use_cuda_graph` the training step is recorded into CUDA graphs after a few eager
    warm-up steps and replayed afterwards (fixed input shapes required)."""
    if training and self.use_cuda_graph and self.device.type == "cuda":
      from recml_b200.utils import graphs
      return graphs.GraphedStep(fn, warmup=self.graph_warmup_steps)
    return fn


class ModelParallelPartitioner(DataParallelPartitioner):
  """N-D mesh: `axes=[("data", -1), ("model", 2)]`; the batch is split over `dp_axes`
  and parameters are sharded according to `rules`, a list of `(regex over the dotted
  parameter name, spec)` where `spec` has one mesh-axis name or None per tensor dim
  (the torch rendering of `nn.with_partitioning` + logical→mesh rules,
  `partitioning.py:148-288`).  Sharded parameters are cut in place at init and tagged
  `_recml_partitioned`; their gradients are reduced over the data axes only.
  """

  def __init__(self, axes: Sequence[tuple[str, int]], dp_axes: int = 1,
               rules: Sequence[tuple[str, Sequence[str | None]]] | None = None, *,
               device=None, inputs_are_global: bool = False):
    super().__init__(device=device, inputs_are_global=inputs_are_global)
    world = dist.get_world_size() if dist.is_initialized() else 1
    names = [a for a, _ in axes]
    sizes = [s for _, s in axes]
    if sizes.count(-1) > 1:
      raise ValueError("At most one mesh axis may have size -1.")
    known = int(np.prod([s for s in sizes if s != -1])) if sizes else 1
    sizes = [world // known if s == -1 else s for s in sizes]
    if int(np.prod(sizes)) != world:
      raise ValueError(f"Mesh {list(zip(names, sizes))} does not cover {world} ranks.")
    self.axis_names, self.axis_sizes = names, sizes
    self.dp_axis_names = names[:dp_axes]
    self.rules = [(re.compile(p), tuple(s)) for p, s in (rules or [])]
    self.mesh = np.arange(world).reshape(sizes)
    me = dist.get_rank() if dist.is_initialized() else 0
    self.coords = dict(zip(names, (int(c[0]) for c in np.where(self.mesh == me))))
    self._axis_groups: dict[str, Any] = {}
    if dist.is_initialized() and world > 1:
      for ai, name in enumerate(names):
        moved = np.moveaxis(self.mesh, ai, -1).reshape(-1, sizes[ai])
        for ranks in moved:  # every rank must create every subgroup, in the same order
          g = dist.new_group([int(r) for r in ranks])
          if me in ranks:
            self._axis_groups[name] = g
      # one group spanning all data axes, used for the batch split and gradient mean
      dp_idx = [names.index(n) for n in self.dp_axis_names]
      rest = [i for i in range(len(names)) if i not in dp_idx]
      moved = np.transpose(self.mesh, rest + dp_idx).reshape(
          -1, int(np.prod([sizes[i] for i in dp_idx])))
      for ranks in moved:
        g = dist.new_group([int(r) for r in ranks])
        if me in ranks:
          self.group = g

  def axis_group(self, name: str):
    return self._axis_groups.get(name)

  def spec_for(self, name: str, ndim: int) -> tuple[str | None, ...] | None:
    for pat, spec in self.rules:
      if pat.search(name):
        if len(spec) != ndim:
          raise ValueError(f"Rule {pat.pattern!r} has {len(spec)} dims, {name} has {ndim}.")
        return spec
    return None

  def _shard_state(self, state: state_lib.State) -> state_lib.State:
    with torch.no_grad():
      for name, p in state.params.items():
        spec = getattr(p, "_recml_spec", None) or self.spec_for(name, p.ndim)
        if spec is None:
          continue
        piece = p.data
        for dim, axis in enumerate(spec):
          if axis is None:
            continue
          n, i = self.axis_sizes[self.axis_names.index(axis)], self.coords[axis]
          if piece.shape[dim] % n:
            raise ValueError(f"{name} dim {dim} ({piece.shape[dim]}) not divisible by {n}.")
          piece = piece.chunk(n, dim=dim)[i]
        p.data = piece.contiguous()
        p._recml_partitioned = True
        p._recml_spec = tuple(spec)
    return state

  def partition_init(self, init_fn, *, abstract_batch=None):
    def wrapped(batch):
      st = init_fn(batch)
      if self.world > 1 or (dist.is_initialized() and dist.get_world_size() > 1):
        src = 0
        with torch.no_grad():
          for t in list(st.params.values()) + list(st.mutable.values()):
            dist.broadcast(t, src=src)
      st = self._shard_state(st)
      st.grad_sync = self.all_reduce_grads
      return st
    return wrapped
