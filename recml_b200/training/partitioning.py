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
  """N-D mesh: `axes=[("data", -1), ("model", 2)]`; the batch is split over the first `dp_axes` axes and
  parameters are sharded according to `rules`, a list of `(regex over the dotted parameter name, spec)`
  where `spec` has one mesh-axis name or None per tensor dim (the torch rendering of
  `nn.with_partitioning` + logical→mesh rules, `recml/core/training/partitioning.py:148-288`).

  What the reference leaves to the compiler happens explicitly here.  A sharded parameter exists twice:
  the SHARD (`[out / n, in]` for a spec `("model", None)`) is what the state, the optimizer (so its slots
  are shard-sized) and the checkpoints hold; the model keeps computing with a FULL tensor that is
  re-assembled from the shards (all-gather over the spec's mesh axes) at the start of every step.  After
  backward the full gradient is cut back onto the shard: sliced when the ranks along the axis saw the
  same batch (axis outside the data axes), reduce-scattered when they saw different batches (axis among
  the data axes: fully-sharded data parallelism); the data axes the parameter is not sharded over are
  then averaged.  Layers that are tensor-parallel by construction (`recml_b200.layers.parallel`) own
  their shards already: they are tagged by the layer and only get their mesh placement here.
  """

  def __init__(self, axes: Sequence[tuple[str, int]] = (("batch", -1),), dp_axes: int | None = 1,
               rules: Sequence[tuple[str, Sequence[str | None]]] | None = None, aot_compile: bool = False,
               options: Mapping[str, Any] | None = None, devices: Sequence[Any] | None = None, *,
               device=None, inputs_are_global: bool = False):
    """`aot_compile`, `options` and `devices` are the reference's remaining constructor arguments
    (`recml/core/training/partitioning.py:166-174`): ahead-of-time compilation, compiler options and an explicit
    device list.  There is no compiler here and a process owns the one device it was started on (`device`), so
    they are accepted for experiment files written against the reference and have no effect.  `dp_axes=None`
    makes every axis a data axis, as there."""
    super().__init__(device=device, inputs_are_global=inputs_are_global)
    del aot_compile, options, devices
    if not axes:
      raise ValueError("At least one axis must be specified in `axes`.")
    if dp_axes == 0:
      raise ValueError("Data parallelism axes range must be positive or negative.")
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
    self._sharded: dict[str, tuple[torch.Tensor, torch.Tensor, tuple]] = {}
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

  def axis_size(self, name: str) -> int:
    return self.axis_sizes[self.axis_names.index(name)]

  @property
  def dp_size(self) -> int:
    return int(np.prod([self.axis_size(a) for a in self.dp_axis_names])) if self.dp_axis_names else 1

  def spec_for(self, name: str, ndim: int) -> tuple[str | None, ...] | None:
    for pat, spec in self.rules:
      if pat.search(name):
        if len(spec) != ndim:
          raise ValueError(f"Rule {pat.pattern!r} has {len(spec)} dims, {name} has {ndim}.")
        return spec
    return None

  # -- placement ---------------------------------------------------------------------------------------
  def _grid(self, spec, shard_shape):
    """(global shape, block index, write?) of a shard with mesh spec `spec`; one replica writes it."""
    gshape, index = [], []
    for dim, axis in enumerate(spec):
      n = self.axis_size(axis) if axis is not None else 1
      gshape.append(shard_shape[dim] * n)
      index.append(self.coords[axis] if axis is not None else 0)
    used = {a for a in spec if a is not None}
    write = all(self.coords[a] == 0 for a in self.axis_names if a not in used)
    return tuple(gshape), tuple(index), write

  def _shard_state(self, state: state_lib.State) -> state_lib.State:
    new_params: dict[str, torch.Tensor] = {}
    self._sharded = {}
    with torch.no_grad():
      for name, p in state.params.items():
        tp_spec = getattr(p, "_recml_tp_spec", None)
        if tp_spec is not None:              # a tensor-parallel layer's own shard: placement only
          spec = tuple(tp_spec)
          p._recml_partitioned, p._recml_spec = True, spec
          p._recml_grid = self._grid(spec, tuple(p.shape))
          new_params[name] = p
          continue
        spec = self.spec_for(name, p.ndim)
        if spec is None or all(a is None for a in spec):
          new_params[name] = p
          continue
        piece = p.data
        for dim, axis in enumerate(spec):
          if axis is None:
            continue
          n, i = self.axis_size(axis), self.coords[axis]
          if piece.shape[dim] % n:
            raise ValueError(f"{name} dim {dim} ({piece.shape[dim]}) not divisible by {n}.")
          piece = piece.chunk(n, dim=dim)[i]
        shard = torch.nn.Parameter(piece.contiguous().clone(), requires_grad=p.requires_grad)
        shard._recml_partitioned, shard._recml_spec = True, tuple(spec)
        shard._recml_grid = self._grid(spec, tuple(shard.shape))
        self._sharded[name] = (p, shard, tuple(spec))
        new_params[name] = shard
    state.params = new_params
    if state.optimizer is not None and (self._sharded or any(
        getattr(p, "_recml_partitioned", False) for p in new_params.values())):
      # slots must have the shards' shapes: bind the same update rule to the new parameter set
      state.optimizer = state.optimizer.rebind({n: p for n, p in new_params.items() if p.requires_grad})
      state.optimizer.sq_norm_sync = self._sq_norm_sync
    state.pre_sync = self._scatter_grads
    return state

  # -- per step: shards -> full tensors before compute, full gradients -> shards after backward ----------
  @torch.no_grad()
  def gather_params(self) -> None:
    for full, shard, spec in self._sharded.values():
      piece = shard.data
      for dim in range(len(spec) - 1, -1, -1):
        axis = spec[dim]
        if axis is None or self.axis_size(axis) == 1:
          continue
        parts = [torch.empty_like(piece) for _ in range(self.axis_size(axis))]
        dist.all_gather(parts, piece.contiguous(), group=self._axis_groups[axis])
        piece = torch.cat(parts, dim=dim)
      full.copy_(piece)        # in place and counted: cached bf16 compute copies of `full` notice the change

  @torch.no_grad()
  def _scatter_grads(self, state: state_lib.State) -> None:
    for full, shard, spec in self._sharded.values():
      g = full.grad
      full.grad = None
      if g is None:
        continue
      g = g.to(torch.float32)
      for dim, axis in enumerate(spec):
        if axis is None:
          continue
        n, i = self.axis_size(axis), self.coords[axis]
        if n == 1:
          continue
        if axis in self.dp_axis_names:          # ranks along this axis saw different batches: sum, keep own block
          parts = [c.contiguous() for c in g.chunk(n, dim=dim)]
          out = torch.empty_like(parts[i])
          if dist.get_backend(self._axis_groups[axis]) == "gloo":
            for r in range(n):                 # gloo has no reduce_scatter: n reductions, one kept
              dist.reduce(parts[r], dst=dist.get_global_rank(self._axis_groups[axis], r), group=self._axis_groups[axis])
            out = parts[i]
          else:
            dist.reduce_scatter(out, parts, group=self._axis_groups[axis])
          g = out
        else:                                   # same batch on every rank of the axis: the block is complete
          g = g.chunk(n, dim=dim)[i].contiguous()
      for axis in self.dp_axis_names:           # data axes the parameter is not sharded over
        if axis not in spec and self.axis_size(axis) > 1:
          dist.all_reduce(g, group=self._axis_groups[axis])
      if self.dp_size > 1:
        g = g / self.dp_size
      shard.grad = g.to(shard.dtype)

  def _sq_norm_sync(self, params, grads, sq):
    """Squared gradient norm over ALL shards: the part of `sq` that comes from sharded parameters is summed
    over the mesh axes they are sharded over."""
    by_axes: dict[tuple, torch.Tensor] = {}
    rest = sq.clone()
    for p, g in zip(params, grads):
      spec = getattr(p, "_recml_spec", None)
      axes = tuple(sorted({a for a in (spec or ()) if a is not None and self.axis_size(a) > 1}))
      if not axes:
        continue
      part = (g * g).sum()
      rest = rest - part
      by_axes[axes] = by_axes.get(axes, torch.zeros_like(part)) + part
    for axes, part in by_axes.items():
      for a in axes:
        dist.all_reduce(part, group=self._axis_groups[a])
      rest = rest + part
    return rest

  def all_reduce_grads(self, params: Sequence[torch.Tensor]) -> None:
    """Replicated parameters are averaged over the data group; shards cut from full tensors were averaged
    when their gradients were scattered; a tensor-parallel layer's shards see the same batch along their
    own axis and are averaged over the data group like replicated ones."""
    own = {id(s) for _, s, _ in self._sharded.values()}
    super().all_reduce_grads([p for p in params if id(p) not in own])

  def partition_init(self, init_fn, *, abstract_batch=None):
    def wrapped(batch):
      st = init_fn(batch)
      if dist.is_initialized() and dist.get_world_size() > 1:
        with torch.no_grad():
          for t in list(st.params.values()) + list(st.mutable.values()):
            if getattr(t, "_recml_tp_spec", None) is None:     # a TP layer's shards differ by construction
              dist.broadcast(t, src=0)
      st = self._shard_state(st)
      st.grad_sync = self.all_reduce_grads
      return st
    return wrapped

  def partition_step(self, fn, *, training: bool = False):
    inner = super().partition_step(fn, training=training)

    def step(inputs, state):
      if self._sharded:
        self.gather_params()
      return inner(inputs, state)
    return step
