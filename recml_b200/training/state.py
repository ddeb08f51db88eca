"""Training state: step counter + model parameters + optimizer state.

Plays the role of the reference's `JaxState` / `KerasState`
(`recml/core/training/jax_trainer.py:65-292`).  Those are immutable pytrees because
JAX steps are pure functions; a CUDA step instead updates parameters in place (so
nothing is re-allocated between steps and the step can be replayed from a CUDA graph),
hence `update()` mutates and returns `self`.

Checkpoint tree produced by `state_dict()`:
  step, params/<dotted name>, opt_state/{count, <slot>/<name>}, mutable/<buffer name>,
  sharded/<module path>/...   (per-rank shards of sharded embedding tables)
"""
from __future__ import annotations

from typing import Any, Callable, Mapping

import torch
from torch import nn

from recml_b200.training import optim_factory


def is_sharded_storage(t: torch.Tensor) -> bool:
  """Tensors tagged by the sharded-embedding subsystem are updated inside its fused
  backward kernel and are invisible to the dense optimizer and gradient all-reduce."""
  return bool(getattr(t, "_recml_sharded", False))


class State:
  def __init__(self, *, model: nn.Module | None = None,
               params: Mapping[str, torch.Tensor] | None = None,
               optimizer: optim_factory.Optimizer | None = None, step: int = 0,
               mutable: dict[str, torch.Tensor] | None = None, meta: Any = None):
    self.model = model
    if params is None:
      params = {} if model is None else {
          n: p for n, p in model.named_parameters() if not is_sharded_storage(p)}
    self.params = dict(params)
    self.optimizer = optimizer
    self.step = int(step)
    self.mutable = mutable if mutable is not None else (
        {} if model is None else {n: b for n, b in model.named_buffers()
                                  if not is_sharded_storage(b)})
    self.meta = meta
    # Installed by a partitioner: called with the list of params between backward and the
    # optimizer step (data-parallel gradient all-reduce).
    self.grad_sync: Callable[[list[torch.Tensor]], None] | None = None
    # Installed by a partitioner with sharded parameters: moves the gradients of the gathered (full)
    # tensors the model computed with onto the shards the optimizer owns.
    self.pre_sync: Callable[["State"], None] | None = None

  @classmethod
  def create(cls, *, model: nn.Module | None = None, params=None,
             tx: optim_factory.OptimizerBuilder | None = None, step: int = 0,
             mutable=None, meta=None) -> "State":
    st = cls(model=model, params=params, optimizer=None, step=step, mutable=mutable, meta=meta)
    if tx is not None:
      st.optimizer = tx.init({n: p for n, p in st.params.items() if p.requires_grad})
    return st

  # -- step ---------------------------------------------------------------------
  def update(self, *, grads: Mapping[str, torch.Tensor] | None = None,
             mutable: dict[str, torch.Tensor] | None = None) -> "State":
    """Synchronises gradients, applies the optimizer and advances `step`."""
    if self.optimizer is None:
      raise ValueError("State has no optimizer; create it with `tx=`.")
    if grads is not None:
      for n, g in grads.items():
        self.params[n].grad = g
    if self.pre_sync is not None:
      self.pre_sync(self)
    on_cuda = any(p.is_cuda for p in self.optimizer.params[:1])
    if on_cuda:
      # weight gradients queued during backward (`ops.dense`) run on their own stream; they must be in
      # `.grad` before the gradients are synchronised and applied
      from recml_b200.ops import dense as dense_ops
      dense_ops.join_deferred()
    if self.grad_sync is not None:
      self.grad_sync([p for p in self.optimizer.params if p.grad is not None])
    self.optimizer.step()
    self.optimizer.zero_grad()
    if on_cuda:
      # side streams of the step (embedding backward, occurrence sort) end here, so the step is one unit
      # for whoever comes next on this stream (the next step, a checkpoint, a CUDA-graph capture)
      from recml_b200.utils import streams
      streams.join()
    if mutable is not None:
      self.mutable.update(mutable)
    self.step += 1
    return self

  def __call__(self, *args, **kwargs):
    return self.model(*args, **kwargs)

  def apply(self, *args, **kwargs):
    """Runs the model on the state's parameters (`JaxState.apply`, `recml/core/training/jax_trainer.py:105-107`):
    the module holds them, so this is the module call."""
    return self.model(*args, **kwargs)

  def sync_model_variables(self) -> None:
    """`KerasState.sync_model_variables` copies the state's arrays back into the Keras model
    (`recml/core/training/jax_trainer.py:277-288`).  Here the state's parameters ARE the module's tensors, so there
    is nothing to copy; the method exists for tasks written against the reference."""

  @property
  def opt_state(self) -> dict[str, Any]:
    """The optimizer's slots by name (`recml/core/training/jax_trainer.py:60-62`); empty without an optimizer."""
    return {} if self.optimizer is None else self.optimizer.state_dict()

  # -- introspection (logged by the trainer) ----------------------------------------
  def num_trainable(self) -> int:
    return sum(p.numel() for p in self.params.values() if p.requires_grad)

  def num_non_trainable(self) -> int:
    return (sum(p.numel() for p in self.params.values() if not p.requires_grad)
            + sum(b.numel() for b in self.mutable.values()))

  # -- checkpoint tree -------------------------------------------------------------
  def sharded_modules(self) -> dict[str, nn.Module]:
    if self.model is None:
      return {}
    return {n: m for n, m in self.model.named_modules() if hasattr(m, "sharded_state_dict")}

  def state_dict(self) -> dict[str, Any]:
    sd: dict[str, Any] = {
        "step": torch.tensor(self.step, dtype=torch.int64),
        "params": {n: _leaf_of(p, p.detach()) for n, p in self.params.items()},
        "mutable": {n: b.detach() for n, b in self.mutable.items()},
    }
    if self.optimizer is not None:
      sd["opt_state"] = self.optimizer.state_dict()
      by_name = dict(zip(self.optimizer.names, self.optimizer.params))
      for slot, entries in sd["opt_state"].items():
        if isinstance(entries, dict):
          sd["opt_state"][slot] = {n: _leaf_of(by_name.get(n), t) for n, t in entries.items()}
    sharded = {n or "root": m.sharded_state_dict() for n, m in self.sharded_modules().items()}
    if sharded:
      sd["sharded"] = sharded
    return sd

  @torch.no_grad()
  def load_state_dict(self, sd: Mapping[str, Any], *, restore_optimizer: bool = True,
                      restore_step: bool = True) -> "State":
    for n, p in self.params.items():
      p.copy_(torch.as_tensor(sd["params"][n]).to(p.dtype))
    for n, b in self.mutable.items():
      if n in sd.get("mutable", {}):
        b.copy_(torch.as_tensor(sd["mutable"][n]).to(b.dtype))
    if restore_optimizer and self.optimizer is not None and "opt_state" in sd:
      self.optimizer.load_state_dict(sd["opt_state"])
    for n, m in self.sharded_modules().items():
      m.load_sharded_state_dict(sd["sharded"][n or "root"])
    if restore_step:
      self.step = int(sd["step"])
    return self


def _leaf_of(param, tensor):
  """Checkpoint leaf for `tensor` (a parameter or one of its optimizer slots): a block of a global array
  when the parameter is a shard placed by a partitioner, the tensor itself otherwise."""
  grid = getattr(param, "_recml_grid", None)
  if grid is None or tensor.shape != param.shape:
    return tensor
  from recml_b200.ckpt.manager import ShardedLeaf
  global_shape, index, write = grid
  return ShardedLeaf(tensor.detach(), global_shape, index, tuple(tensor.shape), write=write)


# Names of the reference API (`recml/__init__.py:19-40`).
JaxState = State
KerasState = State
