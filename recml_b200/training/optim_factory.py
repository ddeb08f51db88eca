"""Dense-parameter optimizers built from dataclass factories.

Same fields and numerics as the reference factories (`recml/core/training/
optax_factory.py:44-213`, contract pinned by `optax_factory_test.py:48-161`):

  update = -lr(step) · ( scale(clip_global_norm(g)) + weight_decay·w·mask )

with `scale` = identity (SGD), Adam moments, or root-sum-of-squares (Adagrad).  Unlike
the reference, `freeze_mask` works: matching parameters receive no update.
On CUDA tensors the whole chain runs as ONE fused multi-tensor kernel per bucket
(`recml_b200.ops.multi_tensor_optim`); on CPU the same math runs as torch foreach ops.
"""
from __future__ import annotations

import dataclasses
import math
import re
from typing import Any, Callable, Iterable, Mapping

import torch

from recml_b200.utils import types

Schedule = Callable[[int], float]
Mask = str | Callable[[str, torch.Tensor], bool]


def default_weight_decay_mask(name: str, p: torch.Tensor) -> bool:
  """Decay matrices, not biases / norm scales (`optax_factory.py:26-28`)."""
  del name
  return p.ndim > 1


def _as_mask(mask: Mask | None) -> Callable[[str, torch.Tensor], bool] | None:
  if mask is None:
    return None
  if isinstance(mask, str):
    pattern = re.compile(mask)
    return lambda name, p: pattern.fullmatch(name) is not None or pattern.search(name) is not None
  return mask


def warmup_cosine_decay_schedule(init_value: float, peak_value: float, warmup_steps: int,
                                 decay_steps: int, end_value: float = 0.0) -> Schedule:
  """Linear warm-up then cosine decay; `decay_steps` counts from step 0 (optax semantics)."""
  def fn(step: int) -> float:
    if step < warmup_steps:
      return init_value + (peak_value - init_value) * step / max(warmup_steps, 1)
    t = min(max(step - warmup_steps, 0) / max(decay_steps - warmup_steps, 1), 1.0)
    return end_value + (peak_value - end_value) * 0.5 * (1.0 + math.cos(math.pi * t))
  return fn


@dataclasses.dataclass
class Scaling:
  """Gradient pre-conditioner: kind ∈ {"identity", "adam", "rss"}."""
  kind: str = "identity"
  b1: float = 0.9
  b2: float = 0.999
  eps: float = 1e-8
  initial_accumulator_value: float = 0.1


def scale_by_adam(b1=0.9, b2=0.999, eps=1e-8) -> Scaling:
  return Scaling("adam", b1=b1, b2=b2, eps=eps)


def scale_by_rss(initial_accumulator_value=0.1, eps=1e-7) -> Scaling:
  return Scaling("rss", eps=eps, initial_accumulator_value=initial_accumulator_value)


def identity() -> Scaling:
  return Scaling("identity")


class Optimizer:
  """A configured update rule bound to named parameters.

  `hyperparams["learning_rate"]` is refreshed on every step so trainers can log it
  (the reference exposes it through `inject_stateful_hyperparams`).
  """

  def __init__(self, named_params: Mapping[str, torch.Tensor] | Iterable[tuple[str, torch.Tensor]],
               *, learning_rate: float | Schedule, scaling: Scaling, weight_decay: float | None,
               grad_clip_norm: float | None, weight_decay_mask: Mask, freeze_mask: Mask | None):
    items = list(named_params.items()) if isinstance(named_params, Mapping) else list(named_params)
    # kept so that a partitioner can bind the same update rule to the shards of the parameters
    self._config = dict(learning_rate=learning_rate, scaling=scaling, weight_decay=weight_decay,
                        grad_clip_norm=grad_clip_norm, weight_decay_mask=weight_decay_mask, freeze_mask=freeze_mask)
    # set by a partitioner whose parameters are sharded: sums a squared-norm over the ranks that hold the
    # other shards, so that global-norm clipping sees the whole gradient
    self.sq_norm_sync = None
    freeze = _as_mask(freeze_mask)
    wd_mask = _as_mask(weight_decay_mask) or default_weight_decay_mask
    self.names = [n for n, p in items if not (freeze and freeze(n, p))]
    self.params = [p for n, p in items if not (freeze and freeze(n, p))]
    self.frozen = [n for n, p in items if freeze and freeze(n, p)]
    self.lr = learning_rate
    self.scaling = scaling
    self.weight_decay = weight_decay
    self.grad_clip_norm = grad_clip_norm
    self.decay_flags = [bool(weight_decay is not None and wd_mask(n, p))
                        for n, p in zip(self.names, self.params)]
    self.count = 0
    self.hyperparams: dict[str, float] = {"learning_rate": self._lr_at(0)}
    self.slots: dict[str, list[torch.Tensor]] = {}
    if scaling.kind == "adam":
      self.slots["mu"] = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
      self.slots["nu"] = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
    elif scaling.kind == "rss":
      self.slots["sum_of_squares"] = [
          torch.full_like(p, scaling.initial_accumulator_value, dtype=torch.float32)
          for p in self.params]
    self.last_grad_norm: torch.Tensor | None = None
    if self.params and self.params[0].is_cuda:
      from recml_b200.utils import graphs
      graphs.register(self)

  def _lr_at(self, step: int) -> float:
    return float(self.lr(step)) if callable(self.lr) else float(self.lr)

  def num_params(self) -> int:
    return sum(t.numel() for ts in self.slots.values() for t in ts)

  # -- the update ------------------------------------------------------------
  @torch.no_grad()
  def step(self, grads: list[torch.Tensor | None] | None = None) -> None:
    """Applies one update from `grads` (default: each parameter's `.grad`)."""
    if grads is None:
      grads = [p.grad for p in self.params]
    lr = self._lr_at(self.count)
    self.hyperparams["learning_rate"] = lr
    live = [i for i, g in enumerate(grads) if g is not None]
    if not live:
      self.count += 1
      return
    params = [self.params[i] for i in live]
    gs = [grads[i] for i in live]
    if params[0].is_cuda:
      from recml_b200.ops import multi_tensor_optim
      self.last_grad_norm = multi_tensor_optim.fused_step(self, live, gs, lr)
      self.count += 1
      return
    gs = [g.to(torch.float32) for g in gs]
    if self.grad_clip_norm is not None:
      sq = sum((g * g).sum() for g in gs)
      if self.sq_norm_sync is not None:
        sq = self.sq_norm_sync(params, gs, sq)
      norm = torch.sqrt(sq)
      self.last_grad_norm = norm
      # optax.clip_by_global_norm: g * (clip / max(norm, clip))
      factor = self.grad_clip_norm / torch.clamp(norm, min=self.grad_clip_norm)
      gs = [g * factor for g in gs]
    t = self.count + 1
    kind = self.scaling.kind
    for i, p, g in zip(live, params, gs):
      if kind == "adam":
        mu, nu = self.slots["mu"][i], self.slots["nu"][i]
        mu.mul_(self.scaling.b1).add_(g, alpha=1 - self.scaling.b1)
        nu.mul_(self.scaling.b2).addcmul_(g, g, value=1 - self.scaling.b2)
        mhat = mu / (1 - self.scaling.b1 ** t)
        vhat = nu / (1 - self.scaling.b2 ** t)
        u = mhat / (vhat.sqrt() + self.scaling.eps)
      elif kind == "rss":
        acc = self.slots["sum_of_squares"][i]
        acc.addcmul_(g, g)
        u = torch.where(acc > 0, g * torch.rsqrt(acc + self.scaling.eps), torch.zeros_like(g))
      else:
        u = g
      if self.decay_flags[i]:
        u = u + self.weight_decay * p.to(torch.float32)
      p.add_(u.to(p.dtype), alpha=-lr)
    self.count += 1

  # -- CUDA-graph protocol (`recml_b200.utils.graphs`) ---------------------------------------------
  def graph_snapshot(self):
    return self.count

  def graph_restore(self, count) -> None:
    self.count = count

  def graph_advance(self) -> None:
    self.count += 1

  def graph_pre_replay(self) -> None:
    from recml_b200.ops import multi_tensor_optim
    lr = self._lr_at(self.count)
    self.hyperparams["learning_rate"] = lr
    multi_tensor_optim.push_hyper(self, lr, self.count + 1)

  def zero_grad(self) -> None:
    for p in self.params:
      p.grad = None

  def rebind(self, named_params) -> "Optimizer":
    """A fresh optimizer with this one's configuration over other tensors (slots start from scratch)."""
    new = Optimizer(named_params, **self._config)
    new.count = self.count
    return new

  def reset_step_count(self) -> None:
    """Restarts the schedule / bias-correction clock while keeping the slots (the
    `restore_iterations=False` case of `recml/core/utils/keras_utils.py:293-294`)."""
    self.count = 0
    self.hyperparams["learning_rate"] = self._lr_at(0)

  # -- checkpointing -----------------------------------------------------------
  def state_dict(self) -> dict[str, Any]:
    out: dict[str, Any] = {"count": torch.tensor(self.count, dtype=torch.int64)}
    for slot, tensors in self.slots.items():
      out[slot] = {n: t for n, t in zip(self.names, tensors)}
    return out

  def load_state_dict(self, sd: Mapping[str, Any]) -> None:
    self.count = int(sd["count"])
    for slot, tensors in self.slots.items():
      for n, t in zip(self.names, tensors):
        t.copy_(torch.as_tensor(sd[slot][n]))
    self.hyperparams["learning_rate"] = self._lr_at(self.count)


class OptimizerBuilder:
  """What a factory's `make()` returns: bind it to parameters with `.init(params)`."""

  def __init__(self, **config):
    self.config = config

  def init(self, named_params) -> Optimizer:
    return Optimizer(named_params, **self.config)


class OptimizerFactory(types.Factory[OptimizerBuilder]):
  learning_rate: float | Schedule
  scaling: Scaling = dataclasses.field(default_factory=identity)
  weight_decay: float | None = None
  grad_clip_norm: float | None = None
  weight_decay_mask: Mask = default_weight_decay_mask
  freeze_mask: Mask | None = None

  def make(self) -> OptimizerBuilder:
    return OptimizerBuilder(
        learning_rate=self.learning_rate, scaling=self.scaling, weight_decay=self.weight_decay,
        grad_clip_norm=self.grad_clip_norm, weight_decay_mask=self.weight_decay_mask,
        freeze_mask=self.freeze_mask)


class AdamFactory(types.Factory[OptimizerBuilder]):
  learning_rate: float | Schedule
  b1: float = 0.9
  b2: float = 0.999
  eps: float = 1e-8
  weight_decay: float | None = None
  grad_clip_norm: float | None = None
  weight_decay_mask: Mask = default_weight_decay_mask
  freeze_mask: Mask | None = None

  def make(self) -> OptimizerBuilder:
    return OptimizerFactory(
        learning_rate=self.learning_rate, scaling=scale_by_adam(self.b1, self.b2, self.eps),
        weight_decay=self.weight_decay, grad_clip_norm=self.grad_clip_norm,
        weight_decay_mask=self.weight_decay_mask, freeze_mask=self.freeze_mask).make()


class AdagradFactory(types.Factory[OptimizerBuilder]):
  learning_rate: float | Schedule
  initial_accumulator_value: float = 0.1
  eps: float = 1e-7
  grad_clip_norm: float | None = None
  freeze_mask: Mask | None = None

  def make(self) -> OptimizerBuilder:
    return OptimizerFactory(
        learning_rate=self.learning_rate,
        scaling=scale_by_rss(self.initial_accumulator_value, self.eps),
        grad_clip_norm=self.grad_clip_norm, freeze_mask=self.freeze_mask).make()


class SGDFactory(types.Factory[OptimizerBuilder]):
  learning_rate: float | Schedule
  weight_decay: float | None = None
  grad_clip_norm: float | None = None
  freeze_mask: Mask | None = None

  def make(self) -> OptimizerBuilder:
    return OptimizerFactory(learning_rate=self.learning_rate, weight_decay=self.weight_decay,
                            grad_clip_norm=self.grad_clip_norm, freeze_mask=self.freeze_mask).make()


def create_optimizer_for_sharded_model(model, factory: types.Factory[OptimizerBuilder] | OptimizerBuilder) -> Optimizer:
  """Dense optimizer for a model that contains sharded embeddings.

  The reference needs `create_optimizer_for_sc_model` (`jax_tpu_embedding/sparsecore/lib/flax/linen/
  embed_optimizer.py:77-97`) to route the embedding variables — whose "gradients" are already updated
  tables — around the dense optimizer with an optax `multi_transform`.  Here the tables are buffers of
  `ShardedEmbedding`, updated inside its backward kernel, so the split is structural: this returns
  `factory`'s optimizer over every trainable parameter that is not part of a sharded table."""
  builder = factory.make() if hasattr(factory, "make") else factory
  named = {n: p for n, p in model.named_parameters()
           if p.requires_grad and not getattr(p, "_recml_sharded", False)}
  return builder.init(named)
