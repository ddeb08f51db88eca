"""Embedding specs: features, tables and per-table optimizers.

Field names follow the reference so configs translate directly:
`EmbeddingSpec` ↔ `recml/layers/linen/sparsecore.py:52-91`; `TableSpec`/`FeatureSpec`
and the optimizer specs ↔ the `embedding_spec` module of the reference's embedding
engine (Adagrad `initial_accumulator_value=0.1`, Adam with bias-corrected step size,
AdagradMomentum, FTRL, LaProp, SGD).  Added here: ROW-WISE Adagrad / Adam, which keep
one second-moment scalar per row instead of a table-shaped accumulator.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Callable, Literal

import torch

Combiner = Literal["sum", "mean", "sqrtn"]
LearningRate = float | Callable[[int], float]


@dataclasses.dataclass(frozen=True)
class OptimizerSpec:
  learning_rate: LearningRate = 0.01
  kind = "base"

  def lr(self, step: int) -> float:
    return float(self.learning_rate(step)) if callable(self.learning_rate) else float(self.learning_rate)

  def slot_names(self) -> tuple[str, ...]:
    return ()

  def slot_is_rowwise(self, slot: str) -> bool:
    return False

  def slot_init(self, slot: str) -> float:
    return 0.0

  def slot_bytes_per_row(self, dim: int) -> int:
    """Optimizer-state bytes stored beside each table row (fp32 slots)."""
    return sum(4 if self.slot_is_rowwise(s) else 4 * dim for s in self.slot_names())

  def hyperparams(self, step: int) -> tuple[float, ...]:
    """Scalars handed to the update kernel for this step (first one is the step size)."""
    return (self.lr(step),)


@dataclasses.dataclass(frozen=True)
class SGDOptimizerSpec(OptimizerSpec):
  kind = "sgd"


@dataclasses.dataclass(frozen=True)
class AdagradOptimizerSpec(OptimizerSpec):
  """Element-wise: acc += g²; w -= lr·g/√acc  (no epsilon, accumulator starts at 0.1)."""
  initial_accumulator_value: float = 0.1
  kind = "adagrad"

  def slot_names(self):
    return ("accumulator",)

  def slot_init(self, slot):
    return self.initial_accumulator_value


@dataclasses.dataclass(frozen=True)
class RowWiseAdagradOptimizerSpec(OptimizerSpec):
  """One accumulator per row: s += mean(g²); w -= lr·g/(√s + eps)."""
  initial_accumulator_value: float = 0.0
  eps: float = 1e-8
  kind = "rowwise_adagrad"

  def slot_names(self):
    return ("accumulator",)

  def slot_is_rowwise(self, slot):
    return True

  def slot_init(self, slot):
    return self.initial_accumulator_value

  def hyperparams(self, step):
    return (self.lr(step), self.eps)


@dataclasses.dataclass(frozen=True)
class AdamOptimizerSpec(OptimizerSpec):
  """m += (1-β1)(g-m); v += (1-β2)(g²-v); w -= α_t·m/(√v + ε̂) with
  α_t = lr·√(1-β2^t)/(1-β1^t), ε̂ = ε·√(1-β2^t), t = step+1."""
  beta_1: float = 0.9
  beta_2: float = 0.999
  epsilon: float = 1e-8
  kind = "adam"

  def slot_names(self):
    return ("momentum", "velocity")

  def hyperparams(self, step):
    t = step + 1
    c2 = math.sqrt(1.0 - self.beta_2 ** t)
    return (self.lr(step) * c2 / (1.0 - self.beta_1 ** t), self.beta_1, self.beta_2,
            self.epsilon * c2)


@dataclasses.dataclass(frozen=True)
class RowWiseAdamOptimizerSpec(AdamOptimizerSpec):
  """Adam whose second moment is one scalar per row (v += (1-β2)(mean(g²)-v))."""
  kind = "rowwise_adam"

  def slot_is_rowwise(self, slot):
    return slot == "velocity"


@dataclasses.dataclass(frozen=True)
class AdagradMomentumOptimizerSpec(OptimizerSpec):
  momentum: float = 0.9
  beta2: float = 1.0
  epsilon: float = 1e-10
  exponent: float = 2.0
  use_nesterov: bool = False
  initial_accumulator_value: float = 0.1
  kind = "adagrad_momentum"

  def slot_names(self):
    return ("accumulator", "momentum")

  def slot_init(self, slot):
    return self.initial_accumulator_value if slot == "accumulator" else 0.0

  def hyperparams(self, step):
    return (self.lr(step), self.momentum, self.beta2, self.epsilon, self.exponent,
            1.0 if self.use_nesterov else 0.0)


@dataclasses.dataclass(frozen=True)
class FTRLOptimizerSpec(OptimizerSpec):
  learning_rate_power: float = -0.5
  l1_regularization_strength: float = 0.0
  l2_regularization_strength: float = 0.0
  beta: float = 0.0
  initial_accumulator_value: float = 0.1
  multiply_linear_by_learning_rate: bool = False
  kind = "ftrl"

  def slot_names(self):
    return ("accumulator", "linear")

  def slot_init(self, slot):
    return self.initial_accumulator_value if slot == "accumulator" else 0.0

  def hyperparams(self, step):
    return (self.lr(step), self.learning_rate_power, self.l1_regularization_strength,
            self.l2_regularization_strength, self.beta,
            1.0 if self.multiply_linear_by_learning_rate else 0.0)


@dataclasses.dataclass(frozen=True)
class LaPropOptimizerSpec(OptimizerSpec):
  b1: float = 0.9
  b2: float = 0.95
  eps: float = 1e-30
  kind = "laprop"

  def slot_names(self):
    return ("mu", "nu")

  def hyperparams(self, step):
    t = step + 1
    decay = self.b2 * (1.0 - self.b2 ** (t - 1)) / (1.0 - self.b2 ** t)
    return (self.lr(step), self.b1, decay, self.eps)


@dataclasses.dataclass
class EmbeddingSpec:
  """One sparse feature → one table (tables are shared when specs compare equal on
  (input_dim, embedding_dim, initializer, optimizer) and `table_name` matches)."""
  input_dim: int
  embedding_dim: int
  max_sequence_length: int | None = None
  combiner: Combiner = "mean"
  initializer: Callable[[torch.Tensor, torch.Generator], None] | None = None
  optimizer: OptimizerSpec | None = None
  weight_name: str | None = None
  table_name: str | None = None

  def __post_init__(self):
    if self.max_sequence_length is not None and self.weight_name is not None:
      raise ValueError("`max_sequence_length` and `weight_name` cannot both be set: weighted "
                       "aggregation needs the sequence dimension to be pooled.")
    if self.combiner not in ("sum", "mean", "sqrtn"):
      raise ValueError(f"Unknown combiner {self.combiner!r}")

  def __hash__(self):
    return id(self)


@dataclasses.dataclass
class TableSpec:
  name: str
  vocabulary_size: int
  embedding_dim: int
  optimizer: OptimizerSpec
  combiner: Combiner = "sum"
  initializer: Callable | None = None
  max_ids_per_partition: int = 256          # kept for stats / FDO parity
  max_unique_ids_per_partition: int = 256


@dataclasses.dataclass
class FeatureSpec:
  name: str
  table: TableSpec
  combiner: Combiner
  max_sequence_length: int | None = None
  weight_name: str | None = None


def truncated_normal_init(stddev: float):
  def init(t: torch.Tensor, gen: torch.Generator):
    torch.nn.init.trunc_normal_(t, mean=0.0, std=stddev, a=-2 * stddev, b=2 * stddev, generator=gen)
  return init


def normal_init(stddev: float):
  def init(t, gen):
    t.normal_(0.0, stddev, generator=gen)
  return init


def uniform_init(scale: float):
  def init(t, gen):
    t.uniform_(-scale, scale, generator=gen)
  return init
