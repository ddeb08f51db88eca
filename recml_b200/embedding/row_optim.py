"""Per-row optimizer update rules for embedding tables, in plain torch (fp32).

These are the oracle for the fused CUDA backward kernel and the implementation used by
the CPU / collective backend.  `g` is the gradient already aggregated per unique row.
Operator order follows the reference's update computations (SGD, Adagrad, Adam,
AdagradMomentum, FTRL, LaProp in its `sparse_dense_matmul_grad_with_*` primitives);
row-wise variants follow the usual definition with mean(g²) over the row.
"""
from __future__ import annotations

import torch

from recml_b200.embedding import specs


@torch.no_grad()
def apply(opt: specs.OptimizerSpec, step: int, w: torch.Tensor, g: torch.Tensor,
          slots: dict[str, torch.Tensor]) -> tuple[torch.Tensor, dict[str, torch.Tensor]]:
  """Returns the new rows and new slot rows for the touched rows `w` `[n, D]`."""
  hp = opt.hyperparams(step)
  kind = opt.kind
  if kind == "sgd":
    return w - hp[0] * g, {}
  if kind == "adagrad":
    acc = slots["accumulator"] + g * g
    return w - hp[0] * g / torch.sqrt(acc), {"accumulator": acc}
  if kind == "rowwise_adagrad":
    lr, eps = hp
    acc = slots["accumulator"] + (g * g).mean(dim=1)
    return w - lr * g / (torch.sqrt(acc)[:, None] + eps), {"accumulator": acc}
  if kind == "adam":
    alpha, b1, b2, eps_hat = hp
    m = slots["momentum"] + (1 - b1) * (g - slots["momentum"])
    v = slots["velocity"] + (1 - b2) * (g * g - slots["velocity"])
    return w - alpha * m / (torch.sqrt(v) + eps_hat), {"momentum": m, "velocity": v}
  if kind == "rowwise_adam":
    alpha, b1, b2, eps_hat = hp
    m = slots["momentum"] + (1 - b1) * (g - slots["momentum"])
    v = slots["velocity"] + (1 - b2) * ((g * g).mean(dim=1) - slots["velocity"])
    return w - alpha * m / (torch.sqrt(v)[:, None] + eps_hat), {"momentum": m, "velocity": v}
  if kind == "adagrad_momentum":
    lr, k, beta2, eps, exponent, nesterov = hp
    acc = slots["accumulator"]
    acc = acc + g * g if beta2 == 1.0 else beta2 * acc + (1 - beta2) * g * g
    s = torch.pow(acc + eps, -1.0 / exponent) * g
    mom = k * slots["momentum"] + s
    delta = k * mom + s if nesterov else mom
    return w - lr * delta, {"accumulator": acc, "momentum": mom}
  if kind == "ftrl":
    lr, lr_power, l1, l2, beta, mult = hp
    acc, lin = slots["accumulator"], slots["linear"]
    acc_new = acc + g * g
    p_old, p_new = torch.pow(acc, -lr_power), torch.pow(acc_new, -lr_power)
    if mult:
      lin_new = lin + lr * g - (p_new - p_old) * w
      l1s, den = l1 * lr, p_new + 2 * lr * l2 + beta
    else:
      lin_new = lin + g - ((p_new - p_old) / lr) * w
      l1s, den = l1, (p_new + beta) / lr + 2 * l2
    num = -lin_new if l1 == 0 else torch.clamp(lin_new, -l1s, l1s) - lin_new
    return num / den, {"accumulator": acc_new, "linear": lin_new}
  if kind == "laprop":
    lr, b1, decay, eps = hp
    nu = decay * slots["nu"] + (1 - decay) * (g * g + eps)
    u = g / torch.sqrt(nu)
    mu = b1 * slots["mu"] + (1 - b1 * b1) ** 0.5 * u
    return w - lr * mu, {"mu": mu, "nu": nu}
  raise ValueError(f"Unknown embedding optimizer {kind!r}")
