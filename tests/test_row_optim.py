"""Embedding row-optimizer rules against an independent float64 restatement of the reference's update
computations (`sparse_dense_matmul_grad_with_{sgd,adagrad,adam,adagrad_momentum,ftrl,laprop}.py`) and of
the row-wise variants, over several steps with a step-dependent learning rate."""
import math

import numpy as np
import pytest
import torch

from recml_b200.embedding import row_optim, specs as S


def _run(opt, steps=4, n=6, d=8, seed=0):
  rng = np.random.default_rng(seed)
  w = rng.normal(size=(n, d))
  slots = {s: np.full((n,) if opt.slot_is_rowwise(s) else (n, d), opt.slot_init(s)) for s in opt.slot_names()}
  grads = [rng.normal(size=(n, d)) * 0.3 for _ in range(steps)]
  tw = torch.tensor(w, dtype=torch.float32)
  ts = {k: torch.tensor(v, dtype=torch.float32) for k, v in slots.items()}
  for step, g in enumerate(grads):
    tw, ts = row_optim.apply(opt, step, tw, torch.tensor(g, dtype=torch.float32), ts)
  return w, slots, grads, tw.numpy(), {k: v.numpy() for k, v in ts.items()}


LR = lambda step: 0.05 / (1 + step)


def test_sgd_and_adagrad():
  w, slots, grads, got, _ = _run(S.SGDOptimizerSpec(learning_rate=LR))
  for t, g in enumerate(grads):
    w = w - LR(t) * g
  np.testing.assert_allclose(got, w, rtol=1e-5, atol=1e-6)
  w, slots, grads, got, gs = _run(S.AdagradOptimizerSpec(learning_rate=LR))
  acc = slots["accumulator"]
  assert np.all(acc == 0.1)                                      # the reference's initial accumulator
  for t, g in enumerate(grads):
    acc = acc + g * g
    w = w - LR(t) * g / np.sqrt(acc)                             # no epsilon
  np.testing.assert_allclose(got, w, rtol=1e-5, atol=1e-6)
  np.testing.assert_allclose(gs["accumulator"], acc, rtol=1e-5)


def test_adam_bias_correction_folded_into_step_size():
  opt = S.AdamOptimizerSpec(learning_rate=LR, beta_1=0.9, beta_2=0.99, epsilon=1e-6)
  w, slots, grads, got, gs = _run(opt)
  m, v = slots["momentum"], slots["velocity"]
  for t, g in enumerate(grads):
    c2 = math.sqrt(1 - 0.99 ** (t + 1))
    alpha, eps_hat = LR(t) * c2 / (1 - 0.9 ** (t + 1)), 1e-6 * c2
    m = m + (1 - 0.9) * (g - m)
    v = v + (1 - 0.99) * (g * g - v)
    w = w - alpha * m / (np.sqrt(v) + eps_hat)
  np.testing.assert_allclose(got, w, rtol=2e-5, atol=1e-6)
  np.testing.assert_allclose(gs["velocity"], v, rtol=1e-5, atol=1e-9)


def test_rowwise_adagrad_uses_mean_square_of_the_row():
  opt = S.RowWiseAdagradOptimizerSpec(learning_rate=LR)
  w, slots, grads, got, gs = _run(opt)
  acc = slots["accumulator"]
  assert acc.shape == (6,)
  lr0, eps = opt.hyperparams(0)
  for t, g in enumerate(grads):
    acc = acc + (g * g).mean(1)
    w = w - LR(t) * g / (np.sqrt(acc)[:, None] + eps)
  np.testing.assert_allclose(got, w, rtol=2e-5, atol=1e-6)


@pytest.mark.parametrize("nesterov,beta2", [(False, 1.0), (True, 0.9)])
def test_adagrad_momentum(nesterov, beta2):
  opt = S.AdagradMomentumOptimizerSpec(learning_rate=LR, momentum=0.8, beta2=beta2, epsilon=1e-10, exponent=2.0,
                                       use_nesterov=nesterov)
  w, slots, grads, got, _ = _run(opt)
  acc, mom = slots["accumulator"], slots["momentum"]
  for t, g in enumerate(grads):
    acc = acc + g * g if beta2 == 1.0 else beta2 * acc + (1 - beta2) * g * g
    s = (acc + 1e-10) ** (-1 / 2.0) * g
    mom = 0.8 * mom + s
    w = w - LR(t) * (0.8 * mom + s if nesterov else mom)
  np.testing.assert_allclose(got, w, rtol=2e-5, atol=1e-6)


@pytest.mark.parametrize("mult,l1", [(False, 0.0), (False, 0.01), (True, 0.01)])
def test_ftrl(mult, l1):
  opt = S.FTRLOptimizerSpec(learning_rate=0.05, learning_rate_power=-0.5, l1_regularization_strength=l1,
                            l2_regularization_strength=0.02, beta=0.1, multiply_linear_by_learning_rate=mult)
  w, slots, grads, got, _ = _run(opt)
  acc, lin, lr = slots["accumulator"], slots["linear"], 0.05
  for g in grads:
    acc_new = acc + g * g
    p_old, p_new = acc ** 0.5, acc_new ** 0.5
    if mult:
      lin = lin + lr * g - (p_new - p_old) * w
      l1s, den = l1 * lr, p_new + 2 * lr * 0.02 + 0.1
    else:
      lin = lin + g - ((p_new - p_old) / lr) * w
      l1s, den = l1, (p_new + 0.1) / lr + 2 * 0.02
    num = -lin if l1 == 0 else np.clip(lin, -l1s, l1s) - lin
    w, acc = num / den, acc_new
  np.testing.assert_allclose(got, w, rtol=5e-5, atol=1e-6)


def test_laprop():
  opt = S.LaPropOptimizerSpec(learning_rate=LR, b1=0.9, b2=0.95, eps=1e-30)
  w, slots, grads, got, _ = _run(opt)
  mu, nu = slots["mu"], slots["nu"]
  for t, g in enumerate(grads):
    decay = 0.95 * (1 - 0.95 ** t) / (1 - 0.95 ** (t + 1))
    nu = decay * nu + (1 - decay) * (g * g + 1e-30)
    mu = 0.9 * mu + math.sqrt(1 - 0.81) * (g / np.sqrt(nu))
    w = w - LR(t) * mu
  np.testing.assert_allclose(got, w, rtol=5e-5, atol=1e-6)
