"""Optimizer factories against the optax chains they stand for, written out in plain torch
(the contract of `recml/core/training/optax_factory_test.py:48-161`)."""
import math

import pytest
import torch
from torch import nn

import recml_b200 as recml
from recml_b200.training import optim_factory as O


def _params():
  torch.manual_seed(0)
  m = nn.Sequential(nn.Linear(5, 4), nn.Linear(4, 3))
  return m, {n: p for n, p in m.named_parameters()}


def _grads(named, seed):
  g = torch.Generator().manual_seed(seed)
  return {n: torch.randn(p.shape, generator=g) * 3.0 for n, p in named.items()}


def _clip(grads, max_norm):
  if max_norm is None:
    return grads
  total = math.sqrt(sum(float((g.double() ** 2).sum()) for g in grads.values()))
  scale = min(1.0, max_norm / max(total, 1e-16)) if total > max_norm else 1.0
  return {n: g * scale for n, g in grads.items()}


def _run(factory, steps, chain):
  """Runs `factory` for `steps` steps with fixed gradients and compares with `chain(step, name, g, w)`."""
  m, named = _params()
  ref = {n: p.detach().clone() for n, p in named.items()}
  opt = factory.make().init(list(named.items()))
  clip = getattr(factory, "grad_clip_norm", None)
  for step in range(steps):
    grads = _grads(named, step)
    for n, p in named.items():
      p.grad = grads[n].clone()
    opt.step()
    opt.zero_grad()
    clipped = _clip(grads, clip)
    for n in ref:
      ref[n] = chain(step, n, clipped[n], ref[n])
  for n, p in named.items():
    torch.testing.assert_close(p.detach(), ref[n], rtol=1e-5, atol=1e-6, msg=lambda s, n=n: f"{n}: {s}")
  return opt


def test_adam_factory_is_clip_adam_decay_lr():
  lr, b1, b2, eps, wd = 0.01, 0.9, 0.95, 1e-6, 0.05
  mu, nu = {}, {}

  def chain(step, n, g, w):
    mu[n] = b1 * mu.get(n, torch.zeros_like(g)) + (1 - b1) * g
    nu[n] = b2 * nu.get(n, torch.zeros_like(g)) + (1 - b2) * g * g
    mh, nh = mu[n] / (1 - b1 ** (step + 1)), nu[n] / (1 - b2 ** (step + 1))
    u = mh / (nh.sqrt() + eps)
    if w.ndim > 1:                      # default mask: matrices decay, biases do not
      u = u + wd * w
    return w - lr * u
  _run(recml.AdamFactory(learning_rate=lr, b1=b1, b2=b2, eps=eps, weight_decay=wd, grad_clip_norm=1.0), 5, chain)


def test_adagrad_factory_is_clip_rss_lr():
  lr, acc0, eps = 0.1, 0.1, 1e-7
  acc = {}

  def chain(step, n, g, w):
    acc[n] = acc.get(n, torch.full_like(g, acc0)) + g * g
    return w - lr * g / (acc[n] + eps).sqrt()
  _run(recml.AdagradFactory(learning_rate=lr, initial_accumulator_value=acc0, eps=eps, grad_clip_norm=2.0), 4, chain)


def test_sgd_with_schedule_and_logged_learning_rate():
  sched = O.warmup_cosine_decay_schedule(0.0, 0.5, warmup_steps=3, decay_steps=10, end_value=0.05)
  assert sched(0) == 0.0 and abs(sched(3) - 0.5) < 1e-12 and abs(sched(10) - 0.05) < 1e-12
  assert abs(sched(1) - 0.5 / 3) < 1e-12 and sched(100) == pytest.approx(0.05)
  seen = []

  def chain(step, n, g, w):
    return w - sched(step) * g
  opt = _run(recml.SGDFactory(learning_rate=sched), 6, chain)
  assert opt.hyperparams["learning_rate"] == pytest.approx(sched(5))   # the rate of the last step taken
  del seen


def test_regex_masks_and_freeze():
  lr, wd = 0.1, 0.5

  def chain(step, n, g, w):
    if n.startswith("0."):              # frozen
      return w
    u = g + (wd * w if n.endswith("bias") else 0.0)
    return w - lr * u
  _run(O.OptimizerFactory(learning_rate=lr, weight_decay=wd, weight_decay_mask=r".*bias$", freeze_mask=r"^0\."), 3,
       chain)
  # a callable mask sees (name, tensor)
  f = O.OptimizerFactory(learning_rate=lr, freeze_mask=lambda n, p: p.ndim == 1)
  m, named = _params()
  before = {n: p.detach().clone() for n, p in named.items()}
  opt = f.make().init(list(named.items()))
  for n, p in named.items():
    p.grad = torch.ones_like(p)
  opt.step()
  for n, p in named.items():
    assert torch.equal(p, before[n]) == (p.ndim == 1), n


def test_state_dict_round_trip_continues_identically():
  fac = recml.AdamFactory(learning_rate=0.01, weight_decay=0.01)
  m1, n1 = _params()
  o1 = fac.make().init(list(n1.items()))
  for step in range(3):
    for n, p in n1.items():
      p.grad = _grads(n1, step)[n]
    o1.step()
  m2, n2 = _params()
  for (_, a), (_, b) in zip(n1.items(), n2.items()):
    b.data.copy_(a.data)
  o2 = fac.make().init(list(n2.items()))
  o2.load_state_dict(o1.state_dict())
  for o, named in ((o1, n1), (o2, n2)):
    for n, p in named.items():
      p.grad = _grads(named, 9)[n]
    o.step()
  for (_, a), (_, b) in zip(n1.items(), n2.items()):
    torch.testing.assert_close(a, b)


@pytest.mark.parametrize("clip", [None, 0.5])
def test_adam_and_sgd_factories_follow_torch_optimizers(clip):
  """An independent oracle: AdamFactory is `torch.optim.AdamW` (decoupled decay on the matrices only) behind
  `clip_grad_norm_`, SGDFactory is `torch.optim.SGD`, over ten steps with a cosine schedule."""
  total = 10
  sched = lambda step: 0.02 * 0.5 * (1.0 + math.cos(math.pi * step / total))
  for kind in ("adam", "sgd"):
    m, named = _params()
    twin, twin_named = _params()
    if kind == "adam":
      opt = recml.AdamFactory(learning_rate=sched, b1=0.9, b2=0.98, eps=1e-8, weight_decay=0.1, grad_clip_norm=clip).make() \
          .init(list(named.items()))
      ref = torch.optim.AdamW([{"params": [p for p in twin_named.values() if p.ndim > 1], "weight_decay": 0.1},
                               {"params": [p for p in twin_named.values() if p.ndim <= 1], "weight_decay": 0.0}],
                              lr=1.0, betas=(0.9, 0.98), eps=1e-8)
    else:
      opt = recml.SGDFactory(learning_rate=sched, grad_clip_norm=clip).make().init(list(named.items()))
      ref = torch.optim.SGD(twin_named.values(), lr=1.0)
    for step in range(total):
      grads = _grads(named, step)
      for n in named:
        named[n].grad = grads[n].clone()
        twin_named[n].grad = grads[n].clone()
      if clip is not None:
        torch.nn.utils.clip_grad_norm_(list(twin_named.values()), clip)
      for group in ref.param_groups:
        group["lr"] = sched(step)
      opt.step()
      ref.step()
    for n in named:
      torch.testing.assert_close(named[n].detach(), twin_named[n].detach(), rtol=2e-5, atol=2e-6,
                                 msg=lambda s, n=n, kind=kind: f"{kind} {n}: {s}")
