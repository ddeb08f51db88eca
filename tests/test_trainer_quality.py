"""End-to-end quality of the step-function trainer on a real classification problem: a small CNN on the
8 x 8 handwritten digits that ship with scikit-learn must pass 95 % accuracy on the training stream and on
held-out digits, in `train_and_evaluate` and again in continuous evaluation of the written checkpoints.
The counterpart of the reference's MNIST test (`recml/core/training/jax_trainer_quality_test.py:35-149`;
MNIST itself needs a download)."""
import os

import numpy as np
import pytest
import torch
from torch import nn

import recml_b200 as recml
from recml_b200.data import iterator as iterator_lib

sklearn_datasets = pytest.importorskip("sklearn.datasets")


class _Digits:
  def __init__(self, images, labels, batch, epochs, seed):
    self.images, self.labels, self.batch, self.epochs, self.seed = images, labels, batch, epochs, seed

  def __iter__(self):
    rng = np.random.default_rng(self.seed)
    for _ in range(self.epochs):
      order = rng.permutation(len(self.labels)) if self.seed else np.arange(len(self.labels))
      for at in range(0, len(order) - self.batch + 1, self.batch):
        idx = order[at:at + self.batch]
        yield {"image": self.images[idx], "label": self.labels[idx]}


class _DigitsTask(recml.Task):
  def create_datasets(self):
    d = sklearn_datasets.load_digits()
    images = (d.images / 16.0).astype(np.float32)[:, None]            # [N, 1, 8, 8]
    labels = d.target.astype(np.int64)
    order = np.random.default_rng(0).permutation(len(labels))          # the file is ordered by writer
    tr, va = order[:1500], order[1500:]
    train = _Digits(images[tr], labels[tr], 32, 1000, seed=1)
    val = _Digits(images[va], labels[va], 32, 1, seed=0)
    return iterator_lib.IterableIterator(train), iterator_lib.IterableIterator(val)

  def create_state(self, batch, rng):
    torch.manual_seed(rng.initial_seed())
    model = nn.Sequential(nn.Conv2d(1, 32, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2),
                          nn.Conv2d(32, 64, 3, padding=1), nn.ReLU(), nn.MaxPool2d(2),
                          nn.Flatten(), nn.Linear(64 * 2 * 2, 256), nn.ReLU(), nn.Linear(256, 10))
    return recml.State.create(model=model, tx=recml.SGDFactory(learning_rate=0.1).make())

  def _metrics(self, logits, labels, loss):
    return {"loss": recml.metrics.mean(loss.detach()), "accuracy": recml.metrics.accuracy(labels, logits.detach())}

  def train_step(self, batch, state, rng):
    logits = state.model(batch["image"])
    loss = nn.functional.cross_entropy(logits, batch["label"])
    loss.backward()
    state.update()
    return state, self._metrics(logits, batch["label"], loss)

  def eval_step(self, batch, state):
    with torch.no_grad():
      logits = state.model(batch["image"])
      return self._metrics(logits, batch["label"], nn.functional.cross_entropy(logits, batch["label"]))


def test_digits_e2e(tmp_path):
  task = _DigitsTask()
  trainer = recml.Trainer(partitioner=recml.DataParallelPartitioner(device="cpu"), train_steps=800, steps_per_eval=9,
                          steps_per_loop=100, continuous_eval_timeout=2, model_dir=str(tmp_path), rng_seed=42)
  logs = trainer.train_and_evaluate(task)
  assert logs["train"]["accuracy"] > 0.95
  assert logs["val"]["accuracy"] > 0.95
  assert os.path.isdir(tmp_path / "checkpoints")
  continuous = trainer.evaluate_continuously(task)
  assert continuous["val"]["accuracy"] > 0.95
