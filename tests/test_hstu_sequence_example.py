"""The TFRecord-based HSTU next-item example (padded sequences, last-position logits, compile-and-fit
trainer) on CPU with a small vocabulary."""
import os

import numpy as np
import torch

import recml_b200 as recml
from recml_b200 import config as C
from recml_b200.examples import hstu_sequence_experiment as E


def test_pad_right_keeps_the_most_recent_items():
  values = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9], dtype=np.int64)
  ids, mask = E.pad_right(values, np.array([2, 0, 7]), 4)
  assert ids.tolist() == [[1, 2, 0, 0], [0, 0, 0, 0], [6, 7, 8, 9]]
  assert mask.tolist() == [[1, 1, 0, 0], [0, 0, 0, 0], [1, 1, 1, 1]]


def test_last_position_logits_ignore_the_padding():
  torch.manual_seed(0)
  cfg = E.HSTUModelConfig(vocab_size=50, max_sequence_length=6, model_dim=16, num_heads=2, num_layers=1, dropout=0.0)
  m = E.LastPositionHSTU(cfg).eval()
  ids = torch.tensor([[4, 9, 7, 0, 0, 0]])
  mask = torch.tensor([[1, 1, 1, 0, 0, 0]])
  a = m({"input_ids": ids, "padding_mask": mask})
  ids2 = ids.clone()
  ids2[0, 3:] = torch.tensor([11, 12, 13])                 # whatever sits in the padded slots must not matter
  b = m({"input_ids": ids2, "padding_mask": mask})
  assert a.shape == (1, 50)
  torch.testing.assert_close(a, b)


def test_experiment_trains_and_evaluates(tmp_path):
  vocab = 40
  E.write_synthetic_tfrecords(str(tmp_path / "data" / "train-0.tfrecord"), 600, vocab, max_len=12, seed=0)
  E.write_synthetic_tfrecords(str(tmp_path / "data" / "eval-0.tfrecord"), 128, vocab, max_len=12, seed=1)
  cfg = E.experiment(train_path=str(tmp_path / "data" / "train-*.tfrecord"), eval_path=str(tmp_path / "data" / "eval-*.tfrecord"),
                     model_dir=str(tmp_path / "model"), vocab_size=vocab, batch_size=32, train_steps=120)
  cfg.task.model_config.max_sequence_length = 10
  cfg.task.model_config.model_dim = 32
  cfg.task.model_config.num_layers = 1
  cfg.task.model_config.dropout = 0.0
  cfg.task.model_config.learning_rate = 5e-3
  cfg.task.train_data.max_sequence_length = 10
  cfg.task.eval_data.max_sequence_length = 10
  cfg.trainer.steps_per_loop = 40
  cfg.trainer.steps_per_eval = 4
  hist = recml.run_experiment(C.build(cfg), "train_and_eval")
  assert len(hist["loss"]) == 3 and hist["loss"][-1] < hist["loss"][0]
  assert "val_loss" in hist and "val_accuracy" in hist
  assert hist["loss"][-1] < np.log(vocab)                  # better than the uniform guess
  assert os.path.isdir(os.path.join(tmp_path, "model", "checkpoints"))


def test_step_trainer_variant_trains(tmp_path):
  vocab = 40
  E.write_synthetic_tfrecords(str(tmp_path / "data" / "train-0.tfrecord"), 600, vocab, max_len=12, seed=0)
  E.write_synthetic_tfrecords(str(tmp_path / "data" / "eval-0.tfrecord"), 128, vocab, max_len=12, seed=1)
  cfg = E.step_experiment(train_path=str(tmp_path / "data" / "train-*.tfrecord"),
                          eval_path=str(tmp_path / "data" / "eval-*.tfrecord"), model_dir=str(tmp_path / "model"),
                          vocab_size=vocab, batch_size=32, train_steps=90)
  for part in (cfg.task.model_config, cfg.task.train_data, cfg.task.eval_data):
    part.max_sequence_length = 10
  cfg.task.model_config.model_dim, cfg.task.model_config.num_layers = 32, 1
  cfg.task.model_config.dropout, cfg.task.model_config.learning_rate = 0.0, 5e-3
  cfg.trainer.steps_per_loop, cfg.trainer.steps_per_eval = 30, 4
  cfg.trainer.partitioner = C.Config(recml.DataParallelPartitioner, device="cpu")
  logs = recml.run_experiment(C.build(cfg), "train_and_eval")
  assert logs["train"]["loss"] < np.log(vocab) and "accuracy" in logs["val"]
