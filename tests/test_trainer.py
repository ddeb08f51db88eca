"""Trainer modes, checkpoint cadence, resume, continuous evaluation, partitioners and the
module ("compile-and-fit") trainer — the torch rendering of `jax_trainer_test.py`,
`keras_trainer_test.py` and `partitioning_test.py`."""
import os
import threading

import numpy as np
import pytest
import torch
from torch import nn

import recml_b200 as recml
from recml_b200 import ckpt
from recml_b200.data import iterator as iterator_lib
from recml_b200.training import module_trainer, partitioning


class _Range:
  def __init__(self, n, batch=8, seed=0):
    self.n, self.batch, self.seed = n, batch, seed

  def __iter__(self):
    rng = np.random.default_rng(self.seed)
    for _ in range(self.n):
      x = rng.normal(size=(self.batch, 4)).astype(np.float32)
      yield {"x": x, "y": (x @ np.array([1., -2., 0.5, 3.], dtype=np.float32))[:, None]}


class _Task(recml.Task):
  def __init__(self, named_evals=False, n_train=1000):
    self.named, self.n_train = named_evals, n_train

  def create_datasets(self):
    tr = iterator_lib.IterableIterator(_Range(self.n_train))
    if self.named:
      return tr, {"a": iterator_lib.IterableIterator(_Range(3, seed=1)),
                  "b": iterator_lib.IterableIterator(_Range(2, seed=2))}
    return tr, iterator_lib.IterableIterator(_Range(3, seed=1))

  def create_state(self, batch, rng):
    torch.manual_seed(0)
    return recml.State.create(model=nn.Linear(4, 1), tx=recml.AdamFactory(learning_rate=0.05).make())

  def train_step(self, batch, state, rng):
    loss = ((state.model(batch["x"]) - batch["y"]) ** 2).mean()
    loss.backward()
    state.update()
    return state, {"loss": recml.metrics.mean(loss.detach()), "lr": recml.metrics.scalar(0.05)}

  def eval_step(self, batch, state):
    return {"loss": recml.metrics.mean(((state.model(batch["x"]) - batch["y"]) ** 2).mean())}


def _trainer(d, **kw):
  base = dict(partitioner=recml.DataParallelPartitioner(device="cpu"), model_dir=str(d), train_steps=12,
              steps_per_loop=4, steps_per_eval=3, continuous_eval_timeout=1)
  base.update(kw)
  return recml.Trainer(**base)


@pytest.mark.parametrize("mode", ["train", "eval", "train_and_eval", "continuous_eval"])
def test_modes_and_log_keys(tmp_path, mode):
  if mode == "continuous_eval":
    recml.run_experiment(recml.Experiment(_Task(), _trainer(tmp_path)), "train")
  logs = recml.run_experiment(recml.Experiment(_Task(), _trainer(tmp_path)), mode)
  if mode in ("train", "train_and_eval"):
    assert "loss" in logs["train"]
    assert ckpt.all_steps(os.path.join(tmp_path, "checkpoints")) == [3, 7, 11]
    assert open(os.path.join(tmp_path, "marker.txt")).read() == "COMPLETED"
    assert "optimizer/learning_rate" in logs["train"] and "model/num_trainable_variables" in logs["train"]
  if mode != "train":
    assert "loss" in logs["val"]


def test_named_eval_sets_and_perf_scalars(tmp_path):
  logs = recml.run_experiment(recml.Experiment(_Task(named_evals=True), _trainer(tmp_path, train_steps=10, steps_per_loop=10)),
                              "train_and_eval")
  assert {"train", "val_a", "val_b"} <= set(logs)
  assert logs["train"]["perf/loop_throughput_ex_per_sec"] > 0 and logs["train"]["perf/loop_ms_per_step"] > 0
  assert os.path.isdir(os.path.join(tmp_path, "logs", "val_a"))


def test_training_converges_and_resumes(tmp_path):
  t = _trainer(tmp_path, train_steps=200, steps_per_loop=100, checkpoint_interval=50)
  logs = recml.run_experiment(recml.Experiment(_Task(), t), "train_and_eval")
  assert logs["val"]["loss"] < 0.05
  assert ckpt.all_steps(os.path.join(tmp_path, "checkpoints")) == [49, 99, 149, 199]
  # a second run finds step 199, so there is nothing left to train and weights are the restored ones
  t2 = _trainer(tmp_path, train_steps=200, steps_per_loop=100)
  _, _, state, _, _, step = t2.process_task(_Task(), training=True)
  assert step == 200
  ev = recml.run_experiment(recml.Experiment(_Task(), _trainer(tmp_path, train_steps=200)), "eval")
  np.testing.assert_allclose(ev["val"]["loss"], logs["val"]["loss"], rtol=1e-5)


def test_continuous_eval_follows_a_running_trainer(tmp_path):
  res = {}
  th = threading.Thread(target=lambda: res.update(
      recml.run_experiment(recml.Experiment(_Task(), _trainer(tmp_path, continuous_eval_timeout=2)), "continuous_eval")))
  th.start()
  recml.run_experiment(recml.Experiment(_Task(), _trainer(tmp_path)), "train")
  th.join(timeout=60)
  assert not th.is_alive() and "loss" in res["val"]


def test_half_written_checkpoint_is_skipped(tmp_path):
  recml.run_experiment(recml.Experiment(_Task(), _trainer(tmp_path)), "train")
  os.remove(os.path.join(tmp_path, "checkpoints", "7", "state", "_METADATA"))
  logs = recml.run_experiment(recml.Experiment(_Task(), _trainer(tmp_path)), "continuous_eval")
  assert "loss" in logs["val"]


def test_partitioners_cpu():
  p = recml.NullPartitioner("cpu")
  out = p.shard_inputs({"a": np.ones((4, 2), np.float32), "b": [np.zeros(3)]})
  assert isinstance(out["a"], torch.Tensor) and out["a"].shape == (4, 2) and isinstance(out["b"][0], torch.Tensor)
  dp = recml.DataParallelPartitioner(device="cpu")
  st = dp.partition_init(lambda b: recml.State.create(model=nn.Linear(2, 2), tx=recml.SGDFactory(learning_rate=.1).make()))(None)
  assert st.grad_sync is not None
  mp = recml.ModelParallelPartitioner(axes=[("data", 1), ("model", 1)], rules=[(r"weight", ("model", None))], device="cpu")
  st = mp.partition_init(lambda b: recml.State.create(model=nn.Linear(4, 6), tx=recml.SGDFactory(learning_rate=.1).make()))(None)
  assert st.params["weight"]._recml_spec == ("model", None) and st.params["weight"].shape == (6, 4)
  with pytest.raises(ValueError):
    recml.ModelParallelPartitioner(axes=[("data", 3)], device="cpu")


class _ModTask(recml.KerasTask):
  def create_dataset(self, training):
    n = 40 if training else 3
    return [(torch.from_numpy(b["x"]), torch.from_numpy(b["y"])) for b in _Range(n, seed=0 if training else 1)]

  def create_model(self, **kw):
    torch.manual_seed(0)
    return module_trainer.CompiledModel(nn.Linear(4, 1, bias=False), lambda o, y: ((o - y) ** 2).mean(),
                                        recml.AdamFactory(learning_rate=0.05).make(),
                                        {"mse": lambda y, o: recml.metrics.mean_squared_error(y, o)})


@pytest.mark.parametrize("mode", ["train", "eval", "train_and_eval", "continuous_eval"])
def test_module_trainer_modes(tmp_path, mode):
  mk = lambda: recml.KerasTrainer(model_dir=str(tmp_path), train_steps=20, steps_per_loop=10, steps_per_eval=3,
                                  continuous_eval_timeout=1)
  if mode in ("eval", "continuous_eval"):
    recml.run_experiment(recml.Experiment(_ModTask(), mk()), "train")
  hist = recml.run_experiment(recml.Experiment(_ModTask(), mk()), mode)
  if mode in ("train", "train_and_eval"):
    assert hist["num_params/trainable"][0] == 4 and len(hist["loss"]) == 2
    assert os.path.exists(os.path.join(tmp_path, "model.pt"))
    assert ckpt.all_steps(os.path.join(tmp_path, "checkpoints")) == [0, 1]
    assert os.path.isdir(os.path.join(tmp_path, "checkpoints", "1", "default"))
  if mode == "train_and_eval":
    assert "val_loss" in hist and "val_mse" in hist
  if mode == "eval":
    assert "loss" in hist


def test_callbacks_and_selective_restore(tmp_path):
  from recml_b200.training import callbacks
  seen = []

  class _Spy(callbacks.Callback):
    def on_train_begin(self, logs=None):
      seen.append("begin")

    def on_epoch_end(self, epoch, logs=None):
      seen.append(("epoch", epoch, "loss" in logs))

    def on_train_end(self, logs=None):
      seen.append("end")

  side = os.path.join(tmp_path, "side")
  mgr = ckpt.CheckpointManager(os.path.join(side, "checkpoints"), item_name="default")
  cbs = [_Spy(), callbacks.EpochCheckpointAndRestoreCallback(mgr, marker_path=os.path.join(side, "marker.txt")),
         callbacks.EpochSummaryCallback(os.path.join(side, "logs"), steps_per_epoch=10)]
  trainer = recml.KerasTrainer(model_dir=str(tmp_path), train_steps=20, steps_per_loop=10, callbacks=cbs,
                               enable_checkpointing=False)
  trainer.train(_ModTask())
  assert seen == ["begin", ("epoch", 0, True), ("epoch", 1, True), "end"]
  assert open(os.path.join(side, "marker.txt")).read() == "COMPLETED"
  assert ckpt.all_steps(os.path.join(side, "checkpoints")) == [0, 1]
  assert os.path.isdir(os.path.join(side, "logs", "train"))
  # the epoch summaries sit at step epoch * steps_per_epoch and carry all four parameter counts
  from tensorboard.backend.event_processing import event_accumulator
  acc = event_accumulator.EventAccumulator(os.path.join(side, "logs", "train")).Reload()
  tags = set(acc.Tags()["scalars"])
  assert {"loss", "learning_rate", "steps_per_second", "num_params/trainable", "num_params/non_trainable",
          "num_params/optimizer", "num_params/total"} <= tags
  assert [e.step for e in acc.Scalars("loss")] == [0, 10]
  assert acc.Scalars("num_params/total")[0].value == 4 + 2 * 4    # a 4 -> 1 layer without bias and two Adam slots

  # selective restore into a fresh state
  def fresh():
    torch.manual_seed(1)
    return recml.State.create(model=nn.Linear(4, 1, bias=False), tx=recml.AdamFactory(learning_rate=0.05).make())
  ckdir = os.path.join(side, "checkpoints")
  full = fresh()
  assert callbacks.restore_state(full, ckdir) == 1
  assert full.optimizer.count == 20 and float(full.optimizer.slots["nu"][0].abs().sum()) > 0
  no_opt = fresh()
  callbacks.restore_state(no_opt, ckdir, restore_optimizer_vars=False, restore_steps=False)
  assert torch.equal(no_opt.params["weight"], full.params["weight"])
  assert no_opt.optimizer.count == 0 and float(no_opt.optimizer.slots["nu"][0].abs().sum()) == 0 and no_opt.step == 0
  no_iter = fresh()
  callbacks.restore_state(no_iter, ckdir, step=0, restore_iterations=False)
  assert no_iter.optimizer.count == 0 and float(no_iter.optimizer.slots["nu"][0].abs().sum()) > 0
  with pytest.raises(ValueError):
    callbacks.restore_state(fresh(), ckdir, step=7)
  with pytest.raises(FileNotFoundError):
    callbacks.restore_state(fresh(), os.path.join(tmp_path, "nothing"))


def test_epoch_checkpoint_manager_round_trip(tmp_path):
  """`save_model_variables` / `restore_model_variables` on a `State`, every second epoch
  (`recml/core/utils/keras_utils.py:36-137`); the reference's names resolve to the same classes."""
  from recml_b200.training import callbacks
  assert callbacks.KerasOrbaxCheckpointManager is callbacks.EpochCheckpointManager
  assert callbacks.restore_keras_model is callbacks.restore_state
  mk = lambda seed: (torch.manual_seed(seed),
                     recml.State.create(model=nn.Linear(4, 2), tx=recml.AdamFactory(learning_rate=0.1).make()))[1]
  st = mk(0)
  mgr = callbacks.EpochCheckpointManager(str(tmp_path / "ck"), max_to_keep=2, save_interval_epochs=2)
  for epoch in range(5):
    st.model(torch.randn(3, 4)).sum().backward()
    st.update()
    mgr.save_model_variables(st, epoch, {"loss": 1.0})
  mgr.wait_until_finished()
  assert ckpt.all_steps(str(tmp_path / "ck")) == [2, 4]
  other = mk(1)
  mgr.restore_model_variables(other, 4)
  assert other.step == 5 and torch.equal(other.params["weight"], st.params["weight"])
  assert torch.equal(other.opt_state["mu"]["weight"], st.opt_state["mu"]["weight"])


def test_training_dataset_that_runs_out_is_a_clear_error(tmp_path):
  with pytest.raises(RuntimeError, match="training dataset ended at step 5 of 12"):
    _trainer(tmp_path, train_steps=12, steps_per_loop=4).train(_Task(n_train=5))


def test_model_parallel_partitioner_takes_the_reference_constructor_arguments():
  p = recml.ModelParallelPartitioner(axes=[("data", 1)], dp_axes=None, rules=None, aot_compile=True, options=None,
                                     devices=None, device="cpu")
  assert p.axis_names == ["data"] and p.dp_axis_names == ["data"]
  assert recml.ModelParallelPartitioner(device="cpu").axis_names == ["batch"]
  with pytest.raises(ValueError, match="At least one axis"):
    recml.ModelParallelPartitioner(axes=[], device="cpu")
  with pytest.raises(ValueError, match="positive or negative"):
    recml.ModelParallelPartitioner(axes=[("data", 1)], dp_axes=0, device="cpu")
