"""Criteo pre-batched TFRecord loader, threaded producer and the standalone DLRM trainer."""
import os
import subprocess
import sys

import numpy as np
import pytest

from recml_b200.data import criteo, tfrecord

VOCAB = [50, 7, 1000]
HOT = [3, 1, 5]


def _write(path, n_records, B, seed):
  rng = np.random.default_rng(seed)
  recs, truth = [], []
  for _ in range(n_records):
    labels = rng.integers(0, 2, B)
    dense = rng.normal(size=(B, 13)).astype(np.float32)
    ids = [rng.integers(0, 10 * v, size=(B, m)) for v, m in zip(VOCAB, HOT)]
    ids += [np.zeros((B, 1), np.int64)] * (26 - len(ids))       # the format always carries 26 features
    recs.append(criteo.encode_record(labels, dense, ids))
    truth.append((labels, dense, ids))
  tfrecord.write_tfrecord(path, recs)
  return truth


def test_loader_parses_prebatched_records(tmp_path):
  B = 8
  truth = _write(str(tmp_path / "eval-0.tfrecord"), 3, B, 0)
  dl = criteo.CriteoDataLoader(str(tmp_path / "eval-*.tfrecord"), B, vocab_sizes=VOCAB, multi_hot_sizes=HOT,
                               is_training=False, eval_steps=5)
  batches = list(dl)
  assert len(batches) == 5                       # 3 real + 2 zero-weight padding batches
  for (labels, dense, ids), b in zip(truth, batches):
    np.testing.assert_array_equal(b["label"].numpy(), labels.astype(np.float32))
    np.testing.assert_allclose(b["dense"].numpy(), dense)
    kjt = b["sparse"]
    off = kjt.offsets.numpy()
    assert kjt.keys == ("cat_0", "cat_1", "cat_2") and off[-1] == B * sum(HOT)
    for f in range(3):
      got = kjt.values.numpy()[off[f * B]:off[(f + 1) * B]].reshape(B, HOT[f])
      np.testing.assert_array_equal(got, ids[f] % VOCAB[f])
    assert float(b["weight"].sum()) == B
  assert float(batches[-1]["weight"].sum()) == 0.0
  with pytest.raises(ValueError):
    list(criteo.CriteoDataLoader(str(tmp_path / "eval-*.tfrecord"), B + 1, vocab_sizes=VOCAB, multi_hot_sizes=HOT,
                                 is_training=False))


def test_training_loader_shards_files_and_repeats(tmp_path):
  for i in range(4):
    _write(str(tmp_path / f"train-{i}.tfrecord"), 2, 4, i)
  a = criteo.CriteoDataLoader(str(tmp_path / "train-*"), 4, vocab_sizes=VOCAB, multi_hot_sizes=HOT, process_index=0,
                              process_count=2, shuffle_buffer=3)
  b = criteo.CriteoDataLoader(str(tmp_path / "train-*"), 4, vocab_sizes=VOCAB, multi_hot_sizes=HOT, process_index=1,
                              process_count=2, shuffle_buffer=0)
  assert [os.path.basename(f) for f in a.files] == ["train-0.tfrecord", "train-2.tfrecord"]
  assert [os.path.basename(f) for f in b.files] == ["train-1.tfrecord", "train-3.tfrecord"]
  it = iter(a)
  got = [next(it) for _ in range(11)]            # more than one epoch of 4 records
  assert all(x["dense"].shape == (4, 13) for x in got)


def test_threaded_producer_keeps_order_and_propagates_errors():
  out = list(criteo.ThreadedProducer(range(50), lambda x: {"v": x * x}, num_workers=4, depth=3))
  assert [o["v"] for o in out] == [i * i for i in range(50)]

  def boom(x):
    if x == 5:
      raise RuntimeError("bad record")
    return {"v": x}
  with pytest.raises(RuntimeError):
    list(criteo.ThreadedProducer(range(10), boom, num_workers=2, depth=2))
  it = iter(criteo.ThreadedProducer(iter(int, 1), lambda x: {"v": x}, num_workers=2, depth=2))   # endless source
  assert next(it)["v"] == 0
  it.close()                                      # the producer thread must let go


def test_dummy_batch_shapes():
  b = criteo.dummy_batch(16, HOT, VOCAB)
  assert b["dense"].shape == (16, 13) and b["sparse"].values.numel() == 16 * sum(HOT)
  assert float(b["dense"].max()) <= 0.9 and int(b["sparse"].values.max()) < max(VOCAB)


def test_standalone_trainer_trains_checkpoints_and_evaluates(tmp_path):
  common = [sys.executable, "-m", "recml_b200.examples.dlrm_main", "--batch_size=32", "--vocab_scale=0.00001",
            "--embedding_size=16", "--eval_steps=1", f"--model_dir={tmp_path}", "--producer_workers=2",
            "--producer_depth=4"]
  env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
  r = subprocess.run(common + ["--num_steps=4", "--logging_interval=2", "--eval_interval=2",
                               "--save_checkpoint_interval=2"], capture_output=True, text=True, env=env, timeout=600)
  assert r.returncode == 0, r.stderr[-2000:]
  assert "step 4: loss=" in r.stderr and "Evaluation over 1 steps" in r.stderr
  assert sorted(os.listdir(tmp_path / "checkpoints")) == ["2", "4"]
  r = subprocess.run(common + ["--mode=eval"], capture_output=True, text=True, env=env, timeout=600)
  assert r.returncode == 0, r.stderr[-2000:]
  assert "Found checkpoint at step 4" in r.stderr and "Evaluation over 1 steps" in r.stderr


def test_experiment_launcher_runs_tiny_dlrm(tmp_path):
  env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
  r = subprocess.run([sys.executable, "-m", "recml_b200.examples.run",
                      "--experiment=config:recml_b200.examples.dlrm_experiment.tiny_experiment",
                      f"--experiment=set:trainer.model_dir='{tmp_path}'", "--experiment=set:trainer.train_steps=6",
                      "--mode=train"], capture_output=True, text=True, env=env, timeout=600)
  assert r.returncode == 0, r.stderr[-2000:]
  assert os.path.isdir(tmp_path / "checkpoints")


def test_loader_takes_ids_modulo_vocab_like_numpy_and_rejects_wrong_bag_sizes(tmp_path):
  """Negative ids wrap the way numpy's modulo does; a record whose bags do not have the configured
  multi-hot size is refused."""
  B = 4
  rng = np.random.default_rng(1)
  labels, dense = rng.integers(0, 2, B), rng.normal(size=(B, 13)).astype(np.float32)
  ids = [rng.integers(-10_000, 10_000, size=(B, m)) for m in HOT] + [np.zeros((B, 1), np.int64)] * 23
  tfrecord.write_tfrecord(str(tmp_path / "neg.tfrecord"), [criteo.encode_record(labels, dense, ids)])
  b = next(iter(criteo.CriteoDataLoader(str(tmp_path / "neg.tfrecord"), B, vocab_sizes=VOCAB, multi_hot_sizes=HOT,
                                        is_training=False)))
  want = np.concatenate([np.mod(a, v).reshape(-1) for a, v in zip(ids[:3], VOCAB)])
  np.testing.assert_array_equal(b["sparse"].values.numpy(), want.astype(np.int32))
  wrong = criteo.CriteoDataLoader(str(tmp_path / "neg.tfrecord"), B, vocab_sizes=VOCAB, multi_hot_sizes=[3, 2, 5],
                                  is_training=False)
  with pytest.raises(ValueError):
    next(iter(wrong))


def test_every_module_imports_in_one_process():
  """Both command-line entry points define a `--mode` flag; importing the whole package must still work."""
  import importlib
  import pkgutil
  import recml_b200
  for m in pkgutil.walk_packages(recml_b200.__path__, "recml_b200."):
    importlib.import_module(m.name)
