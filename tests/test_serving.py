"""Export after training and forward-only use of the exported model (`recml_b200.serving`)."""
import json
import os

import torch

from recml_b200 import config as C, run_experiment, serving
from recml_b200.examples import dlrm_experiment as D
from tests import dist_utils


def test_dlrm_export_load_predict(tmp_path):
  """The trainer's final `export_model` writes weights + recipe; the loaded module predicts what the trained
  one predicts, and batch inference returns host tensors in order."""
  cfg = D.tiny_experiment(model_dir=str(tmp_path / "run"), train_steps=6, batch_size=64)
  cfg.trainer.partitioner = C.Config(__import__("recml_b200").DataParallelPartitioner, device="cpu")
  exp = C.build(cfg)
  run_experiment(exp, "train")
  export_dir = tmp_path / "run" / "export"
  recipe = json.load(open(export_dir / "model.json"))
  assert recipe["builder"] == "recml_b200.models.dlrm:DLRMDCNv2" and recipe["step"] == 6
  assert os.path.exists(export_dir / "embedding_spec.json")
  model = serving.load(str(export_dir), device="cpu")
  pred = serving.Predictor(model, forward=lambda m, b: m(b["dense"], b["sparse"]))
  it = exp.task.create_datasets()[0]
  batches = [next(it) for _ in range(3)]
  outs = list(serving.batch_inference(pred, batches))
  assert len(outs) == 3 and outs[0].shape == (64,)
  # the same weights as a fresh restore of the last checkpoint into the training module
  state = exp.task.create_state(batches[0], torch.Generator().manual_seed(0))
  from recml_b200 import ckpt
  mgr = ckpt.CheckpointManager(str(tmp_path / "run" / "checkpoints"), async_save=False)
  state.load_state_dict(mgr.restore(mgr.latest_step(), target=state.state_dict()))
  state.model.eval()
  with torch.no_grad():
    ref = state.model(batches[1]["dense"], batches[1]["sparse"])
  torch.testing.assert_close(outs[1], ref, rtol=1e-5, atol=1e-6)


def test_export_from_two_ranks_loads_on_one(tmp_path):
  """Tables sharded over 2 ranks at training time are served by a single process."""
  d = str(tmp_path / "run")
  res = dist_utils.run_ranks("dlrm_tiny_export", 2, "gloo", "cpu", d)
  model = serving.load(os.path.join(d, "export"), device="cpu")
  for name, t in res[0]["tables"].items():
    torch.testing.assert_close(model.embedding.gather_table(name), t)
