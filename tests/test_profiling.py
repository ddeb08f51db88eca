"""Tracing / profiling helpers on a machine without a GPU: scopes are no-ops, timers report nothing, the
progress reporter measures steps per second and the share of timed side work, the trace is a Chrome trace."""
import json

import pytest
import time

import torch

from recml_b200.data.preprocessing import PreprocessingMode
from recml_b200.utils import profiling


def test_scopes_and_device_timers_without_gpu():
  with profiling.step_annotation("train", 3), profiling.named_scope("dense"):
    x = torch.ones(4).sum()
  assert float(x) == 4.0
  t = profiling.DeviceStepTimer()
  t.start()
  if not torch.cuda.is_available():
    assert t.stop() is None
    timers = profiling.PhaseTimers()
    with timers.phase("lookup"):
      pass
    assert timers.summary() == {}


def test_report_progress_rates_and_shares():
  rp = profiling.ReportProgress(every_secs=0.05)
  rp(0)
  with rp.timed("checkpoint"):
    time.sleep(0.03)
  time.sleep(0.04)
  rp(10)
  assert rp.steps_per_sec is not None and 1 < rp.steps_per_sec < 400


def test_trace_writes_a_chrome_trace(tmp_path):
  path = str(tmp_path / "trace.json")
  with profiling.trace(path):
    torch.randn(64, 64) @ torch.randn(64, 64)
  with open(path) as f:
    assert "traceEvents" in json.load(f)
  with profiling.trace(str(tmp_path / "off.json"), enabled=False):
    pass
  assert not (tmp_path / "off.json").exists()


def test_preprocessing_mode_values():
  assert str(PreprocessingMode.TRAINING) == "training" and PreprocessingMode("eval") is PreprocessingMode.EVAL
  assert {m.value for m in PreprocessingMode} == {"training", "eval", "serving"}


def test_report_progress_writes_scalars_every_n_steps():
  class W:
    def __init__(self):
      self.rows = []
    def write_scalars(self, step, scalars):
      self.rows.append((step, dict(scalars)))
  w = W()
  rp = profiling.ReportProgress(every_secs=1e9, writer=w, every_steps=5)
  for step in range(12):
    rp(step)
  assert [s for s, _ in w.rows] == [5, 10]
  assert set(w.rows[0][1]) == {"steps_per_sec", "uptime"} and w.rows[0][1]["steps_per_sec"] > 0


@pytest.mark.gpu
def test_kernel_timeline_lists_the_kernels_of_a_step(tmp_path):
  x = torch.randn(1 << 20, device="cuda")
  def step():
    (x * 2).sum()
  out = profiling.kernel_timeline(step, str(tmp_path / "t.txt"), steps=4, pick=2)
  text = open(tmp_path / "t.txt").read()
  assert out["kernels_per_step"] >= 2 and "----" in text and "us x" in text
