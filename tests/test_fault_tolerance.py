"""Failure detection without faulting a GPU: missed heartbeats, an injected rank exception, loader
errors surfacing in the consumer, and (GPU) a bounded device-side wait that expires and reports."""
import ctypes
import time

import pytest
import torch

from recml_b200.comm import health
from recml_b200.data import tfrecord_factory as tff


def test_heartbeat_detects_a_silent_rank():
  store = health.DictStore()
  t = [0.0]
  a = health.HealthMonitor(store, 0, 2, interval_s=0.05, timeout_s=1.0, clock=lambda: t[0]).start()
  b = health.HealthMonitor(store, 1, 2, interval_s=0.05, timeout_s=1.0, clock=lambda: t[0],
                           injector=health.FaultInjector("stop_heartbeat:rank=1:step=3")).start()
  time.sleep(0.2)
  t[0] = 0.5
  a.check(step=1); b.check(step=1)
  b.check(step=3)                      # rank 1 stops beating from step 3 on
  time.sleep(0.2)
  a.check(step=3)                      # records the last value it saw
  t[0] = 5.0
  time.sleep(0.2)
  with pytest.raises(health.PeerFailure) as e:
    a.check(step=4)
  assert e.value.ranks == [1]
  b.check(step=4)                      # rank 0 is still alive from rank 1's point of view
  a.stop(); b.stop()


def test_injected_exception_and_parsing():
  inj = health.FaultInjector("raise:rank=0:step=2")
  m = health.HealthMonitor(health.DictStore(), 0, 1, injector=inj).start()
  m.check(step=1)
  with pytest.raises(RuntimeError, match="injected failure"):
    m.check(step=2)
  m.stop()
  assert not health.FaultInjector("").fires("raise", 0, 0)


def test_loader_thread_exception_reaches_the_consumer(tmp_path):
  p = tmp_path / "bad.tfrecord"
  p.write_bytes(b"\x05\x00\x00\x00\x00\x00\x00\x00garbage-garbage-garbage")
  fac = tff.TFDatasetFactory(input_path=str(p), feature_spec={"x": tff.FixedLenFeature((1,))}, global_batch_size=2,
                             prefetch_buffer_size=2)
  with pytest.raises(IOError):
    next(fac.make())


def _run_leave_job(world, announce, tmp_path):
  import os
  import torch.multiprocessing as mp
  from tests import dist_utils, dist_workers
  ctx = mp.spawn(dist_workers.leave_entry, args=(world, dist_utils._free_port(), str(tmp_path), announce),
                 nprocs=world, join=False, start_method="spawn")
  deadline = time.time() + 60
  while time.time() < deadline and not ctx.join(timeout=1.0):
    pass
  for p in ctx.processes:
    assert not p.is_alive(), "a rank is still waiting for the one that left"
  return [torch.load(os.path.join(tmp_path, f"rank{r}.pt"), weights_only=False) for r in range(world)]


def test_announced_leave_is_seen_before_the_next_collective(tmp_path):
  """gloo ranks: the last rank tells the store that it leaves, takes part in one more step and goes; the
  survivors' host check raises `PeerFailure` naming it before they launch another collective."""
  res = _run_leave_job(3, True, tmp_path)
  assert res[2] == {"left_at": 3}
  for r in res[:2]:
    assert r["detected"] == [2] and r["collective_error"] is None
    assert r["steps_done"] == 4          # exactly the steps all ranks took part in (the leaver's last one included)


def test_silent_exit_ends_the_collective_and_the_heartbeat_names_the_rank(tmp_path):
  """gloo ranks: the last rank exits without a word.  The survivor's next collective ends with an error (closed
  socket or the short process-group timeout) instead of hanging, and the heartbeat check then raises
  `PeerFailure` for that rank within the heartbeat timeout."""
  res = _run_leave_job(2, False, tmp_path)
  assert res[1] == {"left_at": 3}
  assert res[0]["detected"] == [1]
  assert res[0]["steps_done"] == 3
  if res[0]["collective_error"] is not None:      # otherwise the heartbeat fired before the collective was tried
    assert res[0]["seconds"] < 9.0


@pytest.mark.gpu
def test_device_wait_expires_and_reports_status():
  from recml_b200.ops import _lib
  lib = _lib.cuda()
  flag = torch.zeros(1, dtype=torch.int64, device="cuda")          # nobody raises it
  status = torch.zeros(4, dtype=torch.int32, device="cuda")
  result = torch.full((1,), -1, dtype=torch.int32, device="cuda")
  t0 = time.time()
  rc = lib.recml_wait_probe(_lib.ptr(flag), ctypes.c_ulonglong(1), ctypes.c_ulonglong(20_000_000), _lib.ptr(status),
                            ctypes.c_int(7), _lib.ptr(result), _lib.stream())
  assert rc == 0
  torch.cuda.synchronize()
  assert time.time() - t0 < 5.0
  assert result.item() == 0 and status.tolist()[:2] == [2, 7]      # kPeerTimeout, detail
  # the context is still usable, and a raised flag is seen at once
  flag.fill_(3)
  status.zero_()
  lib.recml_wait_probe(_lib.ptr(flag), ctypes.c_ulonglong(3), ctypes.c_ulonglong(20_000_000), _lib.ptr(status),
                       ctypes.c_int(7), _lib.ptr(result), _lib.stream())
  torch.cuda.synchronize()
  assert result.item() == 1 and status.tolist()[0] == 0


@pytest.mark.gpu
def test_no_checkpoint_is_written_after_a_device_error_status(tmp_path):
  """A kernel that gave up on a wait leaves a status word; the trainer looks at it before every checkpoint and at
  loop ends, so a step whose collective timed out can never be committed as a good checkpoint.  The status is
  produced by the bounded-wait probe (a flag nothing raises), not by a fault."""
  import os
  import numpy as np
  from torch import nn
  import recml_b200 as recml
  from recml_b200 import ckpt
  from recml_b200.data import iterator as iterator_lib
  from recml_b200.ops import _lib

  class Data:
    def __iter__(self):
      rng = np.random.default_rng(0)
      for _ in range(100):
        x = rng.normal(size=(8, 4)).astype(np.float32)
        yield {"x": x, "y": x.sum(1, keepdims=True)}

  class Task(recml.Task):
    steps = 0

    def create_datasets(self):
      return iterator_lib.IterableIterator(Data())

    def create_state(self, batch, rng):
      return recml.State.create(model=nn.Linear(4, 1).cuda(), tx=recml.AdamFactory(learning_rate=0.05).make())

    def train_step(self, batch, state, rng):
      loss = ((state.model(batch["x"]) - batch["y"]) ** 2).mean()
      loss.backward()
      state.update()
      Task.steps += 1
      if Task.steps == 2:     # a wait that runs out, reported through the library's status word of this device
        flag = torch.zeros(1, dtype=torch.int64, device="cuda")
        result = torch.zeros(1, dtype=torch.int32, device="cuda")
        _lib.cuda().recml_wait_probe(_lib.ptr(flag), ctypes.c_ulonglong(1), ctypes.c_ulonglong(5_000_000),
                                     _lib.ptr(_lib.status_buffer()), ctypes.c_int(9), _lib.ptr(result), _lib.stream())
      return state, {"loss": recml.metrics.mean(loss.detach())}

    def eval_step(self, batch, state):
      return {"loss": recml.metrics.mean(((state.model(batch["x"]) - batch["y"]) ** 2).mean())}

  _lib.check_status()
  trainer = recml.Trainer(partitioner=recml.DataParallelPartitioner(device="cuda"), model_dir=str(tmp_path),
                          train_steps=12, steps_per_loop=4, checkpoint_interval=4)
  with pytest.raises(_lib.DeviceStatusError):
    recml.run_experiment(recml.Experiment(Task(), trainer), "train")
  assert ckpt.all_steps(os.path.join(tmp_path, "checkpoints")) == []
  _lib.check_status()          # the word was cleared by the raise
