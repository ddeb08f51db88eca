"""Host→device staging must hand every tensor its own pinned buffer until the copy has run."""
import numpy as np
import pytest
import torch

from recml_b200.training import partitioning

pytestmark = pytest.mark.gpu


def test_staging_keeps_equal_shaped_tensors_apart_when_host_runs_ahead():
  part = partitioning.NullPartitioner(torch.device("cuda", 0))
  rng = np.random.default_rng(0)
  # keep the device busy so that many batches are staged before the first copy executes
  a = torch.randn(8192, 8192, device="cuda")
  for _ in range(40):
    a = (a @ a) * 1e-4
  host, dev = [], []
  for step in range(12):
    batch = {"x": rng.integers(0, 1 << 30, 50_000).astype(np.int32),
             "y": rng.integers(0, 1 << 30, 50_000).astype(np.int32),
             "z": rng.integers(0, 1 << 30, 50_000).astype(np.int32)}
    host.append(batch)
    dev.append(part.shard_inputs(batch))
  torch.cuda.synchronize()
  for h, d in zip(host, dev):
    for k in h:
      assert np.array_equal(d[k].cpu().numpy(), h[k]), k


def test_device_prefetcher_delivers_batches_in_order_and_intact():
  from recml_b200.data import prefetch
  part = partitioning.NullPartitioner(torch.device("cuda", 0))
  rng = np.random.default_rng(1)
  host = [{"x": rng.integers(0, 1 << 30, 100_000).astype(np.int32), "y": rng.normal(size=(64, 33)).astype(np.float32)}
          for _ in range(9)]
  pf = prefetch.DevicePrefetcher(iter(host), part, depth=2)
  a = torch.randn(4096, 4096, device="cuda")
  got = []
  for dev in pf:
    a = (a @ a) * 1e-4                      # compute on the consuming stream while later copies are in flight
    got.append(dev)
  torch.cuda.synchronize()
  assert len(got) == len(host)
  for h, d in zip(host, got):
    for k in h:
      assert np.array_equal(d[k].cpu().numpy(), h[k]), k
