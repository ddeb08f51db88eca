"""Launch helper for multi-process tests (gloo on CPU, NCCL on GPUs), 127.0.0.1 rendezvous."""
import glob
import os
import socket
import tempfile

import torch
import torch.multiprocessing as mp

from tests import dist_workers


def _free_port() -> int:
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def run_ranks(fn_name: str, world: int, backend: str, *args, timeout: float = 300.0):
  """Runs `dist_workers.<fn_name>(rank, world, *args)` on `world` processes; returns the list of
  per-rank results."""
  result_dir = tempfile.mkdtemp()
  ctx = mp.spawn(dist_workers.entry, args=(world, backend, _free_port(), fn_name, args, result_dir),
                 nprocs=world, join=False, start_method="spawn")
  import time
  deadline = time.time() + timeout
  ok = False
  try:
    while time.time() < deadline:
      if ctx.join(timeout=1.0):   # returns True once every process has exited cleanly
        ok = True
        break
  except Exception:  # a rank raised: its traceback is in the .err file
    pass
  errs = glob.glob(os.path.join(result_dir, "*.err"))
  if errs or not ok:
    for p in ctx.processes:
      if p.is_alive():
        p.terminate()
  if errs:
    raise RuntimeError("rank failed:\n" + open(errs[0]).read())
  if not ok:
    raise TimeoutError(f"{fn_name} did not finish within {timeout}s")
  return [torch.load(os.path.join(result_dir, f"rank{r}.pt"), weights_only=False) for r in range(world)]
