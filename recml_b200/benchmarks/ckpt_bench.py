"""Checkpoint save / restore throughput on the host (no GPU): one large leaf (a table shard) and a few small
ones through `CheckpointManager`, raw or zstd-compressed, as zarr leaves or as an OCDBT store.

  python -m recml_b200.benchmarks.ckpt_bench --rows 4000000 --dim 64 [--compressor zstd] [--ocdbt] [--no-checksums]

Prints one JSON line: bytes, seconds and MB/s of the save (until the commit) and of the restore, and what the
directory holds.  The page cache is warm after the save, so the restore figure is that of memory-speed reads.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import tempfile
import time


def run(rows: int = 4_000_000, dim: int = 64, compressor: str | None = None, use_ocdbt: bool = False,
        checksums: bool = True, directory: str | None = None) -> dict:
  import torch
  from recml_b200 import ckpt
  os.environ["RECML_CKPT_CHECKSUMS"] = "1" if checksums else "0"
  d = tempfile.mkdtemp(dir=directory)
  try:
    state = {"params": {"table": torch.randn(rows, dim), "w": torch.randn(1024, 1024)}, "step": torch.tensor(3)}
    nbytes = sum(t.numel() * t.element_size() for t in (state["params"]["table"], state["params"]["w"]))
    mgr = ckpt.CheckpointManager(d, max_to_keep=2, compressor=compressor, use_ocdbt=use_ocdbt)
    t = time.time()
    mgr.save(1, state)
    mgr.wait_until_finished()
    save_s = time.time() - t
    t = time.time()
    out = mgr.restore(1, target=state)
    restore_s = time.time() - t
    assert torch.equal(out["params"]["table"], state["params"]["table"])
    files = sum(len(fs) for _, _, fs in os.walk(d))
    on_disk = sum(os.path.getsize(os.path.join(dp, f)) for dp, _, fs in os.walk(d) for f in fs)
    return {"bytes": nbytes, "save_s": round(save_s, 3), "save_mb_per_s": round(nbytes / 1e6 / save_s),
            "restore_s": round(restore_s, 3), "restore_mb_per_s": round(nbytes / 1e6 / restore_s),
            "files": files, "bytes_on_disk": on_disk, "compressor": compressor, "ocdbt": use_ocdbt,
            "checksums": checksums}
  finally:
    shutil.rmtree(d, ignore_errors=True)


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--rows", type=int, default=4_000_000)
  ap.add_argument("--dim", type=int, default=64)
  ap.add_argument("--compressor", default=None)
  ap.add_argument("--ocdbt", action="store_true")
  ap.add_argument("--no-checksums", action="store_true")
  ap.add_argument("--dir", default=None, help="where to create the scratch directory (default: the system's)")
  a = ap.parse_args()
  print(json.dumps(run(a.rows, a.dim, a.compressor, a.ocdbt, not a.no_checksums, a.dir)))


if __name__ == "__main__":
  main()
