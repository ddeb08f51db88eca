"""Sharded-embedding collective microbenchmark: fused NVLink kernels vs the NCCL stand-in.

Workload: `--tables` tables with vocabularies log-spaced in [1 M, 40 M] x `--vocab-scale`, dims
cycling through {64, 128, 256}, fp32 weights, bf16 pooled outputs, bag sizes log-spaced in
[1, 100], Zipf(1.05) ids, row-wise Adagrad.  For every per-GPU batch of the sweep it times, on the
device and as the max over ranks,
  forward   ids exchange + lookup + pooling + pooled all-to-all (+ recording what backward needs)
  backward  gradient all-to-all + dedup (radix sort of the occurrence list, counted in the roofline) + row-wise
            Adagrad update
for `backend="fused"` (peer-memory kernels, `csrc/cuda/embedding.cu`) and `backend="collective"`
(NCCL `all_gather` / `all_to_all_single` + torch ops: the stand-in for the reference's own NCCL
path, which cannot be installed).  Each fused number is also reported as a fraction of its
roofline: the slower of (HBM bytes the busiest rank must move / measured copy bandwidth) and
(bytes that rank must put on NVLink / 770 GB/s per direction).

    python -m torch.distributed.run --nproc-per-node 8 -m recml_b200.benchmarks.embedding_bench \
        --batches 1024,8192,32768
"""
from __future__ import annotations

import argparse
import gc
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from recml_b200 import embedding as emb
from recml_b200.data import synthetic
from recml_b200.utils import streams

NVLINK_BPS = 770e9          # measured peer-copy bandwidth per direction per B200 over NVSwitch (900e9 nominal)


def _hbm_bps() -> float:
  here = os.path.dirname(os.path.abspath(__file__))
  path = os.path.join(here, "..", "..", "MEASURED_PEAKS.json")
  try:
    with open(path) as f:
      return float(json.load(f)["hbm_gbs"]) * 1e9
  except (OSError, KeyError, ValueError):
    return 6.65e12         # a measured B200 copy bandwidth, used when the file is absent


def geometry(n_tables: int, vocab_scale: float):
  vocabs = np.exp(np.linspace(np.log(1e6), np.log(40e6), n_tables))
  rng = np.random.default_rng(7)
  rng.shuffle(vocabs)
  vocabs = [max(1000, int(v * vocab_scale)) for v in vocabs]
  dims = [(64, 128, 256)[i % 3] for i in range(n_tables)]
  bags = [max(1, int(round(b))) for b in np.exp(np.linspace(0.0, np.log(100.0), n_tables))]
  rng.shuffle(bags)
  return vocabs, dims, [int(b) for b in bags]


def make_batch(rng, B, vocabs, bags, names):
  vals = [synthetic.zipf_ids(rng, v, (B, b), 1.05).reshape(-1) for v, b in zip(vocabs, bags)]
  lens = np.concatenate([np.full(B, b, dtype=np.int64) for b in bags])
  off = np.zeros(lens.size + 1, dtype=np.int32)
  off[1:] = np.cumsum(lens)
  return emb.KeyedJagged(tuple(names), torch.from_numpy(np.concatenate(vals).astype(np.int32)), torch.from_numpy(off), None, B)


def roofline(module, kjt_dev, B, world, hbm_bps):
  """Per-rank byte counts of the busiest rank → (fwd floor s, bwd floor s, details).  Collective:
  the ids of every rank are gathered on the device to count rows and distinct rows per owner."""
  P = emb.Placement
  names = module.feature_names
  fwd_hbm = np.zeros(world)
  bwd_hbm = np.zeros(world)
  wire = np.zeros(world)
  off = kjt_dev.offsets
  for fi, name in enumerate(names):
    tp = module.plan.tables[module.feature_to_table[name]]
    D = tp.dim
    mine = kjt_dev.values[int(off[fi * B]):int(off[(fi + 1) * B])].long()
    if world > 1:
      parts = [torch.empty_like(mine) for _ in range(world)]
      dist.all_gather(parts, mine)
      ids = torch.cat(parts)
    else:
      ids = mine
    if tp.placement is P.TABLE_WISE:
      owners = torch.full_like(ids, tp.owner)
      wire[tp.owner] += (world - 1) * B * D * 2
    else:
      owners = (ids % world + tp.rotation) % world
      wire += (world - 1) * B * D * 2
    for r in range(world):
      sel = ids[owners == r]
      if sel.numel() == 0:
        continue
      uniq = int(torch.unique(sel).numel())
      fwd_hbm[r] += sel.numel() * D * 4                      # rows gathered
      bwd_hbm[r] += sel.numel() * D * 2 + 2 * uniq * D * 4    # gradient vectors read + rows read and written
      # de-duplication: the radix sort of the (row, gradient index) pairs reads every pair twice and writes it once
      # per 9-bit pass over the significant bits of the local row number
      local_rows = tp.vocab if tp.placement is P.TABLE_WISE else (tp.vocab + world - 1) // world
      passes = max(1, -(-max(1, int(local_rows) - 1).bit_length() // 9))
      bwd_hbm[r] += sel.numel() * 24 * passes
  f = max(fwd_hbm.max() / hbm_bps, wire.max() / NVLINK_BPS)
  b = max(bwd_hbm.max() / hbm_bps, wire.max() / NVLINK_BPS)
  return f, b, {"fwd_hbm_gb": fwd_hbm.max() / 1e9, "bwd_hbm_gb": bwd_hbm.max() / 1e9, "nvlink_gb": wire.max() / 1e9}


def run_case(backend, B, vocabs, dims, bags, device, rank, world, iters, warmup):
  names = [f"t{i}" for i in range(len(vocabs))]
  specs = {n: emb.EmbeddingSpec(v, d, combiner="sum", initializer=emb.specs.uniform_init(0.01))
           for n, v, d in zip(names, vocabs, dims)}
  cfg = emb.ShardedEmbeddingConfig(specs, emb.RowWiseAdagradOptimizerSpec(0.01), backend=backend,
                                   ids_per_sample=dict(zip(names, bags)))
  module = emb.ShardedEmbedding(cfg, device=device)
  rng = np.random.default_rng(100 + rank)
  host = [make_batch(rng, B, vocabs, bags, names) for _ in range(2)]
  dev = [k.to_device(device) for k in host]
  grads = None
  ev = lambda: torch.cuda.Event(enable_timing=True)
  fwd_ms, bwd_ms = [], []
  for it in range(warmup + iters):
    torch.cuda.synchronize()
    if world > 1:
      dist.barrier()
    e0, e1, e2 = ev(), ev(), ev()
    e0.record()
    out = module(dev[it % 2])
    outs = list(out.values()) if isinstance(out, dict) else [out]
    e1.record()
    if grads is None:
      grads = [torch.randn_like(o) * 1e-3 for o in outs]
    torch.autograd.backward(outs, grads)
    # the sort and the table update run on side streams of their own: the timed stream waits for them
    streams.join("emb_bwd", "emb_sort", device=device)
    e2.record()
    torch.cuda.synchronize()
    if it >= warmup:
      fwd_ms.append(e0.elapsed_time(e1))
      bwd_ms.append(e1.elapsed_time(e2))
  t = torch.tensor([float(np.median(fwd_ms)), float(np.median(bwd_ms))], device=device)
  if world > 1:
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
  gathered = dev[0]
  placements = {}
  for tp in module.plan.tables.values():
    placements[tp.placement.value] = placements.get(tp.placement.value, 0) + 1
  return float(t[0]), float(t[1]), module, gathered, placements


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--tables", type=int, default=26)
  ap.add_argument("--vocab-scale", type=float, default=1.0)
  ap.add_argument("--batches", default="1024,8192,32768")
  ap.add_argument("--backends", default="fused,collective")
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--warmup", type=int, default=3)
  args = ap.parse_args()
  world = int(os.environ.get("WORLD_SIZE", "1"))
  rank = int(os.environ.get("RANK", "0"))
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  device = torch.device("cuda", local)
  if world > 1:
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)
  vocabs, dims, bags = geometry(args.tables, args.vocab_scale)
  hbm = _hbm_bps()
  for B in [int(x) for x in args.batches.split(",")]:
    row = {"per_gpu_batch": B, "n_gpus": world, "tables": args.tables, "ids_per_sample": int(sum(bags))}
    for backend in args.backends.split(","):
      if backend == "collective" and world == 1:
        continue
      f, b, module, gathered, placements = run_case(backend, B, vocabs, dims, bags, device, rank, world, args.iters,
                                                    args.warmup)
      row[f"{backend}_fwd_ms"], row[f"{backend}_bwd_ms"] = round(f, 4), round(b, 4)
      if backend == "fused":
        ff, bf, det = roofline(module, gathered, B, world, hbm)
        row.update({"fwd_floor_ms": round(ff * 1e3, 4), "bwd_floor_ms": round(bf * 1e3, 4),
                    "fwd_frac_of_roofline": round(ff * 1e3 / f, 3), "bwd_frac_of_roofline": round(bf * 1e3 / b, 3),
                    "placements": placements, **{k: round(v, 3) for k, v in det.items()}})
      del module, gathered
      gc.collect()                 # module and backend reference each other: without this the tables stay allocated
      torch.cuda.empty_cache()
    if "fused_fwd_ms" in row and "collective_fwd_ms" in row:
      row["fwd_speedup_vs_nccl"] = round(row["collective_fwd_ms"] / row["fused_fwd_ms"], 2)
      row["bwd_speedup_vs_nccl"] = round(row["collective_bwd_ms"] / row["fused_bwd_ms"], 2)
    if rank == 0:
      print(json.dumps(row), flush=True)
  if world > 1:
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
  main()
