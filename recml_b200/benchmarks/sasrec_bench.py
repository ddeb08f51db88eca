"""SASRec training and full-vocabulary evaluation throughput.

Workload: 2 causal transformer blocks, hidden 256, 4 heads, FFN 1024, learned positions, length 200,
batch 512 sequences per GPU of length uniform[5, 200] (right-aligned), item table 20 M x 256
row-sharded, Zipf(1.1) ids; training = BCE on one positive and one sampled negative per position;
evaluation = rank of the held-out last item against the WHOLE vocabulary through the fused
all-gather -> GEMM -> rank-count kernel, then NDCG@10 / Recall@10 / MRR.  Device-timed, max over ranks.

  python -m recml_b200.benchmarks.sasrec_bench [--steps K] [--vocab V]
  (multi-GPU: launch with torch.distributed.run, one process per GPU)
"""
from __future__ import annotations

import argparse
import json
import os


def run(steps: int = 10, warmup: int = 3, vocab: int = 20_000_000, batch: int = 512) -> dict:
  import torch
  import torch.distributed as dist
  from recml_b200.examples import sasrec_experiment as E
  from recml_b200.ops import _lib
  from recml_b200.training import partitioning
  world = dist.get_world_size() if dist.is_initialized() else 1
  device = torch.device("cuda", torch.cuda.current_device())
  cfg = E.SASRecConfig(vocab_size=vocab, batch_size=batch)
  task = E.SASRecTask(cfg, E.SequenceFactory(model=cfg, num_batches=4))
  part = partitioning.DataParallelPartitioner()
  it = task.create_datasets()
  host = [next(it) for _ in range(4)]
  dev = [part.shard_inputs(b) for b in host]
  state = part.partition_init(lambda b: task.create_state(b, torch.Generator().manual_seed(0)))(dev[0])
  rng = torch.Generator(device=device)
  tokens = sum(float(b["padding_mask"].sum()) for b in host) / len(host)

  def timed(fn, n):
    for i in range(max(warmup, 3)):
      fn(i)
    _lib.check_status(device)
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
      fn(i)
    e1.record()
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / n], device=device)
    if world > 1:
      dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms)

  box = {"state": state, "m": None}

  def train(i):
    box["state"], box["m"] = task.train_step(dev[i % 4], box["state"], rng)

  def evaluate(i):
    with torch.no_grad():
      box["m"] = task.eval_step(dev[i % 4], box["state"])

  train_ms = timed(train, steps)
  loss = float(box["m"]["loss"].localize().compute())
  eval_ms = timed(evaluate, max(3, steps // 2))
  _lib.check_status(device)
  return {"metric": "sasrec_train_sequences_per_sec", "value": batch * world / (train_ms * 1e-3), "unit": "sequences/s",
          "ms_per_step": train_ms, "tokens_per_sec": tokens * world / (train_ms * 1e-3), "n_gpus": world, "loss": loss,
          "eval": {"ms_per_step": eval_ms, "sequences_per_sec": batch * world / (eval_ms * 1e-3),
                   "scored_pairs_per_sec": batch * world * float(vocab) / (eval_ms * 1e-3),
                   "ndcg@10": float(box["m"]["ndcg@10"].localize().compute())},
          "config": {"vocab": vocab, "batch_per_gpu": batch, "max_len": cfg.max_positions, "model_dim": cfg.model_dim,
                     "layers": cfg.num_layers, "heads": cfg.num_heads}}


def main():
  import torch
  import torch.distributed as dist
  ap = argparse.ArgumentParser()
  ap.add_argument("--steps", type=int, default=10)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--vocab", type=int, default=20_000_000)
  ap.add_argument("--batch", type=int, default=512)
  args = ap.parse_args()
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  if int(os.environ.get("WORLD_SIZE", "1")) > 1:
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
  out = run(args.steps, args.warmup, args.vocab, args.batch)
  if int(os.environ.get("RANK", "0")) == 0:
    print(json.dumps(out))
  if dist.is_initialized():
    dist.destroy_process_group()


if __name__ == "__main__":
  main()
