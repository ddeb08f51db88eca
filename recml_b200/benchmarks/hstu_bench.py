"""HSTU tokens/s: the packed generative-retrieval training step (item table 10 M × 256 row-sharded,
8 layers, 4 heads × 64, sequence lengths power-law in [16, 4096] with mean ≈ 512, 128 sequences per
GPU, sampled softmax with 512 uniform + 512 in-batch negatives).  Device-timed, max over ranks.

  python -m recml_b200.benchmarks.hstu_bench [--steps K] [--warmup W] [--vocab V]
  (multi-GPU: launch with torch.distributed.run, one process per GPU)
"""
from __future__ import annotations

import argparse
import json
import os


def run(steps: int = 10, warmup: int = 3, vocab: int = 10_000_000, use_graph: bool = False, layers: int = 8,
        sequences: int = 128, timeline: str | None = None) -> dict:
  import torch
  import torch.distributed as dist
  from recml_b200.examples import hstu_experiment as E
  from recml_b200.ops import _lib
  from recml_b200.training import partitioning
  world = dist.get_world_size() if dist.is_initialized() else 1
  device = torch.device("cuda", torch.cuda.current_device())
  cfg = E.HSTUModelConfig(vocab_size=vocab, num_layers=layers, sequences_per_batch=sequences)
  task = E.HSTUTask(cfg, E.PackedSequenceFactory(model=cfg, num_batches=4))
  part = partitioning.DataParallelPartitioner(use_cuda_graph=use_graph)
  it = task.create_datasets()
  host = [next(it) for _ in range(4)]
  dev = [part.shard_inputs(b) for b in host]
  state = part.partition_init(lambda b: task.create_state(b, torch.Generator().manual_seed(0)))(dev[0])
  rng = torch.Generator(device=device)
  tokens = sum(int(b["input_ids"].numel()) for b in host) / len(host)
  i = [0]

  def step():
    nonlocal state
    state, m = task.train_step(dev[i[0] % 4], state, rng)
    i[0] += 1
    return m

  for _ in range(max(warmup, 3)):
    step()
  _lib.check_status(device)
  if world > 1:
    dist.barrier()
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(steps):
    m = step()
  e1.record()
  if world > 1:
    dist.barrier()
  torch.cuda.synchronize()
  ms = torch.tensor([e0.elapsed_time(e1)], device=device)
  tok = torch.tensor([tokens], device=device)
  if world > 1:
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    dist.all_reduce(tok)
  _lib.check_status(device)
  ms_step = float(ms.item()) / steps
  extra = {}
  if timeline:        # after the timed region: the profiler slows the steps it records
    from recml_b200.utils import profiling
    extra["timeline"] = profiling.kernel_timeline(step, timeline)
  return {**extra, "metric": "hstu_train_tokens_per_sec", "value": float(tok.item()) / (ms_step * 1e-3), "unit": "tokens/s",
          "ms_per_step": ms_step, "tokens_per_step": float(tok.item()), "n_gpus": world,
          "loss": float(m["loss"].localize().compute()),
          "config": {"vocab": vocab, "model_dim": cfg.model_dim, "layers": layers, "heads": cfg.num_heads,
                     "sequences_per_gpu": sequences, "negatives": "512 uniform + 512 in-batch"}}


def main():
  import torch
  import torch.distributed as dist
  ap = argparse.ArgumentParser()
  ap.add_argument("--steps", type=int, default=10)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--vocab", type=int, default=10_000_000)
  ap.add_argument("--layers", type=int, default=8)
  ap.add_argument("--sequences", type=int, default=128)
  ap.add_argument("--timeline", default=None, help="write the per-kernel totals and launch order of one step here")
  args = ap.parse_args()
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  if int(os.environ.get("WORLD_SIZE", "1")) > 1:
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
  out = run(args.steps, args.warmup, args.vocab, layers=args.layers, sequences=args.sequences, timeline=args.timeline)
  if int(os.environ.get("RANK", "0")) == 0:
    print(json.dumps(out))
  if dist.is_initialized():
    dist.destroy_process_group()


if __name__ == "__main__":
  main()
