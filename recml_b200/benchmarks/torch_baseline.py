"""Stand-in baseline: DLRM-DCNv2 training step in plain PyTorch + NCCL + cuBLAS.

The reference cannot be installed on this machine (no jax / flax / TPU kernels), so this file is
the comparison arm that CAN be measured on the same box: the same model, batch geometry, optimizers
and synthetic data as `bench.py`, built only from stock parts —
  embeddings   table-wise sharded fp32 tables, `all_to_all_single` of ids, `F.embedding_bag`,
               `all_to_all_single` of bf16 pooled vectors (and of their gradients in backward),
               `torch.unique` + `index_add_` + row-wise Adagrad in torch ops
  dense        `F.linear` under bf16 autocast (cuBLAS), low-rank DCNv2 cross in torch ops
  gradients    one flat NCCL `all_reduce` of all dense gradients, fused `torch.optim.Adam`
None of this framework's kernels or engine is on this path.  It prints the same JSON line as
`bench.py` with `"impl": "torch+nccl+cublas stand-in"`; it is NOT the reference and is labelled so.

    python -m torch.distributed.run --nproc-per-node 8 -m recml_b200.benchmarks.torch_baseline --steps 20
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from recml_b200.data import synthetic


class _A2A(torch.autograd.Function):
  """all_to_all_single whose backward is the reverse exchange."""

  @staticmethod
  def forward(ctx, x, out_splits, in_splits):
    ctx.splits = (out_splits, in_splits)
    out = x.new_empty((sum(out_splits),) + x.shape[1:])
    dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits)
    return out

  @staticmethod
  def backward(ctx, g):
    out_splits, in_splits = ctx.splits
    gx = g.new_empty((sum(in_splits),) + g.shape[1:])
    dist.all_to_all_single(gx, g.contiguous(), in_splits, out_splits)
    return gx, None, None


class ShardedTables:
  """Table-wise placement (largest gather cost first onto the least loaded rank)."""

  def __init__(self, vocabs, bags, dim, rank, world, device, lr=0.01):
    self.vocabs, self.bags, self.dim, self.rank, self.world, self.lr = vocabs, bags, dim, rank, world, lr
    load = [0.0] * world
    self.owner = [0] * len(vocabs)
    for f in sorted(range(len(vocabs)), key=lambda i: -bags[i]):
      o = min(range(world), key=lambda r: load[r])
      self.owner[f] = o
      load[o] += bags[f]
    self.mine = [f for f in range(len(vocabs)) if self.owner[f] == rank]
    g = torch.Generator(device=device).manual_seed(rank)
    self.tables = {f: (torch.rand(vocabs[f], dim, device=device, generator=g) - 0.5) * 0.02 for f in self.mine}
    self.acc = {f: torch.full((vocabs[f],), 0.1, device=device) for f in self.mine}
    self.by_owner = [[f for f in range(len(vocabs)) if self.owner[f] == r] for r in range(world)]

  def forward(self, ids: list[torch.Tensor]) -> tuple[torch.Tensor, list]:
    """ids[f]: [B, bag_f] int64 on every rank → pooled [B, F, dim] bf16 (autograd-connected)."""
    W, B = self.world, ids[0].shape[0]
    send = torch.cat([ids[f].reshape(-1) for r in range(W) for f in self.by_owner[r]]) if W > 1 else None
    per_owner = [sum(B * self.bags[f] for f in self.by_owner[r]) for r in range(W)]
    mine_n = sum(B * self.bags[f] for f in self.mine)
    if W > 1:
      recv = send.new_empty(W * mine_n)
      dist.all_to_all_single(recv, send, [mine_n] * W, per_owner)
      recv = recv.view(W, mine_n)
    pooled, saved = [], []
    at = 0
    for f in self.mine:
      n = B * self.bags[f]
      got = recv[:, at:at + n].reshape(W * B, self.bags[f]) if W > 1 else ids[f]
      at += n
      out = F.embedding_bag(got, self.tables[f], mode="sum")      # [W*B, dim]
      saved.append((f, got))
      pooled.append(out.to(torch.bfloat16).view(W, B, self.dim))
    leaf = (torch.stack(pooled, dim=2) if pooled else torch.empty(W, B, 0, self.dim, device=ids[0].device,
                                                                   dtype=torch.bfloat16))
    leaf = leaf.reshape(W * B * len(self.mine), self.dim).detach().requires_grad_(True)    # rows: (src, b, local f)
    if W > 1:
      out_splits = [B * len(self.by_owner[r]) for r in range(W)]
      in_splits = [B * len(self.mine)] * W
      got = _A2A.apply(leaf, out_splits, in_splits)                 # rows: (owner, b, f of that owner)
      cols, at = [None] * len(self.vocabs), 0
      for r in range(W):
        k = len(self.by_owner[r])
        blk = got[at:at + B * k].view(B, k, self.dim)
        at += B * k
        for j, f in enumerate(self.by_owner[r]):
          cols[f] = blk[:, j]
      res = torch.stack(cols, dim=1)
    else:
      res = leaf.view(B, len(self.mine), self.dim)
    return res, (leaf, saved, B)

  @torch.no_grad()
  def backward_update(self, ctx) -> None:
    leaf, saved, B = ctx
    W = self.world
    g = leaf.grad.view(W * B, len(self.mine), self.dim).float() / W     # mean over the global batch
    for j, (f, got) in enumerate(saved):
      rows = got.reshape(-1)
      per_id = g[:, j].repeat_interleave(self.bags[f], dim=0)
      uniq, inv = torch.unique(rows, return_inverse=True)
      summed = torch.zeros(uniq.numel(), self.dim, device=rows.device).index_add_(0, inv, per_id)
      acc = self.acc[f][uniq] + summed.pow(2).mean(dim=1)
      self.acc[f][uniq] = acc
      self.tables[f][uniq] -= self.lr * summed / (acc.sqrt()[:, None] + 1e-8)


class DenseNet(nn.Module):
  def __init__(self, num_dense, dim, n_feat, bottom=(512, 256, 128), top=(1024, 1024, 512, 256, 1), n_cross=3, rank=512):
    super().__init__()
    dims = [num_dense, *bottom]
    self.bottom = nn.ModuleList(nn.Linear(a, b) for a, b in zip(dims[:-1], dims[1:]))
    d = dim * (n_feat + 1)
    self.u = nn.ParameterList(nn.Parameter(torch.randn(d, rank) * (2.0 / (d + rank)) ** 0.5) for _ in range(n_cross))
    self.v = nn.ParameterList(nn.Parameter(torch.randn(rank, d) * (2.0 / (d + rank)) ** 0.5) for _ in range(n_cross))
    self.b = nn.ParameterList(nn.Parameter(torch.zeros(d)) for _ in range(n_cross))
    dims = [d, *top]
    self.top = nn.ModuleList(nn.Linear(a, b) for a, b in zip(dims[:-1], dims[1:]))

  def forward(self, dense_x, pooled):
    x = dense_x
    for lin in self.bottom:
      x = F.relu(lin(x))
    x0 = torch.cat([x, pooled.flatten(1).to(x.dtype)], dim=1)
    xl = x0
    for u, v, b in zip(self.u, self.v, self.b):
      xl = x0 * ((xl @ u.to(xl.dtype)) @ v.to(xl.dtype) + b.to(xl.dtype)) + xl
    x = xl
    for i, lin in enumerate(self.top):
      x = lin(x)
      if i + 1 < len(self.top):
        x = F.relu(x)
    return x.reshape(-1)


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--steps", type=int, default=20)
  ap.add_argument("--warmup", type=int, default=5)
  ap.add_argument("--global-batch", type=int, default=65536)
  ap.add_argument("--vocab-scale", type=float, default=1.0)
  args = ap.parse_args()
  world = int(os.environ.get("WORLD_SIZE", "1"))
  rank = int(os.environ.get("RANK", "0"))
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  device = torch.device("cuda", local)
  if world > 1:
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)
  B = args.global_batch // world
  vocabs = [max(3, int(v * args.vocab_scale)) for v in synthetic.CRITEO_VOCAB_SIZES]
  bags = list(synthetic.CRITEO_MULTI_HOT_SIZES)
  torch.manual_seed(0)
  tables = ShardedTables(vocabs, bags, 128, rank, world, device)
  net = DenseNet(13, 128, len(vocabs)).to(device)
  params = list(net.parameters())
  if world > 1:
    for p in params:
      dist.broadcast(p.data, 0)
  opt = torch.optim.Adam(params, lr=1e-3, fused=True)
  rng = np.random.default_rng(rank)
  batches = []
  for _ in range(4):
    ids = [torch.from_numpy(synthetic.zipf_ids(rng, v, (B, b), 1.05)).to(device) for v, b in zip(vocabs, bags)]
    dense = torch.from_numpy(synthetic.lognormal_dense(rng, B, 13)).to(device)
    label = torch.from_numpy((rng.random(B) < 0.25).astype(np.float32)).to(device)
    batches.append((ids, dense, label))

  def step(i):
    ids, dense, label = batches[i % len(batches)]
    pooled, ctx = tables.forward(ids)
    with torch.autocast("cuda", dtype=torch.bfloat16):
      logits = net(dense, pooled)
    loss = F.binary_cross_entropy_with_logits(logits.float(), label)
    opt.zero_grad(set_to_none=True)
    loss.backward()
    tables.backward_update(ctx)
    if world > 1:
      flat = torch.cat([p.grad.reshape(-1) for p in params])
      dist.all_reduce(flat)
      flat /= world
      at = 0
      for p in params:
        p.grad.copy_(flat[at:at + p.numel()].view_as(p))
        at += p.numel()
    opt.step()
    return loss

  for i in range(max(args.warmup, 3)):
    step(i)
  torch.cuda.synchronize()
  if world > 1:
    dist.barrier()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for i in range(args.steps):
    loss = step(i)
  e1.record()
  torch.cuda.synchronize()
  ms = torch.tensor([e0.elapsed_time(e1)], device=device)
  if world > 1:
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
  if rank == 0:
    per = float(ms) / args.steps
    print(json.dumps({"metric": "dlrm_dcnv2_train_samples_per_sec", "value": args.global_batch / (per * 1e-3),
                      "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                      "ms_per_step": per, "dtype": "bf16", "data": "synthetic", "scaling": "strong",
                      "impl": "torch+nccl+cublas stand-in (not the reference)", "last_loss": float(loss),
                      "config": {"global_batch": args.global_batch, "per_gpu_batch": B, "vocab_scale": args.vocab_scale,
                                 "placement": "table-wise"}}))
  if world > 1:
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
  main()
