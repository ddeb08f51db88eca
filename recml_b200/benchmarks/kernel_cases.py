"""Small single-kernel workloads for profiling and roofline checks.

  python -m recml_b200.benchmarks.kernel_cases <case> [--iters N]

Each case builds inputs larger than L2 (126 MB) but only a few GB in total, warms up, then times the
kernel with CUDA events and prints achieved bandwidth / FLOP rate against the measured peaks of this
machine (MEASURED_PEAKS.json when present).  The same command line is what `ncu` captures.
Cases: gemm_fwd, gemm_dgrad, gemm_wgrad, gemm_cross, emb_fwd, emb_bwd, hstu_fwd, hstu_bwd, vocab_rank,
layernorm, layernorm_bwd, ssd_fwd, ssd_bwd, mha_fwd, mha_bwd, sampled_softmax.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch


def peaks():
  path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
  if os.path.exists(path):
    d = json.load(open(path))
    return d["hbm_gbs"], d["bf16_tflops"], "of measured"
  return 6650.0, 1590.0, "of fallback"


def timed(fn, iters, flush=None):
  for _ in range(3):
    fn()
  torch.cuda.synchronize()
  total = 0.0
  for _ in range(iters):
    if flush is not None:
      flush.zero_()            # 256 MB write: evicts L2 between timed iterations
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    fn()
    b.record()
    torch.cuda.synchronize()
    total += a.elapsed_time(b)
  return total / iters


def rnd(*shape, scale=0.5):
  return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("case")
  ap.add_argument("--iters", type=int, default=5)
  ap.add_argument("--rows", type=int, default=32768, help="M of the gemm_* cases")
  args = ap.parse_args()
  from recml_b200.ops import _lib, gemm as G
  hbm, tf, tag = peaks()
  flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
  out = {"case": args.case}
  c = args.case
  if c.startswith("gemm"):
    M, N, K = args.rows, 1024, 3456
    if c == "gemm_fwd":
      a, b = rnd(M, K), rnd(N, K)
      bias = torch.randn(N, device="cuda")
      fn = lambda: G.gemm(a, b, bias=bias, relu=True)
    elif c == "gemm_dgrad":
      a, b, aux = rnd(M, N), rnd(N, K), rnd(M, K)
      fn = lambda: G.gemm(a, b, b_mn=True, epi=G.EPI_MASK_RELU, aux0=aux)
    elif c == "gemm_wgrad":
      a, b = rnd(M, N), rnd(M, K)
      fn = lambda: G.gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32)
    else:  # cross layer second product: [M, 512] x [512, 3456] with the x0*v + xl epilogue
      a, b, x0, xl = rnd(M, 512), rnd(K, 512), rnd(M, K), rnd(M, K)
      bias = torch.randn(K, device="cuda")
      fn = lambda: G.gemm(a, b, bias=bias, epi=G.EPI_CROSS, aux0=x0, aux1=xl, want_out2=True)
      N, K = 3456, 512
    ms = timed(fn, args.iters, flush)
    flops = 2.0 * M * N * K
    out.update(ms=ms, tflops=flops / ms / 1e9, frac=flops / ms / 1e9 / tf, of=tag, shape=[M, N, K])
  elif c in ("emb_fwd", "emb_bwd"):
    from recml_b200 import embedding as emb
    from recml_b200.data import synthetic
    vocabs, bags, B, D = [4_000_000, 1_000_000, 50_000, 2_000_000], [20, 3, 1, 8], 16384, 128
    specs = {f"f{i}": emb.EmbeddingSpec(v, D, combiner="sum") for i, v in enumerate(vocabs)}
    m = emb.ShardedEmbedding(emb.ShardedEmbeddingConfig(specs, emb.RowWiseAdagradOptimizerSpec(0.01)), device="cuda")
    rng = np.random.default_rng(0)
    kjt = synthetic.make_dlrm_batch(rng, B, vocabs, bags, names=list(specs))["sparse"].to_device(torch.device("cuda"))
    ids = B * sum(bags)
    if c == "emb_fwd":
      m.eval()
      fn = lambda: m(kjt)
      bytes_ = ids * D * 4 + B * len(bags) * D * 2
    else:
      g = rnd(B, len(bags), D, scale=0.1)
      def fn():
        o = m(kjt)
        o.backward(g)
      bytes_ = ids * D * 4 + B * len(bags) * D * 2 + ids * (D * 2 + 16) + ids * D * 8   # fwd + grads + row RMW bound
    ms = timed(fn, args.iters, flush)
    out.update(ms=ms, gbs=bytes_ / ms / 1e6, frac=bytes_ / ms / 1e6 / hbm, of=tag, ids=ids)
  elif c in ("hstu_fwd", "hstu_bwd"):
    from recml_b200.ops import hstu_attention as A
    from recml_b200.data import synthetic
    rng = np.random.default_rng(0)
    lens = synthetic.powerlaw_lengths(rng, 64, 16, 4096, 1.2)
    T, H, Dh, N = int(lens.sum()), 4, 64, 4096
    offs = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
    q, k, v = (rnd(T, H, Dh).requires_grad_() for _ in range(3))
    pos_w = (torch.randn(2 * N - 1, device="cuda") * 0.1).requires_grad_()
    ts_w = (torch.randn(129, device="cuda") * 0.1).requires_grad_()
    ts = torch.from_numpy(synthetic.exponential_timestamps(rng, lens)).cuda()
    pairs = float(sum(l * (l + 1) / 2 for l in lens))
    if c == "hstu_fwd":
      fn = lambda: A.jagged_pointwise_attention(q.detach(), k.detach(), v.detach(), offs, N, pos_w=pos_w.detach(),
                                                ts_w=ts_w.detach(), timestamps=ts)
      flops = 4.0 * pairs * Dh * H
    else:
      go = rnd(T, H, Dh)
      def fn():
        o = A.jagged_pointwise_attention(q, k, v, offs, N, pos_w=pos_w, ts_w=ts_w, timestamps=ts)
        o.backward(go)
      flops = 14.0 * pairs * Dh * H
    ms = timed(fn, args.iters)
    out.update(ms=ms, tflops_causal=flops / ms / 1e9, tokens=T, pairs=pairs)
  elif c == "vocab_rank":
    from recml_b200.ops import vocab_rank as VR
    rows, D, V = 2048, 256, 1_000_000
    x, shard = rnd(rows, D, scale=0.3), rnd(V, D, scale=0.3)
    tgt = torch.randint(0, V, (rows,), device="cuda")
    pos = (x.float() * shard[tgt].float()).sum(-1)
    r = VR.VocabRanker(rows, D)
    ms = timed(lambda: r.ranks(x, pos, tgt, shard, 1, 0), args.iters, flush)
    flops = 2.0 * rows * V * D
    out.update(ms=ms, tflops=flops / ms / 1e9, frac=flops / ms / 1e9 / tf, of=tag)
  elif c in ("layernorm", "layernorm_bwd"):
    from recml_b200.ops import norm
    x = rnd(1 << 19, 256).requires_grad_()
    w, b = torch.ones(256, device="cuda", requires_grad=True), torch.zeros(256, device="cuda", requires_grad=True)
    if c == "layernorm":
      ms = timed(lambda: norm.layer_norm(x.detach(), w, b, 1e-6), args.iters, flush)
      bytes_ = x.numel() * 4                  # bf16 in + bf16 out
    else:                                     # forward + backward: x, dy in; y, dx out (+ statistics)
      dy = rnd(1 << 19, 256)

      def fb():
        x.grad = w.grad = b.grad = None
        norm.layer_norm(x, w, b, 1e-6).backward(dy)
      ms = timed(fb, args.iters, flush)
      bytes_ = x.numel() * 2 * 5              # forward: x in, y out; backward: x, dy in, dx out
    out.update(ms=ms, gbs=bytes_ / ms / 1e6, frac=bytes_ / ms / 1e6 / hbm, of=tag)
  elif c in ("ssd_fwd", "ssd_bwd"):
    from recml_b200.ops import ssd
    B, L, H, P, N = 512, 200, 8, 64, 64            # Mamba4Rec block at d_model 256: d_inner 512 = 8 heads x 64
    x = (torch.randn(B, L, H, P, device="cuda") * 0.3).requires_grad_()
    a = (-torch.rand(B, L, H, device="cuda") * 0.5).requires_grad_()
    b = (torch.randn(B, L, 1, N, device="cuda") * 0.3).requires_grad_()
    cc = (torch.randn(B, L, 1, N, device="cuda") * 0.3).requires_grad_()
    if c == "ssd_fwd":
      fn = lambda: ssd.ssd_scan(x.detach(), a.detach(), b.detach(), cc.detach())
      bytes_ = (2 * x.numel() + a.numel() + 2 * b.numel() * 1) * 4 + B * H * ((L + 31) // 32) * P * N * 4
    else:
      go = torch.randn(B, L, H, P, device="cuda")
      def fn():
        ssd.ssd_scan(x, a, b, cc).backward(go)
      bytes_ = (4 * x.numel() + 2 * a.numel() + 2 * b.numel() + 2 * B * L * H * N * 2) * 4 + 2 * B * H * ((L + 31) // 32) * P * N * 4
    ms = timed(fn, args.iters, flush)
    steps = float(B) * L * H
    out.update(ms=ms, gbs=bytes_ / ms / 1e6, frac=bytes_ / ms / 1e6 / hbm, of=tag, state_updates_per_s=steps * P * N / ms * 1e3)
  elif c in ("mha_fwd", "mha_bwd"):
    from recml_b200.ops import softmax_attention as sm
    B, L, H, Dh = 512, 200, 4, 64                   # SASRec block: batch 512 per GPU, 200 positions, 4 x 64
    q, k, v = (rnd(B * L, H, Dh).requires_grad_() for _ in range(3))
    offs = torch.arange(B + 1, device="cuda", dtype=torch.int32) * L
    pairs = float(B) * L * (L + 1) / 2
    if c == "mha_fwd":
      fn = lambda: sm.jagged_softmax_attention(q.detach(), k.detach(), v.detach(), offs, L, True)
      flops = 4.0 * pairs * Dh * H
    else:
      go = rnd(B * L, H, Dh)
      def fn():
        sm.jagged_softmax_attention(q, k, v, offs, L, True).backward(go)
      flops = 14.0 * pairs * Dh * H
    ms = timed(fn, args.iters)
    out.update(ms=ms, tflops_causal=flops / ms / 1e9, tokens=B * L)
  elif c == "sampled_softmax":
    from recml_b200.ops import sampled_softmax as S
    T, C = 65536, 1024
    pos = torch.randn(T, device="cuda")
    neg = rnd(T, C)
    cand, tgt = torch.randint(0, 10_000_000, (C,), device="cuda"), torch.randint(0, 10_000_000, (T,), device="cuda")
    w = torch.ones(T, device="cuda")
    ms = timed(lambda: S.sampled_softmax_loss(pos, neg, cand, tgt, w, 0.05), args.iters, flush)
    bytes_ = T * C * 2 * 2                            # logits read (second pass hits L1/L2) + gradient written
    out.update(ms=ms, gbs=bytes_ / ms / 1e6, frac=bytes_ / ms / 1e6 / hbm, of=tag)
  else:
    raise SystemExit(f"unknown case {c}")
  torch.cuda.synchronize()
  _lib.check_status()
  print(json.dumps(out))


if __name__ == "__main__":
  main()
