"""Jagged HSTU attention kernels vs the fp32 torch formula (the reference's own kernel test compares
against the dense formula with atol = rtol = 5e-3, `recml/core/ops/hstu_ops_test.py:45-70`)."""
import numpy as np
import pytest
import torch

from recml_b200.ops import _lib, hstu_attention as A, hstu_cuda

pytestmark = pytest.mark.gpu


def _inputs(lengths, H, Dh, seed=0, with_bias=True, N=None):
  g = torch.Generator().manual_seed(seed)
  T = int(sum(lengths))
  q, k, v = (torch.randn(T, H, Dh, generator=g).mul(0.5).to(torch.bfloat16) for _ in range(3))
  offs = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32)
  N = N or max(lengths)
  pos_w = torch.randn(2 * N - 1, generator=g) * 0.3 if with_bias else None
  ts_w = torch.randn(129, generator=g) * 0.3 if with_bias else None
  rng = np.random.default_rng(seed)
  ts = torch.from_numpy(np.concatenate([1_600_000_000 + np.cumsum(rng.exponential(3600.0, L)).astype(np.int64)
                                        for L in lengths])) if with_bias else None
  return q, k, v, offs, N, pos_w, ts_w, ts


@pytest.mark.parametrize("lengths,H,Dh,bias", [([128], 1, 64, False), ([5, 128, 300, 1, 77], 2, 64, True),
                                               ([700, 33], 4, 64, True), ([260, 130], 2, 128, True)])
def test_forward_matches_reference(lengths, H, Dh, bias):
  q, k, v, offs, N, pos_w, ts_w, ts = _inputs(lengths, H, Dh, with_bias=bias)
  ref = A.jagged_attention_reference(q.float(), k.float(), v.float(), offs, N, pos_w=pos_w, ts_w=ts_w, timestamps=ts)
  cu = lambda t: None if t is None else t.cuda()
  out = A.jagged_pointwise_attention(q.cuda(), k.cuda(), v.cuda(), offs.cuda(), N, pos_w=cu(pos_w), ts_w=cu(ts_w),
                                     timestamps=cu(ts))
  torch.cuda.synchronize()
  _lib.check_status()
  err = (out.float().cpu() - ref).abs().max().item()
  scale = ref.abs().max().item() + 1e-6
  assert err / scale < 2e-2, (err, scale)


def test_backward_matches_reference():
  lengths, H, Dh = [200, 64, 391], 2, 64
  q, k, v, offs, N, pos_w, ts_w, ts = _inputs(lengths, H, Dh, seed=3)
  leaves = [t.float().requires_grad_() for t in (q, k, v)] + [pos_w.clone().requires_grad_(), ts_w.clone().requires_grad_()]
  ref = A.jagged_attention_reference(leaves[0], leaves[1], leaves[2], offs, N, pos_w=leaves[3], ts_w=leaves[4], timestamps=ts)
  go = torch.randn(ref.shape, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
  ref.backward(go.float())
  gl = [t.cuda().requires_grad_() for t in (q, k, v)] + [pos_w.cuda().requires_grad_(), ts_w.cuda().requires_grad_()]
  out = A.jagged_pointwise_attention(gl[0], gl[1], gl[2], offs.cuda(), N, pos_w=gl[3], ts_w=gl[4], timestamps=ts.cuda())
  out.backward(go.cuda())
  torch.cuda.synchronize()
  _lib.check_status()
  for name, a, b in zip("q k v pos_w ts_w".split(), gl, leaves):
    err = (a.grad.float().cpu() - b.grad).abs().max().item()
    scale = b.grad.abs().max().item() + 1e-6
    assert err / scale < 3e-2, (name, err, scale)


def test_hstu_retrieval_trains_on_gpu():
  """Packed HSTU retrieval model (sharded item table, tcgen05 attention / GEMMs, CUDA LayerNorm): the
  first loss matches the CPU run of the same seed and training reduces it."""
  import numpy as np
  from recml_b200.data import synthetic
  from recml_b200.models import hstu_retrieval as H

  def run(device, steps):
    torch.manual_seed(0)
    rng = np.random.default_rng(0)
    b = synthetic.make_hstu_batch(rng, 6, 3000, min_len=4, max_len=200, mean_target=60, num_negatives=64,
                                  token_capacity=1024)
    b = {k: v.to(device) for k, v in b.items()}
    m = H.HSTURetrieval(vocab_size=3000, model_dim=128, num_heads=2, num_layers=2, max_seq_len=256,
                        token_capacity=1024, num_negatives=64, num_in_batch=32, device=device, seed=1)
    opt = torch.optim.Adam(m.encoder.parameters(), 2e-3)
    losses = []
    for _ in range(steps):
      loss, _ = m(**b)
      loss.backward()
      opt.step(); opt.zero_grad()
      losses.append(float(loss.detach()))
    return losses

  lg = run("cuda", 25)
  torch.cuda.synchronize()
  _lib.check_status()
  lc = run("cpu", 1)
  assert abs(lg[0] - lc[0]) < 0.15, (lg[0], lc[0])
  assert lg[-1] < lg[0] * 0.7, lg


@pytest.mark.parametrize("C", [1000, 256, 512, 1024])
def test_sampled_softmax_kernel_matches_torch(C):
  """C = 256 / 512 / 1024 take the kernel that holds a row in registers; other widths the strided one.  The ids
  go past 32 bits, and one candidate shares only its LOW word with a target: it must not be dropped."""
  import torch
  from recml_b200.ops import sampled_softmax as S
  torch.manual_seed(0)
  T = 777
  pos = torch.randn(T, device="cuda") * 0.5
  neg = (torch.randn(T, C, device="cuda") * 0.5).to(torch.bfloat16)
  cand = torch.randint(0, 3000, (C,), device="cuda") + (1 << 33)
  tgt = torch.randint(0, 3000, (T,), device="cuda") + (1 << 33)
  tgt[:50] = cand[:50]                      # accidental hits
  tgt[60] = 5 + (1 << 33)
  cand[7] = 5 + (1 << 34)                   # same low word as target 60, another item
  cand[8] = 5 + (1 << 33)                   # and the real accidental hit beside it
  w = (torch.rand(T, device="cuda") > 0.2).float()
  w[60] = 1.0
  a = [pos.clone().requires_grad_(), neg.clone().requires_grad_()]
  r = [pos.clone().requires_grad_(), neg.float().clone().requires_grad_()]
  loss, hit = S.sampled_softmax_loss(a[0], a[1], cand, tgt, w, 0.05)
  loss_r, hit_r = S.reference(r[0], r[1], cand, tgt, w, 0.05)
  torch.testing.assert_close(loss, loss_r, rtol=1e-4, atol=1e-4)
  torch.testing.assert_close(hit, hit_r, rtol=1e-5, atol=1e-5)
  (loss * 3.0).backward()
  (loss_r * 3.0).backward()
  torch.testing.assert_close(a[0].grad, r[0].grad, rtol=1e-3, atol=1e-5)
  torch.testing.assert_close(a[1].grad.float(), r[1].grad, rtol=2e-2, atol=1e-5)
  assert float(a[1].grad[60, 8]) == 0.0 and float(a[1].grad[60, 7]) != 0.0
  # the plain backward (incoming gradient exactly 1) leaves the stored gradient as the kernel wrote it
  b = [pos.clone().requires_grad_(), neg.clone().requires_grad_()]
  S.sampled_softmax_loss(b[0], b[1], cand, tgt, w, 0.05)[0].backward()
  torch.testing.assert_close(b[1].grad.float() * 3.0, a[1].grad.float(), rtol=2e-2, atol=1e-6)
  torch.testing.assert_close(b[0].grad * 3.0, a[0].grad, rtol=1e-5, atol=1e-7)


def test_attention_accepts_column_slices_of_a_fused_projection():
  """q, k, v handed over as views into one [T, 4, H, Dh] buffer give the same output and gradients."""
  import torch
  from recml_b200.ops import hstu_attention as A
  torch.manual_seed(0)
  T, H, Dh, N = 300, 2, 64, 256
  offs = torch.tensor([0, 130, 300], dtype=torch.int32, device="cuda")
  fused = (torch.randn(T, 4, H, Dh, device="cuda") * 0.5).to(torch.bfloat16)
  outs = []
  for strided in (True, False):
    leaf = fused.clone().requires_grad_()
    _, q, k, v = leaf.unbind(dim=1)
    if not strided:
      q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    o = A.jagged_pointwise_attention(q, k, v, offs, N, causal=True, scale=0.125)
    o.backward(torch.ones_like(o) * 0.01)
    outs.append((o.detach().float(), leaf.grad.float()))
  torch.testing.assert_close(outs[0][0], outs[1][0], rtol=0, atol=0)
  torch.testing.assert_close(outs[0][1], outs[1][1], rtol=1e-2, atol=1e-4)


def _run_cuda(q, k, v, offs, N, pos_w, ts_w, ts, causal, go):
  gl = [t.cuda().requires_grad_() for t in (q, k, v)] + [pos_w.cuda().requires_grad_(), ts_w.cuda().requires_grad_()]
  out = A.jagged_pointwise_attention(gl[0], gl[1], gl[2], offs.cuda(), N, pos_w=gl[3], ts_w=gl[4], timestamps=ts.cuda(),
                                     causal=causal)
  out.backward(go.cuda())
  torch.cuda.synchronize()
  _lib.check_status()
  return out.detach(), [t.grad.detach() for t in gl]


def test_non_causal_with_bias_matches_reference():
  """Full (non-causal) attention with both bias terms: the per-batch time-bucket blocks are then indexed by
  the square (query tile, key tile) grid instead of the causal triangle."""
  lengths, H, Dh = [200, 64, 391], 2, 64
  q, k, v, offs, N, pos_w, ts_w, ts = _inputs(lengths, H, Dh, seed=5)
  leaves = [t.float().requires_grad_() for t in (q, k, v)] + [pos_w.clone().requires_grad_(), ts_w.clone().requires_grad_()]
  ref = A.jagged_attention_reference(leaves[0], leaves[1], leaves[2], offs, N, pos_w=leaves[3], ts_w=leaves[4],
                                     timestamps=ts, causal=False)
  go = torch.randn(ref.shape, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
  ref.backward(go.float())
  out, grads = _run_cuda(q, k, v, offs, N, pos_w, ts_w, ts, False, go)
  assert (out.float().cpu() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6) < 2e-2
  for name, a, b in zip("q k v pos_w ts_w".split(), grads, leaves):
    err = (a.float().cpu() - b.grad).abs().max().item()
    assert err / (b.grad.abs().max().item() + 1e-6) < 3e-2, (name, err)


def test_step_context_is_shared_and_rebuilt_when_a_table_changes():
  """Calls with the same batch and tables share one bias context (tiles built once); changing a table in place
  (what an optimizer step does) gives a new one."""
  from recml_b200.ops import hstu_cuda
  lengths, H, Dh = [300, 17, 260], 2, 64
  q, k, v, offs, N, pos_w, ts_w, ts = _inputs(lengths, H, Dh, seed=7)
  o, tsg, pw, tw = offs.cuda(), ts.cuda(), pos_w.cuda(), ts_w.cuda()
  hstu_cuda._memo.clear()
  out1 = A.jagged_pointwise_attention(q.cuda(), k.cuda(), v.cuda(), o, N, pos_w=pw, ts_w=tw, timestamps=tsg)
  ctx1 = hstu_cuda._memo["bias_ctx"][2]
  out2 = A.jagged_pointwise_attention(q.cuda(), k.cuda(), v.cuda(), o, N, pos_w=pw, ts_w=tw, timestamps=tsg)
  assert hstu_cuda._memo["bias_ctx"][2] is ctx1 and torch.equal(out1, out2)
  pw.add_(0.25)
  out3 = A.jagged_pointwise_attention(q.cuda(), k.cuda(), v.cuda(), o, N, pos_w=pw, ts_w=tw, timestamps=tsg)
  assert hstu_cuda._memo["bias_ctx"][2] is not ctx1 and not torch.equal(out1, out3)
  torch.cuda.synchronize()
  _lib.check_status()


def _compare(ref, got, tol, what):
  err = (got.float().cpu() - ref).abs().max().item()
  scale = ref.abs().max().item() + 1e-6
  assert err / scale < tol, (what, err, scale)


def test_long_sequence_4096_forward_backward():
  """The configuration's longest sequences: 32 x 32 tile pairs per sequence, bias tables of 8191 entries."""
  lengths, H, Dh = [4096, 130], 2, 64
  q, k, v, offs, N, pos_w, ts_w, ts = _inputs(lengths, H, Dh, seed=5)
  leaves = [t.float().requires_grad_() for t in (q, k, v)] + [pos_w.clone().requires_grad_(), ts_w.clone().requires_grad_()]
  ref = A.jagged_attention_reference(leaves[0], leaves[1], leaves[2], offs, N, pos_w=leaves[3], ts_w=leaves[4], timestamps=ts)
  go = torch.randn(ref.shape, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
  ref.backward(go.float())
  gl = [t.cuda().requires_grad_() for t in (q, k, v)] + [pos_w.cuda().requires_grad_(), ts_w.cuda().requires_grad_()]
  out = A.jagged_pointwise_attention(gl[0], gl[1], gl[2], offs.cuda(), N, pos_w=gl[3], ts_w=gl[4], timestamps=ts.cuda())
  out.backward(go.cuda())
  torch.cuda.synchronize()
  _lib.check_status()
  _compare(ref.detach(), out.detach(), 2e-2, "out")
  for name, a, b in zip("q k v pos_w ts_w".split(), gl, leaves):
    _compare(b.grad, a.grad, 3e-2, name)


@pytest.mark.parametrize("causal", [True, False])
def test_window_and_segment_masks_in_the_kernel(causal):
  lengths, H, Dh = [300, 129, 64], 2, 64
  q, k, v, offs, N, pos_w, ts_w, ts = _inputs(lengths, H, Dh, seed=7)
  g = torch.Generator().manual_seed(1)
  seg = torch.cat([torch.sort(torch.randint(0, 3, (L,), generator=g)).values for L in lengths]).to(torch.int32)
  kw = dict(causal=causal, sliding_window_size=37)
  leaves = [t.float().requires_grad_() for t in (q, k, v)]
  ref = A.jagged_attention_reference(*leaves, offs, N, pos_w=pos_w, ts_w=ts_w, timestamps=ts, segment_ids=seg, **kw)
  go = torch.randn(ref.shape, generator=g).to(torch.bfloat16)
  ref.backward(go.float())
  gl = [t.cuda().requires_grad_() for t in (q, k, v)]
  out = A.jagged_pointwise_attention(*gl, offs.cuda(), N, pos_w=pos_w.cuda(), ts_w=ts_w.cuda(), timestamps=ts.cuda(),
                                     segment_ids=seg.cuda(), **kw)
  out.backward(go.cuda())
  torch.cuda.synchronize()
  _lib.check_status()
  _compare(ref.detach(), out.detach(), 2e-2, "out")
  for name, a, b in zip("qkv", gl, leaves):
    _compare(b.grad, a.grad, 3e-2, name)


def test_bias_tables_shared_by_two_layers_get_the_summed_gradient():
  """Two attention calls of one step use the same tables (as the layers of a model do): the step's bias tiles are
  built once, and the tables' gradients, returned by the backward call that runs last, are the sum over both."""
  lengths, H, Dh = [200, 90], 2, 64
  q, k, v, offs, N, pos_w, ts_w, ts = _inputs(lengths, H, Dh, seed=11)
  q2 = (q.float() * 0.7).to(torch.bfloat16)
  lp, lt = pos_w.clone().requires_grad_(), ts_w.clone().requires_grad_()
  r1 = A.jagged_attention_reference(q.float(), k.float(), v.float(), offs, N, pos_w=lp, ts_w=lt, timestamps=ts)
  r2 = A.jagged_attention_reference(q2.float(), k.float(), v.float(), offs, N, pos_w=lp, ts_w=lt, timestamps=ts)
  go = torch.randn(r1.shape, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
  (r1 * go.float()).sum().add((r2 * go.float()).sum() * 0.5).backward()
  gp, gt = pos_w.cuda().requires_grad_(), ts_w.cuda().requires_grad_()
  o, tsg = offs.cuda(), ts.cuda()
  o1 = A.jagged_pointwise_attention(q.cuda(), k.cuda(), v.cuda(), o, N, pos_w=gp, ts_w=gt, timestamps=tsg)
  o2 = A.jagged_pointwise_attention(q2.cuda(), k.cuda(), v.cuda(), o, N, pos_w=gp, ts_w=gt, timestamps=tsg)
  ((o1.float() * go.cuda().float()).sum() + (o2.float() * go.cuda().float()).sum() * 0.5).backward()
  torch.cuda.synchronize()
  _lib.check_status()
  _compare(lp.grad, gp.grad, 3e-2, "pos_w")
  _compare(lt.grad, gt.grad, 3e-2, "ts_w")


def test_dense_hstu_runs_on_the_packed_kernels_and_matches_the_dense_formulation():
  """`HSTU.forward(ids, padding_mask)` on CUDA goes through the packed attention kernels (head dim 64); on CPU the
  same module evaluates the dense `[B, L, L]` formulation.  Same weights, same inputs: same outputs at the valid
  positions, same gradients."""
  from recml_b200.layers import hstu as H
  torch.manual_seed(0)
  B, L, V = 3, 160, 50
  model = H.HSTU(vocab_size=V, max_positions=L, model_dim=128, num_heads=2, num_layers=2, add_head=False,
                 use_relative_bias=True, max_seq_len=L)
  ids = torch.randint(1, V, (B, L))
  lens = torch.tensor([160, 97, 5])
  mask = (torch.arange(L)[None] < lens[:, None]).long()
  ts = torch.cumsum(torch.randint(1, 5000, (B, L)), dim=1)
  ref = model(ids, padding_mask=mask, timestamps=ts)
  w = torch.randn(B, L, 128) * mask[..., None]
  (ref * w).sum().backward()
  ref_grads = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
  model.zero_grad()
  gm = model.cuda()
  assert gm._packed_kernels_apply(torch.empty(B, L, 128, device="cuda"))
  out = gm(ids.cuda(), padding_mask=mask.cuda(), timestamps=ts.cuda())
  (out.float() * w.cuda()).sum().backward()
  torch.cuda.synchronize()
  _lib.check_status()
  m3 = mask[..., None].bool()
  _compare((ref * m3).detach(), (out.float().cpu() * m3).detach(), 4e-2, "hidden states")
  for n, p in gm.named_parameters():
    if n in ref_grads and ref_grads[n].abs().max() > 0:
      _compare(ref_grads[n], p.grad, 8e-2, n)


def test_block_with_fused_activation_node_matches_unfused(monkeypatch):
  """`HSTUBlock.forward_jagged` runs activation + split + attention as one autograd node (fp32 dq consumed by the
  fused SiLU backward, residual added in the output GEMM's epilogue); the unfused composition of the same kernels
  must give the same outputs and parameter gradients."""
  from recml_b200.layers import hstu as hstu_layers
  from recml_b200.ops import hstu_attention as attn_ops
  torch.manual_seed(0)
  D, H = 256, 4
  lens = torch.tensor([300, 17, 129, 256])
  offs = torch.zeros(5, dtype=torch.int64)
  offs[1:] = lens.cumsum(0)
  T = int(offs[-1])
  x = (torch.randn(T, D, device="cuda") * 0.5).to(torch.bfloat16)
  g = (torch.randn(T, D, device="cuda") * 0.1).to(torch.bfloat16)
  pos_w = (torch.randn(2 * 512 - 1, device="cuda") * 0.1).requires_grad_()

  def run(fused: bool):
    torch.manual_seed(1)
    blk = hstu_layers.HSTUBlock(D, H).cuda().to(torch.bfloat16)
    if not fused:
      monkeypatch.setattr(attn_ops, "fused_block_ok", lambda z, hd: False)
    xi = x.clone().requires_grad_()
    pw = pos_w.detach().clone().requires_grad_()
    out = blk.forward_jagged(xi, offs.cuda(), 512, pos_w=pw)
    out.backward(g)
    monkeypatch.undo()
    return out.detach().float(), xi.grad.float(), pw.grad.float(), {n: p.grad.float() for n, p in blk.named_parameters()}

  of, dxf, dpf, gf = run(True)
  ou, dxu, dpu, gu = run(False)
  tol = lambda ref: 2e-2 * float(ref.abs().max()) + 1e-6
  assert float((of - ou).abs().max()) <= tol(ou)
  assert float((dxf - dxu).abs().max()) <= tol(dxu)
  assert float((dpf - dpu).abs().max()) <= tol(dpu)
  for n in gu:
    assert float((gf[n] - gu[n]).abs().max()) <= tol(gu[n]), n


@pytest.mark.parametrize("rate", [0.25, 0.6])
def test_attention_weight_dropout_in_the_kernels(rate):
  """Dropout on the attention weights (reference `recml/layers/keras/hstu.py:386-387`) is applied inside the
  kernels from a counter-based hash of (key, head, query token, key token); forward and backward regenerate the
  same mask.  The oracle applies the same mask, rebuilt with integer tensor ops from the key the call drew."""
  from recml_b200.ops import hstu_attention as A
  torch.manual_seed(3)
  H, Dh = 2, 64
  lens = torch.tensor([200, 70, 130])
  offs = torch.zeros(4, dtype=torch.int64)
  offs[1:] = lens.cumsum(0)
  T = int(offs[-1])
  mk = lambda: (torch.randn(T, H, Dh, device="cuda") * 0.7).to(torch.bfloat16)
  q, k, v = mk(), mk(), mk()
  a = [t.clone().requires_grad_() for t in (q, k, v)]
  r = [t.float().clone().requires_grad_() for t in (q, k, v)]
  out = A.jagged_pointwise_attention(*a, offs.cuda(), 256, causal=True, dropout_p=rate)
  key = int(A.LAST_DROPOUT_KEY.item())
  ref = A.jagged_attention_reference(*r, offs.cuda(), 256, causal=True, dropout_p=rate, dropout_key=key)
  tol = lambda x: 1.5e-2 * float(x.abs().max())
  assert float((out.float() - ref).abs().max()) <= tol(ref)
  # the mask drops about `rate` of the weights and differs between heads and positions
  tok = torch.arange(0, 200, device="cuda")
  keep0 = hstu_cuda.dropout_keep_mask(key, 0, tok, tok, rate)
  keep1 = hstu_cuda.dropout_keep_mask(key, 1, tok, tok, rate)
  assert abs(float(keep0.float().mean()) - (1 - rate)) < 0.02 and bool((keep0 != keep1).any())
  g = (torch.randn_like(ref) * 0.1).to(torch.bfloat16)
  out.backward(g)
  ref.backward(g.float())
  for name, x, y in zip("qkv", a, r):
    assert float((x.grad.float() - y.grad).abs().max()) <= tol(y.grad), name
  # without a rate nothing is dropped
  o0 = A.jagged_pointwise_attention(q, k, v, offs.cuda(), 256, causal=True)
  r0 = A.jagged_attention_reference(q.float(), k.float(), v.float(), offs.cuda(), 256, causal=True)
  assert float((o0.float() - r0).abs().max()) <= tol(r0)
