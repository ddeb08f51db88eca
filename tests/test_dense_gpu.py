"""MLP / DCNv2 autograd nodes and the memory-bound helpers on CUDA vs fp32 torch on CPU."""
import pytest
import torch

from recml_b200.metrics import confusion
from recml_b200.ops import _lib, bce, dense, elementwise as ew
from recml_b200.training import optim_factory

pytestmark = pytest.mark.gpu


def _close(a, b, tol=3e-2):
  a, b = a.float().cpu(), b.float().cpu()
  err = (a - b).abs().max().item()
  scale = b.abs().max().item() + 1e-6
  assert err / scale < tol, f"rel err {err / scale}"


def _ref_mlp_bf16(x, ws, bs, flags, go):
  """fp32 math on bf16-rounded operands and activations (what the kernels see), with the ReLU masks
  taken from the rounded activations; returns output, weight grads, bias grads, input grad."""
  r = lambda t: t.to(torch.bfloat16).float()
  acts = [r(x)]
  for w, b, f in zip(ws, bs, flags):
    z = acts[-1] @ r(w).t() + b
    z = torch.relu(z) if f else z
    acts.append(r(z) if w.shape[0] > 1 else z)
  g = go.float() if ws[-1].shape[0] == 1 else r(go)
  dws, dbs = [], []
  for i in range(len(ws) - 1, -1, -1):
    if flags[i]:
      g = g * (acts[i + 1] > 0)
    dws.insert(0, g.t() @ acts[i])
    dbs.insert(0, g.sum(0))
    g = g @ (ws[i] if ws[i].shape[0] == 1 else r(ws[i]))
    g = r(g)
  return acts[-1], dws, dbs, g


def test_mlp_forward_backward():
  torch.manual_seed(0)
  M, dims = 300, [13, 512, 256, 128]
  ws = [torch.randn(dims[i + 1], dims[i]) * (1.0 / dims[i]) ** 0.5 for i in range(3)]
  bs = [torch.randn(dims[i + 1]) * 0.1 for i in range(3)]
  x = torch.randn(M, 13)
  flags = [True, True, True]
  go = torch.randn(M, dims[-1])
  yr, dws, dbs, _ = _ref_mlp_bf16(x, ws, bs, flags, go)
  pg = [t.clone().cuda().requires_grad_() for t in ws + bs]
  yg = dense.mlp(x.cuda(), pg[:3], pg[3:], flags)
  _close(yg, yr, tol=1e-2)
  yg.backward(go.cuda().to(yg.dtype))
  torch.cuda.synchronize()
  _lib.check_status()
  for a, b in zip(pg, dws + dbs):
    _close(a.grad, b, tol=2e-2)
  # and the fp32 CPU path of the same function agrees in the forward direction
  _close(yg, dense.mlp(x, ws, bs, flags), tol=2e-2)


def test_top_mlp_with_gemv_head():
  torch.manual_seed(1)
  M, dims = 260, [384, 256, 64, 1]
  ws = [torch.randn(dims[i + 1], dims[i]) * (1.0 / dims[i]) ** 0.5 for i in range(3)]
  bs = [torch.randn(dims[i + 1]) * 0.1 for i in range(3)]
  x = (torch.randn(M, 384)).to(torch.bfloat16)
  flags = [True, True, False]
  go = torch.randn(M, 1)
  yr, dws, dbs, dxr = _ref_mlp_bf16(x.float(), ws, bs, flags, go)
  pg = [t.clone().cuda().requires_grad_() for t in ws + bs]
  xg = x.cuda().requires_grad_()
  yg = dense.mlp(xg, pg[:3], pg[3:], flags)
  _close(yg, yr, tol=1e-2)
  yg.backward(go.cuda())
  torch.cuda.synchronize()
  _lib.check_status()
  for a, b in zip(pg + [xg], dws + dbs + [dxr]):
    _close(a.grad, b.reshape(a.grad.shape), tol=2e-2)


@pytest.mark.parametrize("rank", [64, None])
def test_cross_network(rank):
  torch.manual_seed(2)
  M, d, L = 200, 384, 3
  x0 = (torch.randn(M, d) * 0.5).to(torch.bfloat16)
  us = [torch.randn(rank, d) * 0.05 for _ in range(L)] if rank else None
  vs = [torch.randn(d, rank or d) * 0.05 for _ in range(L)]
  bs = [torch.randn(d) * 0.1 for _ in range(L)]
  def leaves(dev):
    mk = lambda t: t.clone().to(dev).requires_grad_()
    return ([mk(t) for t in us] if us else None), [mk(t) for t in vs], [mk(t) for t in bs]
  uc, vc, bc = leaves("cpu")
  ug, vg, bg = leaves("cuda")
  xc, xg = x0.float().requires_grad_(), x0.cuda().requires_grad_()
  yc, yg = dense.cross_network(xc, uc, vc, bc), dense.cross_network(xg, ug, vg, bg)
  _close(yg, yc)
  go = (torch.randn_like(yc) * 0.1)
  yc.backward(go)
  yg.backward(go.cuda().to(yg.dtype))
  torch.cuda.synchronize()
  _lib.check_status()
  for a, b in zip((ug or []) + vg + bg + [xg], (uc or []) + vc + bc + [xc]):
    _close(a.grad, b.grad, tol=5e-2)


def test_bce_fused_matches_reference():
  torch.manual_seed(3)
  n = 10000
  x, y = torch.randn(n) * 2, (torch.rand(n) < 0.25).float()
  rc = bce.bce_with_logits(x, y, grad_scale=1.0 / n)
  rg = bce.bce_with_logits(x.cuda(), y.cuda(), grad_scale=1.0 / n)
  for f in ("loss_sum", "weight_sum", "label_sum", "pred_sum", "correct_sum", "dlogits", "hist_pos", "hist_neg"):
    torch.testing.assert_close(getattr(rg, f).cpu(), getattr(rc, f), atol=1e-2, rtol=1e-4)
  # histograms reproduce the thresholded confusion counts of the metric library exactly
  tp, tn, fp, fn = confusion.estimate_confusion_matrix(torch.sigmoid(x), y, None, confusion.default_thresholds(200))
  tp2, tn2, fp2, fn2 = confusion.confusion_from_histograms(rg.hist_pos.cpu(), rg.hist_neg.cpu())
  torch.testing.assert_close(tp2, tp); torch.testing.assert_close(fp2, fp)


@pytest.mark.parametrize("factory", [
    optim_factory.AdamFactory(learning_rate=1e-2, weight_decay=1e-2, grad_clip_norm=1.0),
    optim_factory.AdagradFactory(learning_rate=1e-2, grad_clip_norm=0.5),
    optim_factory.SGDFactory(learning_rate=1e-2)], ids=["adamw", "adagrad", "sgd"])
def test_fused_optimizer_matches_cpu(factory):
  torch.manual_seed(4)
  shapes = [(300, 70), (70,), (1, 9), (2049,)]
  pc = {f"p{i}": torch.randn(s).requires_grad_() for i, s in enumerate(shapes)}
  pg = {k: v.detach().clone().cuda().requires_grad_() for k, v in pc.items()}
  oc, og = factory.make().init(pc), factory.make().init(pg)
  for _ in range(4):
    for k in pc:
      g = torch.randn_like(pc[k])
      pc[k].grad, pg[k].grad = g, g.cuda()
    oc.step(); og.step()
  for k in pc:
    torch.testing.assert_close(pg[k].detach().cpu(), pc[k].detach(), atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("shape,ld", [((1000, 1024), 1024), ((777, 128), 384), ((513, 72), 72), ((300, 50), 50),
                                      ((4100, 264), 520)])
def test_colsum_matches_fp32_sum(shape, ld):
  """Bias-gradient column sums: the 16-byte path (N % 8 == 0) and the generic one, dense and row-strided."""
  M, N = shape
  torch.manual_seed(3)
  full = torch.randn(M, ld, device="cuda").to(torch.bfloat16)
  x = full[:, :N]
  got = ew.colsum(x)
  want = x.float().sum(0)
  torch.testing.assert_close(got, want, atol=2e-3 * M ** 0.5, rtol=1e-4)
  # accumulation into an existing vector
  again = ew.colsum(x, out=got.clone())
  torch.testing.assert_close(again, 2 * want, atol=4e-3 * M ** 0.5, rtol=1e-4)
