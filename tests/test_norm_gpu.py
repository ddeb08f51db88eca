"""CUDA LayerNorm family against an fp32 torch reference: forward and all gradients, bf16 io; covers the
16-byte backward (D % 8 == 0, D <= 512) and the generic one, with and without gate / bias / rms."""
import pytest
import torch

from recml_b200.ops import norm as norm_ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,D", [(1000, 256), (333, 512), (257, 64), (100, 72), (64, 1024), (5000, 200)])
@pytest.mark.parametrize("gated,rms,has_bias", [(False, False, True), (True, False, True), (True, True, False)])
def test_layer_norm_matches_fp32_reference(M, D, gated, rms, has_bias):
  torch.manual_seed(D + M)
  x = torch.randn(M, D, device="cuda").to(torch.bfloat16).requires_grad_()
  g = torch.randn(M, D, device="cuda").to(torch.bfloat16).requires_grad_() if gated else None
  w = (1 + 0.1 * torch.randn(D, device="cuda")).requires_grad_()
  b = (0.1 * torch.randn(D, device="cuda")).requires_grad_() if has_bias else None
  dy = torch.randn(M, D, device="cuda").to(torch.bfloat16)

  y = norm_ops.layer_norm(x, w, b, 1e-6, gate=g, rms=rms)
  leaves = [t for t in (x, w, b, g) if t is not None]
  got = torch.autograd.grad(y, leaves, dy)

  xr, wr = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
  br = None if b is None else b.detach().clone().requires_grad_()
  gr = None if g is None else g.detach().float().requires_grad_()
  yr = norm_ops._ln_ref(xr, wr, br, 1e-6, rms)
  if gr is not None:
    yr = yr * gr
  want = torch.autograd.grad(yr, [t for t in (xr, wr, br, gr) if t is not None], dy.float())

  torch.testing.assert_close(y.float(), yr, atol=3e-2, rtol=3e-2)
  for a, e in zip(got, want):
    scale = float(e.abs().max()) + 1e-6
    assert float((a.float() - e).abs().max()) / scale < 2e-2, (a.shape, float((a.float() - e).abs().max()), scale)
