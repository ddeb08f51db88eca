"""CUDA selective scan (SSD recurrence) and depthwise conv + SiLU against the plain fp32 torch formulations."""
import pytest
import torch

from recml_b200.ops import ssd

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,L,H,P,N,init_dim", [(3, 70, 2, 16, 32, 0), (2, 200, 4, 64, 64, 3), (2, 33, 3, 32, 16, 4),
                                                (1, 8, 1, 8, 64, 0)])
def test_scan_matches_recurrence(B, L, H, P, N, init_dim):
  torch.manual_seed(0)
  dev = "cuda"
  x = torch.randn(B, L, H, P, device=dev) * 0.5
  a = -torch.rand(B, L, H, device=dev) * 0.7
  b = torch.randn(B, L, 1, N, device=dev) * 0.5
  c = torch.randn(B, L, 1, N, device=dev) * 0.5
  init = None
  if init_dim == 3:
    init = torch.randn(H, P, N, device=dev) * 0.3
  elif init_dim == 4:
    init = torch.randn(B, H, P, N, device=dev) * 0.3
  leaves = [t.clone().requires_grad_() for t in (x, a, b, c)] + ([init.clone().requires_grad_()] if init is not None else [])
  ref_leaves = [t.clone().requires_grad_() for t in (x, a, b, c)] + ([init.clone().requires_grad_()] if init is not None else [])
  y = ssd.ssd_scan_recurrent_kernel(*leaves[:4], leaves[4] if init is not None else None)
  ri = ref_leaves[4] if init is not None else None
  if ri is not None and ri.dim() == 3:
    ri = ri[None].expand(B, -1, -1, -1)
  y_ref = ssd.ssd_recurrent(*ref_leaves[:4], ri)
  torch.testing.assert_close(y, y_ref, rtol=2e-4, atol=2e-4)
  g = torch.randn_like(y)
  y.backward(g)
  y_ref.backward(g)
  for name, u, v in zip(("dx", "da", "db", "dc", "dinit"), leaves, ref_leaves):
    torch.testing.assert_close(u.grad, v.grad, rtol=2e-3, atol=2e-3, msg=lambda m, n=name: f"{n}: {m}")


@pytest.mark.parametrize("B,L,H,P,init_dim", [(2, 200, 4, 64, 0), (3, 128, 2, 64, 3), (2, 300, 2, 128, 4), (5, 37, 8, 64, 0),
                                              (1, 520, 1, 64, 0)])
def test_tensor_core_quadratic_form_matches_recurrence(B, L, H, P, init_dim):
  """P == N in {64, 128} takes the decay mode of the attention kernels: operands are rounded to bf16 (the oracle
  gets the same rounded inputs), products accumulate in fp32, so the tolerance is that of bf16 scores."""
  torch.manual_seed(2)
  dev = "cuda"
  rb = lambda t: t.to(torch.bfloat16).float()
  x = rb(torch.randn(B, L, H, P, device=dev) * 0.5)
  a = -torch.rand(B, L, H, device=dev) * 0.7
  a[:, ::7] *= 8.0                                        # some strong forgetting steps
  b = rb(torch.randn(B, L, 1, P, device=dev) * 0.3)
  c = rb(torch.randn(B, L, 1, P, device=dev) * 0.3)
  init = None
  if init_dim == 3:
    init = torch.randn(H, P, P, device=dev) * 0.3
  elif init_dim == 4:
    init = torch.randn(B, H, P, P, device=dev) * 0.3
  mk = lambda: [t.clone().requires_grad_() for t in (x, a, b, c)] + ([init.clone().requires_grad_()] if init is not None else [])
  leaves, ref_leaves = mk(), mk()
  assert ssd._quad_supported(x, b)
  y = ssd.ssd_scan(*leaves[:4], 64, leaves[4] if init is not None else None)
  ri = ref_leaves[4] if init is not None else None
  if ri is not None and ri.dim() == 3:
    ri = ri[None].expand(B, -1, -1, -1)
  y_ref = ssd.ssd_recurrent(*ref_leaves[:4], ri)
  tol = lambda ref: 1.5e-2 * float(ref.abs().max())
  assert float((y - y_ref).abs().max()) <= tol(y_ref)
  g = rb(torch.randn_like(y))
  y.backward(g)
  y_ref.backward(g)
  for name, u, v in zip(("dx", "da", "db", "dc", "dinit"), leaves, ref_leaves):
    err = float((u.grad - v.grad).abs().max())
    assert err <= tol(v.grad), f"{name}: {err} vs max {float(v.grad.abs().max())}"
    rel = float((u.grad - v.grad).norm() / v.grad.norm())
    assert rel < 1e-2, f"{name}: relative l2 error {rel}"


@pytest.mark.parametrize("K,use_bias", [(4, True), (4, False), (3, True), (2, False)])
def test_conv_silu_matches_torch(K, use_bias):
  torch.manual_seed(1)
  x = torch.randn(3, 37, 80, device="cuda")
  w = torch.randn(80, K, device="cuda") * 0.5
  bias = torch.randn(80, device="cuda") * 0.1 if use_bias else None
  a = [t.clone().requires_grad_() for t in (x, w)] + ([bias.clone().requires_grad_()] if use_bias else [])
  r = [t.clone().requires_grad_() for t in (x, w)] + ([bias.clone().requires_grad_()] if use_bias else [])
  y = ssd.conv1d_silu(*a)
  y_ref = ssd.causal_depthwise_conv1d_silu(*r)
  torch.testing.assert_close(y, y_ref, rtol=1e-5, atol=1e-5)
  g = torch.randn_like(y)
  y.backward(g)
  y_ref.backward(g)
  for u, v in zip(a, r):
    torch.testing.assert_close(u.grad, v.grad, rtol=1e-4, atol=1e-4)


def test_mamba4rec_trains_on_gpu():
  from recml_b200.layers import mamba
  torch.manual_seed(0)
  m = mamba.Mamba4Rec(vocab_size=500, model_dim=64, mlp_expand=4, num_heads=4, num_layers=2, d_expand=2, d_state=32,
                      chunk_size=32).cuda()
  ids = torch.randint(1, 500, (8, 40), device="cuda")
  opt = torch.optim.Adam(m.parameters(), 1e-3)
  losses = []
  for _ in range(8):
    out = m(ids)
    logits = out if out.dim() == 3 else out[0]
    loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), ids[:, 1:].reshape(-1))
    opt.zero_grad()
    loss.backward()
    opt.step()
    losses.append(float(loss))
  assert losses[-1] < losses[0] and all(l == l for l in losses)
