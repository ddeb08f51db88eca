"""Softmax mode of the tcgen05 attention kernels against the dense fp32 formulation."""
import math

import pytest
import torch

from recml_b200.ops import softmax_attention as sm

pytestmark = pytest.mark.gpu


def _dense(q, k, v, padding_mask, causal):
  B, L = q.shape[:2]
  mask = sm.merge_masks(B, L, q.device, padding_mask=padding_mask, causal=causal)
  return sm.softmax_attention(q, k, v, mask)


@pytest.mark.parametrize("B,L,H,Dh,causal,pad", [(3, 200, 4, 64, True, "left"), (2, 256, 2, 64, False, "right"),
                                                 (4, 50, 2, 64, True, None), (2, 130, 1, 128, True, "left"),
                                                 (2, 128, 2, 64, False, None), (2, 700, 2, 64, True, "right"),
                                                 (1, 1100, 1, 128, False, "left"), (2, 513, 2, 64, False, None)])
def test_structured_attention_matches_dense(B, L, H, Dh, causal, pad):
  torch.manual_seed(0)
  dev = "cuda"
  q, k, v = (torch.randn(B, L, H, Dh, device=dev).to(torch.bfloat16).float() for _ in range(3))
  # keys grow along the sequence so that the running maximum of a row keeps rising from tile to tile
  k = (k * torch.linspace(0.5, 2.0, L, device=dev)[None, :, None, None]).to(torch.bfloat16).float()
  padding_mask = None
  if pad is not None:
    lens = torch.randint(L // 3, L + 1, (B,), device=dev)
    ar = torch.arange(L, device=dev)[None]
    padding_mask = (ar >= (L - lens)[:, None]) if pad == "left" else (ar < lens[:, None])
  a = [t.clone().requires_grad_() for t in (q, k, v)]
  r = [t.clone().requires_grad_() for t in (q, k, v)]
  out = sm.structured_attention(*a, padding_mask, causal)
  ref = _dense(*r, padding_mask, causal)
  valid = padding_mask if padding_mask is not None else torch.ones(B, L, dtype=torch.bool, device=dev)
  w = valid[..., None, None].float()
  torch.testing.assert_close(out * w, ref * w, rtol=2e-2, atol=2e-2)
  if padding_mask is not None:
    assert float((out * (1 - w)).abs().max()) == 0.0          # padded queries come back as zeros
  g = torch.randn_like(out) * w
  out.backward(g)
  ref.backward(g)
  for name, x, y in zip("qkv", a, r):
    torch.testing.assert_close(x.grad * w, y.grad * w, rtol=3e-2, atol=3e-2, msg=lambda m, n=name: f"d{n}: {m}")


def test_sasrec_block_uses_the_kernel_and_trains():
  from recml_b200.layers import sasrec
  torch.manual_seed(0)
  m = sasrec.SASRec(vocab_size=300, max_positions=64, model_dim=128, mlp_dim=256, num_heads=2, num_layers=2).cuda()
  ids = torch.randint(1, 300, (8, 64), device="cuda")
  mask = torch.ones(8, 64, dtype=torch.bool, device="cuda")
  mask[:, :10] = False
  opt = torch.optim.Adam(m.parameters(), 1e-3)
  losses = []
  for _ in range(6):
    logits = m(ids, padding_mask=mask)
    loss = torch.nn.functional.cross_entropy(logits[:, 10:-1].reshape(-1, logits.shape[-1]).float(), ids[:, 11:].reshape(-1))
    opt.zero_grad()
    loss.backward()
    opt.step()
    losses.append(float(loss.detach()))
  assert all(l == l for l in losses) and losses[-1] < losses[0]


@pytest.mark.parametrize("rate,L,causal", [(0.2, 200, True), (0.5, 330, False)])
def test_attention_dropout_in_the_softmax_kernels(rate, L, causal):
  """Dropout on the softmax weights (reference `recml/layers/keras/sasrec.py:89-101`: the decoder blocks are built
  with the model's dropout rate) runs inside the kernels: the weights are normalised over ALL visible keys, then dropped and
  rescaled before they multiply the values.  The oracle rebuilds the mask from the key that the call drew."""
  from recml_b200.ops import hstu_attention as A, hstu_cuda
  torch.manual_seed(5)
  B, H, Dh = 2, 2, 64
  dev = "cuda"
  q, k, v = ((torch.randn(B, L, H, Dh, device=dev) * 0.8).to(torch.bfloat16).float() for _ in range(3))
  a = [t.clone().requires_grad_() for t in (q, k, v)]
  r = [t.clone().requires_grad_() for t in (q, k, v)]
  out = sm.structured_attention(*a, None, causal, dropout_p=rate, training=True)
  key = int(A.LAST_DROPOUT_KEY.item())
  # the kernels number tokens over the packed batch: sequence b holds tokens b * L .. b * L + L - 1
  keep = torch.stack([torch.stack([hstu_cuda.dropout_keep_mask(key, h, torch.arange(b * L, (b + 1) * L, device=dev),
                                                                torch.arange(b * L, (b + 1) * L, device=dev), rate)
                                   for h in range(H)]) for b in range(B)])            # [B, H, L, L]
  s = torch.einsum("bqhd,bkhd->bhqk", r[0], r[1]) / math.sqrt(Dh)
  if causal:
    s = s.masked_fill(~torch.tril(torch.ones(L, L, dtype=torch.bool, device=dev)), float("-inf"))
  p = torch.softmax(s, -1) * keep.float() / (1.0 - rate)
  ref = torch.einsum("bhqk,bkhd->bqhd", p, r[2])
  torch.testing.assert_close(out, ref, rtol=2e-2, atol=2e-2)
  assert abs(float(keep.float().mean()) - (1 - rate)) < 0.02
  g = torch.randn_like(out)
  out.backward(g)
  ref.backward(g)
  for name, x, y in zip("qkv", a, r):
    torch.testing.assert_close(x.grad, y.grad, rtol=3e-2, atol=3e-2, msg=lambda m, n=name: f"d{n}: {m}")
  # evaluation mode drops nothing
  o_eval = sm.structured_attention(q, k, v, None, causal, dropout_p=rate, training=False)
  torch.testing.assert_close(o_eval, _dense(q, k, v, None, causal), rtol=2e-2, atol=2e-2)
