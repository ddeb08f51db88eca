"""tcgen05 GEMM vs a plain PyTorch fp32 reference of the same contraction."""
import pytest
import torch

from recml_b200.ops import _lib
from recml_b200.ops import gemm as G

pytestmark = pytest.mark.gpu


def _rand(*shape):
  return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)


def _check(out, ref, tol=2e-2):
  torch.cuda.synchronize()
  _lib.check_status()
  err = (out.float() - ref.float()).abs().max().item()
  scale = ref.float().abs().max().item() + 1e-6
  assert err / scale < tol, f"max err {err} scale {scale}"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (300, 136, 200),
                                   (1024, 512, 3456), (130, 3456, 512), (64, 8, 16)])
def test_tn(M, N, K):
  a, b = _rand(M, K), _rand(N, K)
  _check(G.gemm(a, b), G.gemm_reference(a.cpu(), b.cpu()).cuda())


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (300, 136, 200), (512, 3456, 512)])
def test_b_mn_major(M, N, K):
  a, b = _rand(M, K), _rand(K, N)
  _check(G.gemm(a, b, b_mn=True), G.gemm_reference(a.cpu(), b.cpu(), b_mn=True).cuda())


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (136, 304, 1000), (512, 3456, 2048)])
def test_both_mn_major_f32_out(M, N, K):
  a, b = _rand(K, M), _rand(K, N)
  out = G.gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32)
  ref = G.gemm_reference(a.cpu(), b.cpu(), a_mn=True, b_mn=True, out_dtype=torch.float32).cuda()
  _check(out, ref)
  acc = torch.ones(M, N, device="cuda")
  G.gemm(a, b, a_mn=True, b_mn=True, accumulate_into=acc)
  _check(acc, ref + 1.0)


def test_bias_relu_and_epilogues():
  M, N, K = 384, 264, 320
  a, b = _rand(M, K), _rand(N, K)
  bias = torch.randn(N, device="cuda")
  x0, xl = _rand(M, N), _rand(M, N)
  _check(G.gemm(a, b, bias=bias, relu=True),
         G.gemm_reference(a.cpu(), b.cpu(), bias=bias.cpu(), relu=True).cuda())
  out, v = G.gemm(a, b, bias=bias, epi=G.EPI_CROSS, aux0=x0, aux1=xl, want_out2=True)
  ref, vref = G.gemm_reference(a.cpu(), b.cpu(), bias=bias.cpu(), epi=G.EPI_CROSS, aux0=x0.cpu(),
                               aux1=xl.cpu(), want_out2=True)
  _check(out, ref.cuda())
  _check(v, vref.cuda())
  _check(G.gemm(a, b, epi=G.EPI_MASK_RELU, aux0=x0),
         G.gemm_reference(a.cpu(), b.cpu(), epi=G.EPI_MASK_RELU, aux0=x0.cpu()).cuda())
  _check(G.gemm(a, b, epi=G.EPI_MUL_ADD, aux0=x0, aux1=xl),
         G.gemm_reference(a.cpu(), b.cpu(), epi=G.EPI_MUL_ADD, aux0=x0.cpu(), aux1=xl.cpu()).cuda())
  _check(G.gemm(a, b, epi=G.EPI_ADD, aux0=x0),
         G.gemm_reference(a.cpu(), b.cpu(), epi=G.EPI_ADD, aux0=x0.cpu()).cuda())
  _check(G.gemm(a, b, epi=G.EPI_ADD, aux0=x0, aux1=xl),
         G.gemm_reference(a.cpu(), b.cpu(), epi=G.EPI_ADD, aux0=x0.cpu(), aux1=xl.cpu()).cuda())
