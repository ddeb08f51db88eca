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


def test_checked_build_guard_words():
  """The RECML_DEBUG build puts guard words around kernel outputs; a GEMM whose N is not a tile multiple and an
  embedding lookup leave them intact (run in a child process: the build flavour is fixed at import time)."""
  import os
  import subprocess
  import sys
  code = (
      "import torch\n"
      "from recml_b200.ops import _lib, gemm as G\n"
      "assert _lib.DEBUG and 'dbg' in _lib._build.cuda_lib_path()\n"
      "a = torch.randn(300, 72, device='cuda', dtype=torch.bfloat16); b = torch.randn(200, 72, device='cuda', dtype=torch.bfloat16)\n"
      "y = G.gemm(a, b); _lib.debug_check()\n"
      "torch.testing.assert_close(y.float(), a.float() @ b.float().t(), rtol=3e-2, atol=3e-1)\n"
      "t = _lib.debug_empty((8, 8), torch.float32, 'cuda', 'probe'); t.view(-1)[:64].fill_(1.0)\n"
      "base = t.view(-1); torch.as_strided(base, (80,), (1,)).fill_(2.0)\n"     # runs 16 floats past the payload
      "try:\n  _lib.debug_check(); print('MISSED')\nexcept _lib.DeviceStatusError as e:\n  print('CAUGHT', e)\n")
  env = dict(os.environ, RECML_DEBUG="1")
  out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=900,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
  assert out.returncode == 0, out.stderr[-2000:]
  assert "CAUGHT" in out.stdout and "probe" in out.stdout
