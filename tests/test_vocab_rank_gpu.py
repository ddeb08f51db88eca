"""Fused all-gather → GEMM → rank-count kernel vs the fp32 matmul oracle (single GPU)."""
import pytest
import torch

from recml_b200.metrics import ranking
from recml_b200.ops import _lib, vocab_rank as VR

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,D,V", [(128, 256, 5000), (300, 64, 777), (512, 128, 40000)])
def test_counts_match_oracle(rows, D, V):
  g = torch.Generator().manual_seed(0)
  x = (torch.randn(rows, D, generator=g) * 0.3).to(torch.bfloat16).cuda()
  shard = (torch.randn(V, D, generator=g) * 0.3).to(torch.bfloat16).cuda()
  target = torch.randint(0, V, (rows,), generator=g).cuda()
  pos = (x.float() * shard[target].float()).sum(-1)
  ranker = VR.VocabRanker(rows, D)
  for _ in range(2):     # twice: device-side sequence numbers and buffer parity advance
    ranks = ranker.ranks(x, pos, target, shard, 1, 0)
    torch.cuda.synchronize()
    _lib.check_status()
  ref = 1 + VR.counts_reference(x, shard, pos, target, 1, 0).long()
  # scores within rounding distance of the positive may fall on either side of the comparison
  s = x.float() @ shard.float().t()
  near = ((s - pos[:, None]).abs() < 2e-3 * s.abs().max()).sum(1)
  assert bool(((ranks - ref).abs() <= near).all()), (ranks[:8], ref[:8])
  assert float((ranks == ref).float().mean()) > 0.9
  full = ranking.rank_of_target(s, target)
  assert float((full - ref).abs().float().mean()) < 1.0
