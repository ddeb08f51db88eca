"""Device id de-duplication against `torch.unique`."""
import pytest
import torch

from recml_b200.ops import id_ops




@pytest.mark.gpu
@pytest.mark.parametrize("n,vocab", [(1, 10), (37, 5), (5000, 300), (100_003, 1_000_000), (300_000, 40_000_000), (4096, 1)])
def test_unique_ids_match_torch_unique(n, vocab):
  g = torch.Generator().manual_seed(n)
  ids = torch.randint(0, vocab, (n,), generator=g, dtype=torch.int32).cuda()
  unique, inverse, count = id_ops.unique_ids(ids, max_id=vocab - 1)
  u_ref, inv_ref = torch.unique(ids.long(), return_inverse=True)
  m = int(count.item())
  assert m == u_ref.numel()
  torch.testing.assert_close(unique[:m].long(), u_ref)
  torch.testing.assert_close(inverse.long(), inv_ref)
  # the inverse expands the distinct ids back to the input
  torch.testing.assert_close(unique[inverse.long()], ids)
  # without the bound the sort walks all 31 bits and gives the same answer
  unique2, inverse2, count2 = id_ops.unique_ids(ids)
  assert int(count2.item()) == m
  torch.testing.assert_close(unique2[:m], unique[:m])
  torch.testing.assert_close(inverse2, inverse)


def test_unique_ids_cpu_path():
  ids = torch.tensor([5, 3, 5, 9, 3], dtype=torch.int32)
  unique, inverse, count = id_ops.unique_ids(ids)
  assert int(count) == 3 and unique[:3].tolist() == [3, 5, 9] and inverse.tolist() == [1, 0, 1, 2, 0]
