"""Per-batch memo of the attention front end: aliases of a tensor hit, in-place changes and new
parameters miss, and the table keeps a fixed set of entries however many batches pass."""
import torch

from recml_b200.ops import hstu_cuda as H


def test_alias_hits_and_version_bump_misses():
  H._memo.clear()
  calls = []
  src = torch.arange(8, dtype=torch.int64)

  def make():
    calls.append(1)
    return src.clone()

  a = H._remember("ts32", src, make)
  b = H._remember("ts32", src.view(8), make)            # a new tensor object over the same storage
  assert a is b and len(calls) == 1
  src.add_(1)                                            # in-place change bumps the version counter
  c = H._remember("ts32", src, make)
  assert c is not a and len(calls) == 2
  d = H._remember("ts32", src, make, extra=(1,))         # same tensor, other parameters
  assert d is not c and len(calls) == 3


def test_table_does_not_grow_with_batches():
  H._memo.clear()
  for T in range(100, 140):
    offs = torch.tensor([0, T], dtype=torch.int32)
    H._remember("tiles_f", offs, lambda: T, (T,))
    H._remember("tiles_b", offs, lambda: T, (T,))
    H._remember("buckets", offs, lambda: T, (T, 4096, 128, True))
  assert set(H._memo) == {"tiles_f", "tiles_b", "buckets"}


def test_offsets32_is_stable_per_batch():
  H._memo.clear()
  o64 = torch.tensor([0, 5, 9], dtype=torch.int64)
  a, b = H.offsets32(o64), H.offsets32(o64)
  assert a is b and a.dtype == torch.int32
  o32 = torch.tensor([0, 5, 9], dtype=torch.int32)
  assert H.offsets32(o32) is o32
