"""Device-count radix sort (`csrc/cuda/radix_sort.cu`) against a stable host sort."""
import ctypes

import numpy as np
import pytest
import torch

from recml_b200.ops import _lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,cap,bits,skew", [(1, 64, 5, False), (4095, 4096, 9, False), (4097, 9000, 17, True),
                                              (300_000, 400_000, 25, True), (1_000_003, 1_000_003, 28, True),
                                              (70_000, 70_000, 32, False)])
def test_sort_pairs_matches_stable_host_sort(n, cap, bits, skew):
  lib = _lib.cuda()
  rng = np.random.default_rng(n)
  hi = (1 << bits) - 1
  keys = rng.integers(0, hi + 1, size=n, dtype=np.uint64).astype(np.uint32)
  if skew:   # Zipf-like head: one key takes a fifth of the entries, a few more take another fifth
    keys[rng.random(n) < 0.2] = 7 & hi
    sel = rng.random(n) < 0.2
    keys[sel] = rng.integers(0, 16, size=int(sel.sum())).astype(np.uint32) & hi
  vals = np.arange(n, dtype=np.uint32)
  dev = torch.device("cuda")
  def buf(a):
    t = torch.full((cap,), -1, dtype=torch.int32, device=dev)     # entries beyond n are never read
    t[:n] = torch.from_numpy(a.view(np.int32)).to(dev)
    return t
  ka, va = buf(keys), buf(vals)
  kb, vb = torch.empty_like(ka), torch.empty_like(va)
  count = torch.tensor([n], dtype=torch.int32, device=dev)
  words = int(lib.recml_radix_sort_scratch_words(ctypes.c_longlong(cap)))
  scratch = torch.empty(words, dtype=torch.int32, device=dev)
  status = _lib.status_buffer(dev)
  for _ in range(2):     # twice: the scratch needs no clearing between calls
    rc = lib.recml_radix_sort_pairs(_lib.ptr(ka), _lib.ptr(va), _lib.ptr(kb), _lib.ptr(vb), _lib.ptr(count),
                                    ctypes.c_longlong(cap), ctypes.c_int(bits), _lib.ptr(scratch), _lib.ptr(status),
                                    _lib.stream())
    assert rc in (0, 1)
    torch.cuda.synchronize()
    _lib.check_status()
    ko, vo = (ka, va) if rc == 0 else (kb, vb)
    order = np.argsort(keys, kind="stable")
    np.testing.assert_array_equal(ko[:n].cpu().numpy().view(np.uint32), keys[order])
    np.testing.assert_array_equal(vo[:n].cpu().numpy().view(np.uint32), vals[order])
    # restore the input for the second round (the sort ping-pongs between the buffers)
    ka, va = buf(keys), buf(vals)


def test_count_beyond_capacity_is_clamped_by_readers():
  """The forward kernel's occurrence counter may run past the capacity; the sort is launched over the
  capacity and must only touch entries below min(count, capacity)."""
  lib = _lib.cuda()
  dev = torch.device("cuda")
  cap = 5000
  keys = torch.randint(0, 1 << 12, (cap,), dtype=torch.int32, device=dev)
  vals = torch.arange(cap, dtype=torch.int32, device=dev)
  kb, vb = torch.empty_like(keys), torch.empty_like(vals)
  count = torch.tensor([cap + 777], dtype=torch.int32, device=dev)
  scratch = torch.empty(int(lib.recml_radix_sort_scratch_words(ctypes.c_longlong(cap))), dtype=torch.int32, device=dev)
  ref = keys.cpu().numpy().copy()
  rc = lib.recml_radix_sort_pairs(_lib.ptr(keys), _lib.ptr(vals), _lib.ptr(kb), _lib.ptr(vb), _lib.ptr(count),
                                  ctypes.c_longlong(cap), ctypes.c_int(12), _lib.ptr(scratch),
                                  _lib.ptr(_lib.status_buffer(dev)), _lib.stream())
  torch.cuda.synchronize()
  out = (keys if rc == 0 else kb).cpu().numpy()
  np.testing.assert_array_equal(out, np.sort(ref, kind="stable"))
