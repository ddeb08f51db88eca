"""Device-side id de-duplication (`id_unique`): the distinct ids of a list, their number, and the inverse map.

The reference de-duplicates ids per partition on the host before they reach the embedding engine
(`jax_tpu_embedding/sparsecore/lib/core/input_preprocessing.py:27-252`).  Here the embedding backward
merges duplicates itself (sort + run reduction), and this op is the stand-alone form for callers that want
the distinct rows of a batch: statistics for feedback-directed sizing, evaluation code that scores every
distinct candidate once, the NCCL stand-in backend.  On CUDA it is the library's radix sort followed by three
small kernels (`csrc/cuda/id_unique.cu`); nothing is read back to the host.
"""
from __future__ import annotations

import ctypes

import torch


def unique_ids(ids: torch.Tensor, max_id: int | None = None):
  """`ids` int32 / int64 `[n]`, non-negative.  Returns `(unique, inverse, count)`: `unique [n]` int32 holds the
  distinct ids in increasing order in its first `count` entries (the rest is unspecified), `inverse [n]` int32
  gives for every input position the index of its id in `unique`, `count` is an int32 tensor of one element on
  the ids' device.  `max_id` (an upper bound of the ids) shortens the sort; default: all 31 bits."""
  n = ids.numel()
  if not ids.is_cuda or n == 0:
    u, inv = torch.unique(ids.reshape(-1).to(torch.int64), return_inverse=True)
    unique = torch.zeros(n, dtype=torch.int32, device=ids.device)
    unique[:u.numel()] = u.to(torch.int32)
    return unique, inv.to(torch.int32), torch.tensor([u.numel()], dtype=torch.int32, device=ids.device)
  from recml_b200.ops import _lib
  lib = _lib.cuda()
  dev = ids.device
  keys = [ids.reshape(-1).to(torch.int32).clone(), torch.empty(n, dtype=torch.int32, device=dev)]
  vals = [torch.arange(n, dtype=torch.int32, device=dev), torch.empty(n, dtype=torch.int32, device=dev)]
  n_dev = torch.tensor([n], dtype=torch.int32, device=dev)
  key_bits = 31 if max_id is None else max(1, int(max_id).bit_length())
  sort_scratch = torch.empty(int(lib.recml_radix_sort_scratch_words(ctypes.c_longlong(n))), dtype=torch.int32, device=dev)
  which = lib.recml_radix_sort_pairs(_lib.ptr(keys[0]), _lib.ptr(vals[0]), _lib.ptr(keys[1]), _lib.ptr(vals[1]),
                                     _lib.ptr(n_dev), ctypes.c_longlong(n), ctypes.c_int(key_bits),
                                     _lib.ptr(sort_scratch), _lib.ptr(_lib.status_buffer(dev)), _lib.stream())
  if which < 0:
    raise _lib.NativeError(f"radix sort failed with code {which}")
  _lib.LAUNCHES["count"] += 4 * ((key_bits + 8) // 9) - 1      # four kernels per sort pass
  unique = torch.empty(n, dtype=torch.int32, device=dev)
  inverse = torch.empty(n, dtype=torch.int32, device=dev)
  count = torch.zeros(1, dtype=torch.int32, device=dev)
  scratch = torch.empty(int(lib.recml_id_unique_scratch_words(ctypes.c_longlong(n))), dtype=torch.int32, device=dev)
  _lib.check_rc(lib.recml_id_unique_sorted(_lib.ptr(keys[which]), _lib.ptr(vals[which]), _lib.ptr(n_dev),
                                           ctypes.c_longlong(n), _lib.ptr(unique), _lib.ptr(inverse), _lib.ptr(count),
                                           _lib.ptr(scratch), _lib.stream()), "id_unique")
  return unique, inverse, count
