"""The allocation-free embedding update entry point (`recml_emb_bwd_update_static`).

Who needs it: callers that may not allocate device memory at the time of the call — a serving or
training process whose whole memory budget was handed out at start-up, or a host application that
uses this library without torch's allocator.  They pass tables, optimizer state, the sorted
occurrence lists and gradients as usual; the scratch that the ordinary entry point receives from
the caller is a fixed array inside the library here.

The test drives both entry points through their exported C symbols on identical inputs — row-wise
Adagrad over occurrence lists with hot rows whose runs span many 128-entry ranges, which is exactly
what the scratch is for — twice in a row with different data, and requires the updated tables and
optimizer state to agree within the tolerance of the other embedding tests.  The second round
proves that leftovers of the first call in the shared array do not leak into the next one.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, n_occ, rows, dim, n_vec):
  rng = np.random.default_rng(seed)
  hot = rng.integers(0, 4, size=n_occ // 2)                       # 4 rows take half of all occurrences
  cold = rng.integers(4, rows, size=n_occ - hot.size)
  keys = np.sort(np.concatenate([hot, cold])).astype(np.int32)
  vals = rng.integers(0, n_vec, size=n_occ).astype(np.int32)
  grads = (rng.normal(size=(n_vec, dim)) * 0.1).astype(np.float32)
  dev = torch.device("cuda")
  return (torch.from_numpy(keys).to(dev), torch.from_numpy(vals).to(dev),
          torch.from_numpy(grads).to(dev).to(torch.bfloat16))


def _params(fused, keys, vals, grads, count, table, slot, scratch, status, dim):
  bp = fused.BwdParams()
  bp.keys, bp.vals, bp.occ_gain, bp.n_occ = keys.data_ptr(), vals.data_ptr(), None, count.data_ptr()
  bp.grads, bp.val_scale = grads.data_ptr(), dim
  bp.table, bp.slot0, bp.slot1 = table.data_ptr(), slot.data_ptr(), None
  bp.dloc, bp.opt = dim, fused.OPT["rowwise_adagrad"]
  for i, v in enumerate((0.05, 1e-8, 0, 0, 0, 0)):
    bp.hp[i] = v
  bp.grad_scale = 1.0
  bp.scratch = None if scratch is None else scratch.data_ptr()
  bp.wait_flags, bp.W, bp.status = None, 1, status.data_ptr()
  return bp


def test_static_scratch_entry_matches_regular_entry_twice():
  from recml_b200 import _build
  from recml_b200.embedding import fused
  lib = ctypes.CDLL(_build.build()["cuda"])           # the exported C symbols, no Python wrapper in between
  regular, static = lib.recml_emb_bwd_update, lib.recml_emb_bwd_update_static
  rows, dim, n_vec = 5000, 128, 4096
  dev = torch.device("cuda")
  status = torch.zeros(4, dtype=torch.int32, device=dev)
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  err = ctypes.create_string_buffer(256)
  torch.manual_seed(0)
  table_a = torch.randn(rows, dim, device=dev)
  table_b = table_a.clone()
  slot_a = torch.zeros(rows, device=dev)
  slot_b = slot_a.clone()
  for rnd, n_occ in enumerate((60000, 35001)):
    keys, vals, grads = _inputs(10 + rnd, n_occ, rows, dim, n_vec)
    count = torch.tensor([n_occ], dtype=torch.int32, device=dev)
    scratch = torch.zeros((n_occ + 127) // 128, dim, device=dev)
    pa = _params(fused, keys, vals, grads, count, table_a, slot_a, scratch, status, dim)
    assert regular(ctypes.byref(pa), ctypes.c_longlong(n_occ), ctypes.c_int(0), ctypes.c_int(0), stream) == 0
    pb = _params(fused, keys, vals, grads, count, table_b, slot_b, None, status, dim)
    rc = static(ctypes.byref(pb), ctypes.c_longlong(n_occ), ctypes.c_int(0), stream, err, ctypes.c_int(256))
    assert rc == 0, err.value
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    # fp32 atomics make the summation order of hot rows free, hence a tolerance rather than equality
    torch.testing.assert_close(table_b, table_a, atol=3e-3, rtol=3e-3)
    torch.testing.assert_close(slot_b, slot_a, atol=3e-3, rtol=3e-3)
    assert float((table_a - table_b).abs().max()) < 3e-3
  # the update really happened (hot rows moved)
  assert float(slot_a[:4].min()) > 0


def test_static_scratch_entry_rejects_oversize_requests():
  from recml_b200 import _build
  from recml_b200.embedding import fused
  lib = ctypes.CDLL(_build.build()["cuda"])
  dev = torch.device("cuda")
  status = torch.zeros(4, dtype=torch.int32, device=dev)
  dummy = torch.zeros(8, device=dev)
  idx = torch.zeros(8, dtype=torch.int32, device=dev)
  err = ctypes.create_string_buffer(256)
  stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  p = _params(fused, idx, idx, dummy.to(torch.bfloat16), idx, dummy, dummy, None, status, 128)
  rc = lib.recml_emb_bwd_update_static(ctypes.byref(p), ctypes.c_longlong(262144 + 1), ctypes.c_int(0), stream, err,
                                       ctypes.c_int(256))
  assert rc == -21 and b"MAX_OCC" in err.value
  p.dloc = 256
  rc = lib.recml_emb_bwd_update_static(ctypes.byref(p), ctypes.c_longlong(64), ctypes.c_int(0), stream, err,
                                       ctypes.c_int(256))
  assert rc == -22 and b"MAX_DIM" in err.value
