"""ctypes driver of the jagged HSTU attention kernels (`csrc/cuda/hstu_attention.cu`)."""
from __future__ import annotations

import ctypes

import torch

from recml_b200.ops import _lib

c_int, c_float, c_vp = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


class _Params(ctypes.Structure):
  _fields_ = [("T", c_int), ("H", c_int), ("Dh", c_int), ("B", c_int), ("max_seq_len", c_int),
              ("num_buckets", c_int), ("causal", c_int), ("scale", c_float), ("inv_n", c_float),
              ("seq_offsets", c_vp), ("tile_seq", c_vp), ("tile_row0", c_vp), ("timestamps", c_vp),
              ("pos_w", c_vp), ("ts_w", c_vp), ("out", c_vp), ("dq", c_vp), ("dk", c_vp), ("dv", c_vp),
              ("dpos_w", c_vp), ("dts_w", c_vp), ("status", c_vp), ("softmax", c_int), ("lse", c_vp),
              ("delta", c_vp), ("ld_q", c_int), ("ld_k", c_int), ("ld_v", c_int), ("ld_do", c_int),
              ("bucket_cache", c_vp), ("pair_base", c_vp), ("cap_pairs", c_int)]


_ok: bool | None = None


def available() -> bool:
  global _ok
  if _ok is None:
    try:
      _ok = int(_lib.cuda().recml_hstu_struct_size()) == ctypes.sizeof(_Params)
    except Exception:  # pylint: disable=broad-except
      _ok = False
  return _ok


# Every layer of a model (and its backward) passes the SAME seq_offsets / timestamps tensors: what is
# derived from them is computed once per batch and remembered for the tensor object it came from.
_memo: dict[str, tuple] = {}


def _remember(kind: str, src: torch.Tensor, make, extra: tuple = ()):
  """One remembered value per kind (a fixed set of kinds, so the table cannot grow with the batches seen),
  valid while `src` keeps its storage, shape and version and `extra` is unchanged.  The entry
  holds `src` itself, so its storage cannot be handed to another tensor in the meantime: a tensor object
  with the same address, layout and version counter is an alias of it (autograd hands the backward pass
  such aliases of what the forward saved)."""
  key = (src.data_ptr(), src._version, tuple(src.shape), tuple(src.stride()), src.dtype, extra)
  hit = _memo.get(kind)
  if hit is not None and hit[0] == key:
    return hit[2]
  val = make()
  _memo[kind] = (key, src, val)
  return val


def _ts32(timestamps):
  """Seconds relative to the earliest timestamp of the batch as int32 (the kernels only use differences)."""
  if timestamps is None:
    return None
  if timestamps.dtype == torch.int32:
    return timestamps.contiguous()
  return _remember("ts32", timestamps, lambda: (timestamps - timestamps.min()).to(torch.int32).contiguous())


def offsets32(seq_offsets: torch.Tensor) -> torch.Tensor:
  """`seq_offsets` as contiguous int32, the same tensor object for every call of a batch (what is derived
  from the offsets is remembered per tensor, so a fresh conversion per layer would defeat it)."""
  if seq_offsets.dtype == torch.int32 and seq_offsets.is_contiguous():
    return seq_offsets
  return _remember("offs32", seq_offsets, lambda: seq_offsets.to(torch.int32).contiguous())


def _tiles(seq_offsets: torch.Tensor, T: int, backward: bool = False):
  """Work-sorted tile list of the batch (heaviest tiles first); the backward kernel, which walks key
  tiles, has its own order."""
  return _remember("tiles_b" if backward else "tiles_f", seq_offsets, lambda: _make_tiles(seq_offsets, T, backward), (T,))


def _make_tiles(seq_offsets: torch.Tensor, T: int, backward: bool = False):
  B = seq_offsets.numel() - 1
  cap = (T + 127) // 128 + B
  tile_seq = torch.empty(cap, dtype=torch.int32, device=seq_offsets.device)
  tile_row0 = torch.zeros(cap, dtype=torch.int32, device=seq_offsets.device)
  _lib.check_rc(_lib.cuda().recml_hstu_tile_list(_lib.ptr(seq_offsets), c_int(B), _lib.ptr(tile_seq),
                                                 _lib.ptr(tile_row0), c_int(cap), c_int(int(backward)),
                                                 _lib.stream()), "hstu_tile_list")
  return tile_seq, tile_row0, cap


BUCKET_CACHE_MAX_BYTES = 1 << 30


def _bucket_cache(seq_offsets, ts32, T: int, max_seq_len: int, num_buckets: int, causal: bool):
  """Time-bucket indices of every (query tile, key tile) pair of the batch as uint8 blocks of 128 x 128,
  computed once per batch: all heads, all layers and both passes read the same ones.  Returns
  (cache, pair_base, cap_pairs) or None when the blocks would not fit the size limit (the kernels then
  compute the buckets inline)."""
  if ts32 is None or num_buckets + 1 > 256:
    return None
  B = seq_offsets.numel() - 1
  cap = (T + 127) // 128 + B
  max_nt = (max_seq_len + 127) // 128
  cap_pairs = cap * ((max_nt + 2) // 2 if causal else max_nt)
  if cap_pairs * 16384 > BUCKET_CACHE_MAX_BYTES:
    return None

  def make():
    tiles = _tiles(seq_offsets, T)
    cache = torch.empty(cap_pairs * 16384, dtype=torch.uint8, device=seq_offsets.device)
    pair_base = torch.empty(B + 1, dtype=torch.int32, device=seq_offsets.device)
    _lib.check_rc(_lib.cuda().recml_hstu_bucket_cache(
        _lib.ptr(seq_offsets), c_int(B), _lib.ptr(tiles[0]), _lib.ptr(tiles[1]), c_int(tiles[2]), _lib.ptr(ts32),
        c_int(num_buckets), c_int(int(causal)), c_int(max_nt), _lib.ptr(pair_base), _lib.ptr(cache), c_int(cap_pairs),
        _lib.stream()), "hstu_bucket_cache")
    return cache, pair_base, cap_pairs, seq_offsets   # the offsets the blocks were made for stay alive with them

  hit = _remember("buckets", ts32, make, (T, max_seq_len, num_buckets, bool(causal)))
  same = hit[3] is seq_offsets or (hit[3].data_ptr() == seq_offsets.data_ptr() and hit[3]._version == seq_offsets._version)
  return hit if same else None


def rows_ok(t: torch.Tensor) -> bool:
  """`[T, H, Dh]` bf16 whose heads are contiguous and whose rows start on 16-byte boundaries: a plain tensor
  or a column slice of a wider matrix (e.g. one of the u|q|k|v blocks of a fused projection)."""
  H, Dh = t.shape[1], t.shape[2]
  return (t.dtype == torch.bfloat16 and t.stride(2) == 1 and t.stride(1) == Dh and t.stride(0) >= H * Dh
          and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0)


def as_rows(t: torch.Tensor) -> torch.Tensor:
  return t if rows_ok(t) else t.contiguous()


def _params(q, seq_offsets, timestamps, pos_w, ts_w, max_seq_len, causal, scale, tiles, k=None, v=None, do=None):
  T, H, Dh = q.shape
  p = _Params()
  p.ld_q = q.stride(0)
  p.ld_k = k.stride(0) if k is not None else 0
  p.ld_v = v.stride(0) if v is not None else 0
  p.ld_do = do.stride(0) if do is not None else 0
  p.T, p.H, p.Dh, p.B, p.max_seq_len = T, H, Dh, seq_offsets.numel() - 1, max_seq_len
  p.num_buckets = ts_w.numel() - 1 if ts_w is not None else 0
  p.causal, p.scale, p.inv_n = int(causal), scale, 1.0 / max_seq_len
  p.seq_offsets, p.tile_seq, p.tile_row0 = seq_offsets.data_ptr(), tiles[0].data_ptr(), tiles[1].data_ptr()
  p.timestamps = timestamps.data_ptr() if (timestamps is not None and ts_w is not None) else None
  p.pos_w = pos_w.data_ptr() if pos_w is not None else None
  p.ts_w = ts_w.data_ptr() if (ts_w is not None and timestamps is not None) else None
  p.status = _lib.status_buffer(q.device).data_ptr()
  if p.ts_w is not None:
    bc = _bucket_cache(seq_offsets, timestamps, T, max_seq_len, p.num_buckets, bool(causal))
    if bc is not None:
      p.bucket_cache, p.pair_base, p.cap_pairs = bc[0].data_ptr(), bc[1].data_ptr(), bc[2]
  return p


def forward(q, k, v, seq_offsets, timestamps, pos_w, ts_w, max_seq_len, causal, scale):
  assert rows_ok(q) and rows_ok(k) and rows_ok(v)
  timestamps = _ts32(timestamps)
  pos_w = None if pos_w is None else pos_w.detach().float().contiguous()
  ts_w = None if ts_w is None else ts_w.detach().float().contiguous()
  tiles = _tiles(seq_offsets, q.shape[0])
  out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
  p = _params(q, seq_offsets, timestamps, pos_w, ts_w, max_seq_len, causal, scale, tiles, k, v)
  p.out = out.data_ptr()
  keep = (timestamps, pos_w, ts_w, tiles)  # referenced until the launch is enqueued
  _lib.check_rc(_lib.cuda().recml_hstu_attn_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), ctypes.byref(p),
                                                c_int(tiles[2]), _lib.stream()), "hstu_attn_fwd")
  del keep
  return out


def backward(do, q, k, v, seq_offsets, timestamps, pos_w, ts_w, max_seq_len, causal, scale):
  """Gradients w.r.t. q, k, v, pos_w, ts_w."""
  lib = _lib.cuda()
  if not hasattr(lib._lib, "recml_hstu_attn_bwd"):
    return _backward_reference(do, q, k, v, seq_offsets, timestamps, pos_w, ts_w, max_seq_len, causal, scale)
  timestamps = _ts32(timestamps)
  pw = None if pos_w is None else pos_w.detach().float().contiguous()
  tw = None if ts_w is None else ts_w.detach().float().contiguous()
  tiles = _tiles(seq_offsets, q.shape[0], backward=True)
  do = as_rows(do)
  dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
  dk, dv = (torch.empty(k.shape, dtype=k.dtype, device=k.device) for _ in range(2))
  dpos = torch.zeros_like(pw) if pw is not None else None
  dts = torch.zeros_like(tw) if (tw is not None and timestamps is not None) else None
  p = _params(q, seq_offsets, timestamps, pw, tw, max_seq_len, causal, scale, tiles, k, v, do)
  p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
  p.dpos_w = dpos.data_ptr() if dpos is not None else None
  p.dts_w = dts.data_ptr() if dts is not None else None
  _lib.check_rc(lib.recml_hstu_attn_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(do),
                                        ctypes.byref(p), c_int(tiles[2]), _lib.stream()), "hstu_attn_bwd")
  return (dq.to(q.dtype), dk, dv, None if dpos is None else dpos.to(pos_w.dtype),
          None if ts_w is None else (dts.to(ts_w.dtype) if dts is not None else torch.zeros_like(ts_w)))


def _backward_reference(do, q, k, v, seq_offsets, timestamps, pos_w, ts_w, max_seq_len, causal, scale):
  from recml_b200.ops import hstu_attention as A
  with torch.enable_grad():
    leaves = [t.detach().float().requires_grad_() for t in (q, k, v)]
    pw = None if pos_w is None else pos_w.detach().float().requires_grad_()
    tw = None if ts_w is None else ts_w.detach().float().requires_grad_()
    o = A.jagged_attention_reference(*leaves, seq_offsets, max_seq_len, pos_w=pw, ts_w=tw, timestamps=timestamps,
                                     causal=causal, scale=scale)
    params = leaves + [t for t in (pw, tw) if t is not None]
    grads = list(torch.autograd.grad(o, params, do.float(), allow_unused=True))
  dq, dk, dv = (g.to(q.dtype) for g in grads[:3])
  rest = grads[3:]
  dpos = rest.pop(0) if pw is not None else None
  dts = rest.pop(0) if tw is not None else None
  return dq, dk, dv, dpos, dts


# ---- softmax mode: the same kernels with P = softmax(scale * QK^T) over the visible keys ----------------------
SOFTMAX_MAX_LEN = 256


def softmax_forward(q, k, v, seq_offsets, max_seq_len, causal, scale):
  """Jagged softmax attention; returns (out `[T, H, Dh]` bf16, row log-sum-exp `[T, H]` fp32)."""
  assert rows_ok(q) and rows_ok(k) and rows_ok(v)
  assert max_seq_len <= SOFTMAX_MAX_LEN
  tiles = _tiles(seq_offsets, q.shape[0])
  out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
  lse = torch.empty(q.shape[0], q.shape[1], dtype=torch.float32, device=q.device)
  p = _params(q, seq_offsets, None, None, None, max_seq_len, causal, scale, tiles, k, v)
  p.out, p.softmax, p.lse = out.data_ptr(), 1, lse.data_ptr()
  _lib.check_rc(_lib.cuda().recml_hstu_attn_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), ctypes.byref(p),
                                                c_int(tiles[2]), _lib.stream()), "softmax_attn_fwd")
  return out, lse


def softmax_backward(do, out, lse, q, k, v, seq_offsets, max_seq_len, causal, scale):
  tiles = _tiles(seq_offsets, q.shape[0], backward=True)
  do = as_rows(do)
  delta = (do.float() * out.float()).sum(-1).contiguous()          # [T, H]
  dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
  dk, dv = (torch.empty(k.shape, dtype=k.dtype, device=k.device) for _ in range(2))
  p = _params(q, seq_offsets, None, None, None, max_seq_len, causal, scale, tiles, k, v, do)
  p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
  p.softmax, p.lse, p.delta = 1, lse.data_ptr(), delta.data_ptr()
  _lib.check_rc(_lib.cuda().recml_hstu_attn_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(do), ctypes.byref(p),
                                                c_int(tiles[2]), _lib.stream()), "softmax_attn_bwd")
  return dq.to(q.dtype), dk, dv
