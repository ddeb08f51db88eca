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
              ("dpos_w", c_vp), ("dts_w", c_vp), ("status", c_vp), ("mode", c_int), ("lse", c_vp),
              ("delta", c_vp), ("ld_q", c_int), ("ld_k", c_int), ("ld_v", c_int), ("ld_do", c_int),
              ("bucket_cache", c_vp), ("pair_base", c_vp), ("cap_pairs", c_int), ("bias_tiles", c_vp),
              ("dbias_tiles", c_vp), ("window", c_int), ("segment_ids", c_vp), ("cum", c_vp),
              ("cum_pitch", ctypes.c_longlong), ("qk_shared", c_int), ("dk_acc", c_vp), ("dcum", c_vp), ("v_rows", c_vp),
              ("dropout_key", c_vp), ("drop_threshold", ctypes.c_uint), ("keep_scale", ctypes.c_float)]

MODE_SILU, MODE_SOFTMAX, MODE_DECAY, MODE_SILU_DROPOUT, MODE_SOFTMAX_DROPOUT = 0, 1, 2, 3, 4


class _BiasParams(ctypes.Structure):
  _fields_ = [("seq_offsets", c_vp), ("tile_seq", c_vp), ("tile_row0", c_vp), ("pair_base", c_vp), ("causal", c_int),
              ("cap_pairs", c_int), ("max_seq_len", c_int), ("window", c_int), ("num_buckets", c_int),
              ("segment_ids", c_vp), ("pos_w", c_vp), ("ts_w", c_vp), ("bucket_cache", c_vp), ("tiles", c_vp),
              ("dbias", c_vp), ("dpos_w", c_vp), ("dts_w", c_vp), ("status", c_vp)]


_ok: bool | None = None


def available() -> bool:
  global _ok
  if _ok is None:
    try:
      _ok = (int(_lib.cuda().recml_hstu_struct_size()) == ctypes.sizeof(_Params) and
             int(_lib.cuda().recml_hstu_bias_struct_size()) == ctypes.sizeof(_BiasParams))
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


# Per-pair blocks (time buckets 16 KB, bias 32 KB, bias gradient 64 KB) are sized for the worst case the
# token capacity allows; beyond this many pairs the caller falls back to the torch formulation.
MAX_PAIRS = 1 << 17


def _pair_capacity(T: int, B: int, max_seq_len: int, causal: bool) -> tuple[int, int, int]:
  """(tile capacity, tiles of the longest sequence, pair capacity): with n_i 128-row tiles per sequence,
  sum n_i <= cap and n_i <= max_nt bound the pairs (n_i (n_i + 1) / 2 causal, n_i^2 full) by cap times
  (max_nt + 1) / 2, respectively max_nt."""
  cap = (T + 127) // 128 + B
  max_nt = (max_seq_len + 127) // 128
  cap_pairs = cap * (max_nt + 1) // 2 + 1 if causal else cap * max_nt
  return cap, max_nt, cap_pairs


def _bucket_cache(seq_offsets, ts32, T: int, max_seq_len: int, num_buckets: int, causal: bool):
  """Time-bucket indices of every (query tile, key tile) pair of the batch as uint8 blocks of 128 x 128,
  computed once per batch: the bias tiles of the step and the bias-gradient pass read them.  Returns
  (cache, pair_base, cap_pairs, seq_offsets)."""
  B = seq_offsets.numel() - 1
  cap, max_nt, cap_pairs = _pair_capacity(T, B, max_seq_len, causal)

  def make():
    tiles = _tiles(seq_offsets, T)
    cache = torch.empty(cap_pairs * 16384, dtype=torch.uint8, device=seq_offsets.device)
    pair_base = torch.empty(B + 1, dtype=torch.int32, device=seq_offsets.device)
    _lib.check_rc(_lib.cuda().recml_hstu_bucket_cache(
        _lib.ptr(seq_offsets), c_int(B), _lib.ptr(tiles[0]), _lib.ptr(tiles[1]), c_int(tiles[2]), _lib.ptr(ts32),
        c_int(num_buckets), c_int(int(causal)), c_int(max_nt), _lib.ptr(pair_base), _lib.ptr(cache), c_int(cap_pairs),
        _lib.stream()), "hstu_bucket_cache")
    _lib.LAUNCHES["count"] += 1
    return cache, pair_base, cap_pairs, seq_offsets   # the offsets the blocks were made for stay alive with them

  hit = _remember("buckets", ts32, make, (T, max_seq_len, num_buckets, bool(causal)))
  same = hit[3] is seq_offsets or (hit[3].data_ptr() == seq_offsets.data_ptr() and hit[3]._version == seq_offsets._version)
  if not same:          # same timestamps tensor, other offsets: rebuild
    _memo.pop("buckets", None)
    hit = _remember("buckets", ts32, make, (T, max_seq_len, num_buckets, bool(causal)))
  return hit


def _ident(t):
  return None if t is None else (t.data_ptr(), t._version, tuple(t.shape))


# Free lists of the per-pair block buffers (hundreds of megabytes each): a context takes what it needs and gives
# it back when it dies, so a training loop keeps re-using the same two buffers while two contexts that are alive
# at the same time (say a causal and a full call whose backward passes come later) never share one.
_free: dict[tuple, list[torch.Tensor]] = {}


def _take(kind: str, numel: int, dtype, device, zero: bool = False) -> torch.Tensor:
  key = (kind, str(device), dtype)
  pool = _free.setdefault(key, [])
  for i, t in enumerate(pool):
    if t.numel() >= numel:
      pool.pop(i)
      if zero and getattr(t, "_recml_dirty", False):
        t.zero_()
        t._recml_dirty = False
      return t
  pool.clear()            # too small for what is needed now: let them go
  return (torch.zeros if zero else torch.empty)(numel, dtype=dtype, device=device)


def _give_back(kind: str, t: torch.Tensor) -> None:
  pool = _free.setdefault((kind, str(t.device), t.dtype), [])
  if len(pool) < 2:
    pool.append(t)


class BiasContext:
  """What every attention call of one training step shares: the bias tiles of the batch (built once, from the
  relative-position / time-bucket tables, the masks and the batch's lengths and timestamps) and the block
  buffer into which every backward call adds its score gradients.  The LAST backward call of the step (the
  count of forward calls that can reach a backward is kept here) turns that buffer into the gradients of the
  two tables and returns them; the earlier ones return none for the tables, which autograd treats as zero."""

  def __init__(self, seq_offsets, ts32, pos_w, ts_w, T, max_seq_len, causal, window, segment_ids):
    lib = _lib.cuda()
    dev = seq_offsets.device
    B = seq_offsets.numel() - 1
    self.seq_offsets, self.ts32, self.segment_ids = seq_offsets, ts32, segment_ids
    self.causal, self.window, self.max_seq_len, self.T = bool(causal), window, max_seq_len, T
    self.pos_w = None if pos_w is None else pos_w.detach().float().contiguous()
    self.ts_w = None if (ts_w is None or ts32 is None) else ts_w.detach().float().contiguous()
    self.num_buckets = self.ts_w.numel() - 1 if self.ts_w is not None else 0
    self.tiles_f = _tiles(seq_offsets, T)
    cap, self.max_nt, self.cap_pairs = _pair_capacity(T, B, max_seq_len, causal)
    if self.cap_pairs > MAX_PAIRS:
      raise MemoryError(f"{self.cap_pairs} tile pairs exceed the per-pair cache limit ({MAX_PAIRS})")
    self.bucket_cache = None
    if self.ts_w is not None:
      bc = _bucket_cache(seq_offsets, ts32, T, max_seq_len, self.num_buckets, causal)
      self.bucket_cache, self.pair_base = bc[0], bc[1]
    else:
      self.pair_base = torch.empty(B + 1, dtype=torch.int32, device=dev)
      _lib.check_rc(lib.recml_hstu_pair_base(_lib.ptr(seq_offsets), c_int(B), c_int(int(causal)),
                                             _lib.ptr(self.pair_base), _lib.stream()), "hstu_pair_base")
    self.tiles = _take("bias_tiles", self.cap_pairs * 16384, torch.bfloat16, dev)
    self.dbias = None
    self.pending = 0
    self.want_bias_grad = False
    _lib.check_rc(lib.recml_hstu_bias_tiles(ctypes.byref(self._params()), c_int(self.tiles_f[2]), c_int(self.max_nt),
                                            _lib.stream()), "hstu_bias_tiles")

  def _params(self, dpos=None, dts=None) -> _BiasParams:
    p = _BiasParams()
    p.seq_offsets, p.tile_seq, p.tile_row0 = self.seq_offsets.data_ptr(), self.tiles_f[0].data_ptr(), self.tiles_f[1].data_ptr()
    p.pair_base, p.causal, p.cap_pairs, p.max_seq_len = self.pair_base.data_ptr(), int(self.causal), self.cap_pairs, self.max_seq_len
    p.window = -1 if self.window is None else int(self.window)
    p.num_buckets = self.num_buckets
    p.segment_ids = None if self.segment_ids is None else self.segment_ids.data_ptr()
    p.pos_w = None if self.pos_w is None else self.pos_w.data_ptr()
    p.ts_w = None if self.ts_w is None else self.ts_w.data_ptr()
    p.bucket_cache = None if self.bucket_cache is None else self.bucket_cache.data_ptr()
    p.tiles = self.tiles.data_ptr()
    p.dbias = None if self.dbias is None else self.dbias.data_ptr()
    p.dpos_w = None if dpos is None else dpos.data_ptr()
    p.dts_w = None if dts is None else dts.data_ptr()
    p.status = _lib.status_buffer(self.seq_offsets.device).data_ptr()
    return p

  def gradient_blocks(self) -> torch.Tensor:
    """The fp32 block buffer the backward kernels reduce into (all zeros between steps: the gradient pass
    clears what it reads; a step that was abandoned half-way leaves it marked dirty and it is cleared here)."""
    if self.dbias is None:
      self.dbias = _take("bias_grads", self.cap_pairs * 16384, torch.float32, self.seq_offsets.device, zero=True)
      self.dbias._recml_dirty = True
    return self.dbias

  def __del__(self):
    try:
      if getattr(self, "tiles", None) is not None:
        _give_back("bias_tiles", self.tiles)
      if getattr(self, "dbias", None) is not None:
        _give_back("bias_grads", self.dbias)        # still marked dirty: cleared by whoever takes it next
    except Exception:  # pylint: disable=broad-except
      pass

  def table_gradients(self, pos_w, ts_w):
    dpos = torch.zeros_like(self.pos_w) if self.pos_w is not None else None
    dts = torch.zeros_like(self.ts_w) if self.ts_w is not None else None
    if self.dbias is not None and (dpos is not None or dts is not None):
      _lib.check_rc(_lib.cuda().recml_hstu_bias_grads(ctypes.byref(self._params(dpos, dts)), c_int(self.tiles_f[2]),
                                                      c_int(self.max_nt), _lib.stream()), "hstu_bias_grads")
      self.dbias._recml_dirty = False
      _give_back("bias_grads", self.dbias)
      self.dbias = None
    out_pos = None if (pos_w is None or dpos is None) else dpos.to(pos_w.dtype)
    out_ts = None if ts_w is None else (dts.to(ts_w.dtype) if dts is not None else torch.zeros_like(ts_w))
    return out_pos, out_ts


def bias_context(seq_offsets, timestamps, pos_w, ts_w, T, max_seq_len, causal, window=None, segment_ids=None) -> BiasContext:
  """The step's shared context: one per (batch, table values, mask description); every layer's call finds it."""
  ts32 = _ts32(timestamps)
  if segment_ids is not None and segment_ids.dtype != torch.int32:
    segment_ids = _remember("seg32", segment_ids, lambda: segment_ids.to(torch.int32).contiguous())
  extra = (T, max_seq_len, bool(causal), window, _ident(ts32), _ident(pos_w), _ident(ts_w), _ident(segment_ids))
  return _remember("bias_ctx", seq_offsets,
                   lambda: BiasContext(seq_offsets, ts32, pos_w, ts_w, T, max_seq_len, causal, window, segment_ids), extra)


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
  p.window = -1
  return p


def _attach(p: _Params, bc: BiasContext) -> None:
  p.pair_base, p.cap_pairs, p.bias_tiles = bc.pair_base.data_ptr(), bc.cap_pairs, bc.tiles.data_ptr()


def _set_dropout(p: _Params, dropout, mode: int = MODE_SILU_DROPOUT) -> None:
  """`dropout` = (rate, key): key is an int64 device tensor of one element that seeds the mask."""
  if dropout is None:
    return
  rate, key = dropout
  p.mode = mode
  p.dropout_key = key.data_ptr()
  p.drop_threshold = min(int(rate * 4294967296.0), 4294967295)
  p.keep_scale = 1.0 / (1.0 - rate)


def dropout_keep_mask(key: int, head: int, q_tokens: torch.Tensor, k_tokens: torch.Tensor, rate: float) -> torch.Tensor:
  """The kernels' keep / drop decision for (head, query token, key token), restated with integer tensor ops:
  boolean `[len(q_tokens), len(k_tokens)]`.  For tests and for callers that need the mask of a small case."""
  M = 0xFFFFFFFF

  def mix(x):
    x = x ^ (x >> 16)
    x = (x * 0x7feb352d) & M
    x = x ^ (x >> 15)
    x = (x * 0x846ca68b) & M
    return x ^ (x >> 16)

  key &= 0xFFFFFFFFFFFFFFFF
  lo, hi = key & M, key >> 32
  q = q_tokens.to(torch.int64)
  kk = k_tokens.to(torch.int64)
  row = mix((lo ^ ((q * 0x9E3779B1) & M) ^ (((head + 1) * 0x85EBCA6B) & M)) & M)
  x = mix((row[:, None] ^ (((kk * 0xC2B2AE35) & M) + hi)[None, :] & M) & M)
  return x >= min(int(rate * 4294967296.0), 4294967295)


def forward(q, k, v, seq_offsets, bc: BiasContext, max_seq_len, causal, scale, dropout=None):
  assert rows_ok(q) and rows_ok(k) and rows_ok(v)
  tiles = _tiles(seq_offsets, q.shape[0])
  out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
  p = _params(q, seq_offsets, None, None, None, max_seq_len, causal, scale, tiles, k, v)
  _attach(p, bc)
  _set_dropout(p, dropout)
  p.out = out.data_ptr()
  _lib.check_rc(_lib.cuda().recml_hstu_attn_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), ctypes.byref(p),
                                                c_int(tiles[2]), _lib.stream()), "hstu_attn_fwd")
  return out


def backward(do, q, k, v, seq_offsets, bc: BiasContext, max_seq_len, causal, scale, dq_fp32: bool = False,
             dropout=None):
  """Gradients w.r.t. q, k, v; the score gradients go into the context's block buffer when a bias table
  wants a gradient.  `dq_fp32` returns dq as the kernel accumulated it (fp32) for a caller that converts it
  in a pass of its own."""
  lib = _lib.cuda()
  tiles = _tiles(seq_offsets, q.shape[0], backward=True)
  do = as_rows(do)
  dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
  dk, dv = (torch.empty(k.shape, dtype=k.dtype, device=k.device) for _ in range(2))
  p = _params(q, seq_offsets, None, None, None, max_seq_len, causal, scale, tiles, k, v, do)
  _attach(p, bc)
  p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
  _set_dropout(p, dropout)
  if bc.want_bias_grad:
    p.dbias_tiles = bc.gradient_blocks().data_ptr()
  _lib.check_rc(lib.recml_hstu_attn_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(do),
                                        ctypes.byref(p), c_int(tiles[2]), _lib.stream()), "hstu_attn_bwd")
  return (dq if dq_fp32 else dq.to(q.dtype)), dk, dv


# ---- softmax mode: the same kernels with P = softmax(scale * QK^T) over the visible keys ----------------------


def softmax_forward(q, k, v, seq_offsets, max_seq_len, causal, scale, dropout=None):
  """Jagged softmax attention; returns (out `[T, H, Dh]` bf16, row log-sum-exp `[T, H]` fp32).  With
  `dropout` = (rate, key) the normalised weights are dropped and rescaled before they multiply the values;
  the log-sum-exp is that of all visible keys."""
  assert rows_ok(q) and rows_ok(k) and rows_ok(v)
  tiles = _tiles(seq_offsets, q.shape[0])
  out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
  lse = torch.empty(q.shape[0], q.shape[1], dtype=torch.float32, device=q.device)
  p = _params(q, seq_offsets, None, None, None, max_seq_len, causal, scale, tiles, k, v)
  p.out, p.mode, p.lse = out.data_ptr(), MODE_SOFTMAX, lse.data_ptr()
  _set_dropout(p, dropout, MODE_SOFTMAX_DROPOUT)
  _lib.check_rc(_lib.cuda().recml_hstu_attn_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), ctypes.byref(p),
                                                c_int(tiles[2]), _lib.stream()), "softmax_attn_fwd")
  return out, lse


def softmax_backward(do, out, lse, q, k, v, seq_offsets, max_seq_len, causal, scale, dropout=None):
  tiles = _tiles(seq_offsets, q.shape[0], backward=True)
  do = as_rows(do)
  delta = (do.float() * out.float()).sum(-1).contiguous()          # [T, H]
  dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
  dk, dv = (torch.empty(k.shape, dtype=k.dtype, device=k.device) for _ in range(2))
  p = _params(q, seq_offsets, None, None, None, max_seq_len, causal, scale, tiles, k, v, do)
  p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
  p.mode, p.lse, p.delta = MODE_SOFTMAX, lse.data_ptr(), delta.data_ptr()
  _set_dropout(p, dropout, MODE_SOFTMAX_DROPOUT)
  _lib.check_rc(_lib.cuda().recml_hstu_attn_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(do), ctypes.byref(p),
                                                c_int(tiles[2]), _lib.stream()), "softmax_attn_bwd")
  return dq.to(q.dtype), dk, dv


# ---- decay mode: the quadratic ("attention") form of a diagonal state-space recurrence -----------------------
#   y[l] = sum_{s <= l} (c_l . b_s) * exp(cum[l] - cum[s]) * x_s        cum = inclusive prefix sum of a <= 0
# c and b play the parts of q and k and are shared by all heads; x is v.
CUM_PAD = 128
LOG2E = 1.4426950408889634


def _decay_params(c, b, x, cum2, seq_offsets, max_seq_len, tiles, do=None):
  p = _params(x, seq_offsets, None, None, None, max_seq_len, True, 1.0, tiles, x, x, do)
  p.ld_q, p.ld_k = c.stride(0), b.stride(0)
  p.inv_n = 1.0
  p.mode, p.qk_shared, p.cum, p.cum_pitch = MODE_DECAY, 1, cum2.data_ptr(), cum2.stride(0)
  return p


def decay_forward(c, b, x, cum2, seq_offsets, max_seq_len):
  """c, b `[T, N]` bf16, x `[T, H, N]` bf16, cum2 `[H, >= T + 128]` fp32 (prefix sums times log2 e).  Returns
  y `[T, H, N]` bf16."""
  assert rows_ok(x) and c.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and c.stride(1) == 1 and b.stride(1) == 1
  assert c.shape[1] == x.shape[2] == b.shape[1] and cum2.stride(1) == 1 and cum2.shape[1] >= x.shape[0] + CUM_PAD
  tiles = _tiles(seq_offsets, x.shape[0])
  out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
  p = _decay_params(c, b, x, cum2, seq_offsets, max_seq_len, tiles)
  p.out = out.data_ptr()
  _lib.check_rc(_lib.cuda().recml_hstu_attn_fwd(_lib.ptr(c), _lib.ptr(b), _lib.ptr(x), ctypes.byref(p),
                                                c_int(tiles[2]), _lib.stream()), "decay_attn_fwd")
  return out


def decay_backward(do, c, b, x, cum2, seq_offsets, max_seq_len):
  """Returns (dc `[T, N]` fp32, db `[T, N]` fp32, dx `[T, H, N]` bf16, dcum `[H, pitch]` fp32 w.r.t. the natural-log
  prefix sums)."""
  tiles = _tiles(seq_offsets, x.shape[0], backward=True)
  do = as_rows(do)
  dc = torch.zeros(c.shape, dtype=torch.float32, device=c.device)
  db = torch.zeros(b.shape, dtype=torch.float32, device=b.device)
  dx = torch.empty(x.shape, dtype=x.dtype, device=x.device)
  dcum = torch.zeros(cum2.shape, dtype=torch.float32, device=x.device)
  p = _decay_params(c, b, x, cum2, seq_offsets, max_seq_len, tiles, do)
  p.dq, p.dk_acc, p.dv, p.dcum, p.v_rows = dc.data_ptr(), db.data_ptr(), dx.data_ptr(), dcum.data_ptr(), x.data_ptr()
  _lib.check_rc(_lib.cuda().recml_hstu_attn_bwd(_lib.ptr(c), _lib.ptr(b), _lib.ptr(x), _lib.ptr(do), ctypes.byref(p),
                                                c_int(tiles[2]), _lib.stream()), "decay_attn_bwd")
  return dc, db, dx, dcum
