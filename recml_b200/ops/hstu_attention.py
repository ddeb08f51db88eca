"""HSTU pointwise (SiLU) attention.

  O = mask( silu(Q·Kᵀ·scale + bias) / n ) · V

Dense form `[B, L, H, Dh]` with an explicit `[B, L, L]` mask / bias is what the reference's model
computes (`recml/layers/keras/hstu.py:356-390`); the reference also ships a block-sparse TPU kernel
for the same math with causal / full / sliding-window masks and segment ids
(`recml/core/ops/hstu_ops.py:196-270,829-1046`; dense oracle in `hstu_ops_test.py:45-58`).  The
B200 path is JAGGED: sequences are packed back to back (`seq_offsets`), cost follows Σ Lᵢ² instead
of B·L², and the learned relative-position / time-bucket bias (`hstu.py:91-113,190-237`) is
computed inside the kernel from `pos_w[2N-1]`, `ts_w[buckets+1]` and the timestamps.  Its
normaliser is the configured `max_seq_len` (the reference divides by the padded length).
"""
from __future__ import annotations

import enum
import math

import torch

BUCKET_SIZE = 0.301


class MaskType(enum.Enum):
  CAUSAL = "causal"
  FULL = "full"


def time_buckets(delta: torch.Tensor, num_buckets: int) -> torch.Tensor:
  """clip(int(log(clip(|Δt|, 1, 1e9)) / 0.301), 0, num_buckets)."""
  v = delta.abs().clamp(min=1, max=int(1e9)).to(torch.float32)
  return torch.clamp((torch.log(v) / BUCKET_SIZE).to(torch.int64), 0, num_buckets)


def relative_bias_dense(L: int, pos_w: torch.Tensor | None, ts_w: torch.Tensor | None,
                        timestamps: torch.Tensor | None) -> torch.Tensor | None:
  """`[B or 1, L, L]` bias: pos_w[(j − i) + N − 1] + ts_w[bucket(t_ext[i+1] − t[j])] where
  t_ext appends the last timestamp once more."""
  bias = None
  if pos_w is not None:
    n = (pos_w.numel() + 1) // 2
    i = torch.arange(L, device=pos_w.device)
    bias = pos_w[(i[None, :] - i[:, None]) + n - 1][None]
  if ts_w is not None and timestamps is not None:
    ext = torch.cat([timestamps, timestamps[:, -1:]], dim=1)
    delta = ext[:, 1:, None] - ext[:, None, :-1]
    tb = ts_w[time_buckets(delta, ts_w.numel() - 1)]
    bias = tb if bias is None else bias + tb
  return bias


def pointwise_attention_dense(q, k, v, attention_mask=None, attention_bias=None, *, scaled: bool = False,
                              normalizer: float | None = None, dropout_p: float = 0.0, training: bool = False):
  """q, k, v `[B, L, H, Dh]`; mask / bias `[B, L, L]` (bias broadcast over heads)."""
  L = q.shape[1]
  qf = q.float() / math.sqrt(q.shape[-1]) if scaled else q.float()
  s = torch.einsum("bthd,bshd->bhts", qf, k.float())
  if attention_bias is not None:
    s = s + attention_bias[:, None].float()
  p = torch.nn.functional.silu(s)
  if not scaled:
    p = p / (normalizer if normalizer is not None else L)
  if attention_mask is not None:
    p = torch.where(attention_mask[:, None].bool(), p, torch.zeros_like(p))
  if training and dropout_p > 0:
    p = torch.nn.functional.dropout(p, dropout_p)
  return torch.einsum("bhts,bshd->bthd", p, v.float()).to(q.dtype)


def attention_mask(mask_type: MaskType | str, Lq: int, Lk: int, *, sliding_window_size: int | None = None,
                   q_offset: int = 0, device=None) -> torch.Tensor:
  """`[Lq, Lk]` bool mask of the reference op: causal (key j visible to query i when j <= i) or full,
  intersected with a window that is INCLUSIVE on both sides, i - w <= j <= i + w (the reference builds it
  as `LocalMask(window_size=(w, w), offset=0)`, `recml/core/ops/hstu_ops.py:940-945`), so a causal window
  of size w sees w + 1 keys.  `q_offset` is the position of query row 0 (queries sharded along the sequence)."""
  mask_type = MaskType(mask_type)
  i = torch.arange(Lq, device=device)[:, None] + q_offset
  j = torch.arange(Lk, device=device)[None, :]
  m = (j <= i) if mask_type is MaskType.CAUSAL else torch.ones(Lq, Lk, dtype=torch.bool, device=device)
  if sliding_window_size is not None:
    m = m & (j >= i - sliding_window_size) & (j <= i + sliding_window_size)
  return m


def pointwise_attention(mask_type: MaskType | str, q, k, v, *, q_segment_ids=None, kv_segment_ids=None,
                        sliding_window_size: int | None = None, scale: float | None = None, q_offset: int = 0,
                        normalizer: float | None = None):
  """API of the reference op on `[B, L, H, Dh]`: P = mask(silu(Q·Kᵀ·scale) / L_q); masks combine
  causal / full, a sliding window (inclusive: query i sees keys i−w..i+w) and equal segment ids.
  `q_offset` / `normalizer` serve the sequence-sharded mode, where a rank holds a slice of the queries."""
  B, Lq, H, Dh = q.shape
  Lk = k.shape[1]
  m = attention_mask(mask_type, Lq, Lk, sliding_window_size=sliding_window_size, q_offset=q_offset, device=q.device)
  m = m[None].expand(B, Lq, Lk)
  if q_segment_ids is not None:
    kv_seg = q_segment_ids if kv_segment_ids is None else kv_segment_ids
    m = m & (q_segment_ids[:, :, None] == kv_seg[:, None, :])
  s = torch.einsum("bthd,bshd->bhts", q.float(), k.float()) * (scale if scale is not None else 1.0)
  p = torch.nn.functional.silu(s) / (normalizer if normalizer is not None else Lq)
  p = torch.where(m[:, None], p, torch.zeros_like(p))
  return torch.einsum("bhts,bshd->bthd", p, v.float()).to(q.dtype)


class _AllGatherSeq(torch.autograd.Function):
  """Concatenates the ranks' `[B, L/W, ...]` slices along dim 1; backward sums the gradients of every
  rank's copy and keeps the own slice (a reduce-scatter)."""

  @staticmethod
  def forward(ctx, x, group):
    import torch.distributed as dist
    ctx.group = group
    n = dist.get_world_size(group)
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=1)

  @staticmethod
  def backward(ctx, g):
    import torch.distributed as dist
    n, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
    g = g.contiguous()
    dist.all_reduce(g, group=ctx.group)
    return g.chunk(n, dim=1)[r].contiguous(), None


def q_sharded_pointwise_attention(mask_type: MaskType | str, q, k, v, *, group=None, segment_ids=None,
                                  sliding_window_size: int | None = None, scale: float | None = None):
  """The reference op's `q_seq_shards` mode (`recml/core/ops/hstu_ops.py:847-848,1018-1040`): every rank of
  `group` holds a contiguous slice of the SEQUENCE (`[B, L / W, H, Dh]` of q, k, v and `[B, L / W]` segment
  ids).  Keys and values are all-gathered (their gradients reduce-scattered in backward), the queries stay
  where they are, and each rank computes its rows of the output with the mask shifted to its position;
  the normaliser is the full length, so the concatenation of the ranks' outputs equals the unsharded op."""
  import torch.distributed as dist
  if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
    return pointwise_attention(mask_type, q, k, v, q_segment_ids=segment_ids,
                               sliding_window_size=sliding_window_size, scale=scale)
  n, r = dist.get_world_size(group), dist.get_rank(group)
  Lq = q.shape[1]
  k_all, v_all = _AllGatherSeq.apply(k, group), _AllGatherSeq.apply(v, group)
  kv_seg = None
  if segment_ids is not None:
    parts = [torch.empty_like(segment_ids) for _ in range(n)]
    dist.all_gather(parts, segment_ids.contiguous(), group=group)
    kv_seg = torch.cat(parts, dim=1)
  return pointwise_attention(mask_type, q, k_all, v_all, q_segment_ids=segment_ids, kv_segment_ids=kv_seg,
                             sliding_window_size=sliding_window_size, scale=scale, q_offset=r * Lq,
                             normalizer=float(Lq * n))


def jagged_attention_reference(q, k, v, seq_offsets, max_seq_len: int, *, pos_w=None, ts_w=None,
                               timestamps=None, causal: bool = True, scale: float = 1.0,
                               sliding_window_size: int | None = None, segment_ids=None, dropout_p: float = 0.0,
                               dropout_key: int | None = None):
  """fp32 torch oracle for the packed kernel: q, k, v `[T, H, Dh]`, `seq_offsets [B+1]`.  With `dropout_key`
  the attention weights are dropped with the kernels' own mask (`hstu_cuda.dropout_keep_mask`); with a rate and
  no key, by `torch.nn.functional.dropout`."""
  out = torch.zeros_like(q, dtype=torch.float32)
  offs = seq_offsets.tolist()
  for b in range(len(offs) - 1):
    a, e = offs[b], offs[b + 1]
    L = e - a
    if L == 0:
      continue
    ts = None if timestamps is None else timestamps[a:e][None]
    bias = relative_bias_dense(L, pos_w, ts_w, ts)
    s = torch.einsum("thd,shd->hts", q[a:e].float(), k[a:e].float()) * scale
    if bias is not None:
      s = s + bias.float()
    p = torch.nn.functional.silu(s) / max_seq_len
    m = attention_mask("causal" if causal else "full", L, L, sliding_window_size=sliding_window_size, device=q.device)
    if segment_ids is not None:
      m = m & (segment_ids[a:e, None] == segment_ids[None, a:e])
    p = torch.where(m[None], p, torch.zeros_like(p))
    if dropout_p > 0 and dropout_key is not None:
      from recml_b200.ops import hstu_cuda
      tok = torch.arange(a, e, device=q.device)
      keep = torch.stack([hstu_cuda.dropout_keep_mask(dropout_key, h, tok, tok, dropout_p) for h in range(q.shape[1])])
      p = torch.where(keep, p / (1.0 - dropout_p), torch.zeros_like(p))
    elif dropout_p > 0:
      p = torch.nn.functional.dropout(p, dropout_p)
    out[a:e] = torch.einsum("hts,shd->thd", p, v[a:e].float())
  return out.to(q.dtype)


LAST_DROPOUT_KEY: torch.Tensor | None = None     # key of the most recent dropout mask (tests read it back)


def _draw_dropout(rate: float, device):
  """(rate, key) for the kernels, or None: the key is one random int64 drawn on the device (no host sync; under
  CUDA-graph capture it comes from the generator's captured state like any other random op)."""
  global LAST_DROPOUT_KEY
  if not rate or rate <= 0.0:
    return None
  if rate >= 1.0:
    raise ValueError("attention dropout rate must be below 1")
  key = torch.empty(1, dtype=torch.int64, device=device).random_()
  LAST_DROPOUT_KEY = key
  return (float(rate), key)


class _JaggedAttnFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, q, k, v, pos_w, ts_w, seq_offsets, timestamps, max_seq_len, causal, scale, window, segment_ids,
              dropout_p=0.0):
    from recml_b200.ops import hstu_cuda
    bc = hstu_cuda.bias_context(seq_offsets, timestamps, pos_w, ts_w, q.shape[0], max_seq_len, causal, window,
                                segment_ids)
    drop = _draw_dropout(dropout_p, q.device)
    o = hstu_cuda.forward(q, k, v, seq_offsets, bc, max_seq_len, causal, scale, dropout=drop)
    ctx.save_for_backward(q, k, v, pos_w, ts_w, seq_offsets)
    ctx.meta = (max_seq_len, causal, scale)
    ctx.drop = drop
    ctx.bias_ctx = bc
    if any(ctx.needs_input_grad):       # this call may see a backward: the step's last one finishes the bias tables
      bc.pending += 1
      bc.want_bias_grad = bc.want_bias_grad or ctx.needs_input_grad[3] or ctx.needs_input_grad[4]
    return o

  @staticmethod
  def backward(ctx, do):
    from recml_b200.ops import hstu_cuda
    q, k, v, pos_w, ts_w, seq_offsets = ctx.saved_tensors
    max_seq_len, causal, scale = ctx.meta
    bc = ctx.bias_ctx
    dq, dk, dv = hstu_cuda.backward(do, q, k, v, seq_offsets, bc, max_seq_len, causal, scale, dropout=ctx.drop)
    bc.pending -= 1
    dpos = dts = None
    if bc.pending <= 0 and bc.want_bias_grad:
      dpos, dts = bc.table_gradients(pos_w, ts_w)
      bc.want_bias_grad = False
    return dq, dk, dv, dpos, dts, None, None, None, None, None, None, None, None


class _SiluSplitAttnFn(torch.autograd.Function):
  """(u, attention(q, k, v)) with u | q | k | v = silu(z) for the pre-activation `z [T, 4 H Dh]` of a block's
  fused projection.  One pass computes the activation; the backward takes dq from the attention kernels as the
  fp32 they accumulate and forms dz = (du | dq | dk | dv) * silu'(z) in one pass (no cast, no concatenation, no
  separate activation backward)."""

  @staticmethod
  def forward(ctx, z, num_heads, pos_w, ts_w, seq_offsets, timestamps, max_seq_len, causal, scale, window, segment_ids,
              dropout_p=0.0):
    from recml_b200.ops import elementwise as ew, hstu_cuda
    T, W4 = z.shape
    D = W4 // 4
    u2, qkv = ew.silu_split(z)
    u = u2.view(T, num_heads, D // num_heads)
    q, k, v = qkv.view(T, 3, num_heads, D // num_heads).unbind(1)
    bc = hstu_cuda.bias_context(seq_offsets, timestamps, pos_w, ts_w, T, max_seq_len, causal, window, segment_ids)
    drop = _draw_dropout(dropout_p, z.device)
    o = hstu_cuda.forward(q, k, v, seq_offsets, bc, max_seq_len, causal, scale, dropout=drop)
    ctx.save_for_backward(z, qkv, pos_w, ts_w, seq_offsets)
    ctx.meta = (max_seq_len, causal, scale, num_heads)
    ctx.drop = drop
    ctx.bias_ctx = bc
    bc.pending += 1
    bc.want_bias_grad = bc.want_bias_grad or ctx.needs_input_grad[2] or ctx.needs_input_grad[3]
    return u, o

  @staticmethod
  def backward(ctx, du, do):
    from recml_b200.ops import elementwise as ew, hstu_cuda
    z, qkv, pos_w, ts_w, seq_offsets = ctx.saved_tensors
    max_seq_len, causal, scale, num_heads = ctx.meta
    bc = ctx.bias_ctx
    T, D = z.shape[0], z.shape[1] // 4
    q, k, v = qkv.view(T, 3, num_heads, D // num_heads).unbind(1)
    dq, dk, dv = hstu_cuda.backward(do, q, k, v, seq_offsets, bc, max_seq_len, causal, scale, dq_fp32=True,
                                    dropout=ctx.drop)
    bc.pending -= 1
    dpos = dts = None
    if bc.pending <= 0 and bc.want_bias_grad:
      dpos, dts = bc.table_gradients(pos_w, ts_w)
      bc.want_bias_grad = False
    g0 = du.reshape(T, D)
    if g0.dtype != torch.bfloat16 or g0.stride(1) != 1 or g0.stride(0) % 8:
      g0 = g0.to(torch.bfloat16).contiguous()
    dz = ew.silu_bwd_gather4(z, g0, dq.view(T, D), dk.view(T, D), dv.view(T, D))
    return dz, None, dpos, dts, None, None, None, None, None, None, None, None


def silu_split_attention(z, num_heads: int, seq_offsets, max_seq_len: int, *, pos_w=None, ts_w=None, timestamps=None,
                         causal: bool = True, scale: float = 1.0, sliding_window_size: int | None = None,
                         segment_ids=None, dropout_p: float = 0.0):
  """`z [T, 4 D]` bf16, contiguous: the pre-activation of an HSTU block's u | q | k | v projection.  Returns
  (u `[T, H, Dh]`, attention output `[T, H, Dh]`); CUDA only (callers check `fused_block_ok`)."""
  from recml_b200.ops import hstu_cuda
  return _SiluSplitAttnFn.apply(z, num_heads, pos_w, ts_w, hstu_cuda.offsets32(seq_offsets), timestamps, max_seq_len,
                                causal, scale, sliding_window_size, segment_ids, dropout_p)


def fused_block_ok(z: torch.Tensor, head_dim: int) -> bool:
  if not (z.is_cuda and z.dtype == torch.bfloat16 and z.is_contiguous() and head_dim in (64, 128)):
    return False
  from recml_b200.ops import hstu_cuda
  return hstu_cuda.available()


def jagged_pointwise_attention(q, k, v, seq_offsets, max_seq_len: int, *, pos_w=None, ts_w=None,
                               timestamps=None, causal: bool = True, scale: float = 1.0,
                               sliding_window_size: int | None = None, segment_ids=None, dropout_p: float = 0.0):
  """Packed HSTU attention.  CUDA bf16 inputs with head dim 64 or 128 run the sm_100a kernels (masks —
  causal, sequence ends, an inclusive sliding window, equal segment ids `[T]` — and the learned bias all
  arrive through the step's bias tiles); everything else takes the torch oracle (differentiable through
  autograd)."""
  if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128):
    from recml_b200.ops import hstu_cuda
    if hstu_cuda.available():
      return _JaggedAttnFn.apply(hstu_cuda.as_rows(q), hstu_cuda.as_rows(k), hstu_cuda.as_rows(v), pos_w, ts_w,
                                 hstu_cuda.offsets32(seq_offsets), timestamps, max_seq_len, causal, scale,
                                 sliding_window_size, segment_ids, dropout_p)
  return jagged_attention_reference(q, k, v, seq_offsets, max_seq_len, pos_w=pos_w, ts_w=ts_w,
                                    timestamps=timestamps, causal=causal, scale=scale,
                                    sliding_window_size=sliding_window_size, segment_ids=segment_ids,
                                    dropout_p=dropout_p)
