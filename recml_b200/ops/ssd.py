"""State-space duality (SSD) scan of Mamba2 and the depthwise causal conv that precedes it.

  h_t = exp(a_t)·h_{t−1} + b_t ⊗ x_t ,   y_t = c_t · h_t          (per head; b, c shared in a group)

Computed chunk-wise like the reference (`recml/layers/keras/mamba.py:53-146`): inside a chunk the
output is a masked "attention" (C·Bᵀ ⊙ decay)·X, chunk end-states are carried by a short
sequential recurrence, and the carried state contributes C·state·decay.  `ssd_recurrent` is the
plain O(L) recurrence used as the oracle.  On CUDA the chunk kernels are `csrc/cuda/ssd.cu`.
"""
from __future__ import annotations

import ctypes

import torch


def ssd_recurrent(x, a, b, c, initial_state=None):
  """x `[B, L, H, P]`, a `[B, L, H]`, b / c `[B, L, G, N]` → y `[B, L, H, P]` (fp32 recurrence)."""
  B, L, H, P = x.shape
  G, N = b.shape[-2:]
  rep = H // G
  h = torch.zeros(B, H, P, N, dtype=torch.float32, device=x.device) if initial_state is None \
      else initial_state.float().clone()
  ys = []
  bf, cf = b.float().repeat_interleave(rep, dim=2), c.float().repeat_interleave(rep, dim=2)
  for t in range(L):
    h = h * torch.exp(a[:, t].float())[..., None, None] + x[:, t].float()[..., None] * bf[:, t][:, :, None, :]
    ys.append(torch.einsum("bhpn,bhn->bhp", h, cf[:, t]))
  return torch.stack(ys, dim=1).to(x.dtype)


def ssd_chunked(x, a, b, c, block_len: int, initial_states=None):
  """Same contract as the reference's `ssd_minimal_discrete` (L must be a multiple of block_len)."""
  B, L, H, P = x.shape
  G, N = b.shape[-2:]
  assert L % block_len == 0, "sequence length must be a multiple of the chunk size"
  assert G == 1 or G == H, "groups must be 1 or equal to heads"
  C = L // block_len
  xf = x.float().reshape(B, C, block_len, H, P)
  af = a.float().reshape(B, C, block_len, H).permute(0, 3, 1, 2)           # [B, H, C, l]
  bf = b.float().reshape(B, C, block_len, G, N).expand(B, C, block_len, H, N) if G == 1 else \
      b.float().reshape(B, C, block_len, H, N)
  cf = c.float().reshape(B, C, block_len, G, N).expand(B, C, block_len, H, N) if G == 1 else \
      c.float().reshape(B, C, block_len, H, N)
  cum = torch.cumsum(af, dim=-1)                                            # inclusive prefix of a
  # intra-chunk: decay[l, s] = exp(cum[l] − cum[s]) for s ≤ l
  diff = cum[..., :, None] - cum[..., None, :]
  tri = torch.tril(torch.ones(block_len, block_len, dtype=torch.bool, device=x.device))
  decay = torch.where(tri, torch.exp(diff.masked_fill(~tri, 0.0)), torch.zeros((), device=x.device))
  scores = torch.einsum("bclhn,bcshn->bhcls", cf, bf) * decay
  y_diag = torch.einsum("bhcls,bcshp->bclhp", scores, xf)
  # chunk end states
  to_end = torch.exp(cum[..., -1:] - cum)                                   # [B, H, C, l]
  states = torch.einsum("bclhn,bhcl,bclhp->bchpn", bf, to_end, xf)
  # carry across chunks (sequential over C, tiny)
  carry = torch.zeros(B, H, P, N, dtype=torch.float32, device=x.device) if initial_states is None \
      else initial_states.float().reshape(B, H, P, N)
  chunk_decay = torch.exp(cum[..., -1])                                     # [B, H, C]
  prev = []
  for ci in range(C):
    prev.append(carry)
    carry = carry * chunk_decay[:, :, ci][..., None, None] + states[:, ci]
  prev = torch.stack(prev, dim=1)                                           # state entering each chunk
  y_off = torch.einsum("bclhn,bchpn,bhcl->bclhp", cf, prev, torch.exp(cum))
  return (y_diag + y_off).reshape(B, L, H, P).to(x.dtype)


ssd_minimal_discrete = ssd_chunked        # the reference's name (`recml/layers/keras/mamba.py:53-146`)


def segsum(x):
  """`out[..., i, j] = x[..., j + 1] + ... + x[..., i]` for j <= i and -inf above the diagonal: the log of the
  decay between two positions (`recml/layers/keras/mamba.py:30-50`), here as a difference of prefix sums."""
  T = x.shape[-1]
  cum = torch.cumsum(x, dim=-1)
  tri = torch.tril(torch.ones(T, T, dtype=torch.bool, device=x.device))
  return (cum[..., :, None] - cum[..., None, :]).masked_fill(~tri, float("-inf"))


def causal_depthwise_conv1d_silu(x, weight, bias=None):
  """x `[B, L, C]`, weight `[C, K]` (tap k multiplies x[t − (K−1) + k]); SiLU fused."""
  K = weight.shape[1]
  xp = torch.nn.functional.pad(x.float().transpose(1, 2), (K - 1, 0))
  y = torch.nn.functional.conv1d(xp, weight.float()[:, None, :], None if bias is None else bias.float(),
                                 groups=weight.shape[0])
  return torch.nn.functional.silu(y).transpose(1, 2).to(x.dtype)


# ---- CUDA path (`csrc/cuda/ssd.cu`) -----------------------------------------------------------------------
class _ScanParams(ctypes.Structure):
  _fields_ = [("x", ctypes.c_void_p), ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("c", ctypes.c_void_p),
              ("init", ctypes.c_void_p), ("init_batch_stride", ctypes.c_longlong), ("y", ctypes.c_void_p),
              ("ckpt", ctypes.c_void_p), ("B", ctypes.c_int), ("L", ctypes.c_int), ("H", ctypes.c_int),
              ("P", ctypes.c_int), ("N", ctypes.c_int), ("n_ckpt", ctypes.c_int), ("dy", ctypes.c_void_p),
              ("dx", ctypes.c_void_p), ("da", ctypes.c_void_p), ("db", ctypes.c_void_p), ("dc", ctypes.c_void_p),
              ("dinit", ctypes.c_void_p)]


def _cuda_supported(x, b) -> bool:
  P, N = x.shape[-1], b.shape[-1]
  # the backward keeps 9 state matrices of a (batch, head) pair in shared memory
  return x.is_cuda and b.shape[-2] == 1 and P in (8, 16, 32, 64) and N in (16, 32, 64) and 9 * P * (N + 4) * 4 < 200_000


class _ScanFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, a, b, c, init):
    from recml_b200.ops import _lib
    lib = _lib.cuda()
    assert lib.recml_ssd_struct_size() == ctypes.sizeof(_ScanParams)
    B, L, H, P = x.shape
    N = b.shape[-1]
    xf, af = x.float().contiguous(), a.float().contiguous()
    bf, cf = b.float().reshape(B, L, N).contiguous(), c.float().reshape(B, L, N).contiguous()
    initf = None if init is None else init.float().contiguous()
    interval = lib.recml_ssd_ckpt_interval()
    n_ckpt = (L + interval - 1) // interval
    y = torch.empty_like(xf)
    ckpt = torch.empty(B, H, n_ckpt, P, N, dtype=torch.float32, device=x.device)
    p = _ScanParams()
    p.x, p.a, p.b, p.c = xf.data_ptr(), af.data_ptr(), bf.data_ptr(), cf.data_ptr()
    p.init = None if initf is None else initf.data_ptr()
    p.init_batch_stride = 0 if initf is None or initf.dim() == 3 else H * P * N
    p.y, p.ckpt = y.data_ptr(), ckpt.data_ptr()
    p.B, p.L, p.H, p.P, p.N, p.n_ckpt = B, L, H, P, N, n_ckpt
    _lib.check_rc(lib.recml_ssd_scan(ctypes.byref(p), ctypes.c_int(0), _lib.stream()), "ssd_scan_fwd")
    ctx.save_for_backward(xf, af, bf, cf, ckpt)
    ctx.meta = (x.dtype, a.dtype, b.dtype, c.dtype, b.shape, None if init is None else (init.dtype, init.dim()))
    return y.to(x.dtype)

  @staticmethod
  def backward(ctx, dy):
    from recml_b200.ops import _lib
    lib = _lib.cuda()
    xf, af, bf, cf, ckpt = ctx.saved_tensors
    xdt, adt, bdt, cdt, bshape, init_meta = ctx.meta
    B, L, H, P = xf.shape
    N = bf.shape[-1]
    dyf = dy.float().contiguous()
    dx, da = torch.empty_like(xf), torch.empty_like(af)
    db = torch.empty(B, L, H, N, dtype=torch.float32, device=xf.device)
    dc = torch.empty_like(db)
    dinit = torch.empty(B, H, P, N, dtype=torch.float32, device=xf.device) if init_meta is not None else None
    p = _ScanParams()
    p.x, p.a, p.b, p.c = xf.data_ptr(), af.data_ptr(), bf.data_ptr(), cf.data_ptr()
    p.ckpt = ckpt.data_ptr()
    p.B, p.L, p.H, p.P, p.N, p.n_ckpt = B, L, H, P, N, ckpt.shape[2]
    p.dy, p.dx, p.da, p.db, p.dc = dyf.data_ptr(), dx.data_ptr(), da.data_ptr(), db.data_ptr(), dc.data_ptr()
    p.dinit = None if dinit is None else dinit.data_ptr()
    _lib.check_rc(lib.recml_ssd_scan(ctypes.byref(p), ctypes.c_int(1), _lib.stream()), "ssd_scan_bwd")
    gi = None
    if dinit is not None:
      gi = (dinit.sum(0) if init_meta[1] == 3 else dinit).to(init_meta[0])
    return (dx.to(xdt), da.to(adt), db.sum(2).reshape(bshape).to(bdt), dc.sum(2).reshape(bshape).to(cdt), gi)


# ---- tensor-core path: the quadratic form on the attention kernels' decay mode ------------------------------
QUAD_MAX_LEN = 1024      # beyond this the O(L^2) form costs more than the recurrence


def _quad_supported(x, b) -> bool:
  from recml_b200.ops import hstu_cuda
  P, N = x.shape[-1], b.shape[-1]
  return (x.is_cuda and b.shape[-2] == 1 and P == N and P in (64, 128) and x.shape[1] <= QUAD_MAX_LEN and
          hstu_cuda.available())


_dense_offsets: dict = {}


def _offsets_for(B: int, L: int, device) -> torch.Tensor:
  key = (B, L, str(device))
  if key not in _dense_offsets:
    if len(_dense_offsets) > 16:
      _dense_offsets.clear()
    _dense_offsets[key] = (torch.arange(B + 1, device=device, dtype=torch.int32) * L).contiguous()
  return _dense_offsets[key]


class _QuadFn(torch.autograd.Function):
  """y[l] = sum_{s <= l} (c_l . b_s) exp(cum[l] - cum[s]) x_s over each sequence: scores, decay mask and the
  product with x run on the tensor cores (`csrc/cuda/hstu_attention.cu`, decay mode), the chunk-wise
  formulation of the reference (`recml/layers/keras/mamba.py:53-146`) with the whole sequence as one chunk."""

  @staticmethod
  def forward(ctx, x, a, b, c):
    from recml_b200.ops import hstu_cuda
    B, L, H, P = x.shape
    T = B * L
    offs = _offsets_for(B, L, x.device)
    cum = torch.cumsum(a.float(), dim=1)                                     # [B, L, H]
    cum2 = torch.empty(H, T + hstu_cuda.CUM_PAD, dtype=torch.float32, device=x.device)
    cum2[:, T:].zero_()
    torch.mul(cum.permute(2, 0, 1).reshape(H, T), hstu_cuda.LOG2E, out=cum2[:, :T])
    xb = x.reshape(T, H, P).to(torch.bfloat16).contiguous()
    bb = b.reshape(T, P).to(torch.bfloat16).contiguous()
    cb = c.reshape(T, P).to(torch.bfloat16).contiguous()
    y = hstu_cuda.decay_forward(cb, bb, xb, cum2, offs, L)
    ctx.save_for_backward(xb, bb, cb, cum2, offs)
    ctx.meta = (x.dtype, a.dtype, b.dtype, c.dtype, tuple(x.shape), tuple(b.shape))
    return y.reshape(B, L, H, P).to(x.dtype)

  @staticmethod
  def backward(ctx, dy):
    from recml_b200.ops import hstu_cuda
    xb, bb, cb, cum2, offs = ctx.saved_tensors
    xdt, adt, bdt, cdt, xshape, bshape = ctx.meta
    B, L, H, P = xshape
    T = B * L
    do = dy.reshape(T, H, P).to(torch.bfloat16)
    dc, db, dx, dcum = hstu_cuda.decay_backward(do, cb, bb, xb, cum2, offs, L)
    # cum[l] = sum_{t <= l} a[t]  =>  da[t] = sum_{l >= t} dcum[l]
    g = dcum[:, :T].reshape(H, B, L)
    da = (g.sum(-1, keepdim=True) - torch.cumsum(g, dim=-1) + g).permute(1, 2, 0)
    return (dx.reshape(xshape).to(xdt), da.to(adt), db.reshape(bshape).to(bdt), dc.reshape(bshape).to(cdt))


def _initial_state_term(a, c, initial_states):
  """Contribution of the state the sequence starts from: y_off[l] = exp(cum[l]) * (h0 c_l)."""
  B, L, H = a.shape
  cum = torch.cumsum(a.float(), dim=1)
  h0 = initial_states.float()
  cf = c.float().reshape(B, L, -1)
  if h0.dim() == 3:
    proj = torch.einsum("bln,hpn->blhp", cf, h0)
  else:
    proj = torch.einsum("bln,bhpn->blhp", cf, h0)
  return proj * torch.exp(cum)[..., None]


def ssd_scan(x, a, b, c, block_len: int = 64, initial_states=None):
  """The SSD recurrence over the whole sequence: x `[B, L, H, P]`, a `[B, L, H]`, b / c `[B, L, G, N]`,
  initial state `[H, P, N]` or `[B, H, P, N]`.  On CUDA with one group and P == N in {64, 128} this is the
  tensor-core quadratic form (bf16 operands, fp32 accumulation); other CUDA shapes with one group take the
  register-resident scan kernel (fp32); elsewhere the chunked formulation with zero padding to a multiple of
  `block_len`."""
  if _quad_supported(x, b):
    y = _QuadFn.apply(x, a, b, c)
    if initial_states is not None:
      y = y + _initial_state_term(a, c, initial_states).to(y.dtype)
    return y
  if _cuda_supported(x, b):
    return _ScanFn.apply(x, a, b, c, initial_states)
  L = x.shape[1]
  pad = (-L) % block_len
  if pad:
    f = torch.nn.functional.pad
    x, a = f(x, (0, 0, 0, 0, 0, pad)), f(a, (0, 0, 0, pad))
    b, c = f(b, (0, 0, 0, 0, 0, pad)), f(c, (0, 0, 0, 0, 0, pad))
  init = initial_states
  if init is not None and init.dim() == 3:
    init = init[None].expand(x.shape[0], -1, -1, -1)
  return ssd_chunked(x, a, b, c, block_len, init)[:, :L]


def ssd_scan_recurrent_kernel(x, a, b, c, initial_states=None):
  """The fp32 scan kernel regardless of shape preferences (tests and precision comparisons)."""
  assert _cuda_supported(x, b)
  return _ScanFn.apply(x, a, b, c, initial_states)


class _ConvFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, weight, bias):
    from recml_b200.ops import _lib
    lib = _lib.cuda()
    B, L, C = x.shape
    xf, wf = x.float().contiguous(), weight.float().contiguous()
    bf = None if bias is None else bias.float().contiguous()
    y = torch.empty_like(xf)
    _lib.check_rc(lib.recml_conv1d_silu_fwd(_lib.ptr(xf), _lib.ptr(wf), None if bf is None else _lib.ptr(bf), _lib.ptr(y),
                                            ctypes.c_int(B), ctypes.c_int(L), ctypes.c_int(C),
                                            ctypes.c_int(weight.shape[1]), _lib.stream()), "conv1d_silu_fwd")
    ctx.save_for_backward(xf, wf, bf if bf is not None else torch.empty(0, device=x.device))
    ctx.meta = (x.dtype, weight.dtype, None if bias is None else bias.dtype)
    return y.to(x.dtype)

  @staticmethod
  def backward(ctx, dy):
    from recml_b200.ops import _lib
    lib = _lib.cuda()
    xf, wf, bf = ctx.saved_tensors
    xdt, wdt, bdt = ctx.meta
    B, L, C = xf.shape
    dyf = dy.float().contiguous()
    dx, du, dw = torch.empty_like(xf), torch.empty_like(xf), torch.empty_like(wf)
    dbias = torch.empty(C, dtype=torch.float32, device=xf.device) if bdt is not None else None
    _lib.check_rc(lib.recml_conv1d_silu_bwd(
        _lib.ptr(xf), _lib.ptr(wf), _lib.ptr(bf) if bdt is not None else None, _lib.ptr(dyf), _lib.ptr(dx), _lib.ptr(du),
        _lib.ptr(dw), None if dbias is None else _lib.ptr(dbias), ctypes.c_int(B), ctypes.c_int(L), ctypes.c_int(C),
        ctypes.c_int(wf.shape[1]), _lib.stream()), "conv1d_silu_bwd")
    return dx.to(xdt), dw.to(wdt), None if dbias is None else dbias.to(bdt)


def conv1d_silu(x, weight, bias=None):
  """Depthwise causal conv + SiLU: the CUDA kernels for 2..4 taps on a GPU, the torch formulation elsewhere."""
  if x.is_cuda and 2 <= weight.shape[1] <= 4:
    return _ConvFn.apply(x, weight, bias)
  return causal_depthwise_conv1d_silu(x, weight, bias)
