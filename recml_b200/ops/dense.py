"""Dense building blocks on the tcgen05 GEMM: MLP stacks and DCNv2 cross networks as single
autograd nodes, so activations stay bf16, ReLU masks are fused into the data-gradient GEMM
epilogues and no transposes are materialised (weight / data gradients use the MN-major operand
modes of the kernel).  CPU tensors take an fp32 torch path with identical semantics.

Reference math: MLP `Dense → ReLU` stacks and `xl ← x0 ⊙ ((xl·U)·V + b) + xl`
(`recml/examples/dlrm_experiment.py:136-177`).
"""
from __future__ import annotations

import torch

from recml_b200.ops import elementwise as ew
from recml_b200.ops import gemm as G
from recml_b200.utils import streams

# ---- deferred weight gradients ------------------------------------------------------------------------
# A backward pass is a chain of data-gradient GEMMs (each needs the previous one) with a weight-gradient
# GEMM hanging off every link.  Only the chain is on the critical path: what consumes its end (the
# embedding backward, which is bound by memory latency, not by the tensor cores) can start as soon as
# the chain is done if the weight gradients are computed afterwards, beside it, on another stream.
# Nodes created with deferral therefore queue their weight-gradient work instead of running it;
# `flush_deferred()` runs the queue on the "wgrad" side stream (ordered after everything issued so far
# on the current stream), stores the results in `.grad` and fires the parameters' post-accumulate hooks
# (the bucketed gradient all-reduce); `State.update` flushes what is left and joins the stream before
# the optimizer step.  Such a node receives DETACHED views of its parameters and delivers every one of
# their gradients itself: autograd runs a parameter's accumulation node (and its hooks) even when
# backward() returns no gradient for it, which would announce a gradient that does not exist yet.
_pending: list = []


def _deliver(p: torch.Tensor, g: torch.Tensor) -> None:
  """What autograd's AccumulateGrad node does for a gradient returned by backward()."""
  if g.shape != p.shape:
    g = g.reshape(p.shape)
  if g.dtype != p.dtype:
    g = g.to(p.dtype)
  if p.grad is None:
    p.grad = g
  else:
    p.grad.add_(g)
  hooks = getattr(p, "_post_accumulate_grad_hooks", None)
  if hooks:
    for h in list(hooks.values()):
      h(p)


def flush_deferred() -> None:
  """Runs the queued weight-gradient work on the "wgrad" side stream."""
  if not _pending:
    return
  work = list(_pending)
  _pending.clear()
  s = streams.fork("wgrad", priority=-1)
  with torch.cuda.stream(s):
    for tensors, fn in work:
      streams.keep_alive_on(s, *tensors)
      fn()


def join_deferred() -> None:
  """Flushes the queue and makes the current stream wait for the weight gradients."""
  flush_deferred()
  streams.join("wgrad")



def bf16_weight(p: torch.Tensor) -> torch.Tensor:
  """bf16 compute copy of an fp32 parameter, refreshed when the parameter changed.  The fused
  optimizer writes this copy itself and stamps the version, so steady-state steps never cast."""
  if p.dtype == torch.bfloat16:
    return p.detach()
  cp = getattr(p, "_recml_bf16", None)
  if cp is None or cp.shape != p.shape or cp.device != p.device:
    cp = torch.empty_like(p, dtype=torch.bfloat16)
    p._recml_bf16 = cp
    p._recml_bf16_version = -1
  if getattr(p, "_recml_bf16_version", -1) != p._version:
    ew.cast_bf16(p.detach(), out=cp)
    p._recml_bf16_version = p._version
  return cp


def _as_bf16_rows(x: torch.Tensor, k_pad: int) -> torch.Tensor:
  """Input matrix as bf16 with a 16-byte row pitch (zero-padded columns)."""
  if x.dtype == torch.bfloat16 and x.stride(-1) == 1 and x.stride(0) % 8 == 0 and x.shape[1] == k_pad:
    return x
  if x.dtype == torch.float32:
    return ew.cast_pad_rows(x, k_pad)
  out = torch.zeros(x.shape[0], k_pad, dtype=torch.bfloat16, device=x.device)
  out[:, :x.shape[1]] = x
  return out


class MLPFn(torch.autograd.Function):
  """y = MLP(x).  `relu_flags[i]` says whether layer i is followed by ReLU.  A last layer with one
  output unit runs as a fused GEMV and returns fp32 `[M]`... as `[M, 1]`."""

  @staticmethod
  def forward(ctx, x, relu_flags, out, targets, *params):
    n = len(relu_flags)
    # targets = (weights, biases): the real parameters when `params` are detached stand-ins (deferral)
    ctx.defer, ctx.targets = targets is not None, targets
    weights, biases = params[:n], params[n:]
    k0 = weights[0].shape[1]
    k_pad = (k0 + 7) // 8 * 8
    h = _as_bf16_rows(x.detach(), k_pad)
    acts, w16s = [h], []
    for i, (w, b) in enumerate(zip(weights, biases)):
      if w.shape[0] == 1 and i == n - 1:
        w16s.append(None)
        y = ew.gemv_fwd(h, w.detach().reshape(-1), None if b is None else b.detach())
        if relu_flags[i]:
          y = torch.relu(y)
        h = y[:, None]
      else:
        # the bf16 compute copy hangs on the real parameter (the optimizer refreshes it there)
        w16 = bf16_weight(targets[0][i] if targets is not None else w)
        if w16.shape[1] != h.shape[1]:   # first layer: pad K to the input's padded width
          wp = torch.zeros(w16.shape[0], h.shape[1], dtype=torch.bfloat16, device=w16.device)
          wp[:, :w16.shape[1]] = w16
          w16 = wp
        w16s.append(w16)
        h = G.gemm(h, w16, bias=None if b is None else b.detach(), relu=bool(relu_flags[i]),
                   out=out if i == n - 1 else None)
      acts.append(h)
    ctx.relu_flags, ctx.acts, ctx.w16s = relu_flags, acts, w16s
    ctx.weights, ctx.biases = weights, biases
    ctx.x_shape, ctx.x_dtype, ctx.need_dx = x.shape, x.dtype, x.requires_grad
    return h

  @staticmethod
  def backward(ctx, dy):
    relu, acts, w16s = ctx.relu_flags, ctx.acts, ctx.w16s
    weights, biases = ctx.weights, ctx.biases
    n = len(relu)
    dws, dbs = [None] * n, [None] * n
    g = dy
    defer = ctx.defer
    tw, tb = ctx.targets if defer else (weights, biases)

    def wgrad(i, g, x_i):
      """Weight and bias gradient of layer i from its output gradient `g` (bf16) and input `x_i`."""
      w = weights[i]
      dw = G.gemm(g, x_i, a_mn=True, b_mn=True, out_dtype=torch.float32)
      dw = dw if dw.shape[1] == w.shape[1] else dw[:, :w.shape[1]].contiguous()
      db = ew.colsum(g) if biases[i] is not None else None
      return dw, db

    def queue(i, g, x_i):
      def run(i=i, g=g, x_i=x_i):
        dw, db = wgrad(i, g, x_i)
        # the bias first: gradients reach the hooks in the order autograd would deliver them (reverse
        # parameter order), which is the order the all-reduce buckets are laid out in
        if db is not None:
          _deliver(tb[i], db)
        _deliver(tw[i], dw)
      _pending.append(((g, x_i), run))

    for i in range(n - 1, -1, -1):
      x_i, y_i, w = acts[i], acts[i + 1], weights[i]
      prev_relu = i > 0 and relu[i - 1]
      need_dx = i > 0 or ctx.need_dx
      if w16s[i] is None:   # GEMV output layer
        gv = g.reshape(-1).to(torch.float32)
        if relu[i]:
          gv = torch.where(y_i.reshape(-1) > 0, gv, torch.zeros_like(gv))
        dw = torch.zeros(w.numel(), dtype=torch.float32, device=w.device)
        db = torch.zeros(1, dtype=torch.float32, device=w.device) if biases[i] is not None else None
        g = ew.gemv_bwd(x_i, w.detach().reshape(-1), gv.contiguous(), prev_relu, dw, db)
        if defer:    # computed on the chain anyway: delivered at once
          if db is not None:
            _deliver(tb[i], db)
          _deliver(tw[i], dw.view_as(w))
        else:
          dws[i], dbs[i] = dw.view_as(w), db
        continue
      if g.dtype != torch.bfloat16:
        g = g.to(torch.bfloat16)
      if i == n - 1 and relu[i]:
        g = ew.relu_mask(g, y_i)       # hidden layers get their mask from the GEMM epilogue below
      if defer:
        queue(i, g, x_i)
      else:
        dws[i], dbs[i] = wgrad(i, g, x_i)
      if need_dx:
        if prev_relu:
          g = G.gemm(g, w16s[i], b_mn=True, epi=G.EPI_MASK_RELU, aux0=x_i)
        else:
          g = G.gemm(g, w16s[i], b_mn=True)
    dx = None
    if ctx.need_dx:
      dx = g[:, :ctx.x_shape[1]].to(ctx.x_dtype)
    return (dx, None, None, None, *dws, *dbs)


def mlp(x: torch.Tensor, weights, biases, relu_flags, out: torch.Tensor | None = None,
        defer_wgrad: bool = False) -> torch.Tensor:
  """Functional MLP.  weights[i]: `[out, in]`; biases[i]: `[out]` or None.  `out` (CUDA only): a bf16
  `[M, out_features]` view, possibly strided, that receives the last layer's result.  `defer_wgrad`
  (CUDA only): weight gradients are queued during backward and computed by `flush_deferred()`."""
  if not x.is_cuda:
    h = x.to(torch.float32)
    for w, b, r in zip(weights, biases, relu_flags):
      h = torch.nn.functional.linear(h, w, b)
      if r:
        h = torch.relu(h)
    return h
  flags = tuple(bool(r) for r in relu_flags)
  if defer_wgrad and x.requires_grad and torch.is_grad_enabled():
    det = lambda t: None if t is None else t.detach()
    return MLPFn.apply(x, flags, out, (tuple(weights), tuple(biases)), *[det(w) for w in weights],
                       *[det(b) for b in biases])
  return MLPFn.apply(x, flags, out, None, *weights, *biases)


class CrossNetFn(torch.autograd.Function):
  """DCNv2 cross stack.  Low-rank layer params: (U `[r, d]`, V `[d, r]`, b `[d]`) with
  v = (xl·Uᵀ)·Vᵀ + b; full-rank layer params: (None, W `[d, d]`, b)."""

  @staticmethod
  def forward(ctx, x0, n_layers, low_rank, targets, *params):
    # targets = (us, vs, bs): the real parameters when `params` are detached stand-ins (deferral)
    ctx.defer, ctx.targets = targets is not None, targets
    x0 = x0.detach()
    if x0.dtype != torch.bfloat16 or x0.stride(-1) != 1:
      x0 = x0.to(torch.bfloat16).contiguous()
    us = params[:n_layers] if low_rank else [None] * n_layers
    vs = params[n_layers:2 * n_layers] if low_rank else params[:n_layers]
    bs = params[2 * n_layers:] if low_rank else params[n_layers:]
    xl, saved = x0, []
    for i in range(n_layers):
      v16 = bf16_weight(targets[1][i] if targets is not None else vs[i])
      if low_rank:
        u16 = bf16_weight(targets[0][i] if targets is not None else us[i])
        u = G.gemm(xl, u16)
        out, v = G.gemm(u, v16, bias=bs[i].detach(), epi=G.EPI_CROSS, aux0=x0, aux1=xl, want_out2=True)
        saved.append((xl, u, v, u16, v16))
      else:
        out, v = G.gemm(xl, v16, bias=bs[i].detach(), epi=G.EPI_CROSS, aux0=x0, aux1=xl, want_out2=True)
        saved.append((xl, None, v, None, v16))
      xl = out
    ctx.saved, ctx.x0, ctx.low_rank, ctx.n = saved, x0, low_rank, n_layers
    return xl

  @staticmethod
  def backward(ctx, g):
    x0, n = ctx.x0, ctx.n
    if g.dtype != torch.bfloat16 or g.stride(-1) != 1 or g.stride(0) != x0.stride(0):
      g = g.to(torch.bfloat16).contiguous()
    dx0 = torch.empty_like(x0)
    dus, dvs, dbs = [None] * n, [None] * n, [None] * n
    tus, tvs, tbs = ctx.targets if ctx.defer else (None, None, None)
    for i in range(n - 1, -1, -1):
      xl, u, v, u16, v16 = ctx.saved[i]
      # dv = g⊙x0 ; dx0 (+)= g⊙v ; db = column sums of dv, all in one pass
      dv, dbs[i] = ew.cross_bwd_ew(g, x0, v, dx0, accumulate=i != n - 1, want_colsum=True)
      if ctx.defer:
        _deliver(tbs[i], dbs[i])
        dbs[i] = None
      wg = lambda a, b: G.gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32)
      if ctx.low_rank:
        du = G.gemm(dv, v16, b_mn=True)                                             # [M, r]
        if ctx.defer:
          def run(i=i, dv=dv, u=u, du=du, xl=xl):
            _deliver(tvs[i], wg(dv, u))
            _deliver(tus[i], wg(du, xl))
          _pending.append(((dv, u, du, xl), run))
        else:
          dvs[i] = wg(dv, u)                                                        # [d, r]
          dus[i] = wg(du, xl)                                                       # [r, d]
        # dxl = du·U + g; layer 0's xl IS x0, so its product also takes the accumulated dx0
        g = G.gemm(du, u16, b_mn=True, epi=G.EPI_ADD, aux0=g, aux1=dx0 if i == 0 else None)
      else:
        if ctx.defer:
          def run(i=i, dv=dv, xl=xl):
            _deliver(tvs[i], wg(dv, xl))
          _pending.append(((dv, xl), run))
        else:
          dvs[i] = wg(dv, xl)                                                       # [d, d]
        g = G.gemm(dv, v16, b_mn=True, epi=G.EPI_ADD, aux0=g, aux1=dx0 if i == 0 else None)
    dx0 = g
    if ctx.low_rank:
      return (dx0, None, None, None, *dus, *dvs, *dbs)
    return (dx0, None, None, None, *dvs, *dbs)


def cross_network(x0: torch.Tensor, us, vs, bs, defer_wgrad: bool = False) -> torch.Tensor:
  """`us` None → full-rank layers (`vs[i]` is `[d, d]`).  `defer_wgrad` as in `mlp`."""
  low_rank = us is not None
  if not x0.is_cuda:
    x0f = x0.to(torch.float32)
    xl = x0f
    for i in range(len(vs)):
      h = torch.nn.functional.linear(xl, us[i]) if low_rank else xl
      xl = x0f * torch.nn.functional.linear(h, vs[i], bs[i]) + xl
    return xl
  params = (*us, *vs, *bs) if low_rank else (*vs, *bs)
  if defer_wgrad and x0.requires_grad and torch.is_grad_enabled():
    targets = (tuple(us) if low_rank else None, tuple(vs), tuple(bs))
    return CrossNetFn.apply(x0, len(vs), low_rank, targets, *[t.detach() for t in params])
  return CrossNetFn.apply(x0, len(vs), low_rank, None, *params)


class JoinColumnsFn(torch.autograd.Function):
  """Declares that `full[:, :k]` was produced by `left` and `full[:, k:]` by `right` (both already
  written in place), so the concat costs no copy and its gradient is two views.  Its backward is where
  the data-gradient chain of the layers above ends, so queued weight-gradient work is started here."""

  @staticmethod
  def forward(ctx, left, right, full):
    ctx.k = left.shape[1]
    return full.detach()

  @staticmethod
  def backward(ctx, g):
    flush_deferred()
    return g[:, :ctx.k], g[:, ctx.k:], None


class LinearFn(torch.autograd.Function):
  """Single linear layer (+ optional ReLU, or + a residual added in the GEMM's epilogue) for callers outside
  an MLP stack; works on the last dim of an arbitrary-rank bf16 activation."""

  @staticmethod
  def forward(ctx, x, w, b, relu, residual=None):
    shp = x.shape
    x2 = x.detach().reshape(-1, shp[-1])
    if x2.dtype != torch.bfloat16 or x2.stride(-1) != 1 or x2.stride(0) % 8:
      x2 = x2.to(torch.bfloat16).contiguous()
    w16 = bf16_weight(w)
    if residual is not None:
      r2 = residual.detach().reshape(-1, w.shape[0])
      if r2.dtype != torch.bfloat16 or r2.stride(-1) != 1 or r2.stride(0) % 8:
        r2 = r2.to(torch.bfloat16).contiguous()
      y = G.gemm(x2, w16, bias=None if b is None else b.detach(), epi=G.EPI_ADD, aux0=r2)
    else:
      y = G.gemm(x2, w16, bias=None if b is None else b.detach(), relu=relu)
    ctx.save = (x2, w16, y if relu else None)
    ctx.has_bias, ctx.shape, ctx.dtype, ctx.w_dtype = b is not None, shp, x.dtype, w.dtype
    ctx.res = None if residual is None else (residual.shape, residual.dtype)
    return y.view(*shp[:-1], w.shape[0])

  @staticmethod
  def backward(ctx, dy):
    x2, w16, y = ctx.save
    g = dy.reshape(-1, dy.shape[-1])
    if g.dtype != torch.bfloat16 or g.stride(-1) != 1 or g.stride(0) % 8:
      g = g.to(torch.bfloat16).contiguous()
    if y is not None:
      g = ew.relu_mask(g, y)
    dw = G.gemm(g, x2, a_mn=True, b_mn=True, out_dtype=torch.float32)
    db = ew.colsum(g) if ctx.has_bias else None
    dx = G.gemm(g, w16, b_mn=True).view(ctx.shape).to(ctx.dtype)
    dres = None if ctx.res is None else dy.reshape(ctx.res[0]).to(ctx.res[1])
    return dx, dw.to(ctx.w_dtype), db, None, dres


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None, relu: bool = False,
           residual: torch.Tensor | None = None):
  """y = x w^T + b (+ ReLU) (+ residual).  `residual` (same shape as y) is added in the GEMM's epilogue."""
  if not x.is_cuda or w.shape[0] % 8 or w.shape[1] % 8:
    y = torch.nn.functional.linear(x.to(w.dtype), w, b)
    y = torch.relu(y) if relu else y
    return y if residual is None else y + residual.to(y.dtype)
  assert not (relu and residual is not None)
  return LinearFn.apply(x, w, b, relu, residual)
