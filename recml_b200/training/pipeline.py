"""Software pipelining of embedding work against dense work across steps.

The reference's auto-pipelining (`jax_tpu_embedding/sparsecore/lib/auto_pipelining/
auto_pipelining.py:134-214`) splits a jitted train step into embedding-lookup / dense /
embedding-update programs and runs, in step i, `update(i-2)` and `lookup(i)` on the SparseCores
while `dense(i-1)` runs on the TensorCores; the carried state is `(activations_1, args_1,
updates_0)` and two `finalize` calls drain it.  Lookups therefore see tables that miss the last two
updates: the schedule changes the numerics, so it is opt-in.

Here the three programs are explicit callables and the two engines are CUDA streams:

  lookup(batch)                  -> activations            (embedding stream)
  dense(activations, batch)      -> (emb_grads, results)   (main stream)
  update(emb_grads, activations) -> None                   (embedding stream)

`PipelinedStep.__call__(batch)` issues `update(i-2)`, `lookup(i)` on the embedding stream and
`dense(i-1)` on the caller's stream, ordered by events, and returns the results of step i-1 (None
for the first call).  `finalize()` runs the two drain steps and returns the last results.

`for_sharded_embedding` builds the three callables for a model whose embedding is a
`ShardedEmbedding`: the lookup keeps the autograd node of the embedding output, the dense stage
works on a detached copy and the update stage feeds the copy's gradient into that node, which runs
the exchange + row-optimizer kernels.  Two lookups are in flight before the first update, so the
embedding backend must keep per-call state: the collective backend does by construction; the fused
NVLink backend is switched to two occurrence lists per table stack and launch-time sequence numbers
(`FusedBackend.set_pipeline_depth(2)`, done here before its first lookup).
"""
from __future__ import annotations

import contextlib
import dataclasses
from typing import Any, Callable

import torch


@dataclasses.dataclass
class _InFlight:
  batch: Any = None
  activations: Any = None
  ready: Any = None          # event: activations produced


class PipelinedStep:
  def __init__(self, lookup: Callable[[Any], Any], dense: Callable[[Any, Any], tuple[Any, Any]],
               update: Callable[[Any, Any], None], *, device: torch.device | None = None):
    self._lookup, self._dense, self._update = lookup, dense, update
    self._cuda = device is not None and device.type == "cuda"
    self._device = device
    self._emb_stream = torch.cuda.Stream(device=device) if self._cuda else None
    self._stage1: _InFlight | None = None      # looked up, waiting for its dense stage
    self._stage0: tuple[Any, Any, Any] | None = None   # (emb_grads, activations, event) waiting for the update
    self.steps_issued = 0

  # -- stream helpers (no-ops on CPU) ----------------------------------------------------------------
  def _on_emb(self):
    return torch.cuda.stream(self._emb_stream) if self._cuda else contextlib.nullcontext()

  def _event(self, stream=None):
    if not self._cuda:
      return None
    ev = torch.cuda.Event()
    ev.record(stream if stream is not None else torch.cuda.current_stream(self._device))
    return ev

  def _wait(self, stream, ev):
    if self._cuda and ev is not None:
      stream.wait_event(ev)

  def _run(self, batch):
    main = torch.cuda.current_stream(self._device) if self._cuda else None
    # embedding engine: update(i-2) then lookup(i)
    new1 = None
    with self._on_emb():
      if self._stage0 is not None:
        grads, acts, grads_ready = self._stage0
        self._wait(self._emb_stream, grads_ready)
        self._update(grads, acts)
        self._stage0 = None
      if batch is not None:
        if self._cuda:
          self._emb_stream.wait_stream(main)      # the batch was staged on the caller's stream
        acts = self._lookup(batch)
        new1 = _InFlight(batch, acts, self._event(self._emb_stream))
    # dense engine: dense(i-1)
    results = None
    if self._stage1 is not None:
      prev = self._stage1
      self._wait(main, prev.ready)
      grads, results = self._dense(prev.activations, prev.batch)
      self._stage0 = (grads, prev.activations, self._event(main))
    self._stage1 = new1
    return results

  def __call__(self, batch):
    self.steps_issued += 1
    return self._run(batch)

  def finalize(self):
    """Drains the pipeline: dense of the last batch, then its update; returns the last results."""
    results = self._run(None)
    self._run(None)
    if self._cuda:
      torch.cuda.current_stream(self._device).wait_stream(self._emb_stream)
    return results


def for_sharded_embedding(embedding, dense_fn: Callable[[torch.Tensor, Any], tuple[torch.Tensor, Any]],
                          get_ids: Callable[[Any], Any], *, device: torch.device | None = None) -> PipelinedStep:
  """Pipeline for `embedding` (a `ShardedEmbedding`).  `dense_fn(activations, batch)` must run the
  dense forward + backward + dense optimizer step and return `(loss, results)`; it receives
  activations that require grad, and their `.grad` after it returns is what the update stage
  pushes to the table owners."""
  backend = getattr(embedding, "_backend", None)
  if hasattr(backend, "set_pipeline_depth") and backend.pipeline_depth < 2:
    backend.set_pipeline_depth(2)

  def lookup(batch):
    with torch.enable_grad():
      out = embedding(get_ids(batch))
    return out

  def dense(acts, batch):
    leaf = acts.detach().requires_grad_(True)
    _, results = dense_fn(leaf, batch)
    return leaf.grad, results

  def update(grads, acts):
    if grads is not None:
      acts.backward(grads)

  return PipelinedStep(lookup, dense, update, device=device)
