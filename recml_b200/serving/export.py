"""Export a trained model for serving and load it back for batch inference.

Layout of an export directory:
  model.json              {"builder": "package.module:Class", "kwargs": {...}, "step": n}
  embedding_spec.json     side-car describing every sharded-embedding module (`embedding/spec_sidecar`)
  weights/<step>/state/   dense parameters and buffers as full arrays, embedding tables as global arrays
                          written shard by shard (the checkpoint format of `recml_b200.ckpt`, no optimizer
                          slots) — a row-sharded table restores on any world size
`load` rebuilds the module from the recipe (a serving job may pass other sharding keyword arguments, e.g.
one GPU instead of eight) and fills it; `Predictor` runs it in eval mode without autograd.
"""
from __future__ import annotations

import importlib
import json
import os
from typing import Any, Callable, Iterable, Iterator, Mapping

import torch
import torch.distributed as dist
from torch import nn

from recml_b200 import ckpt
from recml_b200.training import state as state_lib

MODEL_FILE = "model.json"
SPEC_FILE = "embedding_spec.json"


def _rank() -> int:
  return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _jsonable(v: Any) -> Any:
  if isinstance(v, (list, tuple)):
    return [_jsonable(x) for x in v]
  if isinstance(v, Mapping):
    return {str(k): _jsonable(x) for k, x in v.items()}
  if isinstance(v, (int, float, str, bool)) or v is None:
    return v
  if isinstance(v, torch.dtype):
    return {"__dtype__": str(v).split(".")[-1]}
  return {"__repr__": repr(v)}


def _from_json(v: Any) -> Any:
  if isinstance(v, list):
    return [_from_json(x) for x in v]
  if isinstance(v, dict):
    if "__dtype__" in v:
      return getattr(torch, v["__dtype__"])
    if "__repr__" in v:
      raise ValueError(f"export recipe holds a value that cannot be rebuilt: {v['__repr__']}")
    return {k: _from_json(x) for k, x in v.items()}
  return v


def _weights_tree(model: nn.Module, with_slots: bool = False) -> dict[str, Any]:
  params = {n: p.detach() for n, p in model.named_parameters() if not state_lib.is_sharded_storage(p)}
  buffers = {n: b.detach() for n, b in model.named_buffers() if not state_lib.is_sharded_storage(b)}
  tree: dict[str, Any] = {"params": params, "mutable": buffers}
  sharded = {}
  for name, mod in model.named_modules():
    if hasattr(mod, "sharded_state_dict"):
      sd = mod.sharded_state_dict()
      if not with_slots:
        sd = {k: ({"table": v["table"]} if isinstance(v, dict) and "table" in v else v) for k, v in sd.items()}
      sharded[name or "root"] = sd
  if sharded:
    tree["sharded"] = sharded
  return tree


def export(model: nn.Module, export_dir: str, *, builder: str | None = None, kwargs: Mapping[str, Any] | None = None,
           step: int = 0) -> str:
  """Collective over the job's ranks (every rank writes its table shards; rank 0 writes the rest).
  `builder` is "package.module:Class"; `builder(**kwargs, device=..., group=...)` must rebuild the module.
  A layer that carries `get_config()` (`layers.utils.Configurable`) needs neither: its class and config are the
  recipe, the counterpart of a saved `model.keras` (`recml/core/training/keras_trainer.py:99`)."""
  if builder is None:
    if not hasattr(model, "get_config"):
      raise ValueError("export needs a builder for a module without get_config()")
    builder = "recml_b200.layers.utils:build_from_config"
    kwargs = {"cls": f"{type(model).__module__}:{type(model).__qualname__}", "config": model.get_config()}
  if _rank() == 0:
    os.makedirs(export_dir, exist_ok=True)
  mgr = ckpt.CheckpointManager(os.path.join(export_dir, "weights"), async_save=False, max_to_keep=None)
  mgr.save(step, _weights_tree(model), force=True)
  mgr.close()
  if _rank() == 0:
    with open(os.path.join(export_dir, MODEL_FILE), "w") as f:
      json.dump({"builder": builder, "kwargs": _jsonable(dict(kwargs or {})), "step": int(step)}, f, indent=1)
    from recml_b200.embedding import spec_sidecar
    docs = {name or "root": spec_sidecar.describe(mod) for name, mod in model.named_modules()
            if hasattr(mod, "sharded_state_dict") and hasattr(mod, "plan")}
    with open(os.path.join(export_dir, SPEC_FILE), "w") as f:
      json.dump(docs, f, indent=1)
  if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
    dist.barrier()
  return export_dir


def load(export_dir: str, *, device: torch.device | str | None = None, group=None,
         overrides: Mapping[str, Any] | None = None) -> nn.Module:
  """Rebuilds the exported module on this job's ranks and fills it with the exported weights."""
  with open(os.path.join(export_dir, MODEL_FILE)) as f:
    recipe = json.load(f)
  mod_name, cls_name = recipe["builder"].split(":")
  builder: Callable[..., nn.Module] = getattr(importlib.import_module(mod_name), cls_name)
  kwargs = _from_json(recipe["kwargs"])
  kwargs.update(overrides or {})
  model = builder(**kwargs, device=device, group=group)
  mgr = ckpt.CheckpointManager(os.path.join(export_dir, "weights"), async_save=False, max_to_keep=None)
  tree = mgr.restore(recipe["step"], target=_weights_tree(model))
  with torch.no_grad():
    params = dict(model.named_parameters())
    buffers = dict(model.named_buffers())
    for n, v in tree.get("params", {}).items():
      params[n].copy_(torch.as_tensor(v).to(params[n].dtype))
    for n, v in tree.get("mutable", {}).items():
      buffers[n].copy_(torch.as_tensor(v).to(buffers[n].dtype))
    mods = dict(model.named_modules())
    for name, sd in tree.get("sharded", {}).items():
      mods["" if name == "root" else name].load_sharded_state_dict(sd)   # slots are not part of an export
  model.eval()
  return model


class Predictor:
  """Forward-only use of a module: eval mode, no autograd, inputs moved to the module's device."""

  def __init__(self, model: nn.Module, *, forward: Callable[[nn.Module, Any], Any] | None = None):
    self.model = model.eval()
    self._forward = forward
    p = next(iter(model.parameters()), None)
    self.device = p.device if p is not None else torch.device("cpu")

  def _to_device(self, x: Any) -> Any:
    if isinstance(x, torch.Tensor):
      return x.to(self.device, non_blocking=True)
    if hasattr(x, "to_device"):
      return x.to_device(self.device, None)
    if isinstance(x, Mapping):
      return {k: self._to_device(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
      return type(x)(self._to_device(v) for v in x)
    return x

  @torch.no_grad()
  def predict(self, batch: Any) -> Any:
    batch = self._to_device(batch)
    if self._forward is not None:
      return self._forward(self.model, batch)
    if isinstance(batch, Mapping):
      return self.model(**batch)
    if isinstance(batch, (list, tuple)):
      return self.model(*batch)
    return self.model(batch)


def batch_inference(predictor: Predictor, batches: Iterable[Any], *, max_batches: int | None = None
                    ) -> Iterator[torch.Tensor]:
  """Yields the host copy of every batch's predictions; the device→host copy of batch i overlaps the
  forward pass of batch i+1 (pinned buffers, one event per batch)."""
  pending = None
  for i, batch in enumerate(batches):
    if max_batches is not None and i >= max_batches:
      break
    out = predictor.predict(batch)
    if isinstance(out, torch.Tensor) and out.is_cuda:
      host = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
      host.copy_(out, non_blocking=True)
      ev = torch.cuda.Event()
      ev.record()
      if pending is not None:
        pending[1].synchronize()
        yield pending[0]
      pending = (host, ev)
    else:
      yield out
  if pending is not None:
    pending[1].synchronize()
    yield pending[0]
