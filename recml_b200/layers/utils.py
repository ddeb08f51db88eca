"""Layer helpers (`recml/layers/keras/utils.py:22-147`): attention masks, activations, the L2
embedding post-processor, rotary encodings."""
from __future__ import annotations

import copy
from typing import Any

import torch


def clone_initializer(initializer: Any) -> Any:
  return copy.deepcopy(initializer)


def make_attention_mask(mask: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
  """`[B, L]` padding mask → `[B, L, L]` pairwise mask."""
  return (mask.unsqueeze(-1) * mask.unsqueeze(-2)).to(dtype)


def make_causal_mask(mask: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
  return torch.tril(make_attention_mask(mask, dtype))


def gelu_approximate(x: torch.Tensor) -> torch.Tensor:
  return torch.nn.functional.gelu(x, approximate="tanh")


def relu_squared(x: torch.Tensor) -> torch.Tensor:
  return torch.relu(x) ** 2


def norm_embedding_post_processor(inputs: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
  """Scales every embedding to unit L2 norm (norm clipped below at eps)."""
  return inputs / inputs.norm(dim=-1, keepdim=True).clamp_min(eps)


def apply_rotary_encoding(x: torch.Tensor, *, positions: torch.Tensor | None = None,
                          max_wavelength: int) -> torch.Tensor:
  """RoPE on `[*batch, L, H, Dh]` (Dh even): halves are rotated by position/timescale."""
  if x.shape[-1] % 2:
    raise ValueError(f"Embedding dimension must be even, but got {x.shape[-1]} for input of shape {tuple(x.shape)}.")
  if x.ndim < 4:
    raise ValueError(f"Unexpected input shape: {tuple(x.shape)}. Expected shape of rank 4 or greater.")
  L, half = x.shape[-3], x.shape[-1] // 2
  if positions is None:
    positions = torch.arange(L, device=x.device).expand(*x.shape[:-3], L)
  elif tuple(positions.shape) != tuple(x.shape[:-2]):
    raise ValueError(f"Positions must be of shape: {tuple(x.shape[:-2])} but got shape: {tuple(positions.shape)}.")
  exponents = (2.0 / x.shape[-1]) * torch.arange(half, dtype=torch.float32, device=x.device)
  timescale = float(max_wavelength) ** exponents
  radians = positions.to(torch.float32)[..., None] / timescale          # [..., L, half]
  radians = radians[..., None, :]                                        # [..., L, 1, half]
  sin, cos = torch.sin(radians), torch.cos(radians)
  x1, x2 = x[..., :half].float(), x[..., half:].float()
  return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


def large_negative_for_attention(dtype: torch.dtype) -> float:
  return -3e4 if dtype == torch.float16 else -1e9


# ---- constructor-argument round trip ----------------------------------------------------------------------


def _config_value(v: Any) -> Any:
  """A constructor argument as something JSON can hold: functions become their dotted import path, a nested
  layer its class and its own config."""
  if isinstance(v, Configurable):
    return {"layer": f"{type(v).__module__}:{type(v).__qualname__}", "config": v.get_config()}
  if callable(v) and not isinstance(v, torch.nn.Module) and hasattr(v, "__module__") and hasattr(v, "__qualname__"):
    return {"callable": f"{v.__module__}.{v.__qualname__}"}
  if isinstance(v, torch.dtype):
    return {"dtype": str(v).removeprefix("torch.")}
  if isinstance(v, (list, tuple)):
    return [_config_value(x) for x in v]
  if isinstance(v, dict):
    return {str(k): _config_value(x) for k, x in v.items()}
  return v


def _config_restore(v: Any) -> Any:
  if isinstance(v, dict) and set(v) == {"callable"}:
    import importlib
    parts = v["callable"].split(".")
    for cut in range(len(parts) - 1, 0, -1):              # longest importable module prefix, then attributes
      try:
        obj = importlib.import_module(".".join(parts[:cut]))
      except ImportError:
        continue
      for name in parts[cut:]:
        obj = getattr(obj, name)
      return obj
    raise ImportError(f"cannot resolve {v['callable']!r}")
  if isinstance(v, dict) and set(v) == {"dtype"}:
    return getattr(torch, v["dtype"])
  if isinstance(v, dict) and set(v) == {"layer", "config"}:
    return build_from_config(v["layer"], v["config"])
  if isinstance(v, list):
    return [_config_restore(x) for x in v]
  if isinstance(v, dict):
    return {k: _config_restore(x) for k, x in v.items()}
  return v


class Configurable:
  """`get_config()` / `from_config()` for a layer, the pair every layer of the reference carries
  (`recml/layers/keras/hstu.py:115-127,165-174,476-492,623-628`, `sasrec.py:165-170`, `bert4rec.py:194-208`,
  `mamba.py:417-424,528,622,747-752`).  The config is the constructor call: the arguments the outermost `__init__`
  received (defaults included), with functions written as dotted import paths so that the dictionary survives
  JSON; `cls(**config)` and `cls.from_config(config)` rebuild an identically shaped, freshly initialised layer.
  """

  def __init_subclass__(cls, **kwargs):
    super().__init_subclass__(**kwargs)
    init = cls.__dict__.get("__init__")
    if init is None:
      return
    import functools
    import inspect
    sig = inspect.signature(init)

    @functools.wraps(init)
    def wrapped(self, *args, **kw):
      if "_init_config" not in self.__dict__:               # the outermost constructor wins
        bound = sig.bind(self, *args, **kw)
        bound.apply_defaults()
        cfg = {}
        for name, value in list(bound.arguments.items())[1:]:
          kind = sig.parameters[name].kind
          if kind is inspect.Parameter.VAR_KEYWORD:
            cfg.update(value)
          elif kind is not inspect.Parameter.VAR_POSITIONAL:
            cfg[name] = value
        object.__setattr__(self, "_init_config", cfg)
      init(self, *args, **kw)

    cls.__init__ = wrapped

  def get_config(self) -> dict[str, Any]:
    return {k: _config_value(v) for k, v in self.__dict__["_init_config"].items()}

  @classmethod
  def from_config(cls, config: dict[str, Any]):
    return cls(**{k: _config_restore(v) for k, v in config.items()})


def build_from_config(cls: str, config: dict[str, Any], device=None, group=None):
  """Rebuilds a `Configurable` layer from `"package.module:Class"` and its `get_config()` dictionary on
  `device`: the recipe `serving.export` writes for a layer that is exported without a builder of its own."""
  import importlib
  mod_name, cls_name = cls.split(":")
  layer = getattr(importlib.import_module(mod_name), cls_name).from_config(config)
  return layer.to(device) if device is not None else layer
