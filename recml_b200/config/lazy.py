"""A minimal lazy configuration graph (Fiddle-like semantics, no Fiddle dependency).

The reference configures experiments with `fdl.Config(cls, **kw)` objects that stay
mutable until `fdl.build` instantiates them bottom-up (`recml/examples/
dlrm_experiment.py:360-405`); a sub-config referenced from several places builds to
ONE shared instance, and `fiddle.selectors.select(cfg, Type)` bulk-edits every node
of a type (`recml/examples/dlrm_experiment_test.py:41-54`).  This module provides
exactly those semantics: `Config`, `build`, `select`, dotted `set_path`.
"""
from __future__ import annotations

import ast
import copy
import inspect
from typing import Any, Callable, Generic, Iterator, TypeVar

T = TypeVar("T")
_MISSING = object()


class Config(Generic[T]):
  """A mutable description of the call `fn_or_cls(*args, **kwargs)`.

  Arguments are read and written as attributes (`cfg.trainer.train_steps = 10`).
  Positional arguments are bound to parameter names at construction time so
  that every argument is addressable by name.
  """

  __slots__ = ("__fn__", "__arguments__", "__signature__")

  def __init__(self, fn_or_cls: Callable[..., T], /, *args, **kwargs):
    object.__setattr__(self, "__fn__", fn_or_cls)
    try:
      sig = inspect.signature(fn_or_cls)
    except (TypeError, ValueError):
      sig = None
    object.__setattr__(self, "__signature__", sig)
    bound: dict[str, Any] = {}
    if args:
      if sig is None:
        raise TypeError(f"{fn_or_cls!r} has no signature; pass keywords only.")
      bound.update(sig.bind_partial(*args).arguments)
    for k, v in kwargs.items():
      self._check_name(k)
      bound[k] = v
    object.__setattr__(self, "__arguments__", bound)

  # -- attribute protocol ---------------------------------------------------
  def _check_name(self, name: str) -> None:
    sig = self.__signature__
    if sig is None:
      return
    if name in sig.parameters:
      return
    if any(p.kind is inspect.Parameter.VAR_KEYWORD for p in sig.parameters.values()):
      return
    raise AttributeError(
        f"{getattr(self.__fn__, '__name__', self.__fn__)!r} has no parameter "
        f"{name!r}; valid: {list(sig.parameters)}")

  def __getattr__(self, name: str) -> Any:
    args = object.__getattribute__(self, "__arguments__")
    if name in args:
      return args[name]
    sig = object.__getattribute__(self, "__signature__")
    if sig is not None and name in sig.parameters:
      default = sig.parameters[name].default
      if default is not inspect.Parameter.empty:
        return default
    raise AttributeError(f"No value set for argument {name!r}.")

  def __setattr__(self, name: str, value: Any) -> None:
    self._check_name(name)
    self.__arguments__[name] = value

  def __delattr__(self, name: str) -> None:
    del self.__arguments__[name]

  def __eq__(self, other: Any) -> bool:
    return (isinstance(other, Config) and self.__fn__ is other.__fn__
            and self.__arguments__ == other.__arguments__)

  def __hash__(self):
    return id(self)

  def __repr__(self) -> str:
    name = getattr(self.__fn__, "__qualname__", repr(self.__fn__))
    body = ", ".join(f"{k}={v!r}" for k, v in self.__arguments__.items())
    return f"Config[{name}]({body})"

  def __deepcopy__(self, memo):
    new = Config.__new__(Config)
    memo[id(self)] = new
    object.__setattr__(new, "__fn__", self.__fn__)
    object.__setattr__(new, "__signature__", self.__signature__)
    object.__setattr__(new, "__arguments__", copy.deepcopy(self.__arguments__, memo))
    return new


def _walk(value: Any, seen: set[int]) -> Iterator[Config]:
  if isinstance(value, Config):
    if id(value) in seen:
      return
    seen.add(id(value))
    yield value
    for v in value.__arguments__.values():
      yield from _walk(v, seen)
  elif isinstance(value, (list, tuple, set, frozenset)):
    for v in value:
      yield from _walk(v, seen)
  elif isinstance(value, dict):
    for v in value.values():
      yield from _walk(v, seen)


class Selection:
  """The set of nodes of `root` whose callable is (a subclass of) `target`."""

  def __init__(self, root: Config, target: Any):
    self._nodes = [
        n for n in _walk(root, set())
        if n.__fn__ is target or (inspect.isclass(n.__fn__) and inspect.isclass(target)
                                  and issubclass(n.__fn__, target))]

  def __iter__(self) -> Iterator[Config]:
    return iter(self._nodes)

  def __len__(self) -> int:
    return len(self._nodes)

  def set(self, **kwargs) -> None:
    for n in self._nodes:
      for k, v in kwargs.items():
        setattr(n, k, v)

  def replace(self, value: Any) -> None:
    raise NotImplementedError("Replace nodes by assigning on their parent.")


def select(root: Config, target: Any) -> Selection:
  return Selection(root, target)


def build(value: Any, _memo: dict[int, Any] | None = None) -> Any:
  """Instantiates a config graph bottom-up; shared nodes build exactly once."""
  memo = {} if _memo is None else _memo
  if isinstance(value, Config):
    if id(value) in memo:
      return memo[id(value)]
    kwargs = {k: build(v, memo) for k, v in value.__arguments__.items()}
    sig = value.__signature__
    if sig is not None:
      var_pos = [p.name for p in sig.parameters.values()
                 if p.kind is inspect.Parameter.VAR_POSITIONAL]
      pos_only = [p.name for p in sig.parameters.values()
                  if p.kind is inspect.Parameter.POSITIONAL_ONLY]
      args = [kwargs.pop(n) for n in pos_only if n in kwargs]
      for n in var_pos:
        args.extend(kwargs.pop(n, ()))
      out = value.__fn__(*args, **kwargs)
    else:
      out = value.__fn__(**kwargs)
    memo[id(value)] = out
    return out
  if isinstance(value, list):
    return [build(v, memo) for v in value]
  if isinstance(value, tuple):
    built = [build(v, memo) for v in value]
    return type(value)(*built) if hasattr(value, "_fields") else tuple(built)
  if isinstance(value, dict):
    return {k: build(v, memo) for k, v in value.items()}
  return value


def set_path(root: Config, dotted: str, value: Any) -> None:
  """`set_path(cfg, "a.b[0].c", v)`: attribute / item path assignment."""
  node = ast.parse(dotted.strip(), mode="eval").body

  def resolve(n: ast.AST) -> Any:
    if isinstance(n, ast.Name):
      return getattr(root, n.id)
    if isinstance(n, ast.Attribute):
      return getattr(resolve(n.value), n.attr)
    if isinstance(n, ast.Subscript):
      return resolve(n.value)[ast.literal_eval(n.slice)]
    raise SyntaxError(f"Unsupported path expression: {dotted!r}")

  if isinstance(node, ast.Name):
    setattr(root, node.id, value)
  elif isinstance(node, ast.Attribute):
    setattr(resolve(node.value), node.attr, value)
  elif isinstance(node, ast.Subscript):
    resolve(node.value)[ast.literal_eval(node.slice)] = value
  else:
    raise SyntaxError(f"Unsupported path expression: {dotted!r}")
