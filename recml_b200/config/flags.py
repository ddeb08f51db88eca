"""Command-line configuration of a lazy `Config` through one repeated absl flag.

Same user-facing grammar as the reference flag (`recml/core/utils/config.py:33-136`,
exercised by `recml/core/utils/config_test.py:65-156`):

  --experiment=config:<fn | pkg.module.fn>[(literal args)]   base config
  --experiment=fiddler:<fn | pkg.module.fn>[(literal args)]  mutator fn(cfg, *args)
  --experiment=set:<dotted.path>=<python literal>            single assignment

Directives apply in command-line order.  The module that defined the base config
becomes the default namespace for later un-dotted fiddler names.
"""
from __future__ import annotations

import ast
import dataclasses
import importlib
import inspect
import re
import types
from typing import Any

from absl import flags

from recml_b200.config import lazy


@dataclasses.dataclass(frozen=True)
class CallExpression:
  """`name` or `name(lit, k=lit)` split into its parts; arguments must be literals."""

  func_name: str
  args: tuple[Any, ...]
  kwargs: dict[str, Any]

  _HEAD = re.compile(r"\s*([A-Za-z_][\w\.]*)\s*(\(.*\))?\s*", re.S)

  @classmethod
  def parse(cls, text: str) -> "CallExpression":
    m = cls._HEAD.fullmatch(text)
    if m is None:
      raise SyntaxError(f"Expected a function name or call expression; got {text!r}")
    name, arglist = m.group(1), m.group(2)
    if arglist is None:
      return cls(name, (), {})
    # Parse the parenthesised part as the argument list of a dummy call.
    try:
      call = ast.parse("_" + arglist, mode="eval").body
    except SyntaxError as e:
      raise SyntaxError(f"Malformed arguments in {text!r}: {e}") from e
    if not isinstance(call, ast.Call):
      raise SyntaxError(f"Expected a call expression; got {text!r}")
    pos, kw = [], {}
    for a in call.args:
      if isinstance(a, ast.Starred):
        raise SyntaxError("*args is not supported.")
      pos.append(cls._literal(a, text))
    for k in call.keywords:
      if k.arg is None:
        raise SyntaxError("**kwargs is not supported.")
      kw[k.arg] = cls._literal(k.value, text)
    return cls(name, tuple(pos), kw)

  @staticmethod
  def _literal(node: ast.AST, text: str) -> Any:
    try:
      return ast.literal_eval(node)
    except ValueError as e:
      raise SyntaxError(
          f"Arguments must be literals; got {ast.unparse(node)!r} in {text!r}") from e


def _import_symbol(dotted: str, base: types.ModuleType | None, what: str) -> Any:
  """Longest importable module prefix of `dotted`, then getattr the remainder."""
  parts = dotted.split(".")
  if base is not None:
    parts = base.__name__.split(".") + parts
  for cut in range(len(parts) - 1, 0, -1):
    try:
      obj = importlib.import_module(".".join(parts[:cut]))
    except ModuleNotFoundError:
      continue
    for depth, piece in enumerate(parts[cut:]):
      if not hasattr(obj, piece):
        public = ", ".join(repr(n) for n in dir(obj) if not n.startswith("_"))
        raise AttributeError(
            f"{what} {dotted!r}: {'.'.join(parts[:cut + depth])!r} has no attribute "
            f"{piece!r}; available names: {public}")
      obj = getattr(obj, piece)
    return obj
  raise ModuleNotFoundError(f"{what} {dotted!r}: no importable module prefix.")


def resolve_callable(name: str, module: types.ModuleType | None, what: str) -> Any:
  if module is not None and hasattr(module, name):
    return getattr(module, name)
  if "." in name:
    if module is not None:
      try:
        return _import_symbol(name, module, what)
      except (ModuleNotFoundError, AttributeError):
        pass
    try:
      return _import_symbol(name, None, what)
    except ModuleNotFoundError as e:
      raise ValueError(f"{what} {name!r}: {e}") from e
  avail = [] if module is None else [
      n for n in dir(module) if not n.startswith("_") and callable(getattr(module, n))]
  raise ValueError(f"{what} {name!r}: unresolved name; available: {', '.join(avail)}")


class FiddleFlag(flags.MultiFlag):
  """Repeated flag whose value is the `Config` produced by applying all directives."""

  def __init__(self, *args, default_module: types.ModuleType | None = None,
               pyref_policy: Any | None = None, **kwargs):
    self.default_module = default_module
    self.pyref_policy = pyref_policy
    self._directives: list[str] = []
    self._config: Any = None
    self._built = False
    super().__init__(*args, **kwargs)

  def parse(self, arguments):
    new = [arguments] if isinstance(arguments, str) else list(arguments or ())
    self._directives.extend(new)
    self._built = False
    self.present += len(new)
    self.using_default_value = False

  def _apply(self, directive: str) -> None:
    kind, sep, body = directive.partition(":")
    if not sep:
      raise ValueError(f"Expected '<config|fiddler|set>:...'; got {directive!r}")
    if kind == "config":
      if self._config is not None:
        raise ValueError("Only one `config:` directive is allowed.")
      expr = CallExpression.parse(body)
      fn = resolve_callable(expr.func_name, self.default_module,
                            "Could not init a buildable from")
      self.default_module = inspect.getmodule(fn)
      as_buildable = getattr(fn, "as_buildable", None)
      cfg = (as_buildable or fn)(*expr.args, **expr.kwargs)
      if cfg is None:
        raise ValueError(f"Could not init a buildable from {body!r}: returned None.")
      self._config = cfg
    elif kind == "fiddler":
      if self._config is None:
        raise ValueError("A `config:` directive must precede `fiddler:`.")
      expr = CallExpression.parse(body)
      fn = resolve_callable(expr.func_name, self.default_module, "Could not load fiddler")
      out = fn(self._config, *expr.args, **expr.kwargs)
      if out is not None:
        self._config = out
    elif kind == "set":
      if self._config is None:
        raise ValueError("A `config:` directive must precede `set:`.")
      path, eq, literal = body.partition("=")
      if not eq:
        raise ValueError(f"Expected 'set:<path>=<literal>'; got {directive!r}")
      try:
        value = ast.literal_eval(literal.strip())
      except (ValueError, SyntaxError):
        value = literal.strip()
      lazy.set_path(self._config, path, value)
    else:
      raise ValueError(f"Unknown directive {kind!r} in {directive!r}")

  @property
  def value(self):
    if not self._built:
      self._config = None
      for d in self._directives:
        self._apply(d)
      self._built = True
    return self._config if self._directives else self.default

  @value.setter
  def value(self, v):
    self.default_value = v

  def serialize(self) -> str:
    return " ".join(f"--{self.name}={d}" for d in self._directives)


def DEFINE_fiddle_config(name: str, *, default: Any = None, help_string: str,  # pylint: disable=invalid-name
                         pyref_policy: Any | None = None,
                         flag_values: flags.FlagValues = flags.FLAGS,
                         required: bool = False) -> flags.FlagHolder:
  """Declares `--<name>` taking `config:`, `fiddler:` and `set:` directives."""
  flag = FiddleFlag(flags.ArgumentParser(), flags.ArgumentSerializer(), name, default,
                    help_string, default_module=None, pyref_policy=pyref_policy)
  return flags.DEFINE_flag(flag, flag_values=flag_values, required=required)
