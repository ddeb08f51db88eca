"""Small Python helpers (reference: `recml/core/utils/py_utils.py:21-27`)."""
import inspect
from typing import Callable


def has_argument(fn: Callable, arg_name: str) -> bool:
  """True if `fn` accepts `arg_name` explicitly or through `**kwargs`."""
  params = inspect.signature(fn).parameters
  if arg_name in params:
    return True
  return any(p.kind is inspect.Parameter.VAR_KEYWORD for p in params.values())
