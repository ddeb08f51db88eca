"""Config graph, the `config:/fiddler:/set:` flag and dataclass factories
(cases follow `recml/core/utils/config_test.py` and `types_test.py`)."""
import dataclasses

import pytest
from absl import flags

from recml_b200 import config as C
from recml_b200.utils import py_utils, types

_ME = __name__


@dataclasses.dataclass
class _X:
  value: int


@dataclasses.dataclass
class _Y:
  value: int


@dataclasses.dataclass
class _Object:
  x: _X
  y: _Y


def config_1() -> C.Config:
  return C.Config(_Object, x=C.Config(_X, value=1), y=C.Config(_Y, value=2))


def fiddler_1(cfg):
  cfg.x.value = 3


def fiddler_2(cfg, value: int):
  cfg.y.value = value


def _flag():
  return C.FiddleFlag(flags.ArgumentParser(), None, "test_flag", None, "help")


@pytest.mark.parametrize("args,want", [
    ([f"config:{_ME}.config_1"], (1, 2)),
    ([f"config:{_ME}.config_1", "fiddler:fiddler_1", "fiddler:fiddler_2(value=4)"], (3, 4)),
    ([f"config:{_ME}.config_1", f"fiddler:{_ME}.fiddler_2(3)"], (1, 3)),
    ([f"config:{_ME}.config_1", "set:x.value=0", "set:y.value=0"], (0, 0))])
def test_fiddle_flag(args, want):
  f = _flag()
  f.parse(args)
  expected = C.Config(_Object, x=C.Config(_X, value=want[0]), y=C.Config(_Y, value=want[1]))
  assert f.value == expected
  obj = C.build(f.value)
  assert (obj.x.value, obj.y.value) == want


def test_invalid_fiddle_flag():
  f = _flag()
  f.parse([f"config:{_ME}.config_3"])
  with pytest.raises(AttributeError, match="Could not init a buildable from .*"):
    _ = f.value
  f = _flag()
  f.parse([f"config:{_ME}.config_1", "fiddler:fiddler_3"])
  with pytest.raises(ValueError):
    _ = f.value


def test_call_expression():
  e = C.CallExpression.parse("fn('foo', False, x=[1, 2])")
  assert (e.func_name, e.args, e.kwargs) == ("fn", ("foo", False), {"x": [1, 2]})
  assert C.CallExpression.parse("a.b.fn") == C.CallExpression("a.b.fn", (), {})
  for bad in ("fn(*a)", "fn(**k)", "fn(x=y)", "1fn", "fn(1"):
    with pytest.raises(SyntaxError):
      C.CallExpression.parse(bad)


def test_shared_subconfig_builds_once_and_select():
  shared = C.Config(_X, value=7)
  root = C.Config(_Object, x=shared, y=C.Config(_Y, value=1))
  holder = C.Config(dict, a=root, b=shared)
  built = C.build(holder)
  assert built["a"].x is built["b"]
  C.select(root, _X).set(value=9)
  assert shared.value == 9 and len(C.select(root, _X)) == 1
  with pytest.raises(AttributeError):
    shared.nope = 1


def test_dataclass_transforms():
  class A(types.Dataclass):
    a: int
    b: str = "x"

  class F(types.FrozenDataclass):
    a: int

  class B(A):
    c: float = 1.0

  assert A(1).replace(b="y") == A(1, "y")
  assert B(1, c=2.0).c == 2.0
  f = F(1)
  with pytest.raises(dataclasses.FrozenInstanceError):
    f.a = 2
  assert f.replace(a=3).a == 3


def test_object_factory():
  class Obj:
    def __init__(self, x, y):
      self.x, self.y = x, y

  fac = types.ObjectFactory(type=Obj, x=1, y=2)
  o = fac.make()
  assert (o.x, o.y) == (1, 2)
  assert fac.replace(x=5).make().x == 5
  with pytest.raises(ValueError):
    types.ObjectFactory(Obj)
  with pytest.raises(ValueError):
    types.ObjectFactory(x=1)


def test_has_argument():
  def f(a, **kw): ...
  def g(a): ...
  assert py_utils.has_argument(f, "zzz") and py_utils.has_argument(g, "a") and not py_utils.has_argument(g, "b")
