"""Dataclass-style configuration primitives.

Covers the reference's `recml/core/utils/types.py:26-157`: a base class that
turns every subclass into a dataclass (`Dataclass`, `FrozenDataclass`), the
`Factory[T]` contract (`make()` builds the run-time object) and `ObjectFactory`,
which wraps an arbitrary constructor so that a library accepting factories can be
handed a plain class plus keyword arguments.
"""
from __future__ import annotations

import abc
import dataclasses
from typing import Any, Generic, Protocol, TypeVar

from typing_extensions import dataclass_transform

T = TypeVar("T")


def _install(cls, frozen: bool, kwargs: dict) -> None:
  if frozen:
    kwargs.setdefault("frozen", True)
  dataclasses.dataclass(**kwargs)(cls)
  cls.replace = lambda self, **updates: dataclasses.replace(self, **updates)


@dataclass_transform(field_specifiers=(dataclasses.field,))
class Dataclass:
  """Subclasses become (mutable) dataclasses and gain `.replace(**updates)`."""

  def __init_subclass__(cls, **kwargs):
    _install(cls, False, kwargs)


@dataclass_transform(field_specifiers=(dataclasses.field,), frozen_default=True)
class FrozenDataclass:
  """Subclasses become frozen dataclasses and gain `.replace(**updates)`."""

  def __init_subclass__(cls, **kwargs):
    _install(cls, True, kwargs)


class Factory(abc.ABC, Generic[T], Dataclass):
  """A dataclass whose `make()` builds an object needing run-time information."""

  @abc.abstractmethod
  def make(self, *args, **kwargs) -> T:
    """Builds the object instance."""


class FactoryProtocol(Protocol, Generic[T]):
  def make(self, *args, **kwargs) -> T: ...
  def replace(self, **overrides) -> Any: ...


class _BoundObjectFactory(Factory):
  """Base of the per-call dataclass synthesised by `ObjectFactory`."""

  def __init_subclass__(cls, **kwargs):  # fields are supplied by make_dataclass
    pass

  def make(self):
    kw = {f.name: getattr(self, f.name) for f in dataclasses.fields(self)
          if f.name != "type"}
    return getattr(self, "type")(**kw)


class ObjectFactory(Factory[T]):
  """`ObjectFactory(type=Cls, a=1).make()` == `Cls(a=1)`; keyword-only."""

  def __new__(cls, *args, **kwargs):
    if args:
      raise ValueError(f"ObjectFactory takes keyword arguments only, got {args}.")
    if "type" not in kwargs:
      raise ValueError(f"ObjectFactory requires a `type` keyword, got {kwargs}.")
    sub = dataclasses.make_dataclass(
        cls.__name__, [(k, type(v)) for k, v in kwargs.items()],
        bases=(_BoundObjectFactory,), kw_only=True)
    return sub(**kwargs)

  def make(self) -> T:  # pragma: no cover - replaced by the synthesised class
    raise NotImplementedError
