"""Flatten / unflatten nested dict-list trees with Orbax-style dotted leaf keys."""
from __future__ import annotations

from typing import Any, Iterator


def flatten(tree: Any, prefix: tuple[str, ...] = ()) -> Iterator[tuple[tuple[str, ...], Any]]:
  if isinstance(tree, dict):
    for k in tree:
      yield from flatten(tree[k], prefix + (str(k),))
  elif isinstance(tree, (list, tuple)):
    for i, v in enumerate(tree):
      yield from flatten(v, prefix + (str(i),))
  else:
    yield prefix, tree


def unflatten(items: dict[tuple[str, ...], Any]) -> Any:
  root: dict[str, Any] = {}
  for path, v in items.items():
    node = root
    for p in path[:-1]:
      node = node.setdefault(p, {})
    node[path[-1]] = v
  return root


def key_types(tree: Any, prefix: tuple[str, ...] = ()) -> dict[tuple[str, ...], str]:
  """Container kind at every interior path ("dict" | "list" | "tuple")."""
  out = {}
  if isinstance(tree, dict):
    out[prefix] = "dict"
    for k, v in tree.items():
      out.update(key_types(v, prefix + (str(k),)))
  elif isinstance(tree, (list, tuple)):
    out[prefix] = "list" if isinstance(tree, list) else "tuple"
    for i, v in enumerate(tree):
      out.update(key_types(v, prefix + (str(i),)))
  return out


def restore_containers(tree: Any, kinds: dict[tuple[str, ...], str], prefix=()) -> Any:
  if not isinstance(tree, dict):
    return tree
  built = {k: restore_containers(v, kinds, prefix + (k,)) for k, v in tree.items()}
  kind = kinds.get(prefix, "dict")
  if kind in ("list", "tuple"):
    seq = [built[str(i)] for i in range(len(built))]
    return seq if kind == "list" else tuple(seq)
  return built
