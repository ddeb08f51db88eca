"""JSON side-car describing an embedding configuration and its placement.

The reference serialises its stacked-table specs as a protobuf
(`jax_tpu_embedding/sparsecore/lib/proto/embedding_spec_pb2.py`: per stack its name, padded dim and
vocabulary, shard counts, and per table the name, vocabulary, dim, row offset and shard rotation
inside the stack, plus the feature list) so that export tools can un-stack checkpoints without the
training program.  Here the same information, plus the placement plan of this framework, is a
plain JSON document written next to a checkpoint: no protobuf runtime is needed to read it.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Mapping

from recml_b200.embedding import layout_compat
from recml_b200.embedding import planner as planner_lib
from recml_b200.embedding import specs as specs_lib

FORMAT = "recml_b200.embedding_spec/1"

_OPTIMIZERS = {cls.kind: cls for cls in (
    specs_lib.SGDOptimizerSpec, specs_lib.AdagradOptimizerSpec, specs_lib.RowWiseAdagradOptimizerSpec,
    specs_lib.AdamOptimizerSpec, specs_lib.RowWiseAdamOptimizerSpec, specs_lib.AdagradMomentumOptimizerSpec,
    specs_lib.FTRLOptimizerSpec, specs_lib.LaPropOptimizerSpec)}


def optimizer_to_dict(opt: specs_lib.OptimizerSpec) -> dict[str, Any]:
  d = {"kind": opt.kind}
  for f in dataclasses.fields(opt):
    v = getattr(opt, f.name)
    d[f.name] = v if not callable(v) else {"schedule": getattr(v, "__name__", "callable"), "value_at_0": float(v(0))}
  return d


def optimizer_from_dict(d: Mapping[str, Any]) -> specs_lib.OptimizerSpec:
  cls = _OPTIMIZERS[d["kind"]]
  kw = {}
  for f in dataclasses.fields(cls):
    if f.name in d:
      v = d[f.name]
      kw[f.name] = v["value_at_0"] if isinstance(v, dict) else v   # schedules come back as their initial value
  return cls(**kw)


def describe(module, *, reference_shards: int | None = None) -> dict[str, Any]:
  """Document for a `ShardedEmbedding`: features, tables (with optimizer), this framework's
  placement and, when `reference_shards` is given, the reference stack layout of the same tables."""
  cfg = module.config
  tables, feature_to_table = cfg.table_specs()
  doc: dict[str, Any] = {"format": FORMAT, "world": module.world, "features": [], "tables": [], "stacks": []}
  for fname, s in cfg.specs.items():
    doc["features"].append({"name": fname, "table": feature_to_table[fname], "combiner": s.combiner,
                            "max_sequence_length": s.max_sequence_length, "weight_name": s.weight_name})
  for t in tables:
    tp = module.plan.tables[t.name]
    doc["tables"].append({
        "name": t.name, "vocabulary_size": t.vocabulary_size, "embedding_dim": t.embedding_dim,
        "optimizer": optimizer_to_dict(t.optimizer),
        "placement": tp.placement.value, "owner": tp.owner, "rotation": tp.rotation, "stack": tp.stack})
  for i, st in enumerate(module.plan.stacks):
    doc["stacks"].append({"index": i, "dim": st.dim, "optimizer": st.optimizer.kind, "tables": list(st.tables)})
  if reference_shards:
    groups: dict[int, list] = {}
    for t in tables:
      groups.setdefault((t.embedding_dim + 7) // 8 * 8, []).append((t.name, t.vocabulary_size, t.embedding_dim))
    doc["reference_layout"] = []
    for members in groups.values():
      lay = layout_compat.stack_layout(members, reference_shards)
      doc["reference_layout"].append({
          "stack_name": lay.name, "num_shards": lay.num_shards, "padded_embedding_dim": lay.padded_dim,
          "rows_per_shard": lay.rows_per_shard,
          "tables": [dataclasses.asdict(t) for t in lay.tables]})
  return doc


def write(module, path: str, **kw) -> str:
  """Writes the side-car (rank 0 only does the I/O); returns the path."""
  import torch.distributed as dist
  doc = describe(module, **kw)
  if not dist.is_initialized() or dist.get_rank() == 0:
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
      json.dump(doc, f, indent=1, sort_keys=True)
    os.replace(tmp, path)
  return path


def read(path: str) -> dict[str, Any]:
  with open(path) as f:
    doc = json.load(f)
  if doc.get("format") != FORMAT:
    raise ValueError(f"{path}: not an embedding spec side-car ({doc.get('format')!r})")
  return doc


def table_specs(doc: Mapping[str, Any]) -> list[specs_lib.TableSpec]:
  return [specs_lib.TableSpec(t["name"], t["vocabulary_size"], t["embedding_dim"], optimizer_from_dict(t["optimizer"]))
          for t in doc["tables"]]


def placement_overrides(doc: Mapping[str, Any]) -> dict[str, planner_lib.Placement]:
  """Placement of every table as recorded, to rebuild the same plan in another job."""
  return {t["name"]: planner_lib.Placement(t["placement"]) for t in doc["tables"]}


def reference_layouts(doc: Mapping[str, Any]) -> list[layout_compat.StackLayout]:
  out = []
  for s in doc.get("reference_layout", []):
    tabs = tuple(layout_compat.TableInStack(**t) for t in s["tables"])
    out.append(layout_compat.StackLayout(s["stack_name"], s["num_shards"], s["padded_embedding_dim"],
                                         s["rows_per_shard"], tabs))
  return out
