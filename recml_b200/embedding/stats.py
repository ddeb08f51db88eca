"""Placement statistics measured on a batch: how a feature's ids spread over the residue classes `id % world`.

The reference sizes its per-partition buffers from recorded statistics of the input (feedback-directed
optimisation: `max_ids_per_partition`, `max_unique_ids_per_partition`,
`jax_tpu_embedding/sparsecore/lib/fdo/file_fdo_client.py`).  Here the same two quantities, taken per residue
class on the first batch and summed over the ranks, feed the sharding planner: a row-sharded table puts class q on
rank (q + rotation) % world, so they say what every rank would carry, and distinct ids (row read-modify-writes,
cache misses) are weighed apart from occurrences.
"""
from __future__ import annotations

from typing import Mapping

import torch
import torch.distributed as dist

from recml_b200.embedding.jagged import KeyedJagged


def batch_residue_stats(kjt: KeyedJagged, world: int, group=None) -> Mapping[str, tuple[list[float], list[float]]] | None:
  """`{feature: (ids per sample by class, distinct ids per sample by class)}` over the GLOBAL batch (a collective:
  every rank calls it with its local batch and gets the same result), or None for a single rank.  Distinct ids are
  counted per rank and added up, which counts an id that several ranks saw several times: an upper bound that is
  tight for the large tables whose placement it decides."""
  if world <= 1:
    return None
  names = tuple(kjt.keys)
  B = kjt.batch_size()
  vals, offs = kjt.values, kjt.offsets
  bounds = offs[::B].tolist() if offs.numel() == len(names) * B + 1 else None
  if bounds is None:
    return None
  out = torch.zeros(len(names), 2, world, dtype=torch.float64, device=vals.device)
  for i in range(len(names)):
    ids = vals[bounds[i]:bounds[i + 1]].long()
    if ids.numel() == 0:
      continue
    out[i, 0] = torch.bincount(ids % world, minlength=world)[:world].double()
    out[i, 1] = torch.bincount(torch.unique(ids) % world, minlength=world)[:world].double()
  if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
    if dist.get_backend(group) == "nccl" and not out.is_cuda:
      out = out.cuda()
    dist.all_reduce(out, group=group)
    denom = float(B * dist.get_world_size(group))
  else:
    denom = float(B)
  out = (out / denom).cpu()
  return {n: (out[i, 0].tolist(), out[i, 1].tolist()) for i, n in enumerate(names)}
