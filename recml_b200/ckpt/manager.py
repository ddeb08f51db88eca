"""Checkpoint manager with the directory layout the reference's trainers produce.

Reference behaviour being reproduced (`recml/core/training/jax_trainer.py:461-552`,
`recml/core/utils/keras_utils.py:37-137`): checkpoints live in
`<model_dir>/checkpoints/<step>/` holding one sub-directory per item ("state" for the
trainer's composite save, "default" for single-item saves) plus a "metrics" JSON item
and `_CHECKPOINT_METADATA`; saves are asynchronous, a `should_save_fn(step, last)`
decides which steps are kept, and at most `max_to_keep` steps stay on disk.

A checkpoint is staged in `<step>.orbax-checkpoint-tmp-<n>` and renamed to `<step>`
once every rank finished writing, so a reader never sees a partial step directory;
`commit_success.txt` is written last inside it as the completion marker.  In a multi-rank job
the ranks agree on success before the rename: if any rank failed to write its shards the
staging directory is removed, nothing is committed or rotated out, and every rank raises.
`async_save` moves the file writes to a background thread (tensors that live in host memory are copied first).
In a multi-rank job the ranks then agree through marker files in the staging directory instead of a collective,
so nothing touches the process group off the main thread; `wait_until_finished` (and the next `save`) raises on
every rank when the checkpoint was not committed.  A synchronous multi-rank save agrees with a collective.
"""
from __future__ import annotations

import json
import os
import shutil
import threading
import time
from typing import Any, Callable, Iterator, Mapping

import numpy as np
import torch
import torch.distributed as dist

from recml_b200.ckpt import tree as tree_lib
from recml_b200.ckpt import zarr_io

CHECKPOINT_METADATA = "_CHECKPOINT_METADATA"
TREE_METADATA = "_METADATA"
SHARDING_FILE = "_sharding"
COMMIT_FILE = "commit_success.txt"
TMP_MARK = ".orbax-checkpoint-tmp-"


class ShardedLeaf:
  """A tensor that is one block of a larger global array.

  `global_shape` is the full array, `grid_index` the block coordinate of this rank's
  `local` block and `chunk_shape` the block size; the block grid becomes the zarr
  chunk grid.  `write` is False on ranks that hold a replica which another rank saves.
  """

  def __init__(self, local: torch.Tensor, global_shape, grid_index, chunk_shape=None, write=True, mod=None):
    self.local = local
    self.global_shape = tuple(int(s) for s in global_shape)
    self.grid_index = tuple(int(i) for i in grid_index)
    self.chunk_shape = tuple(int(s) for s in (chunk_shape or local.shape))
    self.write = write
    # Row-sharded embedding tables are stored in MOD layout, `[W, ceil(V / W), ...]` with block r holding the
    # rows whose id is r modulo W.  `mod = {"vocab": V, "world": W}` records that, so that a job with another
    # world size can pick its own residue class out of the stored blocks (`_read_mod_resharded`).
    self.mod = dict(mod) if mod else None


def _rank_world(group=None) -> tuple[int, int]:
  if dist.is_available() and dist.is_initialized():
    return dist.get_rank(group), dist.get_world_size(group)
  return 0, 1


def _barrier(group=None):
  if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
    dist.barrier(group=group)


def is_step_dir(name: str) -> bool:
  return name.isdigit()


def all_steps(directory: str) -> list[int]:
  if not os.path.isdir(directory):
    return []
  return sorted(int(n) for n in os.listdir(directory)
                if is_step_dir(n) and os.path.isdir(os.path.join(directory, n)))


def latest_step(directory: str) -> int | None:
  steps = all_steps(directory)
  return steps[-1] if steps else None


class CheckpointManager:
  def __init__(self, directory: str, *, max_to_keep: int | None = 5,
               should_save_fn: Callable[[int, int | None], bool] | None = None,
               save_interval_steps: int = 1, async_save: bool = True,
               item_name: str = "state", compressor: str | None = None, group=None, use_ocdbt: bool = False,
               commit_timeout_s: float = 1800.0):
    self.directory = os.fspath(directory)
    self.max_to_keep = max_to_keep
    self.should_save_fn = should_save_fn
    self.save_interval_steps = save_interval_steps
    self.async_save = async_save
    self.item_name = item_name
    self.compressor = compressor
    self.group = group
    # True: every item is written as an OCDBT store (the reference's default: `manifest.ocdbt`, `d/`, one
    # `ocdbt.process_<rank>` store per writing rank) instead of one directory per array.  Reading detects
    # the form by itself.
    self.use_ocdbt = use_ocdbt
    # how long rank 0 waits for the other ranks' shards (and they for its commit) in a multi-rank asynchronous save
    self.commit_timeout_s = commit_timeout_s
    self._thread: threading.Thread | None = None
    self._error: BaseException | None = None
    self._last_saved: int | None = None
    self._seq = 0
    rank, _ = _rank_world(group)
    if rank == 0:
      os.makedirs(self.directory, exist_ok=True)
    _barrier(group)

  # -- queries ----------------------------------------------------------------------
  def all_steps(self) -> list[int]:
    return all_steps(self.directory)

  def latest_step(self) -> int | None:
    return latest_step(self.directory)

  def should_save(self, step: int) -> bool:
    if self.should_save_fn is not None:
      return bool(self.should_save_fn(step, self._last_saved))
    return step % self.save_interval_steps == 0

  # -- save ---------------------------------------------------------------------------
  def save(self, step: int, state: Mapping[str, Any], *, metrics: Mapping[str, Any] | None = None,
           force: bool = False) -> bool:
    if not force and not self.should_save(step):
      return False
    self.wait_until_finished()
    rank, world = _rank_world(self.group)
    # Snapshot to host NOW (the step may mutate the tensors right after we return): device tensors are copied
    # to the host anyway; tensors that live in host memory are copied too when the files are written in the
    # background, or the writer would read them while the next steps change them
    snapshot = self.async_save
    staged: list[tuple[tuple[str, ...], Any]] = []
    for path, leaf in tree_lib.flatten(state):
      if isinstance(leaf, ShardedLeaf):
        arr, dt = zarr_io.to_host_numpy(leaf.local, copy=snapshot) if leaf.write else (None, None)
        staged.append((path, ("sharded", leaf, arr, dt,
                              zarr_io.to_host_numpy(leaf.local[:0])[1])))
      elif rank == 0:
        staged.append((path, ("full",) + zarr_io.to_host_numpy(leaf, copy=snapshot)))
      else:
        staged.append((path, ("skip",)))
    kinds = tree_lib.key_types(state)
    self._seq += 1
    tmp = os.path.join(self.directory, f"{step}{TMP_MARK}{self._seq}")
    final = os.path.join(self.directory, str(step))
    if rank == 0:
      if os.path.exists(final):
        shutil.rmtree(final)
      os.makedirs(os.path.join(tmp, self.item_name), exist_ok=True)
    _barrier(self.group)

    def work():
      try:
        self._write(tmp, staged, kinds, metrics, rank, world)
      except BaseException as e:  # surfaced by wait_until_finished
        self._error = e

    if self.async_save and world == 1:
      self._thread = threading.Thread(target=lambda: (work(), self._finalize(step, tmp, final)),
                                      name="recml-ckpt", daemon=True)
      self._thread.start()
    elif self.async_save:
      self._thread = threading.Thread(target=self._write_and_agree, args=(step, tmp, final, rank, world, work),
                                      name="recml-ckpt", daemon=True)
      self._thread.start()
    else:
      work()
      ok = self._all_ranks_ok(self._error is None)
      if rank == 0:
        if ok:
          self._finalize(step, tmp, final)
        else:
          shutil.rmtree(tmp, ignore_errors=True)
      _barrier(self.group)
      err, self._error = self._error, None
      if not ok:
        if err is not None:
          raise err
        raise RuntimeError(f"checkpoint {step}: another rank failed to write its shards; nothing was committed")
    self._last_saved = step
    return True

  def _write_and_agree(self, step, tmp, final, rank, world, work) -> None:
    """The background half of a multi-rank asynchronous save.  No collective runs off the main thread: every
    rank leaves a marker file in the temporary directory when its shards are written (or failed), rank 0 commits
    once all markers say ok and removes the directory otherwise, and the other ranks learn the outcome from the
    directory names.  The ranks must see one file system (one node, or a shared mount)."""
    work()
    kind = "ok" if self._error is None else "failed"
    try:
      with open(os.path.join(tmp, f".rank_{rank}.{kind}"), "w"):
        pass
    except OSError as e:
      self._error = self._error or e
    deadline = time.time() + self.commit_timeout_s
    nothing = RuntimeError(f"checkpoint {step}: a rank failed to write its shards (or did not finish within "
                           f"{self.commit_timeout_s:.0f} s); nothing was committed")
    if rank == 0:
      done, failed = [], []
      while time.time() <= deadline:
        names = os.listdir(tmp) if os.path.isdir(tmp) else []
        done = [n for n in names if n.startswith(".rank_") and n.endswith(".ok")]
        failed = [n for n in names if n.startswith(".rank_") and n.endswith(".failed")]
        if failed or len(done) == world:
          break
        time.sleep(0.01)
      if len(done) == world and not failed and self._error is None:
        for n in done:
          os.remove(os.path.join(tmp, n))
        self._finalize(step, tmp, final)
      else:
        shutil.rmtree(tmp, ignore_errors=True)
        self._error = self._error or nothing
      return
    while time.time() <= deadline:
      if os.path.isdir(final) and not os.path.isdir(tmp):
        return                                       # committed
      if not os.path.isdir(tmp):
        self._error = self._error or nothing         # rank 0 gave up
        return
      time.sleep(0.01)
    self._error = self._error or nothing

  def _all_ranks_ok(self, ok: bool) -> bool:
    """True when every rank of the group reports success (also a barrier)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(self.group) == 1:
      return ok
    flags: list[Any] = [None] * dist.get_world_size(self.group)
    dist.all_gather_object(flags, bool(ok), group=self.group)
    return all(flags)

  def _write(self, tmp, staged, kinds, metrics, rank, world):
    item = os.path.join(tmp, self.item_name)
    meta_tree, sharding = {}, {}
    pending = []     # (array dir, chunk index, array): written together by the native chunk writer
    for path, rec in staged:
      key = ".".join(path)
      leaf_dir = os.path.join(item, key)
      if rec[0] == "full":
        _, arr, dt = rec
        zarr_io.write_zarray(leaf_dir, arr.shape, arr.shape, dt, self.compressor)
        pending.append((leaf_dir, [0] * arr.ndim, arr))
        meta_tree[key] = {"key_path": list(path), "shape": list(arr.shape), "dtype": dt,
                          "value_type": "array"}
        sharding[key] = {"sharding_type": "replicated"}
      elif rec[0] == "sharded":
        _, leaf, arr, dt, dt_all = rec
        if rank == 0:
          zarr_io.write_zarray(leaf_dir, leaf.global_shape, leaf.chunk_shape, dt_all,
                               self.compressor)
        else:
          os.makedirs(leaf_dir, exist_ok=True)
        if arr is not None:
          if tuple(arr.shape) != leaf.chunk_shape:  # edge block: pad to the chunk shape
            full = np.zeros(leaf.chunk_shape, dtype=arr.dtype)
            full[tuple(slice(0, s) for s in arr.shape)] = arr
            arr = full
          pending.append((leaf_dir, leaf.grid_index, arr))
        meta_tree[key] = {"key_path": list(path), "shape": list(leaf.global_shape),
                          "dtype": dt_all, "value_type": "array"}
        sharding[key] = {"sharding_type": "block", "chunk_shape": list(leaf.chunk_shape)}
        if leaf.mod:
          sharding[key]["mod"] = leaf.mod
    if self.use_ocdbt:
      self._write_ocdbt(item, pending, rank, world)
    else:
      zarr_io.write_chunks_parallel(pending, self.compressor)
    if rank == 0:
      with open(os.path.join(item, TREE_METADATA), "w") as f:
        json.dump({"tree_metadata": meta_tree,
                   "containers": {".".join(k): v for k, v in kinds.items()},
                   "use_zarr3": False, "use_ocdbt": bool(self.use_ocdbt)}, f)
      with open(os.path.join(item, SHARDING_FILE), "w") as f:
        json.dump(sharding, f)
      if metrics is not None:
        os.makedirs(os.path.join(tmp, "metrics"), exist_ok=True)
        with open(os.path.join(tmp, "metrics", "metrics"), "w") as f:
          json.dump(_jsonable(metrics), f)
      with open(os.path.join(tmp, CHECKPOINT_METADATA), "w") as f:
        json.dump({"item_handlers": {self.item_name: "recml_b200.ckpt.PyTreeZarr",
                                     **({"metrics": "json"} if metrics is not None else {})},
                   "metrics": _jsonable(metrics or {}),
                   "init_timestamp_nsecs": time.time_ns(),
                   "commit_timestamp_nsecs": time.time_ns()}, f)

  def _write_ocdbt(self, item, pending, rank, world):
    """This rank's chunks (and, on rank 0, every array's `.zarray`) as the store `ocdbt.process_<rank>` of the
    item; rank 0 also writes the item's own (empty) manifest, whose presence marks the item as an OCDBT one.
    The `.zarray` files that `_write` put into per-array directories are folded in and removed."""
    from recml_b200.ckpt import ocdbt
    import glob
    w = ocdbt.Writer(os.path.join(item, f"ocdbt.process_{rank}"))
    if rank == 0:
      for meta in glob.glob(os.path.join(item, "*", ".zarray")):
        key = os.path.basename(os.path.dirname(meta))
        with open(meta, "rb") as f:
          w.add(f"{key}/.zarray", f.read())
    for leaf_dir, index, arr in pending:
      key = f"{os.path.basename(leaf_dir)}/{zarr_io.chunk_name(index)}"
      if self.compressor == "zstd":
        w.add(key, zarr_io.zstd_compress(arr))
      else:
        w.add_array(key, arr)           # written from the array's own memory at the commit
    w.commit(compress_nodes=zarr_io.zstd_available())
    if rank == 0:
      ocdbt.Writer(item).commit(compress_nodes=False)
    if world == 1:
      self._drop_array_dirs(item)

  @staticmethod
  def _drop_array_dirs(item):
    for name in os.listdir(item):
      d = os.path.join(item, name)
      if os.path.isdir(d) and not name.startswith("ocdbt.process_") and name != "d":
        shutil.rmtree(d, ignore_errors=True)

  def _finalize(self, step, tmp, final):
    if self._error:
      return
    if self.use_ocdbt:        # every rank has folded the per-array directories into its store by now
      self._drop_array_dirs(os.path.join(tmp, self.item_name))
    with open(os.path.join(tmp, COMMIT_FILE), "w") as f:
      f.write("Checkpoint commit was successful.")
    os.replace(tmp, final)
    self._gc()

  def _gc(self):
    if self.max_to_keep is None:
      return
    steps = self.all_steps()
    for s in steps[:max(0, len(steps) - self.max_to_keep)]:
      shutil.rmtree(os.path.join(self.directory, str(s)), ignore_errors=True)

  def wait_until_finished(self) -> None:
    if self._thread is not None:
      self._thread.join()
      self._thread = None
    if self._error:
      err, self._error = self._error, None
      raise err

  def close(self) -> None:
    self.wait_until_finished()

  # -- restore ----------------------------------------------------------------------
  def restore(self, step: int | None = None, target: Mapping[str, Any] | None = None,
              item_name: str | None = None) -> Any:
    """Reads a step.  Without `target` returns the stored tree of host tensors.  With a
    `target` tree (same structure) only those leaves are read; a `ShardedLeaf` target
    reads just its own block of the global array, so a checkpoint written by W ranks
    restores on any other world size."""
    self.wait_until_finished()
    if step is None:
      step = self.latest_step()
      if step is None:
        raise FileNotFoundError(f"No checkpoints under {self.directory}")
    return restore_tree(os.path.join(self.directory, str(step), item_name or self.item_name), target)

  def metrics(self, step: int) -> Any:
    with open(os.path.join(self.directory, str(step), "metrics", "metrics")) as f:
      return json.load(f)


def restore_tree(item: str, target: Mapping[str, Any] | None = None) -> Any:
  if not os.path.exists(os.path.join(item, TREE_METADATA)):
    raise FileNotFoundError(f"{item} is not a complete checkpoint item")
  with open(os.path.join(item, TREE_METADATA)) as f:
    meta = json.load(f)
  from recml_b200.ckpt import ocdbt
  in_store = ocdbt.is_store(item)
  leaf_at = (lambda key: ocdbt.leaf_path(item, key)) if in_store else (lambda key: os.path.join(item, key))
  if target is None:
    leaves = {tuple(m["key_path"]): zarr_io.read_region(leaf_at(key))
              for key, m in meta["tree_metadata"].items()}
    kinds = {tuple(k.split(".")) if k else (): v for k, v in meta.get("containers", {}).items()}
    return tree_lib.restore_containers(tree_lib.unflatten(leaves), kinds)
  out = {}
  sharding_meta = {}
  if os.path.exists(os.path.join(item, SHARDING_FILE)):
    with open(os.path.join(item, SHARDING_FILE)) as f:
      sharding_meta = json.load(f)
  for path, leaf in tree_lib.flatten(target):
    key = ".".join(path)
    if key not in meta["tree_metadata"]:
      raise KeyError(f"Checkpoint has no leaf {key!r}")
    leaf_dir = leaf_at(key)
    if isinstance(leaf, ShardedLeaf):
      stored_shape = tuple(zarr_io.read_meta(leaf_dir)["shape"])
      stored_mod = (sharding_meta.get(key) or {}).get("mod")
      if stored_shape != leaf.global_shape or (stored_mod is None) != (leaf.mod is None):
        out[path] = _read_resharded(leaf_dir, stored_shape, stored_mod, leaf)
        continue
      start = [i * c for i, c in zip(leaf.grid_index, leaf.chunk_shape)]
      stop = [min(s + c, g) for s, c, g in zip(start, leaf.chunk_shape, leaf.global_shape)]
      out[path] = zarr_io.read_region(leaf_dir, start, stop)
    else:
      out[path] = zarr_io.read_region(leaf_dir)
  return tree_lib.restore_containers(tree_lib.unflatten(out), tree_lib.key_types(target))


def _read_resharded(leaf_dir: str, stored_shape, stored_mod, leaf: ShardedLeaf) -> torch.Tensor:
  """This rank's block of a row-sharded array whose layout on disk differs from the target's.

  MOD layout is `[W, ceil(V / W), ...]`, block b = rows with id % W == b at position id // W; the logical
  layout is `[V, ...]`.  Handled: MOD(W) -> MOD(W'), MOD(W) -> logical row block, logical -> MOD(W').  An id
  lies in stored block b and in wanted residue class r of W' iff id = b (mod W) and id = r (mod W'), which
  has solutions only when b = r modulo gcd(W, W'), so only those blocks are read."""
  import math
  nd = len(stored_shape)
  dtype = zarr_io.read_region(leaf_dir, [0] * nd, [0] * nd).dtype
  if stored_mod is not None:
    vocab, w_old = int(stored_mod["vocab"]), int(stored_shape[0])
    tail = tuple(stored_shape[2:])

    def blocks(keep_block):
      for b in range(w_old):
        n_b = (vocab - b + w_old - 1) // w_old if vocab > b else 0      # rows of block b that exist
        if n_b == 0 or not keep_block(b):
          continue
        block = zarr_io.read_region(leaf_dir, [b, 0] + [0] * len(tail), [b + 1, n_b] + list(tail))[0]
        yield b + torch.arange(n_b, dtype=torch.int64) * w_old, block

    if leaf.mod is not None:                                   # MOD(W) -> MOD(W')
      w_new, rows_new, r = leaf.global_shape[0], leaf.global_shape[1], leaf.grid_index[0]
      out = torch.zeros((1, rows_new) + tail, dtype=dtype)
      g = math.gcd(w_old, w_new)
      for ids, block in blocks(lambda b: (b - r) % g == 0):
        keep = (ids % w_new) == r
        out[0, ids[keep] // w_new] = block[keep]
      return out
    if leaf.global_shape != (vocab,) + tail:
      raise ValueError(f"{leaf_dir}: stored MOD layout of a [{vocab}, ...] table does not fit target "
                       f"{leaf.global_shape}")
    start = leaf.grid_index[0] * leaf.chunk_shape[0]            # MOD(W) -> rows [start, stop) of the table
    stop = min(start + leaf.chunk_shape[0], vocab)
    out = torch.zeros((stop - start,) + tail, dtype=dtype)
    for ids, block in blocks(lambda b: True):
      keep = (ids >= start) & (ids < stop)
      out[ids[keep] - start] = block[keep]
    return out
  if leaf.mod is None or tuple(stored_shape[1:]) != tuple(leaf.global_shape[2:]):
    raise ValueError(f"{leaf_dir} was stored with global shape {tuple(stored_shape)}, the target expects "
                     f"{leaf.global_shape}; only row-sharded (MOD) leaves can change their world size")
  w_new, rows_new, r = leaf.global_shape[0], leaf.global_shape[1], leaf.grid_index[0]   # logical -> MOD(W')
  full = zarr_io.read_region(leaf_dir)
  mine = full[r::w_new]
  out = torch.zeros((1, rows_new) + tuple(stored_shape[1:]), dtype=dtype)
  out[0, :mine.shape[0]] = mine
  return out


def _jsonable(x: Any) -> Any:
  if isinstance(x, Mapping):
    return {str(k): _jsonable(v) for k, v in x.items()}
  if isinstance(x, (list, tuple)):
    return [_jsonable(v) for v in x]
  if isinstance(x, torch.Tensor):
    x = x.detach().cpu().numpy()
  if isinstance(x, np.ndarray):
    return x.tolist()
  if isinstance(x, (np.floating, np.integer)):
    return x.item()
  return x


def checkpoints_iterator(directory: str, *, timeout: float | None = None,
                         timeout_fn: Callable[[], bool] | None = None,
                         min_interval_secs: float = 0.0,
                         poll_secs: float = 0.5) -> Iterator[int]:
  """Yields each new complete step as it appears.  After `timeout` seconds without a
  new step, `timeout_fn()` is asked: True ends the iteration, False keeps waiting
  (the reference's `ocp.checkpoint_utils.checkpoints_iterator`, used by continuous
  evaluation `jax_trainer.py:871-875`)."""
  last: int | None = None
  while True:
    deadline = None if timeout is None else time.time() + timeout
    found = None
    while True:
      steps = [s for s in all_steps(directory) if last is None or s > last]
      if steps:
        found = steps[-1] if last is None and False else steps[0]
        break
      if deadline is not None and time.time() >= deadline:
        break
      time.sleep(poll_secs)
    if found is None:
      if timeout_fn is None or timeout_fn():
        # one last look so a step committed right before the marker is not lost
        steps = [s for s in all_steps(directory) if last is None or s > last]
        if not steps:
          return
        found = steps[0]
      else:
        continue
    last = found
    start = time.time()
    yield found
    rest = min_interval_secs - (time.time() - start)
    if rest > 0:
      time.sleep(rest)
