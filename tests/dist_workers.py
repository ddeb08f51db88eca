"""Worker functions executed by every rank of the multi-process tests (importable module so that
`torch.multiprocessing.spawn` can pickle them)."""
import os
import sys
import traceback

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _init(rank, world, backend, port):
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                    LOCAL_RANK=str(rank))
  if backend == "nccl":
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
  else:
    dist.init_process_group("gloo", rank=rank, world_size=world)


def entry(rank, world, backend, port, fn_name, args, result_dir):
  try:
    _init(rank, world, backend, port)
    out = globals()[fn_name](rank, world, *args)
    torch.save(out, os.path.join(result_dir, f"rank{rank}.pt"))
  except Exception:  # pylint: disable=broad-except
    with open(os.path.join(result_dir, f"rank{rank}.err"), "w") as f:
      f.write(traceback.format_exc())
    raise
  finally:
    if dist.is_initialized():
      try:
        dist.barrier()
        dist.destroy_process_group()
      except Exception:  # pylint: disable=broad-except
        pass


def save_row_wise_tables(rank, world, device_type, ckpt_dir, fail_rank, use_ocdbt=False):
  """Trains a row-sharded (MOD) embedding for two steps and checkpoints it.  With `fail_rank` >= 0 that
  rank's chunk writer raises, and the save must commit nothing on any rank."""
  from recml_b200 import ckpt, embedding as emb
  from recml_b200.ckpt import zarr_io
  specs = {"a": emb.EmbeddingSpec(37, 8, combiner="sum"), "b": emb.EmbeddingSpec(10, 8, combiner="sum")}
  cfg = emb.ShardedEmbeddingConfig(specs, emb.AdagradOptimizerSpec(learning_rate=0.1), sharding_strategy="MOD",
                                   backend="collective")
  m = emb.ShardedEmbedding(cfg, device="cpu")
  gen = np.random.default_rng(rank)
  for _ in range(2):
    feats = {k: [gen.integers(0, s.input_dim, size=3).tolist() for _ in range(4)] for k, s in specs.items()}
    out = m(emb.KeyedJagged.from_lists(feats))
    (out if isinstance(out, torch.Tensor) else sum(o.sum() for o in out.values())).sum().backward()
  mgr = ckpt.CheckpointManager(ckpt_dir, async_save=False, use_ocdbt=use_ocdbt)
  mgr.save(1, {"sharded": m.sharded_state_dict()})           # a good checkpoint first
  raised = None
  if fail_rank >= 0:
    real = zarr_io.write_chunks_parallel
    if rank == fail_rank:
      def boom(*a, **k):
        raise IOError("disk full (injected)")
      zarr_io.write_chunks_parallel = boom
    try:
      mgr.save(2, {"sharded": m.sharded_state_dict()})
    except Exception as e:  # pylint: disable=broad-except
      raised = type(e).__name__
    zarr_io.write_chunks_parallel = real
  tables = {n: m.gather_table(n) for n in specs}
  slots = {n: m.gather_table(n, "accumulator") for n in specs}
  return {"tables": tables, "slots": slots, "raised": raised, "steps": mgr.all_steps(),
          "listing": sorted(os.listdir(ckpt_dir))}


def async_multi_rank_save(rank, world, device_type, ckpt_dir, fail_rank):
  """An asynchronous save from two ranks: `save` returns while a (slowed) writer thread still runs, the tensors
  change meanwhile, and the committed checkpoint holds what they were at the call.  With `fail_rank` >= 0 that
  rank's writer raises: nothing is committed and every rank raises at `wait_until_finished`."""
  import time
  from recml_b200 import ckpt
  from recml_b200.ckpt import zarr_io
  local = torch.full((4, 3), float(rank + 1))
  whole = torch.arange(6, dtype=torch.float32)
  tree = lambda: {"shard": ckpt.ShardedLeaf(local, (4 * world, 3), (rank, 0)), "whole": whole}
  mgr = ckpt.CheckpointManager(ckpt_dir, async_save=True, commit_timeout_s=30.0)
  real = zarr_io.write_chunks_parallel
  def slow(*a, **k):
    time.sleep(1.0 if rank == 1 else 0.05)
    if rank == fail_rank:
      raise IOError("disk full (injected)")
    return real(*a, **k)
  zarr_io.write_chunks_parallel = slow
  torch.distributed.barrier()        # both ranks enter the save together: the timing below is the save's own
  t = time.time()
  mgr.save(1, tree())
  returned_after = time.time() - t
  local.add_(100.0)                  # training goes on while the files are written
  whole.add_(100.0)
  raised = None
  try:
    mgr.wait_until_finished()
  except Exception as e:  # pylint: disable=broad-except
    raised = f"{type(e).__name__}: {e}"
  zarr_io.write_chunks_parallel = real
  torch.distributed.barrier()
  out = {"returned_after": returned_after, "raised": raised, "steps": mgr.all_steps(),
         "listing": sorted(os.listdir(ckpt_dir))}
  if raised is None:
    back = mgr.restore(1, target=tree())
    out["shard"], out["whole"] = back["shard"], back["whole"]
  return out


class _ToyNet(torch.nn.Module):
  def __init__(self, tp_group=None):
    super().__init__()
    from recml_b200.layers import dense, parallel
    torch.manual_seed(0)
    self.a = dense.Linear(8, 16, activation="relu")
    self.b = dense.Linear(16, 16, activation="relu")
    self.tp = parallel.TensorParallelMLP(16, 32, 16, group=tp_group) if tp_group != "none" else None
    self.c = dense.Linear(16, 1)

  def forward(self, x):
    h = self.b(self.a(x))
    if self.tp is not None:
      h = h + self.tp(h)
    return self.c(h).reshape(-1)


def _toy_batches(steps, n):
  g = torch.Generator().manual_seed(7)
  return [(torch.randn(n, 8, generator=g), torch.randn(n, generator=g)) for _ in range(steps)]


def sharded_state_training(rank, world, device_type, axes, dp_axes, rules, steps, ckpt_dir, with_tp):
  """Trains a small MLP whose parameters are sharded by `rules` over the mesh `axes`; returns the final
  FULL parameters (gathered) and the loss history, for comparison with a replicated single-process run."""
  from recml_b200 import ckpt
  from recml_b200.training import optim_factory, partitioning, state as state_lib
  dev = torch.device("cuda", rank) if device_type == "cuda" else torch.device("cpu")
  part = partitioning.ModelParallelPartitioner(axes, dp_axes=dp_axes, rules=rules, device=dev) if world > 1 or axes \
      else partitioning.NullPartitioner(dev)
  tp_group = part.axis_group("model") if (with_tp and hasattr(part, "axis_group")) else (None if with_tp else "none")
  factory = optim_factory.AdamFactory(learning_rate=1e-2, grad_clip_norm=1.0)
  state = part.partition_init(lambda b: state_lib.State.create(model=_ToyNet(tp_group).to(dev), tx=factory.make()))(None)
  dp = getattr(part, "dp_size", 1)
  # data-parallel rank = position along the data axes (ranks along "model" see the same slice)
  dp_rank = 0
  if hasattr(part, "coords"):
    for a in part.dp_axis_names:
      dp_rank = dp_rank * part.axis_size(a) + part.coords[a]
  losses = []

  def train_step(batch, st):
    x, y = batch
    loss = ((st.model(x) - y) ** 2).mean()
    loss.backward()
    st.update()
    return st, loss.detach()

  step = part.partition_step(train_step, training=True)
  n = 16
  for x, y in _toy_batches(steps, n):
    sl = slice(dp_rank * n // dp, (dp_rank + 1) * n // dp)
    state, loss = step((x[sl].to(dev), y[sl].to(dev)), state)
    losses.append(float(loss))
  shapes = {k: tuple(p.shape) for k, p in state.params.items()}
  slot_shapes = {k: tuple(t.shape) for k, t in zip(state.optimizer.names, state.optimizer.slots["mu"])}
  restored_ok = None
  if ckpt_dir:
    mgr = ckpt.CheckpointManager(ckpt_dir, async_save=False)
    mgr.save(steps, state.state_dict())
    before = {k: p.detach().clone() for k, p in state.params.items()}
    with torch.no_grad():
      for p in state.params.values():
        p.zero_()
    state.load_state_dict(mgr.restore(steps, target=state.state_dict()))
    # shards come back bit-exact; replicated leaves are rank 0's copy, equal up to float reassociation
    restored_ok = all(torch.allclose(before[k], p, rtol=1e-5, atol=1e-7) for k, p in state.params.items()) and all(
        torch.equal(before[k], p) for k, p in state.params.items() if getattr(p, "_recml_partitioned", False))
    stored = {k: tuple(v.shape) for k, v in mgr.restore(steps)["params"].items()} if rank == 0 else None
  else:
    stored = None
  if hasattr(part, "gather_params"):
    part.gather_params()
  full = {k: p.detach().cpu().clone() for k, p in state.model.named_parameters() if "tp." not in k}
  return {"losses": losses, "full": full, "shapes": shapes, "slot_shapes": slot_shapes, "restored_ok": restored_ok,
          "stored": stored}


def leave_entry(rank, world, port, result_dir, announce):
  """A job whose last rank leaves between steps (host-side failure: no GPU involved).  With `announce`
  it tells the store first; without, it just exits.  Every rank exits through os._exit so that nobody
  waits in a barrier for a rank that is gone."""
  import datetime
  import time
  from recml_b200.comm import health
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
  dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
  store = dist.distributed_c10d._get_default_store()   # pylint: disable=protected-access
  mon = health.HealthMonitor(store, rank, world, interval_s=0.05, timeout_s=1.0).start()
  out = {"steps_done": 0, "detected": None, "collective_error": None, "seconds": None}
  t = torch.ones(4)
  leave_step = 3
  t0 = time.time()
  try:
    for step in range(200):
      mon.check(step)                       # host check BEFORE anything that waits for peers
      leaving = rank == world - 1 and step == leave_step
      if leaving and announce:
        # announced one step ahead: the leaver still takes part in this step's collective, which no peer can
        # finish before the announcement is in the store, so every peer sees it at its next check
        mon.leave()
      elif leaving:
        torch.save({"left_at": step}, os.path.join(result_dir, f"rank{rank}.pt"))
        os._exit(0)
      try:
        dist.all_reduce(t)
        if leaving:
          torch.save({"left_at": step}, os.path.join(result_dir, f"rank{rank}.pt"))
          os._exit(0)
      except Exception as e:  # the peer's socket closed or the process-group timeout ran out
        out["collective_error"] = type(e).__name__
        t0 = time.time()
        while True:                         # the heartbeat names the culprit once it has been silent long enough
          mon.check(step)
          time.sleep(0.05)
          if time.time() - t0 > 10:
            break
        break
      out["steps_done"] += 1
      time.sleep(0.02)
  except health.PeerFailure as e:
    out["detected"], out["seconds"] = list(e.ranks), time.time() - t0
  torch.save(out, os.path.join(result_dir, f"rank{rank}.pt"))
  os._exit(0)


# ---------------------------------------------------------------------------------------------------
def _emb_specs():
  from recml_b200 import embedding as emb
  vocabs = [50, 3000, 7, 400]
  combs = ["sum", "sum", "mean", "sqrtn"]
  return vocabs, {f"f{i}": emb.EmbeddingSpec(v, 64, combiner=c) for i, (v, c) in enumerate(zip(vocabs, combs))}


def _global_batch(seed, B_global, vocabs, bags):
  from recml_b200 import embedding as emb
  from recml_b200.data import synthetic
  rng = np.random.default_rng(seed)
  feats = {f"f{i}": [synthetic.zipf_ids(rng, v, (int(rng.integers(0, b + 1)),), 1.05).tolist()
                     for _ in range(B_global)] for i, (v, b) in enumerate(zip(vocabs, bags))}
  return feats


def sharded_embedding_steps(rank, world, device_type, backend_name, placements, opt_kind, steps):
  """Runs `steps` lookups + updates with the requested placements; returns this rank's outputs of
  every step and the final un-sharded tables."""
  from recml_b200 import embedding as emb
  vocabs, specs = _emb_specs()
  bags = [3, 9, 2, 5]
  P = emb.Placement
  overrides = {f"f{i}": P(p) for i, p in enumerate(placements)}
  opt = {"rowwise_adagrad": emb.RowWiseAdagradOptimizerSpec(0.1), "adam": emb.AdamOptimizerSpec(0.02),
         "sgd": emb.SGDOptimizerSpec(0.1)}[opt_kind]
  device = torch.device("cuda", rank) if device_type == "cuda" else torch.device("cpu")
  cfg = emb.ShardedEmbeddingConfig(specs, opt, placement_overrides=overrides, backend=backend_name, seed=5)
  m = emb.ShardedEmbedding(cfg, device=device)
  m.grad_scale = 1.0   # the test feeds identical per-sample gradients for every world size
  outs = []
  B_global = 32 * world if world > 1 else 64
  if world == 1:
    B_global = 64
  for step in range(steps):
    feats = _global_batch(100 + step, 64, vocabs, bags)     # same 64-sample global batch for any world
    per = 64 // world
    mine = {k: v[rank * per:(rank + 1) * per] for k, v in feats.items()}
    kjt = emb.KeyedJagged.from_lists(mine).to_device(device)
    out = m(kjt)
    g = torch.from_numpy(np.random.default_rng(500 + step).normal(size=(64, len(specs), 64)).astype(np.float32))
    g = (g * 0.1).to(torch.bfloat16).float()[rank * per:(rank + 1) * per]
    out.backward(g.to(device).to(out.dtype))
    outs.append(out.detach().float().cpu())
  if device.type == "cuda":
    torch.cuda.synchronize()
    from recml_b200.ops import _lib
    _lib.check_status(device)
  backend = getattr(m, "_backend", None)
  if world > 1 and hasattr(backend, "partition_stats"):
    # the bucketizing id push counted, per row-sharded feature, the ids it sent to every owner
    stats = backend.partition_stats()
    for fname, per_owner in stats.items():
      tp = m.plan.tables[m.feature_to_table[fname]]
      ids = np.concatenate([np.asarray(r, dtype=np.int64) for r in mine[fname]]) if len(mine[fname]) else np.zeros(0, np.int64)
      want = [int(((ids % world + tp.rotation) % world == r).sum()) for r in range(world)]
      assert per_owner == want, (fname, per_owner, want)
  tables = {n: m.gather_table(n).cpu() for n in m.plan.tables}
  return {"outs": outs, "tables": tables}


def allreduce_grads(rank, world, device_type, sizes, nvls=None):
  """Fused NVLink reducer (CUDA) / flat-bucket reducer (CPU) vs a plain all_reduce mean.  `nvls`
  forces the in-switch (`multimem`) reduce step on or off; None keeps the default."""
  from recml_b200.comm import grad_reducer
  device = torch.device("cuda", rank) if device_type == "cuda" else torch.device("cpu")
  gen = torch.Generator().manual_seed(17 + rank)
  params = [torch.zeros(s, device=device, requires_grad=True) for s in sizes]
  results = []
  red = grad_reducer.make_reducer(None, device)
  if nvls is not None and hasattr(red, "use_nvls"):
    red.use_nvls = bool(nvls)
  for it in range(3):
    for p in params:
      p.grad = torch.randn(p.shape, generator=gen).to(device)
    ref = []
    for p in params:
      t = p.grad.clone()
      dist.all_reduce(t)
      ref.append(t / world)
    red.average_grads(params)
    if device.type == "cuda":
      torch.cuda.synchronize()
    results.append(max(float((p.grad - r).abs().max() / (r.abs().max() + 1e-6)) for p, r in zip(params, ref)))
  ms = None
  if device.type == "cuda":
    from recml_b200.ops import _lib
    _lib.check_status(device)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    dist.barrier()
    torch.cuda.synchronize()
    ev[0].record()
    for _ in range(10):
      red.average_grads(params)
    ev[1].record()
    torch.cuda.synchronize()
    _lib.check_status(device)
    ms = ev[0].elapsed_time(ev[1]) / 10
  buf = getattr(red, "buf", None)
  return {"max_rel_err": results, "reducer": type(red).__name__, "ms": ms,
          "multicast": bool(buf is not None and buf.multicast_ptr), "nvls": getattr(red, "use_nvls", False)}


def dlrm_tiny_training(rank, world, device_type, steps, use_graph=False):
  """BASELINE config 1 (tiny DLRM-DCNv2) as a data-parallel + sharded-embedding job."""
  import tempfile
  from recml_b200 import config as C, run_experiment
  from recml_b200.examples import dlrm_experiment as D
  d = tempfile.mkdtemp() if rank == 0 else None
  box = [d]
  dist.broadcast_object_list(box, src=0)
  cfg = D.tiny_experiment(model_dir=box[0], train_steps=steps, batch_size=256)
  if device_type == "cpu":
    cfg.trainer.partitioner = C.Config(__import__("recml_b200").DataParallelPartitioner, device="cpu")
  if use_graph:
    cfg.trainer.partitioner = C.Config(__import__("recml_b200").DataParallelPartitioner, use_cuda_graph=True)
  exp = C.build(cfg)
  logs = run_experiment(exp, "train_and_eval")
  import os as _os
  return {"loss": float(logs["train"]["loss"]), "val_loss": float(logs["val"]["loss"]),
          "ckpts": sorted(_os.listdir(_os.path.join(box[0], "checkpoints")))}


def q_sharded_attention(rank, world, device_type):
  """Sequence-sharded HSTU attention on `world` ranks: this rank's output rows and input gradients."""
  from recml_b200.ops import hstu_attention as A
  g = torch.Generator().manual_seed(3)
  B, L, H, Dh = 2, 24, 2, 8
  q, k, v = (torch.randn(B, L, H, Dh, generator=g) for _ in range(3))
  seg = torch.tensor([[0] * 10 + [1] * 14, [0] * 24])
  go = torch.randn(B, L, H, Dh, generator=g)
  n = L // world
  sl = slice(rank * n, (rank + 1) * n)
  leaves = [t[:, sl].clone().requires_grad_() for t in (q, k, v)]
  out = A.q_sharded_pointwise_attention("causal", *leaves, segment_ids=seg[:, sl], sliding_window_size=6, scale=0.3)
  out.backward(go[:, sl])
  return {"out": out.detach(), "grads": [t.grad for t in leaves]}


def dlrm_tiny_export(rank, world, device_type, model_dir):
  """Trains the tiny DLRM on `world` ranks with row-sharded tables; the trainer's final export is collective."""
  from recml_b200 import config as C, run_experiment
  from recml_b200.examples import dlrm_experiment as D
  cfg = D.tiny_experiment(model_dir=model_dir, train_steps=4, batch_size=64)
  cfg.task.model.row_wise_min_bytes = 0          # every table row-wise: shards on both ranks
  cfg.trainer.partitioner = C.Config(__import__("recml_b200").DataParallelPartitioner, device="cpu")
  exp = C.build(cfg)
  run_experiment(exp, "train")
  # the trained module is not returned by the trainer: rebuild it from the last checkpoint
  from recml_b200 import ckpt
  it = exp.task.create_datasets()[0]
  state = exp.task.create_state(next(it), torch.Generator().manual_seed(0))
  mgr = ckpt.CheckpointManager(os.path.join(model_dir, "checkpoints"), async_save=False)
  state.load_state_dict(mgr.restore(mgr.latest_step(), target=state.state_dict()))
  emb_mod = state.model.embedding
  return {"tables": {n: emb_mod.gather_table(n) for n in emb_mod.plan.tables},
          "placements": {n: str(tp.placement) for n, tp in emb_mod.plan.tables.items()}}


def vocab_rank_sharded(rank, world, device_type, rows, D, V):
  """Ranks over a MOD-row-sharded item matrix vs the single-process fp32 ranks."""
  from recml_b200.ops import vocab_rank as VR
  device = torch.device("cuda", rank) if device_type == "cuda" else torch.device("cpu")
  g = torch.Generator().manual_seed(0)
  x_all = (torch.randn(rows * world, D, generator=g) * 0.3).to(torch.bfloat16)
  items = (torch.randn(V, D, generator=g) * 0.3).to(torch.bfloat16)
  target_all = torch.randint(0, V, (rows * world,), generator=g)
  pos_all = (x_all.float() * items[target_all].float()).sum(-1)
  sl = slice(rank * rows, (rank + 1) * rows)
  shard = items[rank::world].contiguous().to(device)        # local row i <-> global id i*world + rank
  ranker = VR.VocabRanker(rows, D, None, device)
  out = None
  for _ in range(2):
    out = ranker.ranks(x_all[sl].to(device), pos_all[sl].to(device), target_all[sl].to(device), shard, world, rank)
  if device.type == "cuda":
    torch.cuda.synchronize()
    from recml_b200.ops import _lib
    _lib.check_status(device)
  s = x_all[sl].float() @ items.float().t()
  ref = 1 + ((s > pos_all[sl][:, None]) & (torch.arange(V)[None] != target_all[sl][:, None])).sum(1)
  near = ((s - pos_all[sl][:, None]).abs() < 2e-3 * s.abs().max()).sum(1)
  return {"max_excess": int(((out.cpu() - ref).abs() - near).max()), "exact": float((out.cpu() == ref).float().mean())}


def sequence_experiment(rank, world, device_type, which, steps):
  import tempfile
  from recml_b200 import config as C, run_experiment
  d = tempfile.mkdtemp() if rank == 0 else None
  box = [d]
  dist.broadcast_object_list(box, src=0)
  if which == "sasrec":
    from recml_b200.examples import sasrec_experiment as E
  else:
    from recml_b200.examples import hstu_experiment as E
  cfg = E.tiny_experiment(model_dir=box[0], train_steps=steps)
  if device_type == "cpu":
    cfg.trainer.partitioner = C.Config(__import__("recml_b200").DataParallelPartitioner, device="cpu")
  logs = run_experiment(C.build(cfg), "train_and_eval")
  return {k: {kk: float(vv) for kk, vv in v.items() if not kk.startswith(("perf", "model", "optimizer"))}
          for k, v in logs.items()}

