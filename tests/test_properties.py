"""Property tests (hypothesis) of host-side invariants: whatever the tables and the world size, the planner
places every table once, stores every row exactly once across the ranks and decides the same on every rank;
the reference stacking layout round-trips and addresses rows as its rule says; the host id partition agrees
with a numpy restatement."""
import os

import numpy as np
import pytest

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st      # noqa: E402

from recml_b200.embedding import id_pipeline as ip, layout_compat as lc, planner as P, specs as S   # noqa: E402


@settings(max_examples=60, deadline=None, derandomize=True)
@given(vocabs=st.lists(st.integers(1, 5_000_000), min_size=1, max_size=12),
       hots=st.lists(st.floats(0.5, 120.0), min_size=12, max_size=12),
       dim=st.sampled_from([8, 64, 128]), world=st.sampled_from([1, 2, 3, 4, 8]),
       replicate=st.sampled_from([0, 100]), budget_gb=st.sampled_from([1, 140]))
def test_planner_places_every_row_once_and_identically_on_every_rank(vocabs, hots, dim, world, replicate, budget_gb):
  opt = S.RowWiseAdagradOptimizerSpec(learning_rate=0.01)
  tables = [S.TableSpec(f"t{i}", v, dim, opt) for i, v in enumerate(vocabs)]
  ids = {t.name: hots[i] for i, t in enumerate(tables)}
  plans = [P.plan_tables(tables, world, r, ids_per_sample=ids, replicate_max_rows=replicate,
                         rank_budget_bytes=budget_gb << 30) for r in range(world)]
  ref = plans[0]
  assert set(ref.tables) == {t.name for t in tables}
  for t in tables:
    tps = [p.tables[t.name] for p in plans]
    assert len({(tp.placement, tp.owner, tp.rotation) for tp in tps}) == 1
    tp = tps[0]
    if tp.placement is P.Placement.REPLICATED:
      assert all(x.local_rows == t.vocabulary_size and x.local_dim == dim for x in tps)
    elif tp.placement is P.Placement.COLUMN_WISE:
      assert sum(x.local_dim for x in tps) == dim and all(x.local_rows == t.vocabulary_size for x in tps)
    else:
      assert sum(x.local_rows for x in tps) == t.vocabulary_size
      assert all(x.local_dim == dim for x in tps if x.local_rows)
    if tp.placement is P.Placement.TABLE_WISE:
      assert 0 <= tp.owner < world and all((x.local_rows > 0) == (r == tp.owner) for r, x in enumerate(tps))
    if tp.placement is P.Placement.ROW_WISE:
      # rank r holds the rows whose id is congruent to (r - rotation) mod world
      for r, x in enumerate(tps):
        q = (r - tp.rotation) % world
        assert x.local_rows == len(range(q, t.vocabulary_size, world))
  # rows of one stack do not overlap on a rank
  for p in plans:
    spans = {}
    for tp in p.tables.values():
      if tp.local_rows and tp.stack >= 0:          # replicated tables are dense parameters outside the stacks
        spans.setdefault(tp.stack, []).append((tp.row_base, tp.row_base + tp.local_rows))
    for spans_of_stack in spans.values():
      spans_of_stack.sort()
      assert all(a[1] <= b[0] for a, b in zip(spans_of_stack, spans_of_stack[1:]))


@settings(max_examples=60, deadline=None, derandomize=True)
@given(shapes=st.lists(st.tuples(st.integers(1, 70), st.integers(1, 9)), min_size=1, max_size=5),
       shards=st.sampled_from([1, 2, 4, 8]), rotation=st.integers(0, 3), seed=st.integers(0, 100))
def test_reference_stack_layout_round_trips_and_addresses_rows(shapes, shards, rotation, seed):
  rng = np.random.default_rng(seed)
  tabs = {f"t{i}": rng.normal(size=s).astype(np.float32) for i, s in enumerate(shapes)}
  lay = lc.stack_layout([(n, *t.shape) for n, t in tabs.items()], num_shards=shards, rotation=rotation)
  stacked = lc.to_reference_stack(lay, tabs)
  back = lc.from_reference_stack(lay, stacked)
  for n, t in tabs.items():
    np.testing.assert_array_equal(back[n], t)
  per_shard = stacked.reshape(shards, lay.rows_per_shard, -1)
  for n, t in tabs.items():
    for row in {0, t.shape[0] // 2, t.shape[0] - 1}:
      shard, local = lc.reference_location(lay, n, row)
      np.testing.assert_array_equal(per_shard[shard, local, :t.shape[1]], t[row])


@settings(max_examples=60, deadline=None, derandomize=True)
@given(lens=st.lists(st.integers(0, 6), min_size=1, max_size=30), shards=st.integers(1, 8), rotation=st.integers(0, 7),
       vocab=st.integers(1, 50), cap=st.integers(0, 6), seed=st.integers(0, 1000), weighted=st.booleans())
def test_id_partition_matches_a_numpy_restatement(lens, shards, rotation, vocab, cap, seed, weighted):
  rng = np.random.default_rng(seed)
  offs = np.zeros(len(lens) + 1, np.int32)
  offs[1:] = np.cumsum(lens)
  ids = rng.integers(0, vocab, int(offs[-1]))
  gains = rng.integers(1, 4, ids.size).astype(np.float32) if weighted else None
  rows, samples, g, ptr, stats = ip.partition_csr(ids, offs, shards, rotation=rotation, gains=gains,
                                                  max_ids_per_partition=cap)
  # restatement: (shard, row, sample) triples with summed gains, sorted, capped per shard
  merged = {}
  for b in range(len(lens)):
    for i in range(offs[b], offs[b + 1]):
      key = ((int(ids[i]) % shards + rotation) % shards, int(ids[i]) // shards, b)
      merged[key] = merged.get(key, 0.0) + (float(gains[i]) if weighted else 1.0)
  want, dropped, max_ids, max_unique = [], 0, 0, 0
  for s in range(shards):
    entries = sorted(k for k in merged if k[0] == s)
    kept = entries if cap <= 0 else entries[:cap]
    dropped += len(entries) - len(kept)
    max_ids = max(max_ids, len(kept))
    max_unique = max(max_unique, len({k[1] for k in kept}))
    want += kept
    assert ptr[s + 1] - ptr[s] == len(kept)
  assert [(r, b) for _, r, b in want] == list(zip(rows.tolist(), samples.tolist()))
  np.testing.assert_allclose(g, [merged[k] for k in want])
  assert (stats.max_ids_per_partition, stats.max_unique_ids_per_partition, stats.dropped_ids) == (max_ids, max_unique, dropped)


@settings(max_examples=25, deadline=None, derandomize=True)
@given(n=st.integers(200, 3000), pos_rate=st.floats(0.1, 0.9), sep=st.floats(0.0, 3.0), seed=st.integers(0, 10_000),
       weighted=st.booleans())
def test_auc_metrics_agree_with_scikit_learn(n, pos_rate, sep, seed, weighted):
  """The 200-threshold AUC estimates against scikit-learn's exact curves (an independent implementation) on
  random scores of varying separability, merged from two halves the way the trainer merges steps."""
  sk = pytest.importorskip("sklearn.metrics")
  from recml_b200 import metrics as M
  rng = np.random.default_rng(seed)
  y = (rng.random(n) < pos_rate).astype(np.float32)
  if y.min() == y.max():
    y[0], y[1] = 0.0, 1.0
  logits = rng.normal(size=n) + sep * (y - 0.5)
  p = 1.0 / (1.0 + np.exp(-logits))
  w = rng.integers(1, 4, n).astype(np.float32) if weighted else None
  half = n // 2
  parts = [(slice(0, half)), (slice(half, n))]
  roc = [M.aucroc(y[s], p[s], None if w is None else w[s]) for s in parts]
  pr = [M.aucpr(y[s], p[s], None if w is None else w[s]) for s in parts]
  got_roc = float(roc[0].merge(roc[1]).compute())
  got_pr = float(pr[0].merge(pr[1]).compute())
  want_roc = sk.roc_auc_score(y, p, sample_weight=w)
  prec, rec, _ = sk.precision_recall_curve(y, p, sample_weight=w)
  want_pr = sk.auc(rec, prec)
  assert abs(got_roc - want_roc) < 0.02, (got_roc, want_roc)
  assert abs(got_pr - want_pr) < 0.03, (got_pr, want_pr)


@settings(max_examples=25, deadline=None, derandomize=True)
@given(n=st.integers(1, 40), c=st.integers(2, 60), k=st.integers(1, 20), seed=st.integers(0, 10_000))
def test_ranking_metrics_agree_with_scikit_learn(n, c, k, seed):
  """NDCG@K and top-K accuracy with one relevant item per row against scikit-learn (distinct scores: ties are
  broken differently by design — a tie counts against the target here)."""
  sk = pytest.importorskip("sklearn.metrics")
  import torch
  from recml_b200 import metrics as M
  rng = np.random.default_rng(seed)
  scores = rng.permuted(np.tile(np.arange(c, dtype=np.float32), (n, 1)), axis=1) / c      # distinct per row
  y = rng.integers(0, c, n)
  rel = np.zeros((n, c), dtype=np.float32)
  rel[np.arange(n), y] = 1.0
  kk = min(k, c)
  got_ndcg = float(M.ndcg_at_k(torch.from_numpy(y), torch.from_numpy(scores), k=kk).compute())
  got_rec = float(M.recall_at_k(torch.from_numpy(y), torch.from_numpy(scores), k=kk).compute())
  want_ndcg = sk.ndcg_score(rel, scores, k=kk) if c > 1 else 1.0
  want_rec = float(np.mean([(np.argsort(-scores[i])[:kk] == y[i]).any() for i in range(n)]))
  assert abs(got_ndcg - want_ndcg) < 1e-5 and abs(got_rec - want_rec) < 1e-6
  ranks = np.array([1 + int((scores[i] > scores[i, y[i]]).sum()) for i in range(n)])
  assert abs(float(M.mrr(torch.from_numpy(y), torch.from_numpy(scores)).compute()) - float(np.mean(1.0 / ranks))) < 1e-6


def test_cpu_reference_ops_agree_with_torch_builtins():
  """The plain-torch formulations that serve as oracles for the CUDA kernels, themselves checked against torch's
  own operators: attention vs `scaled_dot_product_attention`, the causal depthwise convolution vs `conv1d`, the
  layer / RMS norm vs `layer_norm` / `rms_norm`, the multi-head attention layer vs `nn.MultiheadAttention`."""
  import torch
  import torch.nn.functional as F
  from recml_b200.layers import transformer
  from recml_b200.ops import norm as norm_ops, softmax_attention as sm, ssd
  torch.manual_seed(0)
  B, L, H, Dh = 3, 17, 2, 8
  q, k, v = (torch.randn(B, L, H, Dh) for _ in range(3))
  pad = torch.ones(B, L, dtype=torch.bool)
  pad[0, :5] = False
  pad[2, 11:] = False
  for causal in (False, True):
    mask = sm.merge_masks(B, L, q.device, padding_mask=pad, causal=causal)
    got = sm.softmax_attention(q, k, v, mask)
    want = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                          attn_mask=mask[:, None]).transpose(1, 2)
    rows = mask.any(-1)                      # a query that sees no key has no defined output
    torch.testing.assert_close(got[rows], want[rows], rtol=1e-5, atol=1e-5)

  C, K = 6, 4
  x, w, b = torch.randn(B, L, C), torch.randn(C, K), torch.randn(C)
  got = ssd.causal_depthwise_conv1d_silu(x, w, b)
  want = F.silu(F.conv1d(x.transpose(1, 2), w[:, None, :], b, padding=K - 1, groups=C)[..., :L]).transpose(1, 2)
  torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)

  D = 12
  x, g, beta = torch.randn(5, 7, D), torch.randn(D), torch.randn(D)
  torch.testing.assert_close(norm_ops.layer_norm(x, g, beta, 1e-5), F.layer_norm(x, (D,), g, beta, 1e-5), rtol=1e-5, atol=1e-5)
  torch.testing.assert_close(norm_ops.layer_norm(x, g, None, 1e-5, rms=True), F.rms_norm(x, (D,), g, 1e-5), rtol=1e-5, atol=1e-5)

  # the attention layer with its weights copied into torch's module
  E = H * Dh
  mine = transformer.MultiHeadAttention(E, H).eval()
  ref = torch.nn.MultiheadAttention(E, H, batch_first=True).eval()
  with torch.no_grad():
    mine.qkv_bias.normal_()
    mine.out_bias.normal_()
    ref.in_proj_weight.copy_(mine.qkv)             # rows q | k | v in both
    ref.in_proj_bias.copy_(mine.qkv_bias)
    ref.out_proj.weight.copy_(mine.out)
    ref.out_proj.bias.copy_(mine.out_bias)
  h = torch.randn(B, L, E)
  got = mine(h, sm.merge_masks(B, L, h.device, padding_mask=pad, causal=True))
  got2 = mine(h, None, padding_mask=pad, causal=True, structured=True)
  causal = torch.triu(torch.ones(L, L, dtype=torch.bool), 1)
  want, _ = ref(h, h, h, key_padding_mask=~pad, attn_mask=causal, need_weights=False)
  rows = pad          # padded queries are undefined
  torch.testing.assert_close(got[rows], want[rows], rtol=1e-4, atol=1e-5)
  torch.testing.assert_close(got2[rows], want[rows], rtol=1e-4, atol=1e-5)


@settings(max_examples=30, deadline=None, derandomize=True)
@given(bags=st.lists(st.lists(st.integers(0, 19), min_size=0, max_size=5), min_size=1, max_size=9),
       combiner=st.sampled_from(["sum", "mean", "sqrtn"]), weighted=st.booleans(), seed=st.integers(0, 1000))
def test_embedding_lookup_agrees_with_embedding_bag(bags, combiner, weighted, seed):
  """The sharded-embedding module on one CPU rank and the host oracle `cpu_lookup` against
  `torch.nn.functional.embedding_bag` (sum, mean; weighted sums through `per_sample_weights`) and the
  definition of the sqrtn combiner (sum / sqrt(sum of squared weights))."""
  import torch
  import torch.nn.functional as F
  from recml_b200 import embedding as emb
  rng = np.random.default_rng(seed)
  V, D = 20, 8
  cfg = emb.ShardedEmbeddingConfig({"f": emb.EmbeddingSpec(V, D, combiner=combiner)}, emb.SGDOptimizerSpec(0.1),
                                   backend="collective", seed=seed)
  m = emb.ShardedEmbedding(cfg, device="cpu")
  table = m.gather_table("f")
  weights = {"f": [[float(x) for x in rng.integers(1, 4, len(b))] for b in bags]} if weighted else None
  kjt = emb.KeyedJagged.from_lists({"f": bags}, weights)
  out = m(kjt)
  out = out["f"] if isinstance(out, dict) else out.reshape(len(bags), -1)
  host = emb.cpu_lookup(cfg, {"f": table}, kjt)["f"]
  flat = torch.tensor([i for b in bags for i in b], dtype=torch.long)
  offs = torch.tensor(np.cumsum([0] + [len(b) for b in bags[:-1]]), dtype=torch.long)
  w = torch.tensor([x for b in weights["f"] for x in b]) if weighted else None
  if combiner == "mean" and not weighted:
    want = F.embedding_bag(flat, table, offs, mode="mean")
  else:
    want = F.embedding_bag(flat, table, offs, mode="sum", per_sample_weights=w)
    ww = [np.asarray(x, dtype=np.float64) if weighted else np.ones(len(b)) for b, x in
          zip(bags, weights["f"] if weighted else bags)]
    if combiner == "mean":
      den = torch.tensor([x.sum() for x in ww], dtype=torch.float32)
    elif combiner == "sqrtn":
      den = torch.tensor([np.sqrt((x ** 2).sum()) for x in ww], dtype=torch.float32)
    else:
      den = torch.ones(len(bags))
    want = torch.where(den[:, None] > 0, want / den[:, None].clamp_min(1e-30), torch.zeros(()))
  torch.testing.assert_close(host, want, rtol=1e-5, atol=1e-6)
  torch.testing.assert_close(out.float(), want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("kind", ["sgd", "adagrad"])
def test_embedding_training_follows_torch_embedding_bag_and_optimizer(kind):
  """Five training steps of the sharded-embedding module on one CPU rank (update inside the backward, duplicate
  ids in a batch, empty bags) against `nn.EmbeddingBag` trained by `torch.optim.SGD` / `Adagrad`."""
  import torch
  from torch import nn
  from recml_b200 import embedding as emb
  torch.manual_seed(0)
  rng = np.random.default_rng(0)
  V, D, B, lr = 30, 6, 12, 0.2
  spec = emb.SGDOptimizerSpec(lr) if kind == "sgd" else emb.AdagradOptimizerSpec(lr, initial_accumulator_value=0.1)
  cfg = emb.ShardedEmbeddingConfig({"f": emb.EmbeddingSpec(V, D, combiner="sum")}, spec, backend="collective", seed=1)
  m = emb.ShardedEmbedding(cfg, device="cpu")
  ref = nn.EmbeddingBag(V, D, mode="sum")
  with torch.no_grad():
    ref.weight.copy_(m.gather_table("f"))
  opt = torch.optim.SGD(ref.parameters(), lr=lr) if kind == "sgd" else \
      torch.optim.Adagrad(ref.parameters(), lr=lr, initial_accumulator_value=0.1, eps=0.0)
  head = torch.randn(D)
  for _ in range(5):
    bags = [rng.integers(0, V, int(rng.integers(0, 5))).tolist() for _ in range(B)]
    bags[3] = [7, 7, 7]                                  # one row three times in a bag
    kjt = emb.KeyedJagged.from_lists({"f": bags})
    out = m(kjt)
    out = out["f"] if isinstance(out, dict) else out.reshape(B, -1)
    ((out.float() * head).sum(-1) ** 2).sum().backward()
    flat = torch.tensor([i for b in bags for i in b], dtype=torch.long)
    offs = torch.tensor(np.cumsum([0] + [len(b) for b in bags[:-1]]), dtype=torch.long)
    opt.zero_grad()
    ((ref(flat, offs) * head).sum(-1) ** 2).sum().backward()
    opt.step()
    torch.testing.assert_close(m.gather_table("f"), ref.weight.detach(), rtol=1e-4, atol=1e-5)


@settings(max_examples=30, deadline=None, derandomize=True)
@given(n=st.integers(1, 500), seed=st.integers(0, 10_000), weighted=st.booleans(), scale=st.floats(0.1, 30.0))
def test_bce_reference_agrees_with_torch_and_its_histograms_with_the_auc_metrics(n, seed, weighted, scale):
  """The loss op's host formulation (the oracle of the CUDA kernel): loss and gradient against
  `binary_cross_entropy_with_logits` + autograd, and its two histograms against the threshold-based confusion
  counts that the AUC metrics use."""
  import torch
  import torch.nn.functional as F
  from recml_b200 import metrics as M
  from recml_b200.metrics import confusion
  from recml_b200.ops import bce
  g = torch.Generator().manual_seed(seed)
  x = (torch.randn(n, generator=g) * scale).requires_grad_()
  y = (torch.rand(n, generator=g) < 0.3).float()
  w = torch.randint(1, 4, (n,), generator=g).float() if weighted else None
  r = bce.bce_with_logits(x.detach(), y, w, grad_scale=1.0 / n)
  want = F.binary_cross_entropy_with_logits(x, y, weight=w, reduction="sum")
  torch.testing.assert_close(r.loss_sum, want.detach(), rtol=1e-5, atol=1e-5)
  (want / n).backward()
  torch.testing.assert_close(r.dlogits, x.grad, rtol=1e-5, atol=1e-7)
  tp, tn, fp, fn = confusion.confusion_from_histograms(r.hist_pos, r.hist_neg)
  p = torch.sigmoid(x.detach())
  etp, etn, efp, efn = confusion.estimate_confusion_matrix(p, y, w, thresholds=confusion.default_thresholds(200))
  for got, exp in ((tp, etp), (tn, etn), (fp, efp), (fn, efn)):
    np.testing.assert_allclose(np.asarray(got, dtype=np.float64), np.asarray(exp, dtype=np.float64), rtol=0, atol=1e-3)
  np.testing.assert_allclose(float(M.HistogramAUCROC(pos_hist=r.hist_pos, neg_hist=r.hist_neg).compute()),
                             float(M.aucroc(y, p, w).compute()), atol=1e-6)


@settings(max_examples=80, deadline=None, derandomize=True)
@given(shape=st.lists(st.integers(1, 13), min_size=1, max_size=3), data=st.data(),
       form=st.sampled_from(["raw", "raw_clipped", "zstd", "ocdbt"]), seed=st.integers(0, 1000))
def test_region_reads_of_any_chunk_grid_equal_numpy_slicing(tmp_path_factory, shape, data, form, seed):
  """`read_region` has a general path and several direct ones (whole rows of raw chunks, a chunk that is exactly
  the request, row ranges out of an OCDBT value); whatever the chunk grid, the stored form and the requested
  region, the result is the slice numpy gives."""
  import json
  import torch
  from recml_b200.ckpt import ocdbt, zarr_io
  if form == "zstd" and not zarr_io.zstd_available():
    return
  nd = len(shape)
  chunks = [data.draw(st.integers(1, s + 2)) for s in shape]
  start = [data.draw(st.integers(0, s - 1)) for s in shape]
  stop = [data.draw(st.integers(a + 1, s)) for a, s in zip(start, shape)]
  arr = np.random.default_rng(seed).normal(size=shape).astype(np.float32)
  d = str(tmp_path_factory.mktemp("zr"))
  leaf = os.path.join(d, "leaf")
  comp = "zstd" if form == "zstd" else None
  zarr_io.write_zarray(leaf, shape, chunks, "<f4", comp)
  grid = [(s + c - 1) // c for s, c in zip(shape, chunks)]
  pieces = {}
  for idx in np.ndindex(*grid):
    sl = tuple(slice(i * c, min((i + 1) * c, s)) for i, c, s in zip(idx, chunks, shape))
    full = np.zeros(chunks, dtype=np.float32)                    # edge chunks are stored at full chunk shape
    part = arr[sl]
    full[tuple(slice(0, n) for n in part.shape)] = part
    clip_rows = form == "raw_clipped" and idx[0] == grid[0] - 1  # ... or clipped along the first dimension
    pieces[idx] = np.ascontiguousarray(full[:part.shape[0]] if clip_rows else full)
  if form == "ocdbt":
    w = ocdbt.Writer(d, max_inline_value_bytes=16)
    w.add("leaf/.zarray", open(os.path.join(leaf, ".zarray"), "rb").read())
    for idx, piece in pieces.items():
      w.add_array("leaf/" + zarr_io.chunk_name(idx), piece)
    w.commit(compress_nodes=False, node_fanout=4)
    os.remove(os.path.join(leaf, ".zarray"))
    path = ocdbt.leaf_path(d, "leaf")
  else:
    for idx, piece in pieces.items():
      zarr_io.write_chunk(leaf, idx, piece, comp)
    path = leaf
  want = arr[tuple(slice(a, b) for a, b in zip(start, stop))]
  np.testing.assert_array_equal(zarr_io.read_region(path, start, stop).numpy(), want)
  np.testing.assert_array_equal(zarr_io.read_region(path).numpy(), arr)


@pytest.mark.parametrize("normalize_first", [True, False])
def test_transformer_block_equals_torch_encoder_layer(normalize_first):
  """The SASRec (pre-norm, causal) and BERT4Rec (post-norm) blocks against `nn.TransformerEncoderLayer` carrying the
  same weights: attention with padding and causal masks, tanh-GELU feed-forward, both residual arrangements."""
  import torch
  from torch import nn
  from recml_b200.layers import transformer
  torch.manual_seed(0)
  B, L, E, H, FF = 3, 11, 16, 4, 40
  mine = transformer.TransformerBlock(E, FF, H, normalize_first=normalize_first, causal=normalize_first,
                                      layer_norm_epsilon=1e-5).eval()
  with torch.no_grad():
    for p in mine.parameters():
      if p.ndim == 1:
        p.add_(torch.randn_like(p) * 0.1)
  ref = nn.TransformerEncoderLayer(E, H, FF, dropout=0.0, activation=lambda x: nn.functional.gelu(x, approximate="tanh"),
                                   layer_norm_eps=1e-5, batch_first=True, norm_first=normalize_first).eval()
  with torch.no_grad():
    ref.self_attn.in_proj_weight.copy_(mine.attn.qkv)
    ref.self_attn.in_proj_bias.copy_(mine.attn.qkv_bias)
    ref.self_attn.out_proj.weight.copy_(mine.attn.out)
    ref.self_attn.out_proj.bias.copy_(mine.attn.out_bias)
    ref.norm1.weight.copy_(mine.attn_norm_w); ref.norm1.bias.copy_(mine.attn_norm_b)
    ref.norm2.weight.copy_(mine.ffn_norm_w); ref.norm2.bias.copy_(mine.ffn_norm_b)
    ref.linear1.weight.copy_(mine.ffn_in); ref.linear1.bias.copy_(mine.ffn_in_bias)
    ref.linear2.weight.copy_(mine.ffn_out); ref.linear2.bias.copy_(mine.ffn_out_bias)
  x = torch.randn(B, L, E)
  pad = torch.ones(B, L, dtype=torch.bool)
  pad[1, 8:] = False                                 # right padding: every real query still sees a key
  got = mine(x, padding_mask=pad)
  causal = torch.triu(torch.ones(L, L, dtype=torch.bool), 1) if normalize_first else None
  with torch.no_grad():
    want = ref(x, src_mask=causal, src_key_padding_mask=~pad)
  torch.testing.assert_close(got[pad], want[pad], rtol=1e-4, atol=1e-5)


def test_sampled_softmax_reference_is_cross_entropy_over_the_kept_candidates():
  """The loss op's host formulation (the oracle of its CUDA kernel) against `cross_entropy` over [positive |
  candidates that are not the row's own target] built row by row."""
  import torch
  import torch.nn.functional as F
  from recml_b200.ops import sampled_softmax as S
  torch.manual_seed(0)
  T, C, temp = 23, 17, 0.2
  pos, neg = torch.randn(T), torch.randn(T, C)
  cand = torch.randint(0, 40, (C,))
  tgt = torch.randint(0, 40, (T,))
  tgt[:5] = cand[:5]                       # accidental hits
  w = (torch.rand(T) > 0.3).float()
  loss, hit = S.reference(pos, neg, cand, tgt, w, temp)
  nll, hits = [], []
  for t in range(T):
    keep = cand != tgt[t]
    logits = torch.cat([pos[t:t + 1], neg[t][keep]]) / temp
    nll.append(F.cross_entropy(logits[None], torch.zeros(1, dtype=torch.long)))
    hits.append(float(logits.argmax() == 0))
  want = (torch.stack(nll) * w).sum() / w.sum().clamp_min(1.0)
  torch.testing.assert_close(loss, want, rtol=1e-5, atol=1e-6)
  torch.testing.assert_close(hit, (torch.tensor(hits) * w).sum() / w.sum().clamp_min(1.0))


@pytest.mark.parametrize("scaled,use_bias", [(False, False), (True, True)])
def test_hstu_block_equals_a_loop_restatement(scaled, use_bias):
  """The dense HSTU block against its definition written with explicit loops over batch, head and position
  (`recml/layers/keras/hstu.py:356-460`): LN, one u|q|k|v projection with SiLU, SiLU attention weights divided by
  the padded length (or scaled queries), masked, then LN over (heads, head dim) gated by u, output projection,
  residual."""
  import math
  import torch
  import torch.nn.functional as F
  from recml_b200.layers import hstu
  torch.manual_seed(0)
  B, L, D, H = 2, 6, 8, 2
  Dh = D // H
  blk = hstu.HSTUBlock(D, H, use_bias=use_bias, scaled_pointwise_attn=scaled, layer_norm_epsilon=1e-5).eval()
  with torch.no_grad():
    for p in blk.parameters():
      if p.ndim <= 2 and p is not blk.uqkv and p is not blk.out:
        p.add_(torch.randn_like(p) * 0.1)
  x = torch.randn(B, L, D)
  mask = torch.tril(torch.ones(L, L, dtype=torch.bool))[None].repeat(B, 1, 1)
  mask[1, :, 0] = False                                   # a padded key in the second sequence
  mask[1, 0, 0] = True
  bias = torch.randn(B, L, L) * 0.3
  got = blk(x, mask, bias)
  n = F.layer_norm(x, (D,), blk.input_norm_w, blk.input_norm_b, 1e-5)
  z = F.silu(F.linear(n, blk.uqkv, blk.uqkv_bias)).reshape(B, L, 4, H, Dh)
  u, q, k, v = z[:, :, 0], z[:, :, 1], z[:, :, 2], z[:, :, 3]
  attn = torch.zeros(B, L, H, Dh)
  for b in range(B):
    for h in range(H):
      for t in range(L):
        for s in range(L):
          if not mask[b, t, s]:
            continue
          qv = q[b, t, h] / math.sqrt(Dh) if scaled else q[b, t, h]
          wgt = F.silu(qv @ k[b, s, h] + bias[b, t, s])
          attn[b, t, h] += (wgt if scaled else wgt / L) * v[b, s, h]
  y = F.layer_norm(attn, (H, Dh), blk.attn_norm_w, blk.attn_norm_b, 1e-5) * u
  want = F.linear(y.reshape(B, L, D), blk.out, blk.out_bias) + x
  torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)


def test_mamba2_layer_equals_a_token_by_token_recurrence():
  """The Mamba2 layer (chunked scan over the whole sequence) against the same layer run as a recurrence, one token
  at a time with an explicit convolution window and state `h <- exp(dt A) h + dt x B^T`, `y = h C`
  (`recml/layers/keras/mamba.py:253-360`), using the layer's own weights."""
  import torch
  import torch.nn.functional as F
  from recml_b200.layers import mamba
  torch.manual_seed(0)
  B, L, D = 2, 12, 8
  layer = mamba.Mamba2(D, d_state=4, d_conv=3, expand=2, nheads=4, chunk_size=4, use_dense_bias=True, use_conv_bias=True).eval()
  with torch.no_grad():
    for p in layer.parameters():
      if p.ndim == 1 and p is not layer.dt_bias and p is not layer.a_log:
        p.add_(torch.randn_like(p) * 0.1)
  x_in = torch.randn(B, L, D)
  got = layer(x_in)
  H, P, N, K = layer.nheads, layer.headdim, layer.d_state, layer.d_conv
  a = -torch.exp(layer.a_log)
  out = torch.zeros(B, L, D)
  for bi in range(B):
    h = torch.zeros(H, P, N)
    window = torch.zeros(K, layer.d_inner + 2 * N)             # the last K pre-convolution rows, oldest first
    for t in range(L):
      u = x_in[bi, t]
      z = F.linear(u, layer.z_proj, layer.z_bias)
      xbc = F.linear(u, layer.xbc_proj, layer.xbc_bias)
      dt = F.softplus(F.linear(u, layer.dt_proj, layer.dt_proj_bias) + layer.dt_bias)       # [H]
      window = torch.cat([window[1:], xbc[None]])
      conv = F.silu((window * layer.conv_weight.t()).sum(0) + layer.conv_bias)
      xs, bt, ct = conv[:layer.d_inner].reshape(H, P), conv[layer.d_inner:layer.d_inner + N], conv[layer.d_inner + N:]
      h = torch.exp(dt * a)[:, None, None] * h + (dt[:, None] * xs)[:, :, None] * bt[None, None, :]
      y = (h * ct[None, None, :]).sum(-1).reshape(-1) * F.silu(z)
      y = y * torch.rsqrt(y.pow(2).mean() + 1e-5) * layer.norm_w + layer.norm_b
      out[bi, t] = F.linear(y, layer.out_proj, layer.out_bias)
  torch.testing.assert_close(got, out, rtol=1e-4, atol=1e-5)
