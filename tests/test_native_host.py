"""Native host library: id packing / partitioning vs numpy, TFRecord + tf.Example round trips, the
TFRecord dataset factory, CRC-32C vectors, parallel chunk I/O."""
import ctypes
import os

import numpy as np
import pytest
import torch

from recml_b200.data import tfrecord, tfrecord_factory as tff
from recml_b200.embedding import id_pipeline as ip
from recml_b200.embedding.jagged import KeyedJagged
from recml_b200.ops import _lib


def test_crc32c_known_vectors():
  assert tfrecord.crc32c(b"123456789") == 0xE3069283
  assert tfrecord.crc32c(b"") == 0
  assert tfrecord.crc32c(bytes(32)) == 0x8A9136AA


def test_pack_jagged_matches_python():
  rng = np.random.default_rng(0)
  B = 37
  feats, lists = {}, {}
  for f in range(5):
    lens = rng.integers(0, 6, B).astype(np.int32)
    ids = rng.integers(0, 1000, int(lens.sum()))
    feats[f"f{f}"] = (ids, lens)
    offs = np.concatenate([[0], np.cumsum(lens)])
    lists[f"f{f}"] = [ids[offs[b]:offs[b + 1]].tolist() for b in range(B)]
  a, b = ip.pack_jagged(feats), KeyedJagged.from_lists(lists)
  assert torch.equal(a.values, b.values) and torch.equal(a.offsets, b.offsets) and a.batch_size() == B


def test_partition_csr_merges_duplicates_and_counts():
  ids = np.array([5, 5, 2, 9, 4, 4, 4, 13], np.int32)      # bags: [5,5,2] [9] [4,4,4,13]
  offs = np.array([0, 3, 4, 8], np.int32)
  rows, samples, gains, ptr, st = ip.partition_csr(ids, offs, shards=4)
  # shard = id % 4: 5,9,13 -> 1 ; 2 -> 2 ; 4 -> 0 ; local row = id // 4
  got = sorted(zip(np.repeat(np.arange(4), np.diff(ptr)).tolist(), rows.tolist(), samples.tolist(), gains.tolist()))
  assert got == [(0, 1, 2, 3.0), (1, 1, 0, 2.0), (1, 2, 1, 1.0), (1, 3, 2, 1.0), (2, 0, 0, 1.0)]
  assert (st.max_ids_per_partition, st.max_unique_ids_per_partition, st.dropped_ids) == (3, 3, 0)
  *_, st2 = ip.partition_csr(ids, offs, shards=4, max_ids_per_partition=2)
  assert st2.dropped_ids == 1 and st2.max_ids_per_partition == 2


def test_stats_recorder_roundtrip(tmp_path):
  r = ip.StatsRecorder(str(tmp_path), 0)
  r.record("t", ip.PartitionStats(5, 3, 0)); r.record("t", ip.PartitionStats(4, 9, 2))
  r.publish()
  r1 = ip.StatsRecorder(str(tmp_path), 1)
  r1.record("t", ip.PartitionStats(8, 1, 1)); r1.publish()
  s = r.load()["t"]
  assert (s.max_ids_per_partition, s.max_unique_ids_per_partition, s.dropped_ids) == (8, 9, 3)


def _write(path, n, seed=0):
  rng = np.random.default_rng(seed)
  recs, truth = [], []
  for i in range(n):
    seq = rng.integers(1, 10**12, int(rng.integers(0, 7))).tolist()
    dense = rng.normal(size=3).astype(np.float32).tolist()
    truth.append((seq, dense, i % 2))
    recs.append(tfrecord.encode_example({"sequence": seq, "dense": dense, "label": [i % 2], "tag": [b"x"]}))
  tfrecord.write_tfrecord(path, recs)
  return truth


def test_tfrecord_roundtrip_and_corruption(tmp_path):
  p = str(tmp_path / "a.tfrecord")
  truth = _write(p, 50)
  rf = tfrecord.RecordFile(p)
  assert len(rf) == 50
  rows = np.arange(50)
  vals, lens = rf.parse(rows, "sequence", "int64")
  assert lens.tolist() == [len(t[0]) for t in truth] and vals.tolist() == [v for t in truth for v in t[0]]
  np.testing.assert_allclose(rf.parse(rows, "dense", "float32", 3), np.array([t[1] for t in truth], np.float32))
  assert rf.parse(rows, "label", "int64", 1)[:, 0].tolist() == [t[2] for t in truth]
  assert rf.parse(rows[:3], "missing", "int64", 2, default=-1).tolist() == [[-1, -1]] * 3
  raw = bytearray(open(p, "rb").read())
  raw[40] ^= 0xFF
  open(p, "wb").write(raw)
  with pytest.raises(IOError):
    tfrecord.RecordFile(p)


def test_tfrecord_factory_batches_labels_and_sharding(tmp_path):
  for k in range(4):
    _write(str(tmp_path / f"part-{k}.tfrecord"), 20, seed=k)
  spec = {"sequence": tff.VarLenFeature("int64"), "dense": tff.FixedLenFeature((3,), "float32"),
          "label": tff.FixedLenFeature((1,), "int64")}
  fac = tff.TFDatasetFactory(input_path=str(tmp_path / "part-*.tfrecord"), feature_spec=spec, global_batch_size=8,
                             label_name="label", sharding_info=tff.DatasetShardingInfo(2, 1))
  it = fac.make()
  batches = list(it)
  assert len(batches) == 2 * (20 // 4)           # files 1 and 3, per-process batch 8 / 2 = 4
  feats, label = batches[0]
  assert feats["dense"].shape == (4, 3) and label.shape == (4, 1) and feats["sequence"]["lengths"].shape == (4,)
  assert tff.DatasetShardingInfo(4, 0).per_process_batch_size(64) == 16
  dbg = tff.TFDatasetFactory(input_path=str(tmp_path / "part-0.tfrecord"), feature_spec=spec, global_batch_size=4,
                             debug=True).make()
  a, b = next(dbg), next(dbg)
  assert a is b


def test_parallel_chunk_io(tmp_path):
  lib = _lib.host()
  n = 12
  bufs = [np.random.default_rng(i).integers(0, 255, 1000 + i, dtype=np.uint8) for i in range(n)]
  paths = [str(tmp_path / f"c{i}").encode() for i in range(n)]
  P = ctypes.c_void_p
  cp = (ctypes.c_char_p * n)(*paths)
  bp = (P * n)(*[b.ctypes.data for b in bufs])
  sz = (ctypes.c_longlong * n)(*[b.size for b in bufs])
  crcs = (ctypes.c_uint32 * n)()
  assert lib.recml_write_chunks(n, cp, bp, sz, crcs, 0) == 0
  outs = [np.empty_like(b) for b in bufs]
  op = (P * n)(*[o.ctypes.data for o in outs])
  assert lib.recml_read_chunks(n, cp, op, sz) == 0
  for a, b, c in zip(bufs, outs, crcs):
    assert np.array_equal(a, b) and c == tfrecord.crc32c(a.tobytes())
  assert not any(f.endswith(".partial") for f in os.listdir(tmp_path))


def test_factory_filter_rebatch_interleave_and_sequence_examples(tmp_path):
  import numpy as np
  from recml_b200.data import tfrecord, tfrecord_factory as F
  # three files of 10 records each; record id = file * 100 + index
  for f in range(3):
    recs = [tfrecord.encode_sequence_example({"id": [f * 100 + i], "w": [float(i)]},
                                             {"hist": [[i, i + 1]] * (i % 3), "score": [[0.5 * s] for s in range(i % 2 + 1)]})
            for i in range(10)]
    tfrecord.write_tfrecord(str(tmp_path / f"part-{f}.tfrecord"), recs)
  spec = {"id": F.FixedLenFeature((), "int64"), "w": F.FixedLenFeature((), "float")}
  seq = {"hist": F.VarLenFeature("int64"), "score": F.VarLenFeature("float")}
  sharding = F.DatasetShardingInfo(num_processes=1, process_index=0)
  fac = F.TFDatasetFactory(input_path=str(tmp_path / "part-*.tfrecord"), feature_spec=spec, sequence_feature_spec=seq,
                           global_batch_size=4, cycle_length=3, block_length=2, prefetch_buffer_size=0,
                           sharding_info=sharding, drop_remainder=False)
  batches = list(fac.make())
  ids = np.concatenate([b["id"] for b in batches])
  # interleave: two records from each of the three files in turn
  assert ids[:8].tolist() == [0, 1, 100, 101, 200, 201, 2, 3] and sorted(ids.tolist()) == sorted(
      f * 100 + i for f in range(3) for i in range(10))
  b0 = batches[0]                       # records 0, 1, 100, 101
  assert b0["hist"]["steps"].tolist() == [0, 1, 0, 1] and b0["hist"]["lengths"].tolist() == [0, 2, 0, 2]
  assert b0["hist"]["values"].tolist() == [1, 2, 1, 2]
  assert b0["score"]["steps"].tolist() == [1, 2, 1, 2] and np.allclose(b0["score"]["values"], [0, 0, 0.5, 0, 0, 0.5])
  # vectorised filter keeps even ids and re-batches the survivors into full batches
  fac2 = F.TFDatasetFactory(input_path=str(tmp_path / "part-*.tfrecord"), feature_spec=spec, sequence_feature_spec=seq,
                            global_batch_size=4, prefetch_buffer_size=0, sharding_info=sharding,
                            filter_fn=lambda feats: feats["id"] % 2 == 0)
  out = list(fac2.make())
  assert all(len(b["id"]) == 4 for b in out) and len(out) == 3        # 15 survivors -> 3 full batches, remainder dropped
  kept = np.concatenate([b["id"] for b in out])
  assert (kept % 2 == 0).all() and kept.tolist() == [0, 2, 4, 6, 8, 100, 102, 104, 106, 108, 200, 202]
  assert sum(int(b["hist"]["lengths"].sum()) for b in out) == sum(2 * (i % 3) for i in (0, 2, 4, 6, 8)) * 2 + 2 * (0 + 2)
  # shuffle window: a permutation of the same records
  fac3 = F.TFDatasetFactory(input_path=str(tmp_path / "part-*.tfrecord"), feature_spec=spec, global_batch_size=5,
                            shuffle=True, shuffle_buffer_size=7, prefetch_buffer_size=0, sharding_info=sharding)
  got = np.concatenate([b["id"] for b in fac3.make()])
  assert sorted(got.tolist()) == sorted(ids.tolist()) and got.tolist() != sorted(got.tolist())


def test_parse_many_matches_per_feature_parse(tmp_path):
  """One pass over each record for all features gives what one call per feature gives: fixed-length with
  defaults and truncation, variable-length, features missing from some records, any request order."""
  from recml_b200.data import tfrecord
  rng = np.random.default_rng(5)
  recs = []
  for i in range(700):
    f = {"label": [int(rng.integers(0, 2))], "d0": [float(rng.normal())], "d1": [float(x) for x in rng.normal(size=3)]}
    if i % 3:
      f["ids_a"] = [int(x) for x in rng.integers(0, 1 << 40, int(rng.integers(0, 9)))]
    if i % 5:
      f["ids_b"] = [int(x) for x in rng.integers(0, 100, int(rng.integers(1, 4)))]
    f["w"] = [float(x) for x in rng.random(int(rng.integers(0, 5)))]
    recs.append(tfrecord.encode_example(f))
  path = str(tmp_path / "many.tfrecord")
  tfrecord.write_tfrecord(path, recs)
  rf = tfrecord.RecordFile(path)
  rows = rng.permutation(len(rf))[:650]
  specs = [("ids_b", "int64", 2, -1), ("w", "float", 0, 0), ("label", "int64", 1, 0), ("absent", "int64", 2, 7),
           ("d1", "float", 2, 0.5), ("ids_a", "int64", 0, 0), ("d0", "float", 1, 0.0), ("gone", "float", 0, 0)]
  many = rf.parse_many(rows, specs)
  for name, dtype, fixed, default in specs:
    if fixed:
      np.testing.assert_array_equal(many[name], rf.parse(rows, name, dtype, fixed, default))
    else:
      vals, lens = rf.parse(rows, name, dtype)
      np.testing.assert_array_equal(many[name][0], vals)
      np.testing.assert_array_equal(many[name][1], lens)
  assert (many["absent"] == 7).all() and many["gone"][0].size == 0


@pytest.mark.parametrize("shards,rotation,cap", [(8, 0, 0), (3, 2, 0), (4, 1, 5000)])
def test_partition_csr_large_batch_matches_numpy(shards, rotation, cap):
  """Large batches take the per-shard radix sort: order, merged gains, shard pointers, statistics and
  dropping beyond the cap must equal a numpy restatement."""
  rng = np.random.default_rng(shards)
  B, bag = 4096, 12
  ids = (rng.zipf(1.2, B * bag) % 300000).astype(np.int32)
  offs = np.arange(0, B * bag + 1, bag, dtype=np.int32)
  gains = rng.random(B * bag).astype(np.float32)
  rows, samples, g, ptr, st = ip.partition_csr(ids, offs, shards, rotation=rotation, gains=gains, max_ids_per_partition=cap)
  shard = (ids % shards + rotation) % shards
  row = ids // shards
  sample = np.repeat(np.arange(B), bag)
  order = np.lexsort((sample, row, shard))
  key = np.stack([shard[order], row[order], sample[order]], 1)
  first = np.r_[True, (key[1:] != key[:-1]).any(1)]
  grp = np.cumsum(first) - 1
  merged = np.bincount(grp, weights=gains[order].astype(np.float64))
  ks, kr, km = key[first, 0], key[first, 1], key[first, 2]
  keep = np.ones(ks.size, bool)
  if cap:
    rank_in_shard = np.arange(ks.size) - np.searchsorted(ks, ks, side="left")
    keep = rank_in_shard < cap
  np.testing.assert_array_equal(rows, kr[keep])
  np.testing.assert_array_equal(samples, km[keep])
  np.testing.assert_allclose(g, merged[keep], rtol=1e-5)
  np.testing.assert_array_equal(ptr, np.r_[0, np.cumsum(np.bincount(ks[keep], minlength=shards))])
  assert st.dropped_ids == int((~keep).sum())
  assert st.max_ids_per_partition == int(np.bincount(ks[keep], minlength=shards).max())


def test_parse_many_feature_lists_match_parse_sequence(tmp_path):
  from recml_b200.data import tfrecord
  rng = np.random.default_rng(9)
  recs = []
  for i in range(300):
    steps = int(rng.integers(0, 12))
    ctx = {"user": [int(rng.integers(0, 1000))]}
    lists = {"item": [[int(rng.integers(0, 5000))] for _ in range(steps)],
             "ts": [[float(rng.random()), float(rng.random())] for _ in range(steps)]}
    if i % 4 == 0:
      lists.pop("ts")
    recs.append(tfrecord.encode_sequence_example(ctx, lists))
  path = str(tmp_path / "seq.tfrecord")
  tfrecord.write_tfrecord(path, recs)
  rf = tfrecord.RecordFile(path)
  rows = np.arange(len(rf))
  many = rf.parse_many(rows, [("item", "int64", 0, 0, "list"), ("user", "int64", 1, 0), ("ts", "float", 0, 0, "list")])
  np.testing.assert_array_equal(many["user"], rf.parse(rows, "user", "int64", 1))
  for name, dtype in (("item", "int64"), ("ts", "float")):
    vals, lens, steps = rf.parse_sequence(rows, name, dtype)
    np.testing.assert_array_equal(many[name][0], vals)
    np.testing.assert_array_equal(many[name][1], lens)
    np.testing.assert_array_equal(many[name][2], steps)


@pytest.mark.parametrize("sizes,cycle,block", [([7, 3, 10], 2, 2), ([5, 5, 5, 5], 4, 1), ([9], 3, 4), ([4, 11, 2, 6, 1], 3, 3),
                                               ([6, 6], 1, 5)])
def test_interleave_order_matches_record_by_record_definition(tmp_path, sizes, cycle, block):
  """The block-wise (numpy) interleave must give the order of the plain definition: `cycle_length` files open,
  `block_length` records from each in turn, a finished file replaced by the next pending one."""
  from recml_b200.data import tfrecord, tfrecord_factory as F
  for fi, n in enumerate(sizes):
    tfrecord.write_tfrecord(str(tmp_path / f"part-{fi:02d}.tfrecord"),
                            [tfrecord.encode_example({"x": [fi * 1000 + r]}) for r in range(n)])
  fac = F.TFDatasetFactory(input_path=str(tmp_path / "part-*.tfrecord"), global_batch_size=1,
                           feature_spec={"x": F.FixedLenFeature((1,), "int64")}, cycle_length=cycle, block_length=block,
                           prefetch_buffer_size=0, sharding_info=F.DatasetShardingInfo(1, 0))
  got = [int(b["x"][0, 0]) for b in fac.make()]
  pending = [(fi, list(range(n))) for fi, n in enumerate(sizes)]
  active, want = [], []
  while pending or active:
    while pending and len(active) < cycle:
      active.append(pending.pop(0))
    nxt = []
    for fi, rows in active:
      want += [fi * 1000 + r for r in rows[:block]]
      if rows[block:]:
        nxt.append((fi, rows[block:]))
    active = nxt
  assert got == want


def test_data_benchmark_runs_on_a_small_file():
  from recml_b200.benchmarks import data_bench
  out = data_bench.run(examples=300)
  assert out["features"] == 40 and out["one_pass_parse_examples_per_s"] > 0 and out["factory_examples_per_s"] > 0


def test_repeat_fills_batches_across_epochs(tmp_path):
  """`repeat` repeats the records before batching: an input of 5 records gives batches of 4 that run
  across epoch boundaries, and `num_epochs` bounds the total."""
  from recml_b200.data import tfrecord, tfrecord_factory as F
  tfrecord.write_tfrecord(str(tmp_path / "five.tfrecord"), [tfrecord.encode_example({"x": [r]}) for r in range(5)])
  fac = F.TFDatasetFactory(input_path=str(tmp_path / "five.tfrecord"), global_batch_size=4, repeat=True, num_epochs=3,
                           feature_spec={"x": F.FixedLenFeature((1,), "int64")}, prefetch_buffer_size=0,
                           sharding_info=F.DatasetShardingInfo(1, 0))
  got = [b["x"][:, 0].tolist() for b in fac.make()]
  assert got == [[0, 1, 2, 3], [4, 0, 1, 2], [3, 4, 0, 1]]           # 15 records, the last 3 dropped
  big = F.TFDatasetFactory(input_path=str(tmp_path / "five.tfrecord"), global_batch_size=8, repeat=True,
                           feature_spec={"x": F.FixedLenFeature((1,), "int64")}, prefetch_buffer_size=0,
                           sharding_info=F.DatasetShardingInfo(1, 0))
  it = iter(big.make())
  assert next(it)["x"][:, 0].tolist() == [0, 1, 2, 3, 4, 0, 1, 2]


def test_criteo_example_factory_packs_with_the_host_id_pipeline(tmp_path):
  """Per-example Criteo records -> batches whose `sparse` entry is the jagged layout of the embedding (feature
  major, the ids in record order) built by the native packer, with per-table shard statistics recorded."""
  from recml_b200.embedding import id_pipeline
  from recml_b200.examples import dlrm_experiment as D
  vocab, bags = (50, 1000, 7), (2, 5, 1)
  cfg = D.ModelConfig(vocab_sizes=vocab, bag_sizes=bags, num_dense=4)
  rng = np.random.default_rng(0)
  rows = []
  for i in range(24):
    f = {"label": [float(i % 2)], "dense": [float(x) for x in rng.random(4)]}
    for c, (v, b) in enumerate(zip(vocab, bags)):
      f[f"cat_{c}"] = [int(x) for x in rng.integers(0, v, int(rng.integers(0, b + 1)))]
    rows.append(f)
  tfrecord.write_tfrecord(str(tmp_path / "criteo-0.tfrecord"), [tfrecord.encode_example(f) for f in rows])
  fac = D.CriteoExampleFactory(model=cfg, input_path=str(tmp_path / "criteo-*.tfrecord"), batch_size=8,
                               is_training=False, stats_dir=str(tmp_path / "fdo"))
  it = fac.make()
  seen = 0
  for batch in it:
    kjt = batch["sparse"]
    B = kjt.batch_size()
    assert kjt.keys == ("cat_0", "cat_1", "cat_2") and batch["dense"].shape == (B, 4) and batch["label"].shape == (B,)
    offs, vals = kjt.offsets.numpy(), kjt.values.numpy()
    for c in range(3):
      for b in range(B):
        want = rows[seen + b][f"cat_{c}"]
        got = vals[offs[c * B + b]:offs[c * B + b + 1]].tolist()
        assert got == want
    seen += B
  assert seen == 24
  path = it.stats_recorder.publish()
  assert os.path.exists(path)
  stats = id_pipeline.StatsRecorder(str(tmp_path / "fdo")).load()
  assert set(stats) == {"cat_0", "cat_1", "cat_2"} and stats["cat_1"].max_ids_per_partition >= 1


def test_factory_directory_groups_unsharded_reading_and_repeated_file_lists(tmp_path):
  """`group_uris_by_dir` reads, shards and interleaves whole directories with the lexically largest first
  (`recml/core/data/tf_dataset_factory.py:151-162,809-868`); `sharding=False` gives every process the whole
  input; `repeat_files` repeats the file list before it is dealt out to the processes (`:470-478`)."""
  def write_ids(path, ids):
    os.makedirs(os.path.dirname(path), exist_ok=True)
    tfrecord.write_tfrecord(path, [tfrecord.encode_example({"id": [i]}) for i in ids])
  write_ids(str(tmp_path / "Span-0" / "Shard-0"), [0, 1])
  write_ids(str(tmp_path / "Span-0" / "Shard-1"), [2, 3])
  write_ids(str(tmp_path / "Span-1" / "Shard-0"), [10, 11, 12])
  files = sorted(str(p) for p in tmp_path.glob("Span-*/Shard-*"))
  groups = tff.get_file_groups(files)
  assert groups == [files[2], files[0] + "," + files[1]]
  with pytest.raises(ValueError):
    tff.get_file_groups([])
  spec = {"id": tff.FixedLenFeature((1,), "int64")}
  mk = lambda **kw: tff.TFDatasetFactory(**{**dict(input_path=str(tmp_path / "Span-*" / "Shard-*"), feature_spec=spec,
                                                   global_batch_size=1, prefetch_buffer_size=0), **kw})
  ids = lambda fac: [int(x) for b in fac.make() for x in np.asarray(b["id"]).reshape(-1)]
  assert mk().input_filepaths == files
  assert ids(mk()) == [0, 1, 2, 3, 10, 11, 12]
  assert ids(mk(group_uris_by_dir=True)) == [10, 11, 12, 0, 1, 2, 3]              # newest directory first
  # directories are the unit of sharding: process 1 of 2 reads all of Span-0 and nothing of Span-1
  two = lambda i, **kw: mk(global_batch_size=2, drop_remainder=False, sharding_info=tff.DatasetShardingInfo(2, i), **kw)
  assert ids(two(1, group_uris_by_dir=True)) == [0, 1, 2, 3]
  assert ids(two(0, group_uris_by_dir=True)) == [10, 11, 12]
  # and of interleaving: one record from each directory in turn
  assert ids(mk(group_uris_by_dir=True, cycle_length=2)) == [10, 0, 11, 1, 12, 2, 3]
  assert ids(two(1, sharding=False)) == [0, 1, 2, 3, 10, 11, 12]
  # three files over two processes: process 0 gets files 0 and 2; with the list repeated before sharding its
  # second pass starts at offset 3, so it gets file 1 there
  assert ids(two(0, repeat=True, num_epochs=2)) == [0, 1, 10, 11, 12] * 2
  assert ids(two(0, repeat=True, repeat_files=True, num_epochs=2)) == [0, 1, 10, 11, 12, 2, 3]
  assert ids(mk(preprocessor=lambda b: {"id": b["id"] + 100}, preprocessors=[lambda b: {"id": b["id"] * 2}]))[0] == 200
  assert ids(mk(cache_reading=True, repeat=True, num_epochs=2)) == [0, 1, 2, 3, 10, 11, 12] * 2
  with pytest.raises(ValueError, match="not supported"):
    mk(file_format=tff.FileFormat.SSTABLE).make().__next__()


def test_malformed_examples_raise_instead_of_parsing_to_defaults(tmp_path):
  """A record that does not decode to its last byte (truncated, or a length that runs past the record) is an
  error in every parse entry point, as it is for TensorFlow's example parser; valid neighbours do not hide it."""
  good = tfrecord.encode_example({"a": [1, 2, 3], "f": [0.5, 1.5], "s": [b"xy"]})
  seq = tfrecord.encode_sequence_example({"a": [7]}, {"steps": [[1, 2], [3]]})
  cases = {"truncated": good[:len(good) - 3], "overlong_length": bytes([0x0a, 0x7f]) + good[2:],
           "garbage": bytes(range(200, 230))}
  for name, bad in cases.items():
    p = str(tmp_path / f"{name}.tfrecord")
    tfrecord.write_tfrecord(p, [good, bad, good])
    rows = np.arange(3)
    for call in (lambda rf: rf.parse_many(rows, [("a", "int64", 0, 0), ("f", "float32", 2, 0.0)]),
                 lambda rf: rf.parse(rows, "a", "int64"),
                 lambda rf: rf.parse_sequence(rows, "steps", "int64")):
      with pytest.raises(ValueError, match="record 1 is not a valid"):
        call(tfrecord.RecordFile(p))
    ok = tfrecord.RecordFile(p)
    assert ok.parse(np.array([0, 2]), "a", "int64")[0].tolist() == [1, 2, 3, 1, 2, 3]     # the valid ones still parse
  p = str(tmp_path / "ok.tfrecord")
  tfrecord.write_tfrecord(p, [good, seq])
  rf = tfrecord.RecordFile(p)
  rf.validate(np.arange(2))
  vals, lens, steps = rf.parse_sequence(np.arange(2), "steps", "int64")
  assert vals.tolist() == [1, 2, 3] and steps.tolist() == [0, 2]


def test_id_preprocessing_rejects_inputs_it_cannot_index():
  """A negative id, lengths that do not add up to the ids, a shard count of zero: errors, not reads or writes
  past the buffers (the native code trusts what the wrappers let through); a rotation outside [0, shards) wraps."""
  ids = np.array([5, -3, 7], dtype=np.int64)
  offs = np.array([0, 2, 3], dtype=np.int32)
  with pytest.raises(ValueError, match="negative id"):
    ip.partition_csr(ids, offs, 4)
  with pytest.raises(ValueError, match="shards"):
    ip.partition_csr(np.abs(ids), offs, 0)
  a = ip.partition_csr(np.abs(ids), offs, 4, rotation=1)
  b = ip.partition_csr(np.abs(ids), offs, 4, rotation=-3)
  assert all(np.array_equal(x, y) for x, y in zip(a[:4], b[:4]))
  with pytest.raises(ValueError, match="summing to"):
    ip.pack_jagged({"a": (np.arange(4), np.array([2, 3], dtype=np.int32))})
  with pytest.raises(ValueError, match="lengths of 1 samples"):
    ip.pack_jagged({"a": (np.arange(2), np.array([1, 1], dtype=np.int32)), "b": (np.arange(2), np.array([2], dtype=np.int32))})


def test_tfrecord_index_rejects_frames_that_run_past_the_file(tmp_path):
  """A length field of 2^63 - 1 (read as a negative offset once), a cut-off frame and stray bytes after the last
  frame are corruption with and without checksum verification."""
  good = tfrecord.encode_example({"a": [1, 2]})
  p = str(tmp_path / "x.tfrecord")
  tfrecord.write_tfrecord(p, [good, good])
  raw = open(p, "rb").read()
  frame = len(raw) // 2
  cases = {"huge_length": raw[:frame] + (2**63 - 1).to_bytes(8, "little") + raw[frame + 8:],
           "negative_length": raw[:frame] + (2**64 - 40).to_bytes(8, "little") + raw[frame + 8:],
           "cut_frame": raw[:-5], "stray_tail": raw + b"\\x01\\x02\\x03"}
  for name, blob in cases.items():
    q = str(tmp_path / f"{name}.tfrecord")
    open(q, "wb").write(blob)
    for verify in (True, False):
      with pytest.raises(IOError, match="corrupt TFRecord"):
        tfrecord.RecordFile(q, verify=verify)
  assert len(tfrecord.RecordFile(p)) == 2
