"""Host input pipeline throughput (CPU only): TFRecord indexing + CRC check and `tf.Example` parsing of
Criteo-shaped per-example records (1 label, 13 float features, 26 variable-length id features) by the
native parser, one call per feature versus one pass for all features, the dataset factory end to end, and the
loader of pre-batched Criteo records.

  python -m recml_b200.benchmarks.data_bench [--examples N] [--threads T]

Prints one JSON line.  The file is written to a temporary directory and removed afterwards.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import time


def run(examples: int = 20000, seed: int = 0) -> dict:
  import numpy as np
  from recml_b200.data import tfrecord
  rng = np.random.default_rng(seed)
  specs = ([("label", "int64", 1, 0)] + [(f"dense_{j}", "float", 1, 0.0) for j in range(13)] +
           [(f"cat_{j}", "int64", 0, 0) for j in range(26)])
  with tempfile.TemporaryDirectory() as d:
    path = os.path.join(d, "examples.tfrecord")
    recs = []
    for _ in range(examples):
      f = {"label": [int(rng.integers(0, 2))]}
      for j in range(13):
        f[f"dense_{j}"] = [float(rng.normal())]
      for j in range(26):
        f[f"cat_{j}"] = [int(x) for x in rng.integers(0, 1 << 30, int(rng.integers(1, 16)))]
      recs.append(tfrecord.encode_example(f))
    tfrecord.write_tfrecord(path, recs)
    size = os.path.getsize(path)
    t = time.perf_counter()
    rf = tfrecord.RecordFile(path, verify=True)
    t_index = time.perf_counter() - t
    rows = np.arange(len(rf))
    rf.parse_many(rows[:64], specs)                      # start the thread pool
    t = time.perf_counter()
    for name, dtype, fixed, default in specs:
      rf.parse(rows, name, dtype, fixed, default)
    t_each = time.perf_counter() - t
    best = float("inf")
    for _ in range(3):
      t = time.perf_counter()
      rf.parse_many(rows, specs)
      best = min(best, time.perf_counter() - t)
    # the dataset factory end to end: record order, batching, parsing, label pop (batch 4096, no prefetch thread)
    from recml_b200.data import tfrecord_factory as F
    spec = {n: (F.FixedLenFeature((fl,), dt) if fl else F.VarLenFeature(dt)) for n, dt, fl, _ in specs}
    fac = F.TFDatasetFactory(input_path=path, global_batch_size=4096, feature_spec=spec, label_name="label", repeat=True,
                             prefetch_buffer_size=0, sharding_info=F.DatasetShardingInfo(1, 0))
    it = iter(fac.make())
    next(it)
    t = time.perf_counter()
    n_batches = max(4, examples // 4096)
    for _ in range(n_batches):
      next(it)
    t_fac = time.perf_counter() - t
    # pre-batched Criteo records (one record = one batch of 4096 samples, 214 ids per sample) through the loader
    from recml_b200.data import criteo
    hot = [3, 2, 1, 2, 6, 1, 1, 1, 1, 7, 3, 8, 1, 6, 9, 5, 1, 1, 1, 12, 100, 27, 10, 3, 1, 1]
    cpath, B = os.path.join(d, "criteo.tfrecord"), 4096
    tfrecord.write_tfrecord(cpath, [criteo.encode_record(rng.integers(0, 2, B), rng.normal(size=(B, 13)).astype(np.float32),
                                                         [rng.integers(0, 1000, (B, m)) for m in hot]) for _ in range(4)])
    it = iter(criteo.CriteoDataLoader(cpath, B, vocab_sizes=[1000] * 26, multi_hot_sizes=hot, is_training=True, shuffle_buffer=1))
    next(it)
    t = time.perf_counter()
    for _ in range(16):
      next(it)
    t_criteo = time.perf_counter() - t
  return {"examples": examples, "factory_examples_per_s": n_batches * 4096 / t_fac,
          "criteo_prebatched_samples_per_s": 16 * B / t_criteo, "file_mb": size / 1e6, "features": len(specs),
          "index_crc_ms": t_index * 1e3, "index_crc_mb_per_s": size / 1e6 / t_index,
          "per_feature_parse_examples_per_s": examples / t_each,
          "one_pass_parse_examples_per_s": examples / best, "one_pass_mb_per_s": size / 1e6 / best,
          "host_threads": int(os.environ.get("RECML_HOST_THREADS", os.cpu_count() or 1))}


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--examples", type=int, default=20000)
  ap.add_argument("--threads", type=int, default=0, help="host threads of the native pool (0: all cores)")
  args = ap.parse_args()
  if args.threads > 0:
    os.environ["RECML_HOST_THREADS"] = str(args.threads)
  print(json.dumps(run(args.examples)))


if __name__ == "__main__":
  main()
