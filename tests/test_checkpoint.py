"""Checkpoint manager: layout, round trips (dense, bf16, sharded leaves restored under a different
sharding), retention, save policy, async completion, zstd chunks, the checkpoints iterator."""
import json
import os
import threading
import time

import numpy as np
import pytest
import torch

from recml_b200 import ckpt
from recml_b200.ckpt import zarr_io


def _tree():
  return {"step": torch.tensor(7), "params": {"w": torch.randn(5, 3), "b": torch.randn(3).to(torch.bfloat16)},
          "opt_state": {"count": torch.tensor(3), "mu": [torch.zeros(2), torch.ones(2, 2)]}}


def test_layout_and_roundtrip(tmp_path):
  m = ckpt.CheckpointManager(str(tmp_path), async_save=False)
  t = _tree()
  assert m.save(11, t, metrics={"train": {"loss": 0.5}})
  d = tmp_path / "11"
  assert (d / "_CHECKPOINT_METADATA").exists() and (d / "state" / "_METADATA").exists()
  assert (d / "state" / "_sharding").exists() and (d / "commit_success.txt").exists()
  assert (d / "state" / "params.w" / ".zarray").exists() and (d / "state" / "params.w" / "0.0").exists()
  z = json.load(open(d / "state" / "params.w" / ".zarray"))
  assert z["shape"] == [5, 3] and z["dtype"] == "<f4" and z["zarr_format"] == 2
  assert json.load(open(d / "state" / "params.b" / ".zarray"))["dtype"] == "bfloat16"
  assert m.metrics(11)["train"]["loss"] == 0.5
  back = m.restore(11)
  torch.testing.assert_close(back["params"]["w"], t["params"]["w"])
  assert back["params"]["b"].dtype == torch.bfloat16 and torch.equal(back["params"]["b"], t["params"]["b"])
  assert isinstance(back["opt_state"]["mu"], list) and back["opt_state"]["mu"][1].shape == (2, 2)
  tgt = m.restore(11, target={"params": {"w": torch.zeros(5, 3)}})
  torch.testing.assert_close(tgt["params"]["w"], t["params"]["w"])
  with pytest.raises(KeyError):
    m.restore(11, target={"params": {"nope": torch.zeros(1)}})
  with pytest.raises(FileNotFoundError):
    ckpt.restore_tree(str(tmp_path / "11" / "missing"))


def test_retention_policy_and_async(tmp_path):
  keep = {3, 7, 11}
  m = ckpt.CheckpointManager(str(tmp_path), max_to_keep=2, should_save_fn=lambda s, _: s in keep)
  for s in range(12):
    m.save(s, {"x": torch.full((4,), float(s))})
  m.wait_until_finished()
  assert m.all_steps() == [7, 11] and m.latest_step() == 11
  assert float(m.restore()["x"][0]) == 11.0
  assert not [n for n in os.listdir(tmp_path) if "tmp" in n]
  assert m.save(5, {"x": torch.zeros(1)}, force=True)
  m.close()


def test_sharded_leaf_resharding(tmp_path):
  """A table saved as two row blocks is read back whole, and as three uneven blocks."""
  full = torch.arange(40, dtype=torch.float32).reshape(10, 4)
  m = ckpt.CheckpointManager(str(tmp_path), async_save=False)
  # one process plays both ranks: write block 0, then block 1 into the same step directory
  a = ckpt.ShardedLeaf(full[:5], (10, 4), (0, 0), (5, 4))
  m.save(0, {"t": a})
  zarr_io.write_chunk(str(tmp_path / "0" / "state" / "t"), (1, 0), full[5:].numpy(), None)
  torch.testing.assert_close(m.restore(0)["t"], full)
  for lo, hi in [(0, 4), (4, 8), (8, 10)]:
    got = zarr_io.read_region(str(tmp_path / "0" / "state" / "t"), [lo, 0], [hi, 4])
    torch.testing.assert_close(got, full[lo:hi])
  tgt = ckpt.ShardedLeaf(torch.zeros(4, 4), (10, 4), (1, 0), (4, 4))
  torch.testing.assert_close(m.restore(0, target={"t": tgt})["t"], full[4:8])


@pytest.mark.parametrize("new_world", [1, 3, 4])
def test_mod_sharded_leaf_restores_on_another_world_size(tmp_path, new_world):
  """A row-sharded table saved by 2 ranks in MOD layout (block b = ids with id % 2 == b) is read back by
  jobs of 1, 3 and 4 ranks, each rank getting exactly its residue class; a plain block leaf whose global
  shape changed is refused."""
  V, D, W = 11, 3, 2
  full = torch.arange(V * D, dtype=torch.float32).reshape(V, D)
  rows = (V + W - 1) // W
  m = ckpt.CheckpointManager(str(tmp_path), async_save=False)
  mod = {"vocab": V, "world": W}
  blocks = [full[b::W] for b in range(W)]
  m.save(0, {"t": ckpt.ShardedLeaf(blocks[0][None], (W, rows, D), (0, 0, 0), (1, rows, D), mod=mod)})
  pad = torch.zeros(rows, D)
  pad[:blocks[1].shape[0]] = blocks[1]
  zarr_io.write_chunk(str(tmp_path / "0" / "state" / "t"), (1, 0, 0), pad[None].numpy(), None)
  rows_new = (V + new_world - 1) // new_world
  for r in range(new_world):
    want = full[r::new_world]
    tgt = ckpt.ShardedLeaf(torch.zeros(1, want.shape[0], D), (new_world, rows_new, D), (r, 0, 0), (1, rows_new, D),
                           mod={"vocab": V, "world": new_world})
    got = m.restore(0, target={"t": tgt})["t"]
    torch.testing.assert_close(got[0][:want.shape[0]], want)
  plain = ckpt.ShardedLeaf(torch.zeros(1, rows_new, D), (new_world + 5, rows_new, D), (0, 0, 0), (1, rows_new, D))
  with pytest.raises(ValueError, match="does not fit target"):
    m.restore(0, target={"t": plain})


@pytest.mark.skipif(not zarr_io.zstd_available(), reason="libzstd not loadable")
def test_zstd_chunks(tmp_path):
  m = ckpt.CheckpointManager(str(tmp_path), async_save=False, compressor="zstd")
  x = torch.zeros(1000, 16)
  m.save(1, {"x": x})
  assert os.path.getsize(tmp_path / "1" / "state" / "x" / "0.0") < x.numel()
  assert json.load(open(tmp_path / "1" / "state" / "x" / ".zarray"))["compressor"]["id"] == "zstd"
  torch.testing.assert_close(m.restore(1)["x"], x)
  # the frames carry a content checksum: one flipped bit anywhere in a stored chunk fails the restore
  y = torch.randn(300, 16)
  m.save(2, {"x": y})
  chunk = tmp_path / "2" / "state" / "x" / "0.0"
  raw = bytearray(chunk.read_bytes())
  for at in (len(raw) // 3, len(raw) - 1):
    bad = bytearray(raw)
    bad[at] ^= 0x10
    chunk.write_bytes(bytes(bad))
    with pytest.raises(IOError, match="zstd"):
      m.restore(2)
  chunk.write_bytes(bytes(raw))
  torch.testing.assert_close(m.restore(2)["x"], y)


def test_checkpoints_iterator_sees_new_steps_and_stops_on_marker(tmp_path):
  m = ckpt.CheckpointManager(str(tmp_path), async_save=False)
  m.save(1, {"x": torch.zeros(1)})
  done = threading.Event()

  def writer():
    time.sleep(0.3)
    m.save(2, {"x": torch.zeros(1)})
    time.sleep(0.3)
    done.set()

  th = threading.Thread(target=writer); th.start()
  seen = list(ckpt.checkpoints_iterator(str(tmp_path), timeout=0.5, timeout_fn=done.is_set, poll_secs=0.05))
  th.join()
  assert seen == [1, 2]


def test_row_range_reads_match_general_path(tmp_path):
  """The native reader (uncompressed arrays chunked along rows) returns what the chunk-by-chunk reader
  returns for whole arrays and for row ranges that start and end inside chunks; a missing chunk file
  still raises FileNotFoundError."""
  import numpy as np
  import pytest
  from recml_b200.ckpt import zarr_io
  rng = np.random.default_rng(0)
  full = rng.normal(size=(1000, 24)).astype(np.float32)
  path = str(tmp_path / "arr")
  os.makedirs(path)
  zarr_io.write_zarray(path, full.shape, (256, 24), "<f4", None)
  items = [(path, [ci, 0], full[ci * 256:(ci + 1) * 256]) for ci in range(4)]
  zarr_io.write_chunks_parallel(items)
  for lo, hi in [(0, 1000), (100, 700), (255, 257), (512, 1000), (999, 1000)]:
    got = zarr_io.read_region(path, [lo, 0], [hi, 24]).numpy()
    np.testing.assert_array_equal(got, full[lo:hi])
  cols = zarr_io.read_region(path, [10, 3], [20, 9]).numpy()      # not whole rows: general path
  np.testing.assert_array_equal(cols, full[10:20, 3:9])
  os.remove(os.path.join(path, "2.0"))
  with pytest.raises(FileNotFoundError):
    zarr_io.read_region(path, [0, 0], [1000, 24])


def test_edge_case_leaves_round_trip(tmp_path):
  """Empty arrays, 0-d scalars (they stay 0-d), bf16 and integer leaves, nested containers."""
  state = {"empty": torch.zeros(0, 4), "half": torch.randn(5, 3).to(torch.bfloat16), "count": torch.tensor(7),
           "grid": torch.arange(10).view(2, 5), "nested": {"v": torch.randn(3), "rate": torch.tensor(2.5)}}
  m = ckpt.CheckpointManager(str(tmp_path))
  m.save(1, state)
  m.wait_until_finished()
  out = m.restore(1)
  for got, want in ((out[k], state[k]) for k in ("empty", "half", "count", "grid")):
    assert got.dtype == want.dtype and got.shape == want.shape and torch.equal(got, want)
  assert torch.equal(out["nested"]["v"], state["nested"]["v"]) and out["nested"]["rate"].shape == ()


def test_ocdbt_store_roundtrip_with_compressed_multilevel_tree(tmp_path):
  """The key-value layer alone: 600 keys, values inline and out of line, a fan-out of 8 (three tree levels),
  zstd-compressed nodes; a flipped byte in the manifest is detected by its checksum."""
  from recml_b200.ckpt import ocdbt
  d = str(tmp_path / "kv")
  w = ocdbt.Writer(d, max_inline_value_bytes=64)
  vals = {f"leaf{i}/.zarray": b"{meta %d}" % i for i in range(300)}
  vals.update({f"leaf{i}/0.0": os.urandom(500 + i) for i in range(300)})
  for k, v in vals.items():
    w.add(k, v)
  w.commit(compress_nodes=True, node_fanout=8)
  assert sorted(os.listdir(d)) == ["d", "manifest.ocdbt"]
  s = ocdbt.Store(d)
  assert s.keys() == sorted(vals)
  assert all(s.get(k) == v for k, v in vals.items())
  s.close()
  raw = bytearray(open(os.path.join(d, "manifest.ocdbt"), "rb").read())
  raw[20] ^= 0xFF
  open(os.path.join(d, "manifest.ocdbt"), "wb").write(bytes(raw))
  with pytest.raises(IOError, match="checksum"):
    ocdbt.Store(d)


def test_checkpoint_in_ocdbt_form_is_detected_and_restored(tmp_path):
  """`use_ocdbt=True` writes the item as `manifest.ocdbt` + `ocdbt.process_0/`; restore (whole tree, and a
  sharded target reading its block) detects the form from the files."""
  tree = {"step": torch.tensor(7), "params": {"w": torch.arange(24, dtype=torch.float32).reshape(6, 4),
                                               "b": torch.randn(5).to(torch.bfloat16)}}
  m = ckpt.CheckpointManager(str(tmp_path), async_save=False, use_ocdbt=True, compressor="zstd" if zarr_io.zstd_available() else None)
  m.save(3, tree)
  item = tmp_path / "3" / "state"
  names = sorted(os.listdir(item))
  assert "manifest.ocdbt" in names and "ocdbt.process_0" in names and "params.w" not in names
  assert json.load(open(item / "_METADATA"))["use_ocdbt"] is True
  back = ckpt.CheckpointManager(str(tmp_path), async_save=False).restore(3)
  torch.testing.assert_close(back["params"]["w"], tree["params"]["w"])
  torch.testing.assert_close(back["params"]["b"], tree["params"]["b"])
  assert int(back["step"]) == 7
  tgt = {"params": {"w": ckpt.ShardedLeaf(torch.zeros(3, 4), (6, 4), (1, 0), (3, 4))}}
  torch.testing.assert_close(m.restore(3, target=tgt)["params"]["w"], tree["params"]["w"][3:])


def test_truncated_chunk_raises_instead_of_restoring_zeros(tmp_path):
  """A chunk file that lost its tail is an error on restore, with or without a sharded target; the one short
  form that is accepted is the last chunk along the first dimension stored with exactly the rows that exist."""
  tree = {"w": torch.arange(4096, dtype=torch.float32).reshape(64, 64), "b": torch.randn(33).to(torch.bfloat16)}
  m = ckpt.CheckpointManager(str(tmp_path), async_save=False)
  m.save(1, tree)
  back = ckpt.CheckpointManager(str(tmp_path), async_save=False).restore(1, target=tree)
  assert torch.equal(back["w"], tree["w"])
  chunk = tmp_path / "1" / "state" / "w" / "0.0"
  raw = chunk.read_bytes()
  chunk.write_bytes(raw[:len(raw) - 100])
  with pytest.raises(IOError, match="chunk holds"):
    ckpt.CheckpointManager(str(tmp_path), async_save=False).restore(1, target=tree)
  # a writer that clips its last chunk: 10 rows of 4 in chunks of 4 rows, the last chunk stored with 2 rows
  d = tmp_path / "clipped"
  os.makedirs(d)
  full = np.arange(40, dtype=np.float32).reshape(10, 4)
  zarr_io.write_zarray(str(d), (10, 4), (4, 4), "<f4", None)
  for ci in range(3):
    zarr_io.write_chunk(str(d), [ci, 0], full[ci * 4:(ci + 1) * 4], None)
  assert torch.equal(zarr_io.read_region(str(d)), torch.from_numpy(full))
  assert torch.equal(zarr_io.read_region(str(d), [7, 1], [10, 3]), torch.from_numpy(full[7:10, 1:3]))
  (d / "2.0").write_bytes((d / "2.0").read_bytes()[:-4])
  with pytest.raises(IOError, match="clipped last chunk"):
    zarr_io.read_region(str(d))


def test_raw_chunks_carry_segment_checksums(tmp_path, monkeypatch):
  """Uncompressed chunks get a CRC-32C per 16 MB segment in a dot-file beside them; a flipped bit fails the restore
  on the fast whole-file path and on the general path, a checkpoint without the dot-files still restores, and
  RECML_CKPT_CHECKSUMS=0 switches the check off."""
  monkeypatch.setattr(zarr_io, "_SEGMENT_BYTES", 4096)            # several segments in a small array
  tree = {"w": torch.arange(3 * 4096, dtype=torch.float32).reshape(96, 128), "s": torch.tensor(2.5)}
  m = ckpt.CheckpointManager(str(tmp_path), async_save=False)
  m.save(1, tree)
  leaf = tmp_path / "1" / "state" / "w"
  side = json.load(open(leaf / ".0.0.crc32c"))
  assert side["segment_bytes"] == 4096 and len(side["crc32c"]) == 12
  assert torch.equal(m.restore(1, target=tree)["w"], tree["w"])
  raw = bytearray((leaf / "0.0").read_bytes())
  raw[5000] ^= 0x01
  (leaf / "0.0").write_bytes(bytes(raw))
  with pytest.raises(IOError, match=r"checksum mismatch in bytes \[4096, 8192\)"):
    m.restore(1, target=tree)                                      # whole rows, read by the native reader
  with pytest.raises(IOError, match="checksum mismatch"):
    zarr_io.read_region(str(leaf), [0, 3], [96, 64])               # a column range: the general path
  monkeypatch.setenv("RECML_CKPT_CHECKSUMS", "0")
  assert not torch.equal(m.restore(1, target=tree)["w"], tree["w"])   # unchecked: the flipped bit comes back
  monkeypatch.delenv("RECML_CKPT_CHECKSUMS")
  os.remove(leaf / ".0.0.crc32c")                                  # another writer's checkpoint has no dot-files
  assert m.restore(1, target=tree)["w"].shape == (96, 128)


def test_ocdbt_large_values_go_through_the_parallel_zero_copy_path(tmp_path):
  """A leaf larger than one 16 MB I/O segment in OCDBT form: written from the array's own memory and read
  straight into the restored tensor (several threads, several segments); a row range of it and a store-level
  `read_into` with a buffer of the wrong size take their own paths."""
  from recml_b200.ckpt import ocdbt
  big = torch.arange(5_000_000, dtype=torch.float32).reshape(50_000, 100) * 0.5        # 20 MB
  tree = {"big": big, "half": torch.randn(1000, 8).to(torch.bfloat16), "step": torch.tensor(4)}
  m = ckpt.CheckpointManager(str(tmp_path), async_save=True, use_ocdbt=True)
  m.save(1, tree)
  m.wait_until_finished()
  back = ckpt.CheckpointManager(str(tmp_path), async_save=False).restore(1, target=tree)
  assert torch.equal(back["big"], big) and torch.equal(back["half"], tree["half"]) and int(back["step"]) == 4
  item = os.path.join(str(tmp_path), "1", "state")
  rows = zarr_io.read_region(ocdbt.leaf_path(item, "big"), [123, 0], [4567, 100])
  assert torch.equal(rows, big[123:4567])
  store = ocdbt.open_store(item)
  buf = np.empty(big.numel(), dtype=np.float32)
  store.read_into("big/0.0", buf)
  assert np.array_equal(buf, big.numpy().reshape(-1))
  with pytest.raises(ValueError, match="holds"):
    store.read_into("big/0.0", np.empty(10, dtype=np.float32))
  part = np.empty(1000, dtype=np.float32)
  store.read_range_into("big/0.0", 4 * 777, part)                     # floats 777 .. 1776 of the value
  assert np.array_equal(part, big.numpy().reshape(-1)[777:1777])
  with pytest.raises(IOError, match="code -2"):
    store.read_range_into("big/0.0", big.numel() * 4 - 100, part)     # runs past the value
  with pytest.raises(FileNotFoundError):
    store.read_range_into("nothing/0", 0, part)


def test_async_save_snapshots_host_tensors(tmp_path):
  """An asynchronous save of tensors that live in host memory writes what they held when `save` was called, not
  what later steps made of them while the writer thread ran (device tensors are copied to the host anyway)."""
  w = torch.zeros(2_000_000)
  m = ckpt.CheckpointManager(str(tmp_path), async_save=True)
  m.save(1, {"w": w, "n": np.zeros(4, dtype=np.float32)})
  for k in range(1, 30):          # "training" goes on while the chunk is written
    w.add_(1.0)
  m.wait_until_finished()
  back = m.restore(1)
  assert float(back["w"].abs().max()) == 0.0
