"""Sequence-model layers on CPU: parameter counts of the reference tests (`hstu_test.py`,
`sasrec_test.py`, `bert4rec_test.py`), shapes, Mamba SSD vs the recurrence (`mamba_test.py`), layer
utilities (`utils_test.py`), jagged vs dense HSTU, and the tiny HSTU retrieval experiment."""
import math

import numpy as np
import pytest
import torch

from recml_b200.layers import bert4rec, hstu, mamba, sasrec, utils
from recml_b200.ops import hstu_attention as A
from recml_b200.ops import norm as norm_ops
from recml_b200.ops import ssd

IDS = torch.tensor([[1, 2, 3], [4, 5, 0]])
PAD = torch.tensor([[1, 1, 1], [1, 1, 0]])
n_params = lambda m: sum(p.numel() for p in m.parameters())


def test_hstu_param_count_and_shape():
  m = hstu.HSTU(vocab_size=500, max_positions=20, model_dim=32, num_heads=4, num_layers=3, dropout=0.1)
  assert n_params(m) == 500 * 32 + 20 * 32 + 3 * ((32 * 32 * 4 + 32 * 32) + (2 * 32) * 2) + 2 * 32 + 500 * 32
  assert m(IDS, padding_mask=PAD).shape == (2, 3, 500)
  with pytest.raises(ValueError):
    m(IDS)


def test_sasrec_and_bert4rec_param_counts():
  blk = ((32 + 1) * 32 * 3 + (32 + 1) * 32) + 2 * 32 + (32 + 1) * 64 + (64 + 1) * 32 + 2 * 32
  m = sasrec.SASRec(vocab_size=500, max_positions=20, model_dim=32, mlp_dim=64, num_heads=4, num_layers=3, dropout=0.1)
  assert n_params(m) == 500 * 32 + 20 * 32 + 3 * blk + 2 * 32
  assert m(IDS, padding_mask=PAD).shape == (2, 3, 500)
  b = bert4rec.BERT4Rec(vocab_size=500, max_positions=20, num_types=5, model_dim=32, mlp_dim=64, num_heads=4,
                        num_layers=3, dropout=0.1)
  assert n_params(b) == 500 * 32 + 5 * 32 + 20 * 32 + 2 * 32 + 3 * blk + (32 + 1) * 32 + 2 * 32 + 500
  out = b(IDS, type_ids=torch.zeros_like(IDS), padding_mask=PAD, mask_positions=torch.tensor([[0], [1]]))
  assert out.shape == (2, 1, 500)
  with pytest.raises(ValueError):
    b(IDS)


def test_sasrec_is_causal():
  torch.manual_seed(0)
  m = sasrec.SASRec(vocab_size=50, max_positions=8, model_dim=16, mlp_dim=32, num_heads=2, num_layers=2).eval()
  a = torch.tensor([[1, 2, 3, 4]])
  b = torch.tensor([[1, 2, 9, 9]])
  ya, yb = m(a, padding_mask=torch.ones_like(a)), m(b, padding_mask=torch.ones_like(b))
  torch.testing.assert_close(ya[:, :2], yb[:, :2])
  assert not torch.allclose(ya[:, 2:], yb[:, 2:])


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_ssd_chunked_matches_recurrence(seed):
  g = torch.Generator().manual_seed(seed)
  B, L, H, P, N = 1, 256, 4, 16, 16
  x = torch.randn(B, L, H, P, generator=g)
  a = -torch.rand(B, L, H, generator=g)
  b, c = torch.randn(B, L, 1, N, generator=g), torch.randn(B, L, 1, N, generator=g)
  torch.testing.assert_close(ssd.ssd_chunked(x, a, b, c, 64), ssd.ssd_recurrent(x, a, b, c), atol=1e-4, rtol=1e-4)
  init = torch.randn(B, H, P, N, generator=g)
  torch.testing.assert_close(ssd.ssd_chunked(x, a, b, c, 32, init), ssd.ssd_recurrent(x, a, b, c, init), atol=1e-4,
                             rtol=1e-4)


def test_mamba4rec_shapes_and_padding():
  m = mamba.Mamba4Rec(500, 32, 4, 4, 2, 2, d_state=16, chunk_size=8)
  y = m(IDS, padding_mask=PAD)
  assert y.shape == (2, 3, 500)
  h = mamba.Mamba4Rec(500, 32, 4, 4, 2, 2, d_state=16, chunk_size=8, add_head=False)(IDS, padding_mask=PAD)
  assert float(h[1, 2].abs().max()) == 0.0
  conv = ssd.causal_depthwise_conv1d_silu(torch.ones(1, 5, 2), torch.tensor([[0., 0., 0., 1.], [1., 1., 1., 1.]]))
  torch.testing.assert_close(conv[0, :, 0], torch.nn.functional.silu(torch.ones(5)))
  torch.testing.assert_close(conv[0, :, 1], torch.nn.functional.silu(torch.tensor([1., 2., 3., 4., 4.])))


def test_layer_utils():
  mask = torch.tensor([[1, 1, 0]])
  np.testing.assert_array_equal(utils.make_attention_mask(mask)[0].numpy(), [[1, 1, 0], [1, 1, 0], [0, 0, 0]])
  np.testing.assert_array_equal(utils.make_causal_mask(mask)[0].numpy(), [[1, 0, 0], [1, 1, 0], [0, 0, 0]])
  x = torch.tensor([[[3.0, 4.0], [0.0, 0.0]]])
  torch.testing.assert_close(utils.norm_embedding_post_processor(x)[0, 0], torch.tensor([0.6, 0.8]))
  torch.testing.assert_close(utils.relu_squared(torch.tensor([-1.0, 2.0])), torch.tensor([0.0, 4.0]))
  r = utils.apply_rotary_encoding(torch.ones(1, 2, 1, 4), max_wavelength=10000)
  torch.testing.assert_close(r[0, 0, 0], torch.ones(4))
  c, s_ = math.cos(1.0), math.sin(1.0)
  torch.testing.assert_close(r[0, 1, 0, 0], torch.tensor(c - s_))
  torch.testing.assert_close(r[0, 1, 0, 2], torch.tensor(c + s_))
  with pytest.raises(ValueError):
    utils.apply_rotary_encoding(torch.ones(1, 2, 1, 3), max_wavelength=10)
  assert utils.large_negative_for_attention(torch.float16) == -3e4


def test_relative_bias_layers_and_jagged_equals_dense():
  torch.manual_seed(0)
  N = 6
  pos = hstu.RelativePositionalBias(N)
  b = pos(torch.zeros(1, N))
  assert b.shape == (1, N, N)
  assert float(b[0, 2, 5]) == float(pos.pos_biases[(5 - 2) + N - 1])
  tb = hstu.RelativeBucketedTimeAndPositionBasedBias(8, position_bias_layer=pos)
  ts = torch.tensor([[0, 10, 100, 1000, 5000, 9000]])
  full = tb(ts)
  i, j = 1, 0
  want = tb.ts_w[min(int(math.log(100 - 0) / 0.301), 8)] + pos.pos_biases[(j - i) + N - 1]
  torch.testing.assert_close(full[0, i, j], want)
  # packed attention == dense attention with the same causal mask and bias
  lengths = [6, 3]
  q, k, v = (torch.randn(9, 2, 8) for _ in range(3))
  offs = torch.tensor([0, 6, 9], dtype=torch.int32)
  tsp = torch.cat([ts[0], torch.tensor([5, 50, 500])])
  out = A.jagged_attention_reference(q, k, v, offs, N, pos_w=pos.pos_biases, ts_w=tb.ts_w, timestamps=tsp)
  dense = A.pointwise_attention_dense(q[None, :6], k[None, :6], v[None, :6], torch.tril(torch.ones(1, 6, 6)), full)
  torch.testing.assert_close(out[:6], dense[0], atol=1e-5, rtol=1e-5)


def test_pointwise_attention_api_masks():
  torch.manual_seed(1)
  q, k, v = (torch.randn(1, 5, 1, 4) for _ in range(3))
  seg = torch.tensor([[0, 0, 1, 1, 1]])
  out = A.pointwise_attention("causal", q, k, v, q_segment_ids=seg)
  s = torch.einsum("bthd,bshd->bhts", q, k)
  p = torch.nn.functional.silu(s) / 5
  m = torch.tril(torch.ones(5, 5)).bool() & (seg[0][:, None] == seg[0][None, :])
  ref = torch.einsum("bhts,bshd->bthd", p * m, v)
  torch.testing.assert_close(out, ref)
  w = A.pointwise_attention(A.MaskType.CAUSAL, q, k, v, sliding_window_size=2)
  # inclusive window, as the reference's LocalMask(window_size=(2, 2)): query i sees keys i-2 .. i
  m2 = torch.tril(torch.ones(5, 5)).bool() & (torch.arange(5)[None, :] >= torch.arange(5)[:, None] - 2)
  torch.testing.assert_close(w, torch.einsum("bhts,bshd->bthd", p * m2, v))


def test_layer_norm_variants_cpu():
  x = torch.randn(4, 3, 8)
  w, b = torch.rand(8) + 0.5, torch.randn(8)
  torch.testing.assert_close(norm_ops.layer_norm(x, w, b, 1e-6), torch.nn.functional.layer_norm(x, (8,), w, b, 1e-6))
  w2, b2 = torch.rand(3, 8) + 0.5, torch.randn(3, 8)
  torch.testing.assert_close(norm_ops.layer_norm(x, w2, b2, 1e-6, norm_dims=2),
                             torch.nn.functional.layer_norm(x, (3, 8), w2, b2, 1e-6))
  rms = norm_ops.layer_norm(x, w, None, 1e-5, rms=True)
  torch.testing.assert_close(rms, x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w)


def test_tiny_hstu_retrieval_experiment(tmp_path):
  from recml_b200 import config as C, run_experiment
  from recml_b200.examples import hstu_experiment as E
  cfg = E.tiny_experiment(model_dir=str(tmp_path), train_steps=40)
  cfg.trainer.partitioner = C.Config(__import__("recml_b200").DataParallelPartitioner, device="cpu")
  logs = run_experiment(C.build(cfg), "train_and_eval")
  assert logs["train"]["loss"] < 3.0 and "hit@1_sampled" in logs["val"]


def test_layers_round_trip_through_their_config(tmp_path):
  """`get_config()` holds the constructor call (JSON-serialisable, functions as import paths) and
  `from_config` rebuilds a layer with the same parameter shapes — the reference's Keras layers carry the same
  pair (`recml/layers/keras/hstu.py:476-492,623-628`, `sasrec.py:165-170`, `bert4rec.py:194-208`, `mamba.py:747-752`).
  A layer exported without a builder reloads from that config with its weights."""
  import json
  from recml_b200 import serving
  from recml_b200.layers import bert4rec, hstu, mamba, sasrec
  layers = [
      hstu.HSTU(vocab_size=50, max_positions=16, model_dim=32, num_heads=2, num_layers=2, dropout=0.1),
      hstu.HSTUBlock(32, 2, use_bias=True, scaled_pointwise_attn=True),
      hstu.RelativeBucketedTimeAndPositionBasedBias(num_buckets=16, position_bias_layer=hstu.RelativePositionalBias(16)),
      sasrec.SASRec(vocab_size=50, max_positions=16, model_dim=32, mlp_dim=64, num_heads=2, num_layers=1),
      bert4rec.BERT4Rec(vocab_size=50, max_positions=16, num_types=3, model_dim=32, mlp_dim=64, num_heads=2, num_layers=1),
      mamba.Mamba4Rec(50, 32, 2, 4, 1, 2, d_state=16, chunk_size=8),
  ]
  for layer in layers:
    cfg = json.loads(json.dumps(layer.get_config()))
    twin = type(layer).from_config(cfg)
    assert {n: p.shape for n, p in twin.named_parameters()} == {n: p.shape for n, p in layer.named_parameters()}
    assert twin.get_config() == layer.get_config()
  block_cfg = layers[1].get_config()
  assert block_cfg["activation"] == {"callable": "torch.nn.functional.silu"} and block_cfg["use_bias"] is True
  assert layers[0].get_config()["num_layers"] == 2 and layers[0].get_config()["max_seq_len"] is None

  model = layers[3].eval()
  serving.export(model, str(tmp_path / "sasrec"))
  loaded = serving.load(str(tmp_path / "sasrec"), device="cpu")
  ids = torch.randint(1, 50, (3, 16))
  with torch.no_grad():
    torch.testing.assert_close(loaded(ids), model(ids))


def test_compute_output_shape_matches_the_forward():
  from recml_b200.layers import bert4rec, hstu, mamba, sasrec
  ids = torch.randint(1, 50, (3, 16))
  for add_head in (True, False):
    models = [hstu.HSTU(vocab_size=50, max_positions=16, model_dim=32, num_heads=2, num_layers=1, add_head=add_head),
              sasrec.SASRec(vocab_size=50, max_positions=16, model_dim=32, mlp_dim=64, num_heads=2, num_layers=1,
                            add_head=add_head),
              mamba.Mamba4Rec(50, 32, 2, 4, 1, 2, d_state=16, chunk_size=8, add_head=add_head)]
    mask = torch.ones(3, 16, dtype=torch.bool)
    for m in models:
      assert tuple(m.eval()(ids, padding_mask=mask).shape) == tuple(m.compute_output_shape(ids.shape)), type(m).__name__
  b = bert4rec.BERT4Rec(vocab_size=50, max_positions=16, model_dim=32, mlp_dim=64, num_heads=2, num_layers=1).eval()
  pos = torch.randint(0, 16, (3, 5))
  assert tuple(b(ids, padding_mask=torch.ones(3, 16, dtype=torch.bool), mask_positions=pos).shape) == tuple(b.compute_output_shape(ids.shape, pos.shape))


def test_segsum_is_the_log_decay_between_positions():
  from recml_b200.ops import ssd
  x = torch.randn(2, 3, 7, dtype=torch.float64)
  out = ssd.segsum(x)
  for i in range(7):
    for j in range(7):
      want = x[..., j + 1:i + 1].sum(-1) if j <= i else torch.full((2, 3), float("-inf"), dtype=torch.float64)
      torch.testing.assert_close(out[..., i, j], want)
  assert ssd.ssd_minimal_discrete is ssd.ssd_chunked
