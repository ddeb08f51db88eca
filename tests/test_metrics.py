"""Golden-value tests for the metrics library (cases follow the reference's table-driven tests in
`recml/core/metrics/*_test.py`); every metric is checked through `compute()` and
`localize().compute()`."""
import numpy as np
import pytest
import torch

from recml_b200 import metrics as M


def _both(metric):
  return np.asarray(metric.compute()), np.asarray(metric.localize().compute())


CONF_CASES = [
    (np.array([[0, 0, 1, 1, 0], [1, 1, 1, 1, 1], [0, 1, 0, 1, 0], [1, 1, 1, 1, 1]]),
     np.array([[0, 1, 0, 1, 0], [0, 0, 1, 1, 1], [1, 1, 1, 1, 0], [0, 0, 0, 0, 1]]), None, [0.5],
     [7.0], [3.0], [7.0], [3.0]),
    (np.array([[0, 0, 1, 1, 0], [1, 1, 1, 1, 1], [0, 1, 0, 1, 0], [1, 1, 1, 1, 1]]),
     np.array([[0, 1, 0, 1, 0], [0, 0, 1, 1, 1], [1, 1, 1, 1, 0], [0, 0, 0, 0, 1]]),
     np.array([1.0, 1.5, 2.0, 2.5]), [0.5], [12.0], [4.0], [14.0], [5.0]),
    (np.array([[0.9, 0.2, 0.8, 0.1], [0.2, 0.9, 0.7, 0.6], [0.1, 0.2, 0.4, 0.3], [0.0, 1.0, 0.7, 0.3]]),
     np.array([[0, 1, 1, 0], [1, 0, 0, 0], [0, 0, 0, 0], [1, 1, 1, 1]]), None, [0.15, 0.5, 0.85],
     [6.0, 3.0, 1.0], [2.0, 5.0, 7.0], [7.0, 4.0, 2.0], [1.0, 4.0, 6.0]),
    (np.array([[0.9, 0.2, 0.8, 0.1], [0.2, 0.9, 0.7, 0.6], [0.1, 0.2, 0.4, 0.3], [0.0, 1.0, 0.7, 0.3]]),
     np.array([[0, 1, 1, 0], [1, 0, 0, 0], [0, 0, 0, 0], [1, 1, 1, 1]]),
     np.array([[1.0, 2.0, 3.0, 5.0], [7.0, 11.0, 13.0, 17.0], [19.0, 23.0, 29.0, 31.0], [5.0, 15.0, 10.0, 0]]),
     [0.15, 0.5, 0.85], [37.0, 28.0, 15.0], [24.0, 107.0, 137.0], [125.0, 42.0, 12.0], [5.0, 14.0, 27.0]),
]


@pytest.mark.parametrize("pred,lab,w,th,tp,tn,fp,fn", CONF_CASES)
def test_estimate_confusion_matrix(pred, lab, w, th, tp, tn, fp, fn):
  out = M.estimate_confusion_matrix(pred, lab, w, th)
  for got, want in zip(out, (tp, tn, fp, fn)):
    np.testing.assert_allclose(got.numpy(), want)


def test_confusion_unsorted_thresholds_and_errors():
  p, l = np.array([0.1, 0.6, 0.9]), np.array([0, 1, 1])
  a = M.estimate_confusion_matrix(p, l, None, [0.8, 0.2])
  b = M.estimate_confusion_matrix(p, l, None, [0.2, 0.8])
  np.testing.assert_allclose(a[0].numpy(), b[0].numpy()[::-1])
  with pytest.raises(ValueError):
    M.estimate_confusion_matrix(np.zeros((2, 2)), np.zeros((2, 3)))
  with pytest.raises(ValueError):
    M.estimate_confusion_matrix(np.zeros((2, 2)), np.zeros((2, 2)), np.zeros((3,)))


def test_precision_recall_fbeta():
  y = np.array([0, 1, 1, 0, 1, 1]); p = np.array([0.1, 0.9, 0.8, 0.7, 0.2, 0.6])
  # threshold .5: tp=3 fp=1 fn=1
  for m, want in ((M.precision(y, p), 0.75), (M.recall(y, p), 0.75), (M.f1_score(y, p), 0.75)):
    for v in _both(m):
      np.testing.assert_allclose(v, want, rtol=1e-6)
  f2 = M.fbeta_score(y, p, beta=2.0)
  np.testing.assert_allclose(f2.compute(), (0.75 * 0.75 * 3) / (0.75 * 2 + 0.75))
  np.testing.assert_allclose(M.precision(y, p, threshold=[0.5, 0.85]).compute(), [0.75, 1.0])
  merged = M.precision(y, p).merge(M.precision(y, p))
  np.testing.assert_allclose(merged.compute(), 0.75)


def test_aucpr_goldens():
  y, p = np.array([0, 0, 1, 1]), np.array([0, 0.5, 0.3, 0.9], dtype="float32")
  for v in _both(M.aucpr(y, p, np.array([1, 2, 3, 4]), num_thresholds=3)):
    np.testing.assert_allclose(v, 2.416 / 7 + 4 / 7, rtol=1e-3)
  for v in _both(M.aucpr(y, p, np.array([-1, -2, -3, -4]), num_thresholds=3)):
    np.testing.assert_allclose(v, 0.0, atol=1e-7)


@pytest.mark.parametrize("y,p,w,logits,want", [
    ([0, 0, 1, 1], [0, 0, 1, 1], None, False, 1.0),
    ([0, 0, 1, 1], [0, 0.5, 0.3, 0.9], None, False, 0.75),
    ([0, 0, 1, 1], list(-np.log(1.0 / (np.array([0, 0.5, 0.3, 0.9]) + 1e-12) - 1.0)), None, True, 0.75),
    ([0, 0, 1, 1], [0, 0.5, 0.3, 0.9], [1, 2, 3, 4], False, 0.7855)])
def test_aucroc_goldens(y, p, w, logits, want):
  m = M.aucroc(np.array(y), np.array(p), None if w is None else np.array(w), from_logits=logits, num_thresholds=3)
  for v in _both(m):
    np.testing.assert_allclose(v, want, rtol=1e-3)


@pytest.mark.parametrize("w,recall,want", [(None, 0.8, 2.0 / 3), (None, 0.6, 0.75),
                                           ([2, 1, 2, 1, 2, 1, 2, 2, 1, 2], 7.0 / 8, 0.7)])
def test_precision_at_recall(w, recall, want):
  y = np.array([0, 0, 0, 0, 0, 1, 1, 1, 1, 1])
  p = np.array([0.0, 0.1, 0.2, 0.5, 0.6, 0.2, 0.5, 0.6, 0.8, 0.9])
  m = M.precision_at_recall(y, p, None if w is None else np.array(w), recall=recall)
  for v in _both(m):
    np.testing.assert_allclose(v, want, rtol=1e-3)
  with pytest.raises(ValueError):
    m.merge(M.precision_at_recall(y, p, recall=0.123))


def test_mean_metrics_goldens():
  acc = M.accuracy(np.array([1, 0, 1, 0]), np.array([[0.2, 0.8], [0.8, 0.2], [0.1, 0.9], [0.6, 0.4]]))
  for v in _both(acc):
    np.testing.assert_allclose(v, 1.0)
  acc = M.accuracy(np.array([[1, 0, 1, 0]]), np.array([[[0.2, 0.8], [0.1, 0.9], [0.3, 0.7], [0.4, 0.6]]]),
                   np.array([[1, 2, 3, 4]]))
  np.testing.assert_allclose(acc.compute(), 0.4)
  y = np.array([[1], [4], [2], [3], [3], [1], [0], [5]])
  p = np.array([[[0.1, 0.7, 0.5, 0.3, 0.2, 0.0]], [[0.2, 0.8, 0.0, 0.1, 0.4, 0.3]], [[0.1, 0.2, 0.4, 0.8, 0.0, 0.3]],
                [[1.0, 0.9, 0.1, 0.3, 0.2, 0.0]]] * 2)
  for k, want in zip([1, 2, 3, 4, 5, 6], [0.25, 0.5, 0.75, 0.75, 0.875, 1.0]):
    for v in _both(M.top_k_accuracy(y, p, k=k)):
      np.testing.assert_allclose(v, want)
  m = M.top_k_accuracy(np.array([0, 1, 1, 0]), np.array([[0.1, 0.7], [0.2, 0.4], [0.1, 0.3], [0.2, 0.1]]),
                       np.array([0.2, 0.6, 0.1, 0.1]), k=1)
  np.testing.assert_allclose(m.compute(), 0.8)
  np.testing.assert_allclose(M.binary_accuracy(np.array([1, 0, 1, 0]), np.array([0.4, 0.6, 0.8, 0.2])).compute(), 0.5)
  np.testing.assert_allclose(M.binary_accuracy(np.array([[1, 0, 1, 0]]), np.array([[0.8, 0.6, 0.7, 0.6]]),
                                               np.array([[1, 2, 3, 4]]), threshold=0.75).compute(), 0.7)
  np.testing.assert_allclose(M.mean_squared_error(np.array([0.3, 0.5, 0.7, 0.9]),
                                                  np.array([0.4, 0.6, 0.8, 0.2])).compute(), 0.13, rtol=1e-3)
  np.testing.assert_allclose(M.mean_squared_error(np.array([[0.3, 0.6, 0.2, 0.6]]), np.array([[0.8, 0.6, 0.7, 0.6]]),
                                                  np.array([0.5])).compute(), 0.125, rtol=1e-3)


def test_reduction_metrics_and_broadcast_rules():
  m = M.mean(np.array([1.0, 2.0, 3.0]))
  np.testing.assert_allclose(m.merge(M.mean(np.array([5.0]))).compute(), 11.0 / 4)
  np.testing.assert_allclose(M.mean(np.array([[1., 2.], [3., 4.]]), np.array([1., 0.])).compute(), 1.5)
  np.testing.assert_allclose(M.mean(np.array([[1., 2.], [3., 4.]]), np.array([[1.], [3.]])).compute(), (3 + 21) / 8)
  np.testing.assert_allclose(M.sum(np.array([1., 2.]), np.array([2., 2.])).compute(), 6.0)
  np.testing.assert_allclose(M.mean(np.float32(4.0)).compute(), 4.0)
  with pytest.raises(ValueError):
    M.mean(np.zeros((2, 3)), np.zeros((2, 2)))
  with pytest.raises(ValueError):
    M.mean(np.zeros((2, 3)), np.zeros((3,)))
  Sq = M.Mean.from_fun(lambda a, b: (a - b) ** 2)
  np.testing.assert_allclose(Sq.from_model_output(np.array([1., 2.]), np.array([0., 0.]),
                                                  weights=np.array([1., 3.])).compute(), 13 / 4)


def test_scalar_metric_last_value_wins():
  a, b = M.scalar(1.0), M.scalar(torch.tensor([2.0]))
  assert float(a.merge(b).compute()) == 2.0
  assert float(b.localize().compute()) == 2.0
  with pytest.raises(ValueError):
    M.scalar(np.zeros(3))


def test_ranking_metrics():
  logits = torch.tensor([[0.1, 0.9, 0.3, 0.2], [0.5, 0.1, 0.4, 0.45], [0.0, 0.2, 0.1, 0.9]])
  y = torch.tensor([1, 2, 0])          # ranks 1, 3, 4
  np.testing.assert_allclose(M.rank_of_target(logits, y).numpy(), [1, 3, 4])
  np.testing.assert_allclose(M.recall_at_k(y, logits, k=3).compute(), 2 / 3)
  np.testing.assert_allclose(M.hit_rate_at_k(y, logits, k=1).compute(), 1 / 3)
  np.testing.assert_allclose(M.ndcg_at_k(y, logits, k=3).compute(), (1 + 1 / np.log2(4)) / 3, rtol=1e-6)
  np.testing.assert_allclose(M.mrr(y, logits).compute(), (1 + 1 / 3 + 1 / 4) / 3, rtol=1e-6)
  np.testing.assert_allclose(M.recall_at_k(y, logits, torch.tensor([1., 0., 1.]), k=3).compute(), 0.5)


def test_accumulator_and_writer(tmp_path):
  w = M.AsyncMultiWriter(log_dir=str(tmp_path), name="train")
  acc = M.MetricAccumulator(w)
  acc.accumulate({"loss": M.mean(np.array([1.0, 3.0])), "lr": M.scalar(0.1)}, 0)
  acc.accumulate({"loss": M.mean(np.array([5.0])), "lr": M.scalar(0.2)}, 1)
  out = acc.compute_and_log_scalars(1)
  np.testing.assert_allclose(out["loss"], 3.0)
  np.testing.assert_allclose(out["lr"], 0.2, rtol=1e-6)
  assert any(f.startswith("events.out") for f in __import__("os").listdir(tmp_path / "train"))
  assert acc.compute_and_log_scalars(2) == {}


def test_histogram_auc_states_match_confusion_states():
  """AUC metrics that keep the loss kernel's histograms as state give the same value as the ones built from the
  confusion counts, also after merging steps."""
  import numpy as np
  import torch
  from recml_b200 import metrics as M
  rng = np.random.default_rng(0)
  T = 200
  parts = []
  for _ in range(3):
    hp = torch.from_numpy(rng.random(T + 1).astype(np.float32) * 10)
    hn = torch.from_numpy(rng.random(T + 1).astype(np.float32) * 30)
    parts.append((hp, hn))
  for hist_cls, cls in ((M.HistogramAUCPR, M.AUCPR), (M.HistogramAUCROC, M.AUCROC)):
    a = b = None
    for hp, hn in parts:
      x = hist_cls(pos_hist=hp, neg_hist=hn)
      tp, tn, fp, fn = M.confusion_from_histograms(hp, hn)
      y = cls(true_positives=tp, true_negatives=tn, false_positives=fp, false_negatives=fn)
      a = x if a is None else a.merge(x)
      b = y if b is None else b.merge(y)
    assert abs(a.localize().compute() - b.localize().compute()) < 1e-5
