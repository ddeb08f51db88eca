"""Public metrics API (names of `recml/core/metrics/__init__.py:19-34` plus the ranking
metrics the reference README promises)."""
from recml_b200.metrics.base import Metric, ScalarMetric, scalar
from recml_b200.metrics.confusion import (AUCPR, AUCROC, HistogramAUCPR, HistogramAUCROC, FBeta, Precision, PrecisionAtRecall,
                                          Recall, aucpr, aucroc, default_thresholds,
                                          confusion_from_histograms, estimate_confusion_matrix, f1_score,
                                          fbeta_score,
                                          precision, precision_at_recall, recall)
from recml_b200.metrics.mean import (accuracy, binary_accuracy, mean_squared_error,
                                     top_k_accuracy)
from recml_b200.metrics.ranking import (hit_rate_at_k, mrr, ndcg_at_k, rank_of_target,
                                        recall_at_k)
from recml_b200.metrics.reduction import Mean, ReductionMetric, Sum, mean, sum  # pylint: disable=redefined-builtin
from recml_b200.metrics.tools import (AsyncMultiWriter, MetricAccumulator, compute_metrics,
                                      merge_metrics)
