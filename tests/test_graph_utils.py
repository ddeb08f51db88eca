"""Host-side pieces of the CUDA-graph step wrapper that do not need a GPU."""
import torch

from recml_b200 import metrics as M
from recml_b200.utils import graphs


def test_fast_clone_gathers_per_dtype_and_keeps_structure():
  """The step's outputs leave the replayed graph through one concatenation per dtype: the copies must equal the
  sources, keep shapes / dtypes / tree structure, and must not alias the (static) sources."""
  a, b = torch.arange(6, dtype=torch.float32).reshape(2, 3), torch.tensor(3.5)
  c, d = torch.tensor([1, 2, 3], dtype=torch.int64), torch.tensor(7, dtype=torch.int64)
  tree = {"loss": M.mean(b), "pair": (a, c), "count": d, "lonely": torch.tensor([1.0], dtype=torch.float64)}
  out = graphs._clone_tree(tree, fast=True)
  assert isinstance(out["loss"], type(tree["loss"])) and set(out) == set(tree)
  for x, y in ((out["pair"][0], a), (out["pair"][1], c), (out["count"], d), (out["lonely"], tree["lonely"])):
    assert x.dtype == y.dtype and x.shape == y.shape and torch.equal(x, y) and x.data_ptr() != y.data_ptr()
  a.add_(1.0)
  b.add_(1.0)
  assert float(out["pair"][0][0, 0]) == 0.0 and float(out["loss"].localize().compute()) == 3.5
