import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
  config.addinivalue_line("markers", "multigpu: needs 2+ CUDA devices")


def pytest_collection_modifyitems(config, items):
  try:
    import torch
    has_gpu = torch.cuda.is_available()
    ngpu = torch.cuda.device_count() if has_gpu else 0
  except Exception:  # pylint: disable=broad-except
    has_gpu, ngpu = False, 0
  for item in items:
    if "gpu" in item.keywords and not has_gpu:
      item.add_marker(pytest.mark.skip(reason="no CUDA device"))
    if "multigpu" in item.keywords and ngpu < 2:
      item.add_marker(pytest.mark.skip(reason="needs 2+ CUDA devices"))
