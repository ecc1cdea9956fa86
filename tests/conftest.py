"""Test configuration: path to the in-tree package, the `gpu` marker."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "pallas-mosaic-gpu_b200"))
sys.path.insert(0, ROOT)

# GPU tests synchronise after every kernel call and raise if a kernel reported a
# bounded wait that ran out.
os.environ.setdefault("SPLASH_CHECK_STATUS", "1")


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


def pytest_collection_modifyitems(config, items):
  try:
    import torch
    has_gpu = torch.cuda.is_available()
  except Exception:  # noqa: BLE001
    has_gpu = False
  if has_gpu:
    return
  skip = pytest.mark.skip(reason="no CUDA device")
  for item in items:
    if "gpu" in item.keywords:
      item.add_marker(skip)
