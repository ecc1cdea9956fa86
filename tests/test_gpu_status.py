"""The device status word reaches the caller without an explicit check.

A kernel that abandons a bounded wait leaves the status word non-zero, and every later
launch given that word returns at entry.  No kernel is made to time out here: the word is
set from the host, which is all a later launch can see of an earlier failure.
"""

import numpy as np
import pytest
import torch

import splash_attention_mgpu as sa
from splash_attention_mgpu import _ffi
from splash_attention_mgpu import splash_attention as api

pytestmark = pytest.mark.gpu


def test_failure_surfaces_at_the_next_call_and_clears(monkeypatch):
  monkeypatch.delenv("SPLASH_CHECK_STATUS", raising=False)
  dev = torch.device("cuda:0")
  s, d = 256, 64
  g = torch.Generator().manual_seed(0)
  q, k, v = (torch.randn(2, s, d, generator=g).to(torch.bfloat16).to(dev) for _ in range(3))
  kernel = sa.make_splash_mha(sa.CausalMask((s, s)))
  good = kernel(q, k, v)
  torch.cuda.synchronize()
  sa.check_device_status()
  # What a timed-out kernel leaves behind: {code, site, block, step}.
  api._status_word(dev).copy_(torch.tensor([1, 9, 3, 5], dtype=torch.int32))
  kernel(q, k, v)            # returns at entry on the device; its outputs are not valid
  torch.cuda.synchronize()   # the queued copy of the word has landed
  with pytest.raises(_ffi.SplashLibraryError, match="wait site 9, block 3, step 5"):
    kernel(q, k, v)
  # The word was cleared by the failing call: the library works again.
  again = kernel(q, k, v)
  torch.cuda.synchronize()
  sa.check_device_status()
  assert torch.equal(again, good)


def test_explicit_check_reports_and_clears():
  dev = torch.device("cuda:0")
  api._status_word(dev).copy_(torch.tensor([1, 2, 0, 0], dtype=torch.int32))
  with pytest.raises(_ffi.SplashLibraryError, match="wait site 2"):
    sa.check_device_status()
  sa.check_device_status()
  assert api._status_word(dev).cpu().tolist() == [0, 0, 0, 0]


def test_status_copy_does_not_queue_behind_the_callers_copies(monkeypatch):
  """A caller that streams results to the host keeps a bulk device-to-host copy in flight.  The
  16-byte copy of the status word must not sit behind it on the caller's stream, or the caller's
  next kernels wait for the whole bulk copy: two calls in a row have to finish while a copy of
  several hundred MiB, started before them on another stream, is still running."""
  monkeypatch.delenv("SPLASH_CHECK_STATUS", raising=False)
  dev = torch.device("cuda:0")
  s, d = 256, 64
  g = torch.Generator().manual_seed(1)
  q, k, v = (torch.randn(2, s, d, generator=g).to(torch.bfloat16).to(dev) for _ in range(3))
  kernel = sa.make_splash_mha(sa.CausalMask((s, s)))
  kernel(q, k, v)
  kernel(q, k, v)
  torch.cuda.synchronize()
  big = torch.empty(768 << 20, dtype=torch.uint8, device=dev)
  host = torch.empty(768 << 20, dtype=torch.uint8).pin_memory()
  copies = torch.cuda.Stream(dev)
  copy_done, calls_done = torch.cuda.Event(), torch.cuda.Event()
  torch.cuda.synchronize()
  with torch.cuda.stream(copies):
    host.copy_(big, non_blocking=True)   # >= 10 ms on a PCIe 5 link
    copy_done.record(copies)
  kernel(q, k, v)
  kernel(q, k, v)                        # would wait for the first call's status copy, hence for `big`
  calls_done.record(torch.cuda.current_stream(dev))
  calls_done.synchronize()
  still_copying = not copy_done.query()
  torch.cuda.synchronize()
  sa.check_device_status()
  assert still_copying, "the calls finished only after the bulk copy: they were queued behind it"
