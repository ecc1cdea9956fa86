"""tcgen05 operand descriptors on the device: a single-tile GEMM through the C ABI in
every operand form the attention kernels use, against a plain f32 matmul."""

import ctypes

import numpy as np
import pytest
import torch

from splash_attention_mgpu import _ffi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("a_mode,b_mode", [(0, 0), (2, 1), (0, 1), (1, 0), (1, 1), (2, 0), (4, 2), (0, 2), (4, 0)])
@pytest.mark.parametrize("n,kd", [(128, 128), (64, 64), (256, 64), (64, 256), (128, 192)])
def test_umma_selftest(a_mode, b_mode, n, kd, dtype):
  lib = _ffi.load()
  dev = torch.device("cuda:0")
  g = torch.Generator().manual_seed(n * 1000 + kd + a_mode * 10 + b_mode)
  a = torch.randn(128, kd, generator=g).to(dtype).to(dev)
  b = torch.randn(n, kd, generator=g).to(dtype).to(dev)
  want = a.float() @ b.float().T
  a_in = a.T.contiguous() if a_mode == 1 else a.contiguous()
  b_in = b.T.contiguous() if b_mode == 1 else b.contiguous()
  d = torch.zeros(128, n, dtype=torch.float32, device=dev)
  status = torch.zeros(4, dtype=torch.int32, device=dev)
  rc = lib.splash_selftest_umma(a_in.data_ptr(), b_in.data_ptr(), d.data_ptr(), n, kd, a_mode, b_mode,
                                _ffi.DTYPE_BF16 if dtype == torch.bfloat16 else _ffi.DTYPE_F16,
                                status.data_ptr(), torch.cuda.current_stream().cuda_stream)
  _ffi.check(rc, "selftest")
  torch.cuda.synchronize()
  assert status.tolist() == [0, 0, 0, 0], f"device status {status.tolist()}"
  np.testing.assert_allclose(d.cpu().numpy(), want.cpu().numpy(), atol=2e-2, rtol=1e-3)


def test_a_wait_that_runs_out_is_reported_and_the_context_survives():
  # Mode 3 of the self-test waits on a barrier nothing arrives on: the bounded wait gives
  # up after about a second, the kernel unwinds, and the status word names the wait.
  lib = _ffi.load()
  status = torch.zeros(4, dtype=torch.int32, device="cuda:0")
  a_in = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda:0")
  b_in = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda:0")
  d = torch.zeros(128, 64, dtype=torch.float32, device="cuda:0")
  rc = lib.splash_selftest_umma(a_in.data_ptr(), b_in.data_ptr(), d.data_ptr(), 64, 64, 3, 0, _ffi.DTYPE_BF16,
                                status.data_ptr(), torch.cuda.current_stream().cuda_stream)
  _ffi.check(rc, "selftest")
  torch.cuda.synchronize()
  assert status.cpu().tolist() == [1, 102, 0, 7]
  # The device is still usable: an ordinary self-test on a fresh status word passes.
  status.zero_()
  test_umma_selftest(0, 0, 64, 64, torch.bfloat16)
