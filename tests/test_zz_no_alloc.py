"""splash_bwd_fused_static: the fused backward for callers that may not allocate.

Some hosts of this library run it from inside another runtime's execute callback (an
XLA custom call, a serving plugin) or after their memory pool has been sealed; they
cannot call cudaMalloc and have no scratch to lend.  For them the library carries a
fixed 16 MiB f32 dQ accumulator of its own.  This test drives that entry point through
the C ABI twice in a row (the array keeps the previous call's contents, so the second
call proves it is cleared) and compares dq, dk, dv with the regular entry point, which
takes caller scratch, and with the CPU oracle.  Around the second call it reads the
driver's free-memory figure, which must not move, and it hands the entry point a bogus
`dq_acc` pointer, which must be ignored.  It also checks that an oversized problem is
refused.

The file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""

import ctypes

import numpy as np
import pytest
import torch

import splash_attention_mgpu as sa
from oracle import dense_attention as oracle
from splash_attention_mgpu import _ffi
from splash_attention_mgpu import splash_attention as impl

pytestmark = pytest.mark.gpu


def _setup(s, h, seed):
  dev = torch.device("cuda:0")
  d = 128
  kernel = sa.make_splash_mha(sa.CausalMask((s, s)))
  g = torch.Generator().manual_seed(seed)
  q = (torch.randn(1, h, s, d, generator=g) * d ** -0.5).to(torch.bfloat16).to(dev)
  k = torch.randn(1, h, s, d, generator=g).to(torch.bfloat16).to(dev)
  v = torch.randn(1, h, s, d, generator=g).to(torch.bfloat16).to(dev)
  do = torch.randn(1, h, s, d, generator=g).to(torch.bfloat16).to(dev)
  out, (lse,) = kernel(q, k, v, save_residuals=True)
  lib = _ffi.load()
  stream = torch.cuda.current_stream().cuda_stream
  delta = torch.empty(1, h, s, dtype=torch.float32, device=dev)
  _ffi.check(lib.splash_bwd_delta(out.data_ptr(), do.data_ptr(), delta.data_ptr(), h * s, d, _ffi.DTYPE_BF16,
                                  stream), "delta")
  _, cols = kernel._bwd_schedules(dev)
  keep = dict(q=q, k=k, v=v, do=do, lse=lse, delta=delta, cols=cols, out=out)

  def params(dq, dk, dv):
    p = impl._base_params(kernel, q, k, v, None, cols)
    p.d_out, p.lse, p.delta = do.data_ptr(), lse.data_ptr(), delta.data_ptr()
    p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    p.block_q, p.block_kv, p.num_stages = 128, 128, 2
    return p

  return lib, stream, params, keep


def _grads_like(keep):
  return torch.empty_like(keep["q"]), torch.empty_like(keep["k"]), torch.empty_like(keep["v"])


def test_static_scratch_matches_caller_scratch_twice():
  lib, stream, params, keep = _setup(s=1024, h=4, seed=11)
  # Reference result: the regular entry point with scratch from the caller.
  want = _grads_like(keep)
  p = params(*want)
  acc = torch.empty(lib.splash_bwd_fused_workspace_bytes(ctypes.byref(p)) // 4, dtype=torch.float32, device="cuda:0")
  p.dq_acc = acc.data_ptr()
  _ffi.check(lib.splash_bwd_fused(ctypes.byref(p), stream), "fused")
  torch.cuda.synchronize()
  sa.check_device_status()
  s = keep["q"].shape[2]
  ref = oracle.attention_backward(np.tril(np.ones((s, s), bool))[None], keep["q"], keep["k"], keep["v"], keep["do"])
  for attempt in range(2):
    got = _grads_like(keep)
    for t in got:
      t.fill_(float("nan"))
    p = params(*got)
    # No scratch from the caller; whatever stands in the field is ignored (second call: a bogus address).
    p.dq_acc = None if attempt == 0 else 0x10
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    _ffi.check(lib.splash_bwd_fused_static(ctypes.byref(p), stream), "fused static")
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    if attempt == 1:  # the first call on a device may load the kernels' code; the second allocates nothing
      assert free_after == free_before, f"device free memory moved by {free_before - free_after} bytes"
    sa.check_device_status()
    for name, a, b, r in zip(("dq", "dk", "dv"), got, want, ref):
      a, b = a.float().cpu().numpy(), b.float().cpu().numpy()
      assert np.isfinite(a).all(), (attempt, name)
      rel = np.abs(a - b).max() / np.abs(b).max()
      assert rel < 2e-2, f"call {attempt}, {name}: relative difference {rel} to the regular entry point"
      rel = np.abs(a - r).max() / np.abs(r).max()
      assert rel < 2e-2, f"call {attempt}, {name}: relative error {rel} against the oracle"


def test_static_scratch_refuses_oversized_problems():
  # 1 x 8 x 8192 x 128 f32 = 32 MiB > the 16 MiB built in.
  lib, stream, params, keep = _setup(s=8192, h=8, seed=12)
  got = _grads_like(keep)
  p = params(*got)
  rc = lib.splash_bwd_fused_static(ctypes.byref(p), stream)
  assert rc == _ffi.SPLASH_BUDGET_EXCEEDED
  assert "too large" in _ffi.last_error()
  with pytest.raises(ValueError, match="too large"):
    _ffi.check(rc, "fused static")
