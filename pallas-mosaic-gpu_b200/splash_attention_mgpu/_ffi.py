"""ctypes binding of libsplash_sm100.so (the C ABI declared in include/splash_sm100.h).

The library is built in-tree next to this file (`csrc/Makefile`).  There is no
CPU fallback: if the library is missing, or a call is made without a CUDA
device, the error is raised to the caller.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int, c_int32,
                    c_int64, c_void_p)

LIB_NAME = "libsplash_sm100.so"
# SPLASH_LIB_PATH points at an alternative build of the same library (e.g. a tuning build).
LIB_PATH = os.environ.get("SPLASH_LIB_PATH") or os.path.join(os.path.dirname(os.path.abspath(__file__)), LIB_NAME)

SPLASH_OK = 0
SPLASH_INVALID_ARGUMENT = -1
SPLASH_UNSUPPORTED = -2
SPLASH_BUDGET_EXCEEDED = -3
SPLASH_CUDA_ERROR = -4
SPLASH_DEVICE_TIMEOUT = -5

DTYPE_BF16 = 0
DTYPE_F16 = 1

# Every symbol include/splash_sm100.h declares; the CPU test-suite checks that
# the built library exports all of them.
EXPORTED_SYMBOLS = (
    "splash_fwd128",
    "splash_fwd256",
    "splash_bwd_delta",
    "splash_bwd_dq",
    "splash_bwd_dkv",
    "splash_bwd_fused",
    "splash_bwd_fused_workspace_bytes",
    "splash_bwd_fused_static",
    "splash_seg_ranges_bytes",
    "splash_read_status",
    "splash_status_string",
    "splash_last_error",
    "splash_selftest_umma",
)


class SplashParams(Structure):
  """Mirror of `struct SplashParams`; field order and types must match the header."""

  _fields_ = [
      ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("d_out", c_void_p),
      ("lse", c_void_p), ("delta", c_void_p),
      ("seg_q", c_void_p), ("seg_kv", c_void_p),
      ("num_steps", c_void_p), ("block_order", c_void_p),
      ("block_list", c_void_p), ("block_kind", c_void_p),
      ("mask_block", c_void_p), ("partial_blocks", c_void_p),
      ("mask_desc", c_void_p),
      ("out", c_void_p), ("lse_out", c_void_p),
      ("dq", c_void_p), ("dk", c_void_p), ("dv", c_void_p),
      ("dq_acc", c_void_p), ("status", c_void_p),
      ("batch", c_int32), ("heads", c_int32), ("kv_heads", c_int32),
      ("q_len", c_int32), ("kv_len", c_int32),
      ("head_dim", c_int32), ("head_dim_v", c_int32),
      ("dtype", c_int32), ("mask_heads", c_int32), ("max_steps", c_int32),
      ("num_partial_blocks", c_int32),
      ("block_q", c_int32), ("block_kv", c_int32),
      ("num_stages", c_int32), ("sub_block", c_int32),
      ("mask_value", c_float), ("soft_cap", c_float),
      ("seg_ranges", c_void_p),
  ]


class SplashLibraryError(RuntimeError):
  pass


_lib = None


def load():
  """Loads the shared library once; raises if it has not been built."""
  global _lib
  if _lib is not None:
    return _lib
  if not os.path.exists(LIB_PATH):
    raise SplashLibraryError(
        f"{LIB_NAME} is not built (expected at {LIB_PATH}); run `make -C csrc`"
        " or `python -c 'import __graft_entry__ as g; g.build()'`.")
  lib = ctypes.CDLL(LIB_PATH)
  for name in ("splash_fwd128", "splash_fwd256", "splash_bwd_dq",
               "splash_bwd_dkv", "splash_bwd_fused", "splash_bwd_fused_static"):
    if hasattr(lib, name):
      fn = getattr(lib, name)
      fn.argtypes = [POINTER(SplashParams), c_void_p]
      fn.restype = c_int
  if hasattr(lib, "splash_bwd_delta"):
    lib.splash_bwd_delta.argtypes = [c_void_p, c_void_p, c_void_p, c_int64,
                                     c_int32, c_int32, c_void_p]
    lib.splash_bwd_delta.restype = c_int
  if hasattr(lib, "splash_seg_ranges_bytes"):
    lib.splash_seg_ranges_bytes.argtypes = [POINTER(SplashParams)]
    lib.splash_seg_ranges_bytes.restype = c_int64
  if hasattr(lib, "splash_bwd_fused_workspace_bytes"):
    lib.splash_bwd_fused_workspace_bytes.argtypes = [POINTER(SplashParams)]
    lib.splash_bwd_fused_workspace_bytes.restype = c_int64
  lib.splash_read_status.argtypes = [c_void_p, POINTER(c_int32 * 4), c_void_p]
  lib.splash_read_status.restype = c_int
  lib.splash_status_string.argtypes = [c_int]
  lib.splash_status_string.restype = c_char_p
  lib.splash_last_error.argtypes = []
  lib.splash_last_error.restype = c_char_p
  lib.splash_selftest_umma.argtypes = [c_void_p, c_void_p, c_void_p, c_int32,
                                       c_int32, c_int32, c_int32, c_int32,
                                       c_void_p, c_void_p]
  lib.splash_selftest_umma.restype = c_int
  _lib = lib
  return lib


def last_error() -> str:
  return load().splash_last_error().decode()


def check(status: int, what: str) -> None:
  """Maps a SplashStatus to the exception type the reference raises."""
  if status == SPLASH_OK:
    return
  detail = last_error()
  if status == SPLASH_UNSUPPORTED:
    raise NotImplementedError(f"{what}: {detail}")
  if status in (SPLASH_INVALID_ARGUMENT, SPLASH_BUDGET_EXCEEDED):
    raise ValueError(f"{what}: {detail}")
  raise SplashLibraryError(
      f"{what}: {load().splash_status_string(status).decode()}: {detail}")
