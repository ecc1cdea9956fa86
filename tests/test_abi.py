"""The C ABI: the built library loads and exports every symbol include/splash_sm100.h
declares, and the ctypes mirror of SplashParams matches the header field for field.
No compute calls are made here."""

import ctypes
import os
import re

from splash_attention_mgpu import _ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "splash_sm100.h")


def _header_text():
  with open(HEADER) as f:
    return re.sub(r"/\*.*?\*/", "", f.read(), flags=re.S)


def test_library_exports_every_declared_symbol():
  text = _header_text()
  declared = set(re.findall(r"\b(splash_\w+)\s*\(", text))
  assert declared == set(_ffi.EXPORTED_SYMBOLS)
  lib = ctypes.CDLL(_ffi.LIB_PATH)
  for name in declared:
    assert hasattr(lib, name), name


def test_params_struct_mirrors_the_header():
  text = _header_text()
  body = re.search(r"typedef struct SplashParams \{(.*?)\} SplashParams;", text, flags=re.S).group(1)
  fields = []
  for decl in body.split(";"):
    decl = decl.strip()
    if not decl:
      continue
    names = [n.strip().lstrip("*").strip() for n in decl.split(",")]
    names[0] = names[0].split()[-1].lstrip("*")
    fields.extend(names)
  assert fields == [name for name, _ in _ffi.SplashParams._fields_]
  # 22 pointers, 15 int32, 2 floats, padding to pointer alignment, then the appended scratch pointer.
  assert ctypes.sizeof(_ffi.SplashParams) == 22 * 8 + 15 * 4 + 2 * 4 + 4 + 8
  assert _ffi.SplashParams.seg_ranges.offset == 248


def test_status_strings_and_argument_checks_need_no_gpu():
  lib = _ffi.load()
  assert lib.splash_status_string(0) == b"ok"
  assert b"budget" in lib.splash_status_string(_ffi.SPLASH_BUDGET_EXCEEDED)
  p = _ffi.SplashParams()
  assert lib.splash_fwd128(ctypes.byref(p), None) == _ffi.SPLASH_INVALID_ARGUMENT
  assert b"non-null" in lib.splash_last_error()
  assert lib.splash_bwd_fused(ctypes.byref(p), None) == _ffi.SPLASH_INVALID_ARGUMENT
  assert lib.splash_selftest_umma(None, None, None, 128, 128, 0, 0, 0, None, None) == _ffi.SPLASH_INVALID_ARGUMENT
