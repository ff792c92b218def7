"""ctypes binding of libftq_b200.so (the C ABI declared in include/ftq_b200.h).

There is no fallback of any kind: if the library is missing or a call fails,
the caller gets a RuntimeError carrying the library's own message.
"""
from __future__ import annotations

import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libftq_b200.so")

F32, F16, BF16 = 0, 1, 2

_c = ctypes
_vp, _i, _i64, _f, _sz = _c.c_void_p, _c.c_int, _c.c_int64, _c.c_float, _c.c_size_t
_fp = _c.POINTER(_c.c_float)

# name -> (restype, argtypes); the same list is what tests use to check that
# every symbol the header declares is exported.
SIGNATURES = {
    "ftq_version": (_i, []),
    "ftq_last_error": (_c.c_char_p, []),
    "ftq_packed_dim": (_i, [_i, _i]),
    "ftq_page_bytes": (_i64, [_i, _i, _i]),
    "ftq_encode": (_i, [_vp, _i, _i64, _i, _i64, _i, _fp, _fp, _vp, _vp, _vp]),
    "ftq_decode_dense": (_i, [_vp, _vp, _i, _i64, _i, _i, _fp, _fp, _vp, _vp]),
    "ftq_rht": (_i, [_vp, _vp, _i, _i64, _i, _fp, _i, _vp]),
    "ftq_qk_scores": (_i, [_vp, _vp, _vp, _i, _fp, _f, _i, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "ftq_decode_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "ftq_flash_decode": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _fp, _fp, _fp, _f, _i, _i, _vp,
                              _i, _i, _i, _i, _i, _vp, _i, _vp, _sz, _vp]),
    "ftq_paged_store": (_i, [_vp, _vp, _i, _i64, _i, _i, _i64, _i64, _i, _i, _fp, _fp, _fp, _vp,
                             _i64, _vp, _i, _i64, _i64, _vp]),
    "ftq_paged_decode_attn": (_i, [_vp, _i, _vp, _i, _vp, _i64, _i64, _i, _vp, _i, _vp, _i, _i,
                                   _i, _i, _i, _i, _i, _fp, _fp, _fp, _f, _vp, _sz, _vp]),
    "ftq_paged_decode_attn_static": (_i, [_vp, _i, _vp, _i, _vp, _i64, _i64, _i, _vp, _i, _vp, _i,
                                          _i, _i, _i, _i, _i, _i, _fp, _fp, _fp, _f, _vp]),
    "ftq_paged_decode_status": (_i, [_vp, _i, _i, _i, _i, _i, _i, _vp, _c.POINTER(_c.c_int)]),
    "ftq_v0_store": (_i, [_vp, _vp, _i, _i64, _i, _i, _i64, _i64, _i, _i, _fp, _fp, _fp, _vp,
                          _i64, _i, _i, _vp, _vp]),
    "ftq_v0_gather": (_i, [_vp, _i64, _i, _i, _i, _i, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _vp]),
    "ftq_tq_slot_bytes": (_i, [_i, _i, _i]),
    "ftq_tq_store": (_i, [_vp, _vp, _i, _i64, _i, _i, _i64, _i64, _i, _i, _i, _i, _fp, _vp, _i64,
                          _i64, _i64, _i, _vp, _vp]),
    "ftq_tq_store_layers": (_i, [_vp, _vp, _i, _i64, _i, _i, _i64, _i64, _i, _i, _i, _i, _fp, _vp,
                                 _i64, _i64, _i64, _i, _vp, _i, _i64, _i64, _i64, _vp]),
    "ftq_tq_decode": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _i64, _i64, _i64, _i, _vp, _i, _vp, _vp,
                           _i, _i, _i, _i, _i, _fp, _c.c_float, _i, _vp, _vp, _i, _vp, _vp, _i, _vp,
                           _vp]),
    "ftq_tq_decode_layers": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _i64, _i64, _i64, _i, _vp, _i, _vp,
                                  _vp, _i, _i, _i, _i, _i, _fp, _c.c_float, _i, _vp, _vp, _i, _vp,
                                  _vp, _i, _vp, _i, _i64, _i64, _vp]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once).  Raises RuntimeError if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m fused_turboquant_b200.build` "
                "(nvcc, sm_100a). There is no CPU or Triton fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def is_available() -> bool:
    """True when the CUDA library is built and a CUDA device is visible."""
    import torch

    return os.path.exists(LIB_PATH) and torch.cuda.is_available()


def check(rc: int, what: str) -> None:
    """Turn a negative status into the exception the reference surface raises."""
    if rc == 0:
        return
    msg = load().ftq_last_error().decode("utf-8", "replace")
    if rc == -1 and ("bits must be" in msg or "head_dim" in msg):
        raise ValueError(msg)
    raise RuntimeError(f"{what} failed ({rc}): {msg}")


def fptr(arr):
    """float32 numpy array -> POINTER(c_float) (or None)."""
    if arr is None:
        return None
    return arr.ctypes.data_as(_fp)
