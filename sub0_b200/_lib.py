"""ctypes binding of ``libcda_b200.so`` (declarations: ``include/cda_b200.h``).

The library is the only compute path of this package.  If it is missing the import fails loudly; nothing here falls
back to PyTorch or CPU code.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
# $CDA_B200_LIBRARY selects another build of the same library (e.g. one compiled with different tuning constants).
LIB_PATH = Path(os.environ["CDA_B200_LIBRARY"]) if os.environ.get("CDA_B200_LIBRARY") else _PKG / "libcda_b200.so"

CDA_OK = 0
CDA_ERR_BAD_ARG, CDA_ERR_BAD_SHAPE, CDA_ERR_BAD_ALIGN, CDA_ERR_UNSUPPORTED = -1, -2, -3, -4
CDA_ERR_N_TOO_LARGE, CDA_ERR_WORKSPACE, CDA_ERR_LAUNCH = -5, -6, -7

_p, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); one entry per declaration in include/cda_b200.h
PROTOTYPES = {
    "cda_b200_version": (_i, []),
    "cda_b200_last_error_string": (C.c_char_p, []),
    "cda_b200_slot_bytes": (_i, [_i, _i]),
    "cda_b200_paged_encode": (_i, [_p, _p, _p, _p, _p, _p, _i64, _i, _i64, _i, _i, _i, _p]),
    "cda_b200_quantize_rotated": (_i, [_p, _i64, _p, _i, _p, _p, _p]),
    "cda_b200_hadamard128": (_i, [_p, _p, _i64, _f, _p]),
    "cda_b200_decode_plan_splits": (_i, [_i, _i, _i, _i]),
    "cda_b200_decode_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "cda_b200_decode": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _sz, _i, _i, _i, _i, _i, _i, _i64, _i, _i, _i, _f, _i, _p]),
    "cda_b200_decode_partial": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _sz, _i, _i, _i, _i, _i, _i, _i64, _i,
                                     _i, _i, _f, _i, _p]),
    "cda_b200_decode_lse": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _sz, _i, _i, _i, _i, _i, _i, _i64, _i, _i, _i, _f, _i,
                                 _p]),
    "cda_b200_decode_partial_packed": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _sz, _i, _i, _i, _i, _i, _i, _i64, _i, _i, _i,
                                            _f, _i, _p]),
    "cda_b200_merge_partials": (_i, [_p, _p, _p, _i, _i64, _p, _i, _p]),
    "cda_b200_merge_partials_packed": (_i, [_p, _i, _i64, _p, _i, _p]),
    "cda_b200_decode_exchange_bytes": (_sz, [_i, _i, _i]),
    "cda_b200_exchange_alloc": (_i, [_sz, _p]),
    "cda_b200_exchange_free": (_i, [_p]),
    "cda_b200_exchange_export": (_i, [_p, _p]),
    "cda_b200_exchange_import": (_i, [_p, _p]),
    "cda_b200_exchange_close": (_i, [_p]),
    "cda_b200_decode_exchange": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _sz, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i64,
                                      _i, _i, _i, _f, _i, _p]),
    "cda_b200_decode_static": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i64, _i, _i, _i, _f, _i, _p]),
    "cda_b200_decode_static_status": (_i, [_p]),
    "cda_b200_decode_scalar": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i64, _i, _i, _i, _f, _p]),
    "cda_b200_cache_to_dense_rotated": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i64, _i, _i, _i, _p]),
    "cda_b200_prefill_varlen": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _i, _i64, _i, _i,
                                     _i, _f, _p]),
    "cda_b200_varlen_fwd_hadamard": (_i, [_p, _p, _p, _p, _p, _p, _p, _i64, _i, _i, _i, _i, _i, _f, _p]),
    "cda_b200_varlen_fwd_hadamard_mma": (_i, [_p, _p, _p, _p, _p, _p, _p, _i64, _i, _i, _i, _i, _i, _f, _p]),
    "cda_b200_prefill_fault": (_i, []),
    "cda_b200_prefill_status": (_i, []),
    "cda_b200_prefill_clear_status": (_i, []),
    "cda_b200_prefill_debug": (_i, [_i, _i]),
    "cda_b200_dequantize_rows": (_i, [_p, _p, _p, _p, _i64, _i, _p]),
}


class LibraryMissing(ImportError):
    """``libcda_b200.so`` has not been built (``python -m sub0_b200.build``) -- there is no fallback path."""


def _load() -> C.CDLL:
    if not LIB_PATH.is_file():
        raise LibraryMissing(f"{LIB_PATH} not found: build it with `python -m sub0_b200.build` (needs nvcc, sm_100a). "
                             "sub0_b200 has no CPU or PyTorch fallback.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)          # AttributeError here means header and library disagree
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()

_EXC = {
    CDA_ERR_BAD_ARG: ValueError, CDA_ERR_BAD_SHAPE: ValueError, CDA_ERR_BAD_ALIGN: ValueError,
    CDA_ERR_UNSUPPORTED: NotImplementedError, CDA_ERR_N_TOO_LARGE: ValueError, CDA_ERR_WORKSPACE: ValueError,
    CDA_ERR_LAUNCH: RuntimeError,
}


def last_error() -> str:
    return lib.cda_b200_last_error_string().decode()


def check(rc: int) -> None:
    """Turn a negative status into the Python exception type the reference wrappers raise for that class of error."""
    if rc != CDA_OK:
        raise _EXC.get(rc, RuntimeError)(f"libcda_b200: {last_error()} (status {rc})")
