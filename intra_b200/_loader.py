"""ctypes binding of libintra_b200.so (the C ABI declared in include/intra_b200.h).

The library is the only implementation of the attention path: if it has not been built, importing
this module raises ImportError (build it with `python -m intra_b200.build`); nothing falls back to
PyTorch or to the CPU.
"""
from __future__ import annotations

import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "_lib", "libintra_b200.so")

OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_CUDA, ERR_DEVICE, ERR_KERNEL = 0, -1, -2, -3, -4, -5, -6

_I64x3 = ctypes.POINTER(ctypes.c_int64)
_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float

# name -> (restype, argtypes); every symbol include/intra_b200.h declares.
SIGNATURES = {
    "intra_b200_fwd_llm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _I64x3, _I64x3, _I64x3, _I64x3,
                                _i, _i, _i, _f, _i, _vp]),
    "intra_b200_fwd_image": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _I64x3, _I64x3, _I64x3, _I64x3,
                                  _i, _i, _f, _i, _vp]),
    "intra_b200_fwd_llm_lse": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _I64x3, _I64x3, _I64x3, _I64x3,
                                    _i, _i, _i, _f, _i, _vp]),
    "intra_b200_fwd_image_lse": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _I64x3, _I64x3, _I64x3, _I64x3,
                                      _i, _i, _f, _i, _vp]),
    "intra_b200_fwd_llm_noalloc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _I64x3, _I64x3, _I64x3, _I64x3,
                                        _i, _i, _i, _f, _i, _vp, ctypes.POINTER(_i)]),
    "intra_b200_strerror": (ctypes.c_char_p, [_i]),
    "intra_b200_last_cuda_error": (_i, []),
    "intra_b200_device_status": (_i, [_i, ctypes.POINTER(_i), _i]),
    "intra_b200_visited_host": (_i, [_i, _i, _i, _i, _vp]),
    "intra_b200_visited_pairs_host": (_i, [_i, _i, _i, _i, _vp]),
    "intra_b200_visited_device": (_i, [_i, _i, _i, _i, _vp, _i, _vp]),
    "intra_b200_tile_counts": (_i, [_i, _i, _i, _i, ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]),
    "intra_b200_selftest_umma": (_i, [_vp, _vp, _vp, _f, _vp, _vp, _i, _vp]),
    "intra_b200_test_tma_rows": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _I64x3, _I64x3, _I64x3, _i, _i, _i,
                                      _vp, _vp, _vp, _vp, _vp, ctypes.POINTER(ctypes.c_int64),
                                      ctypes.POINTER(ctypes.c_int64), _i, _vp]),
    "intra_b200_interleave_heads": (_i, [_vp, _vp, _i, ctypes.c_int64, ctypes.c_int64, _i, _vp]),
    "intra_b200_test_force_path": (_i, [_i, _i]),
    "intra_b200_test_kernel_form": (_i, [_i, _i, _i, _i, _i, _i]),
    "intra_b200_test_poke_status": (_i, [_i, _i]),
    "intra_b200_test_wait_timeout": (_i, [_i, _vp, _i, _vp]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is not built; run `python -m intra_b200.build` (needs nvcc)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as err:  # library older than this file
            raise ImportError(f"{LIB_PATH} lacks {name}; rebuild with `python -m intra_b200.build --force`") from err
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def strerror(status: int) -> str:
    return lib.intra_b200_strerror(status).decode()


def strides3(t) -> ctypes.Array:
    """{batch, token, head} element strides of a (B, S, H, 128) tensor as int64[3]."""
    return (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
