"""ctypes binding of ``libdaisy_b200.so`` (the C ABI declared in ``include/daisy_b200.h``).

There is no fallback: if the shared library has not been built, or a call returns a negative
status, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdaisy_b200.so")

OK, EINVAL, EUNSUPPORTED, EALIGN, EWORKSPACE, ECUDA, ETIMEOUT, ENODEV = 0, -1, -2, -3, -4, -5, -6, -7
NORM_Q, NORM_K, NORM_V, ROPE, QKV_DEFAULT, WRITE_RING, OUT_BTHD, KV_BHTD, Q_IN_KERNEL, BOUNDED_QK = 1, 2, 4, 8, 15, 16, 32, 64, 128, 256
WINDOW_BLOCKS = 512
CACHE_FP16 = 1024
KDA_L2NORM_QK, KDA_OUT_FP32 = 1, 2
KDA_GATE_ROUND_BF16 = 1
KDA_CONV_SILU = 1
KDA_NORM_SIGMOID, KDA_NORM_SWISH, KDA_NORM_SWISH_SIGMOID = 0, 1, 2

_vp, _i, _i64, _f, _u, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_uint, C.c_size_t

# name -> (restype, argtypes); every symbol include/daisy_b200.h declares
SIGNATURES = {
    "daisy_b200_version": (_i, []),
    "daisy_b200_strerror": (C.c_char_p, [_i]),
    "daisy_b200_sm_count": (_i, []),
    "daisy_b200_qkv_prep": (_i, [_vp] * 3 + [_i64] * 9 + [_vp] * 2 + [_vp] * 3 + [_vp] + [_i64] * 3 + [_vp] + [_i] * 4 + [_f, _u, _vp]),
    "daisy_b200_qkv_gemm": (_i, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _vp] + [_vp, _i64, _vp] + [_i] * 5 + [_f, _u, _vp, _vp]),
    "daisy_b200_qkv_gemm_ring": (_i, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _vp] + [_vp, _i64, _vp] + [_vp, _vp, _i64, _i64, _i64, _i, _i] +
                                 [_i] * 5 + [_f, _u, _vp, _vp]),
    "daisy_b200_gemm_nt": (_i, [_vp, _i64, _vp, _i64, _vp, _i64, _i, _i, _i, _vp, _vp]),
    "daisy_b200_swa_prefill_workspace_bytes": (_sz, [_i] * 4),
    "daisy_b200_swa_prefill_fwd": (_i, [_vp] * 3 + [_i64] * 9 + [_vp] * 2 + [_vp] + [_i64] * 3 + [_vp] * 2 +
                                   [_i] * 5 + [_f, _f, _vp, _i64, _u, _vp, _sz, _vp, _vp]),
    "daisy_b200_swa_attend": (_i, [_vp] * 3 + [_i64] * 9 + [_vp] + [_i64] * 3 + [_i] * 5 + [_f, _vp, _i64, _u, _vp, _vp]),
    "daisy_b200_swa_attend_lse": (_i, [_vp] * 3 + [_i64] * 9 + [_vp] + [_i64] * 3 + [_vp] + [_i] * 5 + [_f, _vp, _i64, _u, _vp, _vp]),
    "daisy_b200_swa_attend_bwd_workspace_bytes": (_sz, [_i] * 3),
    "daisy_b200_swa_attend_bwd": (_i, [_vp] * 5 + [_i64] * 15 + [_vp] * 4 + [_i] * 5 + [_f, _vp, _i64, _u, _vp, _sz, _vp, _vp]),
    "daisy_b200_qkv_prep_bwd": (_i, [_vp] * 3 + [_i64] * 9 + [_vp] * 2 + [_vp] * 6 + [_i] * 4 + [_f, _u, _vp]),
    "daisy_b200_swa_decode_splits": (_i, [_i] * 4),
    "daisy_b200_swa_decode_workspace_bytes": (_sz, [_i] * 4),
    "daisy_b200_swa_decode_step": (_i, [_vp] * 3 + [_i64] * 6 + [_vp] * 2 + [_i64] * 3 + [_i64, _i, _i] +
                                   [_vp] * 2 + [_vp, _i64, _i64] + [_vp] * 2 + [_i] * 3 + [_f, _f, _u] +
                                   [_vp, _sz, _i, _vp, _vp]),
    "daisy_b200_swa_decode_step_dev": (_i, [_vp] * 3 + [_i64] * 6 + [_vp] * 2 + [_i64] * 3 + [_vp, _i, _i] +
                                       [_vp] * 2 + [_i] + [_vp, _i64, _i64] + [_vp] * 2 + [_i] * 3 + [_f, _f, _u] +
                                       [_vp, _sz, _i, _vp, _vp]),
    "daisy_b200_swa_decode_fused_workspace_bytes": (_sz, [_i] * 4),
    "daisy_b200_swa_decode_step_fused": (_i, [_vp] * 3 + [_i64] * 6 + [_vp] * 2 + [_i64] * 3 + [_i64, _vp, _i, _i] +
                                         [_vp] * 2 + [_i] + [_vp, _i64, _i64] + [_vp] * 2 + [_vp, _i64, _i64, _vp] +
                                         [_i] * 3 + [_f, _f, _u] + [_vp, _sz, _i, _vp, _vp]),
    "daisy_b200_gemm_skinny": (_i, [_vp, _i64, _vp, _i64, _vp, _i64, _i, _i, _i, _vp]),
    "daisy_b200_swa_decode_static_capacity": (_sz, []),
    "daisy_b200_swa_decode_step_static": (_i, [_vp] * 3 + [_i64] * 6 + [_vp] * 2 + [_i64] * 3 + [_i64, _i, _i] +
                                          [_vp] * 2 + [_vp, _i64, _i64] + [_vp] * 2 + [_i] * 3 + [_f, _f, _u] +
                                          [_i, _vp, _vp]),
    "daisy_b200_ring_copy_rows": (_i, [_vp] + [_i64] * 3 + [_vp] + [_i64] * 3 + [_i] * 4 + [_i64] + [_i] * 3 + [_vp]),
    "daisy_b200_kda_workspace_bytes": (_sz, [_i] * 5),
    "daisy_b200_kda_chunk_fwd": (_i, [_vp] * 8 + [_i] * 6 + [_f, _u, _vp, _sz, _vp, _vp]),
    "daisy_b200_kda_varlen_workspace_bytes": (_sz, [_i] * 4),
    "daisy_b200_kda_chunk_fwd_varlen": (_i, [_vp] * 8 + [_i] * 5 + [_f, _u, _vp, _i, _vp, _i, _vp, _sz, _vp, _vp]),
    "daisy_b200_kda_short_conv_varlen": (_i, [_vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _vp, _u, _vp]),
    "daisy_b200_kda_recurrent_fwd": (_i, [_vp] * 8 + [_i] * 5 + [_f, _u, _vp]),
    "daisy_b200_kda_gate": (_i, [_vp, _i, _vp, _vp, _vp, _i64, _i, _i, _f, _f, _u, _vp]),
    "daisy_b200_kda_short_conv": (_i, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i, _i, _i, _i, _u, _vp]),
    "daisy_b200_kda_out_norm": (_i, [_vp, _i, _vp, _vp, _i, _vp, _vp, _i64, _i, _f, _i, _vp]),
    "daisy_b200_selftest_umma": (_i, [_vp] * 3 + [_i, _i, _vp, _vp]),
}

_lib = None


class DaisyB200Error(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        msg = lib().daisy_b200_strerror(code).decode() if _lib is not None else "?"
        super().__init__(f"{what}: daisy_b200 status {code} ({msg})")


def lib() -> C.CDLL:
    """Load the library once.  Raises if it is missing -- build it with ``python -m daisy_b200.build``."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} not found: build the CUDA library first (python -m daisy_b200.build); "
                               "daisy_b200 has no CPU or PyTorch fallback")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)          # AttributeError here = library older than this binding: rebuild
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def check(code: int, what: str) -> None:
    if code != OK:
        raise DaisyB200Error(code, what)
