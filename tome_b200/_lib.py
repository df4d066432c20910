"""ctypes binding of ``libtome_b200.so`` (the C ABI declared in ``include/tome_b200.h``).

There is no fallback: if the library has not been built, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int32, c_int64, c_size_t, c_uint64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtome_b200.so")

TOME_F32 = 0
TOME_BF16 = 1

DEV_TARGET_OUT_OF_RANGE = 1
DEV_TIMEOUT = 2
DEV_RAGGED_OVERFLOW = 4
DEV_BLOCK_OUT_OF_RANGE = 8
DEV_NO_CANDIDATE = 16

LMHEAD_ROUND_LOGITS_BF16 = 1

# name -> (restype, argtypes); mirrors include/tome_b200.h one to one
SIGNATURES = {
    "tome_version": (c_int32, []),
    "tome_status_string": (c_char_p, [c_int32]),
    "tome_last_error_string": (c_char_p, []),
    "tome_selftest_bounded_wait": (c_int32, [c_int64, c_void_p, c_void_p, c_void_p]),
    "tome_selective_logprob": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_int64, c_void_p,
                                         c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p]),
    "tome_log_softmax_full": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_int64, c_float,
                                        c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "tome_dual_logprob_kl": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_int64, c_int64,
                                       c_int64, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p]),
    "tome_ragged_logprob": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_int64, c_int64,
                                      c_void_p, c_int64, c_void_p, c_void_p, c_float, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p]),
    "tome_sample_topk_logprob": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_int64, c_float,
                                           c_int32, c_uint64, c_uint64, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_void_p]),
    "tome_sample_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "tome_sample_topk_logprob_ws": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_int64,
                                              c_float, c_int32, c_uint64, c_uint64, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                              c_void_p, c_void_p]),
    "tome_lmhead_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "tome_lmhead_partials": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                       c_void_p, c_float, c_int32, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_size_t, c_void_p, c_void_p]),
    "tome_lmhead_logprob": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p,
                                      c_float, c_int32, c_void_p, c_void_p, c_void_p, c_size_t,
                                      c_void_p, c_void_p]),
    "tome_rmsnorm_bf16": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_float, c_void_p,
                                    c_void_p]),
    "tome_lmhead_static_scratch_bytes": (c_size_t, []),
    "tome_lmhead_logprob_static": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                             c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                                             c_void_p]),
    "tome_gather_paged_kv": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int64,
                                       c_int64, c_int64, c_int32, c_int32, c_int32, c_int64,
                                       c_void_p, c_void_p, c_void_p, c_void_p]),
    "tome_update_paged_kv": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_int32, c_int64, c_int64, c_int64, c_int64,
                                       c_int32, c_int32, c_int32, c_void_p, c_void_p]),
    "tome_combine_triples": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, c_void_p, c_int64,
                                       c_int32, c_int64, c_void_p, c_void_p, c_void_p]),
}


class TomeArgumentError(ValueError):
    """The library rejected an argument before launching anything (negative status)."""


class TomeRuntimeError(RuntimeError):
    """A CUDA error, or a condition reported by a kernel through the device status word."""


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m tome_b200.build` "
            "(there is no CPU or PyTorch fallback for these kernels)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def check(status: int) -> None:
    """Turn a non-zero tome_status into the matching exception."""
    if status == 0:
        return
    name = lib.tome_status_string(status).decode()
    detail = lib.tome_last_error_string().decode()
    if status < 0:
        raise TomeArgumentError(f"{name}: {detail}")
    raise TomeRuntimeError(f"{name}: {detail}")
