"""ctypes binding of libokc_moe_b200.so (the C ABI declared in include/okc_moe.h).

There is no fallback: if the shared library has not been built (``python -m
okc_muse_kernels_b200.build``) loading fails with an ImportError that says so.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# OKC_MOE_LIB selects another build of the same ABI (the instrumented libokc_moe_b200_prof.so)
LIB_PATH = os.environ.get("OKC_MOE_LIB") or os.path.join(_PKG, "libokc_moe_b200.so")

OKC_OK = 0
OKC_ERR_BAD_PLAN = -1
OKC_ERR_BAD_ARG = -2
OKC_ERR_CUDA = -3
OKC_ERR_NO_DEVICE = -4
OKC_ERR_TIMEOUT = -5
OKC_ERR_TOO_LARGE = -6


class Plan(C.Structure):
    """okc_moe_plan"""
    _fields_ = [("hidden", C.c_int32), ("inter", C.c_int32), ("n_experts", C.c_int32), ("top_k", C.c_int32),
                ("local_start", C.c_int32), ("local_count", C.c_int32), ("shared_inter", C.c_int32),
                ("max_tokens", C.c_int32), ("post_norm", C.c_int32), ("reserved", C.c_int32 * 7)]


class Sizes(C.Structure):
    """okc_moe_sizes"""
    _fields_ = [("packed_w13_bytes", C.c_uint64), ("packed_w2_bytes", C.c_uint64), ("workspace_bytes", C.c_uint64),
                ("expert_slots", C.c_uint32), ("routes_per_token", C.c_uint32)]


EP_MAX_RANKS = 16


class EpComm(C.Structure):
    """okc_ep_comm"""
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("tokens", C.c_int32), ("hidden", C.c_int32),
                ("n_experts", C.c_int32), ("wait_limit_ms", C.c_int32), ("reserved", C.c_int32 * 2),
                ("peer", C.c_void_p * EP_MAX_RANKS)]


class Router(C.Structure):
    """okc_router"""
    _fields_ = [("w", C.c_void_p), ("bias", C.c_void_p), ("mode", C.c_int32), ("multiplier", C.c_float),
                ("w_split", C.c_void_p)]


_P = C.c_void_p
_PLAN = C.POINTER(Plan)
_COMM = C.POINTER(EpComm)
# name -> (restype, argtypes); every symbol include/okc_moe.h declares
SIGNATURES = {
    "okc_moe_version": (C.c_int, []),
    "okc_moe_strerror": (C.c_char_p, [C.c_int]),
    "okc_moe_launches_per_step": (C.c_int, []),
    "okc_moe_query": (C.c_int, [_PLAN, C.POINTER(Sizes)]),
    "okc_moe_repack": (C.c_int, [_PLAN, _P, _P, _P, _P, C.c_int, C.c_int, _P, _P, _P]),
    "okc_moe_route": (C.c_int, [_PLAN, _P, C.c_int, C.c_int, C.c_int, _P, _P, _P, _P]),
    "okc_moe_route_hidden": (C.c_int, [_PLAN, C.POINTER(Router), _P, C.c_int64, _P, C.c_int, C.c_int, C.c_int, _P, _P, _P, _P]),
    "okc_moe_router_split": (C.c_int, [_P, C.c_int, C.c_int, _P, _P]),
    "okc_moe_sort": (C.c_int, [_PLAN, _P, _P, C.c_int, C.c_int, C.c_int, _P, _P]),
    "okc_moe_experts": (C.c_int, [_PLAN, _P, _P, _P, _P, _P, C.c_int64, C.c_int, _P, _P, _P, C.c_int, _P]),
    "okc_moe_experts_prenorm": (C.c_int, [_PLAN, _P, _P, _P, _P, _P, C.c_int64, C.c_int, _P, C.c_float, C.c_int, _P, _P, _P,
                                          C.c_int, _P]),
    "okc_moe_experts_profiled": (C.c_int, [_PLAN, _P, _P, _P, _P, _P, C.c_int64, C.c_int, _P, _P, _P, C.c_int, _P,
                                           C.POINTER(C.c_float)]),
    "okc_moe_cast_bf16": (C.c_int, [_P, _P, C.c_int64, _P]),
    "okc_moe_step": (C.c_int, [_PLAN, _P, _P, _P, _P, _P, C.c_int64, _P, C.c_int, C.c_int, C.c_int, _P, _P, _P, _P,
                               _P, C.c_int, _P]),
    "okc_moe_step_static_scratch": (C.c_int, [_PLAN, _P, _P, _P, _P, _P, C.c_int64, _P, C.c_int, C.c_int, C.c_int, _P, _P,
                                              _P, _P, C.c_int, _P]),
    "okc_moe_read_status_static": (C.c_int, [_P, C.POINTER(C.c_int32)]),
    "okc_moe_export_sort": (C.c_int, [_PLAN, _P, C.c_int, _P, _P, _P, _P, C.c_int, _P]),
    "okc_moe_unpack_bf16": (C.c_int, [_PLAN, _P, C.c_int, C.c_int, _P, _P]),
    "okc_moe_probe_wait_timeout": (C.c_int, [_P, _P]),
    "okc_moe_read_status": (C.c_int, [_P, _P, C.POINTER(C.c_int32)]),
    "okc_ep_buffer_bytes": (C.c_uint64, [C.c_int32, C.c_int32, C.c_int32]),
    "okc_ep_views": (C.c_int, [_COMM, C.POINTER(_P), C.POINTER(_P), C.POINTER(_P)]),
    "okc_ep_gather_tokens": (C.c_int, [_COMM, _P, C.c_int64, _P, _P]),
    "okc_ep_reduce_scatter": (C.c_int, [_COMM, _P, _P]),
    "okc_moe_experts_ep": (C.c_int, [_PLAN, _P, _P, _P, _P, _P, C.c_int64, C.c_int, _P, _COMM, _P, _P]),
    "okc_ep_route_gather": (C.c_int, [_PLAN, _COMM, _P, C.c_int64, _P, _P, _P]),
    "okc_ep_routed_views": (C.c_int, [_COMM, C.c_int, C.POINTER(_P), C.POINTER(_P)]),
    "okc_ep_mark_arrived": (C.c_int, [_COMM, C.c_int, C.c_int, _P]),
    "okc_ep_read_status": (C.c_int, [_COMM, _P, C.POINTER(C.c_int32)]),
}

_lib = None


class OkcError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib().okc_moe_strerror(code).decode() if _lib is not None else str(code)
        super().__init__(f"{where}: {msg} ({code})")


def lib():
    """The loaded library (loads it on first use)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m okc_muse_kernels_b200.build` "
                              "(there is no CPU or PyTorch fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(code: int, where: str) -> None:
    if code != OKC_OK:
        raise OkcError(code, where)
