"""ctypes binding of libflyb200.so (declarations in include/flyb200.h).

The library is the only compute path: there is no CPU or eager-PyTorch fallback. If the shared
object has not been built, loading raises with the build command.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p, POINTER

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FLYB200_LIB_PATH") or os.path.join(_PKG_DIR, "lib", "libflyb200.so")

OK = 0
ERR_INVALID_ARGUMENT = -1
ERR_UNSUPPORTED = -2
ERR_CUDA = -3
ERR_WORKSPACE = -4
ERR_DEVICE_TIMEOUT = -5

BF16, F16, F32 = 0, 1, 2


class GemmCfg(ctypes.Structure):
    """Mirror of flyb200_gemm_cfg."""

    _fields_ = [("block_n", c_int32), ("max_ctas", c_int32), ("path", c_int32),
                ("split_k", c_int32)]


class Flyb200Error(RuntimeError):
    """A libflyb200 entry point returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"libflyb200 status {status}: {message}")
        self.status = status


# name -> (restype, argtypes); exactly the symbols include/flyb200.h declares.
SIGNATURES = {
    "flyb200_repack_weight_fp8": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "flyb200_blockscale_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32,
                                        c_int32, c_int32, c_int32, POINTER(GemmCfg), c_void_p]),
    "flyb200_pertoken_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32,
                                      c_int32, c_int32, c_int32, POINTER(GemmCfg), c_void_p]),
    "flyb200_moe_sort": (c_int, [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p,
                                 c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "flyb200_moe_sort_permute": (c_int, [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p,
                                         c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_int32, c_void_p]),
    "flyb200_moe_route_topk": (c_int, [c_void_p, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p]),
    "flyb200_moe_gemm1": (c_int, [c_void_p] * 9 + [c_int32] * 9 + [POINTER(GemmCfg), c_void_p]),
    "flyb200_moe_gemm1_q8": (c_int, [c_void_p] * 10 + [c_int32] * 9 + [POINTER(GemmCfg), c_void_p]),
    "flyb200_moe_gemm2": (c_int, [c_void_p] * 9 + [c_int32] * 10 + [POINTER(GemmCfg), c_void_p]),
    "flyb200_moe_gemm1_pertoken": (c_int, [c_void_p] * 9 + [c_int32] * 9 + [POINTER(GemmCfg), c_void_p]),
    "flyb200_moe_gemm2_pertoken": (c_int, [c_void_p] * 9 + [c_int32] * 10 + [POINTER(GemmCfg), c_void_p]),
    "flyb200_moe_gemm2_reduce_pertoken": (c_int, [c_void_p] * 10 + [c_int32] * 9 + [POINTER(GemmCfg), c_void_p,
                                                  c_size_t, c_int32, c_void_p]),
    "flyb200_moe_gemm2_reduce": (c_int, [c_void_p] * 10 + [c_int32] * 9 + [POINTER(GemmCfg), c_void_p, c_size_t,
                                         c_void_p]),
    "flyb200_moe_gemm2_reduce_noalloc": (c_int, [c_void_p] * 10 + [c_int32] * 9 + [POINTER(GemmCfg), c_void_p]),
    "flyb200_moe_gemm2_reduce_noalloc_max_bytes": (c_size_t, []),
    "flyb200_moe_gemm2_reduce_workspace_bytes": (c_size_t, [c_int32, c_int32, c_int32, c_int32]),
    "flyb200_moe_reduce": (c_int, [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                   c_void_p]),
    "flyb200_quant_1x128": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32,
                                    c_void_p]),
    "flyb200_moe_gather_rows": (c_int, [c_void_p] * 6 + [c_int32] * 5 + [c_void_p]),
    "flyb200_moe_gather_rows_pertoken": (c_int, [c_void_p] * 6 + [c_int32] * 5 + [c_void_p]),
    "flyb200_quant_pertoken": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32,
                                       c_void_p]),
    "flyb200_quant_1x128_devrows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32,
                                            c_void_p]),
    "flyb200_ep_plan_pack": (c_int, [c_void_p] * 4 + [c_int32] * 5 + [c_void_p] * 5),
    "flyb200_ep_gather_packed": (c_int, [c_void_p] * 5 + [c_int32] * 4 + [c_void_p]),
    "flyb200_ep_unpack_meta": (c_int, [c_void_p] + [c_int32] * 6 + [c_void_p] * 4),
    "flyb200_ep_combine": (c_int, [c_void_p] * 4 + [c_int32] * 4 + [c_void_p]),
    "flyb200_ep_buffer_create": (c_int, [c_int64, c_void_p, c_void_p]),
    "flyb200_ep_buffer_open": (c_int, [c_void_p, c_void_p]),
    "flyb200_ep_buffer_close": (c_int, [c_void_p]),
    "flyb200_ep_buffer_destroy": (c_int, [c_void_p]),
    "flyb200_ep_barrier": (c_int, [c_void_p, c_int32, c_int32, c_int64, c_uint32, c_int32, c_void_p]),
    "flyb200_ep_push": (c_int, [c_void_p] * 4 + [c_int32] * 6 + [c_void_p, c_int64] + [c_void_p] * 4),
    "flyb200_ep_pull_combine": (c_int, [c_void_p, c_int64] + [c_void_p] * 3 + [c_int32] * 5 + [c_void_p]),
    "flyb200_ep_reduce_push": (c_int, [c_void_p, c_void_p, c_void_p, c_int64] + [c_int32] * 6 + [c_void_p]),
    "flyb200_int4_repack": (c_int, [c_void_p, c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_void_p]),
    "flyb200_int4_gemm": (c_int, [c_void_p] * 4 + [c_int32] * 3 + [POINTER(GemmCfg), c_void_p]),
    "flyb200_query_device_error": (c_int, [c_void_p, POINTER(c_int32)]),
    "flyb200_last_error_string": (c_char_p, []),
    "flyb200_version": (c_int, []),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m flydsl_b200.build` "
            "(needs nvcc; there is no fallback path)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int) -> None:
    """Raise Flyb200Error for a non-zero status (ValueError for argument errors)."""
    if status == OK:
        return
    msg = load().flyb200_last_error_string().decode("utf-8", "replace")
    if status == ERR_INVALID_ARGUMENT:
        raise ValueError(f"libflyb200: {msg}")
    raise Flyb200Error(status, msg)


def stream_handle(stream) -> int:
    """torch.cuda.Stream | raw int handle | None (torch's current stream) -> cudaStream_t value.

    Mirrors the reference's Stream argument, which accepts a torch stream or a raw handle
    (python/flydsl/expr/typing.py:312-332).
    """
    if stream is None:
        import torch

        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    handle = getattr(stream, "cuda_stream", None)
    if handle is None:
        raise TypeError(f"stream must be a torch.cuda.Stream, an int handle or None, got {type(stream)!r}")
    return int(handle)


def query_device_error(stream=None) -> int:
    """Synchronise `stream`, return the device error word (0 = fine) and clear it."""
    code = c_int32(0)
    status = load().flyb200_query_device_error(stream_handle(stream), ctypes.byref(code))
    if status not in (OK, ERR_DEVICE_TIMEOUT):
        check(status)
    return int(code.value)
