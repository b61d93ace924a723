"""Dense FP8 GEMM with per-token / per-channel scales behind the reference's factory signature.

``compile_preshuffle_gemm_a8(...)`` mirrors kernels/preshuffle_gemm.py:39-52 of the reference for
``in_dtype="fp8"``: keyword-only shape/tile arguments, the same ``ValueError`` conditions, and it
returns a launcher called as ``fn(c, a, b_shuffled, scale_a, scale_b, M, N, stream)`` (reference
launch_gemm, :1269-1303) computing ``C = (A @ B^T) * scale_a[:, None] * scale_b[None, :]`` -- the
contract of run_torch in tests/kernels/test_preshuffle_gemm.py:55-66. The other input types of the
reference factory (int8, int4, fp16, bf16, fp4) are outside this package. Nothing is compiled at run
time: the launcher forwards to ``flyb200_pertoken_gemm`` in the prebuilt CUDA library.
"""
from __future__ import annotations

import ctypes
from typing import Optional

from .. import _lib

_OUT = {"bf16": _lib.BF16, "fp16": _lib.F16}


class PertokenGemmLauncher:
    """Callable returned by the factory. Holds only compile-time constants; buffers are the caller's."""

    def __init__(self, N, K, out_dtype, name, path=0):
        self.N, self.K = int(N), int(K)
        self.out_dtype = out_dtype
        self._out_code = _OUT[out_dtype]
        self._cfg = _lib.GemmCfg(0, 0, int(path), 0)
        self._cfg_ref = ctypes.byref(self._cfg)
        self.__name__ = name
        self._fn = _lib.load().flyb200_pertoken_gemm

    def __call__(self, c, a, b, scale_a, scale_b, m, n, stream=None):
        """c [M,N] bf16/fp16, a [M,K] fp8, b repacked fp8 [N,K] (this package's shuffle_weight),
        scale_a f32 [M], scale_b f32 [N]. Only ``data_ptr()`` of each tensor is read, so flattened
        views are fine. Asynchronous on ``stream``."""
        if getattr(b, "is_shuffled", False) and getattr(b, "flyb200_layout", None) is None:
            raise ValueError("b was repacked by a different shuffle_weight; use flydsl_b200.utils.shuffle_weight")
        if scale_a.numel() < int(m) or scale_b.numel() < int(n):
            raise ValueError("scale_a needs M entries and scale_b N entries (unscaled inputs are not supported)")
        _lib.check(self._fn(c.data_ptr(), a.data_ptr(), b.data_ptr(), scale_a.data_ptr(),
                            scale_b.data_ptr(), int(m), int(n), self.K, self._out_code,
                            self._cfg_ref, _lib.stream_handle(stream)))


def compile_preshuffle_gemm_a8(
    *,
    M: int = 0,
    N: int = 0,
    K: int,
    tile_m: int,
    tile_n: int,
    tile_k: int,
    in_dtype: str = "fp8",
    out_dtype: str = "fp16",
    lds_stage: int = 2,
    use_cshuffle_epilog: bool = False,
    waves_per_eu: Optional[int] = None,
    use_async_copy: bool = False,
    path: str = "auto",
):
    """Build a launcher for ``C = (A @ B^T) * scale_a * scale_b`` with FP8 (e4m3) operands.

    ``tile_m/tile_n/tile_k``, ``lds_stage``, ``use_cshuffle_epilog``, ``waves_per_eu`` and
    ``use_async_copy`` are accepted and validated like the reference does but do not pick the B200
    tile (128 x 256 x 128, whole K accumulated in tensor memory). M and N are run-time arguments of
    the launcher, as in the reference. ``path`` (extension): ``"auto"`` sends M <= 64 to the swap-AB
    split-K decode kernel when that pays off, ``"tiled"`` / ``"decode"`` force one of the two.
    """
    paths = {"auto": 0, "tiled": 1, "decode": 2, "pair": 3}
    if path not in paths:
        raise ValueError(f"path must be one of {tuple(paths)}, got {path!r}")
    if in_dtype not in ("fp8", "int8", "int4", "fp16", "bf16", "fp4"):
        raise ValueError(
            "in_dtype must be one of ('fp8','int8','int4','fp16','bf16','fp4'), " f"got {in_dtype!r}")
    if out_dtype not in ("fp16", "bf16"):
        raise ValueError(f"out_dtype must be 'fp16' or 'bf16', got {out_dtype!r}")
    if in_dtype != "fp8":
        raise NotImplementedError(f"in_dtype {in_dtype!r}: only 'fp8' is built in this package")
    if (int(tile_k) % 64) != 0:
        raise ValueError(f"tile_k_bytes must be divisible by 64, got tile_k_bytes={int(tile_k)} "
                         f"(tile_k={tile_k}, elem_bytes=1)")
    if K % 128 != 0:
        raise ValueError(f"K ({K}) must be divisible by 128 on this build")
    if N and N % 16 != 0:
        raise ValueError(f"N ({N}) must be divisible by 16")
    name = f"pt_gemm_{out_dtype}_t{tile_m}x{tile_n}x{tile_k}"
    return PertokenGemmLauncher(N, K, out_dtype, name, paths[path])
