"""Dense FP8 block-scale GEMM behind the reference's factory signature.

``compile_blockscale_preshuffle_gemm(...)`` mirrors kernels/blockscale_preshuffle_gemm.py:39-52 of
the reference: keyword-only shape/tile arguments, the same ``ValueError`` conditions, and it returns a
launcher called as ``fn(c, a, b_shuffled, scale_a_T_flat, scale_b_flat, M, N, stream)``
(reference launch_gemm, :842-876). Nothing is compiled at run time: the launcher forwards to
``flyb200_blockscale_gemm`` in the prebuilt CUDA library.
"""
from __future__ import annotations

import ctypes

from .. import _lib

_OUT = {"bf16": _lib.BF16, "fp16": _lib.F16}


class BlockscaleGemmLauncher:
    """Callable returned by the factory. Holds only compile-time constants; buffers are the caller's."""

    def __init__(self, M, N, K, out_dtype, block_n, name, path=0, split_k=0):
        self.M, self.N, self.K = int(M), int(N), int(K)
        self.out_dtype = out_dtype
        self._out_code = _OUT[out_dtype]
        self._cfg = _lib.GemmCfg(int(block_n or 0), 0, int(path or 0), int(split_k or 0))
        self._cfg_ref = ctypes.byref(self._cfg)
        self.__name__ = name
        self._fn = _lib.load().flyb200_blockscale_gemm

    def __call__(self, c, a, b, scale_a, scale_b, m, n, stream=None):
        """c [M,N] bf16/fp16, a [M,K] fp8, b repacked fp8 [N,K] (this package's shuffle_weight),
        scale_a f32 [K/128, M] flat, scale_b f32 [ceil(N/128), K/128] flat. Only ``data_ptr()`` of
        each tensor is read, so flattened views are fine. Asynchronous on ``stream``."""
        if getattr(b, "is_shuffled", False) and getattr(b, "flyb200_layout", None) is None:
            raise ValueError("b was repacked by a different shuffle_weight; use flydsl_b200.utils.shuffle_weight")
        _lib.check(self._fn(c.data_ptr(), a.data_ptr(), b.data_ptr(), scale_a.data_ptr(),
                            scale_b.data_ptr(), int(m), int(n), self.K, self._out_code,
                            self._cfg_ref, _lib.stream_handle(stream)))


def compile_blockscale_preshuffle_gemm(
    *,
    M: int,
    N: int,
    K: int,
    tile_m: int,
    tile_n: int,
    tile_k: int,
    scale_block_k: int = 128,
    out_dtype: str = "bf16",
    use_cshuffle_epilog: bool = False,
    waves_per_eu: int = None,
    use_async_copy: bool = False,
    block_n: int = None,
    path: str = "auto",
    split_k: int = None,
):
    """Build a launcher for C = dequant(A) @ dequant(B)^T with 1x128 / 128x128 fp32 block scales.

    ``tile_m/tile_n/tile_k`` are validated like the reference does but do not pick the B200 tile
    (the MMA tile is 128 x block_n x 128; ``block_n`` in {32,64,128,256} overrides the built-in
    heuristic; ``path`` = "auto" | "tiled" | "decode" picks the kernel: M <= 64 defaults to the
    swap-AB split-K decode kernel, ``split_k`` its cluster size). ``use_cshuffle_epilog``, ``waves_per_eu`` and ``use_async_copy`` are AMD tuning
    switches, accepted and ignored.
    """
    if out_dtype not in ("fp16", "bf16"):
        raise ValueError(f"out_dtype must be 'fp16' or 'bf16', got {out_dtype!r}")
    if tile_k % scale_block_k != 0:
        raise ValueError(f"tile_k ({tile_k}) must be divisible by scale_block_k ({scale_block_k})")
    if K % tile_k != 0:
        raise ValueError(f"K ({K}) must be divisible by tile_k ({tile_k})")
    if K % scale_block_k != 0:
        raise ValueError(f"K ({K}) must be divisible by scale_block_k ({scale_block_k})")
    if tile_k % 64 != 0:
        raise ValueError(f"tile_k_bytes must be divisible by 64, got {tile_k}")
    if (tile_m * tile_k) % 256 != 0:
        raise ValueError(f"tile_m*tile_k must be divisible by 256: tile_m={tile_m}, tile_k={tile_k}")
    if ((tile_m * tile_k) // 256) % 4 != 0:
        raise ValueError(f"bytes_per_thread_a ({(tile_m * tile_k) // 256}) must be divisible by 4")
    if scale_block_k != 128:
        raise ValueError(f"scale_block_k must be 128 on this build, got {scale_block_k}")
    if N % 16 != 0:
        raise ValueError(f"N ({N}) must be divisible by 16")
    if block_n not in (None, 0, 32, 64, 128, 256):
        raise ValueError(f"block_n must be one of 32, 64, 128, 256, got {block_n}")
    paths = {"auto": 0, "tiled": 1, "decode": 2}
    if path not in paths:
        raise ValueError(f"path must be one of {sorted(paths)}, got {path!r}")
    if split_k not in (None, 0, 1, 2, 3, 4, 5, 6, 7, 8):
        raise ValueError(f"split_k must be in 1..8, got {split_k}")
    name = f"bs_gemm_{out_dtype}_t128x{block_n or 'auto'}x128_{path}"
    return BlockscaleGemmLauncher(M, N, K, out_dtype, block_n, name, paths[path], split_k)
