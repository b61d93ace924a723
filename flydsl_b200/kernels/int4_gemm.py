"""Weight-only int4 x bf16 GEMM for decode-size batches (M <= 64), CUDA (csrc/int4_gemm.cu).

Contract: ``C = A @ dequant(W)^T`` with ``W`` signed 4-bit values in [-8, 7] and one bf16 scale per
(output row, 128-wide K group), bf16 activations and output, fp32 accumulation. The reference has no
kernel of exactly this format; its nearest code is the W4A16 MoE path (kernels/moe_gemm_2stage.py:
607-630) and the int4 unpack helpers (kernels/mfma_preshuffle_pipeline.py:202-222), so the layout
here is this library's own, produced by :func:`pack_int4_weight`.
"""
from __future__ import annotations

import functools
from typing import Optional, Tuple

import torch

from .. import _lib

GROUP = 128


def quantize_int4_groupwise(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w [N, K]`` float -> (q int8 in [-8, 7] ``[N, K]``, scales bf16 ``[N, K/128]``):
    ``scale = amax(|group|) / 7`` rounded to bf16 (0 -> 1), ``q = round(w / scale)`` clamped.
    Torch ops on whatever device ``w`` lives on (set-up, not a hot path)."""
    N, K = w.shape
    if K % GROUP:
        raise ValueError(f"K ({K}) must be a multiple of {GROUP}")
    g = w.float().reshape(N, K // GROUP, GROUP)
    scale = (g.abs().amax(dim=-1) / 7.0).to(torch.bfloat16)
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = torch.round(g / scale.float().unsqueeze(-1)).clamp_(-8, 7).to(torch.int8).reshape(N, K)
    return q, scale


def pack_int4_weight(q: torch.Tensor, scales: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """int8 values ``[N, K]`` in [-8, 7] + bf16 scales ``[N, K/128]`` -> the kernel's layout:
    packed uint8 ``[K/128, N/8, 4, 8, 16]`` (per group and block of 8 rows: four 16-byte chunks, each
    holding its 8 rows back to back) and scales bf16 ``[K/128, N]`` (CUDA). ``N % 8 == 0``."""
    if not q.is_cuda:
        raise ValueError("pack_int4_weight needs CUDA tensors (this library has no CPU path)")
    N, K = q.shape
    if q.dtype != torch.int8 or K % GROUP or N % 8 or tuple(scales.shape) != (N, K // GROUP):
        raise ValueError("expected int8 [N, K] with K % 128 == 0, N % 8 == 0 and scales [N, K/128]")
    q = q.contiguous()
    scales = scales.to(torch.bfloat16).contiguous()
    wq = torch.empty((K // GROUP, N // 8, 4, 8, 16), dtype=torch.uint8, device=q.device)
    st = torch.empty((K // GROUP, N), dtype=torch.bfloat16, device=q.device)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().flyb200_int4_repack(q.data_ptr(), scales.data_ptr(), N, K, wq.data_ptr(),
                                                   st.data_ptr(), _lib.stream_handle(None)))
    return wq, st


class Int4GemmLauncher:
    """``fn(c, a, wq, scales_t, m, stream)``: c bf16 ``[m, N]``; a bf16 ``[m, K]``; ``wq`` / ``scales_t``
    from :func:`pack_int4_weight`."""

    def __init__(self, N: int, K: int, split_k: Optional[int], path: str = "auto"):
        if path not in ("auto", "stream", "tensor"):
            raise ValueError("path must be 'auto', 'stream' (mma.sync, weights unpacked in registers) or "
                             "'tensor' (tcgen05, weights unpacked through shared memory)")
        self.N, self.K = int(N), int(K)
        self._cfg = _lib.GemmCfg(0, 0, {"auto": 0, "stream": 1, "tensor": 2}[path], int(split_k or 0))
        self._fn = _lib.load().flyb200_int4_gemm

    def __call__(self, c, a, wq, scales_t, m, stream=None):
        import ctypes

        if a.dtype != torch.bfloat16 or c.dtype != torch.bfloat16:
            raise ValueError("int4 GEMM takes bf16 activations and writes bf16")
        if tuple(a.shape) != (int(m), self.K) or tuple(c.shape) != (int(m), self.N):
            raise ValueError(f"expected a [{m}, {self.K}] and c [{m}, {self.N}]")
        if not (a.is_contiguous() and c.is_contiguous()):
            raise ValueError("a and c must be contiguous")
        _lib.check(self._fn(c.data_ptr(), a.data_ptr(), wq.data_ptr(), scales_t.data_ptr(), int(m), self.N,
                            self.K, ctypes.byref(self._cfg), _lib.stream_handle(stream)))


@functools.lru_cache(maxsize=256)
def compile_int4_weight_only_gemm(*, N: int, K: int, group_size: int = GROUP, split_k: Optional[int] = None,
                                  path: str = "auto"):
    """Launcher for ``C[m, N] = A[m, K] @ dequant(W)^T``, ``m <= 64`` chosen per call. ``path`` picks
    the kernel: ``"stream"`` (csrc/int4_stream.cu), ``"tensor"`` (csrc/int4_gemm.cu) or ``"auto"``
    (the default: the former up to 32 tokens, the latter above)."""
    if group_size != GROUP:
        raise ValueError(f"group_size must be {GROUP}")
    if N % 128 or K % 128:
        raise ValueError(f"N and K must be multiples of 128 (N={N}, K={K})")
    return Int4GemmLauncher(N, K, split_k, path)
