"""CPU oracle of the weight-only int4 x bf16 GEMM. TEST INFRASTRUCTURE ONLY: imported by tests/,
the smoke check and bench.py's CPU baseline, never by the product path.

Parity UNPINNED: the reference holds no kernel, test or golden vector for this exact format (signed
int4, groups of 128 along K, bf16 scales, no zero point). The recipe is the one the benchmark
configuration states -- quantise with scale = amax/7 per group, dequantise, matmul -- and the
nearest reference code is the W4A16 dequantisation of kernels/moe_gemm_2stage.py:607-630
(value * scale, no zero point) and the nibble unpack of kernels/mfma_preshuffle_pipeline.py:202-222.
"""
from __future__ import annotations

import numpy as np
import torch

GROUP = 128


def quantize_int4_groupwise_ref(w: torch.Tensor):
    """w [N, K] f32 -> (q int8 [-8, 7], scales bf16 [N, K/128]); scale = amax/7 (0 -> 1), q = round(w/scale)."""
    N, K = w.shape
    g = w.float().reshape(N, K // GROUP, GROUP)
    scale = (g.abs().amax(dim=-1) / 7.0).to(torch.bfloat16)
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = torch.round(g / scale.float().unsqueeze(-1)).clamp(-8, 7).to(torch.int8).reshape(N, K)
    return q, scale


def dequant_int4_ref(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    N, K = q.shape
    return (q.float().reshape(N, K // GROUP, GROUP) * scales.float().unsqueeze(-1)).reshape(N, K)


def int4_gemm_ref(a: torch.Tensor, q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Dequantise, then matmul in fp32: a bf16 [M, K] -> f32 [M, N]."""
    return a.float() @ dequant_int4_ref(q, scales).t()


def pack_int4_ref(q: np.ndarray) -> np.ndarray:
    """The kernel's packed layout in numpy: q int8 [N, K] -> uint8 [K/128, N/8, 4, 8, 16]: per group of
    128 K elements and block of 8 rows, four 16-byte chunks (32 K elements each), each chunk holding
    its 8 rows back to back. Nibble = q + 8; the eight nibbles of a 32-bit little-endian word hold K
    elements e0 e2 e4 e6 e1 e3 e5 e7. N % 8 == 0."""
    N, K = q.shape
    nib = (q.astype(np.int32) + 8).astype(np.uint32).reshape(N, K // GROUP, 16, 8)
    order = [0, 2, 4, 6, 1, 3, 5, 7]
    word = np.zeros((N, K // GROUP, 16), dtype=np.uint32)
    for pos, e in enumerate(order):
        word |= nib[..., e] << np.uint32(4 * pos)
    out = word.reshape(N // 8, 8, K // GROUP, 4, 4).transpose(2, 0, 3, 1, 4).copy()   # [g, n/8, chunk, row, word]
    return out.view(np.uint8).reshape(K // GROUP, N // 8, 4, 8, 16)


def make_int4_case(M: int, N: int, K: int, seed: int = 0, w_std: float = 0.02):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g) * w_std
    q, s = quantize_int4_groupwise_ref(w)
    return {"a": a, "w": w, "q": q, "scales": s}
