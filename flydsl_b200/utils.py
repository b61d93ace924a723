"""Host helpers with the names and argument meaning of the reference's test utilities
(tests/utils.py, tests/kernels/test_moe_gemm.py), backed by the CUDA library.

shuffle_weight        weight repack for the B200 kernels   (reference: tests/utils.py:76-96)
pertoken_quant        amax/dtype-max quantiser (torch ops) (reference: tests/utils.py:29-73)
quant_1x128           1x128 group quantiser, CUDA          (reference: tests/kernels/test_moe_blockscale.py:346-361)
moe_sorting           routing sort, CUDA                   (reference: tests/kernels/test_moe_gemm.py:97-161)
build_routing_buffers sorter wrapper                       (reference: tests/kernels/test_moe_gemm.py:223-295)
route_topk            router top-k + softmax, CUDA         (reference: tests/kernels/test_moe_blockscale.py:228-230)
get_topk_valid_mask   EP slot mask                         (reference: tests/kernels/test_moe_gemm.py:211-220)
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

FP8_DTYPE = torch.float8_e4m3fn  # OCP e4m3 (max 448), the format B200 tensor cores take
FP8_MAX = 448.0
WEIGHT_LAYOUT_TAG = "flyb200_k128_sw128"


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def shuffle_weight(x: torch.Tensor, layout=(16, 16), use_int4: bool = False) -> torch.Tensor:
    """Repack an fp8 weight ``[..., N, K]`` for the B200 kernels; same shape and dtype out.

    Same call as the reference's shuffle_weight, but the byte layout is the B200 one: per leading
    index ``[K/128][N/8][8][128 B]`` with the 128-byte swizzle applied (see csrc/repack.cu). The
    ``layout`` argument is accepted for signature compatibility and ignored. A tensor repacked by
    the reference's function is NOT accepted by these kernels.
    """
    if use_int4:
        raise NotImplementedError("int4 weights are outside the block-scale fp8 path")
    if x.element_size() != 1:
        raise ValueError(f"shuffle_weight expects a 1-byte dtype, got {x.dtype}")
    if x.dim() < 2:
        raise ValueError("shuffle_weight expects [..., N, K]")
    _require_cuda(x, "x")
    n, k = x.shape[-2], x.shape[-1]
    assert n % 16 == 0, f"{n} % 16 == {n % 16}"
    assert k % 128 == 0, f"{k} % 128 == {k % 128}"
    batch = x.numel() // (n * k) if x.numel() else 0
    out = torch.empty_like(x)
    if batch:
        with torch.cuda.device(x.device):
            _lib.check(_lib.load().flyb200_repack_weight_fp8(
                out.data_ptr(), x.data_ptr(), batch, n, k, _lib.stream_handle(None)))
    out.is_shuffled = True
    out.flyb200_layout = WEIGHT_LAYOUT_TAG
    return out


def pertoken_quant(x, scale=None, x_scale=None, scale_dtype=torch.float32,
                   quant_dtype=FP8_DTYPE, dtypeMax=None):
    """Row-wise amax quantiser: ``scale = amax(|row|)/dtypeMax`` (0 -> 1), ``y = x/scale``.

    Same contract as the reference's pertoken_quant (tests/utils.py:29-73), including its
    handling of NaN/Inf inputs; runs as torch ops on whatever device ``x`` lives on. For 1x128
    groups reshape to ``[-1, 128]`` first, for 128x128 blocks bring each block into one row.
    """
    x = x.to(torch.float32)
    hidden = x if x_scale is None else x * x_scale
    if dtypeMax is None:
        dtypeMax = (torch.finfo(quant_dtype).max if quant_dtype.is_floating_point
                    else torch.iinfo(quant_dtype).max)
    hidden = torch.nan_to_num(hidden, nan=0.0, posinf=float(dtypeMax), neginf=-float(dtypeMax))
    if scale is None:
        hi = torch.amax(hidden, dim=-1, keepdim=True)
        lo = torch.amin(hidden, dim=-1, keepdim=True)
        scale = torch.maximum(hi, -lo) / dtypeMax
        scale[scale == 0] = 1
    scale = torch.nan_to_num(scale, nan=1.0, posinf=1.0, neginf=1.0)
    y = (hidden / scale).to(dtype=quant_dtype)
    return y, scale.to(scale_dtype)


def _dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return _lib.BF16
    if dt == torch.float16:
        return _lib.F16
    if dt == torch.float32:
        return _lib.F32
    raise ValueError(f"unsupported dtype {dt}")


def quant_1x128(x: torch.Tensor, stream=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """CUDA 1x128 group quantiser: ``x [rows, cols]`` (f32/f16/bf16) -> (fp8 ``[rows, cols]``,
    scales f32 ``[cols/128, rows]`` i.e. already in the transposed layout the GEMMs read)."""
    _require_cuda(x, "x")
    if x.dim() != 2:
        raise ValueError("quant_1x128 expects [rows, cols]")
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=FP8_DTYPE, device=x.device)
    st = torch.empty((cols // 128, rows), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().flyb200_quant_1x128(
            x.data_ptr(), q.data_ptr(), st.data_ptr(), rows, cols, _dtype_code(x.dtype),
            _lib.stream_handle(stream)))
    return q, st


def quant_pertoken(x: torch.Tensor, num_rows_dev: Optional[torch.Tensor] = None, out=None, scale_out=None,
                   stream=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """CUDA whole-row quantiser, bit for bit ``pertoken_quant`` on f16/bf16 rows: ``x [rows, cols]``
    -> (fp8 ``[rows, cols]``, scales f32 ``[rows]``). ``num_rows_dev`` (device int32) limits the work to
    its first value's leading rows; the other rows of the outputs are left as they are."""
    _require_cuda(x, "x")
    if x.dim() != 2 or x.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("quant_pertoken expects f16/bf16 [rows, cols]")
    rows, cols = x.shape
    if out is None:
        out = torch.empty((rows, cols), dtype=FP8_DTYPE, device=x.device)
    if scale_out is None:
        scale_out = torch.empty((rows,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().flyb200_quant_pertoken(
            x.data_ptr(), out.data_ptr(), scale_out.data_ptr(),
            None if num_rows_dev is None else num_rows_dev.data_ptr(), rows, cols, _dtype_code(x.dtype),
            _lib.stream_handle(stream)))
    return out, scale_out


def moe_sorting(topk_ids: torch.Tensor, topk_weights: torch.Tensor, *, num_experts: int,
                block_size: int, expert_mask: Optional[torch.Tensor] = None,
                num_local_tokens=None, stream=None, permute=None
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """CUDA routing sort with the outputs of moe_sorting_torch_native
    (tests/kernels/test_moe_gemm.py:97-161): (sorted_ids i32, sorted_weights f32,
    sorted_expert_ids i32, num_tokens_post_pad i32[2]).

    ``permute=(x, x_scale_t, x_sorted, x_scale_sorted_t)`` fuses the permute of the activations into
    routing order into the same launch (what ``moe_gather_rows`` does separately): x fp8 ``[T, K]``,
    x_scale_t f32 ``[K/128, T]``, outputs ``[len(sorted_ids), K]`` and ``[K/128, len(sorted_ids)]``."""
    _require_cuda(topk_ids, "topk_ids")
    _require_cuda(topk_weights, "topk_weights")
    if topk_ids.dtype != torch.int32:
        topk_ids = topk_ids.to(torch.int32)
    if topk_weights.dtype != torch.float32:
        topk_weights = topk_weights.to(torch.float32)
    tokens, topk = topk_ids.shape
    dev = topk_ids.device
    max_len = int(topk_ids.numel() + int(num_experts) * int(block_size) - int(topk))
    max_blocks = (max_len + int(block_size) - 1) // int(block_size)
    sorted_ids = torch.empty((max_len,), dtype=torch.int32, device=dev)
    sorted_weights = torch.empty((max_len,), dtype=torch.float32, device=dev)
    sorted_expert_ids = torch.empty((max_blocks,), dtype=torch.int32, device=dev)
    num_post_pad = torch.empty((2,), dtype=torch.int32, device=dev)
    mask_ptr = None
    if expert_mask is not None:
        expert_mask = expert_mask.to(device=dev, dtype=torch.int32).contiguous()
        mask_ptr = expert_mask.data_ptr()
    if num_local_tokens is None:
        nlt = -1
    elif isinstance(num_local_tokens, torch.Tensor):
        nlt = int(num_local_tokens.item())
    else:
        nlt = int(num_local_tokens)
    with torch.cuda.device(dev):
        if permute is None:
            _lib.check(_lib.load().flyb200_moe_sort(
                topk_ids.data_ptr(), topk_weights.data_ptr(), tokens, topk, int(num_experts),
                int(block_size), mask_ptr, nlt, sorted_ids.data_ptr(), sorted_weights.data_ptr(),
                sorted_expert_ids.data_ptr(), num_post_pad.data_ptr(), _lib.stream_handle(stream)))
        else:
            x, xs_t, x_sorted, xs_sorted = permute
            if x.shape[0] != tokens or tuple(x_sorted.shape) != (max_len, x.shape[1]) or \
                    tuple(xs_sorted.shape) != (x.shape[1] // 128, max_len):
                raise ValueError("permute buffers do not match [T, K] -> [T*k + E*block - k, K]")
            _lib.check(_lib.load().flyb200_moe_sort_permute(
                topk_ids.data_ptr(), topk_weights.data_ptr(), tokens, topk, int(num_experts),
                int(block_size), mask_ptr, nlt, sorted_ids.data_ptr(), sorted_weights.data_ptr(),
                sorted_expert_ids.data_ptr(), num_post_pad.data_ptr(), x.data_ptr(), xs_t.data_ptr(),
                x_sorted.data_ptr(), xs_sorted.data_ptr(), int(x.shape[1]), _lib.stream_handle(stream)))
    return sorted_ids, sorted_weights, sorted_expert_ids, num_post_pad


def route_topk(logits: torch.Tensor, topk: int, stream=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """CUDA router of the reference's MoE test (tests/kernels/test_moe_blockscale.py:228-230):
    ``vals, ids = topk(logits)``; ``weights = softmax(vals)``. Returns (ids i32 [T, k], weights f32
    [T, k]); slot order = descending score."""
    _require_cuda(logits, "logits")
    if logits.dim() != 2:
        raise ValueError("route_topk expects [tokens, experts]")
    if logits.dtype != torch.float32:
        logits = logits.float()
    T, E = logits.shape
    ids = torch.empty((T, int(topk)), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, int(topk)), dtype=torch.float32, device=logits.device)
    if T:
        with torch.cuda.device(logits.device):
            _lib.check(_lib.load().flyb200_moe_route_topk(logits.data_ptr(), T, E, int(topk), ids.data_ptr(),
                                                          w.data_ptr(), _lib.stream_handle(stream)))
    return ids, w


def get_topk_valid_mask(topk_ids: torch.Tensor, expert_mask: Optional[torch.Tensor] = None):
    """``valid_mask[t, s] = expert_mask[topk_ids[t, s]]`` (all ones without a mask), int8."""
    if expert_mask is None:
        return torch.ones(topk_ids.shape, dtype=torch.int8, device=topk_ids.device)
    return expert_mask[topk_ids.long()].to(torch.int8)


def build_routing_buffers(*, topk_ids: torch.Tensor, topk_weights: torch.Tensor, experts: int,
                          model_dim: int, tile_m: int, moe_sort_mode: Optional[str] = None):
    """Routing buffers shared by both MoE stages:
    ``(sorted_token_ids, sorted_weights, sorted_expert_ids, num_valid_ids[:1], sorted_size, blocks)``.

    ``moe_sort_mode`` is accepted for signature compatibility; there is one sorter here (CUDA,
    bit-identical to the reference's "torch" mode). ``model_dim`` is unused, as in the reference.
    """
    mode = str(moe_sort_mode or "torch").lower().strip()
    if mode not in ("aiter", "torch"):
        raise ValueError(f"invalid moe_sort_mode={mode!r} (expected 'aiter' or 'torch')")
    ids, weights, expert_ids, post_pad = moe_sorting(
        topk_ids, topk_weights, num_experts=int(experts), block_size=int(tile_m))
    num_valid_ids = post_pad[:1].contiguous()
    return ids, weights, expert_ids, num_valid_ids, int(ids.numel()), int(expert_ids.numel())


def moe_gather_rows(x, scale_t, sorted_ids, num_valid_ids, *, topk: int, by_slot: bool = False,
                    out=None, scale_out=None, stream=None, per_token: bool = False):
    """Activations into routing order for the TMA-fed stage kernels (``a_sorted=True``).

    ``x`` fp8 ``[rows_in, K]`` and ``scale_t`` f32 ``[K/128, rows_in]``; row i of the result is the
    row of sorted position i (token ``t``, or route ``t*topk+slot`` with ``by_slot``), zero for
    padding. Returns ``(x_sorted [len(sorted_ids), K], scale_sorted_t [K/128, len(sorted_ids)])``.
    ``per_token``: one scale per row instead (``scale_t [rows_in]`` -> ``[len(sorted_ids)]``)."""
    _require_cuda(x, "x")
    rows_in, K = x.shape
    rows_out = sorted_ids.numel()
    if out is None:
        out = torch.empty((rows_out, K), dtype=x.dtype, device=x.device)
    if per_token:
        if scale_t.numel() != rows_in:
            raise ValueError(f"per_token gather needs one scale per row ({rows_in}), got {scale_t.numel()}")
        if scale_out is None:
            scale_out = torch.empty((rows_out,), dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            _lib.check(_lib.load().flyb200_moe_gather_rows_pertoken(
                x.data_ptr(), scale_t.data_ptr(), sorted_ids.data_ptr(), num_valid_ids.data_ptr(),
                out.data_ptr(), scale_out.data_ptr(), rows_in, K, int(topk), rows_out, int(bool(by_slot)),
                _lib.stream_handle(stream)))
        return out, scale_out
    if scale_out is None:
        scale_out = torch.empty((K // 128, rows_out), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().flyb200_moe_gather_rows(
            x.data_ptr(), scale_t.data_ptr(), sorted_ids.data_ptr(), num_valid_ids.data_ptr(),
            out.data_ptr(), scale_out.data_ptr(), rows_in, K, int(topk), rows_out, int(bool(by_slot)),
            _lib.stream_handle(stream)))
    return out, scale_out
