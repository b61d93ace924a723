"""Two-stage FP8 block-scale MoE behind the reference's factory signatures
(kernels/moe_blockscale_2stage.py of the reference).

compile_moe_blockscale_gemm1     reference :74-89   -> launcher args of :1165-1214
compile_moe_blockscale_gemm2     reference :1219-1238 -> launcher args of :2390-2440
compile_moe_reduction            reference :2446-2638
MoeGemm2Mode / compile_moe_blockscale_gemm2_ex   reference :2642-2826

The factories validate like the reference, are ``functools.lru_cache``d like the reference, and
return launchers that forward to the prebuilt CUDA library; nothing is compiled at run time.
"""
from __future__ import annotations

import ctypes
import functools
import logging

from .. import _lib

_OUT_CODES = {
    "f16": _lib.F16, "fp16": _lib.F16, "half": _lib.F16,
    "bf16": _lib.BF16, "bfloat16": _lib.BF16,
    "f32": _lib.F32, "fp32": _lib.F32, "float": _lib.F32,
}


def _cfg(block_n, path_bits=0):
    cfg = _lib.GemmCfg(int(block_n or 0), 0, int(path_bits), 0)
    return cfg, ctypes.byref(cfg)


class MoeGemm1Launcher:
    """``fn(out, x, w, scale_x, scale_w, sorted_token_ids, expert_ids, sorted_weights,
    max_token_ids, tokens, inter, k, size_expert_ids, stream)``.

    out f16/bf16 ``[tokens, topk, inter]``; x fp8 ``[tokens, model_dim]``; w fp8 repacked
    ``[E, 2*inter, model_dim]`` (gate rows then up rows per expert); scale_x f32
    ``[model_dim/128, tokens]``; scale_w f32 ``[E*(2*inter/128), model_dim/128]``.
    """

    def __init__(self, model_dim, inter_dim, experts, topk, tile_m, doweight, out_code, block_n,
                 a_sorted=False, out_sorted=False):
        self.model_dim, self.inter_dim = int(model_dim), int(inter_dim)
        self.experts, self.topk, self.tile_m = int(experts), int(topk), int(tile_m)
        self.doweight, self.out_code = int(bool(doweight)), out_code
        self._cfg, self._cfg_ref = _cfg(block_n, (1 if a_sorted else 0) | (2 if out_sorted else 0))
        self._fn = _lib.load().flyb200_moe_gemm1

    def __call__(self, out, x, w, scale_x, scale_w, sorted_token_ids, expert_ids, sorted_weights,
                 max_token_ids, tokens, inter, k, size_expert_ids, stream=None):
        if int(inter) != self.inter_dim or int(k) != self.model_dim:
            raise ValueError(f"launcher was built for inter_dim={self.inter_dim}, model_dim={self.model_dim}; "
                             f"got inter={inter}, k={k}")
        _lib.check(self._fn(
            out.data_ptr(), x.data_ptr(), w.data_ptr(), scale_x.data_ptr(), scale_w.data_ptr(),
            sorted_token_ids.data_ptr(), expert_ids.data_ptr(), sorted_weights.data_ptr(),
            max_token_ids.data_ptr(), int(tokens), self.inter_dim, self.model_dim,
            int(size_expert_ids), self.experts, self.topk, self.tile_m, self.doweight,
            self.out_code, self._cfg_ref, _lib.stream_handle(stream)))

    def quantized(self, out_q, out_scale_t, x, w, scale_x, scale_w, sorted_token_ids, expert_ids,
                  sorted_weights, max_token_ids, tokens, size_expert_ids, stream=None):
        """Stage 1 with the 1x128 re-quantisation fused into its epilogue (routing-order layouts
        only): writes fp8 ``out_q [rows, inter]`` and ``out_scale_t [inter/128, rows]`` -- bit for bit
        what ``quant_1x128`` makes of the 16-bit stage-1 output -- and no 16-bit tensor at all.
        Rows of padding positions are left untouched."""
        _lib.check(_lib.load().flyb200_moe_gemm1_q8(
            out_q.data_ptr(), out_scale_t.data_ptr(), x.data_ptr(), w.data_ptr(), scale_x.data_ptr(),
            scale_w.data_ptr(), sorted_token_ids.data_ptr(), expert_ids.data_ptr(),
            sorted_weights.data_ptr(), max_token_ids.data_ptr(), int(tokens), self.inter_dim,
            self.model_dim, int(size_expert_ids), self.experts, self.topk, self.tile_m, self.doweight,
            self.out_code, self._cfg_ref, _lib.stream_handle(stream)))


class MoeGemm2Launcher:
    """``fn(out, x, w, scale_x, scale_w, sorted_token_ids, expert_ids, sorted_weights,
    num_valid_ids, tokens, n, k, size_expert_ids, stream)``.

    x fp8 ``[tokens*topk, inter]``; w fp8 repacked ``[E, model_dim, inter]``; scale_x f32
    ``[inter/128, tokens*topk]``; scale_w f32 ``[E*(model_dim/128), inter/128]``. With
    ``accumulate=True`` out is ``[tokens, model_dim]``, pre-zeroed by the caller, and routes are
    added atomically; with ``accumulate=False`` out is ``[tokens*topk, model_dim]``.
    """

    def __init__(self, model_dim, inter_dim, experts, topk, tile_m, doweight, accumulate, out_code,
                 block_n, a_sorted=False):
        self.model_dim, self.inter_dim = int(model_dim), int(inter_dim)
        self.experts, self.topk, self.tile_m = int(experts), int(topk), int(tile_m)
        self.doweight, self.accumulate, self.out_code = int(bool(doweight)), int(bool(accumulate)), out_code
        self._cfg, self._cfg_ref = _cfg(block_n, 1 if a_sorted else 0)
        self._fn = _lib.load().flyb200_moe_gemm2

    def __call__(self, out, x, w, scale_x, scale_w, sorted_token_ids, expert_ids, sorted_weights,
                 num_valid_ids, tokens, n, k, size_expert_ids, stream=None):
        if int(n) != self.model_dim or int(k) != self.inter_dim:
            raise ValueError(f"launcher was built for model_dim={self.model_dim}, inter_dim={self.inter_dim}; "
                             f"got n={n}, k={k}")
        _lib.check(self._fn(
            out.data_ptr(), x.data_ptr(), w.data_ptr(), scale_x.data_ptr(), scale_w.data_ptr(),
            sorted_token_ids.data_ptr(), expert_ids.data_ptr(), sorted_weights.data_ptr(),
            num_valid_ids.data_ptr(), int(tokens), self.model_dim, self.inter_dim,
            int(size_expert_ids), self.experts, self.topk, self.tile_m, self.doweight,
            self.accumulate, self.out_code, self._cfg_ref, _lib.stream_handle(stream)))


class MoeReduceLauncher:
    """``fn(X, Y, valid_mask, m_tokens, stream)``: ``Y[t,d] = sum_s X[t,s,d]`` (f32 accumulate)."""

    def __init__(self, topk, model_dim, dtype_code, use_mask):
        self.topk, self.model_dim = int(topk), int(model_dim)
        self.dtype_code, self.use_mask = dtype_code, bool(use_mask)
        self._fn = _lib.load().flyb200_moe_reduce

    def __call__(self, X, Y, valid_mask, m_tokens, stream=None):
        mask_ptr = None
        if self.use_mask:
            if valid_mask is None or valid_mask.numel() != int(m_tokens) * self.topk:
                raise ValueError("use_mask=True needs valid_mask [tokens, topk]")
            if valid_mask.element_size() != 1:
                raise ValueError("valid_mask must be a 1-byte dtype (uint8/int8/bool)")
            mask_ptr = valid_mask.data_ptr()
        _lib.check(self._fn(X.data_ptr(), Y.data_ptr(), mask_ptr, int(m_tokens), self.topk,
                            self.model_dim, self.dtype_code, _lib.stream_handle(stream)))


def _check_tiles(tile_m, tile_k, scale_block_k):
    if int(tile_k) % 64 != 0:
        raise ValueError(f"tile_k_bytes must be divisible by 64, got tile_k_bytes={tile_k} "
                         f"(tile_k={tile_k}, elem_bytes=1)")
    if int(scale_block_k) != 128:
        raise ValueError(f"scale_block_k must be 128 on this build, got {scale_block_k}")
    if not 1 <= int(tile_m) <= 128:
        raise ValueError(f"tile_m must be in [1, 128] (one routing block per 128-row MMA tile), got {tile_m}")


@functools.lru_cache(maxsize=1024)
def compile_moe_blockscale_gemm1(
    *,
    model_dim: int,
    inter_dim: int,
    experts: int,
    topk: int,
    tile_m: int,
    tile_n: int,
    tile_k: int,
    doweight_stage1: bool,
    scale_block_k: int = 128,
    out_dtype: str = "f16",
    use_cshuffle_epilog=None,
    waves_per_eu=None,
    block_n=None,
    a_sorted=False,
    out_sorted=False,
):
    """Stage 1: ``out[t, slot, :] = silu(x[t] @ Wgate[e]^T) * (x[t] @ Wup[e]^T)`` (optionally times
    the route weight). ``tile_m`` must equal the block size the routing buffers were sorted with;
    ``tile_n/tile_k`` are validated only; ``block_n`` (64/128/256 = gate+up MMA width) overrides
    the heuristic. ``use_cshuffle_epilog`` / ``waves_per_eu`` are AMD switches, ignored.

    Extensions (off by default, so the reference call is unchanged): ``a_sorted`` -- ``x`` and
    ``scale_x`` are already in routing order (``utils.moe_gather_rows``), fetched by TMA instead of
    gathered; ``out_sorted`` -- write ``out`` in routing order ``[T*k + E*tile_m - k, inter]``."""
    if out_dtype not in ("f16", "bf16"):
        raise ValueError(f"out_dtype must be 'f16' or 'bf16', got {out_dtype!r}")
    _check_tiles(tile_m, tile_k, scale_block_k)
    if model_dim % scale_block_k != 0:
        raise ValueError(f"model_dim ({model_dim}) must be divisible by scale_block_k ({scale_block_k})")
    if inter_dim % 128 != 0:
        raise ValueError(f"inter_dim ({inter_dim}) must be divisible by 128 (ScaleBlockN)")
    if block_n not in (None, 0, 64, 128, 256):
        raise ValueError(f"block_n must be one of 64, 128, 256, got {block_n}")
    if (a_sorted or out_sorted) and int(tile_m) % 8:
        raise ValueError(f"sorted layouts need tile_m to be a multiple of 8, got {tile_m}")
    return MoeGemm1Launcher(model_dim, inter_dim, experts, topk, tile_m, doweight_stage1,
                            _OUT_CODES[out_dtype], block_n, a_sorted, out_sorted)


@functools.lru_cache(maxsize=1024)
def compile_moe_blockscale_gemm2(
    *,
    model_dim: int,
    inter_dim: int,
    experts: int,
    topk: int,
    tile_m: int,
    tile_n: int,
    tile_k: int,
    doweight_stage2: bool,
    scale_block_k: int = 128,
    out_dtype: str = "f16",
    use_cshuffle_epilog=None,
    accumulate: bool = True,
    waves_per_eu=None,
    block_n=None,
    a_sorted=False,
):
    """Stage 2: ``A2[t*topk+slot] @ W2[e]^T`` (times the route weight when ``doweight_stage2``),
    atomically added into ``out[t]`` (``accumulate=True``) or stored per route. ``a_sorted``: ``x`` /
    ``scale_x`` are in routing order (rows = sorted positions), fetched by TMA."""
    out_s = str(out_dtype).strip().lower()
    if out_s not in _OUT_CODES:
        raise ValueError(f"out_dtype must be 'f16', 'bf16', or 'f32', got {out_dtype!r}")
    out_code = _OUT_CODES[out_s]
    if (not bool(accumulate)) and out_code == _lib.F32:
        raise ValueError("compile_moe_blockscale_gemm2(accumulate=False) only supports out_dtype in {'f16','bf16'}")
    _check_tiles(tile_m, tile_k, scale_block_k)
    if inter_dim % scale_block_k != 0:
        raise ValueError(f"inter_dim ({inter_dim}) must be divisible by scale_block_k ({scale_block_k})")
    if model_dim % 128 != 0:
        raise ValueError(f"model_dim ({model_dim}) must be divisible by 128 (ScaleBlockN)")
    if block_n not in (None, 0, 32, 64, 128, 256):
        raise ValueError(f"block_n must be one of 32, 64, 128, 256, got {block_n}")
    if a_sorted and int(tile_m) % 8:
        raise ValueError(f"sorted layouts need tile_m to be a multiple of 8, got {tile_m}")
    return MoeGemm2Launcher(model_dim, inter_dim, experts, topk, tile_m, doweight_stage2,
                            accumulate, out_code, block_n, a_sorted)


@functools.lru_cache(maxsize=1024)
def compile_moe_reduction(*, topk: int, model_dim: int, dtype_str: str = "f16", use_mask: bool = False):
    """Reduction over the top-k slots, the companion of ``accumulate=False`` stage 2."""
    ds = str(dtype_str).strip().lower()
    if ds not in _OUT_CODES:
        raise ValueError(f"dtype_str must be 'f16', 'bf16' or 'f32', got {dtype_str!r}")
    return MoeReduceLauncher(topk, model_dim, _OUT_CODES[ds], use_mask)


class MoeGemm2Mode:
    """Execution mode for stage 2."""

    ATOMIC = "atomic"  # atomic accumulation into [tokens, model_dim]
    REDUCE = "reduce"  # per-route store, then a fixed-order reduce (deterministic)


class _MoeGemm2ReduceWrapper:
    """Stage 2 in reduce mode: per-route rows into a scratch tensor, then the fixed-order sum over
    the top-k slots -- one C-ABI call. Call signature of the reference's wrapper (:2642-2737):
    ``fn(out, x, w, scale_x, scale_w, sorted_token_ids, expert_ids, sorted_weights, num_valid_ids,
    tokens, n, k, size_expert_ids, valid_mask=None, stream=None)``. The ``[tokens*topk, model_dim]``
    scratch is allocated per call, as the reference does (:2709-2715)."""

    _TORCH_DTYPES = {_lib.F16: "float16", _lib.BF16: "bfloat16", _lib.F32: "float32"}

    def __init__(self, stage2: MoeGemm2Launcher, masked: bool):
        self._stage2 = stage2
        self._masked = bool(masked)

    def __call__(self, out, x, w, scale_x, scale_w, sorted_token_ids, expert_ids, sorted_weights,
                 num_valid_ids, tokens, n, k, size_expert_ids, valid_mask=None, stream=None):
        import torch

        g = self._stage2
        if (int(n), int(k)) != (g.model_dim, g.inter_dim):
            raise ValueError(f"built for model_dim={g.model_dim}, inter_dim={g.inter_dim}; called with n={n}, k={k}")
        tokens = int(tokens)
        mask_ptr = None
        if self._masked:
            if valid_mask is None or valid_mask.numel() != tokens * g.topk or valid_mask.element_size() != 1:
                raise ValueError("this launcher was built with a valid_mask: pass a 1-byte mask [tokens, topk]")
            mask_ptr = valid_mask.data_ptr()
        elif valid_mask is not None:
            logging.getLogger(__name__).warning(
                "a valid_mask was passed to a reduce-mode launcher built without one; it is not applied")
        scratch = torch.empty((tokens * g.topk, g.model_dim), device=out.device,
                              dtype=getattr(torch, self._TORCH_DTYPES[g.out_code]))
        # zero-fill (when there is no mask) -> stage 2 per-route rows -> top-k reduce
        _lib.check(_lib.load().flyb200_moe_gemm2_reduce(
            out.data_ptr(), x.data_ptr(), w.data_ptr(), scale_x.data_ptr(), scale_w.data_ptr(),
            sorted_token_ids.data_ptr(), expert_ids.data_ptr(), sorted_weights.data_ptr(),
            num_valid_ids.data_ptr(), mask_ptr, tokens, g.model_dim, g.inter_dim, int(size_expert_ids),
            g.experts, g.topk, g.tile_m, g.doweight, g.out_code, g._cfg_ref, scratch.data_ptr(),
            scratch.numel() * scratch.element_size(), _lib.stream_handle(stream)))

    @property
    def mode(self) -> str:
        return MoeGemm2Mode.REDUCE


def compile_moe_blockscale_gemm2_ex(
    *,
    model_dim: int,
    inter_dim: int,
    experts: int,
    topk: int,
    tile_m: int,
    tile_n: int,
    tile_k: int,
    doweight_stage2: bool,
    in_dtype: str = "fp8",
    out_dtype: str = "f16",
    use_cshuffle_epilog=None,
    mode: str = MoeGemm2Mode.ATOMIC,
    valid_mask=None,
):
    """Stage 2 with explicit mode control. The reference's version forwards ``in_dtype=`` to a
    factory that does not take it and so cannot be called as shipped (:2784, :2822); this one
    accepts ``in_dtype="fp8"`` only and works."""
    if in_dtype != "fp8":
        raise ValueError(f"block-scale MoE is fp8-only, got in_dtype={in_dtype!r}")
    common = dict(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk,
                  tile_m=tile_m, tile_n=tile_n, tile_k=tile_k, doweight_stage2=doweight_stage2,
                  out_dtype=out_dtype, use_cshuffle_epilog=use_cshuffle_epilog)
    if mode == MoeGemm2Mode.REDUCE:
        stage2 = compile_moe_blockscale_gemm2(accumulate=False, **common)   # validates out_dtype too
        return _MoeGemm2ReduceWrapper(stage2, masked=valid_mask is not None)
    if mode != MoeGemm2Mode.ATOMIC:
        raise ValueError(f"mode must be 'atomic' or 'reduce', got {mode!r}")
    return compile_moe_blockscale_gemm2(accumulate=True, **common)
