"""Two-stage FP8 MoE with per-token activation scales and per-channel weight scales, behind the
reference's factory signatures (kernels/moe_gemm_2stage.py of the reference).

compile_moe_gemm1        reference :93-1264   -> launcher args of :1215-1229
compile_moe_gemm2        reference :1267-2481 -> launcher args of :2431-2446
compile_moe_reduction    reference :2484-2680 (the block-scale module's launcher: same kernel)
MoeGemm2Mode / compile_moe_gemm2_ex   reference :2683-2877

Only ``in_dtype="fp8"`` is built (the data format of the block-scale path's sibling); the other
operand formats the reference lists are accepted as names and refused with NotImplementedError.
Scales: ``scale_x`` one f32 per activation row (``[tokens]`` for stage 1, ``[tokens*topk]`` for stage
2), ``scale_w`` one f32 per output channel of every expert (``[E*2*inter]`` / ``[E*model_dim]``),
as ``tests/kernels/test_moe_gemm.py`` of the reference builds them with ``pertoken_quant``. Weights
are the ``utils.repack_weight`` image of the preshuffled tensor, as for the block-scale kernels.
"""
from __future__ import annotations

import functools
import logging

from .. import _lib
from .moe_blockscale_2stage import MoeGemm2Mode, _OUT_CODES, _cfg, compile_moe_reduction  # noqa: F401

_IN_DTYPES = ("fp8", "fp16", "bf16", "int8", "int8smooth", "int4", "int4_bf16")


def _check_common(in_dtype, group_size, tile_m, tile_k):
    if in_dtype not in _IN_DTYPES:
        raise ValueError(f"in_dtype must be one of {_IN_DTYPES!r}, got {in_dtype!r}")
    if in_dtype != "fp8":
        raise NotImplementedError(f"in_dtype={in_dtype!r} is not built here; only 'fp8' is")
    if int(group_size) > 0:
        raise NotImplementedError("group-wise weight scales belong to the int4_bf16 path, which is not built here")
    if int(tile_k) % 64 != 0:
        raise ValueError(f"tile_k_bytes must be divisible by 64, got tile_k_bytes={tile_k} "
                         f"(tile_k={tile_k}, elem_bytes=1)")
    if not 1 <= int(tile_m) <= 128:
        raise ValueError(f"tile_m must be in [1, 128] (one routing block per 128-row MMA tile), got {tile_m}")


class PertokenMoeGemm1Launcher:
    """``fn(out, x, w, scale_x, scale_w, sorted_token_ids, expert_ids, sorted_weights,
    max_token_ids, tokens, inter, k, size_expert_ids, stream)``.

    out f16/bf16 ``[tokens, topk, inter]``; x fp8 ``[tokens, model_dim]``; w fp8 repacked
    ``[E, 2*inter, model_dim]`` (gate rows then up rows per expert); scale_x f32 ``[tokens]``;
    scale_w f32 ``[E*2*inter]``."""

    def __init__(self, model_dim, inter_dim, experts, topk, tile_m, doweight, out_code,
                 a_sorted=False, out_sorted=False):
        self.model_dim, self.inter_dim = int(model_dim), int(inter_dim)
        self.experts, self.topk, self.tile_m = int(experts), int(topk), int(tile_m)
        self.doweight, self.out_code = int(bool(doweight)), out_code
        self.a_sorted = bool(a_sorted)
        self._cfg, self._cfg_ref = _cfg(0, (1 if a_sorted else 0) | (2 if out_sorted else 0))
        self._fn = _lib.load().flyb200_moe_gemm1_pertoken

    def __call__(self, out, x, w, scale_x, scale_w, sorted_token_ids, expert_ids, sorted_weights,
                 max_token_ids, tokens, inter, k, size_expert_ids, stream=None):
        if int(inter) != self.inter_dim or int(k) != self.model_dim:
            raise ValueError(f"launcher was built for inter_dim={self.inter_dim}, model_dim={self.model_dim}; "
                             f"got inter={inter}, k={k}")
        if (not self.a_sorted and scale_x.numel() < int(tokens)) or \
                scale_w.numel() != self.experts * 2 * self.inter_dim:
            raise ValueError(f"scale_x needs {int(tokens)} values and scale_w {self.experts * 2 * self.inter_dim}; "
                             f"got {scale_x.numel()} and {scale_w.numel()}")
        _lib.check(self._fn(
            out.data_ptr(), x.data_ptr(), w.data_ptr(), scale_x.data_ptr(), scale_w.data_ptr(),
            sorted_token_ids.data_ptr(), expert_ids.data_ptr(), sorted_weights.data_ptr(),
            max_token_ids.data_ptr(), int(tokens), self.inter_dim, self.model_dim,
            int(size_expert_ids), self.experts, self.topk, self.tile_m, self.doweight,
            self.out_code, self._cfg_ref, _lib.stream_handle(stream)))


class PertokenMoeGemm2Launcher:
    """``fn(out, x, w, scale_x, scale_w, sorted_token_ids, expert_ids, sorted_weights,
    num_valid_ids, tokens, n, k, size_expert_ids, stream)``.

    x fp8 ``[tokens*topk, inter]``; w fp8 repacked ``[E, model_dim, inter]``; scale_x f32
    ``[tokens*topk]``; scale_w f32 ``[E*model_dim]``. With ``accumulate=True`` out is
    ``[tokens, model_dim]``, pre-zeroed by the caller, and routes are added atomically; with
    ``accumulate=False`` out is ``[tokens*topk, model_dim]``."""

    def __init__(self, model_dim, inter_dim, experts, topk, tile_m, doweight, accumulate, out_code,
                 a_sorted=False):
        self.model_dim, self.inter_dim = int(model_dim), int(inter_dim)
        self.experts, self.topk, self.tile_m = int(experts), int(topk), int(tile_m)
        self.doweight, self.accumulate, self.out_code = int(bool(doweight)), int(bool(accumulate)), out_code
        self._cfg, self._cfg_ref = _cfg(0, 1 if a_sorted else 0)
        self._fn = _lib.load().flyb200_moe_gemm2_pertoken

    def __call__(self, out, x, w, scale_x, scale_w, sorted_token_ids, expert_ids, sorted_weights,
                 num_valid_ids, tokens, n, k, size_expert_ids, stream=None):
        if int(n) != self.model_dim or int(k) != self.inter_dim:
            raise ValueError(f"launcher was built for model_dim={self.model_dim}, inter_dim={self.inter_dim}; "
                             f"got n={n}, k={k}")
        if scale_w.numel() != self.experts * self.model_dim:
            raise ValueError(f"scale_w needs {self.experts * self.model_dim} values, got {scale_w.numel()}")
        _lib.check(self._fn(
            out.data_ptr(), x.data_ptr(), w.data_ptr(), scale_x.data_ptr(), scale_w.data_ptr(),
            sorted_token_ids.data_ptr(), expert_ids.data_ptr(), sorted_weights.data_ptr(),
            num_valid_ids.data_ptr(), int(tokens), self.model_dim, self.inter_dim,
            int(size_expert_ids), self.experts, self.topk, self.tile_m, self.doweight,
            self.accumulate, self.out_code, self._cfg_ref, _lib.stream_handle(stream)))


@functools.lru_cache(maxsize=1024)
def compile_moe_gemm1(
    *,
    model_dim: int,
    inter_dim: int,
    experts: int,
    topk: int,
    tile_m: int,
    tile_n: int,
    tile_k: int,
    doweight_stage1: bool,
    in_dtype: str = "fp8",
    group_size: int = -1,
    out_dtype: str = "f16",
    use_cshuffle_epilog=None,
    a_sorted=False,
    out_sorted=False,
):
    """Stage 1: ``out[t, slot, :] = silu(g) * u`` with ``[g, u] = (x[t] * scale_x[t]) @ (W1[e] *
    scale_w[e])^T`` (times the route weight when ``doweight_stage1``). ``tile_m`` must equal the
    block size the routing buffers were sorted with; ``tile_n`` / ``tile_k`` are validated only (the
    kernel's tile is 128 x 256 x 128); ``use_cshuffle_epilog`` is an AMD switch, ignored.

    Extensions (off by default, so the reference call is unchanged): ``a_sorted`` -- ``x`` holds one
    row per routing position (``[T*k + E*tile_m - k, model_dim]``, ``scale_x`` one value per such
    row) and is fetched by TMA instead of gathered; ``out_sorted`` -- ``out`` is written in routing
    order too (``[T*k + E*tile_m - k, inter]``)."""
    _check_common(in_dtype, group_size, tile_m, tile_k)
    if (a_sorted or out_sorted) and int(tile_m) % 8:
        raise ValueError(f"sorted layouts need tile_m to be a multiple of 8, got {tile_m}")
    if out_dtype not in ("f16", "bf16"):
        raise ValueError(f"out_dtype must be 'f16' or 'bf16', got {out_dtype!r}")
    if model_dim % 128 or inter_dim % 128:
        raise ValueError(f"model_dim ({model_dim}) and inter_dim ({inter_dim}) must be multiples of 128")
    return PertokenMoeGemm1Launcher(model_dim, inter_dim, experts, topk, tile_m, doweight_stage1,
                                    _OUT_CODES[out_dtype], a_sorted, out_sorted)


@functools.lru_cache(maxsize=1024)
def compile_moe_gemm2(
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
    group_size: int = -1,
    out_dtype: str = "f16",
    use_cshuffle_epilog=None,
    accumulate: bool = True,
    a_sorted=False,
):
    """Stage 2: ``(A2[t*topk+slot] * scale_x) @ (W2[e] * scale_w[e])^T`` (times the route weight
    when ``doweight_stage2``), atomically added into ``out[t]`` (``accumulate=True``) or stored per
    route. ``a_sorted`` (extension): ``x`` / ``scale_x`` hold one row / value per routing position,
    fetched by TMA."""
    _check_common(in_dtype, group_size, tile_m, tile_k)
    if a_sorted and int(tile_m) % 8:
        raise ValueError(f"sorted layouts need tile_m to be a multiple of 8, got {tile_m}")
    out_s = str(out_dtype).strip().lower()
    if out_s not in _OUT_CODES:
        raise ValueError(f"out_dtype must be 'f16', 'bf16', or 'f32', got {out_dtype!r}")
    out_code = _OUT_CODES[out_s]
    if (not bool(accumulate)) and out_code == _lib.F32:
        raise ValueError("compile_moe_gemm2(accumulate=False) only supports out_dtype in {'f16','bf16'}")
    if model_dim % 128 or inter_dim % 128:
        raise ValueError(f"model_dim ({model_dim}) and inter_dim ({inter_dim}) must be multiples of 128")
    return PertokenMoeGemm2Launcher(model_dim, inter_dim, experts, topk, tile_m, doweight_stage2,
                                    accumulate, out_code, a_sorted)


class _MoeGemm2ReduceWrapper:
    """Stage 2 in reduce mode (reference :2689-2780): per-route rows into a scratch tensor, then the
    fixed-order sum over the top-k slots. ``fn(out, x, w, scale_x, scale_w, sorted_token_ids,
    expert_ids, sorted_weights, num_valid_ids, tokens, n, k, size_expert_ids, valid_mask=None,
    stream=None)``. The scratch is allocated per call and, without a mask, zero-filled first when
    ``zero_intermediate`` (rows of routes that the sort dropped are then summed as zeros)."""

    _TORCH_DTYPES = {_lib.F16: "float16", _lib.BF16: "bfloat16", _lib.F32: "float32"}

    def __init__(self, stage2, masked, zero_intermediate):
        self._stage2 = stage2
        self._masked, self._zero = bool(masked), bool(zero_intermediate)

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
            logging.getLogger(__name__).warning("valid_mask provided but use_mask=False; ignoring valid_mask")
        scratch = torch.empty((tokens * g.topk, g.model_dim), device=out.device,
                              dtype=getattr(torch, self._TORCH_DTYPES[g.out_code]))
        _lib.check(_lib.load().flyb200_moe_gemm2_reduce_pertoken(
            out.data_ptr(), x.data_ptr(), w.data_ptr(), scale_x.data_ptr(), scale_w.data_ptr(),
            sorted_token_ids.data_ptr(), expert_ids.data_ptr(), sorted_weights.data_ptr(),
            num_valid_ids.data_ptr(), mask_ptr, tokens, g.model_dim, g.inter_dim, int(size_expert_ids),
            g.experts, g.topk, g.tile_m, g.doweight, g.out_code, g._cfg_ref, scratch.data_ptr(),
            scratch.numel() * scratch.element_size(), int(self._zero), _lib.stream_handle(stream)))

    @property
    def mode(self) -> str:
        return MoeGemm2Mode.REDUCE


def compile_moe_gemm2_ex(
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
    group_size: int = -1,
    out_dtype: str = "f16",
    use_cshuffle_epilog=None,
    mode: str = MoeGemm2Mode.ATOMIC,
    valid_mask=None,
    zero_intermediate: bool = True,
    a_sorted=False,
):
    """Stage 2 with explicit mode control: ``"atomic"`` (accumulate into ``[tokens, model_dim]``) or
    ``"reduce"`` (per-route store, then the top-k reduction; masked when ``valid_mask`` is given)."""
    common = dict(model_dim=model_dim, inter_dim=inter_dim, experts=experts, topk=topk,
                  tile_m=tile_m, tile_n=tile_n, tile_k=tile_k, doweight_stage2=doweight_stage2,
                  in_dtype=in_dtype, group_size=group_size, out_dtype=out_dtype,
                  use_cshuffle_epilog=use_cshuffle_epilog, a_sorted=a_sorted)
    if mode == MoeGemm2Mode.REDUCE:
        stage2 = compile_moe_gemm2(accumulate=False, **common)   # validates out_dtype too
        return _MoeGemm2ReduceWrapper(stage2, valid_mask is not None, zero_intermediate)
    if mode != MoeGemm2Mode.ATOMIC:
        raise ValueError(f"mode must be 'atomic' or 'reduce', got {mode!r}")
    return compile_moe_gemm2(accumulate=True, **common)
