"""Two-stage block-scale MoE layer assembled from the reference-shaped launchers.

The reference ships the two stage kernels and leaves the chaining to its test
(tests/kernels/test_moe_blockscale.py:293-380): routing sort -> stage 1 -> 1x128 re-quantisation ->
stage 2 (-> top-k reduce). ``BlockscaleMoE`` is that chain with persistent buffers, so a step
launches kernels only (sort, gemm1, quant, gemm2[, reduce]) and allocates nothing after warm-up.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .kernels.moe_blockscale_2stage import (
    compile_moe_blockscale_gemm1,
    compile_moe_blockscale_gemm2,
    compile_moe_reduction,
)
from .utils import moe_gather_rows, moe_sorting, quant_1x128, shuffle_weight

_DT_NAME = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}


def _as_torch_stream(stream):
    """torch.cuda.Stream | raw handle | None -> a torch stream object."""
    if stream is None:
        return torch.cuda.current_stream()
    if isinstance(stream, int):
        return torch.cuda.ExternalStream(stream)
    return stream


class BlockscaleMoE:
    """Expert weights (already repacked) plus the launchers and scratch buffers for one layer.

    w1 fp8 ``[E, 2*I, H]`` repacked (gate rows then up rows), w1_scale f32 ``[E, (2I/128)*(H/128)]``;
    w2 fp8 ``[E, H, I]`` repacked, w2_scale f32 ``[E, (H/128)*(I/128)]``.
    ``mode``: "reduce" (per-route store + fixed-order reduce, deterministic) or "atomic".
    """

    def __init__(self, w1, w1_scale, w2, w2_scale, *, topk: int, tile_m: int = 128,
                 mid_dtype=torch.float16, out_dtype=torch.bfloat16, mode: str = "reduce",
                 block_n1: Optional[int] = None, block_n2: Optional[int] = None,
                 sorted_layout: Optional[bool] = None, fused_quant: Optional[bool] = None):
        if mode not in ("reduce", "atomic"):
            raise ValueError(f"mode must be 'reduce' or 'atomic', got {mode!r}")
        self.E, two_i, self.H = w1.shape
        self.I = two_i // 2
        if tuple(w2.shape) != (self.E, self.H, self.I):
            raise ValueError(f"w2 shape {tuple(w2.shape)} does not match w1 {tuple(w1.shape)}")
        self.w1, self.w2 = w1, w2
        self.w1_scale = w1_scale.contiguous().view(-1)
        self.w2_scale = w2_scale.contiguous().view(-1)
        self.topk, self.tile_m, self.mode = int(topk), int(tile_m), mode
        self.mid_dtype, self.out_dtype = mid_dtype, out_dtype
        # Routing-order intermediates: activations are permuted once (one bandwidth-bound pass) and
        # both stages then fetch their A tiles with TMA instead of gathering rows with cp.async;
        # the stage-1 output and its re-quantisation stay in routing order as well.
        # Measured on the 256-expert layer: 4.31 -> 3.76 ms at 128-token blocks, but slightly slower
        # for decode-size batches (one more launch, nothing to hide), hence the default by block size.
        self.sorted_layout = (self.tile_m >= 64 and self.tile_m % 8 == 0) if sorted_layout is None \
            else bool(sorted_layout)
        # Optional: re-quantisation between the stages fused into the stage-1 epilogue (routing-order
        # layouts, 256-wide stage-1 tiles): the 16-bit intermediate is never written. Bit-identical,
        # but measured 3 % slower on the 256-expert layer (the heavier tile epilogue stalls the MMA
        # pipe longer than the separate quantiser kernel takes), so it is off unless asked for.
        can_fuse = self.sorted_layout and block_n1 in (None, 0, 256)
        self.fused_quant = False if fused_quant is None else bool(fused_quant)
        if self.fused_quant and not can_fuse:
            raise ValueError("fused_quant needs sorted_layout and block_n1 in (None, 256)")
        common = dict(model_dim=self.H, inter_dim=self.I, experts=self.E, topk=self.topk,
                      tile_m=self.tile_m, tile_n=256, tile_k=128)
        self.gemm1 = compile_moe_blockscale_gemm1(doweight_stage1=False, out_dtype=_DT_NAME[mid_dtype],
                                                  block_n=block_n1, a_sorted=self.sorted_layout,
                                                  out_sorted=self.sorted_layout, **common)
        self.gemm2 = compile_moe_blockscale_gemm2(doweight_stage2=True, out_dtype=_DT_NAME[out_dtype],
                                                  accumulate=(mode == "atomic"), block_n=block_n2,
                                                  a_sorted=self.sorted_layout, **common)
        self.reduce = compile_moe_reduction(topk=self.topk, model_dim=self.H,
                                            dtype_str=_DT_NAME[out_dtype]) if mode == "reduce" else None
        self._buf = {}

    @classmethod
    def from_unpacked(cls, w1_q, w1_scale, w2_q, w2_scale, **kw):
        """Build from plain row-major fp8 weights (repacks them on the GPU)."""
        return cls(shuffle_weight(w1_q), w1_scale, shuffle_weight(w2_q), w2_scale, **kw)

    def _buffers(self, T: int, dev):
        key = (T, dev)
        b = self._buf.get(key)
        if b is None:
            # rows of the stage-1 output / stage-2 input: routes, or sorted positions incl. padding
            L = (T * self.topk + self.E * self.tile_m - self.topk) if self.sorted_layout else T * self.topk
            b = {
                "rows": L,
                "x_sorted": torch.empty((L, self.H), dtype=torch.float8_e4m3fn, device=dev)
                if self.sorted_layout else None,
                "xs_sorted": torch.empty((self.H // 128, L), dtype=torch.float32, device=dev)
                if self.sorted_layout else None,
                "out1": None if self.fused_quant else torch.zeros((L, self.I), dtype=self.mid_dtype, device=dev),
                "a2_q": torch.zeros((L, self.I), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn),
                "a2_s": torch.zeros((self.I // 128, L), dtype=torch.float32, device=dev),
                "routes": torch.empty((T * self.topk, self.H), dtype=self.out_dtype, device=dev)
                if self.mode == "reduce" else None,
            }
            self._buf[key] = b
        return b

    def forward(self, x_q, x_scale_t, topk_ids, topk_weights, out=None, stream=None,
                routing=None):
        """x_q fp8 ``[T, H]``; x_scale_t f32 ``[H/128, T]``; topk_ids i32 ``[T, k]``; topk_weights f32.
        Returns ``out [T, H]``. ``routing`` may carry precomputed sort buffers
        ``(sorted_ids, sorted_weights, sorted_expert_ids, num_valid_ids)``."""
        with torch.cuda.stream(_as_torch_stream(stream)):
            return self._forward(x_q, x_scale_t, topk_ids, topk_weights, out, routing)

    def _forward(self, x_q, x_scale_t, topk_ids, topk_weights, out, routing):
        # every launch below goes to torch's current stream (stream=None)
        T = x_q.shape[0]
        dev = x_q.device
        b = self._buffers(T, dev)
        permuted = False
        if routing is None:
            # routing-order layouts: the sort kernel also permutes the activations (one launch)
            fuse = self.sorted_layout and x_q.is_contiguous() and x_scale_t.is_contiguous()
            sid, sw, seid, npp = moe_sorting(
                topk_ids, topk_weights, num_experts=self.E, block_size=self.tile_m,
                permute=(x_q, x_scale_t, b["x_sorted"], b["xs_sorted"]) if fuse else None)
            permuted = fuse
        else:
            sid, sw, seid, npp = routing
        nblk = seid.numel()
        mid_code = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}[self.mid_dtype]
        if self.sorted_layout:
            if sid.numel() != b["rows"]:
                raise ValueError("routing buffers do not match this layer's experts/tile_m/topk")
            if not permuted:
                moe_gather_rows(x_q, x_scale_t, sid, npp, topk=self.topk, out=b["x_sorted"],
                                scale_out=b["xs_sorted"])
            if self.fused_quant:
                self.gemm1.quantized(b["a2_q"], b["a2_s"], b["x_sorted"], self.w1, b["xs_sorted"],
                                     self.w1_scale, sid, seid, sw, npp, T, nblk, None)
            else:
                self.gemm1(b["out1"], b["x_sorted"], self.w1, b["xs_sorted"], self.w1_scale, sid, seid, sw,
                           npp, T, self.I, self.H, nblk, None)
                _lib.check(_lib.load().flyb200_quant_1x128_devrows(
                    b["out1"].data_ptr(), b["a2_q"].data_ptr(), b["a2_s"].data_ptr(), npp.data_ptr(),
                    b["rows"], self.I, mid_code, _lib.stream_handle(None)))
        else:
            self.gemm1(b["out1"], x_q, self.w1, x_scale_t, self.w1_scale, sid, seid, sw, npp, T, self.I,
                       self.H, nblk, None)
            _lib.check(_lib.load().flyb200_quant_1x128(
                b["out1"].data_ptr(), b["a2_q"].data_ptr(), b["a2_s"].data_ptr(), T * self.topk, self.I,
                mid_code, _lib.stream_handle(None)))
        if out is None:
            out = torch.empty((T, self.H), dtype=self.out_dtype, device=dev)
        if self.mode == "atomic":
            out.zero_()
            self.gemm2(out, b["a2_q"], self.w2, b["a2_s"], self.w2_scale, sid, seid, sw, npp, T,
                       self.H, self.I, nblk, None)
        else:
            if routing is not None:
                # A caller's routing may drop routes (expert_mask, ids outside the local experts):
                # their rows are never written by stage 2, so they must read as zero in the sum
                # (the reference wrapper zero-fills its intermediate, :2714-2715).
                b["routes"].zero_()
            self.gemm2(b["routes"], b["a2_q"], self.w2, b["a2_s"], self.w2_scale, sid, seid, sw, npp,
                       T, self.H, self.I, nblk, None)
            self.reduce(b["routes"], out, None, T, None)
        return out

    #: kernels one forward() launches (sort[+permute], gemm1, quant, gemm2, reduce | memset+gemm2)
    @property
    def launches_per_step(self) -> int:
        return 4 if (self.sorted_layout and self.fused_quant) else 5



class PertokenMoE:
    """The same chain for the per-token-scale sibling (kernels/moe_gemm_2stage.py of the reference,
    fp8): routing sort -> permute into routing order -> stage 1 -> whole-row re-quantisation -> stage
    2 -> top-k reduce, with persistent buffers. The reference test chains the stage kernels by hand
    and re-quantises with torch on the host side (tests/kernels/test_moe_gemm.py:1236-1330); here
    every step is a kernel of this library.

    w1 fp8 ``[E, 2*I, H]`` repacked (gate rows then up rows), w1_scale f32 ``[E*2*I]`` (one per output
    channel); w2 fp8 ``[E, H, I]`` repacked, w2_scale f32 ``[E*H]``. Activations come with one scale
    per token. ``tile_m`` must be a multiple of 8 (routing-order layouts are always used).
    """

    def __init__(self, w1, w1_scale, w2, w2_scale, *, topk: int, tile_m: int = 128,
                 mid_dtype=torch.float16, out_dtype=torch.bfloat16):
        from .kernels.moe_gemm_2stage import compile_moe_gemm1, compile_moe_gemm2

        self.E, two_i, self.H = w1.shape
        self.I = two_i // 2
        if tuple(w2.shape) != (self.E, self.H, self.I):
            raise ValueError(f"w2 shape {tuple(w2.shape)} does not match w1 {tuple(w1.shape)}")
        if int(tile_m) % 8:
            raise ValueError(f"tile_m must be a multiple of 8, got {tile_m}")
        self.w1, self.w2 = w1, w2
        self.w1_scale = w1_scale.contiguous().view(-1)
        self.w2_scale = w2_scale.contiguous().view(-1)
        self.topk, self.tile_m = int(topk), int(tile_m)
        self.mid_dtype, self.out_dtype = mid_dtype, out_dtype
        common = dict(model_dim=self.H, inter_dim=self.I, experts=self.E, topk=self.topk,
                      tile_m=self.tile_m, tile_n=256, tile_k=128, in_dtype="fp8")
        self.gemm1 = compile_moe_gemm1(doweight_stage1=False, out_dtype=_DT_NAME[mid_dtype], a_sorted=True,
                                       out_sorted=True, **common)
        self.gemm2 = compile_moe_gemm2(doweight_stage2=True, out_dtype=_DT_NAME[out_dtype], accumulate=False,
                                       a_sorted=True, **common)
        self.reduce = compile_moe_reduction(topk=self.topk, model_dim=self.H, dtype_str=_DT_NAME[out_dtype])
        self._buf = {}

    @classmethod
    def from_unpacked(cls, w1_q, w1_scale, w2_q, w2_scale, **kw):
        """Build from plain row-major fp8 weights (repacks them on the GPU)."""
        return cls(shuffle_weight(w1_q), w1_scale, shuffle_weight(w2_q), w2_scale, **kw)

    def _buffers(self, T: int, dev):
        key = (T, dev)
        b = self._buf.get(key)
        if b is None:
            L = T * self.topk + self.E * self.tile_m - self.topk   # sorted positions incl. padding
            b = {
                "rows": L,
                "x_sorted": torch.empty((L, self.H), dtype=torch.float8_e4m3fn, device=dev),
                "xs_sorted": torch.ones((L,), dtype=torch.float32, device=dev),
                "out1": torch.zeros((L, self.I), dtype=self.mid_dtype, device=dev),
                "a2_q": torch.zeros((L, self.I), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn),
                "a2_s": torch.ones((L,), dtype=torch.float32, device=dev),
                "routes": torch.empty((T * self.topk, self.H), dtype=self.out_dtype, device=dev),
            }
            self._buf[key] = b
        return b

    def forward(self, x_q, x_scale, topk_ids, topk_weights, out=None, stream=None, routing=None):
        """x_q fp8 ``[T, H]``; x_scale f32 ``[T]`` (or ``[T, 1]``); topk_ids i32 ``[T, k]``; topk_weights
        f32. Returns ``out [T, H]``. ``routing`` may carry precomputed sort buffers
        ``(sorted_ids, sorted_weights, sorted_expert_ids, num_valid_ids)``."""
        from .utils import quant_pertoken

        with torch.cuda.stream(_as_torch_stream(stream)):
            T = x_q.shape[0]
            dev = x_q.device
            b = self._buffers(T, dev)
            if routing is None:
                sid, sw, seid, npp = moe_sorting(topk_ids, topk_weights, num_experts=self.E,
                                                 block_size=self.tile_m)
            else:
                sid, sw, seid, npp = routing
            if sid.numel() != b["rows"]:
                raise ValueError("routing buffers do not match this layer's experts/tile_m/topk")
            nblk = seid.numel()
            moe_gather_rows(x_q, x_scale.reshape(-1), sid, npp, topk=self.topk, out=b["x_sorted"],
                            scale_out=b["xs_sorted"], per_token=True)
            self.gemm1(b["out1"], b["x_sorted"], self.w1, b["xs_sorted"], self.w1_scale, sid, seid, sw, npp,
                       T, self.I, self.H, nblk, None)
            quant_pertoken(b["out1"], npp, out=b["a2_q"], scale_out=b["a2_s"])
            if out is None:
                out = torch.empty((T, self.H), dtype=self.out_dtype, device=dev)
            if routing is not None:
                b["routes"].zero_()   # a caller's routing may drop routes: their rows must sum as zero
            self.gemm2(b["routes"], b["a2_q"], self.w2, b["a2_s"], self.w2_scale, sid, seid, sw, npp, T,
                       self.H, self.I, nblk, None)
            self.reduce(b["routes"], out, None, T, None)
            return out

    #: kernels one forward() launches: sort, permute, gemm1, quant, gemm2, reduce
    launches_per_step = 6
