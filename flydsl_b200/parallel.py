"""Multi-GPU layer for the block-scale path: one process per GPU, torch.distributed for plumbing.

The reference is single-GPU (it has no collective anywhere); what it offers for expert parallelism
are two hooks, which are used here as designed: the sorter's ``expert_mask`` (skip non-local
experts and compact their ids, tests/kernels/test_moe_gemm.py:103-104,132-141) and the masked
top-k reduce (``valid_mask``, kernels/moe_blockscale_2stage.py:2554-2563).

* Dense GEMM: column (N) sharding. Rank r owns weight rows ``[r*N/W, (r+1)*N/W)`` and the matching
  rows of the 128x128 scale grid, computes ``C[:, shard]``. No collective on the GEMM.
* MoE: expert parallel. Tokens are data-parallel (each rank routes its own tokens); experts are
  split contiguously, ``E/W`` per rank. One exchange each way:
    dispatch   every (token, destination rank) pair is sent once (a token that picked several
               experts of one rank travels once), as one packed row: fp8 activations, their
               1x128 scales, the token's expert ids and route weights;
    local      sort with expert_mask -> stage 1 -> re-quantise -> stage 2 (per-route rows) ->
               masked reduce: one partial output row per received token;
    combine    partial rows go back the same way; the source rank adds a token's partials in a
               fixed rank order (deterministic).
  Three exchange modes (``ExpertParallelMoE(exchange=...)``):
    "peer"   CUDA kernels over peer memory (:class:`PeerExchange`): rows are written straight into
             the destination's receive area and partial rows are read from the rank that computed
             them; only needed rows cross NVLink; two flag barriers per step, no NCCL call;
    "fixed"  two equal-split NCCL all-to-alls on fixed row slots (no host sync; also the gloo path);
    "exact"  NCCL all-to-alls with split sizes (one host sync for the counts).
  Receive buffers are local memory in every mode, which is what the GEMM kernels read.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


# ------------------------------------------------------------------------------------------------
# dense: N-sharded
# ------------------------------------------------------------------------------------------------
def shard_rows(n: int, rank: int, world: int, align: int = 128):
    """Row range of rank ``rank`` when ``n`` rows are split evenly; the split must respect the
    128-row scale blocks so that every shard owns whole scale rows."""
    if n % (world * align) != 0:
        raise ValueError(f"N={n} cannot be split over {world} ranks in multiples of {align}")
    per = n // world
    return rank * per, (rank + 1) * per


class ColumnParallelBlockscaleGemm:
    """This rank's column shard of ``C = dequant(A) @ dequant(B)^T``."""

    def __init__(self, b_q_full_or_shard, b_scale, *, N: int, K: int, rank: int, world: int,
                 out_dtype: str = "bf16", already_sharded: bool = False):
        from .kernels import compile_blockscale_preshuffle_gemm
        from .utils import shuffle_weight

        lo, hi = shard_rows(N, rank, world)
        self.rank, self.world, self.N, self.K = rank, world, N, K
        self.n_local = hi - lo
        if already_sharded:
            b_q, b_s = b_q_full_or_shard, b_scale
        else:
            b_q = b_q_full_or_shard[lo:hi].contiguous()
            b_s = b_scale[lo // 128: hi // 128].contiguous()
        self.b = shuffle_weight(b_q)
        self.b_scale = b_s.contiguous().view(-1)
        self.out_dtype = torch.bfloat16 if out_dtype == "bf16" else torch.float16
        self._out_name = out_dtype
        self._fns = {}
        self._compile = compile_blockscale_preshuffle_gemm

    def forward(self, a_q, a_scale_t, out=None, stream=None):
        """a_q fp8 [M, K] (replicated), a_scale_t f32 [K/128, M]; returns C[:, shard] [M, N/W]."""
        M = a_q.shape[0]
        fn = self._fns.get(M)
        if fn is None:
            fn = self._compile(M=M, N=self.n_local, K=self.K, tile_m=64, tile_n=128, tile_k=128,
                               out_dtype=self._out_name)
            self._fns[M] = fn
        if out is None:
            out = torch.empty((M, self.n_local), dtype=self.out_dtype, device=a_q.device)
        fn(out, a_q, self.b, a_scale_t, self.b_scale, M, self.n_local, stream)
        return out


# ------------------------------------------------------------------------------------------------
# MoE: expert parallel -- index logic (pure torch, device-agnostic; tested on CPU with gloo)
# ------------------------------------------------------------------------------------------------
def plan_dispatch(topk_ids: torch.Tensor, experts_per_rank: int, world: int):
    """For local tokens ``topk_ids [T, k]`` (global expert ids) decide which ranks each token visits.

    Returns
      need    bool [T, W]   token t has at least one expert on rank r
      order   i64  [S]      token index of every sent row, grouped by destination rank, ascending
                            token inside a group (S = need.sum())
      counts  i64  [W]      rows per destination rank
      pos     i64  [T, W]   position of (t, r)'s row inside ``order`` (undefined where not needed)
    """
    T = topk_ids.shape[0]
    dest = torch.div(topk_ids.long(), experts_per_rank, rounding_mode="floor")      # [T, k]
    ranks = torch.arange(world, device=topk_ids.device).view(1, 1, world)
    need = (dest.unsqueeze(-1) == ranks).any(dim=1)                                 # [T, W]
    counts = need.sum(dim=0)
    need_t = need.t().contiguous()                                                  # [W, T]
    flat = need_t.reshape(-1)
    order = torch.nonzero(flat, as_tuple=False).squeeze(1) % max(T, 1)              # rank-major
    pos_t = torch.cumsum(flat.long(), dim=0) - 1                                    # [W*T]
    pos = pos_t.view(world, T).t().contiguous()
    return need, order, counts, pos


def plan_dispatch_fixed(topk_ids: torch.Tensor, experts_per_rank: int, world: int):
    """Sync-free variant of plan_dispatch: every (source, destination) pair owns a fixed block of
    ``T`` row slots, so no count has to travel or reach the host.

    Returns
      need   bool [T, W]
      slot   i64  [T, W]   row slot of token t inside destination r's block (valid where need)
      src    i64  [W*T]    token index feeding send row r*T + s, or -1 for an unused slot
    """
    T = topk_ids.shape[0]
    dest = torch.div(topk_ids.long(), experts_per_rank, rounding_mode="floor")
    ranks = torch.arange(world, device=topk_ids.device).view(1, 1, world)
    need = (dest.unsqueeze(-1) == ranks).any(dim=1)                                 # [T, W]
    slot = torch.cumsum(need.long(), dim=0) - 1                                     # [T, W]
    # scatter without boolean indexing (that would need the count on the host): entries that are
    # not needed go to one spare slot at the end, which is cut off
    src = torch.full((world * T + 1,), -1, dtype=torch.long, device=topk_ids.device)
    flat = (torch.arange(world, device=topk_ids.device).view(1, world) * T + slot)  # [T, W]
    flat = torch.where(need, flat, torch.full_like(flat, world * T))
    tok = torch.arange(T, device=topk_ids.device).view(T, 1).expand(T, world)
    tok = torch.where(need, tok, torch.full_like(tok, -1))
    src.scatter_(0, flat.reshape(-1), tok.reshape(-1))
    return need, slot, src[: world * T]


def pack_rows_fixed(x_q_u8, x_scale, topk_ids, topk_weights, src):
    """Send buffer [W*T, row bytes]; unused slots carry expert id -1 in every top-k position so the
    receiver's sorter drops them."""
    valid = src >= 0
    idx = src.clamp(min=0)
    ids = torch.where(valid.view(-1, 1), topk_ids[idx].to(torch.int32),
                      torch.full_like(topk_ids[idx], -1, dtype=torch.int32))
    n = idx.numel()
    parts = [x_q_u8[idx],
             x_scale[idx].contiguous().view(torch.uint8).view(n, -1),
             ids.contiguous().view(torch.uint8).view(n, -1),
             topk_weights[idx].to(torch.float32).contiguous().view(torch.uint8).view(n, -1)]
    return torch.cat(parts, dim=1).contiguous()


def plan_pack_cuda(x_u8, x_scale, topk_ids, topk_weights, experts_per_rank, world):
    """plan_dispatch_fixed + pack_rows_fixed as two CUDA launches (flyb200_ep_plan_pack)."""
    from . import _lib

    T, H = x_u8.shape
    k = topk_ids.shape[1]
    dev = x_u8.device
    ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
    w = topk_weights if topk_weights.dtype == torch.float32 else topk_weights.float()
    need = torch.empty((T, world), dtype=torch.uint8, device=dev)
    slot = torch.empty((T, world), dtype=torch.int32, device=dev)
    src = torch.empty((world * T,), dtype=torch.int32, device=dev)
    rows = torch.empty((world * T, H + 4 * (H // 128) + 8 * k), dtype=torch.uint8, device=dev)
    _lib.check(_lib.load().flyb200_ep_plan_pack(
        x_u8.data_ptr(), x_scale.contiguous().data_ptr(), ids.contiguous().data_ptr(),
        w.contiguous().data_ptr(), T, H, k, world, experts_per_rank, need.data_ptr(), slot.data_ptr(),
        src.data_ptr(), rows.data_ptr(), _lib.stream_handle(None)))
    return need, slot, rows


def combine_partials_fixed(back, need, slot, out_dtype):
    """out[t] = sum over ranks r (ascending) of back[r*T + slot[t, r]] where needed; fp32."""
    T, W = need.shape
    if back.is_cuda and back.dtype in (torch.bfloat16, torch.float16) and back.shape[1] % 8 == 0:
        from . import _lib

        out = torch.empty((T, back.shape[1]), dtype=back.dtype, device=back.device)
        _lib.check(_lib.load().flyb200_ep_combine(
            back.data_ptr(), need.to(torch.uint8).contiguous().data_ptr(),
            slot.to(torch.int32).contiguous().data_ptr(), out.data_ptr(), T, W, back.shape[1],
            _lib.BF16 if back.dtype == torch.bfloat16 else _lib.F16, _lib.stream_handle(None)))
        return out.to(out_dtype)
    need, slot = need.bool(), slot.long()
    acc = torch.zeros((T, back.shape[1]), dtype=torch.float32, device=back.device)
    base = torch.arange(W, device=back.device).view(1, W) * T
    idx = (base + slot.clamp(min=0))
    for r in range(W):  # fixed order => deterministic
        acc += back[idx[:, r]].float() * need[:, r].view(T, 1).float()
    return acc.to(out_dtype)


def pack_rows(x_q_u8, x_scale, topk_ids, topk_weights, order):
    """One byte row per sent token: [H fp8 | H/128 f32 scales | k i32 ids | k f32 weights]."""
    parts = [x_q_u8[order],
             x_scale[order].contiguous().view(torch.uint8).view(order.numel(), -1),
             topk_ids[order].to(torch.int32).contiguous().view(torch.uint8).view(order.numel(), -1),
             topk_weights[order].to(torch.float32).contiguous().view(torch.uint8).view(order.numel(), -1)]
    return torch.cat(parts, dim=1).contiguous()


def unpack_rows(buf, H: int, k: int):
    """Inverse of pack_rows on the receiving side."""
    R = buf.shape[0]
    nscale = H // 128
    o0, o1, o2, o3 = H, H + 4 * nscale, H + 4 * nscale + 4 * k, H + 4 * nscale + 8 * k
    x_q = buf[:, :o0].contiguous()
    x_s = buf[:, o0:o1].contiguous().view(torch.float32).view(R, nscale)
    ids = buf[:, o1:o2].contiguous().view(torch.int32).view(R, k)
    w = buf[:, o2:o3].contiguous().view(torch.float32).view(R, k)
    return x_q, x_s, ids, w


def combine_partials(recv, need, pos, out_dtype):
    """out[t] = sum over ranks r (ascending) of the partial row (t, r); fp32 accumulate."""
    T, W = need.shape
    H = recv.shape[1]
    padded = torch.cat([recv, torch.zeros((1, H), dtype=recv.dtype, device=recv.device)], dim=0)
    idx = torch.where(need, pos, torch.full_like(pos, recv.shape[0]))
    acc = torch.zeros((T, H), dtype=torch.float32, device=recv.device)
    for r in range(W):  # fixed order => deterministic
        acc += padded[idx[:, r]].float()
    return acc.to(out_dtype)


def exchange_counts(counts: torch.Tensor, group=None) -> torch.Tensor:
    """counts[r] rows go to rank r; returns how many rows each rank sends to me."""
    recv = torch.empty_like(counts)
    dist.all_to_all_single(recv, counts, group=group)
    return recv


def all_to_all_rows(rows: torch.Tensor, send_counts, recv_counts, group=None) -> torch.Tensor:
    """Variable-count row exchange. ``rows`` is grouped by destination rank."""
    out = rows.new_empty((int(sum(recv_counts)),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows, output_split_sizes=list(recv_counts),
                           input_split_sizes=list(send_counts), group=group)
    return out


class ExpertParallelMoE:
    """Expert-parallel wrapper around a local two-stage MoE.

    ``local_fn(x_q_u8 [R,H], x_scale [R,H/128], topk_ids [R,k] (global ids), topk_weights [R,k])``
    must return the partial output ``[R, H]`` that sums only the routes whose expert lives on this
    rank. On GPUs that is :class:`LocalExpertShard` below; tests plug in a CPU function.
    """

    def __init__(self, local_fn: Callable, *, experts: int, topk: int, model_dim: int, rank: int,
                 world: int, group=None, out_dtype=torch.bfloat16, exchange: str = "fixed"):
        if experts % world:
            raise ValueError(f"{experts} experts cannot be split over {world} ranks")
        self.local_fn, self.E, self.k, self.H = local_fn, experts, topk, model_dim
        self.rank, self.world, self.group, self.out_dtype = rank, world, group, out_dtype
        self.experts_per_rank = experts // world
        self.last_stats = {}
        if exchange not in ("fixed", "exact", "peer"):
            raise ValueError("exchange must be 'peer' (CUDA kernels over peer memory), 'fixed' (T row "
                             "slots per rank pair, no host sync) or 'exact' (only the needed rows "
                             "travel; one host sync for the counts)")
        self.exchange = exchange
        self.trace = False
        self.peer = None     # PeerExchange, created on the first "peer" step (needs T)
        self.peer_combine = "push"   # "push": owners receive partial rows; "pull": they fetch them

    def forward(self, x_q, x_scale, topk_ids, topk_weights):
        """x_q fp8/uint8 [T, H]; x_scale f32 [T, H/128] (token-major); ids [T, k]; weights [T, k]."""
        x_u8 = x_q.view(torch.uint8)
        if self.exchange == "fixed":
            return self._forward_fixed(x_u8, x_scale, topk_ids, topk_weights)
        if self.exchange == "peer":
            return self._forward_peer(x_u8, x_scale, topk_ids, topk_weights)
        need, order, counts, pos = plan_dispatch(topk_ids, self.experts_per_rank, self.world)
        recv_counts = exchange_counts(counts, self.group)
        send_l, recv_l = counts.tolist(), recv_counts.tolist()       # one host sync per step
        rows = pack_rows(x_u8, x_scale, topk_ids, topk_weights, order)
        got = all_to_all_rows(rows, send_l, recv_l, self.group)
        rx_q, rx_s, rids, rw = unpack_rows(got, self.H, self.k)
        partial = self.local_fn(rx_q, rx_s, rids, rw)                # [R, H]
        back = all_to_all_rows(partial.contiguous(), recv_l, send_l, self.group)
        self.last_stats = {"sent_rows": int(sum(send_l)), "recv_rows": int(sum(recv_l)),
                           "dispatch_bytes": int(sum(send_l)) * rows.shape[1],
                           "combine_bytes": int(sum(recv_l)) * self.H * partial.element_size()}
        return combine_partials(back, need, pos, self.out_dtype)


def _forward_fixed(self, x_u8, x_scale, topk_ids, topk_weights):
    """Equal-split all-to-alls: nothing depends on a host-visible count, so the whole step is
    enqueued without synchronising (the price: T row slots per destination instead of the ~T*(1 -
    ((W-1)/W)^k) that are needed)."""
    T = x_u8.shape[0]
    marks = []

    def mark(name):  # optional phase timing (self.trace = True): CUDA events, read after the step
        if self.trace and x_u8.is_cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            marks.append((name, e))

    mark("start")
    if x_u8.is_cuda and self.k % 2 == 0:
        need, slot, rows = plan_pack_cuda(x_u8, x_scale, topk_ids, topk_weights, self.experts_per_rank,
                                          self.world)
    else:
        need, slot, src = plan_dispatch_fixed(topk_ids, self.experts_per_rank, self.world)
        rows = pack_rows_fixed(x_u8, x_scale, topk_ids, topk_weights, src)      # [W*T, bytes]
    mark("plan+pack")
    got = torch.empty_like(rows)
    dist.all_to_all_single(got, rows, group=self.group)
    mark("dispatch")
    if got.is_cuda and self.k % 2 == 0 and hasattr(self.local_fn, "forward_packed"):
        partial = self.local_fn.forward_packed(got)                             # rows read in place
    else:
        rx_q, rx_s, rids, rw = unpack_rows(got, self.H, self.k)
        partial = self.local_fn(rx_q, rx_s, rids, rw).contiguous()              # [W*T, H]
    mark("local experts")
    back = torch.empty_like(partial)
    dist.all_to_all_single(back, partial, group=self.group)
    mark("combine a2a")
    self.last_stats = {"sent_rows": self.world * T, "recv_rows": self.world * T,
                       "dispatch_bytes": rows.numel(), "combine_bytes": partial.numel() * partial.element_size()}
    out = combine_partials_fixed(back, need, slot, self.out_dtype)
    mark("sum partials")
    if marks:
        torch.cuda.synchronize()
        self.last_stats["phase_ms"] = {marks[i + 1][0]: round(marks[i][1].elapsed_time(marks[i + 1][1]), 4)
                                       for i in range(len(marks) - 1)}
    return out


ExpertParallelMoE._forward_fixed = _forward_fixed


class _RawCuda:
    """Device memory owned by the C library, exposed to torch without a copy."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1",
                                         "data": (int(ptr), False), "version": 2}


class PeerExchange:
    """The exchange buffers of one rank and its mappings of the peers' buffers.

    Layout of every rank's buffer: receive area ``[W*T, row bytes]`` | partial area ``[W*T, H]``
    (16-bit) | ``W`` barrier flags. Created collectively (every rank of ``group`` must call it with
    the same sizes): one all-gather of the 64-byte IPC handles."""

    def __init__(self, *, tokens: int, model_dim: int, topk: int, rank: int, world: int, device,
                 group=None, limit_ms: int = 2000):
        import ctypes

        from . import _lib

        self.T, self.H, self.k, self.rank, self.world = tokens, model_dim, topk, rank, world
        self.group, self.limit_ms, self.device = group, int(limit_ms), torch.device(device)
        self.row_bytes = model_dim + 4 * (model_dim // 128) + 8 * topk
        al = lambda n: (n + 255) // 256 * 256
        self.recv_off = 0
        self.part_off = al(world * tokens * self.row_bytes)
        self.flag_off = self.part_off + al(world * tokens * model_dim * 2)
        self.nbytes = self.flag_off + 256
        self._lib = _lib.load()
        own = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            _lib.check(self._lib.flyb200_ep_buffer_create(self.nbytes, ctypes.byref(own), handle))
            self.own = int(own.value)
            mine = torch.tensor(list(bytes(handle)), dtype=torch.uint8, device=self.device)
            every = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(every, mine, group=group)
            self._opened = []
            ptrs = []
            for r in range(world):
                if r == rank:
                    ptrs.append(self.own)
                    continue
                raw = (ctypes.c_ubyte * 64)(*every[r].cpu().tolist())
                q = ctypes.c_void_p()
                _lib.check(self._lib.flyb200_ep_buffer_open(raw, ctypes.byref(q)))
                self._opened.append(int(q.value))
                ptrs.append(int(q.value))
            self.peers = (ctypes.c_void_p * world)(*ptrs)
            whole = torch.as_tensor(_RawCuda(self.own, self.nbytes), device=self.device)
            self.recv = whole[: world * tokens * self.row_bytes].view(world * tokens, self.row_bytes)
            self.partial_u8 = whole[self.part_off: self.part_off + world * tokens * model_dim * 2]
            self.epoch = 0
            dist.barrier(group=group)   # every buffer exists and is zeroed before the first push

    def partial(self, dtype):
        return self.partial_u8.view(dtype).view(self.world * self.T, self.H)

    def barrier(self):
        from . import _lib

        self.epoch += 1
        _lib.check(self._lib.flyb200_ep_barrier(self.peers, self.world, self.rank, self.flag_off,
                                                self.epoch, self.limit_ms, _lib.stream_handle(None)))

    def push(self, x_u8, x_scale, topk_ids, topk_weights, experts_per_rank):
        """Plan + write this rank's token rows into the destinations' receive areas."""
        from . import _lib

        T, W, dev = self.T, self.world, x_u8.device
        ids = (topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)).contiguous()
        w = (topk_weights if topk_weights.dtype == torch.float32 else topk_weights.float()).contiguous()
        need = torch.empty((T, W), dtype=torch.uint8, device=dev)
        slot = torch.empty((T, W), dtype=torch.int32, device=dev)
        src = torch.empty((W * T,), dtype=torch.int32, device=dev)
        _lib.check(self._lib.flyb200_ep_push(
            x_u8.data_ptr(), x_scale.contiguous().data_ptr(), ids.data_ptr(), w.data_ptr(), T, self.H,
            self.k, W, self.rank, experts_per_rank, self.peers, self.recv_off, need.data_ptr(),
            slot.data_ptr(), src.data_ptr(), _lib.stream_handle(None)))
        return need, slot

    def reduce_push(self, routes, valid, dtype):
        """Masked top-k reduce of this rank's route rows, written into the owners' back areas (the
        partial area of every buffer doubles as its back area)."""
        from . import _lib

        _lib.check(self._lib.flyb200_ep_reduce_push(
            routes.data_ptr(), valid.data_ptr(), self.peers, self.part_off, self.T, self.world, self.k,
            self.H, self.rank, _lib.BF16 if dtype == torch.bfloat16 else _lib.F16, _lib.stream_handle(None)))

    def combine_local(self, need, slot, dtype):
        """Sum of this rank's tokens over the rows that the owners pushed into the own back area."""
        from . import _lib

        out = torch.empty((self.T, self.H), dtype=dtype, device=need.device)
        _lib.check(self._lib.flyb200_ep_combine(
            self.own + self.part_off, need.data_ptr(), slot.data_ptr(), out.data_ptr(), self.T, self.world,
            self.H, _lib.BF16 if dtype == torch.bfloat16 else _lib.F16, _lib.stream_handle(None)))
        return out

    def pull_combine(self, need, slot, dtype):
        from . import _lib

        out = torch.empty((self.T, self.H), dtype=dtype, device=need.device)
        _lib.check(self._lib.flyb200_ep_pull_combine(
            self.peers, self.part_off, need.data_ptr(), slot.data_ptr(), out.data_ptr(), self.T,
            self.world, self.H, self.rank, _lib.BF16 if dtype == torch.bfloat16 else _lib.F16,
            _lib.stream_handle(None)))
        return out

    def close(self):
        """Collective: unmap the peers' buffers, then free the own one."""
        from . import _lib

        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for q in self._opened:
                _lib.check(self._lib.flyb200_ep_buffer_close(q))
            self._opened = []
            dist.barrier(group=self.group)
            if self.own:
                self.recv = self.partial_u8 = None
                _lib.check(self._lib.flyb200_ep_buffer_destroy(self.own))
                self.own = 0


def _forward_peer(self, x_u8, x_scale, topk_ids, topk_weights):
    """Exchange by CUDA kernels over peer memory; ``local_fn`` must offer ``forward_packed``
    (:class:`LocalExpertShard` does). The whole step is enqueued without a host sync."""
    if not x_u8.is_cuda:
        raise ValueError("exchange='peer' needs CUDA tensors (one GPU per rank)")
    if self.out_dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("exchange='peer' combines 16-bit partial rows")
    if self.k % 2:
        raise ValueError("exchange='peer' needs an even top-k (packed rows must stay 16-byte aligned)")
    T = x_u8.shape[0]
    if self.peer is None or self.peer.T != T:
        if self.peer is not None:
            self.peer.close()
        self.peer = PeerExchange(tokens=T, model_dim=self.H, topk=self.k, rank=self.rank,
                                 world=self.world, device=x_u8.device, group=self.group)
    px = self.peer
    marks = []

    def mark(name):
        if self.trace:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            marks.append((name, e))

    mark("start")
    need, slot = px.push(x_u8, x_scale, topk_ids, topk_weights, self.experts_per_rank)
    mark("plan+push")
    px.barrier()                                   # every rank's rows have landed here
    mark("barrier")
    if self.peer_combine == "push":
        # the top-k reduce stores each partial row straight into the owner's back area
        self.local_fn.forward_packed(
            px.recv, reducer=lambda routes, valid: px.reduce_push(routes, valid, self.out_dtype))
        mark("local experts+push")
        px.barrier()                               # every rank's partial rows have landed here
        mark("barrier 2")
        out = px.combine_local(need, slot, self.out_dtype)
        mark("sum")
    else:
        self.local_fn.forward_packed(px.recv, out=px.partial(self.out_dtype))
        mark("local experts")
        px.barrier()                               # every rank's partial rows are complete
        mark("barrier 2")
        out = px.pull_combine(need, slot, self.out_dtype)
        mark("pull+sum")
    self.last_stats = {"sent_rows": None, "recv_rows": self.world * T, "exchange": "peer"}
    if marks:
        torch.cuda.synchronize()
        self.last_stats["phase_ms"] = {marks[i + 1][0]: round(marks[i][1].elapsed_time(marks[i + 1][1]), 4)
                                       for i in range(len(marks) - 1)}
    return out


ExpertParallelMoE._forward_peer = _forward_peer


class LocalExpertShard:
    """The experts of one rank on its GPU: routing sort over the local experts (routes renumbered to
    local ids, foreign ones dropped), activations
    permuted into routing order, the two TMA-fed GEMM stages, and the masked top-k reduce that yields
    one partial row per received token. Rows whose expert ids are all foreign (or -1) give zeros."""

    def __init__(self, w1, w1_scale, w2, w2_scale, *, experts: int, topk: int, rank: int, world: int,
                 tile_m: int = 128, mid_dtype=torch.float16, out_dtype=torch.bfloat16, fused_quant: bool = False):
        from .kernels import (compile_moe_blockscale_gemm1, compile_moe_blockscale_gemm2,
                              compile_moe_reduction)

        if tile_m % 8:
            raise ValueError("LocalExpertShard uses the routing-order layout: tile_m must be a multiple of 8")
        self.E, self.k, self.rank, self.world = experts, topk, rank, world
        self.EL = experts // world
        if self.EL < topk:
            raise ValueError(f"LocalExpertShard needs experts per rank ({self.EL}) >= topk ({topk}): the routing "
                             "buffers are sized for the local experts")
        self.w1, self.w2 = w1, w2                       # repacked local experts [EL, 2I, H], [EL, H, I]
        self.w1_scale, self.w2_scale = w1_scale.contiguous().view(-1), w2_scale.contiguous().view(-1)
        self.H, self.I = w1.shape[2], w1.shape[1] // 2
        self.tile_m, self.mid_dtype, self.out_dtype = tile_m, mid_dtype, out_dtype
        names = {torch.float16: "f16", torch.bfloat16: "bf16"}
        # routes are renumbered to local expert ids (foreign routes become -1, which the sorter
        # skips like any id outside [0, E)), so sort, routing buffers and stage kernels are sized for
        # the EL local experts: sorted length = R*k + EL*tile_m - k
        common = dict(model_dim=self.H, inter_dim=self.I, experts=self.EL, topk=topk, tile_m=tile_m,
                      tile_n=256, tile_k=128)
        self.gemm1 = compile_moe_blockscale_gemm1(doweight_stage1=False, out_dtype=names[mid_dtype],
                                                  a_sorted=True, out_sorted=True, **common)
        self.gemm2 = compile_moe_blockscale_gemm2(doweight_stage2=True, out_dtype=names[out_dtype],
                                                  accumulate=False, a_sorted=True, **common)
        self.reduce = compile_moe_reduction(topk=topk, model_dim=self.H, dtype_str=names[out_dtype],
                                            use_mask=True)
        self._mid_code = {torch.float16: 1, torch.bfloat16: 0}[mid_dtype]
        self.fused_quant = bool(fused_quant)   # re-quantisation inside the stage-1 epilogue
        self._buf = {}

    def _buffers(self, R, dev):
        b = self._buf.get(R)
        if b is None:
            L = R * self.k + self.EL * self.tile_m - self.k
            b = {"L": L,
                 "x_sorted": torch.empty((L, self.H), dtype=torch.float8_e4m3fn, device=dev),
                 "xs_sorted": torch.empty((self.H // 128, L), dtype=torch.float32, device=dev),
                 "out1": None if self.fused_quant else torch.zeros((L, self.I), dtype=self.mid_dtype, device=dev),
                 "a2_q": torch.zeros((L, self.I), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn),
                 "a2_s": torch.zeros((self.I // 128, L), dtype=torch.float32, device=dev),
                 "routes": torch.empty((R * self.k, self.H), dtype=self.out_dtype, device=dev),
                 "ids": torch.empty((R, self.k), dtype=torch.int32, device=dev),
                 "w": torch.empty((R, self.k), dtype=torch.float32, device=dev),
                 "valid": torch.empty((R, self.k), dtype=torch.uint8, device=dev),
                 "out": torch.empty((R, self.H), dtype=self.out_dtype, device=dev)}
            self._buf[R] = b
        return b

    def __call__(self, x_q_u8, x_scale, topk_ids, topk_weights):
        from .utils import moe_gather_rows

        R = x_q_u8.shape[0]
        if R == 0:
            return torch.zeros((0, self.H), dtype=self.out_dtype, device=x_q_u8.device)
        xs_t = x_scale.t().contiguous()

        def gather(b, sid, npp):
            moe_gather_rows(x_q_u8.view(torch.float8_e4m3fn), xs_t, sid, npp, topk=self.k,
                            out=b["x_sorted"], scale_out=b["xs_sorted"])

        lo = self.rank * self.EL
        local = topk_ids.to(torch.int32) - lo
        local = torch.where((local >= 0) & (local < self.EL), local, torch.full_like(local, -1))
        valid = (local >= 0).to(torch.uint8)
        return self._run(R, x_q_u8.device, local, topk_weights, gather, None, valid)

    def forward_packed(self, rows, out=None, reducer=None):
        """Same as calling the shard on ``unpack_rows(rows)``, but the packed rows
        ``[R, H + 4*H/128 + 8*k]`` (uint8) are read in place: only ids and weights are sliced out,
        activations and scales go straight into routing order. ``reducer(routes [R*k, H], valid
        [R, k])`` replaces the final masked top-k reduce (nothing is returned then)."""
        from . import _lib

        R = rows.shape[0]
        H, k = self.H, self.k
        o1 = H + 4 * (H // 128)
        if rows.shape[1] != o1 + 8 * k or not rows.is_contiguous():
            raise ValueError("forward_packed: rows must be contiguous [R, H + 4*H/128 + 8*k] bytes")
        b = self._buffers(R, rows.device)
        ids, w, valid = b["ids"], b["w"], b["valid"]
        _lib.check(_lib.load().flyb200_ep_unpack_meta(
            rows.data_ptr(), R, H, k, self.EL, self.rank, 1, ids.data_ptr(), w.data_ptr(), valid.data_ptr(),
            _lib.stream_handle(None)))

        def gather(b, sid, npp):
            _lib.check(_lib.load().flyb200_ep_gather_packed(
                rows.data_ptr(), sid.data_ptr(), npp.data_ptr(), b["x_sorted"].data_ptr(),
                b["xs_sorted"].data_ptr(), R, H, k, b["L"], _lib.stream_handle(None)))

        return self._run(R, rows.device, ids, w, gather, out, valid, reducer)

    def _run(self, R, dev, topk_ids, topk_weights, gather, out, valid=None, reducer=None):
        from . import _lib
        from .utils import moe_sorting

        b = self._buffers(R, dev)
        # topk_ids are LOCAL expert ids here (-1 = not this rank's route)
        sid, sw, seid, npp = moe_sorting(topk_ids, topk_weights, num_experts=self.EL,
                                         block_size=self.tile_m)
        nblk = seid.numel()
        gather(b, sid, npp)
        if self.fused_quant:
            self.gemm1.quantized(b["a2_q"], b["a2_s"], b["x_sorted"], self.w1, b["xs_sorted"], self.w1_scale,
                                 sid, seid, sw, npp, R, nblk, None)
        else:
            self.gemm1(b["out1"], b["x_sorted"], self.w1, b["xs_sorted"], self.w1_scale, sid, seid, sw, npp,
                       R, self.I, self.H, nblk, None)
            _lib.check(_lib.load().flyb200_quant_1x128_devrows(
                b["out1"].data_ptr(), b["a2_q"].data_ptr(), b["a2_s"].data_ptr(), npp.data_ptr(), b["L"],
                self.I, self._mid_code, _lib.stream_handle(None)))
        self.gemm2(b["routes"], b["a2_q"], self.w2, b["a2_s"], self.w2_scale, sid, seid, sw, npp, R,
                   self.H, self.I, nblk, None)
        # a route counts here iff its expert lives on this rank
        if valid is None:
            valid = (topk_ids >= 0).to(torch.uint8)
        if reducer is not None:            # e.g. PeerExchange.reduce_push: rows leave this GPU
            reducer(b["routes"], valid)
            return None
        if out is None:
            out = b["out"]
        self.reduce(b["routes"], out, valid, R, None)
        return out
