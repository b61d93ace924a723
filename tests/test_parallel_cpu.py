"""Host logic of the multi-GPU layer on CPU: gloo, world_size 2, the oracle as the expert compute."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flydsl_b200 import parallel as P
from oracle import blockscale_ref as O


def test_shard_rows():
    assert P.shard_rows(7168, 3, 8) == (2688, 3584)
    assert P.shard_rows(24576, 0, 4) == (0, 6144)
    with pytest.raises(ValueError):
        P.shard_rows(2112, 0, 8)


def test_plan_dispatch_and_pack_roundtrip():
    g = torch.Generator().manual_seed(0)
    T, k, E, W = 37, 4, 16, 4
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    need, order, counts, pos = P.plan_dispatch(ids, E // W, W)
    assert need.shape == (T, W) and int(counts.sum()) == order.numel()
    for t in range(T):
        assert set(torch.nonzero(need[t]).flatten().tolist()) == set((ids[t] // (E // W)).tolist())
    # rows grouped by destination rank, token-ascending inside a group, pos points at them
    off = 0
    for r in range(W):
        grp = order[off: off + int(counts[r])]
        assert torch.equal(grp, torch.nonzero(need[:, r]).flatten())
        for j, t in enumerate(grp.tolist()):
            assert int(pos[t, r]) == off + j
        off += int(counts[r])
    H = 256
    x = torch.randint(0, 255, (T, H), generator=g, dtype=torch.uint8)
    xs = torch.rand(T, H // 128, generator=g)
    w = torch.rand(T, k, generator=g)
    rows = P.pack_rows(x, xs, ids, w, order)
    assert rows.shape == (order.numel(), H + 4 * (H // 128) + 8 * k)
    a, b, c, d = P.unpack_rows(rows, H, k)
    assert torch.equal(a, x[order]) and torch.equal(b, xs[order]) and torch.equal(c, ids[order]) and torch.equal(d, w[order])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _ep_worker(rank, world, port, case, T_local, exchange, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    try:
        E, k, H, I = case["w1_q"].shape[0], case["topk_ids"].shape[1], case["x_q"].shape[1], case["w2_q"].shape[2]
        EL = E // world
        lo, hi = rank * EL, (rank + 1) * EL

        def local_fn(xq_u8, xs, ids, w):
            # partial output over this rank's experts only, computed by the CPU oracle
            R = xq_u8.shape[0]
            out = torch.zeros(R, H)
            if R == 0:
                return out.to(torch.bfloat16)
            xq = xq_u8.view(torch.float8_e4m3fn)
            local = (ids >= lo) & (ids < hi)
            ids_l = torch.where(local, ids - lo, torch.full_like(ids, -1))
            out1 = O.torch_stage1_blockscale_ref(xq, case["w1_q"][lo:hi], ids_l, xs, case["w1_scale"][lo:hi], I)
            a2q, a2s = O.quant_1x128(out1.to(torch.float16).float().reshape(-1, I))
            per_route = O.torch_stage2_blockscale_ref(a2q, case["w2_q"][lo:hi], ids_l, w, a2s, case["w2_scale"][lo:hi],
                                                      R, H, I, k, per_route=True)
            out = (per_route * (w * local).reshape(R, k, 1)).sum(1)
            return out.to(torch.bfloat16)

        ep = P.ExpertParallelMoE(local_fn, experts=E, topk=k, model_dim=H, rank=rank, world=world, exchange=exchange)
        sl = slice(rank * T_local, (rank + 1) * T_local)
        out = ep.forward(case["x_q"][sl].view(torch.uint8), case["x_scale"][sl], case["topk_ids"][sl],
                         case["topk_weights"][sl])
        ret[rank] = (out.float(), dict(ep.last_stats))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["fixed", "exact"])
def test_expert_parallel_matches_single_process_oracle(exchange):
    world, T_local = 2, 12
    case = O.make_moe_case(T=world * T_local, H=256, I=128, E=8, topk=3, seed=7, w_std=0.05)
    ref, _, _, _ = O.torch_moe_two_stage_ref(case["x_q"], case["x_scale"], case["w1_q"], case["w1_scale"],
                                             case["w2_q"], case["w2_scale"], case["topk_ids"], case["topk_weights"], 128)
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    mp.spawn(_ep_worker, args=(world, port, case, T_local, exchange, ret), nprocs=world, join=True)
    out = torch.cat([ret[r][0] for r in range(world)], dim=0)
    assert O.max_rel_err(out, ref) <= 1e-2 and O.cosine(out, ref) >= 0.9999
    need, _, _, _ = P.plan_dispatch(case["topk_ids"], 4, world)
    if exchange == "exact":   # every (token, rank) pair travels exactly once
        assert sum(ret[r][1]["sent_rows"] for r in range(world)) == int(need.sum())
        assert sum(ret[r][1]["recv_rows"] for r in range(world)) == int(need.sum())
    else:                     # fixed blocks: T_local slots per rank pair
        assert all(ret[r][1]["sent_rows"] == world * T_local for r in range(world))


def test_plan_dispatch_fixed_slots():
    g = torch.Generator().manual_seed(1)
    T, k, E, W = 23, 3, 12, 4
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    need, slot, src = P.plan_dispatch_fixed(ids, E // W, W)
    need2, _, counts, _ = P.plan_dispatch(ids, E // W, W)
    assert torch.equal(need, need2) and src.numel() == W * T
    for r in range(W):
        block = src[r * T:(r + 1) * T]
        n = int(counts[r])
        assert torch.equal(block[:n], torch.nonzero(need[:, r]).flatten()) and (block[n:] == -1).all()
        for t in torch.nonzero(need[:, r]).flatten().tolist():
            assert int(block[int(slot[t, r])]) == t
