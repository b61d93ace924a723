"""Multi-GPU layer on real GPUs (skipped with fewer than two): N-sharded dense GEMM and the
expert-parallel MoE (NCCL exchanges and the peer-memory exchange), each rank a child process, against the single-process CPU oracle."""
import os
import socket

import pytest
import torch

from oracle import blockscale_ref as O

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, dense, moe, ret):
    import torch.distributed as dist

    from flydsl_b200 import _lib, parallel
    from flydsl_b200.utils import shuffle_weight

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        # dense: every rank computes its column shard
        M, K = dense["a_q"].shape
        N = dense["b_q"].shape[0]
        col = parallel.ColumnParallelBlockscaleGemm(dense["b_q"].to(dev), dense["b_scale"].to(dev), N=N, K=K,
                                                    rank=rank, world=world)
        c = col.forward(dense["a_q"].to(dev), dense["a_scale"].to(dev).t().contiguous())
        # MoE: expert parallel
        E, k, H, I = moe["w1_q"].shape[0], moe["topk_ids"].shape[1], moe["x_q"].shape[1], moe["w2_q"].shape[2]
        EL, TL = E // world, moe["x_q"].shape[0] // world
        lo, hi = rank * EL, (rank + 1) * EL
        shard = parallel.LocalExpertShard(shuffle_weight(moe["w1_q"][lo:hi].to(dev)), moe["w1_scale"][lo:hi].to(dev),
                                          shuffle_weight(moe["w2_q"][lo:hi].to(dev)), moe["w2_scale"][lo:hi].to(dev),
                                          experts=E, topk=k, rank=rank, world=world, tile_m=32)
        sl = slice(rank * TL, (rank + 1) * TL)
        args = (moe["x_q"][sl].to(dev), moe["x_scale"][sl].to(dev), moe["topk_ids"][sl].to(dev),
                moe["topk_weights"][sl].to(dev))
        outs = {}
        for mode in ("fixed", "exact", "peer"):
            ep = parallel.ExpertParallelMoE(shard, experts=E, topk=k, model_dim=H, rank=rank, world=world,
                                            exchange=mode)
            outs[mode] = ep.forward(*args).float().cpu()
            if mode == "peer":
                # further steps reuse the exchange areas and the barrier flags; both combine variants
                # (partial rows pushed to the owner / pulled by the owner) give the same bits
                for variant in ("push", "pull", "push"):
                    ep.peer_combine = variant
                    again = ep.forward(*args).float().cpu()
                    assert torch.equal(again, outs[mode]), variant
                ep.peer.close()
            torch.cuda.synchronize()
            assert _lib.query_device_error() == 0
        # the three exchanges move the same rows and add partials in the same rank order
        assert torch.equal(outs["fixed"], outs["peer"])
        ret[rank] = (c.float().cpu(), outs["peer"], outs["exact"])
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_dense_shards_and_expert_parallel_moe():
    import torch.multiprocessing as mp

    world = 2
    dense = O.make_dense_case(96, 512, 512, seed=1)
    ref_c = O.run_torch_blockscale(dense["a_q"], dense["b_q"], dense["a_scale"], dense["b_scale"], dtype=torch.float32)
    moe = O.make_moe_case(T=64, H=512, I=256, E=8, topk=4, seed=3, w_std=0.05)
    ref_o, _, _, _ = O.torch_moe_two_stage_ref(moe["x_q"], moe["x_scale"], moe["w1_q"], moe["w1_scale"], moe["w2_q"],
                                               moe["w2_scale"], moe["topk_ids"], moe["topk_weights"], 256)
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), dense, moe, ret), nprocs=world, join=True)
    c = torch.cat([ret[r][0] for r in range(world)], dim=1)
    assert O.max_rel_err(c, ref_c) <= 1e-2 and O.cosine(c, ref_c) >= 0.9999
    for i in (1, 2):
        out = torch.cat([ret[r][i] for r in range(world)], dim=0)
        assert O.max_rel_err(out, ref_o) <= 1e-2 and O.cosine(out, ref_o) >= 0.9999
