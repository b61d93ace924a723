"""MoE path on the GPU: routing sort (bit-exact), 1x128 quantiser (bit-exact), top-k reduce, the two
stage GEMMs and the chained layer, against golden vectors and the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import blockscale_ref as O
from tests.helpers import MAX_REL, MAX_REL_ATOMIC16, assert_close_to_oracle, fp8_from_u8, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _sort_gpu(ids, w, E, bs, mask=None, nlt=None):
    from flydsl_b200.utils import moe_sorting

    out = moe_sorting(torch.as_tensor(ids).to(DEV), torch.as_tensor(w).to(DEV), num_experts=E, block_size=bs,
                      expert_mask=None if mask is None else torch.as_tensor(mask).to(DEV), num_local_tokens=nlt)
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in out]


@pytest.mark.parametrize("tag", ["s0", "s1", "s2", "s3", "s4"])
def test_sort_vs_golden_bit_exact(tag):
    g = load_golden("sort.npz")
    T, k, E, bs, nlt = (int(v) for v in g[f"{tag}_cfg"])
    mask = g[f"{tag}_mask"] if g[f"{tag}_mask"].size else None
    sid, sw, seid, npp = _sort_gpu(g[f"{tag}_ids"], g[f"{tag}_w"], E, bs, mask, None if nlt < 0 else nlt)
    assert np.array_equal(sid, g[f"{tag}_sorted_ids"])
    assert np.array_equal(sw, g[f"{tag}_sorted_w"])
    assert np.array_equal(seid, g[f"{tag}_expert_ids"])
    assert np.array_equal(npp, g[f"{tag}_post_pad"])


@pytest.mark.parametrize("T,k,E,bs,hot", [(4096, 8, 256, 128, 0), (256, 8, 256, 16, 16), (32, 8, 256, 16, 16),
                                          (1, 8, 256, 128, 0), (1000, 6, 160, 64, 0)])
def test_sort_vs_oracle_full_size(T, k, E, bs, hot):
    g = torch.Generator().manual_seed(T + k)
    logits = torch.randn(T, E, generator=g)
    if hot:
        logits[:, :hot] += 2.0
    ids, w = O.route_topk(logits, k)
    got = _sort_gpu(ids, w, E, bs)
    want = O.moe_sorting_ref(ids.numpy(), w.numpy(), E, bs)
    for a, b in zip(got, want):
        assert np.array_equal(a, b)
    # properties that hold at any size: every route appears exactly once, blocks are single-expert
    n_valid = int(got[3][0])
    sid = got[0][:n_valid]
    real = sid[sid != ((k << 24) | T)]
    assert real.size == T * k and np.unique(real).size == T * k
    assert n_valid % bs == 0 and (got[2][: n_valid // bs] >= 0).all()


def test_quant_1x128_bit_exact():
    from flydsl_b200.utils import quant_1x128

    g = load_golden("quant.npz")
    q, st = quant_1x128(torch.from_numpy(g["x"]).to(DEV))
    assert np.array_equal(q.cpu().view(torch.uint8).numpy(), g["q"])
    assert np.array_equal(st.cpu().t().numpy(), g["scale"])
    gen = torch.Generator().manual_seed(9)
    for dt in (torch.float16, torch.bfloat16, torch.float32):
        x = (torch.randn(77, 384, generator=gen) * 5).to(dt)
        x[3, :128] = 0
        q, st = quant_1x128(x.to(DEV))
        wq, ws = O.quant_1x128(x.float())
        assert torch.equal(q.cpu().view(torch.uint8), wq.view(torch.uint8)), dt
        assert torch.equal(st.cpu().t().contiguous(), ws), dt


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("T,k,H", [(1, 8, 7168), (129, 6, 5120), (33, 8, 256)])
def test_reduce(dt, T, k, H):
    from flydsl_b200.kernels import compile_moe_reduction

    gen = torch.Generator().manual_seed(T)
    x = torch.randn(T, k, H, generator=gen).to(dt).to(DEV)
    name = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32"}[dt]
    y = torch.empty(T, H, dtype=dt, device=DEV)
    compile_moe_reduction(topk=k, model_dim=H, dtype_str=name)(x, y, None, T, None)
    torch.testing.assert_close(y.float(), x.float().sum(1).to(dt).float(), rtol=1e-2, atol=1e-2)
    mask = (torch.rand(T, k, generator=gen) > 0.4).to(torch.uint8).to(DEV)
    compile_moe_reduction(topk=k, model_dim=H, dtype_str=name, use_mask=True)(x, y, mask, T, None)
    want = (x.float() * mask.view(T, k, 1).float()).sum(1)
    torch.testing.assert_close(y.float(), want.to(dt).float(), rtol=1e-2, atol=1e-2)


def _golden_moe():
    g = load_golden("moe.npz")
    T, H, I, E, k = (int(v) for v in g["cfg"])
    t = {n: torch.from_numpy(g[n]) for n in ("x_scale", "topk_ids", "topk_w", "w1_scale", "w2_scale", "out1",
                                             "a2_scale", "out2")}
    t.update(x_q=fp8_from_u8(g["x_q"]), w1_q=fp8_from_u8(g["w1_q"]), w2_q=fp8_from_u8(g["w2_q"]),
             a2_q=fp8_from_u8(g["a2_q"]))
    return (T, H, I, E, k), t


@pytest.mark.parametrize("tile_m", [16, 32, 128])
@pytest.mark.parametrize("block_n", [None, 64, 256])
def test_stage1_vs_golden(tile_m, block_n):
    from flydsl_b200.kernels import compile_moe_blockscale_gemm1
    from flydsl_b200.utils import build_routing_buffers, shuffle_weight

    (T, H, I, E, k), t = _golden_moe()
    sid, sw, seid, nv, _, blocks = build_routing_buffers(topk_ids=t["topk_ids"].to(DEV), topk_weights=t["topk_w"].to(DEV),
                                                         experts=E, model_dim=H, tile_m=tile_m, moe_sort_mode="torch")
    fn = compile_moe_blockscale_gemm1(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=256,
                                      tile_k=128, doweight_stage1=False, out_dtype="f16", block_n=block_n)
    out1 = torch.zeros(T, k, I, dtype=torch.float16, device=DEV)
    fn(out1.view(-1), t["x_q"].to(DEV).view(-1), shuffle_weight(t["w1_q"].to(DEV)).view(-1),
       t["x_scale"].to(DEV).t().contiguous().view(-1), t["w1_scale"].to(DEV).view(-1), sid, seid, sw, nv, T, I, H,
       blocks, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert_close_to_oracle(out1, t["out1"], f"stage1 tile_m={tile_m} bn={block_n}")


@pytest.mark.parametrize("out_dtype,accumulate", [("f16", True), ("bf16", True), ("f32", True), ("f16", False),
                                                  ("bf16", False)])
@pytest.mark.parametrize("tile_m", [16, 128])
def test_stage2_vs_golden(out_dtype, accumulate, tile_m):
    from flydsl_b200.kernels import compile_moe_blockscale_gemm2, compile_moe_reduction
    from flydsl_b200.utils import build_routing_buffers, shuffle_weight

    (T, H, I, E, k), t = _golden_moe()
    sid, sw, seid, nv, _, blocks = build_routing_buffers(topk_ids=t["topk_ids"].to(DEV), topk_weights=t["topk_w"].to(DEV),
                                                         experts=E, model_dim=H, tile_m=tile_m)
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[out_dtype]
    fn = compile_moe_blockscale_gemm2(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=256,
                                      tile_k=128, doweight_stage2=True, out_dtype=out_dtype, accumulate=accumulate)
    args = (t["a2_q"].to(DEV).view(-1), shuffle_weight(t["w2_q"].to(DEV)).view(-1),
            t["a2_scale"].to(DEV).t().contiguous().view(-1), t["w2_scale"].to(DEV).view(-1), sid, seid, sw, nv, T, H, I,
            blocks, torch.cuda.current_stream())
    if accumulate:
        out = torch.zeros(T, H, dtype=tdt, device=DEV)
        fn(out.view(-1), *args)
    else:
        routes = torch.zeros(T * k, H, dtype=tdt, device=DEV)
        fn(routes.view(-1), *args)
        out = torch.empty(T, H, dtype=tdt, device=DEV)
        compile_moe_reduction(topk=k, model_dim=H, dtype_str=out_dtype)(routes.view(T, k, H), out, None, T, None)
    torch.cuda.synchronize()
    budget = MAX_REL_ATOMIC16 if (accumulate and out_dtype != "f32") else MAX_REL
    assert_close_to_oracle(out, t["out2"], f"stage2 {out_dtype} acc={accumulate} tile_m={tile_m}", max_rel=budget)


def test_gemm2_ex_reduce_mode_matches_atomic():
    from flydsl_b200.kernels import MoeGemm2Mode, compile_moe_blockscale_gemm2_ex
    from flydsl_b200.utils import build_routing_buffers, shuffle_weight

    (T, H, I, E, k), t = _golden_moe()
    sid, sw, seid, nv, _, blocks = build_routing_buffers(topk_ids=t["topk_ids"].to(DEV), topk_weights=t["topk_w"].to(DEV),
                                                         experts=E, model_dim=H, tile_m=32)
    args = (t["a2_q"].to(DEV), shuffle_weight(t["w2_q"].to(DEV)), t["a2_scale"].to(DEV).t().contiguous(),
            t["w2_scale"].to(DEV), sid, seid, sw, nv, T, H, I, blocks)
    outs = {}
    for mode in (MoeGemm2Mode.ATOMIC, MoeGemm2Mode.REDUCE):
        exe = compile_moe_blockscale_gemm2_ex(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=32, tile_n=256,
                                              tile_k=128, doweight_stage2=True, out_dtype="bf16", mode=mode)
        out = torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
        exe(out, *args)
        torch.cuda.synchronize()
        outs[mode] = out
        assert_close_to_oracle(out, t["out2"], f"gemm2_ex {mode}",
                               max_rel=MAX_REL_ATOMIC16 if mode == MoeGemm2Mode.ATOMIC else MAX_REL)


# The reference's own shape grid (tests/kernels/test_moe_blockscale.py:195-210): tile 16x256x128; the
# 256-expert rows are run with 64 experts so the CPU oracle's weight generation stays within seconds.
@pytest.mark.parametrize("T,H,I,E,k", [(16, 7168, 256, 8, 2), (32, 7168, 256, 8, 2), (32, 7168, 256, 64, 8),
                                       (128, 1024, 512, 16, 4)])
@pytest.mark.parametrize("mode", ["reduce", "atomic"])
def test_layer_vs_oracle(T, H, I, E, k, mode):
    from flydsl_b200 import _lib
    from flydsl_b200.moe import BlockscaleMoE

    m = O.make_moe_case(T=T, H=H, I=I, E=E, topk=k, seed=T + E, x_std=1.0, w_std=0.02)
    ref, out1_ref, _, _ = O.torch_moe_two_stage_ref(m["x_q"], m["x_scale"], m["w1_q"], m["w1_scale"], m["w2_q"],
                                                    m["w2_scale"], m["topk_ids"], m["topk_weights"], I)
    layer = BlockscaleMoE.from_unpacked(m["w1_q"].to(DEV), m["w1_scale"].to(DEV), m["w2_q"].to(DEV),
                                        m["w2_scale"].to(DEV), topk=k, tile_m=16, mode=mode)
    xs_t = m["x_scale"].to(DEV).t().contiguous()
    out = layer.forward(m["x_q"].to(DEV), xs_t, m["topk_ids"].to(DEV), m["topk_weights"].to(DEV))
    torch.cuda.synchronize()
    assert _lib.query_device_error() == 0
    assert_close_to_oracle(out, ref, f"layer {T},{H},{I},{E},{k} {mode}",
                           max_rel=MAX_REL_ATOMIC16 if mode == "atomic" else MAX_REL)
    if mode == "reduce":  # fixed summation order: bitwise repeatable
        out2 = layer.forward(m["x_q"].to(DEV), xs_t, m["topk_ids"].to(DEV), m["topk_weights"].to(DEV))
        torch.cuda.synchronize()
        assert torch.equal(out, out2)


def test_sorted_layout_matches_gathered_layout():
    """Routing-order intermediates (activations permuted once, TMA-fed stages) against the
    reference-shaped gather path: same arithmetic, so the results must agree bit for bit in the
    deterministic reduce mode; the helper kernels are checked against torch indexing."""
    from flydsl_b200.moe import BlockscaleMoE
    from flydsl_b200.utils import moe_gather_rows, moe_sorting

    m = O.make_moe_case(T=96, H=1024, I=512, E=16, topk=4, seed=11, hot_experts=2, hot_bias=3.0)
    args = (m["x_q"].to(DEV), m["x_scale"].to(DEV).t().contiguous(), m["topk_ids"].to(DEV), m["topk_weights"].to(DEV))
    outs = {}
    for flag in (False, True):
        layer = BlockscaleMoE.from_unpacked(m["w1_q"].to(DEV), m["w1_scale"].to(DEV), m["w2_q"].to(DEV),
                                            m["w2_scale"].to(DEV), topk=4, tile_m=32, sorted_layout=flag)
        outs[flag] = layer.forward(*args)
    torch.cuda.synchronize()
    assert torch.equal(outs[True], outs[False])
    ref, _, _, _ = O.torch_moe_two_stage_ref(m["x_q"], m["x_scale"], m["w1_q"], m["w1_scale"], m["w2_q"],
                                             m["w2_scale"], m["topk_ids"], m["topk_weights"], 512)
    assert_close_to_oracle(outs[True], ref, "sorted layout")
    # gather helper: rows and scales land at their sorted positions, padding is zero
    sid, sw, seid, npp = moe_sorting(args[2], args[3], num_experts=16, block_size=32)
    xs, ss = moe_gather_rows(args[0], args[1], sid, npp, topk=4)
    n = int(npp[0])
    ids = sid[:n].cpu().long()
    tok = ids & 0xFFFFFF
    valid = tok < 96
    want = torch.zeros(n, 1024, dtype=torch.uint8)
    want[valid] = m["x_q"].view(torch.uint8)[tok[valid]]
    assert torch.equal(xs[:n].cpu().view(torch.uint8), want)
    want_s = torch.zeros(n, 8)
    want_s[valid] = m["x_scale"][tok[valid]]
    assert torch.equal(ss[:, :n].cpu().t().contiguous(), want_s)


@pytest.mark.parametrize("mid", [torch.float16, torch.bfloat16])
def test_stage1_fused_requant_is_bit_identical_to_separate_quantiser(mid):
    """Stage 1 with the 1x128 re-quantisation in its epilogue against stage 1 + the stand-alone
    quantiser: same fp8 bytes and scales on every real route row, same layer output."""
    from flydsl_b200.moe import BlockscaleMoE
    from flydsl_b200.utils import moe_sorting

    T, H, I, E, k = 200, 1024, 512, 8, 4
    m = O.make_moe_case(T=T, H=H, I=I, E=E, topk=k, seed=31, x_std=1.0, w_std=0.05)
    args = (m["x_q"].to(DEV), m["x_scale"].to(DEV).t().contiguous(), m["topk_ids"].to(DEV), m["topk_weights"].to(DEV))
    got = {}
    for fused in (False, True):
        layer = BlockscaleMoE.from_unpacked(m["w1_q"].to(DEV), m["w1_scale"].to(DEV), m["w2_q"].to(DEV),
                                            m["w2_scale"].to(DEV), topk=k, tile_m=64, mid_dtype=mid,
                                            sorted_layout=True, fused_quant=fused)
        out = layer.forward(*args)
        b = layer._buffers(T, args[0].device)
        got[fused] = (out.clone(), b["a2_q"].view(torch.uint8).clone(), b["a2_s"].clone())
    torch.cuda.synchronize()
    sid, _, _, npp = moe_sorting(args[2], args[3], num_experts=E, block_size=64)
    n = int(npp[0])
    real = ((sid[:n] & 0xFFFFFF) < T).cpu()
    assert real.sum() == T * k
    assert torch.equal(got[True][1][:n].cpu()[real], got[False][1][:n].cpu()[real])
    assert torch.equal(got[True][2][:, :n].cpu()[:, real], got[False][2][:, :n].cpu()[:, real])
    assert torch.equal(got[True][0], got[False][0])
    ref, _, _, _ = O.torch_moe_two_stage_ref(m["x_q"], m["x_scale"], m["w1_q"], m["w1_scale"], m["w2_q"],
                                             m["w2_scale"], m["topk_ids"], m["topk_weights"], I)
    if mid == torch.float16:   # the oracle's intermediate is fp16
        assert_close_to_oracle(got[True][0], ref, "fused re-quantisation")


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (37, 64, 6), (512, 256, 8), (5, 1000, 33)])
def test_router_matches_oracle(T, E, k):
    """Router kernel against the oracle's torch.topk + softmax: same experts in the same slot order,
    weights to fp32 rounding of the exponentials."""
    from flydsl_b200.utils import route_topk

    g = torch.Generator().manual_seed(T * 1000 + E)
    logits = torch.randn(T, E, generator=g)
    if E >= 64:
        logits[:, :16] += 2.0     # hot experts, as the decode stress config biases them
    ids_ref, w_ref = O.route_topk(logits, k)
    ids, w = route_topk(logits.to(DEV), k)
    assert torch.equal(ids.cpu(), ids_ref)
    torch.testing.assert_close(w.cpu(), w_ref, rtol=2e-6, atol=1e-7)
    torch.testing.assert_close(w.sum(1).cpu(), torch.ones(T), rtol=1e-5, atol=1e-6)


def test_ep_plan_pack_kernel_matches_torch_logic():
    """The fused expert-parallel dispatch preparation against the device-agnostic torch functions."""
    from flydsl_b200 import parallel as P

    g = torch.Generator().manual_seed(5)
    T, H, k, E, W = 300, 512, 8, 64, 8
    x = torch.randint(0, 255, (T, H), generator=g, dtype=torch.uint8)
    xs = torch.rand(T, H // 128, generator=g)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, k, generator=g)
    need_c, slot_c, rows_c = P.plan_pack_cuda(x.to(DEV), xs.to(DEV), ids.to(DEV), w.to(DEV), E // W, W)
    need_t, slot_t, src_t = P.plan_dispatch_fixed(ids, E // W, W)
    rows_t = P.pack_rows_fixed(x, xs, ids, w, src_t)
    assert torch.equal(need_c.cpu().bool(), need_t)
    assert torch.equal(slot_c.cpu().long()[need_t], slot_t[need_t])
    used = src_t >= 0
    assert torch.equal(rows_c.cpu()[used], rows_t[used])
    id_lo = H + 4 * (H // 128)
    assert torch.equal(rows_c.cpu()[~used][:, id_lo:id_lo + 4 * k], rows_t[~used][:, id_lo:id_lo + 4 * k])  # ids = -1


def test_ep_peer_kernels_two_ranks_emulated_on_one_gpu():
    """Push, packed local experts and pull+sum of the peer-memory exchange with both ranks' buffers
    on this GPU and their kernels issued one after the other on one stream (the flag barrier is
    left to the two-GPU test: kernels that wait for each other must not share a GPU). Against the
    single-process oracle and, bit for bit, against the torch/NCCL-path functions."""
    import ctypes

    from flydsl_b200 import _lib, parallel as P
    from flydsl_b200.utils import shuffle_weight

    W, T, H, I, E, k = 2, 48, 512, 256, 8, 4
    m = O.make_moe_case(T=W * T, H=H, I=I, E=E, topk=k, seed=21, w_std=0.05)
    ref, _, _, _ = O.torch_moe_two_stage_ref(m["x_q"], m["x_scale"], m["w1_q"], m["w1_scale"], m["w2_q"],
                                             m["w2_scale"], m["topk_ids"], m["topk_weights"], 256)
    lib = _lib.load()
    EL = E // W
    row_bytes = H + 4 * (H // 128) + 8 * k
    part_off = (W * T * row_bytes + 255) // 256 * 256
    nbytes = part_off + W * T * H * 2
    bufs, views = [], []
    for r in range(W):
        q, h = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
        _lib.check(lib.flyb200_ep_buffer_create(nbytes, ctypes.byref(q), h))
        bufs.append(int(q.value))
        views.append(torch.as_tensor(P._RawCuda(int(q.value), nbytes), device=DEV))
    peers = (ctypes.c_void_p * W)(*bufs)
    try:
        shards, plans = [], []
        for r in range(W):
            lo, hi = r * EL, (r + 1) * EL
            shards.append(P.LocalExpertShard(
                shuffle_weight(m["w1_q"][lo:hi].to(DEV)), m["w1_scale"][lo:hi].to(DEV),
                shuffle_weight(m["w2_q"][lo:hi].to(DEV)), m["w2_scale"][lo:hi].to(DEV),
                experts=E, topk=k, rank=r, world=W, tile_m=32))
        for r in range(W):      # every rank pushes its tokens
            sl = slice(r * T, (r + 1) * T)
            x = m["x_q"][sl].view(torch.uint8).to(DEV)
            xs, ids = m["x_scale"][sl].to(DEV).contiguous(), m["topk_ids"][sl].to(DEV).to(torch.int32).contiguous()
            w = m["topk_weights"][sl].to(DEV).float().contiguous()
            need = torch.empty((T, W), dtype=torch.uint8, device=DEV)
            slot = torch.empty((T, W), dtype=torch.int32, device=DEV)
            src = torch.empty((W * T,), dtype=torch.int32, device=DEV)
            _lib.check(lib.flyb200_ep_push(x.data_ptr(), xs.data_ptr(), ids.data_ptr(), w.data_ptr(), T, H, k, W,
                                           r, EL, peers, 0, need.data_ptr(), slot.data_ptr(), src.data_ptr(),
                                           _lib.stream_handle(None)))
            plans.append((need, slot))
            # what landed in rank d's receive area is what the packed NCCL path would have sent there
            _, _, rows = P.plan_pack_cuda(x, xs, ids, w, EL, W)
            used = (src >= 0).cpu()
            for d in range(W):
                got = views[d][: W * T * row_bytes].view(W * T, row_bytes)[r * T:(r + 1) * T].cpu()
                u = used[d * T:(d + 1) * T]
                assert torch.equal(got[u], rows[d * T:(d + 1) * T].cpu()[u])
                id_lo = H + 4 * (H // 128)
                assert (got[~u][:, id_lo:id_lo + 4 * k].contiguous().view(torch.int32) == -1).all()
        for r in range(W):      # local experts on the packed rows, partials into the own partial area
            recv = views[r][: W * T * row_bytes].view(W * T, row_bytes)
            part = views[r][part_off:part_off + W * T * H * 2].view(torch.bfloat16).view(W * T, H)
            shards[r].forward_packed(recv, out=part)
            rx = P.unpack_rows(recv, H, k)
            assert torch.equal(shards[r](*rx).clone(), part)          # same result as the unpacked entry
        outs = []
        for r in range(W):      # every rank pulls and sums the partial rows of its tokens
            need, slot = plans[r]
            out = torch.empty((T, H), dtype=torch.bfloat16, device=DEV)
            _lib.check(lib.flyb200_ep_pull_combine(peers, part_off, need.data_ptr(), slot.data_ptr(),
                                                   out.data_ptr(), T, W, H, r, _lib.BF16, _lib.stream_handle(None)))
            # the NCCL path's combine on the same partial rows: back[q*T + j] = rank q's row r*T + j
            back = torch.cat([views[q][part_off:part_off + W * T * H * 2].view(torch.bfloat16).view(W * T, H)
                              [r * T:(r + 1) * T] for q in range(W)], dim=0).contiguous()
            assert torch.equal(P.combine_partials_fixed(back, need, slot, torch.bfloat16), out)
            assert torch.equal(P.combine_partials_fixed(back.cpu(), need.cpu(), slot.cpu(), torch.bfloat16), out.cpu())
            outs.append(out.float().cpu())
        # push variant: the reduce writes each partial row into the owner's back area (= partial
        # area, free again by now), the owner sums its own memory -- same bits as the pull variant
        for r in range(W):
            recv = views[r][: W * T * row_bytes].view(W * T, row_bytes)
            shards[r].forward_packed(recv, reducer=lambda routes, valid, r=r: _lib.check(
                lib.flyb200_ep_reduce_push(routes.data_ptr(), valid.data_ptr(), peers, part_off, T, W, k, H, r,
                                           _lib.BF16, _lib.stream_handle(None))))
        for r in range(W):
            need, slot = plans[r]
            out = torch.empty((T, H), dtype=torch.bfloat16, device=DEV)
            _lib.check(lib.flyb200_ep_combine(bufs[r] + part_off, need.data_ptr(), slot.data_ptr(), out.data_ptr(),
                                              T, W, H, _lib.BF16, _lib.stream_handle(None)))
            assert torch.equal(out.float().cpu(), outs[r])
        torch.cuda.synchronize()
        assert _lib.query_device_error() == 0
        assert_close_to_oracle(torch.cat(outs, dim=0), ref, "peer exchange, two ranks emulated")
    finally:
        torch.cuda.synchronize()
        views.clear()
        for q in bufs:
            _lib.check(lib.flyb200_ep_buffer_destroy(q))


def test_skewed_routing_and_empty_experts():
    """Decode-style stress: hot experts, many experts with zero tokens, tile_m larger than any count."""
    from flydsl_b200.moe import BlockscaleMoE

    m = O.make_moe_case(T=40, H=512, I=256, E=32, topk=4, seed=4, hot_experts=4, hot_bias=4.0)
    counts = torch.bincount(m["topk_ids"].flatten().long(), minlength=32)
    assert (counts == 0).any() and counts.max() > 20
    ref, _, _, _ = O.torch_moe_two_stage_ref(m["x_q"], m["x_scale"], m["w1_q"], m["w1_scale"], m["w2_q"],
                                             m["w2_scale"], m["topk_ids"], m["topk_weights"], 256)
    for tile_m in (16, 128):
        layer = BlockscaleMoE.from_unpacked(m["w1_q"].to(DEV), m["w1_scale"].to(DEV), m["w2_q"].to(DEV),
                                            m["w2_scale"].to(DEV), topk=4, tile_m=tile_m)
        out = layer.forward(m["x_q"].to(DEV), m["x_scale"].to(DEV).t().contiguous(), m["topk_ids"].to(DEV),
                            m["topk_weights"].to(DEV))
        torch.cuda.synchronize()
        assert_close_to_oracle(out, ref, f"skew tile_m={tile_m}")


def test_moe_factories_validate():
    from flydsl_b200.kernels import compile_moe_blockscale_gemm1, compile_moe_blockscale_gemm2

    kw = dict(model_dim=256, inter_dim=128, experts=4, topk=2, tile_m=16, tile_n=256, tile_k=128)
    with pytest.raises(ValueError):
        compile_moe_blockscale_gemm1(doweight_stage1=False, out_dtype="f32", **kw)
    with pytest.raises(ValueError):
        compile_moe_blockscale_gemm2(doweight_stage2=True, out_dtype="f32", accumulate=False, **kw)
    with pytest.raises(ValueError):
        compile_moe_blockscale_gemm2(doweight_stage2=True, out_dtype="int8", **kw)
