"""Per-token-scale FP8 MoE (compile_moe_gemm1 / compile_moe_gemm2 / compile_moe_gemm2_ex) on the GPU,
against the golden vectors made with the reference's torch_moe_gemm1 / torch_moe_gemm2 and against
the CPU oracle on larger seeded cases."""
import pytest
import torch

from oracle import blockscale_ref as O
from tests.helpers import MAX_REL, MAX_REL_ATOMIC16, assert_close_to_oracle, fp8_from_u8, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"
TDT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def _golden():
    g = load_golden("moe_pertoken.npz")
    cfg = tuple(int(v) for v in g["cfg"])
    t = {n: torch.from_numpy(g[n]) for n in ("x_scale", "topk_ids", "topk_w", "w1_scale", "w2_scale", "out1",
                                             "out1_weighted", "a2_scale", "out2", "out2_unweighted")}
    t.update(x_q=fp8_from_u8(g["x_q"]), w1_q=fp8_from_u8(g["w1_q"]), w2_q=fp8_from_u8(g["w2_q"]),
             a2_q=fp8_from_u8(g["a2_q"]))
    return cfg, t


def _routing(ids, tw, E, H, tile_m):
    from flydsl_b200.utils import build_routing_buffers

    sid, sw, seid, nv, _, blocks = build_routing_buffers(topk_ids=ids.to(DEV), topk_weights=tw.to(DEV), experts=E,
                                                         model_dim=H, tile_m=tile_m, moe_sort_mode="torch")
    return sid, sw, seid, nv, blocks


def _stage1(t, cfg, tile_m, doweight, out_dtype="f16"):
    from flydsl_b200.kernels import compile_moe_gemm1
    from flydsl_b200.utils import shuffle_weight

    T, H, I, E, k = cfg
    sid, sw, seid, nv, blocks = _routing(t["topk_ids"], t["topk_w"], E, H, tile_m)
    fn = compile_moe_gemm1(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=256, tile_k=128,
                           doweight_stage1=doweight, in_dtype="fp8", out_dtype=out_dtype)
    out1 = torch.zeros(T, k, I, dtype=TDT[out_dtype], device=DEV)
    fn(out1.view(-1), t["x_q"].to(DEV).view(-1), shuffle_weight(t["w1_q"].to(DEV)).view(-1),
       t["x_scale"].to(DEV).view(-1), t["w1_scale"].to(DEV).view(-1), sid, seid, sw, nv, T, I, H, blocks,
       torch.cuda.current_stream())
    torch.cuda.synchronize()
    return out1


def _stage2(t, cfg, tile_m, doweight, out_dtype, accumulate):
    from flydsl_b200.kernels import compile_moe_gemm2, compile_moe_reduction
    from flydsl_b200.utils import shuffle_weight

    T, H, I, E, k = cfg
    sid, sw, seid, nv, blocks = _routing(t["topk_ids"], t["topk_w"], E, H, tile_m)
    fn = compile_moe_gemm2(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=256, tile_k=128,
                           doweight_stage2=doweight, in_dtype="fp8", out_dtype=out_dtype, accumulate=accumulate)
    args = (t["a2_q"].to(DEV).view(-1), shuffle_weight(t["w2_q"].to(DEV)).view(-1), t["a2_scale"].to(DEV).view(-1),
            t["w2_scale"].to(DEV).view(-1), sid, seid, sw, nv, T, H, I, blocks, torch.cuda.current_stream())
    if accumulate:
        out = torch.zeros(T, H, dtype=TDT[out_dtype], device=DEV)
        fn(out.view(-1), *args)
    else:
        routes = torch.zeros(T * k, H, dtype=TDT[out_dtype], device=DEV)
        fn(routes.view(-1), *args)
        out = torch.empty(T, H, dtype=TDT[out_dtype], device=DEV)
        compile_moe_reduction(topk=k, model_dim=H, dtype_str=out_dtype)(routes.view(T, k, H), out, None, T, None)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("tile_m", [16, 32, 64, 128])
@pytest.mark.parametrize("doweight", [False, True])
def test_stage1_vs_golden(tile_m, doweight):
    cfg, t = _golden()
    out1 = _stage1(t, cfg, tile_m, doweight)
    assert_close_to_oracle(out1, t["out1_weighted" if doweight else "out1"], f"stage1 tile_m={tile_m} w={doweight}")


@pytest.mark.parametrize("out_dtype,accumulate", [("f16", True), ("bf16", True), ("f32", True), ("f16", False),
                                                  ("bf16", False)])
@pytest.mark.parametrize("tile_m", [16, 128])
def test_stage2_vs_golden(out_dtype, accumulate, tile_m):
    cfg, t = _golden()
    out = _stage2(t, cfg, tile_m, True, out_dtype, accumulate)
    budget = MAX_REL_ATOMIC16 if (accumulate and out_dtype != "f32") else MAX_REL
    assert_close_to_oracle(out, t["out2"], f"stage2 {out_dtype} acc={accumulate} tile_m={tile_m}", max_rel=budget)


def test_stage2_unweighted_vs_golden():
    cfg, t = _golden()
    out = _stage2(t, cfg, 32, False, "f32", True)
    assert_close_to_oracle(out, t["out2_unweighted"], "stage2 without route weights")


def _seeded_case(T, H, I, E, k, seed, hot=0):
    g = torch.Generator().manual_seed(seed)
    s = 0.2
    x = torch.randn(T, H, generator=g) * s
    w1 = torch.randn(E, 2 * I, H, generator=g) * s
    w2 = torch.randn(E, H, I, generator=g) * (s / I ** 0.5)
    score = torch.rand(T, E, generator=g)
    if hot:
        score[:, :hot] += 1.0
    vals, ids = torch.topk(score, k=k, dim=1)
    tw = torch.softmax(vals, dim=1).float()
    xq, xs = O.pertoken_quant(x)
    w1q, w1s = O.pertoken_quant(w1)
    w2q, w2s = O.pertoken_quant(w2)
    return dict(x_q=xq, x_scale=xs.reshape(-1), w1_q=w1q, w1_scale=w1s.reshape(-1), w2_q=w2q,
                w2_scale=w2s.reshape(-1), topk_ids=ids.to(torch.int32), topk_w=tw)


# the reference's small and medium rows (tests/kernels/test_moe_gemm.py test_moe_gemm_2stage grid:
# model_dim / inter_dim multiples of 256, 8-16 experts, top-2/4) plus ragged token counts and a case
# with many row blocks per expert and empty experts
@pytest.mark.parametrize("T,H,I,E,k,tile_m,hot", [(64, 1024, 256, 4, 2, 32, 0), (129, 1024, 256, 8, 2, 64, 0),
                                                  (333, 512, 384, 16, 4, 128, 0), (1, 256, 128, 8, 2, 16, 0),
                                                  (700, 256, 128, 8, 2, 128, 2)])
def test_two_stage_chain_vs_oracle(T, H, I, E, k, tile_m, hot):
    """gemm1 -> fp16 -> per-route re-quantisation (the reference's host-side pertoken_quant) -> gemm2
    in reduce mode, each stage against the oracle on the tensors the GPU chain itself produced."""
    from flydsl_b200.kernels import MoeGemm2Mode, compile_moe_gemm2_ex
    from flydsl_b200.utils import pertoken_quant, shuffle_weight

    cfg = (T, H, I, E, k)
    t = _seeded_case(T, H, I, E, k, seed=T + E, hot=hot)
    out1 = _stage1(t, cfg, tile_m, False)
    ids64 = t["topk_ids"].to(torch.int64)
    want1 = O.torch_moe_gemm1_pertoken_ref(t["x_q"], t["w1_q"], t["x_scale"], t["w1_scale"], ids64, t["topk_w"], I)
    assert_close_to_oracle(out1, want1, f"stage1 {cfg}")

    a2q, a2s = pertoken_quant(out1.float())          # [T, k, I] fp8, [T, k, 1]
    sid, sw, seid, nv, blocks = _routing(t["topk_ids"], t["topk_w"], E, H, tile_m)
    exe = compile_moe_gemm2_ex(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=256, tile_k=128,
                               doweight_stage2=True, in_dtype="fp8", out_dtype="bf16", mode=MoeGemm2Mode.REDUCE)
    assert exe.mode == MoeGemm2Mode.REDUCE
    out = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    exe(out, a2q.view(-1), shuffle_weight(t["w2_q"].to(DEV)).view(-1), a2s.view(-1), t["w2_scale"].to(DEV), sid, seid,
        sw, nv, T, H, I, blocks)
    torch.cuda.synchronize()
    want2 = O.torch_moe_gemm2_pertoken_ref(a2q.cpu(), t["w2_q"], a2s.cpu(), t["w2_scale"], ids64, t["topk_w"], H)
    assert_close_to_oracle(out, want2, f"stage2 reduce {cfg}")


def test_gemm2_ex_modes_and_valid_mask():
    from flydsl_b200.kernels import MoeGemm2Mode, compile_moe_gemm2_ex
    from flydsl_b200.utils import shuffle_weight

    cfg, t = _golden()
    T, H, I, E, k = cfg
    sid, sw, seid, nv, blocks = _routing(t["topk_ids"], t["topk_w"], E, H, 32)
    args = (t["a2_q"].to(DEV), shuffle_weight(t["w2_q"].to(DEV)), t["a2_scale"].to(DEV), t["w2_scale"].to(DEV), sid,
            seid, sw, nv, T, H, I, blocks)
    common = dict(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=32, tile_n=256, tile_k=128,
                  doweight_stage2=True, in_dtype="fp8", out_dtype="f16")
    atomic = compile_moe_gemm2_ex(mode=MoeGemm2Mode.ATOMIC, **common)
    out = torch.zeros(T, H, dtype=torch.float16, device=DEV)
    atomic(out, *args)
    torch.cuda.synchronize()
    assert_close_to_oracle(out, t["out2"], "gemm2_ex atomic", max_rel=MAX_REL_ATOMIC16)

    # masked reduce: slot 1 of every odd token is dropped from the sum
    mask = torch.ones(T, k, dtype=torch.uint8, device=DEV)
    mask[1::2, 1] = 0
    masked = compile_moe_gemm2_ex(mode=MoeGemm2Mode.REDUCE, valid_mask=mask, **common)
    out_m = torch.empty(T, H, dtype=torch.float16, device=DEV)
    masked(out_m, *args, valid_mask=mask)
    torch.cuda.synchronize()
    routes = O.torch_moe_gemm2_pertoken_ref(t["a2_q"].view(T, k, I), t["w2_q"], t["a2_scale"], t["w2_scale"],
                                            t["topk_ids"].to(torch.int64), t["topk_w"], H, per_route=True)
    want = (routes * mask.cpu().view(T, k, 1).float()).sum(1)
    assert_close_to_oracle(out_m, want, "gemm2_ex reduce with valid_mask")

    # zero_intermediate=False is allowed when every (token, slot) has a routing position
    nz = compile_moe_gemm2_ex(mode=MoeGemm2Mode.REDUCE, zero_intermediate=False, **common)
    out_nz = torch.empty(T, H, dtype=torch.float16, device=DEV)
    nz(out_nz, *args)
    torch.cuda.synchronize()
    assert_close_to_oracle(out_nz, t["out2"], "gemm2_ex reduce without zero fill")


def test_factories_validate_like_the_reference():
    from flydsl_b200.kernels import compile_moe_gemm1, compile_moe_gemm2, compile_moe_gemm2_ex

    ok = dict(model_dim=256, inter_dim=128, experts=4, topk=2, tile_m=32, tile_n=128, tile_k=128)
    with pytest.raises(ValueError, match="in_dtype must be one of"):
        compile_moe_gemm1(doweight_stage1=False, in_dtype="fp4", **ok)
    with pytest.raises(NotImplementedError):
        compile_moe_gemm1(doweight_stage1=False, in_dtype="int8", **ok)
    with pytest.raises(NotImplementedError):
        compile_moe_gemm2(doweight_stage2=True, in_dtype="int4_bf16", group_size=32, **ok)
    with pytest.raises(ValueError, match="out_dtype must be"):
        compile_moe_gemm2(doweight_stage2=True, out_dtype="i8", **ok)
    with pytest.raises(ValueError, match="accumulate=False"):
        compile_moe_gemm2(doweight_stage2=True, out_dtype="f32", accumulate=False, **ok)
    with pytest.raises(ValueError, match="tile_k_bytes"):
        compile_moe_gemm1(doweight_stage1=False, **{**ok, "tile_k": 96})
    with pytest.raises(ValueError, match="mode must be"):
        compile_moe_gemm2_ex(doweight_stage2=True, mode="sum", **ok)
    fn = compile_moe_gemm1(doweight_stage1=False, **ok)
    assert fn is compile_moe_gemm1(doweight_stage1=False, **ok)   # cached like the reference's factories
    z = torch.zeros(8, dtype=torch.float32, device=DEV)
    with pytest.raises(ValueError, match="built for"):
        fn(z, z, z, z, z, z, z, z, z, 4, 256, 256, 1)


@pytest.mark.parametrize("tile_m", [16, 128])
def test_routing_order_layouts_give_the_same_bits_as_the_gathered_layouts(tile_m):
    """a_sorted / out_sorted (rows fetched by TMA, staged tiles written by the store warps) against
    the reference layouts (rows gathered, [tokens, topk, ...] outputs): same tiles, same arithmetic."""
    from flydsl_b200.kernels import compile_moe_gemm1, compile_moe_gemm2
    from flydsl_b200.utils import pertoken_quant, shuffle_weight

    T, H, I, E, k = cfg = (200, 512, 256, 8, 2)
    t = _seeded_case(T, H, I, E, k, seed=77, hot=1)
    sid, sw, seid, nv, blocks = _routing(t["topk_ids"], t["topk_w"], E, H, tile_m)
    rows = T * k + E * tile_m - k
    tok, slot = (sid[:rows] & 0xFFFFFF).long(), (sid[:rows] >> 24).long()
    valid = tok < T
    x_sorted = torch.zeros(rows, H, dtype=torch.uint8, device=DEV)
    x_sorted[valid] = t["x_q"].to(DEV).view(torch.uint8)[tok[valid]]
    xs_sorted = torch.ones(rows, dtype=torch.float32, device=DEV)
    xs_sorted[valid] = t["x_scale"].to(DEV)[tok[valid]]
    common = dict(model_dim=H, inter_dim=I, experts=E, topk=k, tile_m=tile_m, tile_n=256, tile_k=128)
    w1 = shuffle_weight(t["w1_q"].to(DEV))
    w2 = shuffle_weight(t["w2_q"].to(DEV))

    want1 = _stage1(t, cfg, tile_m, True)
    g1 = compile_moe_gemm1(doweight_stage1=True, a_sorted=True, out_sorted=True, **common)
    out1_sorted = torch.zeros(rows, I, dtype=torch.float16, device=DEV)
    g1(out1_sorted, x_sorted.view(torch.float8_e4m3fn), w1, xs_sorted, t["w1_scale"].to(DEV), sid, seid, sw, nv, T, I,
       H, blocks)
    torch.cuda.synchronize()
    got1 = torch.zeros_like(want1)
    got1[tok[valid], slot[valid]] = out1_sorted[valid]
    assert torch.equal(got1, want1)

    a2q, a2s = pertoken_quant(want1.float())                       # [T, k, I], [T, k, 1]
    a2_sorted = torch.zeros(rows, I, dtype=torch.uint8, device=DEV)
    a2_sorted[valid] = a2q.view(torch.uint8)[tok[valid], slot[valid]]
    a2s_sorted = torch.ones(rows, dtype=torch.float32, device=DEV)
    a2s_sorted[valid] = a2s[tok[valid], slot[valid], 0]
    outs = []
    for a_sorted, x2, s2 in ((False, a2q, a2s), (True, a2_sorted.view(torch.float8_e4m3fn), a2s_sorted)):
        g2 = compile_moe_gemm2(doweight_stage2=False, out_dtype="bf16", accumulate=False, a_sorted=a_sorted, **common)
        routes = torch.zeros(T * k, H, dtype=torch.bfloat16, device=DEV)
        g2(routes, x2, w2, s2, t["w2_scale"].to(DEV), sid, seid, sw, nv, T, H, I, blocks)
        torch.cuda.synchronize()
        outs.append(routes)
    assert torch.equal(outs[0], outs[1])
    want2 = O.torch_moe_gemm2_pertoken_ref(a2q.cpu(), t["w2_q"], a2s.cpu(), t["w2_scale"],
                                           t["topk_ids"].to(torch.int64), t["topk_w"], H, doweight_stage2=False,
                                           per_route=True)
    assert_close_to_oracle(outs[1].view(T, k, H), want2, "stage2 routes, routing-order input")


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_quant_pertoken_is_bit_exact_with_the_torch_quantiser(dt):
    from flydsl_b200.utils import quant_pertoken

    g = torch.Generator().manual_seed(5)
    x = (torch.randn(300, 2048, generator=g) * 3).to(dt)
    x[3] = 0.0                               # all-zero row -> scale 1
    x[5, 7] = float("inf")
    x[6, 9] = float("nan")
    x[7, 11] = float("-inf")
    x[8] *= 1e-4                             # small values
    x[9, :64] = -0.0
    x[10] = x[10].abs().clamp(max=7.0)
    x[10, 0] = 7.0                           # amax = 7 * 2^0: a power-of-two scale, exact ties
    x[11] *= 1e-30 if dt == torch.bfloat16 else 1e-3
    want_q, want_s = O.pertoken_quant(x.float())
    q, s = quant_pertoken(x.to(DEV))
    torch.cuda.synchronize()
    assert torch.equal(s.cpu(), want_s.reshape(-1))
    assert torch.equal(q.cpu().view(torch.uint8), want_q.view(torch.uint8))

    # a device-side row count: rows beyond it are left untouched; odd widths
    x2 = (torch.randn(50, 520, generator=g)).to(dt).to(DEV)
    n = torch.tensor([17], dtype=torch.int32, device=DEV)
    q2 = torch.full((50, 520), 0x7F, dtype=torch.uint8, device=DEV).view(torch.float8_e4m3fn)
    s2 = torch.full((50,), -1.0, dtype=torch.float32, device=DEV)
    quant_pertoken(x2, n, out=q2, scale_out=s2)
    torch.cuda.synchronize()
    wq, ws = O.pertoken_quant(x2.cpu().float())
    assert torch.equal(q2.cpu().view(torch.uint8)[:17], wq.view(torch.uint8)[:17])
    assert torch.equal(s2.cpu()[:17], ws.reshape(-1)[:17])
    assert bool((q2.cpu().view(torch.uint8)[17:] == 0x7F).all()) and bool((s2.cpu()[17:] == -1.0).all())


def test_gather_rows_with_one_scale_per_row():
    from flydsl_b200.utils import moe_gather_rows

    T, H, E, k, tile_m = 77, 256, 8, 2, 16
    t = _seeded_case(T, H, 128, E, k, seed=9)
    sid, sw, seid, nv, blocks = _routing(t["topk_ids"], t["topk_w"], E, H, tile_m)
    xs, ss = moe_gather_rows(t["x_q"].to(DEV), t["x_scale"].to(DEV), sid, nv, topk=k, per_token=True)
    torch.cuda.synchronize()
    valid_rows = int(nv[0])
    tok = (sid[:valid_rows] & 0xFFFFFF).long().cpu()
    ok = tok < T
    want = torch.zeros(valid_rows, H, dtype=torch.uint8)
    want[ok] = t["x_q"].view(torch.uint8)[tok[ok]]
    want_s = torch.zeros(valid_rows)
    want_s[ok] = t["x_scale"][tok[ok]]
    assert torch.equal(xs.cpu().view(torch.uint8)[:valid_rows], want)
    assert torch.equal(ss.cpu()[:valid_rows], want_s)


@pytest.mark.parametrize("T,H,I,E,k,tile_m,hot", [(64, 1024, 256, 4, 2, 32, 0), (333, 512, 384, 16, 4, 128, 0),
                                                  (1, 256, 128, 8, 2, 16, 0), (700, 256, 128, 8, 2, 128, 2),
                                                  (512, 7168, 2048, 8, 4, 128, 0)])
def test_layer_vs_oracle(T, H, I, E, k, tile_m, hot):
    """PertokenMoE (sort, permute, stage 1, whole-row re-quantisation, stage 2, reduce: all kernels)
    against the oracle's chain (stage 1 -> fp16 -> pertoken_quant -> stage 2)."""
    from flydsl_b200.moe import PertokenMoE

    t = _seeded_case(T, H, I, E, k, seed=3 * T + E, hot=hot)
    layer = PertokenMoE.from_unpacked(t["w1_q"].to(DEV), t["w1_scale"].to(DEV), t["w2_q"].to(DEV),
                                      t["w2_scale"].to(DEV), topk=k, tile_m=tile_m)
    out = layer.forward(t["x_q"].to(DEV), t["x_scale"].to(DEV), t["topk_ids"].to(DEV), t["topk_w"].to(DEV))
    out_again = layer.forward(t["x_q"].to(DEV), t["x_scale"].to(DEV), t["topk_ids"].to(DEV), t["topk_w"].to(DEV))
    torch.cuda.synchronize()
    assert torch.equal(out, out_again)        # fixed summation order: deterministic
    ids64 = t["topk_ids"].to(torch.int64)
    out1 = O.torch_moe_gemm1_pertoken_ref(t["x_q"], t["w1_q"], t["x_scale"], t["w1_scale"], ids64, t["topk_w"], I)
    a2q, a2s = O.pertoken_quant(out1.to(torch.float16).float())
    want = O.torch_moe_gemm2_pertoken_ref(a2q, t["w2_q"], a2s, t["w2_scale"], ids64, t["topk_w"], H)
    assert_close_to_oracle(out, want, f"per-token layer {(T, H, I, E, k)}")


@pytest.mark.parametrize("kind", ["pertoken", "blockscale"])
def test_layers_replay_from_a_cuda_graph(kind):
    """Both layer chains are launch-only after warm-up, so a step can be captured once and replayed
    on new inputs written into the same buffers (the reference's tests do the same with their
    testGraph switch, tests/test_common.py:79-91)."""
    from flydsl_b200.moe import BlockscaleMoE, PertokenMoE

    T, H, I, E, k, tile_m = 96, 512, 256, 8, 2, 32
    if kind == "pertoken":
        t = _seeded_case(T, H, I, E, k, seed=21)
        layer = PertokenMoE.from_unpacked(t["w1_q"].to(DEV), t["w1_scale"].to(DEV), t["w2_q"].to(DEV),
                                          t["w2_scale"].to(DEV), topk=k, tile_m=tile_m)
        x_q, x_s = t["x_q"].to(DEV), t["x_scale"].to(DEV)
        t2 = _seeded_case(T, H, I, E, k, seed=22)
        x_q2, x_s2 = t2["x_q"].to(DEV), t2["x_scale"].to(DEV)
    else:
        m = O.make_moe_case(T, H, I, E, k, seed=21)
        layer = BlockscaleMoE.from_unpacked(m["w1_q"].to(DEV), m["w1_scale"].to(DEV), m["w2_q"].to(DEV),
                                            m["w2_scale"].to(DEV), topk=k, tile_m=tile_m)
        t = {"topk_ids": m["topk_ids"], "topk_w": m["topk_weights"]}
        x_q, x_s = m["x_q"].to(DEV), m["x_scale"].t().contiguous().to(DEV)
        m2 = O.make_moe_case(T, H, I, E, k, seed=22)
        t2 = {"topk_ids": m2["topk_ids"], "topk_w": m2["topk_weights"]}
        x_q2, x_s2 = m2["x_q"].to(DEV), m2["x_scale"].t().contiguous().to(DEV)
    ids, tw = t["topk_ids"].to(DEV), t["topk_w"].to(DEV)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(2):
            layer.forward(x_q, x_s, ids, tw, out=out)      # warm-up: buffers, kernel attributes
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        layer.forward(x_q, x_s, ids, tw, out=out)
    # new inputs and routing in the captured buffers
    x_q.copy_(x_q2); x_s.copy_(x_s2); ids.copy_(t2["topk_ids"].to(DEV)); tw.copy_(t2["topk_w"].to(DEV))
    graph.replay()
    torch.cuda.synchronize()
    got = out.clone()
    want = layer.forward(x_q, x_s, ids, tw)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
