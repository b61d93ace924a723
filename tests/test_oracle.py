"""The CPU oracle against (a) golden vectors produced by the reference's own functions and
(b) the reference functions run live when a checkout is mounted. CPU only."""
import numpy as np
import pytest
import torch

from oracle import blockscale_ref as O
from oracle import ref_loader
from tests.helpers import bf16_from_bits, fp8_from_u8, load_golden


@pytest.mark.parametrize("tag", ["a", "b", "c", "q"])
def test_dense_oracle_matches_golden(tag):
    g = load_golden("dense.npz")
    x, w = fp8_from_u8(g[f"{tag}_x"]), fp8_from_u8(g[f"{tag}_w"])
    xs, ws = torch.from_numpy(g[f"{tag}_xs"]), torch.from_numpy(g[f"{tag}_ws"])
    out = O.run_torch_blockscale(x, w, xs, ws, dtype=torch.bfloat16)
    want = bf16_from_bits(g[f"{tag}_c_bf16_bits"])
    # same fp32 operations in the same order => identical bits
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    if f"{tag}_c_f32" in g:
        out32 = O.run_torch_blockscale(x, w, xs, ws, dtype=torch.float32)
        assert torch.equal(out32, torch.from_numpy(g[f"{tag}_c_f32"]))


@pytest.mark.parametrize("tag", ["a", "b"])
def test_pertoken_oracle_matches_golden(tag):
    g = load_golden("pertoken.npz")
    a, b = fp8_from_u8(g[f"{tag}_a"]), fp8_from_u8(g[f"{tag}_b"])
    c = O.run_torch_pertoken(a, b, torch.from_numpy(g[f"{tag}_sa"]), torch.from_numpy(g[f"{tag}_sb"]))
    assert torch.equal(c, torch.from_numpy(g[f"{tag}_c_f32"]))


def test_pertoken_moe_oracle_matches_golden():
    g = load_golden("moe_pertoken.npz")
    T, H, I, E, k = (int(v) for v in g["cfg"])
    ids = torch.from_numpy(g["topk_ids"]).to(torch.int64)
    tw = torch.from_numpy(g["topk_w"])
    xq, w1q, w2q, a2q = (fp8_from_u8(g[n]) for n in ("x_q", "w1_q", "w2_q", "a2_q"))
    xs, w1s, w2s, a2s = (torch.from_numpy(g[n]) for n in ("x_scale", "w1_scale", "w2_scale", "a2_scale"))
    for doweight, key in ((False, "out1"), (True, "out1_weighted")):
        out1 = O.torch_moe_gemm1_pertoken_ref(xq, w1q, xs, w1s, ids, tw, I, doweight_stage1=doweight)
        torch.testing.assert_close(out1, torch.from_numpy(g[key]), rtol=1e-6, atol=1e-6)
    # the chain of the reference test: fp16 rounding, then per-route re-quantisation (bit-exact)
    q, s = O.pertoken_quant(torch.from_numpy(g["out1"]).to(torch.float16).float())
    assert np.array_equal(q.view(torch.uint8).numpy(), g["a2_q"])
    assert np.array_equal(s.reshape(-1).numpy(), g["a2_scale"])
    for doweight, key in ((True, "out2"), (False, "out2_unweighted")):
        out2 = O.torch_moe_gemm2_pertoken_ref(a2q, w2q, a2s, w2s, ids, tw, H, doweight_stage2=doweight)
        torch.testing.assert_close(out2, torch.from_numpy(g[key]), rtol=1e-6, atol=1e-6)


def test_quantisers_match_golden():
    g = load_golden("quant.npz")
    q, s = O.pertoken_quant(torch.from_numpy(g["x"]))
    assert np.array_equal(q.view(torch.uint8).numpy(), g["q"])
    assert np.array_equal(s.numpy(), g["scale"])
    d = load_golden("dense.npz")
    aq, asc = O.quant_1x128(torch.from_numpy(d["q_a_f32"]))
    assert np.array_equal(aq.view(torch.uint8).numpy(), d["q_x"])
    assert np.array_equal(asc.numpy(), d["q_xs"])
    bq, bsc = O.block_quant_128x128(torch.from_numpy(d["q_b_f32"]))
    assert np.array_equal(bq.view(torch.uint8).numpy(), d["q_w"])
    assert np.array_equal(bsc.reshape(d["q_ws"].shape).numpy(), d["q_ws"])


@pytest.mark.parametrize("tag", ["s0", "s1", "s2", "s3", "s4"])
def test_sort_oracle_matches_golden(tag):
    g = load_golden("sort.npz")
    T, k, E, bs, nlt = (int(v) for v in g[f"{tag}_cfg"])
    mask = g[f"{tag}_mask"] if g[f"{tag}_mask"].size else None
    sid, sw, seid, npp = O.moe_sorting_ref(g[f"{tag}_ids"], g[f"{tag}_w"], E, bs, expert_mask=mask,
                                           num_local_tokens=None if nlt < 0 else nlt)
    assert np.array_equal(sid, g[f"{tag}_sorted_ids"])
    assert np.array_equal(sw, g[f"{tag}_sorted_w"])
    assert np.array_equal(seid, g[f"{tag}_expert_ids"])
    assert np.array_equal(npp, g[f"{tag}_post_pad"])


def test_moe_oracle_matches_golden():
    g = load_golden("moe.npz")
    T, H, I, E, k = (int(v) for v in g["cfg"])
    xq, xs = fp8_from_u8(g["x_q"]), torch.from_numpy(g["x_scale"])
    w1q, w1s = fp8_from_u8(g["w1_q"]), torch.from_numpy(g["w1_scale"])
    w2q, w2s = fp8_from_u8(g["w2_q"]), torch.from_numpy(g["w2_scale"])
    ids, tw = torch.from_numpy(g["topk_ids"]), torch.from_numpy(g["topk_w"])
    out, out1, a2q, a2s = O.torch_moe_two_stage_ref(xq, xs, w1q, w1s, w2q, w2s, ids, tw, I)
    # per-expert matmuls are the same calls on the same values; allow only fp32 reassociation noise
    torch.testing.assert_close(out1, torch.from_numpy(g["out1"]), rtol=1e-5, atol=1e-6)
    assert (a2q.view(torch.uint8).numpy() != g["a2_q"]).mean() < 1e-3
    torch.testing.assert_close(a2s, torch.from_numpy(g["a2_scale"]), rtol=1e-5, atol=0)
    torch.testing.assert_close(out, torch.from_numpy(g["out2"]), rtol=1e-4, atol=1e-5)


def test_repack_layout_is_a_permutation():
    w = torch.arange(2 * 16 * 256, dtype=torch.int32).remainder(251).to(torch.uint8).reshape(2, 16, 256)
    r = O.repack_weight_ref(w)
    assert r.shape == w.shape
    assert torch.equal(r.reshape(2, -1).sort(dim=1).values, w.reshape(2, -1).sort(dim=1).values)
    # byte (n=9, k=128+40) of batch 1: kb=1, atom=1, r=1, chunk 2 -> stored chunk 3, byte 8
    off = ((1 * 2 + 1) * 8 + 1) * 128 + ((2 ^ 1) << 4) + 8
    assert r[1].reshape(-1)[off] == w[1, 9, 168]


@pytest.mark.skipif(not ref_loader.available(), reason="reference checkout not mounted")
def test_oracle_matches_live_reference():
    ref = ref_loader.load()
    case = O.make_dense_case(19, 320, 256, seed=3)
    want = ref["run_torch_blockscale"](case["a_q"], case["b_q"], case["a_scale"], case["b_scale"],
                                       dtype=torch.bfloat16)
    got = O.run_torch_blockscale(case["a_q"], case["b_q"], case["a_scale"], case["b_scale"])
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    m = O.make_moe_case(T=40, H=256, I=128, E=8, topk=3, seed=2)
    sid, sw, seid, npp = ref["moe_sorting_torch_native"](m["topk_ids"], m["topk_weights"], num_experts=8,
                                                         block_size=32)
    a, b, c, d = O.moe_sorting_ref(m["topk_ids"].numpy(), m["topk_weights"].numpy(), 8, 32)
    n = int(npp[0])
    assert n == int(d[0]) and np.array_equal(sid.numpy(), a) and np.array_equal(seid.numpy(), c)
    keep = a != ((3 << 24) | 40)
    assert np.array_equal(sw.numpy()[keep], b[keep])
    want1 = ref["torch_stage1_blockscale_ref"](m["x_q"], m["w1_q"], m["topk_ids"], m["x_scale"],
                                               m["w1_scale"], (128, 128), 128)
    got1 = O.torch_stage1_blockscale_ref(m["x_q"], m["w1_q"], m["topk_ids"], m["x_scale"], m["w1_scale"], 128)
    torch.testing.assert_close(got1, want1, rtol=1e-5, atol=1e-6)
