"""Generate the golden fixtures in this directory by running the REFERENCE project's own torch
functions (loaded unmodified from a checkout by oracle/ref_loader.py) on small seeded inputs.

    python tests/golden/make_golden.py [--root /path/to/FlyDSL]

The fixtures pin the CPU oracle (tests/test_oracle.py) and are also compared directly with the CUDA
kernels (tests/test_gpu_*.py). fp8 tensors are stored as their uint8 bytes, bf16 as uint16 bits.
The reference checkout is needed only to run this script, never at test time.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import ref_loader  # noqa: E402

FP8 = torch.float8_e4m3fn


def u8(t):
    return t.contiguous().view(torch.uint8).numpy()


def bits16(t):
    return t.contiguous().view(torch.int16).numpy()


def dense_cases(ref):
    out = {}
    # (M, N, K): M below / not a multiple of the tile, N not a multiple of 128 (half scale block).
    for tag, (M, N, K) in {"a": (33, 384, 256), "b": (7, 320, 384), "c": (130, 128, 128)}.items():
        g = torch.Generator().manual_seed(100 + len(out))
        # the reference test's recipe: positive rand/10 operands, rand scales (:184-188)
        x = (torch.rand((M, K), generator=g, dtype=torch.float32) / 10).to(torch.float16).to(FP8)
        w = (torch.rand((N, K), generator=g, dtype=torch.float32) / 10).to(torch.float16).to(FP8)
        sk, sn = K // 128, (N + 127) // 128
        xs = torch.rand((M, sk), generator=g, dtype=torch.float32)
        ws = torch.rand((sn, sk), generator=g, dtype=torch.float32)
        c32 = ref["run_torch_blockscale"](x, w, xs, ws, dtype=torch.float32)
        c16 = ref["run_torch_blockscale"](x, w, xs, ws, dtype=torch.bfloat16)
        out.update({f"{tag}_x": u8(x), f"{tag}_w": u8(w), f"{tag}_xs": xs.numpy(), f"{tag}_ws": ws.numpy(),
                    f"{tag}_c_f32": c32.numpy(), f"{tag}_c_bf16_bits": bits16(c16)})
    # signed operands (A ~ N(0,1), B ~ N(0,0.02)) quantised through the reference's pertoken_quant
    g = torch.Generator().manual_seed(7)
    M, N, K = 48, 256, 512
    a = torch.randn(M, K, generator=g)
    b = torch.randn(N, K, generator=g) * 0.02
    aq, asc = ref["pertoken_quant"](a.view(-1, 128), quant_dtype=FP8)
    aq, asc = aq.view(M, K), asc.view(M, K // 128)
    rows = b.view(N // 128, 128, K // 128, 128).permute(0, 2, 1, 3).reshape(-1, 128 * 128)
    bq, bsc = ref["pertoken_quant"](rows, quant_dtype=FP8)
    bq = bq.view(N // 128, K // 128, 128, 128).permute(0, 2, 1, 3).reshape(N, K)
    bsc = bsc.view(N // 128, K // 128)
    c16 = ref["run_torch_blockscale"](aq, bq, asc, bsc, dtype=torch.bfloat16)
    out.update({"q_a_f32": a.numpy(), "q_b_f32": b.numpy(), "q_x": u8(aq), "q_w": u8(bq),
                "q_xs": asc.numpy(), "q_ws": bsc.numpy(), "q_c_bf16_bits": bits16(c16)})
    return out


def pertoken_cases(ref):
    """Per-token / per-channel scaled GEMM: the reference test's recipe (rand operands quantised by
    pertoken_quant, tests/kernels/test_preshuffle_gemm.py:141-180) and its run_torch."""
    out = {}
    for tag, (M, N, K) in {"a": (33, 320, 256), "b": (5, 128, 384)}.items():
        g = torch.Generator().manual_seed(200 + len(out))
        a = torch.rand(M, K, generator=g)
        b = torch.rand(N, K, generator=g)
        aq, sa = ref["pertoken_quant"](a, quant_dtype=FP8)
        bq, sb = ref["pertoken_quant"](b, quant_dtype=FP8)
        c32 = ref["run_torch"](aq, bq, sa, sb, bias=None, dtype=torch.float32)
        out.update({f"{tag}_a": u8(aq), f"{tag}_b": u8(bq), f"{tag}_sa": sa.reshape(-1).numpy(),
                    f"{tag}_sb": sb.reshape(-1).numpy(), f"{tag}_c_f32": c32.numpy()})
    return out


def sort_cases(ref):
    out = {}
    cases = {
        "s0": dict(T=37, k=3, E=8, bs=16, mask=None, nlt=None),
        "s1": dict(T=5, k=2, E=16, bs=32, mask=None, nlt=None),          # many empty experts
        "s2": dict(T=64, k=4, E=8, bs=16, mask=[1, 0, 1, 1, 0, 1, 1, 1], nlt=None),
        "s3": dict(T=40, k=2, E=4, bs=8, mask=None, nlt=29),
        "s4": dict(T=300, k=8, E=32, bs=128, mask=None, nlt=None),
    }
    for tag, c in cases.items():
        g = torch.Generator().manual_seed(11 + int(tag[1:]))
        score = torch.rand((c["T"], c["E"]), generator=g)
        vals, ids = torch.topk(score, k=c["k"], dim=1)
        w = torch.softmax(vals, dim=1).float()
        mask = None if c["mask"] is None else torch.tensor(c["mask"], dtype=torch.int32)
        nlt = None if c["nlt"] is None else torch.tensor(c["nlt"])
        sid, sw, seid, npp = ref["moe_sorting_torch_native"](
            ids.to(torch.int32), w, num_experts=c["E"], block_size=c["bs"], expert_mask=mask,
            num_local_tokens=nlt)
        sentinel = (c["k"] << 24) | c["T"]
        sw = torch.where(sid == sentinel, torch.zeros_like(sw), sw)  # reference leaves padding unset
        out.update({f"{tag}_ids": ids.to(torch.int32).numpy(), f"{tag}_w": w.numpy(),
                    f"{tag}_cfg": np.array([c["T"], c["k"], c["E"], c["bs"],
                                            -1 if c["nlt"] is None else c["nlt"]], dtype=np.int32),
                    f"{tag}_mask": np.array(c["mask"] if c["mask"] is not None else [], dtype=np.int32),
                    f"{tag}_sorted_ids": sid.numpy(), f"{tag}_sorted_w": sw.numpy(),
                    f"{tag}_expert_ids": seid.numpy(), f"{tag}_post_pad": npp.numpy()})
    return out


def moe_case(ref):
    T, H, I, E, k = 24, 256, 128, 4, 2
    g = torch.Generator().manual_seed(5)
    s = 0.2  # the reference test's magnitudes (:223, :245, :251)
    x = torch.randn(T, H, generator=g) * s
    xq, xs = ref["pertoken_quant"](x.view(-1, 128), quant_dtype=FP8)
    xq, xs = xq.view(T, H), xs.view(T, H // 128)
    score = torch.rand(T, E, generator=g)
    vals, ids = torch.topk(score, k=k, dim=1)
    tw = torch.softmax(vals, dim=1).float()

    def bq(w):
        n, kk = w.shape
        rows = w.view(n // 128, 128, kk // 128, 128).permute(0, 2, 1, 3).reshape(-1, 128 * 128)
        q, sc = ref["pertoken_quant"](rows, quant_dtype=FP8)
        return q.view(n // 128, kk // 128, 128, 128).permute(0, 2, 1, 3).reshape(n, kk), sc.view(-1)

    w1 = [bq(torch.randn(2 * I, H, generator=g) * s) for _ in range(E)]
    w2 = [bq(torch.randn(H, I, generator=g) * (s / I ** 0.5)) for _ in range(E)]
    w1q, w1s = torch.stack([a for a, _ in w1]), torch.stack([b for _, b in w1])
    w2q, w2s = torch.stack([a for a, _ in w2]), torch.stack([b for _, b in w2])
    out1 = ref["torch_stage1_blockscale_ref"](xq, w1q, ids, xs, w1s, (128, 128), I)
    a2q, a2s = ref["pertoken_quant"](out1.to(torch.float16).float().view(-1, I // 128, 128), quant_dtype=FP8)
    a2q, a2s = a2q.view(-1, I), a2s.squeeze(-1)
    out2 = ref["torch_stage2_blockscale_ref"](a2q, w2q, ids, tw, a2s, w2s, (128, 128), T, H, I, k)
    fused = ref["torch_moe_blockscale_ref"](xq, w1q, w2q, tw, ids, torch.float32, scale_blks=(128, 128),
                                            a_scale=xs, fc1_scale=w1s, fc2_scale=w2s)
    return {"cfg": np.array([T, H, I, E, k], dtype=np.int32), "x_q": u8(xq), "x_scale": xs.numpy(),
            "topk_ids": ids.to(torch.int32).numpy(), "topk_w": tw.numpy(),
            "w1_q": u8(w1q), "w1_scale": w1s.numpy(), "w2_q": u8(w2q), "w2_scale": w2s.numpy(),
            "out1": out1.numpy(), "a2_q": u8(a2q), "a2_scale": a2s.numpy(), "out2": out2.numpy(),
            "fused": fused.numpy()}


def moe_pertoken_case(ref):
    """Per-token-scale MoE, both stages, with the reference test's recipe
    (tests/kernels/test_moe_gemm.py:1236-1300: randn * 0.2 operands quantised by pertoken_quant, rand
    scores, stage-1 output rounded to fp16 and re-quantised per route) and its torch_moe_gemm1 /
    torch_moe_gemm2 (tests/kernels/test_ref.py)."""
    T, H, I, E, k = 24, 256, 128, 4, 2
    g = torch.Generator().manual_seed(11)
    s = 0.2
    x = torch.randn(T, H, generator=g) * s
    w1 = torch.randn(E, 2 * I, H, generator=g) * s
    w2 = torch.randn(E, H, I, generator=g) * (s / I ** 0.5)
    score = torch.rand(T, E, generator=g)
    vals, ids = torch.topk(score, k=k, dim=1)
    tw = torch.softmax(vals, dim=1).float()
    xq, xs = ref["pertoken_quant"](x, quant_dtype=FP8)
    w1q, w1s = ref["pertoken_quant"](w1, quant_dtype=FP8)
    w2q, w2s = ref["pertoken_quant"](w2, quant_dtype=FP8)
    ids64 = ids.to(torch.int64)
    out1 = ref["torch_moe_gemm1"](xq, w1q.view(E * 2 * I, H), xs, w1s.view(E * 2 * I, 1), ids64, tw,
                                  inter_dim=I, doweight_stage1=False)
    out1w = ref["torch_moe_gemm1"](xq, w1q.view(E * 2 * I, H), xs, w1s.view(E * 2 * I, 1), ids64, tw,
                                   inter_dim=I, doweight_stage1=True)
    a2q, a2s = ref["pertoken_quant"](out1.to(torch.float16).float(), quant_dtype=FP8)
    out2 = ref["torch_moe_gemm2"](a2q, w2q, a2s, w2s, ids64, tw, model_dim=H, doweight_stage2=True)
    out2n = ref["torch_moe_gemm2"](a2q, w2q, a2s, w2s, ids64, tw, model_dim=H, doweight_stage2=False)
    return {"cfg": np.array([T, H, I, E, k], dtype=np.int32), "x_q": u8(xq), "x_scale": xs.reshape(-1).numpy(),
            "topk_ids": ids.to(torch.int32).numpy(), "topk_w": tw.numpy(),
            "w1_q": u8(w1q), "w1_scale": w1s.reshape(-1).numpy(), "w2_q": u8(w2q),
            "w2_scale": w2s.reshape(-1).numpy(), "out1": out1.numpy(), "out1_weighted": out1w.numpy(),
            "a2_q": u8(a2q), "a2_scale": a2s.reshape(-1).numpy(), "out2": out2.numpy(),
            "out2_unweighted": out2n.numpy()}


def quant_case(ref):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(20, 128, generator=g) * 3
    x[3] = 0.0                      # all-zero row -> scale 1
    x[5, 7] = float("inf")
    x[6, 9] = float("nan")
    x[8] *= 1e-6                    # tiny values: flush towards 0 in fp8
    q, s = ref["pertoken_quant"](x, quant_dtype=FP8)
    return {"x": x.numpy(), "q": u8(q), "scale": s.numpy()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--root", default=ref_loader.DEFAULT_ROOT)
    a = ap.parse_args()
    if not ref_loader.available(a.root):
        sys.exit(f"reference checkout not found under {a.root}")
    ref = ref_loader.load(a.root)
    torch.set_num_threads(max(1, min(8, os.cpu_count() or 1)))
    np.savez_compressed(os.path.join(HERE, "dense.npz"), **dense_cases(ref))
    np.savez_compressed(os.path.join(HERE, "sort.npz"), **sort_cases(ref))
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **moe_case(ref))
    np.savez_compressed(os.path.join(HERE, "quant.npz"), **quant_case(ref))
    np.savez_compressed(os.path.join(HERE, "pertoken.npz"), **pertoken_cases(ref))
    np.savez_compressed(os.path.join(HERE, "moe_pertoken.npz"), **moe_pertoken_case(ref))
    for f in ("dense.npz", "sort.npz", "moe.npz", "quant.npz", "pertoken.npz", "moe_pertoken.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
