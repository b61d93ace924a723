"""Shared helpers for the tests: golden loading and tolerance checks."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FP8 = torch.float8_e4m3fn

# Parity bar for floating-point outputs (bf16/fp16 results against the fp32 oracle).
MAX_REL = 1e-2
MIN_COS = 0.9999


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name)))


def fp8_from_u8(arr):
    return torch.from_numpy(np.ascontiguousarray(arr)).view(FP8)


def bf16_from_bits(arr):
    return torch.from_numpy(np.ascontiguousarray(arr)).view(torch.bfloat16)


def assert_close_to_oracle(out, ref, what=""):
    from oracle.blockscale_ref import cosine, max_rel_err

    out, ref = out.detach().float().cpu(), ref.detach().float().cpu()
    assert torch.isfinite(out).all(), f"{what}: non-finite output"
    mr, cs = max_rel_err(out, ref), cosine(out, ref)
    assert mr <= MAX_REL and cs >= MIN_COS, f"{what}: max_rel={mr:.3e} (<= {MAX_REL}), cosine={cs:.6f} (>= {MIN_COS})"
    return mr, cs
