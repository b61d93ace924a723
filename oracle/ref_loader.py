"""Load the reference project's own torch oracle functions, unmodified, from a checkout.

TEST INFRASTRUCTURE ONLY (used by tests/golden/make_golden.py and, when a checkout is present, by
tests/test_oracle.py). The reference's hot-path oracles live in test modules that import the AMD
toolchain at the top, so the modules cannot be imported; instead the wanted ``def`` blocks are cut
out of the source text with ``ast`` and executed in a namespace that only holds torch. No reference
source is stored in this repository.
"""
from __future__ import annotations

import ast
import math
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

# a FlyDSL checkout: $FLYDSL_REFERENCE_ROOT, else a directory "reference" beside this repository
DEFAULT_ROOT = os.environ.get("FLYDSL_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")

_WANTED = {
    "tests/kernels/test_blockscale_preshuffle_gemm.py": ["select_tile_config", "run_torch_blockscale"],
    "tests/kernels/test_moe_blockscale.py": ["_expand_blockscale", "torch_stage1_blockscale_ref",
                                             "torch_stage2_blockscale_ref", "torch_moe_blockscale_ref"],
    "tests/kernels/test_moe_gemm.py": ["moe_sorting_torch_native"],
    "tests/kernels/test_preshuffle_gemm.py": ["run_torch"],
    "tests/kernels/test_ref.py": ["torch_moe_gemm1", "torch_moe_gemm2"],
    "tests/utils.py": ["get_dtype_max", "pertoken_quant", "shuffle_weight"],
}


def available(root: str = DEFAULT_ROOT) -> bool:
    return all(os.path.exists(os.path.join(root, rel)) for rel in _WANTED)


class _Dtypes:
    fp32 = torch.float32
    i8 = torch.int8
    fp8 = torch.float8_e4m3fn


def load(root: str = DEFAULT_ROOT) -> dict:
    """Return {function name: callable} for the reference oracle functions."""
    ns = {"torch": torch, "F": F, "math": math, "Optional": Optional, "Tuple": Tuple,
          "BLOCK_SHAPE": (128, 128), "dtypes": _Dtypes}
    for rel, names in _WANTED.items():
        path = os.path.join(root, rel)
        src = open(path, "r", encoding="utf-8").read()
        tree = ast.parse(src)
        for node in tree.body:
            if isinstance(node, ast.FunctionDef) and node.name in names:
                node.decorator_list = []
                seg = ast.get_source_segment(src, node)
                if node.name == "moe_sorting_torch_native":
                    # the only edit: its device assertion (CPU tensors are used here)
                    seg = seg.replace("assert topk_ids.is_cuda and topk_weights.is_cuda", "pass")
                if node.name in ("torch_moe_gemm1", "torch_moe_gemm2"):
                    # the same kind of edit: they allocate their result on "cuda" and assert CUDA inputs
                    seg = seg.replace('device="cuda"', 'device="cpu"')
                    seg = seg.replace("assert a2_fp8.is_cuda and w2_fp8.is_cuda", "pass")
                # strip decorators that sit above the def in the source segment
                seg = seg[seg.index("def "):]
                exec(compile(seg, path, "exec"), ns)  # noqa: S102 - trusted local checkout, test only
    return {n: ns[n] for names in _WANTED.values() for n in names if n in ns}
