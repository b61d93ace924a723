"""CPU-side checks of the boundary: the shared library loads and exports exactly the symbols the
header declares, factories validate like the reference, and nothing computes without a GPU."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "flyb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(flyb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as entry
    from flydsl_b200 import _lib

    entry.build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    declared = _header_symbols()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/flyb200.h but not exported"
    assert sorted(_lib.SIGNATURES) == declared, "ctypes table and header disagree"
    assert lib.flyb200_version() >= 100


def test_dense_factory_validation_matches_reference_rules():
    from flydsl_b200.kernels import compile_blockscale_preshuffle_gemm as f

    ok = dict(M=16, N=256, K=512, tile_m=16, tile_n=64, tile_k=128)
    for bad in (dict(out_dtype="f32"), dict(tile_k=192), dict(K=520), dict(tile_k=64, scale_block_k=64),
                dict(tile_m=3, tile_k=128), dict(N=200), dict(block_n=48)):
        with pytest.raises(ValueError):
            f(**{**ok, **bad})


def test_moe_factory_validation_and_cache():
    from flydsl_b200.kernels import (MoeGemm2Mode, compile_moe_blockscale_gemm1, compile_moe_blockscale_gemm2,
                                     compile_moe_blockscale_gemm2_ex, compile_moe_reduction)

    kw = dict(model_dim=256, inter_dim=128, experts=4, topk=2, tile_m=16, tile_n=256, tile_k=128)
    with pytest.raises(ValueError):
        compile_moe_blockscale_gemm1(doweight_stage1=False, out_dtype="f32", **kw)
    with pytest.raises(ValueError):
        compile_moe_blockscale_gemm2(doweight_stage2=True, out_dtype="f32", accumulate=False, **kw)
    with pytest.raises(ValueError):
        compile_moe_blockscale_gemm2(doweight_stage2=True, **{**kw, "inter_dim": 100})
    with pytest.raises(ValueError):
        compile_moe_blockscale_gemm2(doweight_stage2=True, **{**kw, "tile_m": 256})
    with pytest.raises(ValueError):
        compile_moe_blockscale_gemm2_ex(doweight_stage2=True, in_dtype="int8", **kw)
    a = compile_moe_blockscale_gemm1(doweight_stage1=False, **kw)
    assert a is compile_moe_blockscale_gemm1(doweight_stage1=False, **kw)  # lru_cache like the reference
    ex = compile_moe_blockscale_gemm2_ex(doweight_stage2=True, mode=MoeGemm2Mode.REDUCE, out_dtype="bf16", **kw)
    assert ex.mode == "reduce"
    assert compile_moe_reduction(topk=2, model_dim=256, dtype_str="bf16").topk == 2


def test_no_cpu_fallback():
    from flydsl_b200.utils import pertoken_quant, shuffle_weight

    w = torch.zeros(16, 128, dtype=torch.uint8).view(torch.float8_e4m3fn)
    with pytest.raises(ValueError):
        shuffle_weight(w)  # CPU tensor: refused, never computed on the host
    q, s = pertoken_quant(torch.tensor([[0.0, 0.0], [1.0, -2.0]]), quant_dtype=torch.float8_e4m3fn)
    assert s.flatten().tolist() == [1.0, (torch.tensor(2.0) / 448.0).item()]


def test_stream_handle_forms():
    from flydsl_b200 import _lib

    assert _lib.stream_handle(1234) == 1234
    with pytest.raises(TypeError):
        _lib.stream_handle("nope")
