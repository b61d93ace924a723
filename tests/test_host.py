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


def test_autotuner_keys_cache_and_persistence(tmp_path):
    """Autotuner host logic without a GPU: a fake benchmark decides, the choice is cached per
    (device, M bucket, N, K, dtype) and survives a new tuner object through the JSON file."""
    from flydsl_b200.autotune import Config, GemmAutotuner, default_configs, m_bucket

    assert [m_bucket(m) for m in (1, 2, 3, 32, 33, 4096)] == [1, 2, 4, 32, 64, 4096]
    calls = []

    def fake_bench(call, warmup, rep):
        return call()

    def make_call(cfg):
        if cfg.block_n == 32:
            raise ValueError("not valid for this shape")
        calls.append(cfg)
        cost = {None: 5.0, 256: 2.0, 128: 3.0, 64: 4.0}[cfg.block_n]
        return lambda: cost

    t = GemmAutotuner(cache_dir=str(tmp_path), do_bench_fn=fake_bench, device_name="fake")
    best = t.tune(4096, 7168, 2048, make_call=make_call)
    assert best == Config(block_n=256, path="tiled")
    n = len(calls)
    assert t.tune(3000, 7168, 2048, make_call=make_call) == best and len(calls) == n   # same bucket: cached
    t.tune(100, 7168, 2048, make_call=make_call)
    assert len(calls) > n                                                              # other bucket: tuned
    t2 = GemmAutotuner(cache_dir=str(tmp_path), do_bench_fn=fake_bench, device_name="fake")
    assert t2.tune(4096, 7168, 2048, make_call=lambda cfg: (_ for _ in ()).throw(AssertionError)) == best
    assert any(c.path == "decode" for c in default_configs(16, 7168, 2048))
    assert all(c.path != "decode" for c in default_configs(4096, 7168, 2048))


def test_c_abi_refuses_bad_sizes_before_any_launch():
    """Argument checks that protect vector accesses run on the host before anything is launched, so
    they can be exercised without a GPU: a non-NULL dummy pointer is enough."""
    from flydsl_b200 import _lib

    lib = _lib.load()
    buf = (ctypes.c_ubyte * 4096)()
    base = ctypes.addressof(buf)
    p16 = (base + 15) // 16 * 16
    peers = (ctypes.c_void_p * 2)(p16, p16)
    inval = _lib.ERR_INVALID_ARGUMENT
    # packed expert-parallel row = H + 4*(H/128) + 8*k bytes, copied as 16-byte vectors: H=640 gives
    # 640 + 20 + 32 = 692 bytes, not a multiple of 16
    assert lib.flyb200_ep_push(p16, p16, p16, p16, 4, 640, 4, 2, 0, 4, peers, 0, p16, p16, p16, None) == inval
    assert b"multiple of 16" in lib.flyb200_last_error_string()
    assert lib.flyb200_ep_plan_pack(p16, p16, p16, p16, 4, 640, 4, 2, 4, p16, p16, p16, p16, None) == inval
    assert lib.flyb200_ep_gather_packed(p16, p16, p16, p16, p16, 4, 4, 640, 4, None) == inval
    # the 16-bit quantiser stores 8 bytes at a time: q at 8k+4 is refused
    assert lib.flyb200_quant_1x128(p16, p16 + 4, p16, 2, 128, _lib.BF16, None) == inval
    assert lib.flyb200_quant_1x128_devrows(p16, p16 + 4, p16, p16, 2, 128, _lib.BF16, None) == inval
    # more routes per token than experts would overrun the reference-sized sort buffers
    assert lib.flyb200_moe_sort(p16, p16, 4, 9, 8, 16, None, -1, p16, p16, p16, p16, None) == inval
    assert b"k <= E" in lib.flyb200_last_error_string()
    # the whole-row quantiser reads 16 bytes and writes 8 at a time
    assert lib.flyb200_quant_pertoken(p16, p16 + 4, p16, None, 2, 128, _lib.F16, None) == inval
    assert lib.flyb200_quant_pertoken(p16, p16, p16, None, 2, 132, _lib.F16, None) == inval
    assert lib.flyb200_quant_pertoken(p16, p16, p16, None, 2, 128, _lib.F32, None) == inval
    assert lib.flyb200_moe_gather_rows_pertoken(p16, p16, p16, p16, p16 + 8, p16, 4, 128, 2, 8, 0, None) == inval
    assert lib.flyb200_moe_gather_rows_pertoken(p16, None, p16, p16, p16, p16, 4, 128, 2, 8, 0, None) == inval


def test_pertoken_moe_entries_refuse_bad_arguments_before_any_launch():
    from flydsl_b200 import _lib

    lib = _lib.load()
    buf = (ctypes.c_ubyte * 4096)()
    p16 = (ctypes.addressof(buf) + 15) // 16 * 16
    inval = _lib.ERR_INVALID_ARGUMENT
    ptrs = [p16] * 9
    # T, I/H, H/I, blocks, E, k, tile_m, doweight, out_dtype
    ok1 = [4, 128, 256, 1, 4, 2, 16, 0, _lib.F16]
    cfg = _lib.GemmCfg(128, 0, 0, 0)   # the per-token stages are built for 256-wide tiles only
    assert lib.flyb200_moe_gemm1_pertoken(*ptrs, *ok1, ctypes.byref(cfg), None) == inval
    assert b"block_n 256" in lib.flyb200_last_error_string()
    bad_k = list(ok1); bad_k[5] = 9    # more routes per token than experts
    assert lib.flyb200_moe_gemm1_pertoken(*ptrs, *bad_k, None, None) == inval
    bad_dim = list(ok1); bad_dim[1] = 96
    assert lib.flyb200_moe_gemm1_pertoken(*ptrs, *bad_dim, None, None) == inval
    ok2 = [4, 256, 128, 1, 4, 2, 16, 1, 0, _lib.BF16]    # ..., doweight, accumulate, out_dtype
    assert lib.flyb200_moe_gemm2_pertoken(*ptrs, *ok2, ctypes.byref(cfg), None) == inval
    bad_tile = list(ok2); bad_tile[6] = 129
    assert lib.flyb200_moe_gemm2_pertoken(*ptrs, *bad_tile, None, None) == inval
    # reduce mode: the workspace must be there, aligned and large enough
    red = [p16] * 10 + [4, 256, 128, 1, 4, 2, 16, 1, _lib.BF16]
    assert lib.flyb200_moe_gemm2_reduce_pertoken(*red, None, None, 0, 1, None) == inval
    assert lib.flyb200_moe_gemm2_reduce_pertoken(*red, None, p16, 16, 1, None) == _lib.ERR_WORKSPACE
    assert lib.flyb200_moe_gemm2_reduce_pertoken(*red[:18], _lib.F32, None, p16, 1 << 20, 1, None) == inval
