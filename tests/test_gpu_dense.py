"""Dense FP8 block-scale GEMM on the GPU, through the reference-shaped Python API (which calls the
C ABI), against the golden vectors and the CPU oracle."""
import pytest
import torch

from oracle import blockscale_ref as O
from tests.helpers import assert_close_to_oracle, bf16_from_bits, fp8_from_u8, load_golden

pytestmark = pytest.mark.gpu


def _run_dense(a_q, a_scale, b_q, b_scale, out_dtype="bf16", block_n=None, tiles=(64, 128, 128), **kw):
    from flydsl_b200 import _lib
    from flydsl_b200.kernels import compile_blockscale_preshuffle_gemm
    from flydsl_b200.utils import shuffle_weight

    dev = torch.device("cuda")
    M, K = a_q.shape
    N = b_q.shape[0]
    fn = compile_blockscale_preshuffle_gemm(M=M, N=N, K=K, tile_m=tiles[0], tile_n=tiles[1], tile_k=tiles[2],
                                            out_dtype=out_dtype, block_n=block_n, **kw)
    tdt = torch.bfloat16 if out_dtype == "bf16" else torch.float16
    c = torch.zeros((M, N), dtype=tdt, device=dev)
    b_sh = shuffle_weight(b_q.to(dev))
    sa_t = a_scale.to(dev).t().contiguous().view(-1)
    sb = b_scale.to(dev).contiguous().view(-1)
    fn(c, a_q.to(dev), b_sh, sa_t, sb, M, N, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert _lib.query_device_error() == 0
    return c


def test_repack_matches_layout_oracle():
    from flydsl_b200.utils import shuffle_weight

    g = torch.Generator().manual_seed(1)
    w = torch.randint(0, 256, (3, 48, 384), generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
    got = shuffle_weight(w.cuda()).cpu()
    want = O.repack_weight_ref(w)
    assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
    assert getattr(shuffle_weight(w.cuda()), "is_shuffled", False)


@pytest.mark.parametrize("tag", ["a", "b", "c", "q"])
@pytest.mark.parametrize("block_n", [None, 32, 64, 128, 256])
def test_dense_vs_golden(tag, block_n):
    g = load_golden("dense.npz")
    x, w = fp8_from_u8(g[f"{tag}_x"]), fp8_from_u8(g[f"{tag}_w"])
    xs, ws = torch.from_numpy(g[f"{tag}_xs"]), torch.from_numpy(g[f"{tag}_ws"])
    c = _run_dense(x, xs, w, ws, block_n=block_n)
    assert_close_to_oracle(c, bf16_from_bits(g[f"{tag}_c_bf16_bits"]), f"golden {tag} bn={block_n}")


# The reference's own test grid (tests/kernels/test_blockscale_preshuffle_gemm.py:121-142): its three
# (N, K) pairs at every small M; the M=1024 rows follow in test_dense_reference_large_rows.
@pytest.mark.parametrize("M", [1, 7, 16, 33, 64, 256])
@pytest.mark.parametrize("N,K", [(7168, 2304), (2112, 7168), (3072, 1536)])
@pytest.mark.parametrize("out_dtype", ["bf16", "fp16"])
def test_dense_reference_shapes(M, N, K, out_dtype):
    case = O.make_dense_case(M, N, K, seed=M + N)
    ref = O.run_torch_blockscale(case["a_q"], case["b_q"], case["a_scale"], case["b_scale"], dtype=torch.float32)
    c = _run_dense(case["a_q"], case["a_scale"], case["b_q"], case["b_scale"], out_dtype=out_dtype)
    assert_close_to_oracle(c, ref, f"M={M} N={N} K={K} {out_dtype}")


# Decode-size M runs on the swap-AB split-K kernel (cluster reduction through distributed shared
# memory); every split factor must give the same answer within tolerance, including K ranges that do
# not divide evenly, N tails and M = 1.
@pytest.mark.parametrize("M,N,K", [(1, 256, 384), (5, 2112, 1024), (32, 1536, 7168), (64, 3072, 1536), (17, 320, 2304)])
@pytest.mark.parametrize("split_k", [None, 1, 2, 3, 8])
def test_decode_path_split_k(M, N, K, split_k):
    case = O.make_dense_case(M, N, K, seed=M * 7 + N)
    ref = O.run_torch_blockscale(case["a_q"], case["b_q"], case["a_scale"], case["b_scale"], dtype=torch.float32)
    c = _run_dense(case["a_q"], case["a_scale"], case["b_q"], case["b_scale"], path="decode", split_k=split_k)
    assert_close_to_oracle(c, ref, f"decode M={M} N={N} K={K} split_k={split_k}")
    c2 = _run_dense(case["a_q"], case["a_scale"], case["b_q"], case["b_scale"], path="decode", split_k=split_k)
    assert torch.equal(c, c2)  # fixed reduction order: bitwise repeatable
    t = _run_dense(case["a_q"], case["a_scale"], case["b_q"], case["b_scale"], path="tiled")
    assert_close_to_oracle(t, ref, f"tiled M={M} N={N} K={K}")


@pytest.mark.parametrize("N,K", [(7168, 2304), (2112, 7168), (3072, 1536)])
def test_dense_reference_large_rows(N, K):
    """The M=1024 rows of the reference grid (its `large_shape` marks)."""
    case = O.make_dense_case(1024, N, K, seed=1024 + N)
    ref = O.run_torch_blockscale(case["a_q"], case["b_q"], case["a_scale"], case["b_scale"], dtype=torch.float32)
    c = _run_dense(case["a_q"], case["a_scale"], case["b_q"], case["b_scale"])
    assert_close_to_oracle(c, ref, f"M=1024 N={N} K={K}")


# The shapes the benchmark sweeps: M in {1, 32, 256, 4096, 16384} x three (N, K) pairs. At M >= 4096
# there are several times more tiles than SMs, so every persistent CTA walks 6-30 tiles back to back
# (staging-tile reuse, accumulator rotation across tile boundaries, next-tile scale prefetch).
SWEEP_NK = [(7168, 2048), (4096, 7168), (24576, 1536)]


@pytest.mark.parametrize("N,K", SWEEP_NK)
@pytest.mark.parametrize("M", [1, 32, 256, 4096])
def test_dense_sweep_shapes_default_heuristic(M, N, K):
    case = O.make_dense_case(M, N, K, seed=M + N + K)
    ref = O.run_torch_blockscale(case["a_q"], case["b_q"], case["a_scale"], case["b_scale"], dtype=torch.float32)
    c = _run_dense(case["a_q"], case["a_scale"], case["b_q"], case["b_scale"])
    assert_close_to_oracle(c, ref, f"sweep M={M} N={N} K={K}")
    if M <= 32:   # the same shape through the tiled kernel
        t = _run_dense(case["a_q"], case["a_scale"], case["b_q"], case["b_scale"], path="tiled")
        assert_close_to_oracle(t, ref, f"sweep tiled M={M} N={N} K={K}")


@pytest.mark.parametrize("M,N,K,block_n", [(4096, 7168, 2048, 256), (4096, 7168, 2048, 128), (4096, 4096, 7168, 256),
                                           (16384, 7168, 2048, None), (16384, 7168, 2048, 256),
                                           (4096 + 77, 7168, 2048, 256), (4096, 7168 - 48, 2048, None)])
def test_dense_many_tiles_per_cta(M, N, K, block_n):
    """Headline shape and its neighbours with the tile width forced, plus ragged M and N: every CTA
    processes many tiles; run twice, results must be bitwise repeatable."""
    case = O.make_dense_case(M, N, K, seed=3)
    ref = O.run_torch_blockscale(case["a_q"], case["b_q"], case["a_scale"], case["b_scale"], dtype=torch.float32)
    c = _run_dense(case["a_q"], case["a_scale"], case["b_q"], case["b_scale"], block_n=block_n)
    assert_close_to_oracle(c, ref, f"M={M} N={N} K={K} bn={block_n}")
    c2 = _run_dense(case["a_q"], case["a_scale"], case["b_q"], case["b_scale"], block_n=block_n)
    assert torch.equal(c, c2)


def test_dense_accepts_parameter_tensors():
    """Tensor subclasses such as nn.Parameter are taken like plain tensors (the reference's
    tests/unit/test_jit_stream_param.py:101-175 passes them to its launchers)."""
    from flydsl_b200.kernels import compile_blockscale_preshuffle_gemm
    from flydsl_b200.utils import shuffle_weight

    M, N, K = 48, 512, 1024
    case = O.make_dense_case(M, N, K, seed=8)
    ref = O.run_torch_blockscale(case["a_q"], case["b_q"], case["a_scale"], case["b_scale"], dtype=torch.float32)
    dev = torch.device("cuda")
    w = torch.nn.Parameter(shuffle_weight(case["b_q"].to(dev)), requires_grad=False)
    sb = torch.nn.Parameter(case["b_scale"].to(dev).contiguous().view(-1), requires_grad=False)
    fn = compile_blockscale_preshuffle_gemm(M=M, N=N, K=K, tile_m=64, tile_n=128, tile_k=128)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    fn(c, case["a_q"].to(dev), w, case["a_scale"].to(dev).t().contiguous().view(-1), sb, M, N, None)
    torch.cuda.synchronize()
    assert_close_to_oracle(c, ref, "nn.Parameter operands")


def test_dense_config1_and_m_tail():
    for (M, N, K) in [(128, 1536, 7168), (1024 + 5, 1536, 512)]:
        case = O.make_dense_case(M, N, K, seed=0)
        ref = O.run_torch_blockscale(case["a_q"], case["b_q"], case["a_scale"], case["b_scale"], dtype=torch.float32)
        for bn in (None, 256):
            c = _run_dense(case["a_q"], case["a_scale"], case["b_q"], case["b_scale"], block_n=bn)
            assert_close_to_oracle(c, ref, f"M={M} N={N} K={K} bn={bn}")


def test_dense_is_deterministic_and_stream_forms():
    from flydsl_b200.kernels import compile_blockscale_preshuffle_gemm
    from flydsl_b200.utils import shuffle_weight
    import flydsl_b200 as flyc

    case = O.make_dense_case(96, 512, 1024, seed=5)
    dev = torch.device("cuda")
    fn = compile_blockscale_preshuffle_gemm(M=96, N=512, K=1024, tile_m=32, tile_n=128, tile_k=128)
    a, b = case["a_q"].to(dev), shuffle_weight(case["b_q"].to(dev))
    sa, sb = case["a_scale"].to(dev).t().contiguous().view(-1), case["b_scale"].to(dev).view(-1)
    outs = []
    side = torch.cuda.Stream()
    for stream in (None, torch.cuda.current_stream(), torch.cuda.current_stream().cuda_stream, side):
        c = torch.zeros((96, 512), dtype=torch.bfloat16, device=dev)
        if stream is side:
            side.wait_stream(torch.cuda.current_stream())
        fn(c, a, b, sa, sb, 96, 512, stream)
        torch.cuda.synchronize()
        outs.append(c)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    # flyc.compile-style pre-binding and CUDA-graph capture, as the reference's tests exercise
    c = torch.zeros((96, 512), dtype=torch.bfloat16, device=dev)
    exe = flyc.compile(fn, c, a, b, sa, sb, 96, 512, torch.cuda.current_stream())
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    c.zero_()
    with torch.cuda.graph(graph):
        exe(c, a, b, sa, sb, 96, 512, torch.cuda.current_stream())
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(c, outs[0])


def test_dense_bad_arguments_raise():
    from flydsl_b200.kernels import compile_blockscale_preshuffle_gemm

    with pytest.raises(ValueError):
        compile_blockscale_preshuffle_gemm(M=8, N=128, K=256, tile_m=16, tile_n=64, tile_k=128, out_dtype="f32")
    with pytest.raises(ValueError):
        compile_blockscale_preshuffle_gemm(M=8, N=128, K=200, tile_m=16, tile_n=64, tile_k=128)
    fn = compile_blockscale_preshuffle_gemm(M=8, N=128, K=256, tile_m=16, tile_n=64, tile_k=128)
    z = torch.zeros(8 * 256, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):  # misaligned output pointer is rejected by the C ABI, nothing launches
        fn(z[1:], z, z, z.view(torch.float32), z.view(torch.float32), 8, 128, None)


def test_autotuner_picks_a_valid_configuration(tmp_path):
    """The tuner benchmarks its candidates on the GPU, caches the winner and the tuned launcher
    still matches the oracle."""
    from flydsl_b200.autotune import GemmAutotuner
    from flydsl_b200.utils import shuffle_weight

    DEV = torch.device("cuda")
    M, N, K = 48, 1536, 1024
    tuner = GemmAutotuner(cache_dir=str(tmp_path), warmup=2, rep=5)
    cfg = tuner.tune(M, N, K)
    assert len(tuner.timings[tuner.key(M, N, K)]) >= 4          # several candidates really ran
    assert (tmp_path / "blockscale_gemm.json").exists()
    d = O.make_dense_case(M, N, K, seed=5)
    ref = O.run_torch_blockscale(d["a_q"], d["b_q"], d["a_scale"], d["b_scale"], dtype=torch.float32)
    fn = tuner.tuned_gemm(M=M, N=N, K=K)
    c = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    fn(c, d["a_q"].to(DEV), shuffle_weight(d["b_q"].to(DEV)), d["a_scale"].to(DEV).t().contiguous(),
       d["b_scale"].to(DEV), M, N, None)
    torch.cuda.synchronize()
    assert_close_to_oracle(c, ref, f"tuned {cfg}")


@pytest.mark.parametrize("M,N,K,block_n", [(4500, 512, 12288, None), (4500, 512, 12288, 128), (7000, 768, 7168, 256)])
def test_dense_grouped_tile_order_with_a_short_last_group(M, N, K, block_n):
    """Shapes with enough row blocks for the grouped tile order (groups of 16 / 26 row blocks here),
    M chosen so that the last group is shorter than the others and the last row block is partial."""
    case = O.make_dense_case(M, N, K, seed=M)
    ref = O.run_torch_blockscale(case["a_q"], case["b_q"], case["a_scale"], case["b_scale"], dtype=torch.float32)
    c = _run_dense(case["a_q"], case["a_scale"], case["b_q"], case["b_scale"], block_n=block_n)
    assert_close_to_oracle(c, ref, f"grouped order M={M} N={N} K={K} bn={block_n}")
