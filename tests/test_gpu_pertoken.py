"""Dense FP8 GEMM with per-token / per-channel scales on the GPU, through the reference-shaped Python
API (which calls the C ABI), against the golden vectors and the CPU oracle."""
import pytest
import torch

from oracle import blockscale_ref as O
from tests.helpers import assert_close_to_oracle, fp8_from_u8, load_golden

pytestmark = pytest.mark.gpu


def _run(a_q, sa, b_q, sb, out_dtype="bf16", stream=None, path="auto"):
    from flydsl_b200 import _lib
    from flydsl_b200.kernels import compile_preshuffle_gemm_a8
    from flydsl_b200.utils import shuffle_weight

    dev = torch.device("cuda")
    M, K = a_q.shape
    N = b_q.shape[0]
    fn = compile_preshuffle_gemm_a8(M=M, N=N, K=K, tile_m=64, tile_n=256, tile_k=128, in_dtype="fp8",
                                    out_dtype=out_dtype, path=path)
    tdt = torch.bfloat16 if out_dtype == "bf16" else torch.float16
    c = torch.zeros((M, N), dtype=tdt, device=dev)
    fn(c, a_q.to(dev), shuffle_weight(b_q.to(dev)), sa.to(dev).contiguous().view(-1),
       sb.to(dev).contiguous().view(-1), M, N, stream)
    torch.cuda.synchronize()
    assert _lib.query_device_error() == 0
    return c


def _case(M, N, K, seed):
    """The reference test's recipe (tests/kernels/test_preshuffle_gemm.py:141-160): rand operands
    quantised per row."""
    g = torch.Generator().manual_seed(seed)
    a_q, sa = O.pertoken_quant(torch.rand(M, K, generator=g))
    b_q, sb = O.pertoken_quant(torch.rand(N, K, generator=g))
    return a_q, sa.view(-1), b_q, sb.view(-1)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_pertoken_vs_golden(tag):
    g = load_golden("pertoken.npz")
    a, b = fp8_from_u8(g[f"{tag}_a"]), fp8_from_u8(g[f"{tag}_b"])
    sa, sb = torch.from_numpy(g[f"{tag}_sa"]), torch.from_numpy(g[f"{tag}_sb"])
    want = torch.from_numpy(g[f"{tag}_c_f32"])
    for dt in ("bf16", "fp16"):
        assert_close_to_oracle(_run(a, sa, b, sb, out_dtype=dt), want, f"golden {tag} {dt}")


# The reference's own test grid (tests/kernels/test_preshuffle_gemm.py:70-80), its large shapes with
# M cut to a few row blocks (the CPU oracle has to finish in seconds), plus row and column tails.
@pytest.mark.parametrize("M,N,K", [(16, 5120, 8192), (33, 1024, 2048), (300, 5120, 8320), (261, 2048, 8320),
                                   (1, 16, 128), (129, 272, 256), (640, 7168, 2048)])
@pytest.mark.parametrize("out_dtype", ["bf16", "fp16"])
def test_pertoken_reference_shapes(M, N, K, out_dtype):
    a_q, sa, b_q, sb = _case(M, N, K, seed=M + N)
    want = O.run_torch_pertoken(a_q, b_q, sa, sb)
    got = _run(a_q, sa, b_q, sb, out_dtype=out_dtype, stream=torch.cuda.current_stream())
    assert_close_to_oracle(got, want, f"per-token M={M} N={N} K={K} {out_dtype}")


# Decode-size M on both kernels: the swap-AB split-K kernel (token scale on every K block, channel
# scale once) and the tiled kernel give the same result within the parity bar.
@pytest.mark.parametrize("M,N,K", [(1, 7168, 2048), (16, 4096, 7168), (32, 7168, 2048), (33, 1024, 2048),
                                   (64, 24576, 1536), (7, 272, 256)])
@pytest.mark.parametrize("path", ["decode", "tiled", "auto"])
def test_pertoken_decode_sizes_on_both_kernels(M, N, K, path):
    g = torch.Generator().manual_seed(M + K)
    a_q, sa = O.pertoken_quant(torch.randn(M, K, generator=g))
    b_q, sb = O.pertoken_quant(torch.randn(N, K, generator=g) * 0.05)
    want = O.run_torch_pertoken(a_q, b_q, sa.view(-1), sb.view(-1))
    got = _run(a_q, sa.view(-1), b_q, sb.view(-1), path=path)
    assert_close_to_oracle(got, want, f"per-token {path} M={M} N={N} K={K}")


def test_pertoken_grouped_tile_order_with_a_short_last_group():
    """Enough row blocks for the grouped tile order (groups of 26 at K = 7168), the last group short."""
    g = torch.Generator().manual_seed(11)
    M, N, K = 7000, 768, 7168
    a_q, sa = O.pertoken_quant(torch.randn(M, K, generator=g))
    b_q, sb = O.pertoken_quant(torch.randn(N, K, generator=g) * 0.05)
    want = O.run_torch_pertoken(a_q, b_q, sa.view(-1), sb.view(-1))
    assert_close_to_oracle(_run(a_q, sa.view(-1), b_q, sb.view(-1)), want, "per-token grouped order")


# The CTA-pair kernel (tcgen05.mma.cta_group::2, 256 x 256 tiles over two SMs): forced on shapes with
# one tile, ragged M (a pair whose second CTA has few or no rows), many tiles per pair, the grouped
# tile order, both output types; it must reproduce the single-CTA kernel bit for bit (same products,
# same fp32 accumulation order inside the tensor core, same scaling) and match the oracle.
@pytest.mark.parametrize("M,N,K,out_dtype", [(256, 256, 256, "bf16"), (300, 768, 384, "fp16"), (129 + 256, 512, 2048, "bf16"),
                                             (2048, 6144, 1024, "bf16"), (7000, 768, 7168, "bf16")])
def test_pertoken_cta_pair_kernel(M, N, K, out_dtype):
    g = torch.Generator().manual_seed(M + K)
    a_q, sa = O.pertoken_quant(torch.randn(M, K, generator=g))
    b_q, sb = O.pertoken_quant(torch.randn(N, K, generator=g) * 0.05)
    want = O.run_torch_pertoken(a_q, b_q, sa.view(-1), sb.view(-1))
    pair = _run(a_q, sa.view(-1), b_q, sb.view(-1), out_dtype=out_dtype, path="pair")
    tiled = _run(a_q, sa.view(-1), b_q, sb.view(-1), out_dtype=out_dtype, path="tiled")
    assert_close_to_oracle(pair, want, f"per-token pair M={M} N={N} K={K}")
    assert torch.equal(pair, tiled)
    again = _run(a_q, sa.view(-1), b_q, sb.view(-1), out_dtype=out_dtype, path="pair")
    assert torch.equal(pair, again)


def test_pertoken_pair_path_argument_checks():
    from flydsl_b200.kernels import compile_preshuffle_gemm_a8

    dev = torch.device("cuda")
    fn = compile_preshuffle_gemm_a8(M=128, N=320, K=256, tile_m=64, tile_n=256, tile_k=128, path="pair")
    z = torch.zeros(128 * 320, dtype=torch.float32, device=dev)
    with pytest.raises(ValueError, match="CTA-pair path"):
        fn(z, z, z, z, z, 128, 320, None)


def test_pertoken_signed_operands_and_many_tiles_per_cta():
    """Signed operands (the reference test only uses positive ones) on a shape with several tiles per
    CTA, so that both accumulator buffers and the store hand-off are exercised; twice for
    determinism."""
    g = torch.Generator().manual_seed(3)
    M, N, K = 2048, 6144, 1024
    a_q, sa = O.pertoken_quant(torch.randn(M, K, generator=g))
    b_q, sb = O.pertoken_quant(torch.randn(N, K, generator=g) * 0.05)
    want = O.run_torch_pertoken(a_q, b_q, sa.view(-1), sb.view(-1))
    c1 = _run(a_q, sa.view(-1), b_q, sb.view(-1))
    c2 = _run(a_q, sa.view(-1), b_q, sb.view(-1))
    assert_close_to_oracle(c1, want, "per-token signed")
    assert torch.equal(c1, c2)


def test_pertoken_rejects_bad_arguments():
    from flydsl_b200.kernels import compile_preshuffle_gemm_a8

    with pytest.raises(ValueError):
        compile_preshuffle_gemm_a8(K=256, tile_m=64, tile_n=256, tile_k=128, in_dtype="fp7")
    with pytest.raises(ValueError):
        compile_preshuffle_gemm_a8(K=256, tile_m=64, tile_n=256, tile_k=128, out_dtype="fp32")
    with pytest.raises(NotImplementedError):
        compile_preshuffle_gemm_a8(K=256, tile_m=64, tile_n=256, tile_k=128, in_dtype="int8")
    with pytest.raises(ValueError):
        compile_preshuffle_gemm_a8(K=200, tile_m=64, tile_n=256, tile_k=128)
    fn = compile_preshuffle_gemm_a8(N=256, K=256, tile_m=64, tile_n=256, tile_k=128)
    a = torch.zeros(4, 256, device="cuda").to(torch.float8_e4m3fn)
    c = torch.zeros(4, 256, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        fn(c, a, a, torch.ones(2, device="cuda"), torch.ones(256, device="cuda"), 4, 256)   # scale_a too short
