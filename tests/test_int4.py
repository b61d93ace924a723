"""Weight-only int4 x bf16 decode GEMM: oracle self-checks on CPU, kernel parity on the GPU."""
import numpy as np
import pytest
import torch

from oracle import int4_ref as R
from tests.helpers import assert_close_to_oracle


def test_oracle_quantiser_and_pack_layout():
    c = R.make_int4_case(4, 256, 512, seed=1)
    q, s = c["q"], c["scales"]
    assert q.dtype == torch.int8 and int(q.min()) >= -8 and int(q.max()) <= 7
    assert s.dtype == torch.bfloat16 and tuple(s.shape) == (256, 4)
    # scale = amax/7 (as bf16): dequantised weights are within half a step of the originals
    err = (R.dequant_int4_ref(q, s) - c["w"]).abs().reshape(256, 4, 128).amax(-1)
    assert (err <= 0.5 * s.float() * 1.01 + 1e-8).all()
    # packed layout: unpack by the documented rule and compare
    packed = R.pack_int4_ref(q.numpy())
    assert packed.shape == (4, 32, 4, 8, 16)          # [group, row / 8, chunk, row % 8, 16 bytes]
    words = packed.view(np.uint32).reshape(4, 32, 4, 8, 4).transpose(0, 1, 3, 2, 4).reshape(4, 256, 16)
    order = [0, 2, 4, 6, 1, 3, 5, 7]
    back = np.zeros((4, 256, 16, 8), dtype=np.int32)
    for pos, e in enumerate(order):
        back[..., e] = ((words >> np.uint32(4 * pos)) & 0xF).astype(np.int32) - 8
    assert np.array_equal(back.transpose(1, 0, 2, 3).reshape(256, 512), q.numpy().astype(np.int32))
    # all-zero group -> scale 1, zeros
    z, zs = R.quantize_int4_groupwise_ref(torch.zeros(2, 128))
    assert (zs == 1).all() and (z == 0).all()


@pytest.mark.gpu
def test_gpu_pack_matches_oracle_layout():
    from flydsl_b200.kernels import pack_int4_weight, quantize_int4_groupwise

    c = R.make_int4_case(1, 384, 1024, seed=2)
    q_dev, s_dev = quantize_int4_groupwise(c["w"].cuda())
    assert torch.equal(q_dev.cpu(), c["q"]) and torch.equal(s_dev.cpu(), c["scales"])
    wq, st = pack_int4_weight(c["q"].cuda(), c["scales"].cuda())
    assert np.array_equal(wq.cpu().numpy(), R.pack_int4_ref(c["q"].numpy()))
    assert torch.equal(st.cpu(), c["scales"].t().contiguous())


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K,split_k", [(1, 256, 512, None), (7, 384, 1024, 1), (16, 1024, 2048, 2),
                                           (33, 512, 1024, 4), (64, 1024, 1024, None), (16, 8192, 8192, None),
                                           (64, 8192, 8192, None), (1, 8192, 8192, None),
                                           (17, 128, 128, None), (32, 640, 3072, 8), (48, 256, 8192, 3)])
@pytest.mark.parametrize("path", ["stream", "tensor"])
def test_gpu_int4_gemm_vs_oracle(M, N, K, split_k, path):
    from flydsl_b200 import _lib
    from flydsl_b200.kernels import compile_int4_weight_only_gemm, pack_int4_weight

    c = R.make_int4_case(M, N, K, seed=M + N)
    ref = R.int4_gemm_ref(c["a"], c["q"], c["scales"])
    wq, st = pack_int4_weight(c["q"].cuda(), c["scales"].cuda())
    fn = compile_int4_weight_only_gemm(N=N, K=K, split_k=split_k, path=path)
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    fn(out, c["a"].cuda(), wq, st, M, None)
    out2 = torch.empty_like(out)
    fn(out2, c["a"].cuda(), wq, st, M, torch.cuda.current_stream())
    torch.cuda.synchronize()
    assert _lib.query_device_error() == 0
    assert_close_to_oracle(out, ref, f"int4 {path} M={M} N={N} K={K} split_k={split_k}")
    assert torch.equal(out, out2)                       # fixed summation order


@pytest.mark.gpu
def test_gpu_int4_gemm_rejects_bad_arguments():
    from flydsl_b200.kernels import compile_int4_weight_only_gemm

    with pytest.raises(ValueError):
        compile_int4_weight_only_gemm(N=100, K=128)
    fn = compile_int4_weight_only_gemm(N=128, K=128)
    a = torch.zeros((65, 128), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((65, 128), dtype=torch.bfloat16, device="cuda")
    wq = torch.zeros((1, 128, 64), dtype=torch.uint8, device="cuda")
    st = torch.ones((1, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(Exception):
        fn(c, a, wq, st, 65, None)                      # M > 64 is outside this kernel
