"""The allocation-free stage-2 entry point, flyb200_moe_gemm2_reduce_noalloc.

It exists for callers that cannot give the library scratch memory: a C/C++ serving loop or plug-in
callback that binds the C ABI without any device allocator behind it, or a host that forbids
cudaMalloc once it is running. Instead of a caller workspace it uses a fixed 16 MiB array inside the
library. The test drives it through the C ABI twice in a row and compares each result with the
regular entry point (caller-provided workspace) on the same inputs; the second call uses a slot mask
so that rows left in the shared array by the first call must not leak into the result.

The module name sorts after the other test modules, so in a whole-suite run the shared array is used
after every other test has gone through the library in the same process -- the order in which
state left behind by earlier calls would show.
"""
import ctypes

import pytest
import torch

from tests.helpers import assert_close_to_oracle, fp8_from_u8, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case():
    g = load_golden("moe.npz")
    T, H, I, E, k = (int(v) for v in g["cfg"])
    t = {n: torch.from_numpy(g[n]) for n in ("topk_ids", "topk_w", "w2_scale", "a2_scale", "out2")}
    t.update(w2_q=fp8_from_u8(g["w2_q"]), a2_q=fp8_from_u8(g["a2_q"]))
    return (T, H, I, E, k), t


def _call(lib, name, out, a2, w2, a2s, w2s, routing, mask, dims, tile_m, workspace=None):
    from flydsl_b200 import _lib

    T, H, I, E, k = dims
    sid, sw, seid, nv, blocks = routing
    args = [out.data_ptr(), a2.data_ptr(), w2.data_ptr(), a2s.data_ptr(), w2s.data_ptr(), sid.data_ptr(),
            seid.data_ptr(), sw.data_ptr(), nv.data_ptr(), None if mask is None else mask.data_ptr(),
            T, H, I, blocks, E, k, tile_m, 1, _lib.BF16, None]
    if workspace is not None:
        args += [workspace.data_ptr(), workspace.numel() * workspace.element_size()]
    args.append(torch.cuda.current_stream().cuda_stream)
    return getattr(lib, name)(*args)


def test_noalloc_matches_workspace_entry_on_two_calls_in_a_row():
    from flydsl_b200 import _lib
    from flydsl_b200.utils import build_routing_buffers, shuffle_weight

    lib = _lib.load()
    dims, t = _case()
    T, H, I, E, k = dims
    assert T * k * H * 2 <= lib.flyb200_moe_gemm2_reduce_noalloc_max_bytes()
    a2, w2 = t["a2_q"].to(DEV), shuffle_weight(t["w2_q"].to(DEV))
    a2s, w2s = t["a2_scale"].to(DEV).t().contiguous(), t["w2_scale"].to(DEV).contiguous()
    ids, tw = t["topk_ids"].to(DEV), t["topk_w"].to(DEV)

    # call 1: all experts, no mask (tile_m 32)
    sid, sw, seid, nv, _, blocks = build_routing_buffers(topk_ids=ids, topk_weights=tw, experts=E, model_dim=H, tile_m=32)
    routing = (sid, sw, seid, nv, blocks)
    want1 = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    ws = torch.empty(T * k, H, dtype=torch.bfloat16, device=DEV)
    _lib.check(_call(lib, "flyb200_moe_gemm2_reduce", want1, a2, w2, a2s, w2s, routing, None, dims, 32, workspace=ws))
    got1 = torch.empty_like(want1)
    _lib.check(_call(lib, "flyb200_moe_gemm2_reduce_noalloc", got1, a2, w2, a2s, w2s, routing, None, dims, 32))

    # call 2, straight after: only experts 0 and 2 are "local" (expert-parallel style): their sorter
    # mask drops the other routes and the slot mask tells the reduce which rows exist
    from flydsl_b200.utils import moe_sorting

    emask = torch.tensor([1, 0, 1, 0], dtype=torch.int32, device=DEV)
    sid2, sw2, seid2, npp2 = moe_sorting(ids, tw, num_experts=E, block_size=16, expert_mask=emask)
    # local expert ids are compacted by the sorter: weights of experts 0 and 2 become experts 0 and 1
    w2_local = shuffle_weight(t["w2_q"][[0, 2]].to(DEV))
    w2s_local = t["w2_scale"][[0, 2]].to(DEV).contiguous()
    routing2 = (sid2, sw2, seid2, npp2[:1].contiguous(), seid2.numel())
    slot_mask = emask[ids.long()].to(torch.uint8).contiguous()
    dims2 = (T, H, I, 2, k)
    want2 = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    _lib.check(_call(lib, "flyb200_moe_gemm2_reduce", want2, a2, w2_local, a2s, w2s_local, routing2, slot_mask, dims2, 16,
                     workspace=ws))
    got2 = torch.empty_like(want2)
    _lib.check(_call(lib, "flyb200_moe_gemm2_reduce_noalloc", got2, a2, w2_local, a2s, w2s_local, routing2, slot_mask,
                     dims2, 16))
    torch.cuda.synchronize()
    assert _lib.query_device_error() == 0

    assert_close_to_oracle(got1, want1.float(), "noalloc call 1 vs workspace entry")
    assert_close_to_oracle(got2, want2.float(), "noalloc call 2 vs workspace entry")
    assert torch.equal(got1, want1) and torch.equal(got2, want2)   # same kernels, fixed order
    assert_close_to_oracle(got1, t["out2"], "noalloc call 1 vs reference golden")   # and it is the right answer


def test_noalloc_refuses_what_does_not_fit():
    from flydsl_b200 import _lib

    lib = _lib.load()
    limit = lib.flyb200_moe_gemm2_reduce_noalloc_max_bytes()
    T, k, H = 4096, 8, 7168
    assert T * k * H * 2 > limit
    z = torch.zeros(64, dtype=torch.uint8, device=DEV)
    rc = lib.flyb200_moe_gemm2_reduce_noalloc(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(),
                                              z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), None, T, H, 2048,
                                              8, 256, k, 128, 1, _lib.BF16, None, None)
    assert rc == _lib.ERR_WORKSPACE
    assert b"scratch" in lib.flyb200_last_error_string()
