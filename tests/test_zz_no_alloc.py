"""The scratch-free entry point, lo_fused_moe_block_int8_noalloc, against the ordinary one.

The ordinary entry point takes a workspace from the caller.  This one is for hosts that cannot
get device memory when they need the layer (a serving thread that must not run into cudaMalloc's
device-wide synchronisation, a plugin handed raw pointers by a runtime that owns the allocator, a
foreign-language binding without an allocator handle): its scratch is an array inside the library.
Both are called through the C ABI on the same inputs, twice in a row with different inputs, so the
second call runs on scratch that still holds the first call's intermediates.
"""
import ctypes

import pytest
import torch

from lightop_b200 import synthetic
from util import assert_out_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call(lib, _lib, fn_name, t, ids, M, E, k, H, I, workspace=None):
    cache3 = torch.empty(M * k * H, dtype=torch.bfloat16, device=DEV)
    out = torch.full((M, H), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    head = [t["x"].data_ptr(), t["w1"].data_ptr(), t["w2"].data_ptr(), t["w1_s"].data_ptr(), t["w2_s"].data_ptr(),
            t["w"].data_ptr(), ids.data_ptr(), _lib.LO_I32, 0, E, M, E, k, H, I, cache3.data_ptr(), 0, out.data_ptr(),
            0, 1.0]
    if workspace is None:
        st = getattr(lib, fn_name)(*head, status.data_ptr(), stream)
    else:
        st = getattr(lib, fn_name)(*head, workspace.data_ptr(), workspace.numel(), status.data_ptr(), stream)
    _lib.check(st, fn_name)
    torch.cuda.synchronize()
    assert status.item() == 0
    return out


def test_noalloc_matches_workspace_entry_point_twice():
    from lightop_b200 import _lib
    from oracle import moe_block_int8 as O
    lib = _lib.load()
    E, k, H, I = 8, 2, 256, 512
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=0)
    for call, (M, seed) in enumerate([(32, 1), (19, 7)]):
        x, logits = synthetic.make_activations(M, H, E, seed=seed)
        w, ids = O.route_topk_softmax(logits, k, renormalize=True)
        t = {n: v.to(DEV).contiguous() for n, v in dict(x=x, w1=w1, w2=w2, w1_s=w1_s, w2_s=w2_s, w=w.float()).items()}
        ids_d = ids.to(torch.int32).to(DEV).contiguous()
        ws_bytes = lib.lo_fused_moe_workspace_bytes(M, E, E, k, H, I)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
        ref = _call(lib, _lib, "lo_fused_moe_block_int8", t, ids_d, M, E, k, H, I, workspace=ws)
        got = _call(lib, _lib, "lo_fused_moe_block_int8_noalloc", t, ids_d, M, E, k, H, I)
        assert not torch.isnan(got.float()).any()
        # same kernels, same inputs: the tolerance of the layer tests, and in fact the same bits
        assert_out_close(got, ref, f"no-alloc call {call}")
        assert torch.equal(got, ref)
        # and both agree with the oracle
        assert_out_close(got, O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w, ids), f"oracle, call {call}")


def test_noalloc_rejects_shapes_beyond_its_scratch():
    from lightop_b200 import _lib
    lib = _lib.load()
    # DeepSeek-V3 prefill needs ~350 MB of scratch: refused before anything is launched
    st = lib.lo_fused_moe_block_int8_noalloc(0, 0, 0, 0, 0, 0, 0, _lib.LO_I32, 0, 256, 4096, 256, 8, 7168, 2048,
                                             0, 0, 0, 0, 1.0, 0, 0)
    assert st == 1
    assert b"built-in array" in lib.lo_last_error()
