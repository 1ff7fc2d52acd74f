"""Expert parallelism over peer stores, R ranks emulated on one GPU.

Every "rank" is a set of buffers in the one device's memory; the steps of lightop_b200/ep.py's peer transport run
rank after rank through the C ABI (plan, put into the destination ranks' receive zones, expert-side GEMMs whose
epilogue stores into the source ranks' return zones, gather), with the same host bookkeeping (ep.peer_routes).  No
kernel waits for another, so one GPU can run them in sequence.  The result of every rank must have the bits of the
single-GPU layer on that rank's tokens (the sequence of the reference's own EP test,
test/test_ep_gather_scatter_moe.py:205-296, with the exchange filled in).
"""
import pytest
import torch

from lightop_b200 import synthetic
from oracle import moe_block_int8 as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def lo():
    import lightop_b200
    return lightop_b200


@pytest.mark.parametrize("R,E,k,H,I,tokens", [(2, 8, 2, 256, 256, (40, 17)), (4, 16, 4, 512, 256, (33, 70, 1, 128)),
                                              (3, 12, 3, 384, 128, (0, 25, 300))])
def test_peer_transport_with_emulated_ranks(lo, R, E, k, H, I, tokens):
    from lightop_b200 import _lib, device_status_word
    from lightop_b200.ep import peer_routes
    from lightop_b200.quant import per_token_group_quant_int8
    lib = _lib.load()
    El = E // R
    w1, w2, w1_s, w2_s = [t.to(DEV) for t in synthetic.make_weights(E, H, I, seed=31)]
    rank_of_expert = (torch.arange(E, device=DEV) // El).to(torch.int32)
    stride = int(lib.lo_ep_dispatch_row_bytes(H))
    st = _lib.current_stream(torch.device(DEV))
    xs_, tw_, ti_, inv_, counts_, xq_, xsc_ = [], [], [], [], [], [], []
    for r in range(R):
        M = tokens[r]
        x, logits = synthetic.make_activations(max(M, 1), H, E, seed=40 + r)
        x, logits = x[:M].to(DEV), logits[:M].to(DEV)
        tw = torch.empty(M, k, dtype=torch.float32, device=DEV)
        ti = torch.empty(M, k, dtype=torch.int32, device=DEV)
        if M:
            lo.moe.topk_softmax(tw, ti, None, logits, True)
        xq, xsc = per_token_group_quant_int8(x, 128) if M else (torch.empty(0, H, dtype=torch.int8, device=DEV), torch.empty(0, H // 128, device=DEV))
        dest = torch.empty(M * k, dtype=torch.int32, device=DEV)
        inv = torch.empty(M, k, dtype=torch.int32, device=DEV)
        counts = torch.zeros(R, dtype=torch.int32, device=DEV)
        _lib.check(lib.lo_ep_dispatch_plan(_lib.ptr(ti), _lib.dtype_code(ti.dtype), _lib.ptr(rank_of_expert), M, k, R,
                                           _lib.ptr(dest), _lib.ptr(inv), _lib.ptr(counts), st), "plan")
        xs_.append(x); tw_.append(tw); ti_.append(ti); inv_.append(inv); counts_.append(counts); xq_.append(xq); xsc_.append(xsc)
    mat = torch.stack(counts_).tolist()
    assert [sum(row) for row in mat] == [tokens[r] * k for r in range(R)]
    recv_rows = [sum(mat[s][d] for s in range(R)) for d in range(R)]
    recv = [torch.zeros(max(recv_rows[d], 1) * stride, dtype=torch.uint8, device=DEV) for d in range(R)]
    ret = [torch.zeros(max(tokens[r] * k, 1), H, dtype=torch.bfloat16, device=DEV) for r in range(R)]
    peer_recv = [t.data_ptr() for t in recv]
    peer_ret = [t.data_ptr() for t in ret]
    routes = [peer_routes(mat, me, stride, 2 * H, peer_recv, peer_ret) for me in range(R)]
    tables = []
    for r in range(R):                                   # dispatch: every rank stores into everybody's receive zone
        first_out, seg_dst, first_in, seg_ret = routes[r]
        i32 = torch.tensor(first_out + first_in, dtype=torch.int32, device=DEV)
        i64 = torch.tensor(seg_dst + seg_ret, dtype=torch.int64, device=DEV)
        tables.append((i32, i64))
        _lib.check(lib.lo_ep_dispatch_put(_lib.ptr(xq_[r]), _lib.ptr(xsc_[r]), _lib.ptr(ti_[r]), _lib.dtype_code(ti_[r].dtype),
                                          _lib.ptr(tw_[r]), _lib.ptr(rank_of_expert), _lib.ptr(inv_[r]), tokens[r], k, H, El, R,
                                          i32.data_ptr(), i64.data_ptr(), st), "put")
    for r in range(R):                                   # expert side: result rows go straight to their source's zone
        if recv_rows[r] == 0:
            continue
        sl = slice(r * El, (r + 1) * El)
        a, b, c, d = w1[sl].contiguous(), w2[sl].contiguous(), w1_s[sl].contiguous(), w2_s[sl].contiguous()
        nbytes = lib.lo_expert_rows_packed_workspace_bytes(recv_rows[r], El, H, I)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
        i32, i64 = tables[r]
        _lib.check(lib.lo_expert_rows_block_int8_packed_put(
            _lib.ptr(recv[r]), recv_rows[r], _lib.ptr(a), _lib.ptr(b), _lib.ptr(c), _lib.ptr(d), El, H, I,
            i32.data_ptr() + 4 * R, i64.data_ptr() + 8 * R, R, _lib.ptr(ws), nbytes,
            _lib.ptr(device_status_word(torch.device(DEV))), st), "experts")
        torch.cuda.synchronize()
    for r in range(R):                                   # gather, and the comparison
        M = tokens[r]
        if M == 0:
            continue
        y = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
        ones = torch.ones(M, k, dtype=torch.float32, device=DEV)
        _lib.check(lib.lo_ep_gather(_lib.ptr(ret[r]), _lib.ptr(ti_[r]), _lib.dtype_code(ti_[r].dtype), _lib.ptr(ones),
                                    _lib.ptr(inv_[r]), 0, _lib.ptr(y), M, k, H, st), "gather")
        c13 = torch.empty(M * k * H, dtype=torch.bfloat16, device=DEV)
        local = lo.moe.fused_experts_impl_int8(xs_[r], w1, w2, tw_[r], ti_[r], c13, use_int8_w8a8=True, block_shape=[128, 128],
                                               w1_scale=w1_s, w2_scale=w2_s)
        torch.cuda.synchronize()
        assert torch.equal(y, local), f"rank {r}: max diff {(y.float() - local.float()).abs().max().item()}"
    lo.check_device_status()


def test_peer_buffer_entry_points_and_words_to_host(lo):
    """lo_peer_alloc / lo_peer_export / lo_peer_free on one device (a process does not open its own handle), and the
    kernel-written read of a few words into page-locked memory."""
    import ctypes
    from lightop_b200 import _lib
    lib = _lib.load()
    with torch.cuda.device(DEV):
        p = ctypes.c_void_p()
        _lib.check(lib.lo_peer_alloc(1 << 20, ctypes.byref(p)), "alloc")
        assert p.value
        hb = int(lib.lo_peer_handle_bytes())
        assert hb == 64
        buf = (ctypes.c_uint8 * hb)()
        _lib.check(lib.lo_peer_export(p.value, buf), "export")
        assert any(buf)
        assert lib.lo_peer_alloc(0, ctypes.byref(ctypes.c_void_p())) != 0          # bad size is an error, not a crash
        _lib.check(lib.lo_peer_free(p.value), "free")
        src = torch.arange(37, dtype=torch.int32, device=DEV) * 3 - 5
        dst = torch.zeros(37, dtype=torch.int32).pin_memory()
        _lib.check(lib.lo_words_to_host(_lib.ptr(src), dst.data_ptr(), 37, _lib.current_stream(torch.device(DEV))), "words")
        torch.cuda.synchronize()
    assert torch.equal(dst, src.cpu())
