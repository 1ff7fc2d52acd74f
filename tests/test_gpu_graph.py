"""CUDA-graph capture and replay of the layer, both quantisation modes, and of the routers: the library
neither synchronises nor allocates, so a warmed-up call can be captured and replayed on new inputs."""
import pytest
import torch

from lightop_b200 import synthetic
from oracle import moe_block_int8 as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def lo():
    import lightop_b200
    return lightop_b200


@pytest.mark.parametrize("mode", ["block", "channel"])
def test_layer_graph_replay(lo, mode):
    E, k, M, H, I = 16, 4, 48, 512, 256
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=12)
    if mode == "channel":
        w1_s, w2_s = synthetic.make_channel_scales(E, H, I, seed=12)
        kw = dict(use_int8_w8a8=True, per_channel_quant=True)
    else:
        kw = dict(use_int8_w8a8=True, block_shape=[128, 128])
    w1, w2, w1_s, w2_s = (t.to(DEV) for t in (w1, w2, w1_s, w2_s))
    x_a, logits_a = synthetic.make_activations(M, H, E, seed=13, device=DEV)
    x_b, logits_b = synthetic.make_activations(M, H, E, seed=14, device=DEV)
    x = x_a.clone()
    logits = logits_a.clone()
    tw = torch.empty(M, k, dtype=torch.float32, device=DEV)
    ti = torch.empty(M, k, dtype=torch.int32, device=DEV)
    cache13 = torch.empty(M * k * max(2 * I, H), dtype=torch.bfloat16, device=DEV)

    def step():
        lo.moe.topk_softmax(tw, ti, None, logits, True)
        return lo.moe.fused_experts_impl_int8(x, w1, w2, tw, ti, cache13, w1_scale=w1_s, w2_scale=w2_s, **kw)

    eager_a = step().clone()            # also the warm-up: kernel attributes and tensor maps are set up here
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = step()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, eager_a)
    # new inputs in the captured buffers: the routing, the chunk table and the result all follow
    x.copy_(x_b)
    logits.copy_(logits_b)
    graph.replay()
    torch.cuda.synchronize()
    lo.check_device_status()
    replay_b = y.clone()
    eager_b = step()
    torch.cuda.synchronize()
    assert torch.equal(replay_b, eager_b)
    assert not torch.equal(replay_b, eager_a)


def test_gate_graph_replay(lo):
    # the reference tests graph replay of its gate after the inputs change (docs/moe_fused_gate_dispatch.md:59-64)
    from oracle import moe_gate as OG
    M, E = 64, 256
    g = torch.Generator().manual_seed(2)
    xa, xb = torch.randn(M, E, generator=g), torch.randn(M, E, generator=g)
    bias = torch.randn(E, generator=g).to(DEV)
    x = xa.to(DEV).clone()
    lo.moe.moe_fused_gate(x, bias, 8, 4, 8, 0, 2.5)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        w, ids = lo.moe.moe_fused_gate(x, bias, 8, 4, 8, 0, 2.5)
    for src in (xa, xb):
        x.copy_(src.to(DEV))
        graph.replay()
        torch.cuda.synchronize()
        w_ref, ids_ref = OG.fused_gate(src, bias.cpu(), 8, 4, 8, 0, 2.5)
        assert torch.equal(ids.cpu(), ids_ref)
        torch.testing.assert_close(w.cpu(), w_ref, rtol=2e-5, atol=2e-6)
