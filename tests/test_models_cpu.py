"""nn.Module wrappers: router choices and a trainable MoE block on CPU."""
import torch

import teramoe_b200 as tm
from teramoe_b200.models import MoEBlock, TeraMoELayer, TopKRouter


def test_router_group_limited_topk():
    torch.manual_seed(0)
    r = TopKRouter(32, 16, 4, score_func="sigmoid", num_groups=4, topk_groups=2)
    idx, w = r(torch.randn(50, 32))
    assert idx.shape == (50, 4) and torch.allclose(w.sum(1), torch.ones(50), atol=1e-5)
    groups = (idx // 4)
    assert all(len(set(g.tolist())) <= 2 for g in groups)          # experts come from at most 2 groups
    r2 = TopKRouter(32, 16, 4, score_func="softmax")
    idx2, w2 = r2(torch.randn(7, 32))
    assert (idx2 >= 0).all() and (idx2 < 16).all() and (w2 > 0).all()


def test_block_trains_on_cpu():
    torch.manual_seed(1)
    buf = tm.Buffer(None, device="cpu")
    block = MoEBlock(buf, hidden=64, intermediate=96, num_experts=8, top_k=2, dtype=torch.float32, device="cpu", init_std=0.1)
    opt = torch.optim.SGD(block.parameters(), lr=0.05)
    x = torch.randn(4, 24, 64)
    target = torch.randn(4, 24, 64)
    losses = []
    for _ in range(8):
        opt.zero_grad()
        loss = (block(x) - target).pow(2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
    assert block.moe.router.weight.grad is not None and block.moe.W_gateup.grad.abs().sum() > 0


def test_two_layers_share_one_buffer():
    """Forward of layer 2 runs before backward of layer 1: saved state must not live in reused buffers."""
    torch.manual_seed(2)
    buf = tm.Buffer(None, device="cpu")
    T, H, I, E, K = 48, 64, 96, 8, 2
    x = torch.randn(T, H)
    params = []
    for _ in range(2):
        params.append((torch.randn(E, 2 * I, H) * 0.1, torch.randn(E, H, I) * 0.1, torch.randn(T, E)))

    def run(layer_fn):
        leaves = [x.clone().requires_grad_(True)]
        h = leaves[0]
        ws = []
        for Wg, Wd, logits in params:
            Wg, Wd = Wg.clone().requires_grad_(True), Wd.clone().requires_grad_(True)
            top = torch.topk(logits, K, dim=1)
            w = torch.softmax(top.values, 1).requires_grad_(True)
            h = h + layer_fn(h, top.indices, w, Wg, Wd)
            ws += [Wg, Wd, w]
        h.pow(2).sum().backward()
        return [leaves[0].grad] + [p.grad for p in ws]

    got = run(lambda h, idx, w, Wg, Wd: buf.teramoe_autograd(h, idx, w, Wg, Wd, E))
    want = run(lambda h, idx, w, Wg, Wd: tm.moe_reference(h, idx, w, Wg, Wd))
    for a, b in zip(got, want):
        assert torch.allclose(a, b, atol=1e-4, rtol=1e-4)
