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
