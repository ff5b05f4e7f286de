"""`TeraMoELayer`: router + expert-parallel SwiGLU experts as an nn.Module on top of `Buffer.teramoe_autograd`.

The reference ships the layer op only; its tests build the router by hand
(tests/teramoe_test_utils.py:339-392: sigmoid or softmax scores, optional group-limited top-k, weights
normalised to sum 1).  This module packages the same routing choices so a model can drop the layer in.
Expert weights use the reference layout: W_gateup [E_local, 2I, H] with rows element-interleaved
(g0,u0,g1,u1,...), W_down [E_local, H, I].
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..buffer import Buffer


class TopKRouter(nn.Module):
    """Linear gate -> scores (sigmoid | softmax) -> optional group-limited top-k -> normalised weights."""

    def __init__(self, hidden: int, num_experts: int, top_k: int, score_func: str = "sigmoid", num_groups: int = 1,
                 topk_groups: Optional[int] = None, normalize: bool = True, dtype=torch.float32, device=None):
        super().__init__()
        if score_func not in ("sigmoid", "softmax"):
            raise ValueError("score_func must be 'sigmoid' or 'softmax'")
        if num_experts % num_groups:
            raise ValueError("num_experts must be divisible by num_groups")
        self.num_experts, self.top_k, self.score_func = num_experts, top_k, score_func
        self.num_groups, self.topk_groups, self.normalize = num_groups, topk_groups or num_groups, normalize
        self.weight = nn.Parameter(torch.empty(num_experts, hidden, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=1.0 / math.sqrt(hidden))
        self.register_buffer("expert_bias", torch.zeros(num_experts, dtype=torch.float32, device=device))

    def forward(self, x: torch.Tensor):
        logits = torch.nn.functional.linear(x.float(), self.weight.float())
        scores = torch.sigmoid(logits) if self.score_func == "sigmoid" else torch.softmax(logits, dim=-1)
        select = scores + self.expert_bias            # the bias steers selection only, not the weights
        if self.num_groups > 1 and self.topk_groups < self.num_groups:
            T = select.shape[0]
            g = select.view(T, self.num_groups, -1)
            group_score = g.topk(min(2, g.shape[-1]), dim=-1).values.sum(-1)
            keep = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, group_score.topk(self.topk_groups, dim=-1).indices, True)
            select = torch.where(keep.unsqueeze(-1).expand_as(g), g, torch.full_like(g, float("-inf"))).reshape(T, -1)
        topk_idx = select.topk(self.top_k, dim=-1).indices
        weights = scores.gather(1, topk_idx)
        if self.normalize:
            weights = weights / weights.sum(dim=-1, keepdim=True).clamp(min=1e-20)
        return topk_idx, weights.float()


class TeraMoELayer(nn.Module):
    """y = sum_k w_k * Expert_{e_k}(x), experts sharded over the ranks of `buffer`'s group."""

    def __init__(self, buffer: Buffer, hidden: int, intermediate: int, num_experts: int, top_k: int, score_func: str = "sigmoid",
                 num_groups: int = 1, topk_groups: Optional[int] = None, dtype=torch.bfloat16, device=None, init_std: float = 0.02,
                 **layer_kwargs):
        super().__init__()
        if num_experts % buffer.group_size:
            raise ValueError("num_experts must be divisible by the expert-parallel size")
        device = device if device is not None else buffer.device
        self.buffer, self.num_experts = buffer, num_experts
        self.num_local_experts = num_experts // buffer.group_size
        self.layer_kwargs = layer_kwargs
        self.router = TopKRouter(hidden, num_experts, top_k, score_func, num_groups, topk_groups, device=device)
        self.W_gateup = nn.Parameter(torch.empty(self.num_local_experts, 2 * intermediate, hidden, dtype=dtype, device=device))
        self.W_down = nn.Parameter(torch.empty(self.num_local_experts, hidden, intermediate, dtype=dtype, device=device))
        nn.init.normal_(self.W_gateup, std=init_std)
        nn.init.normal_(self.W_down, std=init_std)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        topk_idx, topk_w = self.router(x2)
        out = self.buffer.teramoe_autograd(x2, topk_idx, topk_w, self.W_gateup, self.W_down, self.num_experts, **self.layer_kwargs)
        return out.reshape(shape)


class MoEBlock(nn.Module):
    """Pre-norm residual block around a TeraMoELayer (the shape an MoE transformer's FFN takes)."""

    def __init__(self, buffer: Buffer, hidden: int, intermediate: int, num_experts: int, top_k: int, eps: float = 1e-6, **kw):
        super().__init__()
        self.norm = nn.RMSNorm(hidden, eps=eps, device=kw.get("device", buffer.device), dtype=kw.get("dtype", torch.bfloat16))
        self.moe = TeraMoELayer(buffer, hidden, intermediate, num_experts, top_k, **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x + self.moe(self.norm(x))
