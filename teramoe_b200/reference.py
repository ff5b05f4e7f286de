"""Plain PyTorch restatement of the MoE layer (any device, any float dtype; fp32 on CPU is the oracle).

out[t] = sum_k W_down[e_k] @ ( w_k * silu(g) * u ),  (g_j, u_j) = (W_gateup[e_k][2j] . x_t, W_gateup[e_k][2j+1] . x_t)

`W_gateup` rows are element-interleaved (g0,u0,g1,u1,...) as in the reference
(tests/test_teramoe_accuracy.py:215-220, csrc/teramoe/teramoe_wrapper.cuh:221-223); the route weight is
folded into the activation before the down projection
(csrc/teramoe/teramoe_sm100_bf16_compute.cuh:667-670).  Entries with topk_idx == -1 are skipped.
Everything is differentiable through autograd, which gives the oracle gradients for x,
topk_weights, W_gateup and W_down.
"""
from __future__ import annotations

import torch


def moe_reference(x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, W_gateup: torch.Tensor,
                  W_down: torch.Tensor) -> torch.Tensor:
    """x [T,H]; topk_idx [T,K] int (global expert ids, -1 = none); topk_weights [T,K];
    W_gateup [E,2I,H]; W_down [E,H,I] with E = number of global experts.  Returns [T,H] in x.dtype."""
    T, H = x.shape
    E = W_gateup.shape[0]
    acc_dtype = torch.float32 if x.dtype in (torch.bfloat16, torch.float16) else x.dtype
    out = torch.zeros(T, H, dtype=acc_dtype, device=x.device)
    for e in range(E):
        t_idx, k_idx = torch.nonzero(topk_idx == e, as_tuple=True)
        if t_idx.numel() == 0:
            continue
        xe = x[t_idx].to(acc_dtype)
        gu = xe @ W_gateup[e].to(acc_dtype).t()
        g, u = gu[:, 0::2], gu[:, 1::2]
        w = topk_weights[t_idx, k_idx].to(acc_dtype)
        act = torch.nn.functional.silu(g) * u * w[:, None]
        y = act @ W_down[e].to(acc_dtype).t()
        out = out.index_add(0, t_idx, y)
    return out.to(x.dtype)


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[E,I,H] x 2 -> [E,2I,H] with rows (g0,u0,g1,u1,...)."""
    E, I, H = w_gate.shape
    return torch.stack([w_gate, w_up], dim=2).reshape(E, 2 * I, H)


def deinterleave_gate_up(w_gateup: torch.Tensor):
    return w_gateup[:, 0::2], w_gateup[:, 1::2]


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - 2<x+1,y+1>/(|x+1|^2+|y+1|^2), the reference's similarity metric (tests/utils.py:39-43)."""
    x, y = x.double() + 1, y.double() + 1
    denom = (x * x + y * y).sum()
    return float(1 - 2 * (x * y).sum() / denom)
