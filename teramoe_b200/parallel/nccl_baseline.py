"""Comparison baseline (not the product): Megatron-style MoE layer built from library pieces only.

permute by expert -> NCCL all_to_all_single -> sort by local expert -> per-expert cuBLAS GEMMs
(gate_up, SwiGLU, down) -> all_to_all_single back -> weighted un-permute.  Autograd comes from
PyTorch, so it keeps what an eager implementation keeps (permuted inputs per slot, gate/up, act).

The reference's own baseline is DeepEP dispatch/combine + TransformerEngine grouped MLP
(tests/teramoe_test_utils.py:134-226); neither library is available offline, and the task names an
NCCL all-to-all + grouped-GEMM layer as the same-box baseline.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        if group is None or dist.get_world_size(group) == 1:
            return x.clone()
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        if ctx.group is None or dist.get_world_size(ctx.group) == 1:
            return g.clone(), None, None, None
        out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return out, None, None, None


class _PermuteRows(torch.autograd.Function):
    """y = x[perm] for a permutation `perm`; the gradient is a gather through the inverse permutation
    (no atomics), which is what a fused permute kernel of a training framework does."""

    @staticmethod
    def forward(ctx, x, perm, inv):
        ctx.save_for_backward(inv)
        return x[perm]

    @staticmethod
    def backward(ctx, g):
        (inv,) = ctx.saved_tensors
        return g[inv], None, None


class NcclMoEBaseline:
    def __init__(self, group: Optional[dist.ProcessGroup], num_experts: int, grouped: bool = False):
        self.group = group
        self.grouped = grouped and hasattr(torch.nn.functional, "grouped_mm")
        self.N = dist.get_world_size(group) if group is not None else 1
        self.E = num_experts
        self.El = num_experts // self.N

    @staticmethod
    def to_chunked(W_gateup: torch.Tensor) -> torch.Tensor:
        """Element-interleaved [E,2I,H] -> gate rows then up rows (the layout a library SwiGLU wants)."""
        return torch.cat([W_gateup[:, 0::2], W_gateup[:, 1::2]], dim=1).contiguous()

    def __call__(self, x, topk_idx, topk_weights, W_gateup, W_down, chunked: bool = False):
        """`chunked=True`: W_gateup holds all gate rows, then all up rows (no strided slicing)."""
        N, E, El = self.N, self.E, self.El
        T, H = x.shape
        K = topk_idx.shape[1]
        flat_e = topk_idx.reshape(-1)
        valid = flat_e >= 0
        ent = torch.nonzero(valid, as_tuple=True)[0]
        e_of = flat_e[ent]
        order = torch.argsort(e_of, stable=True)
        ent = ent[order]
        tok = ent // K
        cnt = torch.bincount(e_of, minlength=E).view(N, El)
        # counts exchange: recv_cnt[s, le] = entries rank s sends for my local expert le
        if N > 1:
            recv_cnt = torch.empty_like(cnt)
            dist.all_to_all_single(recv_cnt, cnt.contiguous(), group=self.group)
        else:
            recv_cnt = cnt
        cnt_h, recv_h = cnt.cpu(), recv_cnt.cpu()                  # host sync, as in Megatron's all-to-all dispatcher
        in_splits = cnt_h.sum(1).tolist()
        out_splits = recv_h.sum(1).tolist()
        all_valid = ent.numel() == T * K
        if all_valid:
            # permutation path: every (token,k) entry is routed, so permute / un-permute are pure gathers
            inv_ent = torch.empty_like(ent)
            inv_ent[ent] = torch.arange(ent.numel(), device=x.device)
            xs = _PermuteRows.apply(x.unsqueeze(1).expand(T, K, H).reshape(T * K, H), ent, inv_ent)
        else:
            xs = x[tok]                                            # [entries, H] permuted by expert (kept by autograd)
        recv = _AllToAll.apply(xs, out_splits, in_splits, self.group)
        # rows arrive grouped by (source, local expert); regroup by local expert
        S = recv.shape[0]
        seg = recv_h.reshape(-1)                                   # [N*El] lengths in arrival order
        starts = torch.cumsum(seg, 0) - seg
        pieces = []
        for le in range(El):
            for s in range(N):
                j = s * El + le
                if seg[j] > 0:
                    pieces.append(torch.arange(int(starts[j]), int(starts[j] + seg[j])))
        sort_idx = (torch.cat(pieces) if pieces else torch.zeros(0, dtype=torch.long)).to(x.device)
        inv = torch.empty_like(sort_idx)
        inv[sort_idx] = torch.arange(S, device=x.device)
        xe = _PermuteRows.apply(recv, sort_idx, inv)
        per_expert = recv_h.sum(0).tolist()
        if self.grouped and chunked and S > 0:
            # one library grouped GEMM per stage (torch.nn.functional.grouped_mm) instead of a loop over experts
            offs = torch.cumsum(recv_cnt.sum(0), 0).to(torch.int32)
            gu = torch.nn.functional.grouped_mm(xe, W_gateup.transpose(-2, -1), offs=offs)
            g, u = gu.chunk(2, dim=1)
            ye = torch.nn.functional.grouped_mm(torch.nn.functional.silu(g) * u, W_down.transpose(-2, -1), offs=offs)
            return self._finish(ye, inv, sort_idx, in_splits, out_splits, all_valid, ent, inv_ent if all_valid else None, tok,
                                topk_weights, T, K, H, x)
        outs = []
        o = 0
        for le in range(El):
            c = per_expert[le]
            if c == 0:
                continue
            a = xe[o:o + c]
            gu = a @ W_gateup[le].t()
            if chunked:
                g, u = gu.chunk(2, dim=1)
                act = torch.nn.functional.silu(g) * u
            else:
                act = torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]
            outs.append(act @ W_down[le].t())
            o += c
        ye = torch.cat(outs) if outs else xe.new_zeros(0, H)
        return self._finish(ye, inv, sort_idx, in_splits, out_splits, all_valid, ent, inv_ent if all_valid else None, tok, topk_weights,
                            T, K, H, x)

    def _finish(self, ye, inv, sort_idx, in_splits, out_splits, all_valid, ent, inv_ent, tok, topk_weights, T, K, H, x):
        y = _PermuteRows.apply(ye, inv, sort_idx)
        back = _AllToAll.apply(y, in_splits, out_splits, self.group)
        if all_valid:
            yk = _PermuteRows.apply(back, inv_ent, ent).view(T, K, H)
            return (yk * topk_weights.to(back.dtype).unsqueeze(-1)).sum(1)
        wsel = topk_weights.reshape(-1)[ent].to(back.dtype)
        out = torch.zeros(T, H, dtype=torch.float32, device=x.device).index_add(0, tok, (back * wsel[:, None]).float())
        return out.to(x.dtype)
