"""Low-latency (inference-style) dispatch / combine API of `Buffer`.

Reference counterparts: teramoe/buffer.py:537-708 (Python API), csrc/kernels/internode_ll.cu:129-463
(dispatch: optional FP8 cast, push to the final per-expert slot), :715-1139 (combine: weighted reduce,
optional LogFMT-10 compression), :1241-1288 (rank-mask maintenance), csrc/config.hpp:133-219 (layout).

Semantics kept: packed per-expert receive tensor [E_local, ranks * max_tokens, H] with per-expert valid
counts, FP8 e4m3 payload with one scale per 128 channels (optionally rounded to a power of two and
packed as UE8M0 bytes), a WEIGHTED combine at the token's rank, the LogFMT-10 numerics of the
combine payload, receive hooks, cumulative receive statistics and the rank mask of the elastic
"shrink" mode.  Transport: the same deterministic push kernels as the training path (one NVSwitch
node, so there is no RDMA double buffer to manage); `clean_low_latency_buffer` is a barrier.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch

from .engine import LayerHandle

FP8_MAX = 448.0
LOGFMT_BITS = 10


@dataclass
class LowLatencyHandle:
    layer: LayerHandle
    max_tokens: int
    hidden: int
    num_experts: int
    slot_index: torch.Tensor     # [valid slots] flat row in the packed [E_local * ranks * max_tokens] layout
    slot_ids: torch.Tensor       # [valid slots] slot-space row


def fp8_quantize(x: torch.Tensor, round_scale: bool = False, use_ue8m0: bool = False):
    """Per-128-channel e4m3 cast (csrc/kernels/internode_ll.cu:220-246, csrc/kernels/utils.cuh:464-499).
    -> (x_fp8 [..., H], scales [..., H/128] fp32, or int32 [..., H/512] holding four UE8M0 exponent bytes)."""
    H = x.shape[-1]
    if H % 128 != 0:
        raise ValueError("hidden size must be a multiple of 128 for FP8 dispatch")
    if use_ue8m0 and not round_scale:
        raise ValueError("UE8M0 scales require round_scale=True")
    xv = x.float().reshape(*x.shape[:-1], H // 128, 128)
    amax = xv.abs().amax(dim=-1).clamp(min=1e-4)
    scale = amax / FP8_MAX
    if round_scale:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    q = (xv / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).reshape(x.shape)
    if use_ue8m0:
        if (H // 128) % 4 != 0:
            raise ValueError("UE8M0 packing needs hidden % 512 == 0")
        expo = (torch.log2(scale).round().to(torch.int32) + 127).clamp(0, 255)
        e4 = expo.reshape(*expo.shape[:-1], -1, 4)
        packed = e4[..., 0] | (e4[..., 1] << 8) | (e4[..., 2] << 16) | (e4[..., 3] << 24)
        return q, packed.to(torch.int32)
    return q, scale


def fp8_dequantize(q: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    H = q.shape[-1]
    if scales.dtype == torch.int32:
        b = torch.stack([(scales >> s) & 0xFF for s in (0, 8, 16, 24)], dim=-1).reshape(*scales.shape[:-1], -1)
        scales = torch.exp2(b.float() - 127)
    xv = q.float().reshape(*q.shape[:-1], H // 128, 128) * scales.unsqueeze(-1)
    return xv.reshape(q.shape).to(dtype)


def logfmt10_roundtrip(x: torch.Tensor) -> torch.Tensor:
    """Numerics of the LogFMT-10 combine payload (csrc/kernels/internode_ll.cu:557-713): per 128 channels,
    if log2(amax) < 0 and the range is not degenerate, every value becomes sign + 9-bit code of
    log2|x| on a grid of 510 steps between max(log_amin, log_amax - 32) and log_amax (code 0 = zero);
    other divisions stay bf16."""
    H = x.shape[-1]
    if H % 128 != 0:
        return x
    xv = x.float().reshape(-1, H // 128, 128)
    ax = xv.abs()
    amax = ax.amax(dim=-1, keepdim=True)
    amin = torch.where(ax > 0, ax, torch.full_like(ax, float("inf"))).amin(dim=-1, keepdim=True)
    log_amax = torch.log2(amax.clamp(min=1e-38))
    log_amin = torch.maximum(torch.log2(amin.clamp(min=1e-38)), log_amax - 32)
    use = (log_amax < 0) & (log_amin < log_amax) & torch.isfinite(amin)
    step = (log_amax - log_amin) / ((1 << (LOGFMT_BITS - 1)) - 2)
    code = torch.floor((torch.log2(ax.clamp(min=1e-38)) - log_amin) / step.clamp(min=1e-30) + 0.5) + 1
    code = torch.where(ax > 0, code.clamp(1, (1 << (LOGFMT_BITS - 1)) - 1), torch.zeros_like(code))
    dec = torch.where(code > 0, torch.exp2((code - 1) * step + log_amin), torch.zeros_like(code)) * torch.sign(xv)
    out = torch.where(use, dec, xv)
    return out.reshape(x.shape).to(x.dtype)


class LowLatencyMixin:
    """Methods mixed into `Buffer` (they use its `_engine`, `_drive`, `_world`, `group_size`)."""

    # ------------------------------------------------------------------ rank mask (elastic shrink)
    def _require_shrink(self):
        if not self.enable_shrink:
            raise RuntimeError("the rank-mask API needs Buffer(enable_shrink=True)")

    def low_latency_update_mask_buffer(self, rank_to_mask: int, mask: bool = False) -> None:
        self._require_shrink()
        if not 0 <= rank_to_mask < self.group_size:
            raise ValueError("rank out of range")
        (self._ll_masked.add if mask else self._ll_masked.discard)(rank_to_mask)

    def low_latency_query_mask_buffer(self, mask_status: torch.Tensor) -> None:
        self._require_shrink()
        mask_status.zero_()
        for r in self._ll_masked:
            mask_status[r] = 1

    def low_latency_clean_mask_buffer(self) -> None:
        self._require_shrink()
        self._ll_masked.clear()

    def clean_low_latency_buffer(self, num_max_dispatch_tokens_per_rank: int, hidden: int, num_experts: int) -> None:
        """Nothing persists between calls in the push design; this only lines the ranks up."""
        def gen():
            yield ("barrier",)
        self._drive(gen())

    # ------------------------------------------------------------------ dispatch
    def low_latency_dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, num_max_dispatch_tokens_per_rank: int, num_experts: int,
                             cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                             dispatch_wait_recv_cost_stats: Optional[torch.Tensor] = None, use_fp8: bool = True,
                             round_scale: bool = False, use_ue8m0: bool = False, async_finish: bool = False,
                             return_recv_hook: bool = False):
        """-> (recv_x | (recv_x_fp8, scales), recv_count [E_local] i32, handle, event, hook).
        recv_x is [E_local, ranks * max_tokens, H]; the first recv_count[e] rows of expert e are valid."""
        N, M = self.group_size, num_max_dispatch_tokens_per_rank
        T, H = x.shape
        if T > M:
            raise ValueError(f"{T} tokens exceed num_max_dispatch_tokens_per_rank={M}")
        El = num_experts // N
        idx = topk_idx
        if self._ll_masked:
            dst = torch.where(idx >= 0, idx // El, torch.zeros_like(idx))
            masked = torch.zeros_like(idx, dtype=torch.bool)
            for r in self._ll_masked:
                masked |= dst == r
            idx = torch.where(masked, torch.full_like(idx, -1), idx)
        idx = idx.contiguous()
        eng = self._engine

        def run():
            h = self._drive(eng.layout_gen(idx, num_experts))
            ones = torch.ones(T, idx.shape[1], dtype=torch.float32, device=x.device)
            tabs, _ = self._drive(eng.dispatch_gen(h, x.contiguous(), ones, with_meta=True))
            eng.snapshot_tables(h, tabs)
            rows = tabs["recv_x"][: h.rows].clone()
            self._release()
            xperm = eng.expand(rows, h)
            counts = h.expert_total_local.to(torch.int32)
            if int(counts.max()) > N * M if counts.numel() else False:
                raise RuntimeError("an expert received more rows than ranks * num_max_dispatch_tokens_per_rank")
            valid = (h.slot_tk >= 0).nonzero(as_tuple=True)[0]
            le = h.mblock_expert.long()[valid // 128]
            pos = valid - h.seg_offsets.long()[le]
            flat = le * (N * M) + pos
            packed = torch.zeros(El * N * M, H, dtype=x.dtype, device=x.device)
            packed[flat] = xperm[valid]
            packed = packed.view(El, N * M, H)
            handle = LowLatencyHandle(h, M, H, num_experts, flat, valid)
            if cumulative_local_expert_recv_stats is not None:
                cumulative_local_expert_recv_stats.add_(counts.to(cumulative_local_expert_recv_stats.dtype))
            if use_fp8:
                q, sc = fp8_quantize(packed, round_scale, use_ue8m0)
                return (q, sc), counts, handle
            return packed, counts, handle

        (recv, counts, handle), ev = self._on_comm_stream(run, None, async_finish, False)
        hook: Optional[Callable] = (lambda: None) if return_recv_hook else None
        return recv, counts, handle, ev, hook

    # ------------------------------------------------------------------ combine
    def get_next_low_latency_combine_buffer(self, handle: LowLatencyHandle) -> torch.Tensor:
        """A [E_local, ranks * max_tokens, H] bf16 tensor that experts may write their outputs into and
        hand to low_latency_combine(zero_copy=True)."""
        El = handle.num_experts // self.group_size
        shape = (El, self.group_size * handle.max_tokens, handle.hidden)
        buf = getattr(self, "_ll_combine_buffer", None)
        if buf is None or tuple(buf.shape) != shape:
            buf = torch.zeros(shape, dtype=torch.bfloat16 if self.device.type == "cuda" else torch.float32, device=self.device)
            self._ll_combine_buffer = buf
        return buf

    def low_latency_combine(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, handle: LowLatencyHandle,
                            use_logfmt: bool = False, zero_copy: bool = False, async_finish: bool = False,
                            return_recv_hook: bool = False, out: Optional[torch.Tensor] = None,
                            combine_wait_recv_cost_stats: Optional[torch.Tensor] = None):
        """Weighted reduce at the token's rank: out[t] = sum_k topk_weights[t,k] * x[row of (t,k)].
        -> (combined_x [T,H], event, hook)."""
        h = handle.layer
        eng = self._engine
        src = self.get_next_low_latency_combine_buffer(handle) if zero_copy else x

        def run():
            H = handle.hidden
            y = torch.zeros(h.slots, H, dtype=src.dtype, device=src.device)
            payload = src.reshape(-1, H)[handle.slot_index]
            if use_logfmt:
                payload = logfmt10_roundtrip(payload)
            y[handle.slot_ids] = payload
            res = self._drive(eng.slots_combine_gen(h, y, topk_weights.float().contiguous()))
            self._release()
            if out is not None:
                out.copy_(res)
                return out
            return res

        res, ev = self._on_comm_stream(run, None, async_finish, False)
        hook: Optional[Callable] = (lambda: None) if return_recv_hook else None
        return res, ev, hook
