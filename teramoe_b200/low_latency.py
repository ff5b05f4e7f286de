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
    layer: Optional[LayerHandle]
    max_tokens: int
    hidden: int
    num_experts: int
    slot_index: Optional[torch.Tensor] = None     # host path: [valid slots] flat row in the packed [E_local * ranks * max_tokens] layout
    slot_ids: Optional[torch.Tensor] = None       # host path: [valid slots] slot-space row
    # kernel path (csrc/lowlat.cu): where every packed row came from, like the reference's handle
    # (packed_recv_src_info, packed_recv_layout_range; teramoe/buffer.py:606-612)
    src_info: Optional[torch.Tensor] = None       # [E_local, ranks*max_tokens] token index at the source
    layout_range: Optional[torch.Tensor] = None   # [E_local, ranks] int64: rows << 32 | first row
    seq: int = 0                                  # call number the flags of this dispatch / its combine carry


def _ll_geometry(N: int, rank: int, E: int, M: int, H: int, use_fp8: bool, use_ue8m0: bool, round_scale: bool, use_logfmt: bool):
    """Byte layout of the low-latency windows in the symmetric arena (csrc/lowlat.h LowLatLayout) -> (list for the
    bindings, total bytes, (flag offset, flag bytes) ranges)."""
    El, G = E // N, H // 128
    d_msg = 16 + ((H + (G if use_ue8m0 else 4 * G)) if use_fp8 else 2 * H)
    d_msg = (d_msg + 15) // 16 * 16
    c_row = G * 272 if use_logfmt else 2 * H
    r256 = lambda v: (v + 255) // 256 * 256
    off_d_stage = 0
    off_d_flags = r256(off_d_stage + El * N * M * d_msg)
    off_c_stage = r256(off_d_flags + El * N * 8)
    off_c_flags = r256(off_c_stage + E * M * c_row)
    total = r256(off_c_flags + E * 8)
    geom = [N, rank, E, M, H, int(use_fp8), int(use_ue8m0), int(round_scale), int(use_logfmt), off_d_stage, off_d_flags, off_c_stage,
            off_c_flags, d_msg, c_row]
    return geom, total, ((off_d_flags, El * N * 8), (off_c_flags, E * 8))


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


def _flatten(v):
    return list(v) if isinstance(v, tuple) else [v]


class LowLatencyMixin:
    """Methods mixed into `Buffer` (they use its `_engine`, `_drive`, `_world`, `group_size`)."""

    # ------------------------------------------------------------------ rank mask (elastic shrink)
    def _require_shrink(self):
        if not self.enable_shrink:
            raise RuntimeError("the rank-mask API needs Buffer(enable_shrink=True)")

    def _ll_mask_tensor(self) -> Optional[torch.Tensor]:
        """Device int[ranks]: 1 = the rank is ignored by the low-latency kernels and by their barrier (nothing is sent
        to it, nothing awaited from it).  Kernels set entries themselves when a wait runs out in shrink mode."""
        if self.device.type != "cuda":
            return None
        if getattr(self, "_ll_mask_dev", None) is None:
            self._ll_mask_dev = torch.zeros(self.group_size, dtype=torch.int32, device=self.device)
        return self._ll_mask_dev

    def low_latency_update_mask_buffer(self, rank_to_mask: int, mask: bool = False) -> None:
        self._require_shrink()
        if not 0 <= rank_to_mask < self.group_size:
            raise ValueError("rank out of range")
        if self.device.type == "cuda":
            self._world.ext.ll_mask_update(self._ll_mask_tensor(), rank_to_mask, 1 if mask else 0)
        else:
            (self._ll_masked.add if mask else self._ll_masked.discard)(rank_to_mask)

    def low_latency_query_mask_buffer(self, mask_status: torch.Tensor) -> None:
        self._require_shrink()
        if self.device.type == "cuda" and mask_status.is_cuda and mask_status.dtype == torch.int32:
            self._world.ext.ll_mask_query(self._ll_mask_tensor(), mask_status)
            return
        mask_status.zero_()
        masked = self._ll_mask_tensor().nonzero().flatten().tolist() if self.device.type == "cuda" else self._ll_masked
        for r in masked:
            mask_status[r] = 1

    def low_latency_clean_mask_buffer(self) -> None:
        self._require_shrink()
        if self.device.type == "cuda":
            self._world.ext.ll_mask_clean(self._ll_mask_tensor())
        else:
            self._ll_masked.clear()

    def clean_low_latency_buffer(self, num_max_dispatch_tokens_per_rank: int, hidden: int, num_experts: int) -> None:
        """The flags of the low-latency windows carry the call number, so nothing has to be cleaned between calls; this
        lines the ranks up (masked ranks left out) like the reference's clean kernel does as a side effect."""
        mask = self._ll_mask_tensor() if self.enable_shrink else None

        def gen():
            yield ("masked_barrier", mask) if mask is not None else ("barrier",)
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
        if x.is_cuda:
            return self._ll_dispatch_cuda(x, topk_idx, M, num_experts, cumulative_local_expert_recv_stats, dispatch_wait_recv_cost_stats,
                                          use_fp8, round_scale, use_ue8m0, async_finish, return_recv_hook)
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

    # ------------------------------------------------------------------ kernel path (csrc/lowlat.cu)
    def _ll_prepare(self, M, H, E, use_fp8, use_ue8m0, round_scale, use_logfmt):
        """Geometry of the windows for these sizes; on a change (or after other users of the arena) the flag words are
        cleared and the ranks cross a barrier, so that no stale bytes can pass for a flag of this call."""
        w = self._world
        geom, total, flag_ranges = _ll_geometry(self.group_size, self.rank, E, M, H, use_fp8, use_ue8m0, round_scale, use_logfmt)
        key = ("ll", M, H, E, geom[13], geom[14])

        def gen():
            yield ("grow", total)
            if w.arena_user != key:
                for off, n in flag_ranges:
                    w.data.view(off, [n // 8], torch.int64).zero_()
                yield ("barrier",)
                w.arena_user = key
            yield ("acquire",)
        self._drive(gen())
        return geom

    def _ll_dispatch_cuda(self, x, topk_idx, M, num_experts, expert_stats, wait_stats, use_fp8, round_scale, use_ue8m0, async_finish,
                          return_recv_hook):
        w, ext = self._world, self._world.ext
        N, T, H = self.group_size, x.shape[0], x.shape[1]
        El, G = num_experts // N, x.shape[1] // 128
        if H % 256 != 0:
            raise ValueError("the low-latency kernels need hidden % 256 == 0")
        if use_ue8m0 and not (use_fp8 and round_scale and H % 512 == 0):
            raise ValueError("UE8M0 scales need use_fp8, round_scale and hidden % 512 == 0")
        mask = self._ll_mask_tensor() if self.enable_shrink else None
        dev = x.device

        def send():
            geom = self._ll_prepare(M, H, num_experts, use_fp8, use_ue8m0, round_scale, getattr(self, "_ll_logfmt", False))
            self._ll_seq = getattr(self, "_ll_seq", 0) + 1
            ext.ll_dispatch_send(geom, x.contiguous(), topk_idx.contiguous(), w.ptr_table(w.data, 0, "data"), self._ll_seq, mask)
            return geom, self._ll_seq

        NM = N * M

        def alloc():
            recv_x = torch.empty(El, NM, H, dtype=torch.float8_e4m3fn if use_fp8 else torch.bfloat16, device=dev)
            scales = None
            if use_fp8:
                scales = (torch.empty(El, G // 4, NM, dtype=torch.int32, device=dev) if use_ue8m0
                          else torch.empty(El, G, NM, dtype=torch.float32, device=dev))
            return (recv_x, scales, torch.empty(El, NM, dtype=torch.int32, device=dev), torch.empty(El, N, dtype=torch.int64, device=dev),
                    torch.empty(El, dtype=torch.int32, device=dev))

        def recv(geom, seq, bufs):
            recv_x, scales, src_info, layout_range, recv_count = bufs
            ext.ll_dispatch_recv(geom, w.data.view(0, [16], torch.uint8), recv_x, scales, src_info, layout_range, recv_count, expert_stats,
                                 wait_stats, seq, mask, bool(self.enable_shrink), w.wait_limit_ms, w.status)
            self._release()

        def results(geom, seq, bufs):
            recv_x, scales, src_info, layout_range, recv_count = bufs
            handle = LowLatencyHandle(None, M, H, num_experts, src_info=src_info, layout_range=layout_range, seq=seq)
            handle.geom = geom
            # scales come back [E_local, ranks*max_tokens, groups] over column-major storage, like the reference's
            return ((recv_x, scales.transpose(1, 2)) if use_fp8 else recv_x), recv_count, handle

        if return_recv_hook:
            # two phases (csrc/kernels/internode_ll.cu: LOW_LATENCY_SEND_PHASE / RECV_PHASE): the call sends, the hook
            # receives into the tensors that the call already hands out
            (geom, seq), ev = self._on_comm_stream(send, None, False, False)
            bufs = alloc()
            state = {"done": False}

            def hook():
                if not state["done"]:
                    state["done"] = True
                    self._on_comm_stream(lambda: recv(geom, seq, bufs), None, False, False)
            recv_out, counts, handle = results(geom, seq, bufs)
            return recv_out, counts, handle, ev, hook

        def both():
            geom, seq = send()
            bufs = alloc()
            recv(geom, seq, bufs)
            return results(geom, seq, bufs)
        (recv_out, counts, handle), ev = self._on_comm_stream(both, None, async_finish, False)
        return recv_out, counts, handle, ev, None

    def _ll_combine_cuda(self, x, topk_idx, topk_weights, handle, use_logfmt, async_finish, return_recv_hook, out, wait_stats):
        w, ext = self._world, self._world.ext
        N, M, H, E = self.group_size, handle.max_tokens, handle.hidden, handle.num_experts
        mask = self._ll_mask_tensor() if self.enable_shrink else None
        T = topk_idx.shape[0]
        geom = list(handle.geom)
        if bool(geom[8]) != bool(use_logfmt):
            # the combine windows of this call have another row format than the dispatch planned for: lay them out again
            self._ll_logfmt = bool(use_logfmt)
            geom = self._ll_prepare(M, H, E, bool(geom[5]), bool(geom[6]), bool(geom[7]), bool(use_logfmt))
        res = out if out is not None else torch.empty(T, H, dtype=torch.bfloat16, device=x.device)

        def send():
            ext.ll_combine_send(geom, x.contiguous(), handle.src_info, handle.layout_range, w.ptr_table(w.data, 0, "data"), handle.seq, mask)

        def recv():
            ext.ll_combine_recv(geom, w.data.view(0, [16], torch.uint8), topk_idx.contiguous(), topk_weights.float().contiguous(), res, wait_stats,
                                handle.seq, mask, bool(self.enable_shrink), w.wait_limit_ms, w.status)
            self._release()
            return res

        if return_recv_hook:
            _, ev = self._on_comm_stream(send, None, False, False)
            state = {"done": False}

            def hook():
                if not state["done"]:
                    state["done"] = True
                    self._on_comm_stream(recv, None, False, False)
            return res, ev, hook
        _, ev = self._on_comm_stream(lambda: (send(), recv())[1], None, async_finish, False)
        return res, ev, None

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
        src = self.get_next_low_latency_combine_buffer(handle) if zero_copy else x
        if handle.src_info is not None:
            return self._ll_combine_cuda(src, topk_idx, topk_weights, handle, use_logfmt, async_finish, return_recv_hook, out,
                                         combine_wait_recv_cost_stats)
        h = handle.layer
        eng = self._engine

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
