"""Index math of deterministic expert-parallel routing, in plain PyTorch.

This is the executable specification of csrc/routing.cu (the CUDA kernels are tested against it)
and the CPU implementation used when tensors live on the host.

For a source rank with topk_idx [T,K] (global expert ids, -1 = none), N ranks, E experts
(El = E/N per rank, rank d owns experts [d*El, (d+1)*El)):

  counts row  C = E + N + 2 ints: per-expert entry counts, per-destination-rank distinct-token
              counts, the sum over tokens of distinct destination ranks, and the token count.
  All ranks all-gather their rows into meta [N, C]; everything below is a pure function of meta.

  slot(t,k)   = seg_off[e] + sum_{s<me} meta[s,e] + j(t,k)       on rank e // El
                seg_off[e] = sum over lower local experts of ceil128(total entries)
                j(t,k) = position of (t,k) among this source's entries of expert e, ordered by
                (t // 32, k, t % 32)  -- the order in which the CUDA kernel's warps visit them
  row(t,d)    = sum_{s<me} meta[s,E+d] + position of t among this source's tokens that hit rank d
  land(t,d)   = exclusive prefix of ndst over tokens + ordinal of d among t's destination ranks

Reference counterparts: csrc/kernels/layout.cu:9-121 (counts, is_token_in_rank) and the prefix
matrices of csrc/kernels/intranode.cu:11-113.  The reference claims slots with receiver-side
atomics (csrc/teramoe/teramoe_orchestrator.cu:1238-1259); here they are a function of the counts.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


def ceil128(v):
    return (v + 127) // 128 * 128


def count_row(topk_idx: torch.Tensor, E: int, N: int) -> torch.Tensor:
    """[E+N+2] int32 counts of one source rank (CPU tensor)."""
    idx = topk_idx.detach().cpu().long()
    T, K = idx.shape
    El = E // N
    valid = (idx >= 0) & (idx < E)
    row = torch.zeros(E + N + 2, dtype=torch.int64)
    if T > 0:
        row[:E] = torch.bincount(idx[valid], minlength=E)
        hit = token_rank_hits(idx, E, N)
        row[E:E + N] = hit.sum(0)
        row[E + N] = hit.sum()
    row[E + N + 1] = T
    return row.to(torch.int32)


def token_rank_hits(topk_idx: torch.Tensor, E: int, N: int) -> torch.Tensor:
    """is_token_in_rank [T,N] bool."""
    idx = topk_idx.detach().cpu().long()
    T, K = idx.shape
    El = E // N
    valid = (idx >= 0) & (idx < E)
    hit = torch.zeros(T, N, dtype=torch.bool)
    if T > 0:
        d = torch.where(valid, idx // El, torch.zeros_like(idx))
        hit.scatter_(1, d, valid)
        # scatter_ with duplicate destinations and mixed values is order dependent: redo with amax
        hit = torch.zeros(T, N, dtype=torch.int64).scatter_reduce_(1, d, valid.long(), reduce="amax").bool()
    return hit


@dataclass
class GlobalLayout:
    """Quantities every rank derives identically from the gathered counts."""
    expert_total: torch.Tensor   # [E]
    seg_off_all: torch.Tensor    # [E]   offset of e's padded segment in its rank's slot space
    slots_padded: torch.Tensor   # [N]   padded slot rows per rank
    rows: torch.Tensor           # [N]   token-once receive rows per rank
    land_rows: torch.Tensor      # [N]   combine landing rows per source rank
    src_off: torch.Tensor        # [N,E] rows of lower sources inside each expert segment
    row_base: torch.Tensor       # [N(dst),N(src)] first receive row of source s on rank d


def global_layout(meta: torch.Tensor, E: int, N: int) -> GlobalLayout:
    meta = meta.detach().cpu().long()
    El = E // N
    cnt = meta[:, :E]
    tot = cnt.sum(0)
    pad = ceil128(tot).view(N, El)
    seg = (torch.cumsum(pad, 1) - pad).reshape(E)
    src_off = torch.cumsum(cnt, 0) - cnt
    rowcnt = meta[:, E:E + N]            # [src, dst]
    row_base = (torch.cumsum(rowcnt, 0) - rowcnt).t().contiguous()   # [dst, src]
    return GlobalLayout(tot, seg, pad.sum(1), rowcnt.sum(0), meta[:, E + N].clone(), src_off, row_base)


@dataclass
class SendLayout:
    send_slot: torch.Tensor  # [T,K] int32  slot on the destination rank (-1 = no expert)
    send_row: torch.Tensor   # [T,N] int32  row in rank d's receive buffer (-1 = not sent)
    land_off: torch.Tensor   # [T]   int32  first landing row of token t
    ndst: torch.Tensor       # [T]   int32  number of distinct destination ranks


def send_layout(topk_idx: torch.Tensor, E: int, N: int, rank: int, gl: GlobalLayout) -> SendLayout:
    idx = topk_idx.detach().cpu().long()
    T, K = idx.shape
    El = E // N
    valid = (idx >= 0) & (idx < E)
    send_slot = torch.full((T, K), -1, dtype=torch.int64)
    if T > 0 and valid.any():
        t_ar = torch.arange(T).view(T, 1).expand(T, K)
        k_ar = torch.arange(K).view(1, K).expand(T, K)
        key = (t_ar // 32) * (K * 32) + k_ar * 32 + (t_ar % 32)
        e_v, key_v = idx[valid], key[valid]
        order = torch.argsort(e_v * (key.max() + 1) + key_v)
        e_sorted = e_v[order]
        first = torch.searchsorted(e_sorted, e_sorted, right=False)
        j = torch.empty_like(order)
        j[order] = torch.arange(order.numel()) - first
        send_slot[valid] = gl.seg_off_all[e_v] + gl.src_off[rank][e_v] + j
    hit = token_rank_hits(idx, E, N)
    pos = torch.cumsum(hit.long(), 0) - hit.long()
    send_row = torch.where(hit, gl.row_base[:, rank].view(1, N) + pos, torch.full((T, N), -1, dtype=torch.int64))
    ndst = hit.sum(1)
    land_off = torch.cumsum(ndst, 0) - ndst
    return SendLayout(send_slot.to(torch.int32), send_row.to(torch.int32), land_off.to(torch.int32), ndst.to(torch.int32))


def wire_rank_plan(topk_idx: torch.Tensor, send_slot: torch.Tensor, E: int, N: int):
    """Once-per-rank wire format of the layer kernel's dispatch (csrc/layer.cu, `wire_rank`), as index math.

    Of a token's entries on one destination rank only the HOME entry carries the row: the one with the smallest slot
    there (slots of a rank grow with the local expert id, so the home is also the first of them the receiver works on).
    The other entries (siblings) get their table entries and `slot_src` = the home's slot; the receiver copies the row.

    -> (home [T,K] bool, src_slot [T,K] int64): src_slot is -1 for invalid entries and for homes, else the home's slot on
    the same rank.  Rows on the wire = home.sum(): one per (token, destination rank)."""
    idx = topk_idx.detach().cpu().long()
    slot = send_slot.detach().cpu().long().view(idx.shape)
    T, K = idx.shape
    El = E // N
    valid = (idx >= 0) & (idx < E) & (slot >= 0)
    dst = torch.where(valid, idx // El, torch.full_like(idx, -1))
    big = torch.iinfo(torch.int64).max
    home_slot = torch.full((T, K), -1, dtype=torch.int64)
    for d in range(N):
        on_d = dst == d
        smallest = torch.where(on_d, slot, torch.full_like(slot, big)).min(dim=1, keepdim=True).values     # [T,1]
        home_slot = torch.where(on_d, smallest.expand(T, K), home_slot)
    home = valid & (slot == home_slot)
    src_slot = torch.where(valid & ~home, home_slot, torch.full_like(slot, -1))
    return home, src_slot


def recv_tables(rank: int, E: int, N: int, gl: GlobalLayout):
    """This rank's segment table and block->expert map: (seg_offsets [El+1], mblock_expert [S/128])."""
    El = E // N
    seg = gl.seg_off_all.view(N, El)[rank]
    tot = gl.expert_total.view(N, El)[rank]
    spad = int(gl.slots_padded[rank])
    seg_offsets = torch.cat([seg, torch.tensor([spad])]).to(torch.int32)
    me = torch.repeat_interleave(torch.arange(El), (ceil128(tot) // 128)).to(torch.int32)
    return seg_offsets, me


def imbalanced_topk(T: int, K: int, E: int, peak_to_mean: float, generator: torch.Generator | None = None,
                    device="cpu") -> torch.Tensor:
    """Sample top-k expert choices from a Zipf-like distribution tuned so that the expected
    max-per-expert load is `peak_to_mean` times the mean (1.0 = uniform)."""
    if peak_to_mean <= 1.0 + 1e-6:
        p = torch.ones(E, dtype=torch.float64)
    else:
        lo, hi = 0.0, 4.0
        for _ in range(60):
            a = (lo + hi) / 2
            p = 1.0 / torch.arange(1, E + 1, dtype=torch.float64) ** a
            # inclusion probability of the hottest expert when drawing K without replacement (approx.)
            q = 1 - (1 - p / p.sum()) ** K
            ratio = float(q.max() / q.mean())
            if ratio < peak_to_mean:
                lo = a
            else:
                hi = a
        p = 1.0 / torch.arange(1, E + 1, dtype=torch.float64) ** ((lo + hi) / 2)
    p = (p / p.sum()).float()
    perm = torch.randperm(E, generator=generator)
    p = p[perm]
    idx = torch.multinomial(p.expand(T, E), K, replacement=False, generator=generator)
    return idx.to(device)
