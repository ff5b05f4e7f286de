"""Grouped expert GEMMs on tcgen05 (csrc/gemm.cu) with plain-PyTorch restatements for CPU tests.

Slot space: rows sorted by local expert, every expert's segment padded to a multiple of 128 rows
(`seg_offsets[e]..seg_offsets[e+1]`), pad rows zero with route weight 0.  `mblock_expert[b]` is
the expert of 128-row block `b`; `num_mblocks` is a device scalar with the live block count.

Reference counterparts: teramoe/buffer.py:745-760 (weight-gradient GEMMs),
csrc/teramoe/teramoe_orchestrator.cu:1813-1876 (forward GEMM pair), :4696-4811 (backward pair).
"""
from __future__ import annotations

import torch

from .._build import load_ext


def _status_check(status: torch.Tensor | None) -> None:
    if status is None:
        return
    s = status.tolist()
    if s[0] != 0:
        raise RuntimeError(f"teramoe_b200 kernel gave up: code={s[0]} site={s[1]} block={s[2]} detail={s[3]}")


def num_droute_parts(I: int) -> int:
    return 2 * ((I + 255) // 256)


def _lay(mblock_expert, num_mblocks, units):
    """Block layout list for the bindings; `units` = (unit_blk, num_units) selects the CTA-pair kernels."""
    return [mblock_expert, num_mblocks] + (list(units) if units is not None else [])


def make_units(mblock_expert: torch.Tensor):
    """Host-side unit table (tests): pairs of consecutive blocks of one expert -> (unit_blk, num_units)."""
    me = mblock_expert.tolist()
    ub, b = [], 0
    while b < len(me):
        e, start = me[b], b
        while b < len(me) and me[b] == e:
            b += 1
        ub += list(range(start, b, 2))
    ub.append(len(me))
    dev = mblock_expert.device
    return torch.tensor(ub, dtype=torch.int32, device=dev), torch.tensor([len(ub) - 1], dtype=torch.int32, device=dev)


def _gathered(rows, gather_rows):
    """Plain restatement of the TMA row gather: slot space <- rows[gather_rows], -1 gives zero rows."""
    g = gather_rows.long()
    return torch.where((g >= 0)[:, None], rows[g.clamp(min=0)], torch.zeros((), dtype=rows.dtype, device=rows.device))


def fwd_gateup(xperm, w_gateup, row_w, mblock_expert, num_mblocks, status=None, num_sms=0, gather_rows=None, units=None):
    """-> (act [S,I], preact [S,2I]).  act = silu(g)*u*row_w, preact = (g,u) interleaved bf16.
    With `gather_rows` [S], `xperm` is a row source [R,H] and slot row s reads xperm[gather_rows[s]]."""
    S, H = (gather_rows.numel() if gather_rows is not None else xperm.shape[0]), xperm.shape[1]
    I = w_gateup.shape[1] // 2
    act = torch.empty(S, I, dtype=xperm.dtype, device=xperm.device)
    preact = torch.empty(S, 2 * I, dtype=xperm.dtype, device=xperm.device)
    if xperm.is_cuda:
        load_ext().gemm_fwd_gateup(xperm, w_gateup, act, preact, row_w, _lay(mblock_expert, num_mblocks, units), gather_rows, status, num_sms)
    else:
        if gather_rows is not None:
            xperm = _gathered(xperm, gather_rows)
        ref_fwd_gateup(xperm, w_gateup, row_w, mblock_expert, int(num_mblocks), act, preact)
    return act, preact


def fwd_down(act, w_down, mblock_expert, num_mblocks, status=None, num_sms=0, units=None, push=None):
    """y[S,H] = act @ W_down[e]^T.  With push = ([arena_ptrs, slot_tk, slot_row, recv_row_base], landing_off) the rows
    are stored straight into their source ranks' landing tables by the GEMM epilogue and None is returned."""
    S, I = act.shape
    H = w_down.shape[1]
    if push is not None:
        load_ext().gemm_fwd_down(act, w_down, None, _lay(mblock_expert, num_mblocks, units), status, num_sms, push[0], push[1])
        return None
    y = torch.empty(S, H, dtype=act.dtype, device=act.device)
    if act.is_cuda:
        load_ext().gemm_fwd_down(act, w_down, y, _lay(mblock_expert, num_mblocks, units), status, num_sms, None, 0)
    else:
        ref_mgroup(act, w_down.transpose(1, 2), mblock_expert, int(num_mblocks), y)
    return y


def bwd_gradact(dyperm, w_down, preact, row_w, mblock_expert, num_mblocks, status=None, num_sms=0, gather_rows=None, units=None):
    """-> (dgu [S,2I], act_w [S,I], droute partial sums [S, parts] fp32)."""
    S, H = (gather_rows.numel() if gather_rows is not None else dyperm.shape[0]), dyperm.shape[1]
    I = w_down.shape[2]
    dgu = torch.empty(S, 2 * I, dtype=dyperm.dtype, device=dyperm.device)
    act_w = torch.empty(S, I, dtype=dyperm.dtype, device=dyperm.device)
    if dyperm.is_cuda:
        parts = torch.empty(S, num_droute_parts(I), dtype=torch.float32, device=dyperm.device)
        load_ext().gemm_bwd_gradact(dyperm, w_down, preact, row_w, dgu, act_w, parts, _lay(mblock_expert, num_mblocks, units), gather_rows, status,
                                    num_sms)
        return dgu, act_w, parts
    if gather_rows is not None:
        dyperm = _gathered(dyperm, gather_rows)
    parts = torch.zeros(S, num_droute_parts(I), dtype=torch.float32)
    ref_bwd_gradact(dyperm, w_down, preact, row_w, mblock_expert, int(num_mblocks), dgu, act_w, parts)
    return dgu, act_w, parts


def bwd_dx(dgu, w_gateup, mblock_expert, num_mblocks, status=None, num_sms=0, units=None, push=None):
    S = dgu.shape[0]
    H = w_gateup.shape[2]
    if push is not None:
        load_ext().gemm_bwd_dx(dgu, w_gateup, None, _lay(mblock_expert, num_mblocks, units), status, num_sms, push[0], push[1])
        return None
    dx = torch.empty(S, H, dtype=dgu.dtype, device=dgu.device)
    if dgu.is_cuda:
        load_ext().gemm_bwd_dx(dgu, w_gateup, dx, _lay(mblock_expert, num_mblocks, units), status, num_sms, None, 0)
    else:
        ref_mgroup(dgu, w_gateup, mblock_expert, int(num_mblocks), dx)
    return dx


def wgrad(a, b, seg_offsets, num_local_experts, status=None, num_sms=0, gather_rows=None, gather_operand=0, cta_pairs=False):
    """dW[e] = a[seg_e]^T @ b[seg_e]  -> [E, a.shape[1], b.shape[1]] bf16 (zeros for empty experts).
    gather_operand 1 / 2: operand a / b is a row source read through gather_rows."""
    M, N = a.shape[1], b.shape[1]
    dw = torch.empty(num_local_experts, M, N, dtype=a.dtype, device=a.device)
    S = gather_rows.numel() if (gather_rows is not None and gather_operand) else a.shape[0]
    if S == 0 or a.shape[0] == 0 or b.shape[0] == 0:
        return dw.zero_()
    if a.is_cuda:
        load_ext().gemm_wgrad(a, b, dw, seg_offsets, gather_rows, gather_operand if gather_rows is not None else 0, cta_pairs, status, num_sms)
    else:
        if gather_rows is not None and gather_operand == 1:
            a = _gathered(a, gather_rows)
        if gather_rows is not None and gather_operand == 2:
            b = _gathered(b, gather_rows)
        offs = seg_offsets.tolist()
        for e in range(num_local_experts):
            s0, s1 = offs[e], offs[e + 1]
            dw[e] = (a[s0:s1].float().t() @ b[s0:s1].float()).to(dw.dtype)
    return dw


# ------------------------------------------------------------------------------------------------
# Plain PyTorch restatements (fp32 math, bf16 rounding where the kernels round).  Used on CPU and as
# the oracle of the GPU numerics tests.
# ------------------------------------------------------------------------------------------------
def ref_mgroup(a, b_kn, mblock_expert, num_mblocks, out):
    """out[blk] = a[blk] @ b_kn[e]; b_kn is [E, K, N] (any strides)."""
    out.zero_()
    me = mblock_expert.tolist()
    for blk in range(num_mblocks):
        r = slice(blk * 128, blk * 128 + 128)
        out[r] = (a[r].float() @ b_kn[me[blk]].float()).to(out.dtype)


def ref_fwd_gateup(xperm, w_gateup, row_w, mblock_expert, num_mblocks, act, preact):
    act.zero_()
    preact.zero_()
    me = mblock_expert.tolist()
    for blk in range(num_mblocks):
        r = slice(blk * 128, blk * 128 + 128)
        gu = xperm[r].float() @ w_gateup[me[blk]].float().t()
        g, u = gu[:, 0::2], gu[:, 1::2]
        act[r] = (g * torch.sigmoid(g) * u * row_w[r].float()[:, None]).to(act.dtype)
        preact[r] = gu.to(preact.dtype)


def ref_bwd_gradact(dyperm, w_down, preact, row_w, mblock_expert, num_mblocks, dgu, act_w, parts):
    dgu.zero_()
    act_w.zero_()
    parts.zero_()
    me = mblock_expert.tolist()
    for blk in range(num_mblocks):
        r = slice(blk * 128, blk * 128 + 128)
        ga = dyperm[r].float() @ w_down[me[blk]].float()  # [128, I]
        g = preact[r, 0::2].float()
        u = preact[r, 1::2].float()
        w = row_w[r].float()[:, None]
        sig = torch.sigmoid(g)
        s = g * sig
        a = s * u
        gaw = ga * w
        d_up = s * gaw
        d_gate = (sig - s * sig + s) * gaw * u
        out = torch.stack([d_gate, d_up], dim=-1).reshape(128, -1)
        dgu[r] = out.to(dgu.dtype)
        act_w[r] = (a * w).to(act_w.dtype)
        parts[r, 0] = (ga * a).sum(dim=1)
