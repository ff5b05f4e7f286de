"""tcgen05 grouped GEMM kernels vs plain PyTorch fp32 (bf16 tolerance)."""
import pytest
import torch

from teramoe_b200.ops import gemm

pytestmark = pytest.mark.gpu


def _layout(counts, device):
    """Padded segment offsets / block->expert map for per-expert row counts."""
    offs = [0]
    me = []
    for e, c in enumerate(counts):
        pad = (c + 127) // 128 * 128
        offs.append(offs[-1] + pad)
        me += [e] * (pad // 128)
    S = offs[-1]
    valid = torch.zeros(S, dtype=torch.bool)
    for e, c in enumerate(counts):
        valid[offs[e]:offs[e] + c] = True
    return (S, torch.tensor(offs, dtype=torch.int32, device=device), torch.tensor(me, dtype=torch.int32, device=device),
            torch.tensor([len(me)], dtype=torch.int32, device=device), valid.to(device))


def _close(a, b, atol=1e-2, rtol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert err <= atol + rtol * ref, f"max err {err} (ref max {ref})"
    if ref > 0:
        cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
        assert cos > 0.999, f"cosine {cos}"


CASES = [
    # H, I, counts
    (256, 512, [100, 0, 300, 128]),
    (512, 256, [5, 700]),
    (1024, 1536, [257, 255, 1, 511, 130]),
]


@pytest.mark.parametrize("H,I,counts", CASES)
def test_forward_pair(H, I, counts):
    dev = "cuda"
    torch.manual_seed(0)
    E = len(counts)
    S, offs, me, nmb, valid = _layout(counts, dev)
    x = (torch.randn(S, H, device=dev) * 0.5).to(torch.bfloat16) * valid[:, None]
    wgu = (torch.randn(E, 2 * I, H, device=dev) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device=dev) * 0.05).to(torch.bfloat16)
    row_w = torch.rand(S, device=dev) * valid
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    act, preact = gemm.fwd_gateup(x, wgu, row_w, me, nmb, status)
    y = gemm.fwd_down(act, wd, me, nmb, status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, status.tolist()
    act_r = torch.empty_like(act)
    pre_r = torch.empty_like(preact)
    gemm.ref_fwd_gateup(x, wgu, row_w, me, len(me.tolist()), act_r, pre_r)
    y_r = torch.empty_like(y)
    gemm.ref_mgroup(act_r, wd.transpose(1, 2), me, len(me.tolist()), y_r)
    _close(preact, pre_r)
    _close(act, act_r)
    _close(y, y_r)


@pytest.mark.parametrize("H,I,counts", CASES)
def test_backward_pair(H, I, counts):
    dev = "cuda"
    torch.manual_seed(1)
    E = len(counts)
    S, offs, me, nmb, valid = _layout(counts, dev)
    dy = (torch.randn(S, H, device=dev) * 0.5).to(torch.bfloat16) * valid[:, None]
    preact = (torch.randn(S, 2 * I, device=dev)).to(torch.bfloat16) * valid[:, None]
    wgu = (torch.randn(E, 2 * I, H, device=dev) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device=dev) * 0.05).to(torch.bfloat16)
    row_w = torch.rand(S, device=dev) * valid
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    dgu, act_w, parts = gemm.bwd_gradact(dy, wd, preact, row_w, me, nmb, status)
    dx = gemm.bwd_dx(dgu, wgu, me, nmb, status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, status.tolist()
    dgu_r, aw_r = torch.empty_like(dgu), torch.empty_like(act_w)
    parts_r = torch.zeros_like(parts)
    gemm.ref_bwd_gradact(dy, wd, preact, row_w, me, len(me.tolist()), dgu_r, aw_r, parts_r)
    dx_r = torch.empty_like(dx)
    gemm.ref_mgroup(dgu_r, wgu, me, len(me.tolist()), dx_r)
    _close(dgu, dgu_r)
    _close(act_w, aw_r)
    _close(parts.sum(1), parts_r.sum(1), atol=5e-2)
    _close(dx, dx_r)


@pytest.mark.parametrize("M,N,counts", [(512, 256, [100, 0, 300, 128]), (1024, 768, [5, 700]), (200, 264, [129, 0])])
def test_wgrad(M, N, counts):
    dev = "cuda"
    torch.manual_seed(2)
    E = len(counts)
    S, offs, me, nmb, valid = _layout(counts, dev)
    a = (torch.randn(S, M, device=dev) * 0.5).to(torch.bfloat16) * valid[:, None]
    b = (torch.randn(S, N, device=dev) * 0.5).to(torch.bfloat16) * valid[:, None]
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    dw = gemm.wgrad(a, b, offs, E, status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, status.tolist()
    o = offs.tolist()
    for e in range(E):
        ref = a[o[e]:o[e + 1]].float().t() @ b[o[e]:o[e + 1]].float()
        _close(dw[e], ref, atol=5e-2)
    assert dw[1].abs().max().item() == 0.0 or counts[1] != 0


@pytest.mark.parametrize("H,I,counts", CASES)
def test_gather_modes_match_dense(H, I, counts):
    """Row-gather operands (TMA gather4 from a token-once row source) give bitwise the dense results."""
    from teramoe_b200._build import load_ext
    if not load_ext().gemm_has_gather4():
        pytest.skip("the gather4 operand modes are only built with -DTMOE_WITH_GATHER4 (measured too slow for the hot path)")
    dev = "cuda"
    torch.manual_seed(3)
    E = len(counts)
    S, offs, me, nmb, valid = _layout(counts, dev)
    R = max(1, int(valid.sum().item()) // 2 + 3)
    rows = (torch.randn(R, H, device=dev) * 0.5).to(torch.bfloat16)
    gidx = torch.where(valid, torch.randint(0, R, (S,), device=dev), torch.full((S,), -1, device=dev)).to(torch.int32)
    dense = gemm._gathered(rows, gidx).contiguous()
    wgu = (torch.randn(E, 2 * I, H, device=dev) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device=dev) * 0.05).to(torch.bfloat16)
    row_w = torch.rand(S, device=dev) * valid
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    a1, p1 = gemm.fwd_gateup(dense, wgu, row_w, me, nmb, st)
    a2, p2 = gemm.fwd_gateup(rows, wgu, row_w, me, nmb, st, gather_rows=gidx)
    assert torch.equal(a1, a2) and torch.equal(p1, p2)
    d1 = gemm.bwd_gradact(dense, wd, p1, row_w, me, nmb, st)
    d2 = gemm.bwd_gradact(rows, wd, p1, row_w, me, nmb, st, gather_rows=gidx)
    for x, y in zip(d1, d2):
        assert torch.equal(x, y)
    other = (torch.randn(S, I, device=dev) * 0.5).to(torch.bfloat16) * valid[:, None]
    w1 = gemm.wgrad(dense, other, offs, E, st)
    w2 = gemm.wgrad(rows, other, offs, E, st, gather_rows=gidx, gather_operand=1)
    assert torch.equal(w1, w2)
    w3 = gemm.wgrad(other, dense, offs, E, st)
    w4 = gemm.wgrad(other, rows, offs, E, st, gather_rows=gidx, gather_operand=2)
    assert torch.equal(w3, w4)
    torch.cuda.synchronize()
    assert st.tolist()[0] == 0


@pytest.mark.parametrize("H,I,counts", CASES + [(512, 512, [128, 256, 0, 384, 129])])
def test_cta_pair_kernels_match_one_cta(H, I, counts):
    """cta_group::2 (256x256 tiles over CTA pairs) kernels give bitwise the one-CTA results."""
    dev = "cuda"
    torch.manual_seed(4)
    E = len(counts)
    S, offs, me, nmb, valid = _layout(counts, dev)
    units = gemm.make_units(me)
    x = (torch.randn(S, H, device=dev) * 0.5).to(torch.bfloat16) * valid[:, None]
    wgu = (torch.randn(E, 2 * I, H, device=dev) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device=dev) * 0.05).to(torch.bfloat16)
    row_w = torch.rand(S, device=dev) * valid
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    a1, p1 = gemm.fwd_gateup(x, wgu, row_w, me, nmb, st)
    a2, p2 = gemm.fwd_gateup(x, wgu, row_w, me, nmb, st, units=units)
    torch.cuda.synchronize()
    assert st.tolist()[0] == 0, st.tolist()
    assert torch.equal(p1, p2) and torch.equal(a1, a2)
    y1 = gemm.fwd_down(a1, wd, me, nmb, st)
    y2 = gemm.fwd_down(a1, wd, me, nmb, st, units=units)
    assert torch.equal(y1, y2)
    d1 = gemm.bwd_gradact(x, wd, p1, row_w, me, nmb, st)
    d2 = gemm.bwd_gradact(x, wd, p1, row_w, me, nmb, st, units=units)
    for u, v in zip(d1, d2):
        assert torch.equal(u, v)
    x1 = gemm.bwd_dx(d1[0], wgu, me, nmb, st)
    x2 = gemm.bwd_dx(d1[0], wgu, me, nmb, st, units=units)
    assert torch.equal(x1, x2)
    w1 = gemm.wgrad(d1[0], x, offs, E, st)
    w2 = gemm.wgrad(d1[0], x, offs, E, st, cta_pairs=True)
    assert torch.equal(w1, w2)
    w3 = gemm.wgrad(x, d1[1], offs, E, st)
    w4 = gemm.wgrad(x, d1[1], offs, E, st, cta_pairs=True)
    assert torch.equal(w3, w4)
    torch.cuda.synchronize()
    assert st.tolist()[0] == 0, st.tolist()
