"""Low-latency API (packed per-expert receive, FP8 payload, weighted combine, rank mask) on CPU ranks."""
import pytest
import torch

import teramoe_b200 as tm
from teramoe_b200.low_latency import fp8_dequantize, fp8_quantize, logfmt10_roundtrip


def _problem(T=40, H=256, E=8, K=3, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g)
    top = torch.topk(torch.randn(T, E, generator=g), K, dim=1)
    return x, top.indices, torch.softmax(top.values, 1)


def test_low_latency_roundtrip_single_rank():
    x, idx, w = _problem()
    E, M = 8, 64
    buf = tm.Buffer(None, device="cpu", low_latency_mode=True)
    stats = torch.zeros(E, dtype=torch.int64)
    recv, counts, handle, ev, hook = buf.low_latency_dispatch(x, idx, M, E, cumulative_local_expert_recv_stats=stats, use_fp8=False,
                                                              return_recv_hook=True)
    hook()
    assert recv.shape == (E, M, 256)
    assert counts.tolist() == torch.bincount(idx.flatten(), minlength=E).tolist() == stats.tolist()
    # every expert's valid rows are exactly the tokens routed to it
    for e in range(E):
        toks = (idx == e).any(1).nonzero().flatten()
        got = recv[e, : counts[e]]
        assert sorted(map(tuple, got.tolist())) == sorted(map(tuple, x[toks].tolist()))
    # experts = identity: combine gives sum_k w[t,k] * x[t] = x[t]
    out, _, _ = buf.low_latency_combine(recv, idx, w, handle)
    assert torch.allclose(out, x, atol=1e-5)
    # zero-copy buffer + preallocated output
    zc = buf.get_next_low_latency_combine_buffer(handle)
    zc.copy_(recv * 2)
    dst = torch.empty_like(x)
    out2, _, _ = buf.low_latency_combine(recv, idx, w, handle, zero_copy=True, out=dst)
    assert out2 is dst and torch.allclose(dst, 2 * x, atol=1e-5)


def test_fp8_and_logfmt_numerics():
    x = torch.randn(16, 512) * 0.3
    q, sc = fp8_quantize(x)
    assert q.dtype == torch.float8_e4m3fn and sc.shape == (16, 4)
    assert (fp8_dequantize(q, sc, torch.float32) - x).abs().max() < 0.05
    q2, packed = fp8_quantize(x, round_scale=True, use_ue8m0=True)
    assert packed.dtype == torch.int32 and packed.shape == (16, 1)
    assert (fp8_dequantize(q2, packed, torch.float32) - x).abs().max() < 0.1
    small = torch.randn(4, 256) * 0.05
    rt = logfmt10_roundtrip(small)
    assert ((rt - small).abs() <= 0.02 * small.abs() + 1e-9).all()
    assert torch.equal(logfmt10_roundtrip(torch.zeros(2, 128)), torch.zeros(2, 128))


def test_rank_mask_api():
    buf = tm.Buffer(None, device="cpu", low_latency_mode=True, enable_shrink=True)
    status = torch.zeros(1, dtype=torch.int32)
    buf.low_latency_update_mask_buffer(0, True)
    buf.low_latency_query_mask_buffer(status)
    assert status.tolist() == [1]
    x, idx, w = _problem(T=8)
    recv, counts, handle, _, _ = buf.low_latency_dispatch(x, idx, 16, 8, use_fp8=False)
    assert counts.sum().item() == 0            # every destination is masked: nothing is sent
    buf.low_latency_clean_mask_buffer()
    buf.low_latency_query_mask_buffer(status)
    assert status.tolist() == [0]
    with pytest.raises(RuntimeError):
        tm.Buffer(None, device="cpu").low_latency_clean_mask_buffer()


def test_unfused_dispatch_fp8_tuple_and_fixed_shape():
    """deepep_dispatch with an (e4m3 rows, scales) payload returns the same bytes in the order of the plain payload;
    num_worst_tokens pads every output to a fixed number of rows."""
    x, idx, w = _problem(T=48, H=512, E=8, K=2, seed=3)
    buf = tm.Buffer(None, device="cpu")
    q, sc = fp8_quantize(x)
    (rq, rs), ridx, rw, counts, handle, _ = buf.deepep_dispatch((q, sc), topk_idx=idx, topk_weights=w, num_experts=8)
    plain, *_ = buf.deepep_dispatch(x, handle=handle)
    assert rq.dtype == q.dtype and rs.dtype == sc.dtype and sum(counts) == idx.numel()
    q2, sc2 = fp8_quantize(plain)
    assert torch.equal(rq.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(rs, sc2)
    (pq, ps), pidx, pw, pcounts, h2, _ = buf.deepep_dispatch((q, sc), topk_idx=idx, topk_weights=w, num_experts=8, num_worst_tokens=96)
    assert pq.shape == (96, 512) and ps.shape == (96, 4) and pidx.shape == (96, 2) and pcounts == []
    assert bool((pidx[rq.shape[0]:] == -1).all()) and torch.equal(pq[: rq.shape[0]].view(torch.uint8), rq.view(torch.uint8))
    comb, _, _ = buf.deepep_combine(fp8_dequantize(pq, ps, torch.float32), h2)
    assert (comb - x).abs().max().item() <= 0.07 * x.abs().max().item()      # one rank: every token comes back once
