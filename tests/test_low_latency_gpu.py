"""The low-latency kernels (csrc/lowlat.cu) on one GPU through the public API, against the plain PyTorch restatements of
the same semantics in teramoe_b200/low_latency.py (fp8_quantize, logfmt10_roundtrip) and a direct evaluation."""
import pytest
import torch

import teramoe_b200 as tm
from teramoe_b200.low_latency import fp8_dequantize, fp8_quantize, logfmt10_roundtrip

pytestmark = pytest.mark.gpu


def _problem(T, H, E, K, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(T, H, generator=g) * 0.3).to(torch.bfloat16).cuda()
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).cuda()
    idx[1, 0] = -1
    w = torch.rand(T, K, generator=g).cuda()
    return x, idx, w


def _expected_rows(idx, e):
    """tokens routed to expert e, in token order (the kernel's deterministic slot order)"""
    return (idx == e).any(dim=1).nonzero().flatten()


@pytest.mark.parametrize("use_fp8,round_scale,use_ue8m0", [(False, False, False), (True, False, False), (True, True, False), (True, True, True)])
def test_low_latency_dispatch_ep1(use_fp8, round_scale, use_ue8m0):
    T, H, E, K, M = 100, 1024, 8, 3, 128
    x, idx, w = _problem(T, H, E, K)
    buf = tm.Buffer(None, int(8e6), low_latency_mode=True, explicitly_destroy=True)
    stats = torch.zeros(E, dtype=torch.int32, device="cuda")
    waits = torch.zeros(1, dtype=torch.int64, device="cuda")
    recv, count, handle, _, hook = buf.low_latency_dispatch(x, idx, M, E, cumulative_local_expert_recv_stats=stats,
                                                            dispatch_wait_recv_cost_stats=waits, use_fp8=use_fp8, round_scale=round_scale,
                                                            use_ue8m0=use_ue8m0)
    assert hook is None
    torch.cuda.synchronize()
    for e in range(E):
        toks = _expected_rows(idx, e)
        assert count[e].item() == toks.numel() == stats[e].item()
        assert torch.equal(handle.src_info[e, : toks.numel()].long(), toks)
        assert (handle.layout_range[e, 0].item() >> 32) == toks.numel() and (handle.layout_range[e, 0].item() & 0xFFFFFFFF) == 0
        if use_fp8:
            q, sc = recv
            assert q.dtype == torch.float8_e4m3fn and q.shape == (E, M, H) and sc.shape == (E, M, H // 512 if use_ue8m0 else H // 128)
            want_q, want_s = fp8_quantize(x[toks], round_scale, use_ue8m0)
            got = fp8_dequantize(q[e, : toks.numel()], sc[e, : toks.numel()].contiguous(), torch.float32)
            want = fp8_dequantize(want_q, want_s, torch.float32)
            got_s = sc[e, : toks.numel()].contiguous()
            if use_ue8m0:
                # power-of-two exponents: identical except where amax / 448 sits within an ulp of a power of two
                assert (got_s == want_s).float().mean().item() >= 0.99
            else:
                assert torch.allclose(got_s, want_s, rtol=1e-6, atol=0), "scales differ from the specification"
            # the cast may differ from the restatement in the last e4m3 bit where a quotient sits on a rounding boundary
            assert (got - want).abs().max().item() <= 0.07 * max(1.0, want.abs().max().item())
            assert (got - x[toks].float()).abs().max().item() <= 0.07 * x.float().abs().max().item()
        else:
            assert torch.equal(recv[e, : toks.numel()], x[toks])
    buf.check_status()
    buf.destroy()


@pytest.mark.parametrize("use_logfmt", [False, True])
def test_low_latency_round_trip_weighted_combine_ep1(use_logfmt):
    T, H, E, K, M = 77, 512, 4, 2, 96
    x, idx, w = _problem(T, H, E, K, seed=3)
    buf = tm.Buffer(None, int(8e6), low_latency_mode=True, explicitly_destroy=True)
    recv, count, handle, _, _ = buf.low_latency_dispatch(x, idx, M, E, use_fp8=False)
    # "experts": y = 0.25 * row * (expert id + 1); small values so that the LogFMT groups qualify (log2 amax < 0)
    y = torch.zeros_like(recv)
    for e in range(E):
        y[e] = (recv[e].float() * 0.25 * (e + 1)).to(torch.bfloat16)
    waits = torch.zeros(1, dtype=torch.int64, device="cuda")
    out, _, _ = buf.low_latency_combine(y, idx, w, handle, use_logfmt=use_logfmt, combine_wait_recv_cost_stats=waits)
    torch.cuda.synchronize()
    want = torch.zeros(T, H, dtype=torch.float32, device="cuda")
    for k in range(K):
        e = idx[:, k]
        valid = e >= 0
        rows = (x.float() * 0.25 * (e.clamp(min=0).float() + 1)[:, None]).to(torch.bfloat16)
        if use_logfmt:
            rows = logfmt10_roundtrip(rows)
        want += torch.where(valid[:, None], w[:, k:k + 1] * rows.float(), torch.zeros((), device="cuda"))
    tol = 2e-2 if use_logfmt else 8e-3
    assert (out.float() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())
    if use_logfmt:
        # the wire format must really be the logarithmic one: compared with the plain sum the result differs a little
        plain, _, _ = buf.low_latency_combine(y, idx, w, handle, use_logfmt=False)
        assert not torch.equal(plain, out)
    buf.check_status()
    buf.destroy()


def test_low_latency_hooks_split_send_and_receive():
    T, H, E, K, M = 64, 512, 4, 2, 64
    x, idx, w = _problem(T, H, E, K, seed=5)
    buf = tm.Buffer(None, int(8e6), low_latency_mode=True, explicitly_destroy=True)
    ref, ref_count, ref_handle, _, _ = buf.low_latency_dispatch(x, idx, M, E, use_fp8=False)
    recv, count, handle, _, hook = buf.low_latency_dispatch(x, idx, M, E, use_fp8=False, return_recv_hook=True)
    assert callable(hook)
    hook()                          # the receive phase runs now and fills the tensors handed out above
    torch.cuda.synchronize()
    assert torch.equal(count, ref_count) and torch.equal(handle.src_info[:, :4], ref_handle.src_info[:, :4])
    for e in range(E):
        n = count[e].item()
        assert torch.equal(recv[e, :n], ref[e, :n])
    out, _, hook2 = buf.low_latency_combine(recv, idx, w, handle, return_recv_hook=True)
    hook2()
    want, _, _ = buf.low_latency_combine(ref, idx, w, ref_handle)
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    buf.destroy()


def test_low_latency_mask_kernels_and_masked_rank():
    T, H, E, K, M = 32, 512, 4, 2, 32
    x, idx, w = _problem(T, H, E, K, seed=7)
    buf = tm.Buffer(None, int(8e6), low_latency_mode=True, explicitly_destroy=True, enable_shrink=True)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    buf.low_latency_query_mask_buffer(st)
    assert st.tolist() == [0]
    buf.low_latency_update_mask_buffer(0, True)
    buf.low_latency_query_mask_buffer(st)
    assert st.tolist() == [1]
    # the only rank is masked: nothing is sent or awaited, every expert receives zero rows, and nothing times out
    recv, count, handle, _, _ = buf.low_latency_dispatch(x, idx, M, E, use_fp8=False)
    torch.cuda.synchronize()
    assert count.tolist() == [0] * E
    buf.low_latency_clean_mask_buffer()
    buf.low_latency_query_mask_buffer(st)
    assert st.tolist() == [0]
    buf.clean_low_latency_buffer(M, H, E)
    recv, count, handle, _, _ = buf.low_latency_dispatch(x, idx, M, E, use_fp8=False)
    assert count.sum().item() == int((idx >= 0).sum())
    buf.check_status()
    buf.destroy()


def test_low_latency_wait_runs_out_masks_the_silent_rank():
    """Shrink mode: a receive whose flags nobody sets gives up after the (short) limit, marks the silent rank in the
    mask instead of raising, and reports zero rows; without shrink mode the same wait reports through the status block."""
    from teramoe_b200.low_latency import _ll_geometry
    T, H, E, K, M = 16, 512, 4, 2, 16
    x, idx, w = _problem(T, H, E, K, seed=9)
    for shrink in (True, False):
        buf = tm.Buffer(None, int(8e6), low_latency_mode=True, explicitly_destroy=True, enable_shrink=shrink)
        world, ext = buf._world, buf._world.ext
        geom = buf._ll_prepare(M, H, E, False, False, False, False)
        mask = buf._ll_mask_tensor()
        bufs = (torch.empty(E, M, H, dtype=torch.bfloat16, device="cuda"), None, torch.empty(E, M, dtype=torch.int32, device="cuda"),
                torch.empty(E, 1, dtype=torch.int64, device="cuda"), torch.empty(E, dtype=torch.int32, device="cuda"))
        # receive for a call number that no send carried: every flag wait runs out after 50 ms
        ext.ll_dispatch_recv(geom, world.data.view(0, [16], torch.uint8), bufs[0], None, bufs[2], bufs[3], bufs[4], None, None, 12345,
                             mask if shrink else None, shrink, 50, world.status)
        torch.cuda.synchronize()
        assert bufs[4].tolist() == [0] * E
        if shrink:
            assert mask.tolist() == [1] and world.status.tolist()[0] == 0
        else:
            with pytest.raises(RuntimeError, match="wait ran out"):
                buf.check_status()
        # the context and the buffer stay usable
        if shrink:
            buf.low_latency_clean_mask_buffer()
        recv, count, handle, _, _ = buf.low_latency_dispatch(x, idx, M, E, use_fp8=False)
        assert count.sum().item() == int((idx >= 0).sum())
        buf.destroy()
