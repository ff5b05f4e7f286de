"""Failure detection on the device without faulting it: a wait whose flag nobody sets runs out its
(short) limit, the kernel writes the status block and returns, the host raises, the context lives on."""
import pytest
import torch

from teramoe_b200.parallel.world import VirtualCluster

pytestmark = pytest.mark.gpu


def test_barrier_wait_runs_out_and_reports():
    cluster = VirtualCluster(2, "cuda")
    try:
        w0 = cluster.worlds[0]
        # only rank 0 enters the barrier: rank 1's flag is never written
        w0.device_barrier(site=700, limit_ms=50)
        torch.cuda.synchronize()
        st = w0.status.tolist()
        assert st[0] == 2 and st[1] == 701, st          # flag timeout, site 700 + missing peer 1
        with pytest.raises(RuntimeError, match="wait ran out"):
            w0.check_status()
        assert w0.status.tolist()[0] == 0                # cleared after reporting
        # the context is still usable
        a = torch.ones(1024, device="cuda")
        assert float((a * 2).sum()) == 2048.0
        # a complete barrier (both ranks signal) passes
        ep = max(w.epoch for w in cluster.worlds) + 1
        for w in cluster.worlds:
            w.epoch = ep - 1
        # rank 1 signals first (its own wait for rank 0 runs out quickly), then rank 0 finds both flags
        cluster.worlds[1].device_barrier(site=800, limit_ms=20)
        cluster.worlds[0].device_barrier(site=900, limit_ms=200)
        torch.cuda.synchronize()
        assert cluster.worlds[0].status.tolist()[0] == 0
        cluster.worlds[1].status.zero_()
    finally:
        cluster.close()


def test_fused_dispatch_gemm_wait_runs_out_and_reports():
    """The compute pairs of the one-kernel dispatch + GEMM wait for arrival counters.  With a sending list of length
    zero no counter ever fills: every wait runs out its limit, the kernel frees its tensor memory and returns, the status
    block names the wait, and the same buffer runs a normal layer afterwards."""
    import teramoe_b200 as tm
    from teramoe_b200 import engine

    torch.manual_seed(3)
    T, H, I, E, K = 256, 256, 256, 4, 2
    x = (torch.randn(T, H, device="cuda") * 0.1).to(torch.bfloat16)
    Wg = (torch.randn(E, 2 * I, H, device="cuda") * 0.02).to(torch.bfloat16)
    Wd = (torch.randn(E, H, I, device="cuda") * 0.02).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(T)])
    w = torch.rand(T, K, device="cuda")
    buf = tm.Buffer(None, int(64e6), explicitly_destroy=True)
    try:
        eng, world = buf._engine, buf._world
        h = buf._drive(eng.layout_gen(idx, E))
        h.topk_weights = w
        h.num_send = torch.zeros_like(h.num_send)          # the dispatch role sends nothing
        world.set_wait_limit_ms(200)                       # waits on "other ranks" give up after 0.2 s instead of 30 s
        buf._drive(eng.fused_dispatch_gemm_gen(h, x, w, Wg, 0))
        torch.cuda.synchronize()
        st = world.status.tolist()
        assert st[0] in (1, 2) and 600 <= st[1] < 660, st  # a flag or mbarrier wait of the fused kernel
        with pytest.raises(RuntimeError, match="wait ran out"):
            world.check_status()
        assert world.status.tolist()[0] == 0
        # with strict status checks the call whose wait ran out is the call that raises
        world.strict_status = True
        h2 = buf._drive(eng.layout_gen(idx, E))
        h2.topk_weights = w
        h2.num_send = torch.zeros_like(h2.num_send)
        with pytest.raises(RuntimeError, match="wait ran out"):
            buf._drive(eng.fused_dispatch_gemm_gen(h2, x, w, Wg, 0))
        world.strict_status = False
        assert world.status.tolist()[0] == 0
        # without them the next call on the buffer raises (the snapshot taken at the end of the failed call)
        h3 = buf._drive(eng.layout_gen(idx, E))
        h3.topk_weights = w
        h3.num_send = torch.zeros_like(h3.num_send)
        buf._drive(eng.fused_dispatch_gemm_gen(h3, x, w, Wg, 0))
        with pytest.raises(RuntimeError, match="wait ran out"):
            buf._drive(eng.layout_gen(idx, E))
        world.set_wait_limit_ms(0)
        assert world.status.tolist()[0] == 0
        # the context and the buffer are still usable
        saved_mode = engine._FUSED_DISPATCH_MODE
        try:
            engine._FUSED_DISPATCH_MODE = "1"
            out = buf.teramoe_forward(x, idx, w, Wg, Wd, E)
        finally:
            engine._FUSED_DISPATCH_MODE = saved_mode
        ref = tm.moe_reference(x.float(), idx, w, Wg.float(), Wd.float())
        torch.cuda.synchronize()
        assert world.status.tolist()[0] == 0
        assert (out.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    finally:
        buf.destroy()
