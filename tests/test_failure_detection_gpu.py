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
