"""Host-side pieces that need no GPU: low-latency window geometry, capacity bookkeeping of the launch-ahead forward,
CPU binding helper, Config invariants."""
import os

import pytest
import torch

from teramoe_b200.config import Config
from teramoe_b200.engine import EPEngine, LayerHandle
from teramoe_b200.low_latency import _ll_geometry
from teramoe_b200.parallel.world import EPWorld
from teramoe_b200.utils import numa


@pytest.mark.parametrize("use_fp8,use_ue8m0,use_logfmt", [(False, False, False), (True, False, False), (True, True, True)])
def test_low_latency_geometry_is_aligned_and_disjoint(use_fp8, use_ue8m0, use_logfmt):
    N, E, M, H = 4, 32, 96, 1024
    geom, total, flags = _ll_geometry(N, 1, E, M, H, use_fp8, use_ue8m0, use_ue8m0, use_logfmt)
    off_d_stage, off_d_flags, off_c_stage, off_c_flags, d_msg, c_row = geom[9:15]
    El, G = E // N, H // 128
    assert d_msg % 16 == 0 and c_row % 16 == 0
    assert d_msg >= 16 + ((H + (G if use_ue8m0 else 4 * G)) if use_fp8 else 2 * H)
    assert c_row == (G * 272 if use_logfmt else 2 * H)
    regions = [(off_d_stage, El * N * M * d_msg), (off_d_flags, El * N * 8), (off_c_stage, E * M * c_row), (off_c_flags, E * 8)]
    for (a, n), (b, _) in zip(regions, regions[1:]):
        assert a % 256 == 0 and a + n <= b
    assert regions[-1][0] + regions[-1][1] <= total
    assert flags == ((off_d_flags, El * N * 8), (off_c_flags, E * 8))


def test_capacities_grow_only_and_do_not_depend_on_the_rank_token_count():
    eng = EPEngine(EPWorld.single("cpu"))
    mk = lambda T: LayerHandle(T, 8, 0, 64, 1, 0, 0, 0, 0, (0, 0, 0, 0), *([None] * 9))
    eng._note_caps(mk(100), (1000, 2048, 100))
    first = eng._caps[(8, 64, 1)]
    assert first[0] >= 1000 and first[1] >= 2048 and first[1] % 128 == 0 and first[2] == 100
    eng._note_caps(mk(7), (500, 1024, 300))          # another rank-local T, smaller rows: same key, capacities only grow
    second = eng._caps[(8, 64, 1)]
    assert second[0] == first[0] and second[1] == first[1] and second[2] == 300
    assert eng._caps_key(mk(100)) == eng._caps_key(mk(7))


def test_bind_to_gpu_without_nvml_changes_nothing(monkeypatch):
    before = os.sched_getaffinity(0)
    monkeypatch.setattr(numa, "gpu_cpu_affinity", lambda i: None)
    assert numa.bind_to_gpu(0) is None
    assert os.sched_getaffinity(0) == before
    # with an affinity answer the process is restricted to the intersection with what it may use
    some = sorted(before)[:1]
    monkeypatch.setattr(numa, "gpu_cpu_affinity", lambda i: some + [10 ** 6])
    assert numa.bind_to_gpu(0) == some
    os.sched_setaffinity(0, before)
    monkeypatch.setenv("TERAMOE_NO_BIND", "1")
    assert numa.bind_to_gpu(0) is None


def test_config_invariants_follow_the_reference():
    c = Config(20, 6, 256, 6, 250)
    assert c.num_max_rdma_chunked_recv_tokens == 252          # rounded up to whole send chunks (csrc/config.hpp:70)
    with pytest.raises(ValueError):
        Config(20, 256, 256, 6, 128)                          # nvl send chunk must be smaller than the receive chunk
    with pytest.raises(ValueError):
        Config(20, 6, 256, 100, 100)                          # rdma send chunk must be smaller than (and at most half of) the receive chunk
    with pytest.raises(ValueError):
        Config(-1)


def test_fusion_rule_follows_flops_per_wire_byte():
    """The combine is pushed from the GEMM epilogue only where the GEMM does enough FLOPs per byte it sends."""
    from teramoe_b200 import engine as eng
    if eng._FUSED_MODE != "auto" or eng._FUSED_DISPATCH_MODE != "auto":
        pytest.skip("fusion forced by the environment")
    assert eng.use_fused_combine(512, 1, False)                      # one rank: nothing crosses a link
    assert not eng.use_fused_combine(512, 8, False) and not eng.use_fused_combine(512, 8, True)
    assert eng.use_fused_combine(2048, 8, False) and eng.use_fused_combine(2048, 8, True)
    assert eng.use_fused_combine(1024, 8, True) and not eng.use_fused_combine(1024, 8, False)   # dX does 2I per byte
    assert eng.flops_per_wire_byte(2048, True) == 2 * eng.flops_per_wire_byte(2048, False)
    if eng.USE_CTA_PAIRS and not eng.USE_TMA_GATHER:
        assert eng.use_fused_dispatch(2048, 8, 0) and not eng.use_fused_dispatch(512, 8, 0)
        assert not eng.use_fused_dispatch(2048, 8, eng.FUSED_DISPATCH_MAX_BYTES + 1)


@pytest.mark.parametrize("N,T,E,K", [(1, 200, 8, 4), (4, 333, 32, 8), (8, 257, 64, 6)])
def test_once_per_rank_wire_plan_covers_every_slot_once(N, T, E, K):
    """Index math of the layer kernel's once-per-rank wire format: one home per (token, destination rank), every other
    entry of the token on that rank points at the home's slot, and the rows on the wire are the distinct-rank count."""
    from teramoe_b200 import layout as L
    g = torch.Generator().manual_seed(N * 1000 + T)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)])
    idx[torch.rand(T, K, generator=g) < 0.1] = -1
    metas = torch.stack([L.count_row(idx, E, N) for _ in range(N)])          # every rank routes the same tokens here
    gl = L.global_layout(metas, E, N)
    sl = L.send_layout(idx, E, N, 0, gl)
    home, src = L.wire_rank_plan(idx, sl.send_slot, E, N)
    valid = idx >= 0
    hits = L.token_rank_hits(idx, E, N)
    assert int(home.sum()) == int(hits.sum())                                # one row per (token, rank) on the wire
    assert bool((home <= valid).all()) and bool((src[~valid] == -1).all()) and bool((src[home] == -1).all())
    El = E // N
    slot = sl.send_slot.long()
    for t in range(T):
        for d in range(N):
            ks = [k for k in range(K) if valid[t, k] and int(idx[t, k]) // El == d]
            if not ks:
                continue
            homes = [k for k in ks if home[t, k]]
            assert len(homes) == 1
            h = homes[0]
            assert int(slot[t, h]) == min(int(slot[t, k]) for k in ks)       # the first slot the receiver works on
            for k in ks:
                if k != h:
                    assert int(src[t, k]) == int(slot[t, h]) and int(src[t, k]) < int(slot[t, k])


def test_bench_reference_arm_prints_its_unavailable_line_and_exits_zero():
    """Contract of the benchmark's reference arm where the reference cannot be installed: one JSON line, exit code 0."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300, cwd=root)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [ln for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and "\n" not in rec["unavailable"]


def _layout_invariants(idx_per_rank, E, N):
    """Every routed entry gets its own slot inside its expert's segment, every (token, rank) hit its own receive row, landing
    rows tile [0, land_rows) -- for ALL ranks together, which is what makes the push model race-free."""
    from teramoe_b200 import layout as L
    El = E // N
    metas = torch.stack([L.count_row(idx, E, N) for idx in idx_per_rank])
    gl = L.global_layout(metas, E, N)
    slots_seen = [set() for _ in range(N)]
    rows_seen = [set() for _ in range(N)]
    for r, idx in enumerate(idx_per_rank):
        sl = L.send_layout(idx, E, N, r, gl)
        idx = idx.long()
        valid = (idx >= 0) & (idx < E)
        assert bool((sl.send_slot[~valid] == -1).all())
        for t, k in valid.nonzero().tolist():
            e = int(idx[t, k])
            d, s = e // El, int(sl.send_slot[t, k])
            lo = int(gl.seg_off_all[e])
            assert lo <= s < lo + int(gl.expert_total[e]), "slot outside the expert's rows"
            assert s not in slots_seen[d], "two entries share a slot"
            slots_seen[d].add(s)
        hit = L.token_rank_hits(idx, E, N)
        assert torch.equal(hit, sl.send_row >= 0)
        for t, d in hit.nonzero().tolist():
            row = int(sl.send_row[t, d])
            assert 0 <= row < int(gl.rows[d]) and row not in rows_seen[d]
            rows_seen[d].add(row)
        assert torch.equal(sl.ndst.long(), hit.sum(1))
        if idx.shape[0]:
            assert int(sl.land_off[0]) == 0 and torch.equal(sl.land_off[1:].long(), torch.cumsum(sl.ndst.long(), 0)[:-1])
            assert int(sl.land_off[-1]) + int(sl.ndst[-1]) == int(gl.land_rows[r])
    for d in range(N):
        assert len(slots_seen[d]) == int(gl.expert_total.view(N, El)[d].sum()) and len(rows_seen[d]) == int(gl.rows[d])
        assert int(gl.slots_padded[d]) % 128 == 0 and int(gl.slots_padded[d]) >= len(slots_seen[d])


def test_layout_invariants_on_edge_cases():
    g = torch.Generator().manual_seed(5)
    cases = [
        (1, 4, [torch.zeros(0, 2, dtype=torch.int64)]),                                        # no tokens at all
        (2, 4, [torch.full((7, 3), -1, dtype=torch.int64), torch.zeros(0, 3, dtype=torch.int64)]),   # nothing routed
        (2, 2, [torch.tensor([[0, 1], [1, 0], [1, -1]]), torch.tensor([[1, 1]])]),             # E == N, a token twice on one expert
        (4, 8, [torch.randint(-1, 8, (300, 1), generator=g) for _ in range(4)]),               # K == 1
        (8, 64, [torch.randint(0, 64, (129 + 31 * r, 8), generator=g) for r in range(8)]),     # duplicates inside a token, uneven T
    ]
    for N, E, idx_per_rank in cases:
        _layout_invariants(idx_per_rank, E, N)


def test_layout_invariants_random():
    hypothesis = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=25, deadline=None, derandomize=True, database=None)
    @given(st.sampled_from([1, 2, 4, 8]), st.integers(1, 4), st.integers(1, 6), st.integers(0, 70), st.integers(0, 2 ** 31 - 1))
    def run(N, el, K, T, seed):
        E = N * el
        g = torch.Generator().manual_seed(seed)
        idx_per_rank = [torch.randint(-1, E, (max(0, T - 9 * r), K), generator=g) for r in range(N)]
        _layout_invariants(idx_per_rank, E, N)

    run()
