"""The whole-layer kernel (csrc/layer.cu): its scheduler's work list, and forward + backward through the public API
against the fp32 oracle and, bit for bit, against the separate kernels (same slots, same tiles, same reduction order)."""
import pytest
import torch

import teramoe_b200 as tm
from teramoe_b200.utils.numerics import assert_close_bf16
from helpers import make_problem, oracle

pytestmark = pytest.mark.gpu


def _set_path(monkeypatch, path):
    """path: "separate" (push / expand / GEMM / reduce kernels), "fused" (dispatch + GEMM kernel, push epilogue),
    "layer" (one kernel per direction)."""
    from teramoe_b200 import engine
    monkeypatch.setattr(engine, "_FUSED_DISPATCH_MODE", "0" if path == "separate" else "1")
    monkeypatch.setattr(engine, "_FUSED_MODE", "0" if path == "separate" else "1")
    monkeypatch.setattr(engine, "_LAYER_KERNEL_MODE", "1" if path == "layer" else "0")


def _run(buf, prob, E, **kw):
    r = prob["ranks"][0]
    x = r["x"].clone().requires_grad_(True)
    w = r["w"].clone().requires_grad_(True)
    Wg = prob["W_gateup"].clone().requires_grad_(True)
    Wd = prob["W_down"].clone().requires_grad_(True)
    out = buf.teramoe_autograd(x, r["idx"], w, Wg, Wd, E, **kw)
    out.backward(r["go"])
    torch.cuda.synchronize()
    return {"out": out.detach(), "dx": x.grad, "dw": w.grad, "dWg": Wg.grad, "dWd": Wd.grad}


@pytest.mark.parametrize("bwd", [False, True])
@pytest.mark.parametrize("U,group,lag,min_lag", [(1, 8, 70, 0), (7, 4, 0, 0), (8, 8, 100, 0), (19, 8, 70, 148), (33, 16, 40, 148), (5, 1, 50, 7),
                                                 (40, 2, 70, 148)])
def test_schedule_covers_every_tile_once_and_respects_dependencies(bwd, U, group, lag, min_lag):
    from teramoe_b200._build import load_ext
    ext = load_ext()
    H, I, T, El, chunk = 1024, 768, 300, 3, 64
    dev = "cuda"
    g = torch.Generator().manual_seed(U)
    order = torch.randperm(U, generator=g).to(torch.int32).to(dev)
    # U units over El experts: expert e owns a contiguous run of units (two blocks each, the last maybe one)
    per = [U // El + (1 if e < U % El else 0) for e in range(El)]
    max_work = ext.moe_layer_max_work(bwd, U, H, I, El, T, chunk)
    work = torch.full((max_work * 4,), -7, dtype=torch.int32, device=dev)
    num_work = torch.zeros(1, dtype=torch.int32, device=dev)
    eu = torch.zeros(2 * El, dtype=torch.int32, device=dev)
    # every unit has two blocks except the last unit of the last expert; 100 valid rows are missing in every expert's last block
    nblk = 2 * U - 1
    unit_blk = torch.tensor([min(2 * u, nblk) for u in range(U + 1)], dtype=torch.int32, device=dev)
    seg = torch.tensor([0] + [min(256 * sum(per[: e + 1]), 128 * nblk) for e in range(El)], dtype=torch.int32, device=dev)
    me = torch.tensor([e for e in range(El) for _ in range((int(seg[e + 1]) - int(seg[e])) // 128)], dtype=torch.int32, device=dev)
    totals = torch.tensor([max(int(seg[e + 1]) - int(seg[e]) - 100, 0) for e in range(El)], dtype=torch.int32, device=dev)
    ext.moe_layer_schedule(bwd, H, I, T, order, torch.tensor([U], dtype=torch.int32, device=dev), seg, unit_blk, me, totals, group, lag, min_lag,
                           chunk, work, num_work, eu)
    n = int(num_work.item())
    raw = work.view(-1, 4)[:n].cpu().tolist()
    # decode (csrc/layer.h): kind = x & 15; GEMM items (unit, column block); weight gradients (expert, row unit, column block)
    items = []
    for x, y, z, w_ in raw:
        k = x & 15
        if k <= 1:
            blk0, two = w_, (x >> 4) & 1
            assert blk0 == int(unit_blk[y]) and two == int(int(unit_blk[y + 1]) - blk0 == 2) and (x >> 8) == int(me[blk0])
            e = int(me[blk0])
            valid_end = int(seg[e]) + int(totals[e])
            assert (z >> 16) & 0xff == max(0, min(128, valid_end - 128 * blk0))
            assert (z >> 24) & 0xff == (max(0, min(128, valid_end - 128 * (blk0 + 1))) if two else 0)
            items.append((k, y, z & 0xffff, 0))
        elif k <= 3:
            e = x >> 8
            assert y == int(seg[e]) and w_ == (int(seg[e + 1]) - int(seg[e])) // 64
            items.append((k, e, (z >> 16) & 0xffff, z & 0xffff))
        else:
            raise AssertionError(f"unknown item kind {k}")
    nb1 = (I + 255) // 256 if bwd else (2 * I + 255) // 256
    nb2 = (H + 255) // 256
    want = {(0, u, nb) for u in range(U) for nb in range(nb1)} | {(1, u, nb) for u in range(U) for nb in range(nb2)}
    got = [(k, a, b) for k, a, b, _ in items if k <= 1]
    assert len(got) == len(set(got)) and set(got) == want
    # a unit's second GEMM comes after ALL items of its first GEMM (a worker waits only for items claimed before its own)
    last_g1 = {}
    for pos, (k, a, b, c) in enumerate(items):
        if k == 0:
            last_g1[a] = pos
    first_g2 = {}
    for pos, (k, a, b, c) in enumerate(items):
        if k == 1:
            assert pos > last_g1[a]
            first_g2.setdefault(a, pos)
    # ... and, while first-GEMM items remain to fill the gap, at least min_lag of them lie in between
    n_g1 = U * nb1
    for u, pos in first_g2.items():
        between = sum(1 for p in range(last_g1[u] + 1, pos) if items[p][0] == 0)
        after = sum(1 for p in range(last_g1[u] + 1, n) if items[p][0] == 0)
        assert between >= min(min_lag, after) - group * nb1, (u, between, after)
    # units are visited in the given order, batch by batch
    first_seen = []
    for k, a, b, c in items:
        if k == 0 and a not in first_seen:
            first_seen.append(a)
    pos_of = {int(u): i for i, u in enumerate(order.cpu().tolist())}
    assert [pos_of[u] // group for u in first_seen] == sorted(pos_of[u] // group for u in first_seen)
    if bwd:
        mu_wd, mu_wg = (H + 255) // 256, (2 * I + 255) // 256
        wd = [(a, b, c) for k, a, b, c in items if k == 2]
        wg = [(a, b, c) for k, a, b, c in items if k == 3]
        assert set(wd) == {(e, m, nb) for e in range(El) for m in range(mu_wd) for nb in range((I + 255) // 256)} and len(wd) == len(set(wd))
        assert set(wg) == {(e, m, nb) for e in range(El) for m in range(mu_wg) for nb in range(nb2)} and len(wg) == len(set(wg))
        assert max(p for p, it in enumerate(items) if it[0] <= 1) < min(p for p, it in enumerate(items) if it[0] in (2, 3))
    assert all(it[0] <= 3 for it in items)      # the reduce of the landed rows is a role of its own, not an item
    first = 0
    for e in range(El):
        assert eu.view(-1, 2)[e].tolist() == [first, per[e]]
        first += per[e]


@pytest.mark.parametrize("T,H,I,E,K,kw", [
    (512, 1024, 1024, 16, 8, {}),
    (300, 512, 256, 8, 4, {"compute_batch_size": 1024, "combine_start_head_percent": 0}),
    (1000, 768, 640, 4, 2, {"compute_batch_size": 4096, "combine_start_head_percent": 100, "num_dispatch_sms": 8}),
    (77, 256, 128, 8, 3, {"total_sms": 64, "num_dispatch_sms": 4, "num_combine_sms": 4}),
])
def test_layer_kernel_ep1_matches_oracle_and_separate_kernels(T, H, I, E, K, kw, monkeypatch):
    prob = make_problem(1, T, H, I, E, K, seed=T, dtype=torch.bfloat16, device="cuda", x_scale=0.1, w_scale=0.02, drop_some=True,
                        empty_expert=1)
    buf = tm.Buffer(None, int(64e6), explicitly_destroy=True)
    res = {}
    for path in ("separate", "layer", "fused"):
        _set_path(monkeypatch, path)
        res[path] = [_run(buf, prob, E, **kw) for _ in range(2)]
        assert buf._engine.last_paths.get("layer_kernel", False) == (path == "layer")
    ref = oracle(prob)[0]
    for name in ("out", "dx", "dw", "dWg", "dWd"):
        assert_close_bf16(res["layer"][0][name].float(), ref[name].cuda().float(), name)
        assert torch.equal(res["layer"][0][name], res["layer"][1][name]), f"{name}: two runs differ"
        assert torch.equal(res["layer"][0][name], res["separate"][0][name]), f"{name}: layer kernel differs from the separate kernels"
        assert torch.equal(res["fused"][0][name], res["separate"][0][name]), f"{name}: fused kernels differ from the separate kernels"
    buf.check_status()
    buf.destroy()


@pytest.mark.parametrize("T,H,I,E,K,kw", [
    (700, 512, 1536, 8, 4, {}),
    (1500, 1024, 512, 16, 8, {"stage": 2, "num_dispatch_sms": 8}),
    (77, 256, 128, 8, 3, {"total_sms": 64, "num_dispatch_sms": 4}),
])
def test_layer_kernel_one_row_per_rank_on_the_wire_is_bitwise_equal(T, H, I, E, K, kw, monkeypatch):
    """TERAMOE_WIRE=rank: a token's row travels once per destination rank and the receiver copies it into the token's other
    slots there.  On one rank all K entries of a token share one row, so every block mixes arrived and copied rows."""
    from teramoe_b200 import engine
    _set_path(monkeypatch, "layer")
    prob = make_problem(1, T, H, I, E, K, seed=T + 1, dtype=torch.bfloat16, device="cuda", x_scale=0.1, w_scale=0.02, drop_some=True,
                        empty_expert=1)
    buf = tm.Buffer(None, int(64e6), explicitly_destroy=True)
    res = {}
    for wire in ("entry", "rank", "entry", "rank"):
        monkeypatch.setattr(engine, "LAYER_WIRE", wire)
        res.setdefault(wire, []).append(_run(buf, prob, E, **kw))
        assert buf._engine.last_paths.get("layer_kernel", False)
    ref = oracle(prob)[0]
    for name in ("out", "dx", "dw", "dWg", "dWd"):
        assert_close_bf16(res["rank"][0][name].float(), ref[name].cuda().float(), name)
        assert torch.equal(res["rank"][0][name], res["entry"][0][name]), f"{name}: wire formats differ"
        assert torch.equal(res["rank"][1][name], res["entry"][1][name]), f"{name}: wire formats differ on the second call"
    buf.check_status()
    buf.destroy()


def test_layer_kernel_zero_tokens_and_changing_routing(monkeypatch):
    """A call without tokens, then calls whose routing changes every step, on one buffer."""
    _set_path(monkeypatch, "layer")
    H, I, E, K = 512, 256, 8, 2
    buf = tm.Buffer(None, int(64e6), explicitly_destroy=True)
    prob = make_problem(1, 64, H, I, E, K, seed=1, dtype=torch.bfloat16, device="cuda", x_scale=0.1, w_scale=0.02)
    Wg, Wd = prob["W_gateup"], prob["W_down"]
    x0 = torch.zeros(0, H, dtype=torch.bfloat16, device="cuda", requires_grad=True)
    out0 = buf.teramoe_autograd(x0, torch.zeros(0, K, dtype=torch.int64, device="cuda"), torch.zeros(0, K, device="cuda"),
                                Wg.clone().requires_grad_(True), Wd.clone().requires_grad_(True), E)
    out0.backward(torch.zeros_like(out0))
    assert out0.shape == (0, H)
    for step in range(6):
        p = make_problem(1, 64 + 50 * step, H, I, E, K, seed=100 + step, dtype=torch.bfloat16, device="cuda", x_scale=0.1, w_scale=0.02,
                         drop_some=True)
        p["W_gateup"], p["W_down"] = Wg, Wd
        got = _run(buf, p, E)
        ref = oracle(p)[0]
        for name in ("out", "dx", "dw", "dWg", "dWd"):
            assert_close_bf16(got[name].float(), ref[name].cuda().float(), f"step {step} {name}")
    buf.check_status()
    buf.destroy()


def test_autotune_sweeps_the_schedule_knobs(monkeypatch):
    """autotune_teramoe walks compute_batch_size x combine_start_head_percent (plus, on request, num_dispatch_sms and stage),
    which shape the work list of the layer kernel; it returns the reference's structure."""
    _set_path(monkeypatch, "layer")
    prob = make_problem(1, 512, 512, 256, 8, 4, seed=3, dtype=torch.bfloat16, device="cuda", x_scale=0.1, w_scale=0.02)
    r = prob["ranks"][0]
    buf = tm.Buffer(None, int(64e6), explicitly_destroy=True)
    best, results = tm.autotune_teramoe(buf, r["x"], r["idx"], r["w"], prob["W_gateup"], prob["W_down"], 8, num_iters=2, warmup_iters=1,
                                        verbose=False, mode="fwd_bwd", compute_batch_sizes=[1024, 4096], combine_start_head_percents=[0, 100],
                                        dispatch_sms_list=[8, 24], stages=[1, 2])
    assert len(results) == 16 and best.time_ms == min(ms for _, _, ms in results)
    assert best.compute_batch_size in (1024, 4096) and best.combine_start_head_percent in (0, 100)
    assert best.extra["num_dispatch_sms"] in (8, 24) and best.extra["stage"] in (1, 2)
    buf.check_status()
    buf.destroy()
