"""CPU plumbing: the whole pipeline (layout, push tables, expert math, combine, autograd) in fp32
against the plain reference layer, single rank and emulated multi-rank."""
import pytest
import torch

import teramoe_b200 as tm
from helpers import compare, make_problem, oracle, run_virtual


def test_config1_single_rank_autograd():
    # T=128, H=256, E=8, top-2, I=512, fp32, seed 0
    prob = make_problem(1, 128, 256, 512, 8, 2, seed=0, x_scale=1.0)
    r = prob["ranks"][0]
    buf = tm.Buffer(None, device="cpu")
    x = r["x"].clone().requires_grad_(True)
    w = r["w"].clone().requires_grad_(True)
    Wg = prob["W_gateup"].clone().requires_grad_(True)
    Wd = prob["W_down"].clone().requires_grad_(True)
    out = buf.teramoe_autograd(x, r["idx"], w, Wg, Wd, 8)
    out.backward(r["go"])
    ref = oracle(prob)[0]
    compare([{"out": out.detach(), "dx": x.grad, "dw": w.grad, "dWg": Wg.grad, "dWd": Wd.grad}], [ref], 1e-4, 1e-4)


@pytest.mark.parametrize("N,T,E,K", [(2, 70, 8, 2), (4, 130, 16, 4), (8, 40, 32, 8)])
def test_virtual_cluster_matches_oracle(N, T, E, K):
    prob = make_problem(N, T, 64, 96, E, K, seed=N, drop_some=True, empty_expert=1, uneven_tokens=True)
    compare(run_virtual(prob, "cpu"), oracle(prob), 1e-4, 1e-4)


def test_activation_saving_policy():
    """Only X once per received token and the pre-activation per slot are kept."""
    prob = make_problem(2, 64, 64, 96, 8, 4, seed=3)
    res = run_virtual(prob, "cpu")
    for r in res:
        s = r["saved"]
        assert s.saved_x.shape == (s.handle.rows, 64)
        assert s.preact.shape == (s.handle.slots, 2 * 96)
        assert s.handle.rows <= s.handle.slots


def test_argument_validation():
    buf = tm.Buffer(None, device="cpu")
    x = torch.randn(4, 64)
    idx = torch.zeros(4, 2, dtype=torch.int64)
    w = torch.ones(4, 2)
    Wg, Wd = torch.randn(2, 64, 64), torch.randn(2, 64, 32)
    with pytest.raises(ValueError):
        buf.teramoe_autograd(x, idx, w, Wg, Wd, 2, compute_batch_size=999)
    with pytest.raises(ValueError):
        buf.teramoe_autograd(x, idx, w, Wg, Wd, 2, num_dispatch_sms=3)
    with pytest.raises(ValueError):
        buf.teramoe_autograd(x, idx, w, Wg, Wd, 3)  # weights say 2 local experts
    with pytest.raises(RuntimeError):
        buf.destroy()  # explicitly_destroy not set
    with pytest.raises(ValueError):
        tm.Buffer(None, num_nvl_bytes=100, device="cpu")


def test_fused_path_rules(monkeypatch):
    """The default rules that pick the fused kernels are pure functions of the shape, the rank count and the table size,
    so every rank takes the same decision."""
    from teramoe_b200 import engine
    monkeypatch.setattr(engine, "_FUSED_DISPATCH_MODE", "auto")
    monkeypatch.setattr(engine, "_FUSED_MODE", "auto")
    monkeypatch.setattr(engine, "USE_CTA_PAIRS", True)
    monkeypatch.setattr(engine, "USE_TMA_GATHER", False)
    assert engine.use_fused_dispatch(2048, 8, 1 << 30) and engine.use_fused_dispatch(2048, 1, 1 << 30)
    assert not engine.use_fused_dispatch(512, 8, 1 << 30)                 # the GEMM is shorter than the transfer
    assert not engine.use_fused_dispatch(2048, 8, 12 * (1 << 30))         # operand table too large for the arena
    assert engine.use_fused_combine(2048, 8, False) and engine.use_fused_combine(1024, 8, True)
    assert not engine.use_fused_combine(1024, 8, False) and engine.use_fused_combine(256, 1, False)
    monkeypatch.setattr(engine, "_FUSED_DISPATCH_MODE", "0")
    assert not engine.use_fused_dispatch(2048, 8, 0)
    # num_dispatch_sms -> CTA pairs that dispatch first (two SMs per pair) unless the environment fixes them
    monkeypatch.setattr(engine, "_pairs_env", None)
    assert engine.dispatch_pairs(0, 32) == 16 and engine.dispatch_pairs(1, 2) == 2 and engine.dispatch_pairs(0, 400) == 48
    assert engine.dispatch_pairs(0, 0) == engine.FUSED_DISPATCH_CLUSTERS[0]
