"""Child process of the multi-process tests: one rank of a gloo (CPU) or nccl (GPU) group.

usage: python mp_worker.py <backend> <case>     (RANK / WORLD_SIZE / MASTER_* come from the environment)
Prints "WORKER_OK <rank>" on success.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import torch
import torch.distributed as dist

import teramoe_b200 as tm
from helpers import compare, make_problem, oracle


def main():
    backend, case = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group("nccl", device_id=dev)
        dtype, tol = torch.bfloat16, 2e-2
    else:
        dev = torch.device("cpu")
        import datetime
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=15))
        dtype, tol = torch.float32, 1e-4
    group = dist.group.WORLD

    if case == "layer":
        T, H, I, E, K = (300, 512, 256, 8 * world, 4) if backend == "nccl" else (60, 64, 96, 4 * world, 2)
        prob = make_problem(world, T, H, I, E, K, seed=5, dtype=dtype, x_scale=0.5, w_scale=0.05, drop_some=True, empty_expert=1,
                            uneven_tokens=True)
        ref = oracle(prob)[rank]
        r = prob["ranks"][rank]
        El = E // world
        buf = tm.Buffer(group, int(1e6) // 128 * 128, explicitly_destroy=True)
        outs = []
        for it in range(3):
            x = r["x"].to(dev).clone().requires_grad_(True)
            w = r["w"].to(dev).clone().requires_grad_(True)
            Wg = prob["W_gateup"][rank * El:(rank + 1) * El].to(dev).clone().requires_grad_(True)
            Wd = prob["W_down"][rank * El:(rank + 1) * El].to(dev).clone().requires_grad_(True)
            out = buf.teramoe_autograd(x, r["idx"].to(dev), w, Wg, Wd, E)
            out.backward(r["go"].to(dev))
            outs.append({"out": out.detach(), "dx": x.grad, "dw": w.grad, "dWg": Wg.grad, "dWd": Wd.grad})
        compare([outs[0]], [ref], tol, tol)
        for n in outs[0]:
            assert torch.equal(outs[0][n], outs[2][n]), f"{n} differs between runs"
        # un-fused API round trip
        idx = r["idx"].to(dev)
        per_rank, _, per_expert, in_rank, _ = buf.get_dispatch_layout(idx, E)
        recv_x, recv_idx, recv_w, counts, handle, _ = buf.deepep_dispatch(r["x"].to(dev), topk_idx=idx, topk_weights=r["w"].to(dev),
                                                                            num_tokens_per_expert=per_expert)
        comb, comb_w, _ = buf.deepep_combine(recv_x, handle, topk_weights=recv_w)
        ndst = in_rank.sum(1).to(comb.dtype)
        expect = (r["x"].to(dev).float() * ndst[:, None].float())
        if expect.numel():
            assert (comb.float() - expect).abs().max().item() <= tol * 4 * max(1.0, expect.abs().max().item())
        valid = idx >= 0
        assert torch.allclose(comb_w[valid], r["w"].to(dev)[valid], atol=1e-6)
        # fixed-shape mode: padded outputs, the same combine result
        worst = 2048   # at least the sum of all ranks' token counts in this problem
        wx, widx, ww, wcounts, whandle, _ = buf.deepep_dispatch(r["x"].to(dev), topk_idx=idx, topk_weights=r["w"].to(dev), num_experts=E,
                                                                num_worst_tokens=worst)
        assert wx.shape[0] == worst and widx.shape[0] == worst and wcounts == []
        assert torch.equal(wx[: recv_x.shape[0]], recv_x) and bool((widx[recv_x.shape[0]:] == -1).all())
        comb2, _, _ = buf.deepep_combine(wx, whandle)
        assert torch.equal(comb2, comb)
        # FP8 payload: (e4m3 rows, per-128-channel scales) travel as raw bytes and arrive in the order of recv_x
        from teramoe_b200.low_latency import fp8_dequantize, fp8_quantize
        x8 = torch.randn(idx.shape[0], 256, generator=torch.Generator().manual_seed(100 + rank)).to(dev).to(r["x"].dtype)
        q, sc = fp8_quantize(x8)
        (rq, rsc), _, _, _, h8, _ = buf.deepep_dispatch((q, sc), topk_idx=idx, topk_weights=r["w"].to(dev), num_experts=E)
        want, *_ = buf.deepep_dispatch(x8, handle=h8)
        assert rq.dtype == q.dtype and rq.shape == want.shape and rsc.shape == (want.shape[0], sc.shape[1])
        if want.numel():
            err = (fp8_dequantize(rq, rsc, torch.float32) - want.float()).abs().max().item()
            assert err <= 0.07 * max(1.0, want.float().abs().max().item()), err
        buf.destroy()
    elif case == "layer_auto":
        # a shape large enough for the default rules to pick the fused kernels (I >= 1536): no environment switches
        from teramoe_b200 import engine
        T, H, I, E, K = 384, 1024, 1536, 2 * world, 2
        prob = make_problem(world, T, H, I, E, K, seed=9, dtype=dtype, x_scale=0.1, w_scale=0.02, drop_some=True, uneven_tokens=True)
        ref = oracle(prob)[rank]
        r = prob["ranks"][rank]
        El = E // world
        buf = tm.Buffer(group, int(1e6) // 128 * 128, explicitly_destroy=True)
        outs = []
        for it in range(2):
            x = r["x"].to(dev).clone().requires_grad_(True)
            w = r["w"].to(dev).clone().requires_grad_(True)
            Wg = prob["W_gateup"][rank * El:(rank + 1) * El].to(dev).clone().requires_grad_(True)
            Wd = prob["W_down"][rank * El:(rank + 1) * El].to(dev).clone().requires_grad_(True)
            out = buf.teramoe_autograd(x, r["idx"].to(dev), w, Wg, Wd, E)
            out.backward(r["go"].to(dev))
            outs.append({"out": out.detach(), "dx": x.grad, "dw": w.grad, "dWg": Wg.grad, "dWd": Wd.grad})
        if dev.type == "cuda":
            assert buf._engine.last_paths["fused_dispatch_gemm"] and buf._engine.last_paths["fused_combine_fwd"], buf._engine.last_paths
        compare([outs[0]], [ref], tol, tol)
        for n in outs[0]:
            assert torch.equal(outs[0][n], outs[1][n]), f"{n} differs between runs"
        buf.destroy()
    elif case == "mismatch":
        # ranks disagree on num_experts: the host-side check must raise on every rank, nothing hangs
        buf = tm.Buffer(group, device=dev)
        try:
            x = torch.randn(8, 64, dtype=dtype, device=dev)
            idx = torch.zeros(8, 2, dtype=torch.int64, device=dev)
            w = torch.ones(8, 2, device=dev)
            Wg, Wd = torch.randn(2, 64, 64, dtype=dtype, device=dev), torch.randn(2, 64, 32, dtype=dtype, device=dev)
            buf.teramoe_autograd(x, idx, w, Wg, Wd, 2 * world + 1)
        except ValueError:
            print(f"WORKER_OK {rank}", flush=True)
            dist.destroy_process_group()
            return
        raise SystemExit("expected ValueError")
    elif case == "absent":
        # the last rank leaves before the first collective: the others must get an exception, not hang
        if rank == world - 1:
            print(f"WORKER_OK {rank}", flush=True)
            os._exit(0)
        buf = tm.Buffer(group, device=dev)
        x = torch.randn(8, 64, dtype=dtype, device=dev)
        idx = torch.zeros(8, 2, dtype=torch.int64, device=dev)
        idx[:, 1] = 1
        w = torch.ones(8, 2, device=dev)
        Wg, Wd = torch.randn(1, 64, 64, dtype=dtype, device=dev), torch.randn(1, 64, 32, dtype=dtype, device=dev)
        try:
            buf.teramoe_autograd(x, idx, w, Wg, Wd, world)
        except Exception as e:  # gloo reports the lost peer (connection closed / timeout)
            print(f"WORKER_OK {rank} ({type(e).__name__})", flush=True)
            os._exit(0)
        raise SystemExit("expected an exception because a rank is absent")
    else:
        raise SystemExit(f"unknown case {case}")
    dist.barrier()
    print(f"WORKER_OK {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
