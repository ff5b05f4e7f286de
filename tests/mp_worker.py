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


class FileComm:
    """Stand-in for an mpi4py communicator (Get_rank / Get_size / bcast / allgather) over a shared directory."""

    def __init__(self, root, rank, size):
        self.root, self.rank, self.size, self.seq = root, rank, size, 0

    def Get_rank(self):
        return self.rank

    def Get_size(self):
        return self.size

    def _put(self, tag, obj):
        import pickle
        tmp = os.path.join(self.root, f".{tag}.{self.rank}.tmp")
        with open(tmp, "wb") as f:
            pickle.dump(obj, f)
        os.replace(tmp, os.path.join(self.root, f"{tag}.{self.rank}"))

    def _get(self, tag, r):
        import pickle
        import time
        path = os.path.join(self.root, f"{tag}.{r}")
        t0 = time.time()
        while not os.path.exists(path):
            if time.time() - t0 > 60:
                raise TimeoutError(path)
            time.sleep(0.01)
        with open(path, "rb") as f:
            return pickle.load(f)

    def allgather(self, obj):
        self.seq += 1
        self._put(f"ag{self.seq}", obj)
        return [self._get(f"ag{self.seq}", r) for r in range(self.size)]

    def bcast(self, obj, root=0):
        self.seq += 1
        if self.rank == root:
            self._put(f"bc{self.seq}", obj)
        return self._get(f"bc{self.seq}", root)


def mpi_comm_case(backend):
    """No process group yet: the buffer builds one from the communicator, then the layer runs as usual."""
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    assert backend == "gloo" and not dist.is_initialized()
    comm = FileComm(os.environ["FILECOMM_DIR"], rank, world)
    buf = tm.Buffer(comm=comm, device="cpu")
    assert dist.is_initialized() and buf.group_size == world and buf.rank == rank
    T, H, I, E, K = 40, 64, 96, 4 * world, 2
    prob = make_problem(world, T, H, I, E, K, seed=9, dtype=torch.float32, x_scale=0.5, w_scale=0.05, uneven_tokens=True)
    ref = oracle(prob)[rank]
    r = prob["ranks"][rank]
    El = E // world
    x = r["x"].clone().requires_grad_(True)
    w = r["w"].clone().requires_grad_(True)
    Wg = prob["W_gateup"][rank * El:(rank + 1) * El].clone().requires_grad_(True)
    Wd = prob["W_down"][rank * El:(rank + 1) * El].clone().requires_grad_(True)
    out = buf.teramoe_autograd(x, r["idx"], w, Wg, Wd, E)
    out.backward(r["go"])
    compare([{"out": out.detach(), "dx": x.grad, "dw": w.grad, "dWg": Wg.grad, "dWd": Wd.grad}], [ref], 1e-4, 1e-4)
    # a second buffer on the now initialised group: the communicator must span it
    buf2 = tm.Buffer(comm=comm, device="cpu")
    assert buf2.group_size == world
    dist.barrier()
    print(f"WORKER_OK {rank}", flush=True)
    dist.destroy_process_group()


def main():
    backend, case = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if case == "mpi_comm":
        return mpi_comm_case(backend)
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
    elif case == "wire_rank":
        # one row per (token, rank) on the wire (TERAMOE_WIRE=rank, set by the test) against one row per entry: same bits
        from teramoe_b200 import engine
        T, H, I, E, K = 384, 1024, 1536, 4 * world, 6
        prob = make_problem(world, T, H, I, E, K, seed=23, dtype=dtype, x_scale=0.5, w_scale=0.05, drop_some=True, uneven_tokens=True)
        ref = oracle(prob)[rank]
        r = prob["ranks"][rank]
        El = E // world
        buf = tm.Buffer(group, int(1e6) // 128 * 128, explicitly_destroy=True)
        res = {}
        for wire in ("entry", "rank", "rank"):
            engine.LAYER_WIRE = wire
            x = r["x"].to(dev).clone().requires_grad_(True)
            w = r["w"].to(dev).clone().requires_grad_(True)
            Wg = prob["W_gateup"][rank * El:(rank + 1) * El].to(dev).clone().requires_grad_(True)
            Wd = prob["W_down"][rank * El:(rank + 1) * El].to(dev).clone().requires_grad_(True)
            out = buf.teramoe_autograd(x, r["idx"].to(dev), w, Wg, Wd, E)
            out.backward(r["go"].to(dev))
            assert buf._engine.last_paths.get("layer_kernel", False), "the default rules must pick the layer kernel for this shape"
            res.setdefault(wire, []).append({"out": out.detach(), "dx": x.grad, "dw": w.grad, "dWg": Wg.grad, "dWd": Wd.grad})
        compare([res["rank"][0]], [ref], tol, tol)
        for n in res["entry"][0]:
            assert torch.equal(res["entry"][0][n], res["rank"][0][n]), f"{n}: wire formats differ"
            assert torch.equal(res["rank"][0][n], res["rank"][1][n]), f"{n}: two runs differ"
        buf.check_status()
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
    elif case == "soak":
        # Buffer reuse under stress: routing re-drawn every step, two layers of different shapes interleaved on ONE buffer
        # (fwd A, fwd B, bwd B, bwd A), a rank without tokens, ranks that exchange nothing, an arena that has to grow
        # mid-run.  Every step the one-kernel path must equal the two-kernel fused path bit for bit (same slots, same tiles,
        # same order of the sums) and the separate kernels within bf16 tolerance (they round once more: a token's rows of
        # one rank are summed there before they travel).
        from teramoe_b200 import engine
        steps = int(os.environ.get("SOAK_STEPS", "200"))
        El = 2
        E = El * world
        shapes = {"A": (256, 512, 256, 4), "B": (192, 1024, 128, 2)}           # T, H, I, K
        gw = torch.Generator().manual_seed(77)
        weights = {}
        for name, (T, H, I, K) in shapes.items():
            Wg_all = (torch.randn(E, 2 * I, H, generator=gw) * 0.02).to(dtype)
            Wd_all = (torch.randn(E, H, I, generator=gw) * 0.02).to(dtype)
            weights[name] = (Wg_all[rank * El:(rank + 1) * El].to(dev), Wd_all[rank * El:(rank + 1) * El].to(dev))
        buf = tm.Buffer(group, int(1e6) // 128 * 128, explicitly_destroy=True)

        def draw(step, name):
            T, H, I, K = shapes[name]
            g = torch.Generator().manual_seed(1000 * step + 10 * rank + (1 if name == "B" else 0))
            Tr = T if step % 7 != 3 else T * 3                                   # every seventh step is larger: the arena grows
            if step % 5 == 2 and rank == world - 1:
                Tr = 0                                                           # a rank without tokens
            x = (torch.randn(Tr, H, generator=g) * 0.1).to(dtype).to(dev)
            logits = torch.randn(Tr, E, generator=g)
            if step % 4 == 1:
                logits[:, : rank * El] = -1e9                                    # only own and higher ranks: some pairs exchange nothing
            top = torch.topk(logits, K, dim=1)
            idx = top.indices.to(torch.int64).to(dev)
            if Tr > 3:
                idx[2, 0] = -1
            return x, idx, torch.softmax(top.values, dim=1).float().to(dev), (torch.randn(Tr, H, generator=g)).to(dtype).to(dev)

        def run_pair(step):
            """fwd A, fwd B, bwd B, bwd A -> all outputs and gradients"""
            res, live = {}, {}
            for name in ("A", "B"):
                x, idx, w, go = draw(step, name)
                Wg, Wd = weights[name]
                leaves = [x.clone().requires_grad_(True), w.clone().requires_grad_(True), Wg.clone().requires_grad_(True),
                          Wd.clone().requires_grad_(True)]
                out = buf.teramoe_autograd(leaves[0], idx, leaves[1], leaves[2], leaves[3], E)
                live[name] = (out, go, leaves)
            for name in ("B", "A"):
                out, go, leaves = live[name]
                out.backward(go)
                res[name] = [out.detach()] + [t.grad for t in leaves]
            return res

        for step in range(steps):
            got = {}
            for path in ("layer", "fused") + (("separate",) if step % 10 == 0 else ()):
                engine._FUSED_DISPATCH_MODE = "0" if path == "separate" else "1"
                engine._FUSED_MODE = "0" if path == "separate" else "1"
                engine._LAYER_KERNEL_MODE = "1" if path == "layer" else "0"
                got[path] = run_pair(step)
            for name in ("A", "B"):
                for i, (a, b) in enumerate(zip(got["layer"][name], got["fused"][name])):
                    assert torch.equal(a, b), f"step {step} layer {name} tensor {i}: one-kernel path differs from the two-kernel fused path"
                if "separate" in got:
                    for i, (a, b) in enumerate(zip(got["layer"][name], got["separate"][name])):
                        if a.numel():
                            err = (a.float() - b.float()).abs().max().item()
                            assert err <= 2e-2 * max(1.0, b.float().abs().max().item()), f"step {step} layer {name} tensor {i}: {err}"
            if step % 50 == 0:
                buf.check_status()
        buf.check_status()
        buf.destroy()
    elif case == "cached_race":
        # a cached-handle dispatch right behind another dispatch: the second call's rows must not land before the first
        # call's result has been copied out, even when one rank's host is slow between the barrier and the copy
        import time
        T, H, E, K = 200, 512, 4 * world, 2
        g = torch.Generator().manual_seed(31 + rank)
        x1 = torch.randn(T, H, generator=g).to(dtype).to(dev)
        x2 = x1 + 100
        logits = torch.randn(T, E, generator=g)
        top = torch.topk(logits, K, dim=1)
        idx, w = top.indices.to(dev), torch.softmax(top.values, 1).to(dev)
        buf = tm.Buffer(group, int(1e6) // 128 * 128, explicitly_destroy=True)
        want, _, _, _, handle, _ = buf.deepep_dispatch(x1, topk_idx=idx, topk_weights=w, num_experts=E)
        eng = buf._engine
        orig = eng.dispatch_gen

        def slow(*a, **k):
            res = yield from orig(*a, **k)
            if rank == 0:
                time.sleep(0.3)                     # the copy of the received rows is enqueued late on this rank
            return res
        eng.dispatch_gen = slow
        for _ in range(3):
            r1, *_ = buf.deepep_dispatch(x1, handle=handle)
            r2, *_ = buf.deepep_dispatch(x2, handle=handle)
            torch.cuda.synchronize() if dev.type == "cuda" else None
            assert torch.equal(r1, want), "rows of the next dispatch landed before the result was copied"
            assert torch.equal(r2, want + 100)
        buf.destroy()
    elif case == "ll":
        # low-latency kernels across ranks: bf16 and fp8 dispatch, weighted combine (plain and LogFMT-10)
        from teramoe_b200.low_latency import fp8_dequantize
        T, H, K, M = 60 + 5 * rank, 1024, 4, 96
        El = 3
        E = El * world
        g = torch.Generator().manual_seed(500 + rank)
        x = (torch.randn(T, H, generator=g) * 0.3).to(dtype).to(dev)
        idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(dev)
        idx[0, 1] = -1
        w = torch.rand(T, K, generator=g).to(dev)
        buf = tm.Buffer(group, int(1e6) // 128 * 128, low_latency_mode=True, explicitly_destroy=True)
        xs = [torch.empty(60 + 5 * r, H, dtype=dtype, device=dev) for r in range(world)]
        ids = [torch.empty(60 + 5 * r, K, dtype=idx.dtype, device=dev) for r in range(world)]
        dist.all_gather(xs, x)
        dist.all_gather(ids, idx)
        for use_fp8 in (False, True):
            stats = torch.zeros(El, dtype=torch.int32, device=dev)
            waits = torch.zeros(world, dtype=torch.int64, device=dev)
            recv, count, handle, _, _ = buf.low_latency_dispatch(x, idx, M, E, cumulative_local_expert_recv_stats=stats,
                                                                 dispatch_wait_recv_cost_stats=waits, use_fp8=use_fp8)
            torch.cuda.synchronize()
            for le in range(El):
                ge = rank * El + le
                want = torch.cat([xs[s][(ids[s] == ge).any(1)] for s in range(world)])
                assert count[le].item() == want.shape[0] == stats[le].item()
                got = fp8_dequantize(recv[0][le, : want.shape[0]], recv[1][le, : want.shape[0]].contiguous(), torch.float32) if use_fp8 \
                    else recv[le, : want.shape[0]].float()
                lim = 0.07 * max(1.0, want.float().abs().max().item()) if use_fp8 else 0.0
                assert (got - want.float()).abs().max().item() <= lim
        recv, count, handle, _, _ = buf.low_latency_dispatch(x, idx, M, E, use_fp8=False)
        y = torch.zeros_like(recv)
        for le in range(El):
            y[le] = (recv[le].float() * 0.25 * ((rank * El + le) % 5 + 1)).to(dtype)
        for use_logfmt in (False, True):
            out, _, _ = buf.low_latency_combine(y, idx, w, handle, use_logfmt=use_logfmt)
            want = torch.zeros(T, H, dtype=torch.float32, device=dev)
            for k in range(K):
                e = idx[:, k]
                rows = (x.float() * 0.25 * ((e.clamp(min=0) % 5).float() + 1)[:, None]).to(dtype).float()
                want += torch.where((e >= 0)[:, None], w[:, k:k + 1] * rows, torch.zeros((), device=dev))
            tol = 3e-2 if use_logfmt else 1e-2
            assert (out.float() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())
        buf.check_status()
        buf.destroy()
    elif case == "fdpass":
        # descriptors between processes: every rank offers an anonymous memory file that names it, twice in a row
        from teramoe_b200.parallel.fdpass import exchange_fds
        for rnd in range(2):
            fd = os.memfd_create(f"rank{rank}")
            os.write(fd, f"rank {rank} round {rnd}".encode())
            fds = exchange_fds(fd, rank, world, group=group)
            assert len(fds) == world and fds[rank] == fd
            for r, f in enumerate(fds):
                assert f >= 0
                os.lseek(f, 0, os.SEEK_SET)
                assert os.read(f, 64).decode() == f"rank {r} round {rnd}", (r, rnd)
            dist.barrier()
            for f in fds:
                os.close(f)
    elif case == "vmm":
        # arenas allocated with virtual memory management and shared as descriptors: the layer must give the same bits
        # as with CUDA IPC arenas (TERAMOE_ARENA=vmm is set by the test; use_fabric=True selects the same allocation)
        T, H, I, E, K = 300, 512, 256, 8 * world, 4
        prob = make_problem(world, T, H, I, E, K, seed=11, dtype=dtype, x_scale=0.5, w_scale=0.05, uneven_tokens=True)
        ref = oracle(prob)[rank]
        r = prob["ranks"][rank]
        El = E // world
        outs = []
        for kind in ("ipc", "vmm", "fabric"):
            buf = tm.Buffer(group, int(1e6) // 128 * 128, explicitly_destroy=True, use_fabric=(kind == "fabric"))
            world_obj = buf._world
            if kind == "vmm":
                # the environment switch, set for this buffer only
                buf.destroy()
                from teramoe_b200.parallel import world as world_mod
                world_mod.ARENA_KIND = "vmm"
                buf = tm.Buffer(group, int(1e6) // 128 * 128, explicitly_destroy=True)
                world_mod.ARENA_KIND = "ipc"
                world_obj = buf._world
            assert world_obj.control.is_vmm() == (kind != "ipc") and world_obj.data.is_vmm() == (kind != "ipc")
            x = r["x"].to(dev).clone().requires_grad_(True)
            w = r["w"].to(dev).clone().requires_grad_(True)
            Wg = prob["W_gateup"][rank * El:(rank + 1) * El].to(dev).clone().requires_grad_(True)
            Wd = prob["W_down"][rank * El:(rank + 1) * El].to(dev).clone().requires_grad_(True)
            out = buf.teramoe_autograd(x, r["idx"].to(dev), w, Wg, Wd, E)
            out.backward(r["go"].to(dev))
            outs.append({"out": out.detach(), "dx": x.grad, "dw": w.grad, "dWg": Wg.grad, "dWd": Wd.grad})
            # a larger call makes the data arena regrow: the new allocation is shared the same way
            big = torch.randn(4096, 1024, dtype=dtype, device=dev)
            bidx = torch.randint(0, E, (4096, K), device=dev)
            rx, *_ = buf.deepep_dispatch(big, topk_idx=bidx, topk_weights=torch.ones(4096, K, device=dev), num_experts=E)
            assert world_obj.data.is_vmm() == (kind != "ipc")
            buf.check_status()
            buf.destroy()
        compare([outs[0]], [ref], tol, tol)
        for other in outs[1:]:
            for n in outs[0]:
                assert torch.equal(outs[0][n], other[n]), f"{n} differs between arena kinds"
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
