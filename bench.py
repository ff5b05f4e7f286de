"""Headline benchmark: bf16 MoE layer forward + backward latency, expert-parallel over N GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 20 --warmup 5

Metric and configuration follow the reference's own benchmark (tests/test_teramoe_performance.py:127-164,
docs/latency.md): one MoE layer (dispatch -> grouped gate_up GEMM -> SwiGLU -> down GEMM -> combine) forward
plus backward, per-iteration CUDA events, here reported as the MAXIMUM over ranks.  Default config: the
DeepSeek-V3-like layer (H=7168, I=2048, 32 experts per rank, top-8, 8192 tokens per rank); per-GPU
work is fixed as N grows (weak scaling; 256 experts at N=8).  Synthetic data, random-init weights.

Prints ONE JSON line on rank 0.  `value` is the device-timed latency; `e2e` is the same step through the
public API with every step's inputs copied from pinned host memory and the loss read back.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: (H, I, experts per rank, top-k, tokens per rank, peak-to-mean)
    "dsv3": (7168, 2048, 32, 8, 8192, 1.0),
    "sparse": (7168, 512, 32, 8, 16384, 1.0),
    "imbalanced": (7168, 2048, 32, 8, 32768, 3.0),
    "mixtral": (4096, 14336, 1, 2, 8192, 1.0),
    "ref_published": (2048, 3072, 16, 6, 8192, 1.0),
    "tiny": (512, 256, 4, 2, 512, 1.0),
}
# closest published reference number per config (ms, fwd+bwd): docs/latency.md:14, EP16, T=8192, P2M 1.0
PUBLISHED_MS = {"ref_published": 11.639}
METRIC = "MoE layer fwd+bwd latency ms (max over ranks)"


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="teramoe", choices=["teramoe", "reference", "nccl"])
    p.add_argument("--config", default="dsv3", choices=sorted(CONFIGS))
    p.add_argument("--tokens", type=int, default=0, help="override tokens per rank")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--baseline-loop", action="store_true", help="--impl nccl: per-expert GEMM loop instead of the library grouped GEMM")
    p.add_argument("--trace", action="store_true", help="print per-phase device times (rank 0, stderr) after the timed region")
    return p.parse_args()


def reference_unavailable():
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference does not build offline (nvshmem needs infiniband/mlx5dv.h; third-party/{cutlass,DeepGEMM,quack} "
                       "submodules are empty) and its fused path only runs on 16/32/64 ranks with IBGDA NICs",
    }))


def main():
    args = parse()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            reference_unavailable()
        return 0

    import torch
    import torch.distributed as dist

    import teramoe_b200 as tm
    from teramoe_b200 import layout as L
    from teramoe_b200._build import load_ext
    from teramoe_b200.utils.timing import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs a torchrun launch with {args.gpus} ranks")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    ext = load_ext()

    H, I, El, K, T, p2m = CONFIGS[args.config]
    if args.tokens:
        T = args.tokens
    N = world
    E = El * N
    if K > E:
        raise SystemExit(f"config {args.config}: top-{K} routing needs at least {K} experts, {N} rank(s) x {El} give {E}; use more GPUs")
    gen = torch.Generator().manual_seed(1234 + rank)
    x_host = (torch.randn(T, H, generator=gen)).to(torch.bfloat16).pin_memory()
    go_host = (torch.randn(T, H, generator=gen)).to(torch.bfloat16).pin_memory()
    if p2m > 1.0:
        idx_host = L.imbalanced_topk(T, K, E, p2m, torch.Generator().manual_seed(99)).to(torch.int64)
        logits = torch.randn(T, K, generator=gen)
    else:
        full = torch.randn(T, E, generator=gen)
        top = torch.topk(full, K, dim=1)
        idx_host, logits = top.indices.to(torch.int64), top.values
    w_host = torch.softmax(logits, dim=1).float().pin_memory()
    idx_host = idx_host.pin_memory()
    wgen = torch.Generator(device=dev).manual_seed(4321 + rank)
    Wg = (torch.randn(El, 2 * I, H, device=dev, generator=wgen) * 0.02).to(torch.bfloat16).requires_grad_(True)
    Wd = (torch.randn(El, H, I, device=dev, generator=wgen) * 0.02).to(torch.bfloat16).requires_grad_(True)

    if args.impl == "nccl":
        from teramoe_b200.parallel.nccl_baseline import NcclMoEBaseline
        # library grouped GEMMs (torch.nn.functional.grouped_mm) unless --baseline-loop asks for one cuBLAS GEMM per expert
        layer = NcclMoEBaseline(group, E, grouped=not args.baseline_loop)
        # the baseline keeps its gate/up weights in the layout a library SwiGLU prefers (gate rows, then up rows)
        Wg = NcclMoEBaseline.to_chunked(Wg.detach()).requires_grad_(True)
        run_layer = lambda x, idx, w: layer(x, idx, w, Wg, Wd, chunked=True)
    else:
        buf = tm.Buffer(group, int(2e9), int(1e9) if world > 8 else 0, explicitly_destroy=True)
        run_layer = lambda x, idx, w: buf.teramoe_autograd(x, idx, w, Wg, Wd, E, num_dispatch_sms=32, num_combine_sms=32)

    x_dev, go_dev, idx_dev, w_dev = x_host.to(dev), go_host.to(dev), idx_host.to(dev), w_host.to(dev)

    def step_device():
        x = x_dev.detach().requires_grad_(True)
        w = w_dev.detach().requires_grad_(True)
        out = run_layer(x, idx_dev, w)
        out.backward(go_dev)
        Wg.grad = None
        Wd.grad = None
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- activation memory, the reference's protocol (tests/teramoe_test_utils.py:229-252)
    for _ in range(2):
        step_device()
    barrier()
    torch.cuda.reset_peak_memory_stats()
    m0 = torch.cuda.memory_allocated()
    xa = x_dev.detach().requires_grad_(True)
    wa = w_dev.detach().requires_grad_(True)
    outa = run_layer(xa, idx_dev, wa)
    torch.cuda.synchronize()
    act_mb = (torch.cuda.memory_allocated() - m0) / 2 ** 20
    outa.backward(go_dev)
    Wg.grad = None
    Wd.grad = None
    del outa, xa, wa
    peak_mb = (torch.cuda.max_memory_allocated() - m0) / 2 ** 20

    # ---- device-timed region: warm-up, then exactly K steps; inputs (weights 2.8 GB/rank) exceed the 126 MB L2
    for _ in range(max(args.warmup, 3)):
        step_device()
    barrier()
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    l0 = ext.launch_count()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    wall0 = time.perf_counter()
    evs[0].record()
    for i in range(args.steps):
        step_device()
        evs[i + 1].record()
    barrier()
    wall_ms = (time.perf_counter() - wall0) * 1e3
    launches = (ext.launch_count() - l0)
    total_ms = evs[0].elapsed_time(evs[-1])
    per_step = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    ms = total_ms / args.steps

    # ---- end to end through the public API: every step copies its inputs from pinned host memory
    # (prefetched on a copy stream, double-buffered) and reads the loss back to the host
    e2e = None
    if not args.no_e2e:
        copy_stream = torch.cuda.Stream()
        slots = [[torch.empty_like(x_dev), torch.empty_like(go_dev), torch.empty_like(idx_dev), torch.empty_like(w_dev)] for _ in range(2)]
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]
        loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()

        def prefetch(i):
            s = i % 2
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[s])
                for d, h in zip(slots[s], (x_host, go_host, idx_host, w_host)):
                    d.copy_(h, non_blocking=True)
                ready[s].record(copy_stream)

        def step_e2e(i, n):
            s = i % 2
            cur = torch.cuda.current_stream()
            cur.wait_event(ready[s])
            if i + 1 < n:
                prefetch(i + 1)
            xd, god, idxd, wd = slots[s]
            x = xd.detach().requires_grad_(True)
            w = wd.detach().requires_grad_(True)
            out = run_layer(x, idxd, w)
            loss = (out * god).sum(dtype=torch.float32) / out.numel()      # scalar the host reads back every step
            out.backward(god)
            consumed[s].record(cur)
            Wg.grad = None
            Wd.grad = None
            loss_host.copy_(loss.detach().reshape(1), non_blocking=True)
            return loss_host

        for c in consumed:
            c.record()
        nw = max(args.warmup, 3)
        prefetch(0)
        for i in range(nw):
            step_e2e(i, nw)
        barrier()
        for c in consumed:
            c.record()
        prefetch(0)
        s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        s_ev.record()
        for i in range(args.steps):
            step_e2e(i, args.steps)
        e_ev.record()
        e_ev.synchronize()
        float(loss_host[0])
        barrier()
        e2e_wall = (time.perf_counter() - t0) * 1e3 / args.steps
        e2e_ms = max(s_ev.elapsed_time(e_ev) / args.steps, 0.0)
        h2d = sum(t.numel() * t.element_size() for t in (x_host, go_host, idx_host, w_host))
        e2e = {"ms": e2e_ms, "wall_ms": e2e_wall, "h2d": h2d, "d2h": 4}

    clocks = sampler.stop() if sampler is not None else None
    if args.trace and args.impl == "teramoe":
        buf.trace(True)
        for _ in range(3):
            step_device()
        rep = buf.trace_report()
        buf.trace(False)
        if rank == 0:
            tot = sum(rep.values())
            print("phase trace (ms, mean of 3 steps; events serialise nothing):", file=sys.stderr)
            for k, v in rep.items():
                print(f"  {k:40s} {v:8.3f}", file=sys.stderr)
            print(f"  {'sum':40s} {tot:8.3f}", file=sys.stderr)
            print("wait times inside the layer kernels (ms per CTA pair):", buf._engine.wait_report(), file=sys.stderr)

    def reduce_max(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms_max = reduce_max(ms)
    act_max = reduce_max(act_mb)
    e2e_max = reduce_max(e2e["ms"]) if e2e else None
    e2e_wall_max = reduce_max(e2e["wall_ms"]) if e2e else None

    if rank == 0:
        flops = 18.0 * T * K * H * I          # fwd 6*S*H*I + bwd 12*S*H*I per rank, S = T*K
        out = {
            "metric": METRIC,
            "value": round(ms_max, 4),
            "unit": "ms",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_max, 4),
            "higher_is_better": False,
            "scaling": "weak",
            "vs_baseline": (round(ms_max / PUBLISHED_MS[args.config], 4) if args.config in PUBLISHED_MS else None),
            "dtype": "bf16",
            "data": "synthetic (random tokens, uniform random top-k routing, random-init weights)",
            "impl": args.impl,
            "config": {"model": f"moe_layer[{args.config}] H={H} I={I} experts/rank={El} experts={E} top{K}", "global_batch": T * world,
                       "seq_len": T, "tokens_per_rank": T, "parallelism": f"ep{world}", "peak_to_mean": p2m,
                       "l2": "inputs larger than L2 (expert weights %.1f GB per rank are re-read every step)" % (El * 3 * H * I * 2 / 1e9)},
            "paths": (dict(getattr(buf._engine, "last_paths", {})) if args.impl == "teramoe" else None),
            "tokens_per_s": round(T * world / (ms_max * 1e-3), 1),
            "tflops_per_gpu": round(flops / (ms_max * 1e-3) / 1e12, 1),
            "activation_mb": round(act_max, 2),
            "peak_mb": round(peak_mb, 2),
            "ms_per_step_rank0_min": round(min(per_step), 4),
            "wall_ms_per_step": round(wall_ms / args.steps, 4),
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if e2e:
            out["e2e"] = {"value": round(e2e_max, 4), "unit": "ms", "wall_ms": round(e2e_wall_max, 4),
                          "h2d_bytes_per_step": int(e2e["h2d"]), "d2h_bytes_per_step": int(e2e["d2h"])}
        print(json.dumps(out), flush=True)
    if args.impl != "nccl":
        buf.destroy()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
