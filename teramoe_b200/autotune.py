"""Grid search over (compute_batch_size, combine_start_head_percent), the two arguments that shape the work list of the
whole-layer kernel (batch size of the schedule; how far the first GEMM runs ahead of the second GEMM + combine push).
`num_dispatch_sms` and `stage` can be swept as well (`dispatch_sms_list`, `stages`); the best of them is recorded in the
result's `extra`.

Same signature and return value as the reference (teramoe/autotune.py:59-177): returns
(AutotuneResult, [(compute_batch_size, percent, ms), ...]).  Differences: the timed region can be
forward + backward (`mode="fwd_bwd"`, what a training step pays; the reference times forward only),
and the time of a configuration is the maximum over ranks, not rank 0's.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

COMPUTE_BATCH_SIZES = [1024, 2048, 4096]
COMBINE_START_HEAD_PERCENTS = [40, 50, 60, 70, 80, 90]


@dataclass
class AutotuneResult:
    compute_batch_size: int
    combine_start_head_percent: int
    time_ms: float
    forward_ms: Optional[float] = None
    backward_ms: Optional[float] = None
    extra: Optional[dict] = None          # {"num_dispatch_sms": ..., "stage": ...} of the best configuration when those were swept


def _barrier(group):
    if dist.is_available() and dist.is_initialized() and (group is not None or dist.get_world_size() > 1):
        dist.barrier(group=group)


def _max_over_ranks(v: float, group, device) -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return v
    t = torch.tensor([v], dtype=torch.float64, device=device if dist.get_backend(group) == "nccl" else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def autotune_teramoe(buffer, x, topk_idx, topk_weights, W_gateup, W_down, num_experts, num_dispatch_sms: int = 24,
                     num_combine_sms: int = 24, total_sms: int = 148, stage: int = 1, num_iters: int = 1000, warmup_iters: int = 10,
                     verbose: bool = True, group: Optional[dist.ProcessGroup] = None, mode: str = "fwd",
                     compute_batch_sizes=None, combine_start_head_percents=None, dispatch_sms_list=None,
                     stages=None) -> Tuple[AutotuneResult, List[Tuple[int, int, float]]]:
    if mode not in ("fwd", "fwd_bwd"):
        raise ValueError("mode must be 'fwd' or 'fwd_bwd'")
    group = group if group is not None else buffer.group
    cbs_list = list(compute_batch_sizes or COMPUTE_BATCH_SIZES)
    pct_list = list(combine_start_head_percents or COMBINE_START_HEAD_PERCENTS)
    cuda = x.is_cuda
    results: List[Tuple[int, int, float]] = []
    best: Optional[AutotuneResult] = None
    grad_out = torch.randn_like(x) if mode == "fwd_bwd" else None
    leaves = None
    if mode == "fwd_bwd":
        leaves = [t.detach().requires_grad_(True) for t in (x, topk_weights, W_gateup, W_down)]

    extra_grid = list(itertools.product(list(dispatch_sms_list or [num_dispatch_sms]), list(stages or [stage])))
    cur = {"num_dispatch_sms": num_dispatch_sms, "stage": stage}

    def step(cbs, pct):
        kw = dict(num_dispatch_sms=cur["num_dispatch_sms"], num_combine_sms=num_combine_sms, total_sms=total_sms, stage=cur["stage"],
                  compute_batch_size=cbs, combine_start_head_percent=pct)
        if mode == "fwd":
            buffer.teramoe_autograd(x, topk_idx, topk_weights, W_gateup, W_down, num_experts, **kw)
        else:
            lx, lw, lg, ld = leaves
            out = buffer.teramoe_autograd(lx, topk_idx, lw, lg, ld, num_experts, **kw)
            out.backward(grad_out)
            for t in leaves:
                t.grad = None

    for (dsm, stg), (cbs, pct) in itertools.product(extra_grid, itertools.product(cbs_list, pct_list)):
        cur["num_dispatch_sms"], cur["stage"] = dsm, stg
        _barrier(group)
        for _ in range(warmup_iters):
            step(cbs, pct)
        if cuda:
            torch.cuda.synchronize()
        _barrier(group)
        if cuda:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(num_iters):
                step(cbs, pct)
            e.record()
            e.synchronize()
            ms = s.elapsed_time(e) / max(num_iters, 1)
        else:
            import time
            t0 = time.perf_counter()
            for _ in range(num_iters):
                step(cbs, pct)
            ms = (time.perf_counter() - t0) * 1e3 / max(num_iters, 1)
        ms = _max_over_ranks(ms, group, x.device)
        results.append((cbs, pct, ms))
        if verbose and buffer.rank == 0:
            more = f" num_dispatch_sms={dsm} stage={stg}" if len(extra_grid) > 1 else ""
            print(f"[autotune] compute_batch_size={cbs} combine_start_head_percent={pct}{more}: {ms:.4f} ms", flush=True)
        if best is None or ms < best.time_ms:
            best = AutotuneResult(cbs, pct, ms, extra=(dict(cur) if len(extra_grid) > 1 else None))
    if verbose and buffer.rank == 0 and best is not None:
        print(f"[autotune] best: compute_batch_size={best.compute_batch_size} "
              f"combine_start_head_percent={best.combine_start_head_percent} ({best.time_ms:.4f} ms)", flush=True)
    return best, results
