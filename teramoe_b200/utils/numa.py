"""Keep a rank's host threads and pinned memory next to its GPU.

A launcher such as torchrun does not bind its workers.  On a two-socket host half of the ranks then run (and first-touch
their pinned staging buffers) on the socket that is NOT attached to their GPU, so every host-to-device copy and every
kernel launch crosses the socket interconnect; with eight ranks copying at once that link becomes the bottleneck of an
end-to-end step.  `bind_to_gpu` asks NVML (a read-only query) which CPUs are local to the GPU and restricts THIS
process to them.  It changes nothing on the GPU.  The reference leaves placement to the job launcher (its tests spawn
unbound workers, tests/utils.py:14-36).
"""
from __future__ import annotations

import os
from typing import Optional


def gpu_cpu_affinity(gpu_index: int) -> Optional[list]:
    """CPUs that NVML reports as local to physical GPU `gpu_index`, or None if that cannot be found out."""
    try:
        import pynvml
    except ImportError:
        return None
    try:
        pynvml.nvmlInit()
    except Exception:
        return None
    try:
        handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        ncpu = os.cpu_count() or 1
        words = (ncpu + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = [64 * i + b for i, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1]
        return cpus or None
    except Exception:
        return None
    finally:
        try:
            pynvml.nvmlShutdown()
        except Exception:
            pass


def bind_to_gpu(local_rank: int) -> Optional[list]:
    """Restrict this process to the CPUs local to its GPU.  Returns the CPU list, or None if nothing was changed
    (no NVML, no affinity information, or the allowed set would become empty)."""
    if os.environ.get("TERAMOE_NO_BIND", "0") == "1" or not hasattr(os, "sched_setaffinity"):
        return None
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    index = local_rank
    if visible:
        ids = [v for v in visible.split(",") if v.strip() != ""]
        if local_rank < len(ids) and ids[local_rank].strip().isdigit():
            index = int(ids[local_rank])
    cpus = gpu_cpu_affinity(index)
    if not cpus:
        return None
    allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
    if not allowed:
        return None
    try:
        os.sched_setaffinity(0, allowed)
    except OSError:
        return None
    return allowed
