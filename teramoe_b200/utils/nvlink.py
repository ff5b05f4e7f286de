"""NVLink reachability check between the GPUs of a group (reference: teramoe/utils.py:64-101).

B200 boards sit behind NVSwitch, so every pair is connected; the check only does work on PCIe
parts, where it asks NVML (read-only queries) whether each pair has an NVLink path.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def check_nvlink_connections(group) -> None:
    if not torch.cuda.is_available():
        return
    name = torch.cuda.get_device_name()
    if "PCIE" not in name.upper():
        return
    try:
        import pynvml
    except ImportError:  # pragma: no cover
        return
    pynvml.nvmlInit()
    try:
        devices = os.environ.get("CUDA_VISIBLE_DEVICES", "0,1,2,3,4,5,6,7").strip(",").split(",")
        physical = int(devices[torch.cuda.current_device()])
        ids = [None] * dist.get_world_size(group)
        dist.all_gather_object(ids, physical, group)
        handles = [pynvml.nvmlDeviceGetHandleByIndex(i) for i in ids]
        for i, hi in enumerate(handles):
            for j, hj in enumerate(handles):
                if i >= j:
                    continue
                status = pynvml.nvmlDeviceGetP2PStatus(hi, hj, pynvml.NVML_P2P_CAPS_INDEX_NVLINK)
                if status != pynvml.NVML_P2P_STATUS_OK:
                    raise RuntimeError(f"GPU {ids[i]} and GPU {ids[j]} are not connected through NVLink")
    finally:
        pynvml.nvmlShutdown()
