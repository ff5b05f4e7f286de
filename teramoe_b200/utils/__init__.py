"""Host-side helpers: CUDA-event wrapper, NVLink topology check, numerics check, timing."""
from .events import EventHandle, EventOverlap
from .nvlink import check_nvlink_connections
from .numerics import numerics_report, assert_close_bf16
from .timing import bench_cuda, ClockSampler, max_over_ranks

__all__ = ["EventHandle", "EventOverlap", "check_nvlink_connections", "numerics_report", "assert_close_bf16", "bench_cuda",
           "ClockSampler", "max_over_ranks"]
