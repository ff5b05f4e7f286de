"""teramoe_b200: Blackwell-native expert-parallel Mixture-of-Experts training library.

Public surface (same names as the reference package, teramoe/__init__.py:1-8):
Buffer, EventOverlap, Config, topk_idx_t, autotune_teramoe, AutotuneResult.
"""
from .config import Config, topk_idx_t
from .utils.events import EventHandle, EventOverlap
from .buffer import Buffer
from .autotune import AutotuneResult, autotune_teramoe
from .reference import moe_reference

__version__ = "0.1.0"
__all__ = ["Buffer", "EventOverlap", "EventHandle", "Config", "topk_idx_t", "autotune_teramoe", "AutotuneResult", "moe_reference"]
