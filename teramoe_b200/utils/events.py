"""CUDA event wrappers with the reference's overlap protocol.

Reference counterparts: csrc/event.hpp:9-40 (EventHandle), teramoe/utils.py:10-61 (EventOverlap).
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch


class EventHandle:
    """A CUDA event recorded on a stream at construction (current stream by default)."""

    def __init__(self, stream: Optional["torch.cuda.Stream"] = None):
        self.event = None
        if torch.cuda.is_available():
            self.event = torch.cuda.Event()
            self.event.record(stream if stream is not None else torch.cuda.current_stream())

    def current_stream_wait(self) -> None:
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)

    def synchronize(self) -> None:
        if self.event is not None:
            self.event.synchronize()


class EventOverlap:
    """Event + the tensors whose lifetime must cover the asynchronous work (a stand-in for
    `record_stream` that also works under CUDA-graph capture)."""

    def __init__(self, event: Optional[EventHandle] = None, extra_tensors: Optional[Tuple[torch.Tensor, ...]] = None) -> None:
        self.event = event
        self.extra_tensors = extra_tensors

    def current_stream_wait(self) -> None:
        assert self.event is not None
        self.event.current_stream_wait()

    def __enter__(self) -> Any:
        return self

    def __exit__(self, exc_type: Any, exc_val: Any, exc_tb: Any) -> None:
        if self.event is not None:
            self.event.current_stream_wait()
