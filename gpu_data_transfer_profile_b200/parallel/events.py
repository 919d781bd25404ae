"""Stream/event plumbing with the DeepEP call shapes.

Parity: `EventOverlap(EventHandle())` seeds `previous_event`, and
`event.current_stream_wait()` joins the communication stream back into the caller's stream
(`DeepEP_v1/deepep_v1_dispatch.py:171-183`). Here both are thin wrappers over
`torch.cuda.Event`; on a machine without CUDA they degrade to no-ops so that CPU tests of the
host logic can construct them.
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch


class EventHandle:
    """An event captured on the stream that was current at construction."""

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
    """Carries an `EventHandle` plus tensors that must stay alive until it fires.
    Usable as a context manager: leaving the block makes the current stream wait."""

    def __init__(self, event: Optional[EventHandle] = None,
                 extra_tensors: Optional[Tuple[Any, ...]] = None):
        self.event = event
        self.extra_tensors = extra_tensors

    def current_stream_wait(self) -> None:
        if self.event is not None:
            self.event.current_stream_wait()

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        self.current_stream_wait()
        return False


topk_idx_t = torch.int64
