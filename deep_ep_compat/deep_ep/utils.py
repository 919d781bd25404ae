"""`from deep_ep.utils import EventHandle, EventOverlap` (the import the reference tries first)."""
from gpu_data_transfer_profile_b200.parallel.events import EventHandle, EventOverlap

__all__ = ["EventHandle", "EventOverlap"]
