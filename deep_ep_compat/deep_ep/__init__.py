"""Drop-in `deep_ep` module backed by `gpu_data_transfer_profile_b200`.

Put this directory on PYTHONPATH (`PYTHONPATH=<repo>/deep_ep_compat:<repo>`) and scripts written
against DeepEP's V1 Python API, such as the reference's `DeepEP_v1/deepep_v1_dispatch.py`,
`DeepEP_v1/deepep_v1_combine.py` and `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py`,
import this library instead: `Buffer`, `Config` size hints, `EventOverlap`, `EventHandle` and
`topk_idx_t` keep the names and call shapes those scripts use (`deepep_v1_dispatch.py:19-56,176-230`).
"""
from gpu_data_transfer_profile_b200.parallel.buffer import Buffer, DispatchHandle, EpStatusError, EpTimeoutError
from gpu_data_transfer_profile_b200.parallel.config import Config
from gpu_data_transfer_profile_b200.parallel.events import EventHandle, EventOverlap, topk_idx_t

__all__ = ["Buffer", "Config", "EventHandle", "EventOverlap", "topk_idx_t", "DispatchHandle",
           "EpStatusError", "EpTimeoutError"]
__version__ = "b200ep-compat"
