"""Small host-side helpers shared by the training scripts.

Same surface as the reference's ``src/himuon/utils.py:11-59``
(``seed_everything``, ``parse_kv_args``, ``merge_kv_args``, ``TimeBudget``)
plus device-side timing helpers used by the benchmarks.
"""

from .misc import TimeBudget, merge_kv_args, parse_kv_args, seed_everything
from .timing import ClockSampler, PhaseTimer, cuda_time_ms, l2_flush_buffer, max_over_ranks, nvtx_range

__all__ = [
    "seed_everything",
    "parse_kv_args",
    "merge_kv_args",
    "TimeBudget",
    "cuda_time_ms",
    "max_over_ranks",
    "l2_flush_buffer",
    "ClockSampler",
    "PhaseTimer",
    "nvtx_range",
]
