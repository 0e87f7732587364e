"""Facts about the GPU that launch plans depend on, asked of the device instead of written into the code."""
from __future__ import annotations

from typing import Dict, Optional

import torch

# What host-only tests of the launch plans assume when there is no device to ask: a B200.
DEFAULT_SM_COUNT = 148

_sm_counts: Dict[int, int] = {}


def sm_count(device: Optional[torch.device] = None) -> int:
    """Multiprocessors of `device` (default: the current one); DEFAULT_SM_COUNT without CUDA."""
    if not torch.cuda.is_available():
        return DEFAULT_SM_COUNT
    index = torch.device(device).index if device is not None else None
    if index is None:
        index = torch.cuda.current_device()
    got = _sm_counts.get(index)
    if got is None:
        got = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return got
