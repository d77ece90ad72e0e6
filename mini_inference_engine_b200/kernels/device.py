"""What the launch plans need to know about the GPU, asked of the device once."""
from __future__ import annotations

import functools

import torch

B200_SMS = 148          # what a plan made without a device (a test of the planning arithmetic on the CPU) assumes


@functools.lru_cache(maxsize=None)
def _properties(index: int):
    return torch.cuda.get_device_properties(index)


def num_sms(device=None) -> int:
    """Streaming multiprocessors of ``device`` (the current one by default)."""
    if not torch.cuda.is_available():
        return B200_SMS
    index = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    return _properties(index).multi_processor_count
