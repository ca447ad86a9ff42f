"""Device facts for the host-side heuristics (role of triton_kernels/target_info.py:60-74).
Unlike the reference (which hard-codes device 0) the current device is queried."""
import functools

import torch

from . import _lib


@functools.lru_cache(maxsize=None)
def _info(device: int):
    info = _lib.MoeDeviceInfo()
    _lib.check(_lib.load().moe_device_info(device, info), "moe_device_info")
    return info


def device_info(device=None):
    return _info(torch.cuda.current_device() if device is None else int(device))


def num_sms(device=None) -> int:
    return device_info(device).sm_count


def cuda_capability_geq(major, minor=0) -> bool:
    i = device_info()
    return (i.cc_major, i.cc_minor) >= (major, minor)


def is_cuda() -> bool:
    return True


def is_hip() -> bool:
    return False
