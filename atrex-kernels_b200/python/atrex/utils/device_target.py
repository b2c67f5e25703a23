"""Which accelerator family and architecture a torch device really is.

Same observable behaviour as the reference's classifier
(python/atrex/utils/device_target.py:25-66): ROCm is recognised before anything
else because it also answers through ``torch.cuda``; an Alibaba PPU is
recognised by its exact product name because it reports a CUDA compute
capability; only then is a device whose name starts with ``NVIDIA`` labelled
``sm<major><minor>``.  A B200 is ``("nvidia", "sm100")``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True, slots=True)
class DeviceTarget:
    family: str
    arch: str
    runtime_version: str | None
    device_index: int


_PPU_ARCH_BY_PRODUCT = {"ZW-M890P": "zwm890p"}


def _device_index(torch, device):
    """-1 for "no accelerator", a non-negative CUDA ordinal otherwise, or a str for a non-CUDA type."""
    if device is None:
        return torch.cuda.current_device() if torch.cuda.is_available() else -1
    if isinstance(device, int):
        return device
    resolved = torch.device(device)
    if resolved.type != "cuda":
        return resolved.type
    return torch.cuda.current_device() if resolved.index is None else resolved.index


def detect_device_target(device: Any = None) -> DeviceTarget:
    import torch  # deferred: importing atrex must not import torch

    index = _device_index(torch, device)
    if isinstance(index, str):
        return DeviceTarget(index, index, None, -1)
    if index < 0:
        return DeviceTarget("unavailable", "unavailable", None, -1)

    props = torch.cuda.get_device_properties(index)
    product = props.name.strip()
    if torch.version.hip is not None:
        gfx = getattr(props, "gcnArchName", "").partition(":")[0]
        return DeviceTarget("amd", gfx or "unknown", torch.version.hip, index)
    if product in _PPU_ARCH_BY_PRODUCT:
        return DeviceTarget("alibaba_ppu", _PPU_ARCH_BY_PRODUCT[product], torch.version.cuda, index)
    if torch.version.cuda is not None and product.upper().startswith("NVIDIA "):
        major, minor = torch.cuda.get_device_capability(index)
        return DeviceTarget("nvidia", f"sm{major}{minor}", torch.version.cuda, index)
    return DeviceTarget("unknown", "unknown", None, index)
