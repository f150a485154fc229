"""Platform capability seam: what the device can do and which kernels the engine may pick.

Reference: ``include/vllm/platforms/interface.h``, ``src/vllm/platforms/{platform,cpu,cuda,
metal,vulkan}.cpp``. Only the CPU oracle and CUDA sm_100a exist here; the Metal and Vulkan
back ends of the reference have no counterpart (no graphics stack on the target machines).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class DeviceCapability:
    major: int
    minor: int

    def as_int(self) -> int:
        return self.major * 10 + self.minor


class Platform:
    name = "base"
    device_type = "cpu"

    def device_capability(self, index: int = 0) -> DeviceCapability | None:
        return None

    def supports_fp8(self) -> bool:
        return False

    def supports_nvfp4(self) -> bool:
        """Block-scaled FP4 tensor cores: compute capability 10.0 - 12.9."""
        return False

    def is_integrated(self) -> bool:
        return False

    def total_memory(self, index: int = 0) -> int:
        return 0

    def attention_backends(self) -> list[str]:
        return ["reference"]

    def residency_policy(self) -> str:
        """Where weights live: "device" (discrete memory) or "unified"."""
        return "device"

    def supports_cuda_graphs(self) -> bool:
        return False


class CpuPlatform(Platform):
    name = "cpu"

    def total_memory(self, index: int = 0) -> int:
        import psutil
        return psutil.virtual_memory().total

    def residency_policy(self) -> str:
        return "unified"


class CudaPlatform(Platform):
    name = "cuda"
    device_type = "cuda"

    def device_capability(self, index: int = 0):
        import torch
        mj, mn = torch.cuda.get_device_capability(index)
        return DeviceCapability(mj, mn)

    def supports_fp8(self) -> bool:
        c = self.device_capability()
        return c is not None and c.as_int() >= 89

    def supports_nvfp4(self) -> bool:
        c = self.device_capability()
        return c is not None and 100 <= c.as_int() <= 129

    def is_blackwell_datacenter(self) -> bool:
        c = self.device_capability()
        return c is not None and c.major == 10

    def total_memory(self, index: int = 0) -> int:
        import torch
        return torch.cuda.get_device_properties(index).total_memory

    def attention_backends(self) -> list[str]:
        return ["tcgen05_paged", "cuda_core_paged"] if self.is_blackwell_datacenter() else ["cuda_core_paged"]

    def supports_cuda_graphs(self) -> bool:
        return True


class UnavailablePlatform(Platform):
    """Metal / Vulkan: named for interface parity only."""

    def __init__(self, name: str):
        self.name = name

    def device_capability(self, index: int = 0):
        raise RuntimeError(f"the {self.name} platform is not available in this build")


def current_platform(device: str | None = None) -> Platform:
    import torch
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    if device.startswith("cuda"):
        return CudaPlatform()
    if device in ("metal", "vulkan"):
        return UnavailablePlatform(device)
    return CpuPlatform()
