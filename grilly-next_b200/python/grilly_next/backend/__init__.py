"""Grilly backend: every op goes through the grilly_core C++ extension (no Python fallback)."""
from ._bridge import NATIVE_AVAILABLE

VULKAN_AVAILABLE = NATIVE_AVAILABLE

from .compute import VulkanCompute  # noqa: E402

__all__ = ["VULKAN_AVAILABLE", "NATIVE_AVAILABLE", "VulkanCompute"]
