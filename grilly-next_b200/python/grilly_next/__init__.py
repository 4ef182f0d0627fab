"""grilly_next, attention / KV-cache subset, CUDA (sm_100a) backend.

Mirrors the reference package's public names (src/grilly_next/__init__.py): Compute,
VulkanCompute, VULKAN_AVAILABLE.  "VULKAN_AVAILABLE" keeps its name for drop-in compatibility; it
is true when the grilly_core extension (here: the CUDA build) can be imported.
"""
from grilly_next.backend import VULKAN_AVAILABLE
from grilly_next.backend.compute import VulkanCompute

Compute = VulkanCompute

__all__ = ["VULKAN_AVAILABLE", "VulkanCompute", "Compute"]
__version__ = "0.5.0.dev0+b200"
