"""Kernel sets: the interface parts are written against and the CUDA implementation."""

from .interface import KernelSet, KvSlot, RotaryTable, StepTensors

__all__ = ["KernelSet", "KvSlot", "RotaryTable", "StepTensors", "make_kernels"]


def make_kernels(dtype, device="cuda:0") -> KernelSet:
    """The product's kernel set for ``dtype`` (torch.bfloat16 or torch.float32)."""
    from .device import DeviceKernels

    return DeviceKernels(dtype, device)
