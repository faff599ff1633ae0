"""Errors of the kernel library, importable without a CUDA device."""


class KernelError(RuntimeError):
    """A kernel refused its input, could not be built or loaded, or reported a fault
    (for instance a bounded wait inside a kernel that gave up)."""
