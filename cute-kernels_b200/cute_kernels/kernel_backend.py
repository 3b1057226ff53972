"""Names kept for signature compatibility with the reference (cute_kernels/kernel_backend.py:7-20,
cute_kernels/cutotune/parameter.py).  There is one backend here: hand-written sm_100a CUDA."""

from enum import Enum


class CutoTuneParameter:
    """Placeholder the reference uses for "let the tuner decide"; accepted and ignored."""


class KernelBackend(Enum):
    cuda = "cuda"
    triton = "triton"


def resolve_backend(kernel_backend) -> None:
    """Accepts None / CutoTuneParameter / KernelBackend.cuda; a Triton request is an error."""
    if kernel_backend is None or isinstance(kernel_backend, CutoTuneParameter) or kernel_backend == KernelBackend.cuda:
        return
    if kernel_backend == KernelBackend.triton:
        raise ValueError("this build has no Triton backend: kernels are sm_100a CUDA only")
    raise ValueError("unexpected kernel_backend")
