"""continuous_count_cute: histogram of expert ids (reference: kernels/continuous_count/__init__.py:12-38)."""

import torch

from . import _lib


def _continuous_count_impl(x: torch.Tensor, output: torch.Tensor, size: int) -> None:
    _lib.require_cuda(x, output)
    with torch.cuda.device(x.device), _lib.launch("continuous_count", 1 if x.numel() else 0):
        st = _lib.lib.ck_continuous_count(
            x.data_ptr(), int(x.dtype == torch.int64), x.numel(), size, output.data_ptr(), _lib.stream_ptr()
        )
    _lib.check(st, "ck_continuous_count")


# opaque to torch.compile, like the reference's cute_op wrapper (utils/custom_op.py:34-57)
_continuous_count_op = torch.library.custom_op(
    "cute_kernels_b200::continuous_count", _continuous_count_impl, mutates_args={"output"}
)


@torch.no_grad()
def continuous_count_cute(x: torch.Tensor, size: int) -> torch.Tensor:
    """Counts the occurrences of the values [0, size) in the 1-D integer tensor ``x``.

    Values outside the range are ignored.  Returns a ``uint32`` tensor of ``size`` elements, equal to
    ``x.bincount(minlength=size).to(torch.uint32)`` for in-range inputs.  Same signature, dtypes
    (int32 / int64) and ``size == 1`` shortcut as the reference.
    """
    if size == 1:
        return torch.tensor([x.numel()], dtype=torch.uint32, device=x.device)

    assert x.dim() == 1, "x should be 1-dimensional"
    assert x.dtype in [torch.int32, torch.long]
    if size > _lib.CK_COUNT_MAX_SIZE:
        raise RuntimeError(f"size ({size}) exceeds the supported maximum of {_lib.CK_COUNT_MAX_SIZE}")

    x = x.contiguous()
    output = torch.empty(size, dtype=torch.uint32, device=x.device)
    (_continuous_count_op if _lib.use_custom_op() else _continuous_count_impl)(x, output, size)
    return output
