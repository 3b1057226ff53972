"""Small host helpers with the reference's names (cute_kernels/utils/random.py:10-15,
cute_kernels/math.py, cute_kernels/utils/contiguous.py)."""

import random
from functools import wraps

import numpy as np
import torch


def set_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def ceil_divide(x: int, y: int) -> int:
    return (x + y - 1) // y


def divide_if_divisible(dividend: int, divisor: int, msg: str = "") -> int:
    assert dividend % divisor == 0, msg
    return dividend // divisor


def ensure_contiguous(func):
    """Makes every tensor argument contiguous before the call (autograd.Function forward/backward)."""

    @wraps(func)
    def inner(*args, **kwargs):
        args = [a.contiguous() if isinstance(a, torch.Tensor) else a for a in args]
        kwargs = {k: (v.contiguous() if isinstance(v, torch.Tensor) else v) for k, v in kwargs.items()}
        return func(*args, **kwargs)

    return inner
