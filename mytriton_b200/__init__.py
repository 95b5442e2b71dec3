"""mytriton_b200 — a B200 (sm_100a) execution backend for mytriton-style kernels.

``import mytriton_b200 as triton; import mytriton_b200.language as tl`` gives the
same ``@triton.jit`` / ``tl.*`` surface as the reference package
(``src/mytriton/__init__.py:1-15``).
"""

from .autotune import Config, autotune
from .compiler import jit
from .cuda_utils import cuda_available


def cdiv(x: int, y: int) -> int:
    return -(-x // y)


def next_power_of_2(value: int) -> int:
    """Smallest power of two that is not below ``value``."""
    if value < 1:
        raise ValueError("value must be positive")
    power = 1
    while power < value:
        power *= 2
    return power


__all__ = ["Config", "autotune", "cdiv", "cuda_available", "jit", "next_power_of_2"]
