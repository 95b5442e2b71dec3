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


def next_power_of_2(value):
    if value <= 0:
        raise ValueError("value must be positive")
    return 1 << (value - 1).bit_length()


__all__ = ["Config", "autotune", "cdiv", "cuda_available", "jit", "next_power_of_2"]
