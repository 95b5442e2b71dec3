"""Expected values, as the reference's execution tests compute them.

TEST INFRASTRUCTURE: not imported by the product.  Every function cites the
reference test that holds the expression.  Inputs and outputs are NumPy arrays;
float32 unless stated.
"""

from __future__ import annotations

import numpy as np


def add(x, y):                      # tests/test_add_kernel.py:254  (x + y)
    return x + y


def copy(x):                        # tests/test_copy_kernel.py:156
    return x.copy()


def sigmoid(x):                     # tests/test_sigmoid_kernel.py:90
    one = np.float32(1.0)
    return one / (one + np.exp(-x))


def relu(x):                        # tests/test_relu_kernel.py:85  (maximum(x, 0))
    return np.maximum(x, np.float32(0.0))


def leaky_relu(x, alpha):           # tests/test_leaky_relu_kernel.py:94
    alpha = np.float32(alpha)
    return np.where(x < np.float32(0.0), alpha * x, x)


def row_sum(x):                     # tests/test_reduce_sum_kernel.py:200
    return np.sum(x, axis=1)


def row_max(x):                     # tests/test_reduce_extremum_kernel.py:182
    return np.max(x, axis=1)


def row_min(x):                     # tests/test_reduce_extremum_kernel.py:183
    return np.min(x, axis=1)


def softmax(x):                     # tests/test_softmax_kernel.py:225-227
    shifted = x - np.max(x, axis=1, keepdims=True)
    numerators = np.exp(shifted)
    return numerators / np.sum(numerators, axis=1, keepdims=True)


def matmul(a, b):                   # tests/test_matmul_2d_kernel.py:189  (a @ b)
    return a @ b


# ---- fp64 references for the tolerance checks the benchmark configurations state

def row_sum_f64(x):
    return np.sum(x.astype(np.float64), axis=1)


def softmax_f64(x):
    x = x.astype(np.float64)
    shifted = x - np.max(x, axis=1, keepdims=True)
    numerators = np.exp(shifted)
    return numerators / np.sum(numerators, axis=1, keepdims=True)


def matmul_f64(a, b):
    """fp64 product of (already bf16-rounded) inputs; the tl.dot yardstick."""
    return a.astype(np.float64) @ b.astype(np.float64)


def relative_frobenius_error(actual, expected_f64) -> float:
    diff = actual.astype(np.float64) - expected_f64
    return float(np.linalg.norm(diff) / np.linalg.norm(expected_f64))


def reduction_relative_error(actual, expected_f64, x) -> float:
    """|error| normalised by the row's sum of magnitudes, so that cancellation in a
    near-zero sum does not make the figure meaningless."""
    scale = np.sum(np.abs(x.astype(np.float64)), axis=1)
    scale = np.where(scale == 0.0, 1.0, scale)
    return float(np.max(np.abs(actual.astype(np.float64) - expected_f64) / scale))


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16, returned widened back to fp32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    out = rounded.astype(np.uint32).view(np.float32).reshape(x.shape)
    return np.where(np.isnan(x), x, out).astype(np.float32)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """The 16-bit patterns of round_to_bf16(x), as uint16."""
    return (round_to_bf16(x).view(np.uint32) >> 16).astype(np.uint16)
