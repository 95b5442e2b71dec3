"""tl.dot K-loops -> TMA-fed tcgen05 GEMM kernels (placeholder until the matcher lands)."""

from __future__ import annotations


def match_gemm_loop(ssa_ops, params):
    return None


def generate_gemm(kernel_name, matched, params, codegen):
    raise NotImplementedError
