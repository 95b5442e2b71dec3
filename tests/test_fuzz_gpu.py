"""Differential fuzzing of the code generator on the GPU.

Seeded random kernels — elementwise expression trees over i32/f32 blocks and scalars,
with rank-2 broadcasting and a final reduction in some of them — are written to a
temporary module, compiled by this backend and run on the device; the CPU oracle
(oracle/ssa_interp.py) interprets the same kernel's printed SSA.  Results must agree to
rtol 1e-5 / atol 1e-5 (the device contracts a*b+c into one FMA and its expf differs
from NumPy's exp in the last ulp), NaNs in the same places.
"""

import importlib.util
import itertools

import numpy as np
import pytest

from mytriton_b200 import device, runtime
from mytriton_b200.ssa import SSAPrinter
from oracle import ssa_interp

pytestmark = pytest.mark.gpu

HEADER = "import mytriton_b200 as triton\nimport mytriton_b200.language as tl\n\n\n"


class ExprGen:
    """Random expressions with a tracked element type ("i" or "f")."""

    def __init__(self, rng, float_leaves, int_leaves):
        self.rng = rng
        self.float_leaves = float_leaves
        self.int_leaves = int_leaves

    def leaf(self, want):
        if want == "i":
            pool = self.int_leaves + [str(int(self.rng.integers(-4, 5)))]
        else:
            pool = self.float_leaves + [repr(float(np.round(self.rng.uniform(-2, 2), 2)))]
        return pool[int(self.rng.integers(len(pool)))]

    def expr(self, depth, want="f"):
        if depth == 0 or self.rng.random() < 0.15:
            return self.leaf(want)
        choice = int(self.rng.integers(8))
        if want == "i":
            lhs, rhs = self.expr(depth - 1, "i"), self.expr(depth - 1, "i")
            if choice < 3:
                return f"({lhs} + {rhs})"
            if choice < 5:
                return f"({lhs} - {rhs})"
            if choice == 5:
                return f"tl.maximum({lhs}, {rhs})"
            if choice == 6:
                return f"({lhs} / {int(self.rng.choice([-3, 2, 3, 5]))})"      # C division
            return f"tl.where({self.cond(depth - 1)}, {lhs}, {rhs})"
        kinds = ("f", "f") if self.rng.random() < 0.6 else ("f", "i")          # mixed promotes to f32
        lhs, rhs = (self.expr(depth - 1, k) for k in self.rng.permutation(kinds))
        if choice == 0:
            return f"({lhs} + {rhs})"
        if choice == 1:
            return f"({lhs} - {rhs})"
        if choice == 2:
            return f"({lhs} * {rhs})"
        if choice == 3:
            return f"({lhs} / ({self.expr(depth - 1, 'f')} * 0.25 + 3.5))"
        if choice == 4:
            return f"tl.minimum({lhs}, {rhs})"
        if choice == 5:
            return f"tl.exp(tl.minimum({self.expr(depth - 1, 'f')}, 3.0))"
        if choice == 6:
            return f"(-{self.expr(depth - 1, 'f')})"
        return f"tl.where({self.cond(depth - 1)}, {lhs}, {rhs})"

    def cond(self, depth):
        kind = "f" if self.rng.random() < 0.5 else "i"
        first = f"({self.expr(depth, kind)} < {self.expr(depth, kind)})"
        if self.rng.random() < 0.3:
            return f"({first} & ({self.expr(depth, 'i')} < {self.expr(depth, 'i')}))"
        return first


def rank1_kernel(rng, name):
    gen = ExprGen(rng, ["a", "b", "s"], ["offs", "n", "lanes"])
    result = gen.expr(3, "f" if rng.random() < 0.8 else "i")
    reduce = rng.random() < 0.35
    lines = [
        "@triton.jit",
        f"def {name}(x0, x1, out, n, s, BLOCK: tl.constexpr):",
        "    pid = tl.program_id(0)",
        "    lanes = tl.arange(0, BLOCK)",
        "    offs = pid * BLOCK + lanes",
        "    mask = offs < n",
        "    a = tl.load(x0 + offs, mask=mask, other=0.5)",
        "    b = tl.load(x1 + offs, mask=mask, other=-1.0)",
        f"    r = {result}",
    ]
    if reduce:
        op = ["tl.sum", "tl.max", "tl.min"][int(rng.integers(3))]
        lines += [f"    total = {op}(tl.where(mask, r, 0 * r))",
                  "    tl.store(out + pid, total, mask=lanes < 1)"]
    else:
        lines += ["    tl.store(out + offs, r, mask=mask)"]
    return "\n".join(lines) + "\n\n\n", reduce


def rank2_kernel(rng, name):
    gen = ExprGen(rng, ["tile", "rowv", "colv", "s"], ["offs_m", "offs_n", "M"])
    result = gen.expr(3, "f")
    lines = [
        "@triton.jit",
        f"def {name}(x0, x1, out, M, N, s, BM: tl.constexpr, BN: tl.constexpr):",
        "    offs_m = tl.program_id(0) * BM + tl.arange(0, BM)[:, None]",
        "    offs_n = tl.program_id(1) * BN + tl.arange(0, BN)[None, :]",
        "    mask = (offs_m < M) & (offs_n < N)",
        "    tile = tl.load(x0 + offs_m * N + offs_n, mask=mask, other=0.25)",
        "    rowv = tl.load(x1 + offs_m, mask=offs_m < M, other=1.0)",
        "    colv = tl.load(x1 + M + offs_n, mask=offs_n < N, other=2.0)",
        f"    r = {result}",
        "    tl.store(out + offs_m * N + offs_n, r, mask=mask)",
    ]
    return "\n".join(lines) + "\n\n\n"


def load_module(tmp_path, name, source):
    path = tmp_path / f"{name}.py"
    path.write_text(HEADER + source)
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def compare(got, want, label, source):
    nan_got, nan_want = np.isnan(got), np.isnan(want)
    assert np.array_equal(nan_got, nan_want), f"{label}: NaN pattern differs\n{source}"
    finite = ~nan_got
    ok = np.isclose(got[finite], want[finite], rtol=1e-5, atol=1e-5) | (got[finite] == want[finite])
    assert ok.all(), (f"{label}: {int((~ok).sum())} of {ok.size} elements differ, worst "
                      f"{np.abs(got[finite] - want[finite])[~ok].max()}\n{source}")


@pytest.mark.parametrize("seed", range(24))
def test_random_rank1_kernels(seed, tmp_path, gpu):
    rng = np.random.default_rng(1000 + seed)
    name = f"fuzz1_{seed}"
    source, reduce = rank1_kernel(rng, name)
    kernel = getattr(load_module(tmp_path, name, source), name)
    block = int(rng.choice([16, 64, 256, 1024]))
    n = int(rng.integers(block // 2 + 1, 3 * block + 7))
    grid = (-(-n // block),)
    x0 = rng.standard_normal(n, dtype=np.float32)
    x1 = rng.standard_normal(n, dtype=np.float32) * 2
    s = float(np.float32(rng.uniform(-1.5, 1.5)))
    out = np.full(grid[0] if reduce else n, 7.0, dtype=np.float32)
    options = [{}, {"num_warps": 1}, {"elems_per_thread": 2}][seed % 3]
    d0, d1, dout = device.to_device(x0), device.to_device(x1), device.to_device(out)
    _, ssa_ops, _ = kernel[grid](d0, d1, dout, n, s, BLOCK=block, **options)
    runtime.synchronize()
    expected = out.copy()
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops),
                   {"x0": x0.copy(), "x1": x1.copy(), "out": expected, "n": n, "s": s}, grid)
    compare(dout.to_host(), expected, name, source)


@pytest.mark.parametrize("seed", range(12))
def test_random_rank2_kernels(seed, tmp_path, gpu):
    rng = np.random.default_rng(5000 + seed)
    name = f"fuzz2_{seed}"
    source = rank2_kernel(rng, name)
    kernel = getattr(load_module(tmp_path, name, source), name)
    bm, bn = [(4, 8), (16, 32), (8, 64), (6, 10), (32, 32), (1, 128)][seed % 6]
    m, n = int(rng.integers(1, 3 * bm)), int(rng.integers(1, 3 * bn))
    grid = (-(-m // bm), -(-n // bn))
    x0 = rng.standard_normal((m, n), dtype=np.float32)
    x1 = rng.standard_normal(m + n, dtype=np.float32)
    s = float(np.float32(rng.uniform(-1.5, 1.5)))
    out = np.full((m, n), 7.0, dtype=np.float32)
    d0, d1, dout = device.to_device(x0), device.to_device(x1), device.to_device(out)
    _, ssa_ops, _ = kernel[grid](d0, d1, dout, m, n, s, BM=bm, BN=bn)
    runtime.synchronize()
    expected = out.copy()
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops),
                   {"x0": x0.copy(), "x1": x1.copy(), "out": expected, "M": m, "N": n, "s": s}, grid)
    compare(dout.to_host(), expected, name, source)


def test_generators_are_deterministic():
    first = [rank1_kernel(np.random.default_rng(1000 + s), "k")[0] for s in range(3)]
    again = [rank1_kernel(np.random.default_rng(1000 + s), "k")[0] for s in range(3)]
    assert first == again and len(set(itertools.chain(first))) == 3
