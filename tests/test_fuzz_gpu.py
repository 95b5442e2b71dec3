"""Differential fuzzing of the code generator on the GPU.

Seeded random kernels — elementwise expression trees over i32/f32 blocks and scalars,
with rank-2 broadcasting, run-time if/else and early returns on scalars, and a final
reduction in some of them — are written to a
temporary module, compiled by this backend and run on the device; the CPU oracle
(oracle/ssa_interp.py) interprets the same kernel's printed SSA.  Results must agree to
rtol 1e-5 / atol 1e-5 (the device contracts a*b+c into one FMA and its expf differs
from NumPy's exp in the last ulp), NaNs in the same places.
"""

import importlib.util
import itertools
import os

import numpy as np
import pytest

from mytriton_b200 import device, runtime
from mytriton_b200.cuda_utils import NVRTC_OPTIONS
from mytriton_b200.ssa import SSAPrinter
from oracle import ssa_interp

HEADER = "import mytriton_b200 as triton\nimport mytriton_b200.language as tl\n\n\n"


class ExprGen:
    """Random expressions with a tracked element type ("i" or "f")."""

    def __init__(self, rng, float_leaves, int_leaves, integers=True):
        self.rng = rng
        self.float_leaves = float_leaves
        self.int_leaves = int_leaves
        self.integers = integers        # False: float-typed subtrees only

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
                operator = ["/", "//", "%"][int(self.rng.integers(3))]        # C division and remainder
                return f"({lhs} {operator} {int(self.rng.choice([-3, 2, 3, 5]))})"
            return f"tl.where({self.cond(depth - 1)}, {lhs}, {rhs})"
        mixed = self.rng.random() >= 0.6 and self.integers
        kinds = ("f", "i") if mixed else ("f", "f")                             # mixed promotes to f32
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
            inner = self.expr(depth - 1, 'f')
            # sin's argument is clamped: the device fuses a*b+c into one rounding, and an argument
            # in the thousands would turn that half-ulp difference into a visible phase error
            function = ["-", "tl.abs", "tl.tanh", "tl.sin(tl.minimum(8.0, tl.maximum(-8.0, ", "tl.sqrt(tl.abs",
                        "tl.log(1.0 + tl.abs"][int(self.rng.integers(6))]
            return f"({function}({inner}){')' * function.count('(')})"
        return f"tl.where({self.cond(depth - 1)}, {lhs}, {rhs})"

    def cond(self, depth):
        kind = "f" if self.rng.random() < 0.5 or not self.integers else "i"
        first = f"({self.expr(depth, kind)} < {self.expr(depth, kind)})"
        if self.rng.random() < 0.3 and self.integers:
            return f"({first} & ({self.expr(depth, 'i')} < {self.expr(depth, 'i')}))"
        return first


def rank1_kernel(rng, name):
    gen = ExprGen(rng, ["a", "b", "s"], ["offs", "n", "lanes"])
    result_kind = "f" if rng.random() < 0.8 else "i"
    result = gen.expr(3, result_kind)
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
    ]
    if rng.random() < 0.25:                      # some programs leave early
        lines.insert(5, f"    if pid > {int(rng.integers(0, 3))}:\n        return")
    if rng.random() < 0.4:                       # run-time if/else on program-uniform scalars
        kind = "f" if result_kind == "f" or rng.random() < 0.5 else "i"
        condition = ["pid < 1", "s < 0.25", "not (n < 40)", "(pid < 2) & (s < 0.0)"][int(rng.integers(4))]
        lines += [f"    if {condition}:", f"        r = {result}", "    else:",
                  f"        r = {gen.expr(2, kind)}"]
    else:
        lines += [f"    r = {result}"]
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
    ]
    if rng.random() < 0.5:        # a reduction along the tile's rows, broadcast back over the tile
        reduce = ["tl.sum", "tl.max", "tl.min"][int(rng.integers(3))]
        lines += [f"    row_stat = {reduce}(tl.where(mask, {gen.expr(2, 'f')}, 0.0), axis=1)",
                  "    r = r + row_stat[:, None] * 0.001"]
    lines += ["    tl.store(out + offs_m * N + offs_n, r, mask=mask)"]
    return "\n".join(lines) + "\n\n\n"


def loop_kernel(rng, name):
    """A run-time loop over row chunks with a carried block and a carried counter, an
    optional run-time if in the body, then a reduction broadcast back over the block."""
    gen = ExprGen(rng, ["a", "b", "acc", "s"], ["cols", "count", "n_cols"])
    update = gen.expr(2, "f")
    lines = [
        "@triton.jit",
        f"def {name}(x0, x1, out, n_cols, s, BLOCK: tl.constexpr):",
        "    row = tl.program_id(0)",
        "    lanes = tl.arange(0, BLOCK)",
        f"    acc = tl.full((BLOCK,), {float(np.round(rng.uniform(-1, 1), 2))}, tl.float32)",
        "    count = 0",
        "    for start in range(0, n_cols, BLOCK):" if rng.random() < 0.6 else
        "    start = 0 - BLOCK\n    while start + BLOCK < n_cols:\n        start = start + BLOCK",
        "        cols = start + lanes",
        "        live = cols < n_cols",
        "        a = tl.load(x0 + row * n_cols + cols, mask=live, other=0.0)",
        "        b = tl.load(x1 + cols, mask=live, other=1.0)",
    ]
    if rng.random() < 0.5:
        lines += [f"        if {['count < 1', 'row < 2', 's < 0.0'][int(rng.integers(3))]}:",
                  f"            acc = tl.where(live, tl.minimum(tl.maximum({update}, -50.0), 50.0), acc)",
                  "        else:",
                  f"            acc = tl.where(live, tl.minimum(tl.maximum({gen.expr(2, 'f')}, -50.0), 50.0), acc)"]
    else:
        lines += [f"        acc = tl.where(live, tl.minimum(tl.maximum({update}, -50.0), 50.0), acc)"]
    lines += [
        "        count = count + 1",
        f"    total = {['tl.sum', 'tl.max', 'tl.min'][int(rng.integers(3))]}(acc)",
        "    tl.store(out + row * BLOCK + lanes, acc + total * 0.001 + count)",
    ]
    return "\n".join(lines) + "\n\n\n"


def load_module(tmp_path, name, source):
    path = tmp_path / f"{name}.py"
    path.write_text(HEADER + source)
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def compare(got, want, label, source, tolerance=1e-5, global_scale=False):
    nan_got, nan_want = np.isnan(got), np.isnan(want)
    assert np.array_equal(nan_got, nan_want), f"{label}: NaN pattern differs\n{source}"
    finite = ~nan_got
    atol = tolerance
    if global_scale and finite.any():        # index factors amplify the accumulator's rounding
        atol = tolerance * max(1.0, float(np.abs(want[finite & np.isfinite(want)]).max(initial=1.0)))
    ok = np.isclose(got[finite], want[finite], rtol=tolerance, atol=atol) | (got[finite] == want[finite])
    assert ok.all(), (f"{label}: {int((~ok).sum())} of {ok.size} elements differ, worst "
                      f"{np.abs(got[finite] - want[finite])[~ok].max()}\n{source}")


def rank1_case(seed, tmp_path):
    """(kernel, source, grid, host arrays by parameter name, launch keywords)."""
    rng = np.random.default_rng(1000 + seed)
    name = f"fuzz1_{seed}"
    source, reduce = rank1_kernel(rng, name)
    kernel = getattr(load_module(tmp_path, name, source), name)
    block = int(rng.choice([16, 64, 256, 1024]))
    n = int(rng.integers(block // 2 + 1, 3 * block + 7))
    grid = (-(-n // block),)
    arrays = {"x0": rng.standard_normal(n, dtype=np.float32),
              "x1": rng.standard_normal(n, dtype=np.float32) * 2,
              "out": np.full(grid[0] if reduce else n, 7.0, dtype=np.float32)}
    scalars = {"n": n, "s": float(np.float32(rng.uniform(-1.5, 1.5)))}
    options = dict(BLOCK=block, **[{}, {"num_warps": 1}, {"elems_per_thread": 2}][seed % 3])
    return kernel, source, grid, arrays, scalars, options


def rank2_case(seed, tmp_path):
    rng = np.random.default_rng(5000 + seed)
    name = f"fuzz2_{seed}"
    source = rank2_kernel(rng, name)
    kernel = getattr(load_module(tmp_path, name, source), name)
    bm, bn = [(4, 8), (16, 32), (8, 64), (6, 10), (32, 32), (1, 128)][seed % 6]
    m, n = int(rng.integers(1, 3 * bm)), int(rng.integers(1, 3 * bn))
    grid = (-(-m // bm), -(-n // bn))
    arrays = {"x0": rng.standard_normal((m, n), dtype=np.float32),
              "x1": rng.standard_normal(m + n, dtype=np.float32),
              "out": np.full((m, n), 7.0, dtype=np.float32)}
    scalars = {"M": m, "N": n, "s": float(np.float32(rng.uniform(-1.5, 1.5)))}
    return kernel, source, grid, arrays, scalars, dict(BM=bm, BN=bn)


def loop_case(seed, tmp_path):
    rng = np.random.default_rng(9000 + seed)
    name = f"fuzz3_{seed}"
    source = loop_kernel(rng, name)
    kernel = getattr(load_module(tmp_path, name, source), name)
    block = int(rng.choice([32, 128, 512, 2048]))
    rows, n_cols = int(rng.integers(1, 6)), int(rng.integers(1, 4 * block))
    arrays = {"x0": rng.standard_normal((rows, n_cols), dtype=np.float32),
              "x1": rng.standard_normal(n_cols, dtype=np.float32),
              "out": np.full((rows, block), 7.0, dtype=np.float32)}
    scalars = {"n_cols": n_cols, "s": float(np.float32(rng.uniform(-1.5, 1.5)))}
    return kernel, source, (rows,), arrays, scalars, dict(BLOCK=block)


SCALE = int(os.environ.get("MYTRITON_FUZZ_SCALE", "1"))      # more seeds for a longer soak
CASES = ([(rank1_case, seed) for seed in range(24 * SCALE)] + [(rank2_case, seed) for seed in range(12 * SCALE)]
         + [(loop_case, seed) for seed in range(16 * SCALE)])
IDS = [f"{make.__name__}-{seed}" for make, seed in CASES]


def call_arguments(kernel, arrays, scalars):
    return [arrays.get(name, scalars.get(name)) for name in kernel.signature.parameters
            if name in arrays or name in scalars]


@pytest.mark.gpu
@pytest.mark.parametrize("make,seed", CASES, ids=IDS)
def test_random_kernels_match_the_oracle(make, seed, tmp_path, gpu):
    kernel, source, grid, arrays, scalars, options = make(seed, tmp_path)
    on_device = {name: device.to_device(array) for name, array in arrays.items()}
    _, ssa_ops, _ = kernel[grid](*call_arguments(kernel, on_device, scalars), **options)
    runtime.synchronize()
    expected = {name: array.copy() for name, array in arrays.items()}
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {**expected, **scalars}, grid)
    compare(on_device["out"].to_host(), expected["out"], kernel.fn.__name__, source,
            tolerance=1e-4 if make is loop_case else 1e-5)      # rounding differences compound over a loop


@pytest.mark.gpu
@pytest.mark.parametrize("make,seed", CASES[::3], ids=IDS[::3])
def test_random_kernels_in_the_other_code_generation_modes(make, seed, tmp_path, gpu):
    """Every third random kernel twice more: with the loop-aware passes off (the code generator
    gets the reference's SSA), and in bounds-check mode (element-by-element accesses behind
    guards).  Both must give what the interpreter gives, and a correct kernel on correctly
    sized arrays must not trip a single guard."""
    from mytriton_b200 import bounds

    kernel, source, grid, arrays, scalars, options = make(seed, tmp_path)
    _, ssa_ops, _ = kernel[grid](*call_arguments(kernel, arrays, scalars), **options)
    expected = {name: array.copy() for name, array in arrays.items()}
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {**expected, **scalars}, grid)
    bounds.check()
    for extra in ({"loop_passes": False}, {"bounds_check": True}):
        mode_options = {key: value for key, value in options.items() if key != "online_softmax" or "bounds_check" not in extra}
        on_device = {name: device.to_device(array) for name, array in arrays.items()}
        kernel[grid](*call_arguments(kernel, on_device, scalars), **mode_options, **extra)
        runtime.synchronize()
        bounds.check(kernel=kernel)
        compare(on_device["out"].to_host(), expected["out"], f"{kernel.fn.__name__} {extra}", source,
                tolerance=1e-4 if make is loop_case else 1e-5)


@pytest.mark.parametrize("make,seed", CASES, ids=IDS)
def test_random_kernels_compile_for_sm_100a(make, seed, tmp_path, runtime_lib):
    """Host only: every generated source gets through NVRTC (no launch)."""
    kernel, source, grid, arrays, scalars, options = make(seed, tmp_path)
    _, _, cuda_src = kernel[grid](*call_arguments(kernel, arrays, scalars), **options)
    runtime_lib.Module(cuda_src, kernel.fn.__name__, NVRTC_OPTIONS)


def dot_epilogue_kernel(rng, name, b_transposed=False, a_transposed=False, b_through_trans=False):
    """The tl.dot K-loop followed by a random elementwise epilogue over the accumulator, a
    column vector, a row vector, a scalar and the element's row and column indices:
    everything the tcgen05 generator fuses.  B is read from a [K, N] array or from its transpose."""
    gen = ExprGen(rng, ["acc", "bias_row", "scale_col", "s"], ["rows", "cols", "M"])
    b_index = "offs_n[None, :] * K + offs_k[:, None]" if b_transposed else "offs_k[:, None] * N + offs_n[None, :]"
    a_index = "offs_k[None, :] * M + offs_m[:, None]" if a_transposed else "offs_m[:, None] * K + offs_k[None, :]"
    lines = [
        "@triton.jit",
        f"def {name}(a, b, bias, scale, c, M, N, K, s, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):",
        "    offs_m = tl.program_id(0) * BM + tl.arange(0, BM)",
        "    offs_n = tl.program_id(1) * BN + tl.arange(0, BN)",
        "    acc = tl.zeros((BM, BN), tl.float32)",
        "    for k0 in range(0, K, BK):",
        "        offs_k = k0 + tl.arange(0, BK)",
        f"        a_tile = tl.load(a + {a_index},",
        "                         mask=(offs_m[:, None] < M) & (offs_k[None, :] < K), other=0.0)",
        *(["        b_tile = tl.trans(tl.load(b + offs_n[:, None] * K + offs_k[None, :],",
           "                                  mask=(offs_n[:, None] < N) & (offs_k[None, :] < K), other=0.0))"]
          if b_through_trans else
          [f"        b_tile = tl.load(b + {b_index},",
           "                         mask=(offs_k[:, None] < K) & (offs_n[None, :] < N), other=0.0)"]),
        "        acc = tl.dot(a_tile, b_tile, acc)",
        "    bias_row = tl.load(bias + offs_n, mask=offs_n < N, other=0.0)[None, :]",
        "    scale_col = tl.load(scale + offs_m, mask=offs_m < M, other=0.0)[:, None]",
        "    rows = offs_m[:, None]",
        "    cols = offs_n[None, :]",
        f"    y = acc + ({gen.expr(3, 'f')})",
        "    tl.store(c + offs_m[:, None] * N + offs_n[None, :], y,",
        "             mask=(offs_m[:, None] < M) & (offs_n[None, :] < N))",
    ]
    return "\n".join(lines) + "\n\n\n"


def dot_case(seed, tmp_path):
    from oracle import numpy_oracle as no

    rng = np.random.default_rng(7000 + seed)
    name = f"fuzz4_{seed}"
    b_transposed = seed % 3 == 2            # every third case reads B from an [N, K] array
    a_transposed = seed % 5 == 3            # every fifth reads A from a [K, M] array
    b_through_trans = seed % 7 == 5         # every seventh loads a [BN, BK] tile of an [N, K] array and transposes it
    b_transposed = b_transposed or b_through_trans
    source = dot_epilogue_kernel(rng, name, b_transposed, a_transposed, b_through_trans)
    kernel = getattr(load_module(tmp_path, name, source), name)
    bn = int(rng.choice([64, 128, 256]))
    bm, bk = [(128, 64), (128, 64), (64, 32), (192, 64), (256, 128)][int(rng.integers(5))]   # some need retiling
    m, n, k = int(rng.integers(1, 300)), int(rng.integers(1, 40)) * 8, int(rng.integers(1, 30)) * 8
    if a_transposed:
        m = -(-m // 8) * 8                  # rows of a [K, M] bf16 array must be whole 16-byte units for TMA
    a = no.round_to_bf16(rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k)))
    b = no.round_to_bf16(rng.standard_normal((k, n), dtype=np.float32))
    if b_transposed:
        b = np.ascontiguousarray(b.T)
    if a_transposed:
        a = np.ascontiguousarray(a.T)
    host = {"a": a, "b": b, "bias": rng.standard_normal(n, dtype=np.float32),
            "scale": rng.standard_normal(m, dtype=np.float32), "c": np.full((m, n), 7.0, np.float32)}
    scalars = {"M": m, "N": n, "K": k, "s": float(np.float32(rng.uniform(-1.5, 1.5)))}
    return kernel, source, (-(-m // bm), -(-n // bn)), host, scalars, dict(BM=bm, BN=bn, BK=bk)


def dot_arguments(kernel, host, scalars):
    from oracle import numpy_oracle as no

    on_device = {name: (device.to_device(no.bf16_bits(array), "bfloat16") if name in ("a", "b")
                        else device.to_device(array)) for name, array in host.items()}
    return on_device, call_arguments(kernel, on_device, scalars)


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(10 * SCALE))
def test_random_dot_epilogues_match_the_oracle(seed, tmp_path, gpu):
    """The fused epilogue of the tensor-core GEMM against the interpreter's fp64 product plus
    the same elementwise SSA: within 1e-4 relative, or 1e-4 of the largest expected magnitude
    (the epilogue may multiply the accumulator's rounding error by an index)."""
    from mytriton_b200 import dot_codegen

    kernel, source, grid, host, scalars, options = dot_case(seed, tmp_path)
    on_device, arguments = dot_arguments(kernel, host, scalars)
    launcher = kernel.launcher(grid, *arguments, **options)
    assert launcher.artifact.plan.kind == "tcgen05", source
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    _, ssa_ops, _ = kernel[grid](*call_arguments(kernel, host_views(host), scalars), **options)
    expected = {name: array.copy() for name, array in host.items()}
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {**expected, **scalars}, grid)
    compare(on_device["c"].to_host(), expected["c"], kernel.fn.__name__, source, tolerance=1e-4,
            global_scale=True)


DOT_VARIANTS = [
    {"cta_group": 2, "tile_n": 256, "cta_rows": 128},      # CTA pairs, two accumulators
    {"cta_group": 2, "tile_n": 256, "cta_rows": 256},      # CTA pairs, 512-row tiles
    {"cta_group": 1, "tile_n": 256},
    {"cta_group": 1, "tile_n": 128, "split_k": 2},
    {"cta_group": 1, "tile_n": 64, "split_k": 3},
    {"cta_group": 1, "split_k": 4},
]


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(10 * SCALE))
def test_random_dot_epilogues_in_every_kernel_variant(seed, tmp_path, gpu):
    """The same random kernels with the kernel variant named explicitly (a launch left to itself
    picks one by the problem's size, and these problems are all small): CTA pairs on both tile
    heights, single CTAs, and units along K whose partial sums the second kernel adds before it
    applies the epilogue."""
    from mytriton_b200 import dot_codegen

    kernel, source, grid, host, scalars, options = dot_case(seed, tmp_path)
    if options["BM"] == 256:
        pytest.skip("a 256-row program tile is a CTA-pair tile of its own: no other variant applies")
    variant = DOT_VARIANTS[seed % len(DOT_VARIANTS)]
    on_device, arguments = dot_arguments(kernel, host, scalars)
    launcher = kernel.launcher(grid, *arguments, **options, **variant)
    notes = launcher.artifact.plan.notes
    assert launcher.artifact.plan.kind == "tcgen05", source
    assert notes["cta_group"] == variant["cta_group"] and notes["split_k"] == variant.get("split_k", 1)
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    _, ssa_ops, _ = kernel[grid](*call_arguments(kernel, host_views(host), scalars), **options)
    expected = {name: array.copy() for name, array in host.items()}
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {**expected, **scalars}, grid)
    compare(on_device["c"].to_host(), expected["c"], kernel.fn.__name__, source, tolerance=1e-4,
            global_scale=True)


def host_views(host):
    """NumPy arguments of the right dtypes for a compile-only call (bf16 for a and b)."""
    import ml_dtypes

    return {name: (array.astype(ml_dtypes.bfloat16) if name in ("a", "b") else array)
            for name, array in host.items()}


@pytest.mark.parametrize("seed", range(10 * SCALE))
def test_random_dot_epilogues_are_fused_and_compile(seed, tmp_path, runtime_lib):
    kernel, source, grid, host, scalars, options = dot_case(seed, tmp_path)
    artifact = kernel.launcher(grid, *call_arguments(kernel, host_views(host), scalars), **options).artifact
    assert artifact.plan.kind == "tcgen05", source
    runtime_lib.Module(artifact.src, kernel.fn.__name__, NVRTC_OPTIONS)


def test_generators_are_deterministic():
    first = [rank1_kernel(np.random.default_rng(1000 + s), "k")[0] for s in range(3)]
    again = [rank1_kernel(np.random.default_rng(1000 + s), "k")[0] for s in range(3)]
    assert first == again and len(set(itertools.chain(first))) == 3
