"""The tl.dot loop matcher (CPU): what lowers to the tcgen05 kernel and what does not."""

import ml_dtypes
import numpy as np
import pytest

from mytriton_b200 import kernels as corpus
import mytriton_b200 as triton
import mytriton_b200.language as tl
from mytriton_b200.cuda_utils import NVRTC_OPTIONS


def operands(m=512, n=512, k=512, dtype=ml_dtypes.bfloat16):
    return (np.zeros((m, k), dtype=dtype), np.zeros((k, n), dtype=dtype), np.zeros((m, n), np.float32))


def plan_of(kernel, grid, *args, **kwargs):
    return kernel.launcher(grid, *args, **kwargs).artifact


def test_plain_gemm_matches_and_both_variants_compile(runtime_lib):
    a, b, c = operands()
    # one CTA per 128-row tile; CTA pairs on 256-row tiles (two accumulators, six stages); CTA
    # pairs on 512-row tiles (the default: one accumulator filling TMEM, four stages)
    for group, rows, stages in ((1, None, 4), (2, 128, 6), (2, 256, 4), (2, None, 4)):
        extra = {} if rows is None else {"cta_rows": rows}
        art = plan_of(corpus.matmul_dot_kernel, (4, 2), a, b, c, 512, 512, 512,
                      BM=128, BN=256, BK=64, cta_group=group, **extra)
        assert art.plan.kind == "tcgen05" and art.plan.cluster == (group, 1, 1)
        assert art.plan.notes["stages"] == stages
        assert art.plan.notes["cta_rows"] == (rows or (128 if group == 1 else 256))
        assert art.plan.dynamic_smem <= 227 * 1024
        match = art.plan.notes["gemm"]
        assert (match.lda, match.ldb, match.ldc, match.k_extent) == ("p:K", "p:N", "p:N", "p:K")
        assert (match.axis_m, match.axis_n, match.m_extent, match.n_extent) == (0, 1, "p:M", "p:N")
        module = runtime_lib.Module(art.src, "matmul_dot_kernel", NVRTC_OPTIONS)
        assert "warning" not in module.log.lower(), module.log


def test_default_pairs_ctas_when_b_splits_in_64_column_boxes():
    a, b, c = operands()
    assert plan_of(corpus.matmul_dot_kernel, (4, 2), a, b, c, 512, 512, 512,
                   BM=128, BN=256, BK=64).plan.cluster == (2, 1, 1)
    assert plan_of(corpus.matmul_dot_kernel, (4, 8), a, b, c, 512, 512, 512,
                   BM=128, BN=64, BK=64).plan.cluster == (1, 1, 1)


def test_256_row_tiles_are_cta_pair_tiles(runtime_lib):
    a, b, c = operands()
    art = plan_of(corpus.matmul_dot_kernel, (2, 2), a, b, c, 512, 512, 512, BM=256, BN=256, BK=64)
    assert art.plan.kind == "tcgen05" and art.plan.cluster == (2, 1, 1) and "BM = 128" in art.src
    runtime_lib.Module(art.src, "matmul_dot_kernel", NVRTC_OPTIONS)
    with pytest.raises(TypeError, match="cta_group must be 2"):
        plan_of(corpus.matmul_dot_kernel, (2, 2), a, b, c, 512, 512, 512, BM=256, BN=256, BK=64, cta_group=1)
    retiled = plan_of(corpus.matmul_dot_kernel, (2, 8), a, b, c, 512, 512, 512, BM=256, BN=64, BK=64)
    assert retiled.plan.kind == "tcgen05"            # 64 columns cannot be split between two CTAs: default tiling
    assert (retiled.plan.notes["gemm"].bn, retiled.plan.notes["gemm"].program_tile) == (256, (256, 64))


def test_skinny_variant_compiles(runtime_lib):
    a = np.zeros((16, 512), dtype=ml_dtypes.bfloat16)
    b = np.zeros((512, 512), dtype=ml_dtypes.bfloat16)
    c = np.zeros((16, 512), np.float32)
    art = plan_of(corpus.matmul_dot_kernel, (1, 2), a, b, c, 16, 512, 512, BM=128, BN=256, BK=64, a_rows=16)
    match = art.plan.notes["gemm"]
    assert (match.bn, match.bk, match.program_tile) == (64, 256, (128, 256)) and art.plan.cluster == (1, 1, 1)
    assert "A_ROWS = 16;" in art.src and art.plan.dynamic_smem <= 227 * 1024
    runtime_lib.Module(art.src, "matmul_dot_kernel", NVRTC_OPTIONS)
    with pytest.raises(ValueError, match="a_rows"):
        plan_of(corpus.matmul_dot_kernel, (1, 2), a, b, c, 16, 512, 512, BM=128, BN=256, BK=64, a_rows=12)
    with pytest.raises(TypeError, match="single-CTA"):
        plan_of(corpus.matmul_dot_kernel, (1, 2), a, b, c, 16, 512, 512, BM=128, BN=256, BK=64, a_rows=16, cta_group=2)


def test_epilogue_is_fused(runtime_lib):
    a, b, c = operands()
    bias, scale = np.zeros(512, np.float32), np.zeros(512, np.float32)
    art = plan_of(corpus.matmul_bias_act_kernel, (4, 2), a, b, bias, scale, c, 512, 512, 512, 0.1,
                  BM=128, BN=256, BK=64)
    assert art.plan.kind == "tcgen05"
    text = " ".join(art.plan.notes["gemm"].epilogue)
    assert "bias[col]" in text and "row_scale[row]" in text and "slope" in text
    runtime_lib.Module(art.src, "matmul_bias_act_kernel", NVRTC_OPTIONS)


def test_index_dependent_epilogue_is_fused(runtime_lib):
    """Row and column indices of the element are available to the fused epilogue (a causal
    mask); the program ids cancel once tile-local coordinates become global ones."""
    a, b, c = operands()
    for group in (1, 2):
        art = plan_of(corpus.matmul_causal_kernel, (4, 2), a, b, c, 512, 512, 512, 3,
                      BM=128, BN=256, BK=64, cta_group=group)
        assert art.plan.kind == "tcgen05"
        text = " ".join(art.plan.notes["gemm"].epilogue)
        assert "row" in text and "col" in text and "shift" in text and "pid" not in text
        runtime_lib.Module(art.src, "matmul_causal_kernel", NVRTC_OPTIONS)


@triton.jit
def uniform_scalar_epilogue_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    """The epilogue adds integers that are the same for every element but no polynomial of the
    scalar arguments: a remainder, a quotient, a minimum."""
    offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
    offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        offs_k = k0 + tl.arange(0, BK)
        acc += tl.dot(tl.load(a + offs_m[:, None] * K + offs_k[None, :]),
                      tl.load(b + offs_k[:, None] * N + offs_n[None, :]))
    acc = acc + (M % -3) + (K // 7) * 0.5 + tl.minimum(M, N - 5)
    tl.store(c + offs_m[:, None] * N + offs_n[None, :], acc)


def test_uniform_scalars_in_the_epilogue_stay_on_the_tensor_cores(runtime_lib):
    """`M % 3`, `K // 7`, `min(M, N)` are opaque to the index algebra; in an epilogue they are
    rendered as C on the scalar arguments instead of pushing the kernel to the SIMT path."""
    a, b, c = operands()
    art = plan_of(uniform_scalar_epilogue_kernel, (4, 2), a, b, c, 512, 512, 512, BM=128, BN=256, BK=64)
    assert art.plan.kind == "tcgen05"
    text = " ".join(art.plan.notes["gemm"].epilogue)
    assert "% (-3)" in text and "/ (7)" in text and "min(" in text and "pid" not in text
    runtime_lib.Module(art.src, "uniform_scalar_epilogue_kernel", NVRTC_OPTIONS)


@triton.jit
def augmented_dot_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    """The other spelling of the K-loop: ``acc += tl.dot(a, b)`` and unmasked loads."""
    offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
    offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        offs_k = k0 + tl.arange(0, BK)
        acc += tl.dot(tl.load(a + offs_m[:, None] * K + offs_k[None, :]),
                      tl.load(b + offs_k[:, None] * N + offs_n[None, :]))
    tl.store(c + offs_m[:, None] * N + offs_n[None, :], acc)


def test_augmented_accumulation_spelling_matches(runtime_lib):
    a, b, c = operands()
    art = plan_of(augmented_dot_kernel, (4, 2), a, b, c, 512, 512, 512, BM=128, BN=256, BK=64)
    assert art.plan.kind == "tcgen05"
    match = art.plan.notes["gemm"]
    assert (match.m_extent, match.n_extent, match.k_extent) == (None, None, "p:K")   # no masks: the grid bounds C
    runtime_lib.Module(art.src, "augmented_dot_kernel", NVRTC_OPTIONS)


def test_pointer_bumping_loop_matches(runtime_lib):
    """Carried pointer blocks advanced by BK and BK*N are induction values; `cols < K - k0`
    is the same bound as `k0 + cols < K`."""
    a, b, c = operands()
    art = plan_of(corpus.matmul_pointer_bump_kernel, (4, 2), a, b, c, 512, 512, 512, BM=128, BN=256, BK=64)
    assert art.plan.kind == "tcgen05"
    match = art.plan.notes["gemm"]
    assert (match.lda, match.ldb, match.ldc, match.k_extent) == ("p:K", "p:N", "p:N", "p:K")
    assert (match.m_extent, match.n_extent) == ("p:M", "p:N")
    runtime_lib.Module(art.src, "matmul_pointer_bump_kernel", NVRTC_OPTIONS)
    small = plan_of(corpus.matmul_pointer_bump_kernel, (32, 32), a, b, c, 512, 512, 512, BM=16, BN=16, BK=16)
    assert small.plan.kind == "simt"                     # carried pointers as i32 offsets in registers
    runtime_lib.Module(small.src, "matmul_pointer_bump_kernel", NVRTC_OPTIONS)


def test_pointer_bumping_loop_in_the_oracle():
    """The interpreter carries pointer blocks through the loop like any other value."""
    from mytriton_b200.ssa import SSAPrinter
    from oracle import ssa_interp

    rng = np.random.default_rng(0)
    m, n, k = 19, 23, 21
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    c = np.zeros((m, n), np.float32)
    _, ssa_ops, _ = corpus.matmul_pointer_bump_kernel[(2, 2)](a, b, c, m, n, k, BM=16, BN=16, BK=8)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"a": a, "b": b, "c": c, "M": m, "N": n, "K": k}, (2, 2))
    assert np.array_equal(c, a @ b)


def test_fp16_operands_select_the_fp16_instruction_format(runtime_lib):
    a, b, c = operands(dtype=np.float16)
    art = plan_of(corpus.matmul_dot_kernel, (4, 2), a, b, c, 512, 512, 512, BM=128, BN=256, BK=64)
    assert art.plan.kind == "tcgen05" and art.plan.notes["gemm"].operand == "f16"
    assert "AB_FORMAT = 0u" in art.src
    bf = plan_of(corpus.matmul_dot_kernel, (4, 2), *operands(), 512, 512, 512, BM=128, BN=256, BK=64)
    assert "AB_FORMAT = 1u" in bf.src
    mixed = (np.zeros((512, 512), np.float16), np.zeros((512, 512), ml_dtypes.bfloat16), c)
    with pytest.raises(TypeError, match="share one element type"):
        plan_of(corpus.matmul_dot_kernel, (4, 2), *mixed, 512, 512, 512, BM=128, BN=256, BK=64)


def test_fp8_operands_use_the_f8f6f4_kind(runtime_lib):
    a, b, c = operands(dtype=ml_dtypes.float8_e4m3fn)
    for group, bn in ((1, 128), (1, 256), (2, 256)):
        art = plan_of(corpus.matmul_dot_kernel, (4, 512 // bn), a, b, c, 512, 512, 512,
                      BM=128, BN=bn, BK=128, cta_group=group)
        assert art.plan.kind == "tcgen05" and art.plan.notes["gemm"].operand == "f8e4m3"
        assert 'MTB_MMA_KIND "f8f6f4"' in art.src and "EB = 1;" in art.src and "unsigned char* a" in art.src
        assert art.plan.dynamic_smem <= 227 * 1024
        module = runtime_lib.Module(art.src, "matmul_dot_kernel", NVRTC_OPTIONS)
        assert "warning" not in module.log.lower(), module.log
    assert plan_of(corpus.matmul_dot_kernel, (4, 4), a, b, c, 512, 512, 512,
                   BM=128, BN=128, BK=128).plan.cluster == (1, 1, 1)       # one 128-byte box per CTA: no pairing
    shallow = plan_of(corpus.matmul_dot_kernel, (4, 2), a, b, c, 512, 512, 512, BM=128, BN=256, BK=64)
    assert shallow.plan.kind == "tcgen05" and shallow.plan.notes["gemm"].bk == 128   # BK below one swizzle row: retiled
    small = plan_of(corpus.matmul_dot_kernel, (32, 32), a, b, c, 512, 512, 512, BM=16, BN=16, BK=16)
    assert small.plan.kind == "simt" and "mtb_e4m3_to_f32" in small.src
    runtime_lib.Module(small.src, "matmul_dot_kernel", NVRTC_OPTIONS)
    a5, b5, _ = operands(dtype=ml_dtypes.float8_e5m2)
    art = plan_of(corpus.matmul_dot_kernel, (4, 2), a5, b5, c, 512, 512, 512, BM=128, BN=256, BK=128)
    assert art.plan.notes["gemm"].operand == "f8e5m2" and "AB_FORMAT = 1u" in art.src and 'MTB_MMA_KIND "f8f6f4"' in art.src
    runtime_lib.Module(art.src, "matmul_dot_kernel", NVRTC_OPTIONS)
    small5 = plan_of(corpus.matmul_dot_kernel, (32, 32), a5, b5, c, 512, 512, 512, BM=16, BN=16, BK=16)
    assert "mtb_e5m2_to_f32" in small5.src
    runtime_lib.Module(small5.src, "matmul_dot_kernel", NVRTC_OPTIONS)


def test_tf32_is_opt_in_for_fp32_operands(runtime_lib):
    a, b, c = operands(dtype=np.float32)
    exact = plan_of(corpus.matmul_dot_kernel, (4, 2), a, b, c, 512, 512, 512, BM=128, BN=256, BK=32)
    assert exact.plan.kind == "simt"                    # no silent rounding of fp32 operands
    for group in (1, 2):
        art = plan_of(corpus.matmul_tf32_kernel, (4, 2), a, b, c, 512, 512, 512,
                      BM=128, BN=256, BK=32, cta_group=group)
        assert art.plan.kind == "tcgen05" and art.plan.notes["gemm"].operand == "tf32"
        assert 'MTB_MMA_KIND "tf32"' in art.src and "AB_FORMAT = 2u" in art.src and "EB = 4;" in art.src
        assert art.plan.dynamic_smem <= 227 * 1024
        module = runtime_lib.Module(art.src, "matmul_tf32_kernel", NVRTC_OPTIONS)
        assert "warning" not in module.log.lower(), module.log
    _, ssa_ops, _ = corpus.matmul_tf32_kernel[(4, 2)](a, b, c, 512, 512, 512, BM=128, BN=256, BK=32)
    from mytriton_b200.ssa import SSAPrinter
    assert "input_precision" in SSAPrinter().print_ops(ssa_ops)
    with pytest.raises(ValueError, match="input_precision"):
        tl.dot(None, None, None, input_precision="fp8")


def test_program_tiles_the_generator_lacks_are_recomputed_in_the_default_tiling(runtime_lib):
    """The loop is proven to be a dense GEMM over the launched grid, so the programs' tile
    shape only says which part of C is covered; the kernel tiles that part its own way."""
    a, b, c = operands()
    for tile, grid in (((64, 64, 32), (8, 8)), ((64, 128, 64), (8, 4)), ((128, 96, 64), (4, 6)), ((192, 64, 48), (3, 8))):
        art = plan_of(corpus.matmul_dot_kernel, grid, a, b, c, 512, 512, 512, BM=tile[0], BN=tile[1], BK=tile[2])
        match = art.plan.notes["gemm"]
        assert art.plan.kind == "tcgen05", tile
        assert (match.bm, match.bn, match.bk, match.program_tile) == (128, 256, 64, tile[:2])
    runtime_lib.Module(art.src, "matmul_dot_kernel", NVRTC_OPTIONS)


def test_small_tiles_and_fp32_operands_take_the_simt_path():
    a, b, c = operands()
    assert plan_of(corpus.matmul_dot_kernel, (32, 32), a, b, c, 512, 512, 512,
                   BM=16, BN=16, BK=16).plan.kind == "simt"
    a32, b32, c32 = operands(dtype=np.float32)
    assert plan_of(corpus.matmul_dot_kernel, (32, 32), a32, b32, c32, 512, 512, 512,
                   BM=16, BN=16, BK=16).plan.kind == "simt"


@triton.jit
def strided_store_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    """Same loop, but C is written to every other row of a [2M, N] array: its row stride is no
    single parameter, so this is not the dense tile the tensor-core kernel stores."""
    pid_m = tl.program_id(0)
    pid_n = tl.program_id(1)
    offs_m = pid_m * BM + tl.arange(0, BM)
    offs_n = pid_n * BN + tl.arange(0, BN)
    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        offs_k = k0 + tl.arange(0, BK)
        a_tile = tl.load(a + offs_m[:, None] * K + offs_k[None, :])
        b_tile = tl.load(b + offs_k[:, None] * N + offs_n[None, :])
        acc = tl.dot(a_tile, b_tile, acc)
    tl.store(c + offs_m[:, None] * (N + N) + offs_n[None, :], acc)


def test_anything_but_the_dense_tile_form_is_not_matched(runtime_lib):
    a, b, c = operands()
    # a large tile that does not match still compiles: the SIMT path stages it in dynamic shared memory
    big = plan_of(strided_store_kernel, (4, 2), a, b, c, 512, 512, 512, BM=128, BN=256, BK=64)
    assert big.plan.kind == "simt" and big.plan.dynamic_smem == (128 * 64 + 64 * 256) * 4
    assert "extern __shared__ float mtb_dot_staging[];" in big.src
    runtime_lib.Module(big.src, "strided_store_kernel", NVRTC_OPTIONS)
    with pytest.raises(TypeError, match="200 KiB"):
        plan_of(strided_store_kernel, (4, 2), a, b, c, 512, 512, 512, BM=128, BN=256, BK=256)
    assert plan_of(strided_store_kernel, (32, 32), a, b, c, 512, 512, 512,
                   BM=16, BN=16, BK=16).plan.kind == "simt"


def test_bounded_wait_probe_kernel_compiles_against_the_prelude(runtime_lib):
    """The kernel the GPU status test launches is built from the GEMM prelude alone."""
    import test_status_gpu
    from mytriton_b200 import dot_codegen

    src = "#define MTB_WAIT_LIMIT 200000ll\n" + dot_codegen._PRELUDE + test_status_gpu.KERNEL
    runtime_lib.Module(src, "starved_wait", NVRTC_OPTIONS)


# ---------------------------------------------------------------- tile maps, guards, transposed C


def test_one_axis_launch_with_grouped_ordering_matches(runtime_lib):
    """`pid // n`, `pid % n` and `min(...)` are program-uniform scalars the matcher keeps as opaque
    symbols; whether the programs of a given grid visit every tile once is checked per launch."""
    from mytriton_b200 import dot_codegen

    a, b, c = operands(1024, 768, 256)
    art = plan_of(corpus.matmul_grouped_kernel, (24,), a, b, c, 1024, 768, 256, BM=128, BN=256, BK=64, GROUP_M=3)
    assert art.plan.kind == "tcgen05"
    match = art.plan.notes["gemm"]
    assert match.tile_map is not None and not match.tile_map.guards and not match.c_transposed
    assert {code for _, (code, _, _) in match.tile_map.opaque} == {"div", "rem", "minimum"}
    runtime_lib.Module(art.src, "matmul_grouped_kernel", NVRTC_OPTIONS)
    names = ["a", "b", "c", "M", "N", "K"]
    args = (a, b, c, 1024, 768, 256)
    assert dot_codegen.launch_tiles(match, (24,), args, names) == (8, 3)
    assert dot_codegen.launch_obstacle(art.plan, (24,), args, names) is None or "aligned" in \
        dot_codegen.launch_obstacle(art.plan, (24,), args, names)
    # too few programs: some tile is never visited; too many: a program divides by zero
    for grid, reason in (((23,), "every tile of a rectangle"), ((25,), "every tile of a rectangle|divides by zero")):
        with pytest.raises(dot_codegen.GemmLaunchError, match=reason):
            dot_codegen.launch_tiles(match, grid, args, names)
    # ragged M: 1000 rows are still 8 tile rows
    assert dot_codegen.launch_tiles(match, (24,), (a, b, c, 1000, 768, 256), names) == (8, 3)


def test_the_program_to_tile_check_follows_c_arithmetic():
    from mytriton_b200.dot_codegen import Bound, Poly, TileMap, _evaluate_tile_map, GemmLaunchError

    pid, n = Poly.sym("pid0"), Poly.sym("p:n")
    opaque = (("s:0", ("div", pid, n)), ("s:1", ("rem", pid, n)))
    plain = TileMap(Poly.sym("s:0"), Poly.sym("s:1"), (), opaque)
    assert _evaluate_tile_map(plain, (12, 1, 1), {"n": 4}) == (3, 4)
    with pytest.raises(GemmLaunchError, match="every tile of a rectangle"):
        _evaluate_tile_map(plain, (11, 1, 1), {"n": 4})
    with pytest.raises(GemmLaunchError, match="divides by zero"):
        _evaluate_tile_map(plain, (12, 1, 1), {"n": 0})
    # a guard `row tile < 2` (written as difference < 0) drops the programs of the third row
    guarded = TileMap(Poly.sym("s:0"), Poly.sym("s:1"), (Bound(Poly.sym("s:0") - Poly.const(2), Poly()),), opaque)
    assert _evaluate_tile_map(guarded, (12, 1, 1), {"n": 4}) == (2, 4)
    # two programs on the same tile
    doubled = TileMap(Poly.sym("s:0"), Poly.const(0), (), opaque)
    with pytest.raises(GemmLaunchError):
        _evaluate_tile_map(doubled, (12, 1, 1), {"n": 4})


def test_early_return_and_transposed_store_match(runtime_lib):
    from mytriton_b200 import dot_codegen

    a, b, _ = operands(512, 512, 256)
    ct = np.zeros((512, 512), np.float32)
    art = plan_of(corpus.matmul_guarded_transposed_kernel, (10,), a, b, ct, 512, 512, 256, BM=128, BN=256, BK=64)
    assert art.plan.kind == "tcgen05"
    match = art.plan.notes["gemm"]
    assert match.c_transposed and match.ldc == "p:M" and len(match.tile_map.guards) == 1
    assert "C_TRANSPOSED = true" in art.src
    runtime_lib.Module(art.src, "matmul_guarded_transposed_kernel", NVRTC_OPTIONS)
    names = ["a", "b", "ct", "M", "N", "K"]
    # ten programs for eight tiles: the two past the last tile row return early
    assert dot_codegen.launch_tiles(match, (10,), (a, b, ct, 512, 512, 256), names) == (4, 2)
    # a bf16 transposed C stays on the SIMT path
    c16 = np.zeros((512, 512), ml_dtypes.bfloat16)
    assert plan_of(corpus.matmul_guarded_transposed_kernel, (8,), a, b, c16, 512, 512, 256,
                   BM=128, BN=256, BK=64).plan.kind == "simt"


def test_a_guard_on_the_loads_alone_is_not_a_gemm():
    """If a program could skip its loads but still store, the stored tile would not be the product."""

    @triton.jit
    def kernel(a, b, c, M, N, K, flag, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        rows = tl.program_id(0) * BM + tl.arange(0, BM)
        cols = tl.program_id(1) * BN + tl.arange(0, BN)
        kk = tl.arange(0, BK)
        acc = tl.zeros((BM, BN), tl.float32)
        live = tl.program_id(0) < flag
        for k0 in range(0, K, BK):
            x = tl.load(a + rows[:, None] * K + (k0 + kk)[None, :], mask=(rows[:, None] < M) & live, other=0.0)
            y = tl.load(b + (k0 + kk)[:, None] * N + cols[None, :], mask=cols[None, :] < N, other=0.0)
            acc = tl.dot(x, y, acc)
        tl.store(c + rows[:, None] * N + cols[None, :], acc, mask=(rows[:, None] < M) & (cols[None, :] < N))

    a, b, c = operands()
    assert plan_of(kernel, (4, 2), a, b, c, 512, 512, 512, 3, BM=128, BN=256, BK=64).plan.kind == "simt"


def test_comparisons_with_or_equal():
    @triton.jit
    def kernel(x, out, n, BLOCK: tl.constexpr):
        offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
        v = tl.load(x + offs, mask=offs < n, other=0.0)
        tl.store(out + offs, tl.where((v >= 0.5) & (offs <= 7), v, 0.0), mask=offs < n)

    from oracle import ssa_interp
    from mytriton_b200.ssa import SSAPrinter

    x = np.array([0.5, 0.25, 1.0, -1.0, 0.75, 0.5, 2.0, 3.0, 4.0, 0.6], np.float32)
    _, ssa_ops, _ = kernel[(1,)](x, np.zeros(10, np.float32), 10, BLOCK=16)
    out = np.zeros(10, np.float32)
    ssa_interp.run(SSAPrinter().print_ops(list(ssa_ops)), {"x": x.copy(), "out": out, "n": 10}, (1,))
    assert np.array_equal(out, np.where((x >= 0.5) & (np.arange(10) <= 7), x, 0.0).astype(np.float32))


def test_tile_height_follows_how_well_the_tiles_fill_the_rounds():
    """74 CTA pairs (a B200): the benchmark shapes and every shard of the sharded run keep the
    512-row tiles; launches of less than one round, or of a little more than a whole number of
    rounds, switch to 256-row tiles."""
    from mytriton_b200.dot_codegen import narrow_tiles_fill_better

    for rows in (8192, 16384, 32768, 65536, 2048, 1024):         # x 8192 columns: full rounds or equal fill
        assert not narrow_tiles_fill_better(rows, 8192, 256, 74), rows
    assert not narrow_tiles_fill_better(4096, 4096, 256, 74)      # 128 vs 256 tiles: both 86 % filled
    assert narrow_tiles_fill_better(4096, 8192, 256, 74)          # 256 tiles = 3.46 rounds vs 512 = 6.92
    assert narrow_tiles_fill_better(2048, 2048, 256, 74)          # 32 tiles for 74 pairs
    assert narrow_tiles_fill_better(512, 8192, 256, 74)
    assert narrow_tiles_fill_better(4000, 5000, 256, 74)          # 160 tiles = 2.16 rounds vs 320 = 4.3
    assert narrow_tiles_fill_better(256, 4096, 256, 74)           # half of every 512-row tile would be empty
    assert not narrow_tiles_fill_better(257, 4096 * 8, 256, 74)   # 128 tiles of 512 rows = 2 rounds; 256 of 256 rows = 4


def test_small_problems_choose_tile_width_and_split_k_by_the_launch_model():
    """148 SMs: sub-wave problems go to single CTAs (narrow tiles for a shallow K, several units
    along a deep K, never so many that a unit has fewer than four k-blocks); problems that fill the
    CTA pairs, or whose depth favours the pairs' shared operand, stay."""
    from mytriton_b200.dot_codegen import small_problem_variant as choose

    assert choose(1024, 1024, 1024, 64, 64, 148) == {"cta_group": 1, "tile_n": 64}
    assert choose(1024, 1024, 8192, 64, 64, 148) == {"cta_group": 1, "tile_n": 256, "split_k": 4}
    assert choose(1536, 1536, 4096, 64, 64, 148) == {"cta_group": 1, "tile_n": 256, "split_k": 2}
    assert choose(512, 512, 16384, 64, 64, 148)["split_k"] >= 8
    assert choose(2048, 2048, 512, 64, 64, 148) == {"cta_group": 1, "tile_n": 256}
    for filled in ((512, 8192, 8192), (4096, 4096, 4096), (8192, 8192, 8192), (3072, 2048, 1024), (4000, 5000, 3000)):
        assert choose(*filled, 64, 64, 148) is None, filled
    assert choose(128, 8192, 8192, 64, 64, 148) is None              # the skinny variant's business
    assert choose(1024, 1024, 1024, 128, 128, 148)["tile_n"] == 128  # fp8: 128 elements per 128-byte row
    picked = choose(300, 300, 520, 64, 64, 148)
    assert "split_k" not in picked or 520 // 64 // picked["split_k"] >= 4


def test_skinny_launches_choose_column_tiles_and_units_along_k():
    """At most 128 rows of C: 128-column tiles with enough units along K to fill 148 SMs (sixteen
    k-blocks per unit at least), 64-column tiles when K cannot be split and wider tiles would leave
    SMs idle."""
    from mytriton_b200.dot_codegen import skinny_options as choose

    assert choose(128, 8192, 8192, 64, 148) == {"a_rows": 128, "tile_n": 128, "split_k": 2}
    assert choose(128, 4096, 16384, 64, 148) == {"a_rows": 128, "tile_n": 128, "split_k": 4}
    assert choose(32, 16384, 4096, 64, 148) == {"a_rows": 32, "tile_n": 128}
    assert choose(16, 8192, 8192, 64, 148) == {"a_rows": 16}            # two units per tile would not pay
    assert choose(16, 1024, 8192, 64, 148) == {"a_rows": 16, "tile_n": 128, "split_k": 4}
    assert choose(128, 8192, 512, 64, 148) == {"a_rows": 128}          # too shallow to split: 128 narrow tiles
    assert choose(16, 64, 8192, 64, 148) == {"a_rows": 16}


def test_b_stored_as_its_transpose_is_the_k_major_operand(runtime_lib):
    """`bt + offs_n[None, :] * K + offs_k[:, None]` reads B from an [N, K] array: matched, flagged,
    and compiled with B as a K-major operand in every kernel variant."""
    a = np.zeros((512, 1024), ml_dtypes.bfloat16)
    bt = np.zeros((768, 1024), ml_dtypes.bfloat16)
    c = np.zeros((512, 768), np.float32)
    for options in ({}, {"cta_rows": 128}, {"cta_group": 1}, {"cta_group": 1, "tile_n": 64, "split_k": 2}, {"a_rows": 64}):
        art = plan_of(corpus.matmul_nt_kernel, (4, 3), a, bt, c, 512, 768, 1024, BM=128, BN=256, BK=64, **options)
        assert art.plan.kind == "tcgen05", options
        match = art.plan.notes["gemm"]
        assert match.b_transposed and (match.ldb, match.n_extent, match.k_extent) == ("p:K", "p:N", "p:K")
        assert "B_KMAJOR = true" in art.src
        runtime_lib.Module(art.src, "matmul_nt_kernel", NVRTC_OPTIONS)
    plain = plan_of(corpus.matmul_dot_kernel, (4, 3), a, np.zeros((1024, 768), ml_dtypes.bfloat16), c, 512, 768, 1024,
                    BM=128, BN=256, BK=64)
    assert not plain.plan.notes["gemm"].b_transposed and "B_KMAJOR = false" in plain.src


def test_a_stored_as_its_transpose_is_the_mn_major_operand(runtime_lib):
    """`at + offs_k[None, :] * M + offs_m[:, None]` reads A from a [K, M] array: matched, flagged,
    compiled with A as an MN-major operand, alone or together with a transposed B; the few-row
    (skinny) variant does not apply to it."""
    at = np.zeros((1024, 512), ml_dtypes.bfloat16)
    b = np.zeros((1024, 768), ml_dtypes.bfloat16)
    bt = np.zeros((768, 1024), ml_dtypes.bfloat16)
    c = np.zeros((512, 768), np.float32)
    for kernel, operands, both in ((corpus.matmul_tn_kernel, (at, b), False), (corpus.matmul_tt_kernel, (at, bt), True)):
        for options in ({}, {"cta_rows": 128}, {"cta_group": 1}, {"cta_group": 1, "tile_n": 64, "split_k": 2}):
            art = plan_of(kernel, (4, 3), *operands, c, 512, 768, 1024, BM=128, BN=256, BK=64, **options)
            assert art.plan.kind == "tcgen05", options
            match = art.plan.notes["gemm"]
            assert match.a_transposed and match.b_transposed == both and (match.lda, match.m_extent) == ("p:M", "p:M")
            assert "A_MMAJOR = true" in art.src and f"B_KMAJOR = {'true' if both else 'false'}" in art.src
            runtime_lib.Module(art.src, kernel.fn.__name__, NVRTC_OPTIONS)
    with pytest.raises(TypeError, match="transposed A"):
        plan_of(corpus.matmul_tn_kernel, (4, 3), at, b, c, 512, 768, 1024, BM=128, BN=256, BK=64, a_rows=64)


def test_stride_arguments_equal_to_one_select_the_layout(runtime_lib):
    """The usual matmul signature passes every stride.  Integer arguments equal to 1 are folded into
    the IR of kernels that use tl.dot (they stay in the parameter list), so one kernel source
    reaches the tensor cores for every storage layout; strides that leave no unit axis do not."""
    bf = ml_dtypes.bfloat16
    m, n, k = 512, 768, 1024
    a, at = np.zeros((m, k), bf), np.zeros((k, m), bf)
    b, bt = np.zeros((k, n), bf), np.zeros((n, k), bf)
    c, ct = np.zeros((m, n), np.float32), np.zeros((n, m), np.float32)
    cases = {
        "NN": ((a, b, c, k, 1, n, 1, n, 1), (False, False, False)),
        "NT": ((a, bt, c, k, 1, 1, k, n, 1), (False, True, False)),
        "TN": ((at, b, c, 1, m, n, 1, n, 1), (True, False, False)),
        "TT": ((at, bt, c, 1, m, 1, k, n, 1), (True, True, False)),
        "C transposed": ((a, b, ct, k, 1, n, 1, 1, m), (False, False, True)),
    }
    for name, ((x, y, z, *strides), want) in cases.items():
        art = plan_of(corpus.matmul_strided_kernel, (4, 3), x, y, z, m, n, k, *strides, BM=128, BN=256, BK=64)
        assert art.plan.kind == "tcgen05", name
        match = art.plan.notes["gemm"]
        assert (match.a_transposed, match.b_transposed, match.c_transposed) == want, name
        assert "int stride_ak" in art.src                      # folded arguments stay parameters
        runtime_lib.Module(art.src, "matmul_strided_kernel", NVRTC_OPTIONS)
    general = plan_of(corpus.matmul_strided_kernel, (4, 3), a, b, c, m, n, k, k, 2, n, 1, n, 1, BM=128, BN=256, BK=64)
    assert general.plan.kind == "simt"
    # kernels without tl.dot are traced as the reference traces them, whatever their arguments
    _, ssa_one, _ = corpus.row_sum_kernel[(1,)](np.zeros((1, 1), np.float32), np.zeros(1, np.float32), 1, BLOCK=16)
    _, ssa_two, _ = corpus.row_sum_kernel[(1,)](np.zeros((1, 2), np.float32), np.zeros(1, np.float32), 2, BLOCK=16)
    from mytriton_b200.ssa import SSAPrinter
    assert SSAPrinter().print_ops(ssa_one) == SSAPrinter().print_ops(ssa_two)


def test_the_tutorial_spelling_of_a_matmul_matches(runtime_lib):
    """A one-axis grid with grouped ordering, stride arguments, pointer blocks advanced in a loop over
    `range(0, cdiv(K, BK))`, masks against `K - k * BK`: the loop index counts k-blocks and is
    rewritten to the depth it stands for."""
    bf = ml_dtypes.bfloat16
    m, n, k = 512, 768, 1000
    a, at, b, bt = np.zeros((m, k), bf), np.zeros((k, m), bf), np.zeros((k, n), bf), np.zeros((n, k), bf)
    c = np.zeros((m, n), np.float32)
    for (x, y, sam, sak, sbk, sbn), want in (((a, b, k, 1, n, 1), (False, False)), ((a, bt, k, 1, 1, k), (False, True)),
                                             ((at, b, 1, m, n, 1), (True, False))):
        art = plan_of(corpus.matmul_tutorial_kernel, (12,), x, y, c, m, n, k, sam, sak, sbk, sbn, n, 1,
                      BM=128, BN=256, BK=64, GROUP_M=4)
        assert art.plan.kind == "tcgen05"
        match = art.plan.notes["gemm"]
        assert (match.a_transposed, match.b_transposed) == want
        assert (match.k_extent, match.bk, match.m_extent, match.n_extent) == ("p:K", 64, "p:M", "p:N")
        assert match.tile_map is not None
        runtime_lib.Module(art.src, "matmul_tutorial_kernel", NVRTC_OPTIONS)


@triton.jit
def block_index_misused_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    """Counts k-blocks but masks against `K - k` instead of `K - k * BK`: no dense K-loop."""
    offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
    offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
    offs_k = tl.arange(0, BK)
    a_ptrs = a + offs_m[:, None] * K + offs_k[None, :]
    b_ptrs = b + offs_k[:, None] * N + offs_n[None, :]
    acc = tl.zeros((BM, BN), tl.float32)
    for k in range(0, tl.cdiv(K, BK)):
        a_tile = tl.load(a_ptrs, mask=offs_k[None, :] < K - k, other=0.0)
        b_tile = tl.load(b_ptrs, mask=offs_k[:, None] < K - k, other=0.0)
        acc = tl.dot(a_tile, b_tile, acc)
        a_ptrs += BK
        b_ptrs += BK * N
    tl.store(c + offs_m[:, None] * N + offs_n[None, :], acc)


def test_a_block_index_used_as_a_depth_is_not_matched():
    a, b, c = operands()
    art = plan_of(block_index_misused_kernel, (4, 2), a, b, c, 512, 512, 512, BM=128, BN=256, BK=64)
    assert art.plan.kind == "simt"


@triton.jit
def modulo_without_store_mask_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    """Rows wrap around modulo M but the store is not masked by M: wrapped rows would be stored."""
    offs_m = (tl.program_id(0) * BM + tl.arange(0, BM)) % M
    offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        offs_k = k0 + tl.arange(0, BK)
        acc += tl.dot(tl.load(a + offs_m[:, None] * K + offs_k[None, :]),
                      tl.load(b + offs_k[:, None] * N + offs_n[None, :]))
    rows = tl.program_id(0) * BM + tl.arange(0, BM)
    tl.store(c + rows[:, None] * N + offs_n[None, :], acc)


def test_indices_taken_modulo_the_extent_stand_for_the_missing_mask(runtime_lib):
    """`offs_m % M` on the operands' indices keeps a ragged tile's addresses inside the array; the
    kernel is a dense GEMM exactly if the store is masked by the same M, which the matcher demands."""
    bf = ml_dtypes.bfloat16
    m, n, k = 500, 700, 1000
    a, b, c = np.zeros((m, k), bf), np.zeros((k, n), bf), np.zeros((m, n), np.float32)
    art = plan_of(corpus.matmul_tutorial_modulo_kernel, (12,), a, b, c, m, n, k, k, 1, n, 1, n, 1,
                  BM=128, BN=256, BK=64, GROUP_M=4)
    assert art.plan.kind == "tcgen05"
    match = art.plan.notes["gemm"]
    assert (match.m_extent, match.n_extent, match.k_extent) == ("p:M", "p:N", "p:K")
    runtime_lib.Module(art.src, "matmul_tutorial_modulo_kernel", NVRTC_OPTIONS)
    unmasked = plan_of(modulo_without_store_mask_kernel, (4, 2), *operands(), 512, 512, 512, BM=128, BN=256, BK=64)
    assert unmasked.plan.kind == "simt"


def test_a_transposed_tile_as_the_operand_of_a_dot_is_seen_through(runtime_lib):
    bf = ml_dtypes.bfloat16
    x, w, y = np.zeros((512, 1024), bf), np.zeros((768, 1024), bf), np.zeros((512, 768), np.float32)
    art = plan_of(corpus.linear_layer_kernel, (4, 3), x, w, y, 512, 768, 1024, BM=128, BN=256, BK=64)
    assert art.plan.kind == "tcgen05"
    match = art.plan.notes["gemm"]
    assert (match.a_transposed, match.b_transposed, match.ldb, match.n_extent, match.k_extent) == (
        False, True, "p:K", "p:N", "p:K")
    runtime_lib.Module(art.src, "linear_layer_kernel", NVRTC_OPTIONS)


@triton.jit
def remainder_in_epilogue_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
    offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        offs_k = k0 + tl.arange(0, BK)
        acc += tl.dot(tl.load(a + offs_m[:, None] * K + offs_k[None, :]),
                      tl.load(b + offs_k[:, None] * N + offs_n[None, :]))
    acc = acc + (offs_m[:, None] % 5) + (offs_n[None, :] % M)
    tl.store(c + offs_m[:, None] * N + offs_n[None, :], acc)


@triton.jit
def wrapped_index_in_epilogue_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    rows = tl.program_id(0) * BM + tl.arange(0, BM)
    wrapped = rows % M
    offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        offs_k = k0 + tl.arange(0, BK)
        acc += tl.dot(tl.load(a + wrapped[:, None] * K + offs_k[None, :]),
                      tl.load(b + offs_k[:, None] * N + offs_n[None, :]))
    acc = acc + wrapped[:, None]                         # here the remainder is data, not addressing
    tl.store(c + rows[:, None] * N + offs_n[None, :], acc, mask=rows[:, None] < M)


def test_a_remainder_is_addressing_only_where_it_addresses_the_operands(runtime_lib):
    """`rows % 5` in an epilogue is elementwise work and is rendered as such; an index read through
    `% M` that also feeds the epilogue cannot be taken for the index itself."""
    a, b, c = operands()
    art = plan_of(remainder_in_epilogue_kernel, (4, 2), a, b, c, 512, 512, 512, BM=128, BN=256, BK=64)
    assert art.plan.kind == "tcgen05"
    text = " ".join(art.plan.notes["gemm"].epilogue)
    assert "% 5" in text and "% (M)" in text.replace("% M", "% (M)")
    runtime_lib.Module(art.src, "remainder_in_epilogue_kernel", NVRTC_OPTIONS)
    mixed = plan_of(wrapped_index_in_epilogue_kernel, (4, 2), a, b, c, 512, 512, 512, BM=128, BN=256, BK=64)
    assert mixed.plan.kind == "simt"


@triton.jit
def residual_with_another_mask_kernel(a, b, residual, c, M, N, K, M2, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    rows = tl.program_id(0) * BM + tl.arange(0, BM)
    cols = tl.program_id(1) * BN + tl.arange(0, BN)
    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        ks = k0 + tl.arange(0, BK)
        acc += tl.dot(tl.load(a + rows[:, None] * K + ks[None, :]), tl.load(b + ks[:, None] * N + cols[None, :]))
    skip = tl.load(residual + rows[:, None] * N + cols[None, :], mask=rows[:, None] < M2, other=0.0)
    tl.store(c + rows[:, None] * N + cols[None, :], acc + skip, mask=(rows[:, None] < M) & (cols[None, :] < N))


def test_a_whole_tile_read_in_the_epilogue_is_fused(runtime_lib):
    """`acc * alpha + residual[rows, cols]`: the tile of the other matrix is read per element at the
    element's own position, guarded like the store; a mask by some other extent is not that guard."""
    bf = ml_dtypes.bfloat16
    a, b = np.zeros((512, 1024), bf), np.zeros((1024, 768), bf)
    residual, c = np.zeros((512, 768), np.float32), np.zeros((512, 768), np.float32)
    for options in ({}, {"cta_group": 1, "split_k": 2}):
        art = plan_of(corpus.matmul_residual_kernel, (4, 3), a, b, residual, c, 512, 768, 1024, 0.5,
                      BM=128, BN=256, BK=64, **options)
        assert art.plan.kind == "tcgen05"
        text = " ".join(art.plan.notes["gemm"].epilogue)
        assert "residual[(long long)row * (N) + col]" in text and "row < m_rows && col < n_cols" in text
        runtime_lib.Module(art.src, "matmul_residual_kernel", NVRTC_OPTIONS)
    other = plan_of(residual_with_another_mask_kernel, (4, 3), a, b, residual, c, 512, 768, 1024, 300,
                    BM=128, BN=256, BK=64)
    assert other.plan.kind == "simt"
