"""tl.dot on the GPU: the tcgen05 path and the SIMT fallback against the fp64
product of the bf16-rounded inputs.  The stated bar is 1e-2 relative Frobenius
error; fp32 accumulation lands several orders of magnitude inside it, so the
tests use 1e-5 and would catch a mis-addressed tile immediately."""

import numpy as np
import pytest

from mytriton_b200 import kernels as corpus
import mytriton_b200 as triton
import mytriton_b200.language as tl
from mytriton_b200 import device, dot_codegen, runtime
from oracle import numpy_oracle as no

pytestmark = pytest.mark.gpu
STATED_TOLERANCE = 1e-2
TEST_TOLERANCE = 1e-5


def run_dot(a, b, bm, bn, bk, **options):
    m, k = a.shape
    n = b.shape[1]
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)          # NaN canary
    grid = (-(-m // bm), -(-n // bn))
    launcher = corpus.matmul_dot_kernel.launcher(grid, da, db, dc, m, n, k, BM=bm, BN=bn, BK=bk, **options)
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    return dc.to_host(), launcher.artifact.plan.kind


def expected(a, b):
    return no.matmul_f64(no.round_to_bf16(a), no.round_to_bf16(b))


def test_single_tile_exact_integers(gpu):
    rng = np.random.default_rng(0)
    a = rng.integers(-3, 4, (128, 64)).astype(np.float32)
    b = rng.integers(-3, 4, (64, 256)).astype(np.float32)
    c, kind = run_dot(a, b, 128, 256, 64)
    assert kind == "tcgen05"
    assert np.array_equal(c, (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32))


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("shape", [(128, 256, 256), (256, 512, 512), (1024, 1024, 1024),
                                   (300, 520, 200), (129, 264, 72), (1000, 8, 64), (384, 256, 128)])
def test_tcgen05_shapes_including_ragged_edges(shape, cta_group, gpu):
    """Both kernel variants: one CTA per 128x256 tile, and CTA pairs on 256x256 tiles
    (an odd number of 128-row tiles leaves the pair's second CTA fully clipped)."""
    m, n, k = shape
    rng = np.random.default_rng(m * 7 + n)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32) / np.float32(np.sqrt(k))
    c, kind = run_dot(a, b, 128, 256, 64, cta_group=cta_group)
    assert kind == "tcgen05"
    assert no.relative_frobenius_error(c, expected(a, b)) < TEST_TOLERANCE < STATED_TOLERANCE


@pytest.mark.parametrize("tile", [(64, 64, 32), (64, 128, 64), (128, 96, 64), (192, 64, 48), (256, 64, 64)])
@pytest.mark.parametrize("shape", [(512, 512, 256), (300, 520, 200), (129, 264, 72)])
def test_program_tiles_recomputed_in_the_kernels_own_tiling(tile, shape, gpu):
    """Program tiles the generator has no kernel for: the covered part of C is computed in
    128 x 256 tiles instead, with the same result."""
    m, n, k = shape
    bm, bn, bk = tile
    rng = np.random.default_rng(m + n + bm + bn)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32)
    c, kind = run_dot(a, b, bm, bn, bk)
    assert kind == "tcgen05"
    assert no.relative_frobenius_error(c, expected(a, b)) < TEST_TOLERANCE


def test_a_grid_that_covers_part_of_c_writes_only_that_part(gpu):
    """Two by three programs of 64 x 64 over a 512 x 512 problem: rows 0..127 and columns
    0..191 are written, everything else keeps its canary."""
    m = n = k = 512
    rng = np.random.default_rng(77)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = corpus.matmul_dot_kernel.launcher((2, 3), da, db, dc, m, n, k, BM=64, BN=64, BK=64)
    assert launcher.artifact.plan.kind == "tcgen05"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    got = dc.to_host()
    assert no.relative_frobenius_error(got[:128, :192], expected(a, b)[:128, :192]) < TEST_TOLERANCE
    untouched = np.ones((m, n), bool)
    untouched[:128, :192] = False
    assert np.isnan(got[untouched]).all()


@pytest.mark.parametrize("shape", [(512, 512, 256), (300, 520, 200), (1000, 264, 72), (129, 256, 64)])
@pytest.mark.parametrize("bn", [128, 256])
def test_256_row_tiles(shape, bn, gpu):
    """BM=256: one program's tile is a whole CTA-pair tile (each CTA holds 128 of its rows)."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + bn)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32)
    c, kind = run_dot(a, b, 256, bn, 64)
    assert kind == "tcgen05"
    assert no.relative_frobenius_error(c, expected(a, b)) < TEST_TOLERANCE


@pytest.mark.parametrize("tile", [(64, 64), (128, 64), (192, 64), (256, 64), (128, 128), (256, 128)])
@pytest.mark.parametrize("stages", [None, 2])
def test_tcgen05_tile_shapes(tile, stages, gpu):
    bn, bk = tile
    rng = np.random.default_rng(bn + bk)
    a = rng.standard_normal((512, 512), dtype=np.float32)
    b = rng.standard_normal((512, 512), dtype=np.float32)
    options = {} if stages is None else {"num_stages": stages}
    c, kind = run_dot(a, b, 128, bn, bk, **options)       # default pairing: cta_group 2 iff BN % 128 == 0
    assert kind == "tcgen05"
    assert no.relative_frobenius_error(c, expected(a, b)) < TEST_TOLERANCE


TF32_TOLERANCE = 2e-3      # operands keep 10 mantissa bits: about 2^-11 relative error per element


def run_tf32(a, b, bn, bk, **options):
    m, k = a.shape
    n = b.shape[1]
    da, db = device.to_device(a), device.to_device(b)
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    grid = (-(-m // 128), -(-n // bn))
    launcher = corpus.matmul_tf32_kernel.launcher(grid, da, db, dc, m, n, k, BM=128, BN=bn, BK=bk, **options)
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert launcher.artifact.plan.kind == "tcgen05"
    return dc.to_host()


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("shape,bn,bk", [((128, 256, 32), 256, 32), ((256, 512, 256), 256, 32),
                                         ((384, 384, 192), 128, 64), ((300, 520, 200), 256, 32),
                                         ((129, 264, 72), 128, 32)])
def test_tf32_operands(shape, bn, bk, cta_group, gpu):
    """fp32 arrays through kind::tf32.  Small integers are exact in tf32, so a wrong tile
    address or descriptor shows as a bit difference; random operands must stay inside the
    tolerance tf32's 10-bit mantissa implies, against the fp64 product of the fp32 inputs."""
    m, n, k = shape
    rng = np.random.default_rng(m + 3 * n + k)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    c = run_tf32(a, b, bn, bk, cta_group=cta_group)
    assert np.array_equal(c, (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32))
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    c = run_tf32(a, b, bn, bk, cta_group=cta_group)
    error = no.relative_frobenius_error(c, no.matmul_f64(a, b))
    assert 1e-6 < error < TF32_TOLERANCE, error        # above 1e-6: the operands really were cut to tf32


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("shape,shift", [((300, 520, 200), 3), ((256, 256, 64), 0), ((129, 264, 72), -40)])
def test_index_dependent_epilogue(shape, shift, cta_group, gpu):
    """A causal mask and a per-row scale computed from the element's own row and column."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + shift)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = corpus.matmul_causal_kernel.launcher((-(-m // 128), -(-n // 256)), da, db, dc, m, n, k, shift,
                                                    BM=128, BN=256, BK=64, cta_group=cta_group)
    assert launcher.artifact.plan.kind == "tcgen05"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    got = dc.to_host()
    rows, cols = np.arange(m)[:, None], np.arange(n)[None, :]
    masked = rows + shift < cols
    assert np.all(np.isneginf(got[masked])) and not np.isinf(got[~masked]).any()
    want = expected(a, b) / (rows + 1)
    assert no.relative_frobenius_error(got[~masked], want[~masked]) < TEST_TOLERANCE


def test_augmented_accumulation_and_unmasked_loads(gpu):
    """``acc += tl.dot(a, b)`` with loads that carry no masks (sizes are tile multiples)."""
    from test_dot_matcher import augmented_dot_kernel

    m, n, k = 256, 512, 192
    rng = np.random.default_rng(21)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = augmented_dot_kernel.launcher((m // 128, n // 256), da, db, dc, m, n, k, BM=128, BN=256, BK=64)
    assert launcher.artifact.plan.kind == "tcgen05"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert no.relative_frobenius_error(dc.to_host(), expected(a, b)) < TEST_TOLERANCE


@pytest.mark.parametrize("tile", [(128, 256, 64), (16, 16, 16)])
@pytest.mark.parametrize("shape", [(256, 512, 256), (300, 520, 200), (129, 264, 72)])
def test_pointer_bumping_loop(shape, tile, gpu):
    """Carried pointer blocks on both paths: tcgen05 (the loop is recognised as the same GEMM)
    and SIMT (offsets carried in registers), with ragged edges in all three dimensions."""
    m, n, k = shape
    bm, bn, bk = tile
    rng = np.random.default_rng(m + n + bm)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = corpus.matmul_pointer_bump_kernel.launcher((-(-m // bm), -(-n // bn)), da, db, dc, m, n, k,
                                                          BM=bm, BN=bn, BK=bk)
    assert launcher.artifact.plan.kind == ("tcgen05" if bm == 128 else "simt")
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert no.relative_frobenius_error(dc.to_host(), expected(a, b)) < TEST_TOLERANCE


@pytest.mark.parametrize("m,n,k", [(1, 512, 256), (16, 1024, 1000), (40, 520, 72), (64, 8192, 1024), (33, 264, 2048),
                                   (100, 1024, 520), (128, 512, 4096)])
def test_skinny_launches_use_the_variant_that_fetches_few_rows(m, n, k, gpu):
    """At most 128 rows of C: the launch picks the kernel variant that loads only those rows
    of A (the MMA still reads 128; the rest is stale shared memory that only reaches rows never
    stored), in 64- or 128-column tiles with deep k-blocks.  Rows past M of a larger buffer keep their canary."""
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    whole = device.empty((m + 8, n)).fill_u32(0x7FC00000)
    launcher = corpus.matmul_dot_kernel.launcher((1, -(-n // 256)), da, db, whole.rows(0, m), m, n, k,
                                                 BM=128, BN=256, BK=64)
    plan = launcher.artifact.plan
    assert plan.kind == "tcgen05" and plan.notes["skinny"] and plan.notes["a_rows"] in (16, 32, 64, 128)
    assert plan.notes["a_rows"] >= m
    assert plan.notes["gemm"].bn in (64, 128) and plan.cluster == (1, 1, 1)
    for _ in range(2):                      # the second launch finds other stale data in shared memory
        launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    got = whole.to_host()
    assert no.relative_frobenius_error(got[:m], expected(a, b)) < TEST_TOLERANCE
    assert np.isnan(got[m:]).all()


def test_operands_tma_cannot_address_use_the_simt_variant(gpu):
    """K = 100 bf16 elements is a 200-byte row: not a whole number of 16-byte units, so no
    tensor map can describe A.  The same kernel then runs in its SIMT variant; aligned
    operands of the same kernel object still take the tensor-core path."""
    rng = np.random.default_rng(41)
    for k, want in ((100, "simt"), (104, "tcgen05")):
        a = rng.standard_normal((140, k), dtype=np.float32)
        b = rng.standard_normal((k, 264), dtype=np.float32)
        c, kind = run_dot(a, b, 128, 256, 64)
        assert kind == want
        assert no.relative_frobenius_error(c, expected(a, b)) < TEST_TOLERANCE


def test_large_tile_that_does_not_match_runs_on_the_simt_path(gpu):
    """C written to every other row of a wider array: not the tensor-core form.  The 128x256x64
    tile is staged in dynamic shared memory (96 KiB) and the result is still right."""
    from test_dot_matcher import strided_store_kernel

    m, n, k = 256, 512, 128
    rng = np.random.default_rng(31)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((2 * m, n)).fill_u32(0x7FC00000)
    launcher = strided_store_kernel.launcher((m // 128, n // 256), da, db, dc, m, n, k, BM=128, BN=256, BK=64)
    assert launcher.artifact.plan.kind == "simt" and launcher.artifact.plan.dynamic_smem > 48 * 1024
    launcher()
    runtime.synchronize()
    got = dc.to_host()
    assert no.relative_frobenius_error(got[0::2], expected(a, b)) < TEST_TOLERANCE
    assert np.isnan(got[1::2]).all()


def test_uniform_scalars_in_the_epilogue(gpu):
    """`M % -3`, `K // 7`, `min(M, N - 5)` in the epilogue: rendered as C on the scalar arguments,
    on the tensor-core path, with C's truncating remainder and quotient."""
    from test_dot_matcher import uniform_scalar_epilogue_kernel

    m, n, k = 256, 512, 192
    rng = np.random.default_rng(37)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = uniform_scalar_epilogue_kernel.launcher((m // 128, n // 256), da, db, dc, m, n, k,
                                                       BM=128, BN=256, BK=64)
    assert launcher.artifact.plan.kind == "tcgen05"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    want = expected(a, b) + (m - 3 * (m // 3)) + (k // 7) * 0.5 + min(m, n - 5)     # 256 % -3 == 1 in C
    assert no.relative_frobenius_error(dc.to_host(), want) < TEST_TOLERANCE


def run_fp8(a8, b8, bn, bk, **options):
    """a8, b8: ml_dtypes.float8_e4m3fn or float8_e5m2 arrays."""
    m, k = a8.shape
    n = b8.shape[1]
    da = device.to_device(a8.view(np.uint8), str(a8.dtype))
    db = device.to_device(b8.view(np.uint8), str(b8.dtype))
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    bm = options.pop("bm", 128)
    launcher = corpus.matmul_dot_kernel.launcher((-(-m // bm), -(-n // bn)), da, db, dc, m, n, k,
                                                 BM=bm, BN=bn, BK=bk, **options)
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    return dc.to_host(), launcher.artifact.plan.kind


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("shape,bk", [((128, 256, 128), 128), ((256, 512, 512), 128), ((384, 256, 512), 256),
                                      ((300, 528, 208), 128), ((129, 272, 80), 128)])
def test_fp8_e4m3_operands(shape, bk, cta_group, gpu):
    """e4m3 arrays through kind::f8f6f4.  Small integers are exact in e4m3, so a wrong tile
    address shows as a bit difference; random operands (already rounded to e4m3) must match
    the fp64 product to fp32-accumulation accuracy."""
    import ml_dtypes

    m, n, k = shape
    rng = np.random.default_rng(2 * m + n + k)
    a8 = rng.integers(-3, 4, (m, k)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
    b8 = rng.integers(-3, 4, (k, n)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
    c, kind = run_fp8(a8, b8, 256, bk, cta_group=cta_group)
    assert kind == "tcgen05"
    assert np.array_equal(c, (a8.astype(np.float64) @ b8.astype(np.float64)).astype(np.float32))
    a8 = rng.standard_normal((m, k)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
    b8 = rng.standard_normal((k, n)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
    c, _ = run_fp8(a8, b8, 256, bk, cta_group=cta_group)
    assert no.relative_frobenius_error(c, a8.astype(np.float64) @ b8.astype(np.float64)) < TEST_TOLERANCE


@pytest.mark.parametrize("bm", [128, 16])
def test_fp8_e5m2_operands(bm, gpu):
    """The other fp8 format (instruction format 1), on the tensor-core and on the SIMT path."""
    import ml_dtypes

    rng = np.random.default_rng(bm)
    a8 = rng.standard_normal((200, 144)).astype(np.float32).astype(ml_dtypes.float8_e5m2)
    b8 = rng.standard_normal((144, 272)).astype(np.float32).astype(ml_dtypes.float8_e5m2)
    c, kind = run_fp8(a8, b8, 256 if bm == 128 else 16, 128 if bm == 128 else 16, bm=bm)
    assert kind == ("tcgen05" if bm == 128 else "simt")
    assert no.relative_frobenius_error(c, a8.astype(np.float64) @ b8.astype(np.float64)) < TEST_TOLERANCE


def test_fp8_simt_path_converts_in_registers(gpu):
    import ml_dtypes

    rng = np.random.default_rng(8)
    a8 = rng.standard_normal((19, 24)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
    b8 = rng.standard_normal((24, 23)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
    c, kind = run_fp8(a8, b8, 16, 16, bm=16)
    assert kind == "simt"
    assert no.relative_frobenius_error(c, a8.astype(np.float64) @ b8.astype(np.float64)) < TEST_TOLERANCE


def test_simt_fallback_small_tiles_odd_sizes(gpu):
    """Tiles the tensor-core generator does not cover (and K not a multiple of 8)."""
    rng = np.random.default_rng(5)
    a = rng.standard_normal((19, 5), dtype=np.float32)
    b = rng.standard_normal((5, 23), dtype=np.float32)
    c, kind = run_dot(a, b, 16, 16, 16)
    assert kind == "simt"
    assert no.relative_frobenius_error(c, expected(a, b)) < TEST_TOLERANCE


def test_linearity_at_full_size(gpu):
    """8192^3 is too big for an fp64 product on the host, so check a size-independent
    property on the device — C(a, b1 + b2) == C(a, b1) + C(a, b2) up to rounding — plus
    an fp64 check on a sample of rows."""
    m = n = k = 8192
    rng = np.random.default_rng(4)
    scale = np.float32(1.0 / np.sqrt(k))
    a = no.round_to_bf16(rng.standard_normal((m, k), dtype=np.float32) * scale)
    b1 = no.round_to_bf16(rng.standard_normal((k, n), dtype=np.float32) * scale)
    c1, kind = run_dot(a, b1, 128, 256, 64)
    assert kind == "tcgen05"
    rows = rng.choice(m, 48, replace=False)
    sample = no.matmul_f64(a[rows], b1)
    assert no.relative_frobenius_error(c1[rows], sample) < TEST_TOLERANCE
    c2, _ = run_dot(a, b1 * np.float32(2.0), 128, 256, 64)     # scaling by 2 is exact in bf16
    assert np.array_equal(c2, c1 * np.float32(2.0))


def test_epilogue_fan_out_writes_every_destination(gpu):
    """The fused all-gather path on one GPU: two destination buffers stand in for this
    rank's C and a peer's C; both must receive the tile rows, bit-identically, and
    nothing outside the shard's rows may be touched."""
    m, n, k = 256, 512, 256
    rng = np.random.default_rng(11)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    total_rows = 3 * m                                   # shard = the middle third
    mine = device.empty((total_rows, n)).fill_u32(0x7FC00000)
    peer = device.empty((total_rows, n)).fill_u32(0x7FC00000)
    shard, peer_shard = mine.rows(m, 2 * m), peer.rows(m, 2 * m)
    corpus.matmul_dot_kernel[(m // 128, n // 256)](
        da, db, shard, m, n, k, BM=128, BN=256, BK=64,
        peer_stores={"c": [shard.ptr, peer_shard.ptr]})
    runtime.synchronize()
    dot_codegen.check_status()
    got_mine, got_peer = mine.to_host(), peer.to_host()
    want = expected(a, b)
    assert no.relative_frobenius_error(got_mine[m:2 * m], want) < TEST_TOLERANCE
    assert np.array_equal(got_mine[m:2 * m], got_peer[m:2 * m])
    for untouched in (got_mine[:m], got_mine[2 * m:], got_peer[:m], got_peer[2 * m:]):
        assert np.isnan(untouched).all()


@pytest.mark.parametrize("cta_group,tile", [(1, (128, 256, 64)), (2, (128, 256, 64)), (None, (16, 16, 16))])
def test_dot_epilogue_fusion_bias_scale_activation(cta_group, tile, gpu):
    """Elementwise work after the K-loop runs on the accumulator in registers (tcgen05
    path) or in the SIMT fallback (small tiles); both must match the fp64 evaluation."""
    bm, bn, bk = tile
    m, n, k = (300, 520, 200) if bm == 128 else (37, 45, 24)
    rng = np.random.default_rng(17)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32)
    scale = rng.random(m, dtype=np.float32) + 0.5
    slope = 0.125
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dbias, dscale = device.to_device(bias), device.to_device(scale)
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    options = {} if cta_group is None else {"cta_group": cta_group}
    launcher = corpus.matmul_bias_act_kernel.launcher(
        (-(-m // bm), -(-n // bn)), da, db, dbias, dscale, dc, m, n, k, slope,
        BM=bm, BN=bn, BK=bk, **options)
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert launcher.artifact.plan.kind == ("tcgen05" if bm == 128 else "simt")
    y = (expected(a, b) + bias.astype(np.float64)[None, :]) * scale.astype(np.float64)[:, None]
    y = np.where(y < 0.0, slope * y, y)
    assert no.relative_frobenius_error(dc.to_host(), y) < TEST_TOLERANCE


@pytest.mark.parametrize("tile,cta_group", [((128, 256, 64), 2), ((128, 256, 64), 1), ((16, 16, 16), None)])
def test_fp16_operands(tile, cta_group, gpu):
    """fp16 A and B (kind::f16 with the fp16 operand format; SIMT path widens with cvt)."""
    bm, bn, bk = tile
    m, n, k = (384, 520, 264) if bm == 128 else (37, 45, 24)
    rng = np.random.default_rng(23)
    a = rng.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    b = rng.standard_normal((k, n), dtype=np.float32).astype(np.float16)
    da, db = device.to_device(a), device.to_device(b)
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    options = {} if cta_group is None else {"cta_group": cta_group}
    launcher = corpus.matmul_dot_kernel.launcher((-(-m // bm), -(-n // bn)), da, db, dc, m, n, k,
                                                 BM=bm, BN=bn, BK=bk, **options)
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert launcher.artifact.plan.kind == ("tcgen05" if bm == 128 else "simt")
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert no.relative_frobenius_error(dc.to_host(), want) < TEST_TOLERANCE


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("shape", [(256, 512, 256), (300, 520, 200), (129, 264, 72)])
def test_bf16_output_is_rounded_to_nearest_even(shape, cta_group, gpu):
    """C in bf16: the accumulator is rounded once, by the store, to nearest even —
    the same cvt the SIMT path uses — and ragged edges are clipped by the tensor map."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.DeviceArray((m, n), "bfloat16")
    runtime.memset_u32(dc.ptr, 0x7FC07FC0, (dc.nbytes + 3) // 4)
    launcher = corpus.matmul_dot_kernel.launcher((-(-m // 128), -(-n // 256)), da, db, dc, m, n, k,
                                                 BM=128, BN=256, BK=64, cta_group=cta_group)
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert launcher.artifact.plan.kind == "tcgen05" and launcher.artifact.plan.notes["gemm"].out == "bf16"
    got = (dc.to_host().astype(np.uint32) << 16).view(np.float32)
    want = expected(a, b)
    assert not np.isnan(got).any()
    # within half a bf16 ulp of the fp64 product (plus the fp32 accumulation error)
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-3)) < 2.0 ** -8 + 1e-4
    # and exactly the rounding of this backend's own fp32 result
    dc32 = device.empty((m, n))
    corpus.matmul_dot_kernel[(-(-m // 128), -(-n // 256))](da, db, dc32, m, n, k, BM=128, BN=256, BK=64,
                                                          cta_group=cta_group)
    runtime.synchronize()
    assert np.array_equal(dc.to_host(), no.bf16_bits(dc32.to_host()))


# ---------------------------------------------------------------- 512-row pair tiles (cta_rows=256)

WIDE_SHAPES = [(512, 256, 64), (512, 512, 512), (1024, 1024, 1024), (300, 520, 200), (129, 264, 72),
               (1000, 8, 64), (640, 256, 128), (1536, 768, 2048), (4096, 512, 320)]


@pytest.mark.parametrize("shape", WIDE_SHAPES)
def test_wide_pair_tiles_exact_integers_and_random(shape, gpu):
    """cta_rows=256: each CTA of a pair holds two 128-row halves that share the B operand (one
    accumulator filling TMEM, first k-blocks of a tile issued half by half).  Small integers are
    exact, so any mis-addressed half, stage or TMEM column shows as a bit difference; tiles
    beyond the ragged edge are clipped by the tensor maps."""
    m, n, k = shape
    rng = np.random.default_rng(5 * m + n + k)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    c, kind = run_dot(a, b, 128, 256, 64, cta_rows=256)
    assert kind == "tcgen05"
    assert np.array_equal(c, (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32))
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32) / np.float32(np.sqrt(k))
    c, _ = run_dot(a, b, 128, 256, 64, cta_rows=256)
    assert no.relative_frobenius_error(c, expected(a, b)) < TEST_TOLERANCE
    # the two tilings add the same products in the same order: identical bits
    c_narrow, _ = run_dot(a, b, 128, 256, 64, cta_rows=128)
    assert np.array_equal(c.view(np.uint32), c_narrow.view(np.uint32))


@pytest.mark.parametrize("options", [{"group_m": 1}, {"group_m": 3}, {"num_stages": 2}, {"num_stages": 3}])
def test_wide_pair_tiles_many_tiles_per_cta(options, gpu):
    """More tiles than CTA pairs (several tiles per CTA: the accumulator hand-over between
    epilogue and MMA thread runs many times), and fewer stages than the half-by-half lead."""
    m, n, k = 8192, 2560, 192
    rng = np.random.default_rng(m + n)
    a = rng.integers(-2, 3, (m, k)).astype(np.float32)
    b = rng.integers(-2, 3, (k, n)).astype(np.float32)
    c, kind = run_dot(a, b, 128, 256, 64, cta_rows=256, **options)
    assert kind == "tcgen05"
    assert np.array_equal(c, (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32))


def test_wide_pair_tiles_fan_out_fused_epilogue_and_bf16_output(gpu):
    m, n, k = 768, 512, 256
    rng = np.random.default_rng(23)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    # two destinations
    mine = device.empty((3 * m, n)).fill_u32(0x7FC00000)
    peer = device.empty((3 * m, n)).fill_u32(0x7FC00000)
    shard, peer_shard = mine.rows(m, 2 * m), peer.rows(m, 2 * m)
    corpus.matmul_dot_kernel[(m // 128, n // 256)](
        da, db, shard, m, n, k, BM=128, BN=256, BK=64, cta_rows=256,
        peer_stores={"c": [shard.ptr, peer_shard.ptr]})
    runtime.synchronize()
    dot_codegen.check_status()
    got_mine, got_peer = mine.to_host(), peer.to_host()
    assert no.relative_frobenius_error(got_mine[m:2 * m], expected(a, b)) < TEST_TOLERANCE
    assert np.array_equal(got_mine[m:2 * m], got_peer[m:2 * m])
    for untouched in (got_mine[:m], got_mine[2 * m:], got_peer[:m], got_peer[2 * m:]):
        assert np.isnan(untouched).all()
    # fused bias / scale / activation
    bias = rng.standard_normal(n, dtype=np.float32)
    scale = rng.random(m, dtype=np.float32) + 0.5
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = corpus.matmul_bias_act_kernel.launcher(
        (m // 128, n // 256), da, db, device.to_device(bias), device.to_device(scale), dc, m, n, k, 0.125,
        BM=128, BN=256, BK=64, cta_rows=256)
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert launcher.artifact.plan.kind == "tcgen05"
    y = (expected(a, b) + bias.astype(np.float64)[None, :]) * scale.astype(np.float64)[:, None]
    y = np.where(y < 0.0, 0.125 * y, y)
    assert no.relative_frobenius_error(dc.to_host(), y) < TEST_TOLERANCE
    # bf16 C: exactly the rounding of the fp32 result
    d16 = device.DeviceArray((m, n), "bfloat16")
    d32 = device.empty((m, n))
    for out in (d16, d32):
        corpus.matmul_dot_kernel[(m // 128, n // 256)](da, db, out, m, n, k, BM=128, BN=256, BK=64, cta_rows=256)
    runtime.synchronize()
    dot_codegen.check_status()
    assert np.array_equal(d16.to_host(), no.bf16_bits(d32.to_host()))


# ---------------------------------------------------------------- one-axis launches, early return, transposed C


@pytest.mark.parametrize("shape,group_m", [((1024, 768, 256), 3), ((1000, 520, 200), 4), ((384, 256, 64), 8),
                                           ((2048, 1024, 512), 2)])
def test_grouped_ordering_on_a_one_axis_grid_uses_the_tensor_cores(shape, group_m, gpu):
    m, n, k = shape
    rng = np.random.default_rng(m + n + k + group_m)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    grid = (-(-m // 128) * -(-n // 256),)
    launcher = corpus.matmul_grouped_kernel.launcher(grid, da, db, dc, m, n, k, BM=128, BN=256, BK=64,
                                                     GROUP_M=group_m)
    assert launcher.artifact.plan.kind == "tcgen05"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert no.relative_frobenius_error(dc.to_host(), expected(a, b)) < TEST_TOLERANCE


def test_a_grid_that_is_no_tiling_of_c_falls_back_to_the_simt_variant(gpu):
    """One program short: some tile is never computed.  The launch must not be replaced by a dense
    GEMM; it runs the kernel as written (SIMT) and leaves that tile untouched."""
    m, n, k = 512, 512, 64
    rng = np.random.default_rng(3)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    corpus.matmul_grouped_kernel[(7,)](da, db, dc, m, n, k, BM=128, BN=256, BK=64, GROUP_M=2)
    runtime.synchronize()
    got, want = dc.to_host(), expected(a, b)
    missing = np.isnan(got)
    assert missing.sum() == 128 * 256                       # exactly one tile was not written
    assert no.relative_frobenius_error(np.where(missing, want, got), want) < TEST_TOLERANCE


@pytest.mark.parametrize("shape,extra_programs", [((512, 512, 256), 2), ((300, 520, 200), 0), ((1024, 256, 128), 5),
                                                  ((129, 264, 72), 1)])
def test_early_return_and_transposed_store_use_the_tensor_cores(shape, extra_programs, gpu):
    m, n, k = shape
    rng = np.random.default_rng(m + 2 * n + k)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dct = device.empty((n, m)).fill_u32(0x7FC00000)
    tiles_n = -(-n // 256)
    grid = (-(-m // 128) * tiles_n + extra_programs * tiles_n,)     # whole extra tile rows return early
    launcher = corpus.matmul_guarded_transposed_kernel.launcher(grid, da, db, dct, m, n, k, BM=128, BN=256, BK=64)
    assert launcher.artifact.plan.kind == "tcgen05"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    got = dct.to_host()
    assert not np.isnan(got).any()
    assert no.relative_frobenius_error(got.T, expected(a, b)) < TEST_TOLERANCE


def test_wide_pair_tiles_with_tf32_and_fp8_operands(gpu):
    import ml_dtypes

    m, n, k = 1024, 512, 512
    rng = np.random.default_rng(99)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    assert np.array_equal(run_tf32(a, b, 256, 32, cta_rows=256), want)
    c, kind = run_fp8(a.astype(ml_dtypes.float8_e4m3fn), b.astype(ml_dtypes.float8_e4m3fn), 256, 128, cta_rows=256)
    assert kind == "tcgen05" and np.array_equal(c, want)


def test_launches_pick_the_tile_height_that_fills_the_gpu(gpu):
    """The 512-row pair tile is the default for a deep K; a launch whose 512-row tiles would fill the
    GPU's CTA pairs worse than 256-row tiles would (512 x 8192: 32 tiles for 74 pairs; 4096 x 8192:
    3.5 rounds), or whose K is shallow (the wide tile's exposed epilogue then costs more than its
    operand traffic saves), uses the 256-row tiling instead (compiled on first need); an explicit
    cta_rows is always honoured."""
    from mytriton_b200.dot_codegen import WIDE_TILE_MIN_DEPTH as deep

    da = device.empty((8192, deep), "bfloat16")   # launchers are built, nothing is launched
    db = device.empty((deep, 8192), "bfloat16")
    dc = device.empty((8192, 8192))
    chosen = {}
    for rows in (8192, 4096, 2048, 512):
        launcher = corpus.matmul_dot_kernel.launcher((rows // 128, 8192 // 256), da, db, dc, rows, 8192, deep,
                                                     BM=128, BN=256, BK=64)
        chosen[rows] = launcher.artifact.plan.notes["cta_rows"]
    assert chosen == {8192: 256, 4096: 128, 2048: 256, 512: 128}
    shallow = corpus.matmul_dot_kernel.launcher((64, 32), da, db, dc, 8192, 8192, deep - 64, BM=128, BN=256, BK=64)
    assert shallow.artifact.plan.notes["cta_rows"] == 128
    forced = corpus.matmul_dot_kernel.launcher((8, 32), da, db, dc, 1024, 8192, 64, BM=128, BN=256, BK=64,
                                               cta_rows=256)
    assert forced.artifact.plan.notes["cta_rows"] == 256


# ---------------------------------------------------------------- split K


@pytest.mark.parametrize("shape,split_k,tile_n", [((256, 512, 1024), 4, None), ((213, 152, 200), 3, None),
                                                  ((384, 520, 1032), 8, 128), ((128, 64, 128), 8, 64),
                                                  ((1024, 1024, 2048), 2, 256)])
def test_split_k_matches_the_oracle_and_repeats_bit_for_bit(shape, split_k, tile_n, gpu):
    """Units of work along K, partial sums added in the order of the splits by a second kernel:
    right at ragged edges, with more splits asked for than there are k-blocks, and the same bits
    on every run."""
    m, n, k = shape
    rng = np.random.default_rng(m + 3 * n + 5 * k + split_k)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32)
    options = {"split_k": split_k, **({} if tile_n is None else {"tile_n": tile_n})}
    first, kind = run_dot(a, b, 128, 256, 64, **options)
    assert kind == "tcgen05"
    assert not np.isnan(first).any()
    assert no.relative_frobenius_error(first, expected(a, b)) < TEST_TOLERANCE
    again, _ = run_dot(a, b, 128, 256, 64, **options)
    assert np.array_equal(first, again)


def test_split_k_applies_the_epilogue_after_the_sum(gpu):
    """bias, row scale and a leaky ReLU are no linear map: they run in the kernel that adds the
    partial sums, once per element; bf16 C and a transposed C are written by that kernel too."""
    m, n, k = 384, 520, 512
    rng = np.random.default_rng(41)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32)
    scale = rng.random(m, dtype=np.float32) + 0.5
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = corpus.matmul_bias_act_kernel.launcher(
        (-(-m // 128), -(-n // 256)), da, db, device.to_device(bias), device.to_device(scale), dc, m, n, k, 0.125,
        BM=128, BN=256, BK=64, split_k=4)
    assert launcher.artifact.plan.kind == "tcgen05" and launcher.artifact.plan.notes["split_k"] == 4
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    y = (expected(a, b) + bias.astype(np.float64)[None, :]) * scale.astype(np.float64)[:, None]
    y = np.where(y < 0.0, 0.125 * y, y)
    assert no.relative_frobenius_error(dc.to_host(), y) < TEST_TOLERANCE
    # bf16 C is the rounding of the fp32 result of the same split
    d16 = device.DeviceArray((m, n), "bfloat16")
    d32 = device.empty((m, n))
    for out in (d16, d32):
        corpus.matmul_dot_kernel[(-(-m // 128), -(-n // 256))](da, db, out, m, n, k, BM=128, BN=256, BK=64, split_k=4)
    runtime.synchronize()
    dot_codegen.check_status()
    assert np.array_equal(d16.to_host(), no.bf16_bits(d32.to_host()))
    # transposed C
    dct = device.empty((n, m)).fill_u32(0x7FC00000)
    tiles = -(-m // 128) * -(-n // 256)
    corpus.matmul_guarded_transposed_kernel[(tiles,)](da, db, dct, m, n, k, BM=128, BN=256, BK=64, split_k=2)
    runtime.synchronize()
    dot_codegen.check_status()
    assert no.relative_frobenius_error(dct.to_host().T, expected(a, b)) < TEST_TOLERANCE


@pytest.mark.parametrize("shape,want", [((1024, 1024, 1024), {"tile_n": 64}), ((512, 512, 4096), {"split_k": True}),
                                        ((1024, 8192, 4096), None)])
def test_small_problems_pick_narrower_tiles_or_split_k_on_their_own(shape, want, gpu):
    """A launch with too few tiles for the GPU's CTA pairs switches to the single-CTA kernel on
    narrower tiles, with several units along a deep K; a launch that fills the GPU keeps the pairs."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = corpus.matmul_dot_kernel.launcher((m // 128, n // 256), da, db, dc, m, n, k, BM=128, BN=256, BK=64)
    notes = launcher.artifact.plan.notes
    if want is None:
        assert notes["cta_group"] == 2 and notes["split_k"] == 1
    else:
        assert notes["cta_group"] == 1
        if "tile_n" in want:
            assert notes["gemm"].bn == want["tile_n"]
        if "split_k" in want:
            assert notes["split_k"] > 1
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert no.relative_frobenius_error(dc.to_host(), expected(a, b)) < TEST_TOLERANCE


@pytest.mark.parametrize("shape", [(100, 520, 4096), (16, 1024, 2048), (128, 8192, 1024), (40, 256, 512)])
def test_skinny_launches_split_k_on_their_own(shape, gpu):
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
    b = rng.standard_normal((k, n), dtype=np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = corpus.matmul_dot_kernel.launcher((1, -(-n // 256)), da, db, dc, m, n, k, BM=128, BN=256, BK=64)
    notes = launcher.artifact.plan.notes
    assert notes["skinny"] and notes["cta_group"] == 1
    want = dot_codegen.skinny_options(notes["a_rows"], n, k, 64, runtime.device_info(runtime.current_device()).sm_count)
    assert notes["split_k"] == want.get("split_k", 1) and notes["gemm"].bn == want.get("tile_n", 64)
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    got = dc.to_host()
    assert not np.isnan(got).any()
    assert no.relative_frobenius_error(got, expected(a, b)) < TEST_TOLERANCE


def test_split_k_and_narrow_tiles_with_tf32_and_fp8_operands(gpu):
    """Small integers are exact in tf32 and fp8, so every unit's k-range and every partial sum's
    place in the workspace shows as a bit difference if it is wrong."""
    import ml_dtypes

    m, n, k = 384, 512, 1024
    rng = np.random.default_rng(77)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    assert np.array_equal(run_tf32(a, b, 256, 32, split_k=4), want)
    assert np.array_equal(run_tf32(a, b, 256, 32, tile_n=64, split_k=3), want)
    assert np.array_equal(run_tf32(a, b, 256, 32), want)                   # whatever the launcher picks
    for options in ({"split_k": 2}, {"tile_n": 128, "split_k": 4}, {}):
        c, kind = run_fp8(a.astype(ml_dtypes.float8_e4m3fn), b.astype(ml_dtypes.float8_e4m3fn), 256, 128, **options)
        assert kind == "tcgen05" and np.array_equal(c, want), options


# ---------------------------------------------------------------- B stored as its transpose


NT_VARIANTS = [{}, {"cta_group": 2, "cta_rows": 128}, {"cta_group": 2, "cta_rows": 256}, {"cta_group": 1},
               {"cta_group": 1, "tile_n": 64}, {"cta_group": 1, "tile_n": 128, "split_k": 3}]


@pytest.mark.parametrize("options", NT_VARIANTS)
@pytest.mark.parametrize("shape", [(256, 512, 256), (1000, 520, 200), (129, 264, 72), (1024, 1024, 1024)])
def test_b_stored_as_its_transpose(shape, options, gpu):
    """A @ Bt.T with Bt [N, K] row-major: small integers (exact in bf16) show a wrong tile address
    or descriptor as a bit difference, at ragged edges too, in every kernel variant."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    bt = rng.integers(-3, 4, (n, k)).astype(np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    dbt = device.to_device(no.bf16_bits(bt), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = corpus.matmul_nt_kernel.launcher((-(-m // 128), -(-n // 256)), da, dbt, dc, m, n, k,
                                                BM=128, BN=256, BK=64, **options)
    assert launcher.artifact.plan.kind == "tcgen05" and launcher.artifact.plan.notes["gemm"].b_transposed
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    want = (a.astype(np.float64) @ bt.astype(np.float64).T).astype(np.float32)
    assert np.array_equal(dc.to_host(), want)


def test_b_transposed_skinny_and_random_operands(gpu):
    rng = np.random.default_rng(5)
    for m, n, k in ((16, 1024, 2048), (100, 520, 4096), (384, 768, 520)):
        a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
        bt = rng.standard_normal((n, k), dtype=np.float32)
        da = device.to_device(no.bf16_bits(a), "bfloat16")
        dbt = device.to_device(no.bf16_bits(bt), "bfloat16")
        dc = device.empty((m, n)).fill_u32(0x7FC00000)
        launcher = corpus.matmul_nt_kernel.launcher((-(-m // 128), -(-n // 256)), da, dbt, dc, m, n, k,
                                                    BM=128, BN=256, BK=64)
        assert launcher.artifact.plan.kind == "tcgen05"
        launcher()
        runtime.synchronize()
        dot_codegen.check_status()
        want = no.matmul_f64(no.round_to_bf16(a), no.round_to_bf16(bt).T)
        assert no.relative_frobenius_error(dc.to_host(), want) < TEST_TOLERANCE


@triton.jit
def matmul_nt_tf32_kernel(a, bt, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
    offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        offs_k = k0 + tl.arange(0, BK)
        a_tile = tl.load(a + offs_m[:, None] * K + offs_k[None, :],
                         mask=(offs_m[:, None] < M) & (offs_k[None, :] < K), other=0.0)
        b_tile = tl.load(bt + offs_n[None, :] * K + offs_k[:, None],
                         mask=(offs_k[:, None] < K) & (offs_n[None, :] < N), other=0.0)
        acc = tl.dot(a_tile, b_tile, acc, input_precision="tf32")
    tl.store(c + offs_m[:, None] * N + offs_n[None, :], acc,
             mask=(offs_m[:, None] < M) & (offs_n[None, :] < N))


@pytest.mark.parametrize("options", [{}, {"cta_group": 2, "cta_rows": 256}, {"cta_group": 1, "split_k": 2}])
def test_b_transposed_with_tf32_and_fp8_operands(options, gpu):
    import ml_dtypes

    m, n, k = 384, 520, 1024
    rng = np.random.default_rng(78)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    bt = rng.integers(-3, 4, (n, k)).astype(np.float32)
    want = (a.astype(np.float64) @ bt.astype(np.float64).T).astype(np.float32)
    grid = (-(-m // 128), -(-n // 256))
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = matmul_nt_tf32_kernel.launcher(grid, device.to_device(a), device.to_device(bt), dc, m, n, k,
                                              BM=128, BN=256, BK=32, **options)
    assert launcher.artifact.plan.kind == "tcgen05" and launcher.artifact.plan.notes["gemm"].operand == "tf32"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert np.array_equal(dc.to_host(), want)
    a8, bt8 = a.astype(ml_dtypes.float8_e4m3fn), bt.astype(ml_dtypes.float8_e4m3fn)
    dc8 = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = corpus.matmul_nt_kernel.launcher(
        grid, device.to_device(a8.view(np.uint8), "float8_e4m3fn"), device.to_device(bt8.view(np.uint8), "float8_e4m3fn"),
        dc8, m, n, k, BM=128, BN=256, BK=128, **options)
    assert launcher.artifact.plan.kind == "tcgen05" and launcher.artifact.plan.notes["gemm"].operand == "f8e4m3"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert np.array_equal(dc8.to_host(), want)


# ---------------------------------------------------------------- A stored as its transpose


@pytest.mark.parametrize("options", NT_VARIANTS)
@pytest.mark.parametrize("shape", [(256, 512, 256), (1000, 520, 200), (136, 264, 72), (1024, 1024, 1024)])
@pytest.mark.parametrize("both", [False, True])
def test_a_stored_as_its_transpose(shape, options, both, gpu):
    """At.T @ B (and At.T @ Bt.T) with At [K, M] row-major: A becomes the MN-major operand.  Small
    integers show a wrong tile address or descriptor as a bit difference, at ragged edges too."""
    m, n, k = shape
    rng = np.random.default_rng(2 * m + n + k + both)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    dat = device.to_device(no.bf16_bits(np.ascontiguousarray(a.T)), "bfloat16")
    db = device.to_device(no.bf16_bits(np.ascontiguousarray(b.T) if both else b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    kernel = corpus.matmul_tt_kernel if both else corpus.matmul_tn_kernel
    launcher = kernel.launcher((-(-m // 128), -(-n // 256)), dat, db, dc, m, n, k, BM=128, BN=256, BK=64, **options)
    match = launcher.artifact.plan.notes["gemm"]
    assert launcher.artifact.plan.kind == "tcgen05" and match.a_transposed and match.b_transposed == both
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert np.array_equal(dc.to_host(), (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32))


@triton.jit
def matmul_tn_tf32_kernel(at, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
    offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        offs_k = k0 + tl.arange(0, BK)
        a_tile = tl.load(at + offs_k[None, :] * M + offs_m[:, None],
                         mask=(offs_m[:, None] < M) & (offs_k[None, :] < K), other=0.0)
        b_tile = tl.load(b + offs_k[:, None] * N + offs_n[None, :],
                         mask=(offs_k[:, None] < K) & (offs_n[None, :] < N), other=0.0)
        acc = tl.dot(a_tile, b_tile, acc, input_precision="tf32")
    tl.store(c + offs_m[:, None] * N + offs_n[None, :], acc,
             mask=(offs_m[:, None] < M) & (offs_n[None, :] < N))


@pytest.mark.parametrize("options", [{}, {"cta_group": 2, "cta_rows": 256}, {"cta_group": 1, "split_k": 2}])
def test_a_transposed_with_tf32_and_fp8_operands(options, gpu):
    import ml_dtypes

    m, n, k = 384, 528, 1024                 # rows of an fp8 B are n bytes: a whole number of 16-byte units
    rng = np.random.default_rng(79)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    at = np.ascontiguousarray(a.T)
    grid = (-(-m // 128), -(-n // 256))
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = matmul_tn_tf32_kernel.launcher(grid, device.to_device(at), device.to_device(b), dc, m, n, k,
                                              BM=128, BN=256, BK=32, **options)
    assert launcher.artifact.plan.kind == "tcgen05" and launcher.artifact.plan.notes["gemm"].operand == "tf32"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert np.array_equal(dc.to_host(), want)
    at8, b8 = at.astype(ml_dtypes.float8_e4m3fn), b.astype(ml_dtypes.float8_e4m3fn)
    dc8 = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = corpus.matmul_tn_kernel.launcher(
        grid, device.to_device(at8.view(np.uint8), "float8_e4m3fn"), device.to_device(b8.view(np.uint8), "float8_e4m3fn"),
        dc8, m, n, k, BM=128, BN=256, BK=128, **options)
    assert launcher.artifact.plan.kind == "tcgen05" and launcher.artifact.plan.notes["gemm"].operand == "f8e4m3"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert np.array_equal(dc8.to_host(), want)


# ---------------------------------------------------------------- strides as arguments


@pytest.mark.parametrize("layout", ["NN", "NT", "TN", "TT", "Ct", "general"])
@pytest.mark.parametrize("shape", [(256, 512, 256), (1000, 520, 200)])
def test_matmul_written_with_stride_arguments(layout, shape, gpu):
    """One kernel source, every storage layout: the strides that equal 1 are folded into the IR per
    call, the matcher sees which axis is contiguous, and all but the general case (no unit stride
    along K for A) run on the tensor cores.  Exact-integer data, bit-exact results."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32)
    a_store, sam, sak = (np.ascontiguousarray(a.T), 1, m) if layout in ("TN", "TT") else (a, k, 1)
    b_store, sbk, sbn = (np.ascontiguousarray(b.T), 1, k) if layout in ("NT", "TT") else (b, n, 1)
    if layout == "general":                                  # A with every second column unused
        wide = np.zeros((m, 2 * k), np.float32)
        wide[:, ::2] = a
        a_store, sam, sak = wide, 2 * k, 2
    da = device.to_device(no.bf16_bits(a_store), "bfloat16")
    db = device.to_device(no.bf16_bits(b_store), "bfloat16")
    c_shape, scm, scn = ((n, m), 1, m) if layout == "Ct" else ((m, n), n, 1)
    dc = device.empty(c_shape).fill_u32(0x7FC00000)
    launcher = corpus.matmul_strided_kernel.launcher((-(-m // 128), -(-n // 256)), da, db, dc, m, n, k,
                                                     sam, sak, sbk, sbn, scm, scn, BM=128, BN=256, BK=64)
    assert launcher.artifact.plan.kind == ("simt" if layout == "general" else "tcgen05")
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    got = dc.to_host()
    assert np.array_equal(got.T if layout == "Ct" else got, want)


@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
@pytest.mark.parametrize("shape,group_m", [((256, 512, 256), 8), ((1000, 520, 200), 3), ((2048, 1024, 1000), 4)])
def test_the_tutorial_spelling(layout, shape, group_m, gpu):
    """A matmul written the common way (one-axis grid with grouped ordering, stride arguments,
    pointer blocks advanced in a loop over k-blocks): bit-exact on exact-integer data, on the
    tensor cores."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k + group_m)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    a_store, sam, sak = (np.ascontiguousarray(a.T), 1, m) if layout == "TN" else (a, k, 1)
    b_store, sbk, sbn = (np.ascontiguousarray(b.T), 1, k) if layout == "NT" else (b, n, 1)
    da = device.to_device(no.bf16_bits(a_store), "bfloat16")
    db = device.to_device(no.bf16_bits(b_store), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    grid = (-(-m // 128) * -(-n // 256),)
    launcher = corpus.matmul_tutorial_kernel.launcher(grid, da, db, dc, m, n, k, sam, sak, sbk, sbn, n, 1,
                                                      BM=128, BN=256, BK=64, GROUP_M=group_m)
    assert launcher.artifact.plan.kind == "tcgen05"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert np.array_equal(dc.to_host(), (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32))


@pytest.mark.parametrize("shape,group_m", [((256, 512, 256), 8), ((1000, 520, 200), 3), ((333, 264, 1000), 2)])
def test_the_tutorial_spelling_with_modulo_indices(shape, group_m, gpu):
    """The operands' indices wrap around modulo M and N instead of being masked; the store's mask
    drops what wrapped.  Bit-exact on exact-integer data, on the tensor cores."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k + group_m)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    dc = device.empty((m, n)).fill_u32(0x7FC00000)
    grid = (-(-m // 128) * -(-n // 256),)
    launcher = corpus.matmul_tutorial_modulo_kernel.launcher(grid, da, db, dc, m, n, k, k, 1, n, 1, n, 1,
                                                             BM=128, BN=256, BK=64, GROUP_M=group_m)
    assert launcher.artifact.plan.kind == "tcgen05"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert np.array_equal(dc.to_host(), (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32))
    # and as written, on the SIMT path: the same bits
    dsimt = device.empty((m, n)).fill_u32(0x7FC00000)
    corpus.matmul_tutorial_modulo_kernel[grid](da, db, dsimt, m, n, k, k, 1, n, 1, n, 1,
                                               BM=128, BN=256, BK=64, GROUP_M=group_m, tensor_cores=False)
    runtime.synchronize()
    assert np.array_equal(dsimt.to_host(), dc.to_host())


@triton.jit
def leaky_relu(x):
    return tl.where(x >= 0, x, 0.01 * x)


@triton.jit
def matmul_f16_out_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    """fp16 operands, an activation from a helper, `.to(tl.float16)` and an fp16 C."""
    offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
    offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        offs_k = k0 + tl.arange(0, BK)
        acc += tl.dot(tl.load(a + offs_m[:, None] * K + offs_k[None, :],
                              mask=(offs_m[:, None] < M) & (offs_k[None, :] < K), other=0.0),
                      tl.load(b + offs_k[:, None] * N + offs_n[None, :],
                              mask=(offs_k[:, None] < K) & (offs_n[None, :] < N), other=0.0))
    out = leaky_relu(acc).to(tl.float16)
    tl.store(c + offs_m[:, None] * N + offs_n[None, :], out, mask=(offs_m[:, None] < M) & (offs_n[None, :] < N))


@pytest.mark.parametrize("options", [{}, {"cta_group": 2, "cta_rows": 256}, {"cta_group": 1, "split_k": 2}])
def test_fp16_c_with_an_activation_and_a_conversion(options, gpu):
    m, n, k = 384, 520, 512
    rng = np.random.default_rng(88)
    a = rng.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    b = (rng.standard_normal((k, n), dtype=np.float32) / np.float32(np.sqrt(k))).astype(np.float16)
    dc = device.DeviceArray((m, n), "float16")
    launcher = matmul_f16_out_kernel.launcher((-(-m // 128), -(-n // 256)), device.to_device(a), device.to_device(b), dc,
                                              m, n, k, BM=128, BN=256, BK=64, **options)
    match = launcher.artifact.plan.notes["gemm"]
    assert launcher.artifact.plan.kind == "tcgen05" and (match.operand, match.out) == ("f16", "f16")
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    exact = a.astype(np.float64) @ b.astype(np.float64)
    want = np.where(exact >= 0, exact, 0.01 * exact)
    got = dc.to_host().astype(np.float64)
    assert not np.isnan(got).any()
    assert no.relative_frobenius_error(got, want) < 1e-3          # fp16 rounding of C: 2^-11 relative per element


@pytest.mark.parametrize("options", [{}, {"cta_group": 2, "cta_rows": 256}, {"cta_group": 1, "tile_n": 128, "split_k": 2}])
@pytest.mark.parametrize("shape", [(256, 512, 256), (1000, 520, 200)])
def test_a_transposed_tile_as_a_dot_operand(shape, options, gpu):
    """`tl.dot(x_tile, tl.trans(w_tile), acc)` with w [N, K]: the matcher reads the tile with its
    coordinates exchanged, which makes B the K-major operand.  Bit-exact on exact-integer data."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    x = rng.integers(-3, 4, (m, k)).astype(np.float32)
    w = rng.integers(-3, 4, (n, k)).astype(np.float32)
    dx = device.to_device(no.bf16_bits(x), "bfloat16")
    dw = device.to_device(no.bf16_bits(w), "bfloat16")
    dy = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = corpus.linear_layer_kernel.launcher((-(-m // 128), -(-n // 256)), dx, dw, dy, m, n, k,
                                                   BM=128, BN=256, BK=64, **options)
    assert launcher.artifact.plan.kind == "tcgen05" and launcher.artifact.plan.notes["gemm"].b_transposed
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert np.array_equal(dy.to_host(), (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32))


@pytest.mark.parametrize("options", [{}, {"cta_group": 2, "cta_rows": 256}, {"cta_group": 1, "split_k": 3}])
@pytest.mark.parametrize("shape", [(256, 512, 256), (1000, 520, 200)])
def test_residual_tile_in_the_epilogue(shape, options, gpu):
    """c = alpha * a @ b + residual with an fp32 and a bf16 residual, and in place (residual is c)."""
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    skip = rng.integers(-8, 9, (m, n)).astype(np.float32)
    da = device.to_device(no.bf16_bits(a), "bfloat16")
    db = device.to_device(no.bf16_bits(b), "bfloat16")
    want = (0.5 * (a.astype(np.float64) @ b.astype(np.float64)) + skip).astype(np.float32)
    grid = (-(-m // 128), -(-n // 256))
    for residual in (device.to_device(skip), device.to_device(no.bf16_bits(skip), "bfloat16")):
        dc = device.empty((m, n)).fill_u32(0x7FC00000)
        launcher = corpus.matmul_residual_kernel.launcher(grid, da, db, residual, dc, m, n, k, 0.5,
                                                          BM=128, BN=256, BK=64, **options)
        assert launcher.artifact.plan.kind == "tcgen05"
        launcher()
        runtime.synchronize()
        dot_codegen.check_status()
        assert np.array_equal(dc.to_host(), want)
    dc = device.to_device(skip)                                  # c += 0.5 * a @ b
    corpus.matmul_residual_kernel[grid](da, db, dc, dc, m, n, k, 0.5, BM=128, BN=256, BK=64, **options)
    runtime.synchronize()
    dot_codegen.check_status()
    assert np.array_equal(dc.to_host(), want)


@triton.jit
def gradient_kernel(xt, dy, dw, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    """dw[M, N] = xt.T @ dy with xt stored [K, M]: a [BK, BM] tile of xt is loaded as it lies in memory
    and transposed in the call."""
    rows = tl.program_id(0) * BM + tl.arange(0, BM)
    cols = tl.program_id(1) * BN + tl.arange(0, BN)
    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        ks = k0 + tl.arange(0, BK)
        x_tile = tl.load(xt + ks[:, None] * M + rows[None, :], mask=(ks[:, None] < K) & (rows[None, :] < M), other=0.0)
        y_tile = tl.load(dy + ks[:, None] * N + cols[None, :], mask=(ks[:, None] < K) & (cols[None, :] < N), other=0.0)
        acc = tl.dot(tl.trans(x_tile), y_tile, acc)
    tl.store(dw + rows[:, None] * N + cols[None, :], acc, mask=(rows[:, None] < M) & (cols[None, :] < N))


@pytest.mark.parametrize("options", [{}, {"cta_group": 2, "cta_rows": 128}, {"cta_group": 1, "split_k": 2}])
def test_a_transposed_tile_as_the_first_operand(options, gpu):
    m, n, k = 520, 264, 1000
    rng = np.random.default_rng(91)
    x = rng.integers(-3, 4, (k, m)).astype(np.float32)
    dy = rng.integers(-3, 4, (k, n)).astype(np.float32)
    dxt = device.to_device(no.bf16_bits(x), "bfloat16")
    ddy = device.to_device(no.bf16_bits(dy), "bfloat16")
    dw = device.empty((m, n)).fill_u32(0x7FC00000)
    launcher = gradient_kernel.launcher((-(-m // 128), -(-n // 256)), dxt, ddy, dw, m, n, k, BM=128, BN=256, BK=64, **options)
    match = launcher.artifact.plan.notes["gemm"]
    assert launcher.artifact.plan.kind == "tcgen05" and match.a_transposed and not match.b_transposed
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    assert np.array_equal(dw.to_host(), (x.astype(np.float64).T @ dy.astype(np.float64)).astype(np.float32))


@triton.jit
def matmul_f16_bias_kernel(a, b, bias, residual, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    """An all-fp16 layer: fp16 operands, fp16 bias vector, fp16 residual tile, fp16 C."""
    rows = tl.program_id(0) * BM + tl.arange(0, BM)
    cols = tl.program_id(1) * BN + tl.arange(0, BN)
    inside = (rows[:, None] < M) & (cols[None, :] < N)
    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        ks = k0 + tl.arange(0, BK)
        acc += tl.dot(tl.load(a + rows[:, None] * K + ks[None, :], mask=(rows[:, None] < M) & (ks[None, :] < K), other=0.0),
                      tl.load(b + ks[:, None] * N + cols[None, :], mask=(ks[:, None] < K) & (cols[None, :] < N), other=0.0))
    shift = tl.load(bias + cols, mask=cols < N, other=0.0)
    skip = tl.load(residual + rows[:, None] * N + cols[None, :], mask=inside, other=0.0)
    tl.store(c + rows[:, None] * N + cols[None, :], (acc + shift[None, :] + skip).to(tl.float16), mask=inside)


@pytest.mark.parametrize("options", [{}, {"cta_group": 1, "split_k": 2}])
def test_fp16_vectors_and_tiles_in_the_epilogue(options, gpu):
    m, n, k = 384, 520, 256
    rng = np.random.default_rng(92)
    a = rng.integers(-3, 4, (m, k)).astype(np.float16)
    b = rng.integers(-3, 4, (k, n)).astype(np.float16)
    bias = rng.integers(-8, 9, n).astype(np.float16)
    skip = rng.integers(-8, 9, (m, n)).astype(np.float16)
    dc = device.DeviceArray((m, n), "float16")
    launcher = matmul_f16_bias_kernel.launcher(
        (-(-m // 128), -(-n // 256)), device.to_device(a), device.to_device(b), device.to_device(bias),
        device.to_device(skip), dc, m, n, k, BM=128, BN=256, BK=64, **options)
    assert launcher.artifact.plan.kind == "tcgen05"
    launcher()
    runtime.synchronize()
    dot_codegen.check_status()
    want = (a.astype(np.float64) @ b.astype(np.float64) + bias.astype(np.float64)[None, :] + skip).astype(np.float16)
    assert np.array_equal(dc.to_host(), want)                   # small integers: exact in fp16 too
