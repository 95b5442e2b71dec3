"""The CTA-pair (``cta_group::2``) variant of the tcgen05 GEMM kernel.

Two CTAs of a 2-CTA cluster (one per SM of a pair) compute one tile of C:
each loads its own rows of A and its own half (BN/2 columns) of B, and the
leader CTA's single MMA thread issues ``tcgen05.mma.cta_group::2`` with M=256,
which reads both CTAs' shared memory and accumulates 128 rows into each CTA's
TMEM.

Two tile heights (``MH`` = 128-row halves per CTA):

* ``MH = 1``: 256 x BN per pair.  32 KiB per CTA and k-block (BK=64, BN=256)
  through L2 -> shared memory, six pipeline stages, two accumulators in TMEM so
  that tile i+1's main loop overlaps tile i's epilogue.
* ``MH = 2``: 512 x BN per pair, two M=256 instructions per k-step that share
  the B operand.  48 KiB per CTA and k-block for twice the arithmetic, i.e. 25 %
  less operand traffic per flop (L2 -> shared memory and, through the larger
  footprint of a wave, DRAM), four stages.  With BN=256 the tile fills TMEM
  (512 columns), so there is one accumulator and the epilogue is exposed; the
  MMA thread hides half of it by starting the next tile's upper half while the
  lower half is still being read out.

No load uses cluster multicast: each CTA fetches its own operand halves with a
plain ``cp.async.bulk.tensor`` whose completion is counted on the *leader's*
mbarrier.  Only ``tcgen05.commit`` is multicast (it arrives on both CTAs'
barriers).  Everything else — roles, double-buffered accumulators, TMA-store
epilogue with peer fan-out, bounded waits and the status word — is as in the
single-CTA kernel (dot_codegen.py), whose prelude this text is appended to.
"""

PAIR_PRELUDE = r'''
MTB_DEV unsigned mtb_cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
MTB_DEV unsigned mtb_mapa(unsigned smem_addr, unsigned rank) {
    unsigned out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
    return out;
}
MTB_DEV void mtb_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
MTB_DEV void mtb_mbar_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory; completion bytes are counted on `bar`, a
// shared::cluster address that may belong to the other CTA of the pair.  No multicast.
MTB_DEV void mtb_tma_load_2d_pair(unsigned dst, const MtbTensorMap* map, unsigned bar, int c_inner, int c_outer) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(c_inner), "r"(c_outer) : "memory");
}
MTB_DEV void mtb_umma_bf16_pair(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::" MTB_MMA_KIND " [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// arrives (once the MMAs issued so far retire) on the barrier at this offset in both CTAs
MTB_DEV void mtb_umma_commit_pair(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(bar), "h"((unsigned short)3) : "memory");
}
'''

PAIR_KERNEL_HEAD = r'''
extern "C" __global__ __launch_bounds__(192, 1)
void @NAME@(@SIGNATURE@, const __grid_constant__ MtbTensorMap map_a,
            const __grid_constant__ MtbTensorMap map_b,
            const __grid_constant__ MtbTensorMaps8 maps_c, int n_dst,
            int grid_m, int grid_n, int m_rows, int n_cols, int k_depth, int ldc,
            unsigned* status) {
    constexpr int BM = @BM@, BN = @BN@, BK = @BK@, STAGES = @STAGES@;   // BM rows per MMA half
    constexpr int MH = @MH@;                          // 128-row halves of the tile per CTA (2*MH*BM rows per pair)
    constexpr int ACCS = @ACCS@;                      // accumulators in TMEM, MH*BN columns each
    constexpr int CTA_ROWS = MH * BM;
    constexpr int HALF_N = BN / 2;                    // columns of B this CTA fetches
    constexpr int EB = @EB@;                          // bytes per operand element (2; 4 for tf32; 1 for fp8)
    constexpr int AE = 128 / EB;                      // elements in one 128-byte swizzle row
    constexpr int UK = 32 / EB;                       // k-depth of one MMA instruction (32 bytes)
    constexpr int A_BYTES = CTA_ROWS * BK * EB;
    constexpr int B_BYTES = BK * HALF_N * EB;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int OUT_BYTES = 32 * 32 * 4;
    constexpr int TMEM_COLS = @TMEM_COLS@;
    constexpr unsigned AB_FORMAT = @AB_FORMAT@u;     // kind::f16: 0 = fp16, 1 = bf16; kind::tf32: 2 = tf32
    // B in memory: [K, N] row-major (the MN-major operand: sub-tiles of [BK][AE]) or its transpose
    // [N, K] (K-major like A: sub-tiles of [HALF_N][AE])
    constexpr bool B_KMAJOR = @B_KMAJOR@;
    // A in memory: [M, K] row-major (K-major: sub-tiles of [CTA_ROWS][AE]) or its transpose [K, M]
    // (the MN-major operand: sub-tiles of [BK][AE], BM / AE of them per 128-row half)
    constexpr bool A_MMAJOR = @A_MMAJOR@;
    constexpr unsigned IDESC = (1u << 4) | (AB_FORMAT << 7) | (AB_FORMAT << 10)
                             | ((A_MMAJOR ? 1u : 0u) << 15) | ((B_KMAJOR ? 0u : 1u) << 16)
                             | ((unsigned)(BN >> 3) << 17) | ((unsigned)((2 * BM) >> 4) << 24);

    extern __shared__ unsigned char mtb_dyn_smem[];
    __shared__ unsigned long long bar_full[STAGES], bar_empty[STAGES], bar_acc_full[ACCS * MH], bar_acc_empty[ACCS * MH];
    __shared__ unsigned tmem_slot;
    __shared__ unsigned abort_word;
    volatile unsigned* abort_flag = &abort_word;

    const unsigned tiles_base = (mtb_smem(mtb_dyn_smem) + 1023u) & ~1023u;
    const unsigned out_base = tiles_base + STAGES * STAGE_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = mtb_cluster_rank();         // 0 = leader of the pair
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int pair_rows = (grid_m + 2 * MH - 1) / (2 * MH);   // tiles of 2*MH*BM rows
    const int num_tiles = pair_rows * grid_n;
    const int num_kb = (k_depth + BK - 1) / BK;

    if (threadIdx.x == 0) {
        abort_word = 0u;
        for (int s = 0; s < STAGES; ++s) { mtb_mbar_init(mtb_smem(&bar_full[s]), 1); mtb_mbar_init(mtb_smem(&bar_empty[s]), 1); }
        for (int s = 0; s < ACCS * MH; ++s) mtb_mbar_init(mtb_smem(&bar_acc_full[s]), 1);
        for (int s = 0; s < ACCS * MH; ++s) mtb_mbar_init(mtb_smem(&bar_acc_empty[s]), 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(mtb_smem(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    mtb_cluster_sync();                               // both CTAs' barriers exist before any remote arrive
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = tmem_slot;

    auto tile_coords = [&](int t, int& pm, int& pn) {
        constexpr int GROUP_M = @GROUP_M@;
        const int per_group = GROUP_M * grid_n;
        const int group = t / per_group;
        const int first = group * GROUP_M;
        const int rows = (pair_rows - first < GROUP_M) ? (pair_rows - first) : GROUP_M;
        const int in_group = t - group * per_group;
        pm = first + in_group % rows;
        pn = in_group / rows;
    };
'''

PAIR_KERNEL_MAINLOOP = r'''
    if (num_kb > 0) {
        if (warp == 0 && lane == 0) {
            // ---------------- TMA producer (both CTAs; bytes counted on the leader's barrier) ----
            unsigned it = 0;
            for (int t = pair; t < num_tiles && !*abort_flag; t += num_pairs) {
                int pm, pn;
                tile_coords(t, pm, pn);
                const int row0 = (pm * 2 + (int)rank) * CTA_ROWS;
                const int col0 = pn * BN + (int)rank * HALF_N;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const unsigned s = it % STAGES, phase = (it / STAGES) & 1u;
                    if (!mtb_mbar_wait(mtb_smem(&bar_empty[s]), phase ^ 1u, abort_flag, status, 0x10u + s)) break;
                    const unsigned full_local = mtb_smem(&bar_full[s]);
                    const unsigned full = mtb_mapa(full_local, 0u);
                    const unsigned a_dst = tiles_base + s * STAGE_BYTES;
                    const unsigned b_dst = a_dst + A_BYTES;
                    if (rank == 0u) mtb_mbar_expect_tx(full_local, 2 * STAGE_BYTES);
                    if (A_MMAJOR) {
                        #pragma unroll
                        for (int j = 0; j < CTA_ROWS / AE; ++j)
                            mtb_tma_load_2d_pair(a_dst + j * (BK * 128), &map_a, full, row0 + j * AE, kb * BK);
                    } else {
                        #pragma unroll
                        for (int j = 0; j < BK / AE; ++j)
                            mtb_tma_load_2d_pair(a_dst + j * (CTA_ROWS * 128), &map_a, full, kb * BK + j * AE, row0);
                    }
                    if (B_KMAJOR) {
                        #pragma unroll
                        for (int j = 0; j < BK / AE; ++j)
                            mtb_tma_load_2d_pair(b_dst + j * (HALF_N * 128), &map_b, full, kb * BK + j * AE, col0);
                    } else {
                        #pragma unroll
                        for (int j = 0; j < HALF_N / AE; ++j)
                            mtb_tma_load_2d_pair(b_dst + j * (BK * 128), &map_b, full, col0 + j * AE, kb * BK);
                    }
                }
            }
        } else if (warp == 1 && lane == 0 && rank == 0u) {
            // ---------------- MMA issuer (leader CTA only) ----------------
            unsigned it = 0, local_tile = 0;
            for (int t = pair; t < num_tiles && !*abort_flag; t += num_pairs, ++local_tile) {
                const unsigned acc = local_tile % ACCS, acc_phase = (local_tile / ACCS) & 1u;
                const unsigned d_tmem = tmem_base + acc * (MH * BN);
                bool ok = true;
                // the MMAs of one k-block for half h of the tile (B is shared by the halves)
                auto issue = [&](unsigned s, int h, int kb) {
                    // One descriptor per operand and stage; the k-steps differ only in the start
                    // address (bits 0-13 of the descriptor, in 16-byte units), so each further
                    // descriptor is one addition of a compile-time constant.  The single issuing
                    // thread must stay well under the ~128 cycles one instruction keeps the tensor
                    // pipe busy.
                    const unsigned stage = tiles_base + s * STAGE_BYTES;
                    const unsigned long long a_first = !A_MMAJOR
                        ? mtb_desc(stage + h * (BM * 128), 16, 1024)
                        : EB == 4
                        ? mtb_desc(stage + h * (BM / AE) * (BK * 128), BK * 128, 512, 1ull)
                        : mtb_desc(stage + h * (BM / AE) * (BK * 128), BK * 128, 1024);
                    const unsigned long long b_first = B_KMAJOR
                        ? mtb_desc(stage + A_BYTES, 16, 1024)
                        : EB == 4
                        ? mtb_desc(stage + A_BYTES, BK * 128, 512, 1ull)
                        : mtb_desc(stage + A_BYTES, BK * 128, 1024);
                    #pragma unroll
                    for (int k = 0; k < BK / UK; ++k) {
                        const unsigned long long a_desc = a_first + (unsigned long long)(
                            (!A_MMAJOR ? (k / 4) * (CTA_ROWS * 128) + (k % 4) * 32
                                       : EB == 4 ? k * 1024 : k * (UK / 8) * 1024) >> 4);
                        const unsigned long long b_desc = b_first + (unsigned long long)(
                            (B_KMAJOR ? (k / 4) * (HALF_N * 128) + (k % 4) * 32
                                      : EB == 4 ? k * 1024 : k * (UK / 8) * 1024) >> 4);
                        mtb_umma_bf16_pair(d_tmem + h * BN, a_desc, b_desc, IDESC, (kb | k) != 0 ? 1u : 0u);
                    }
                };
                // With more than one half per CTA the first `lead` and the last `tail` k-blocks of a
                // tile are issued half by half.  Lead: half 0 starts as soon as the epilogue has read
                // it out, while the previous tile's half 1 is still being drained (the operands of
                // those k-blocks are already in shared memory: the producer does not wait for TMEM).
                // Tail: half 0 finishes `tail` k-blocks before half 1, so its read-out overlaps the
                // rest of half 1's arithmetic.  In between the halves alternate k-step by k-step.
                // Either way a stage is loaded once and used by both halves before it is freed.
                const int lead = MH > 1 ? (num_kb < STAGES ? num_kb : STAGES) : 0;
                const int tail = MH > 1 ? (num_kb - lead < STAGES ? num_kb - lead : STAGES) : 0;
                for (int h = 0; h < MH && ok; ++h) {
                    if (!mtb_mbar_wait(mtb_smem(&bar_acc_empty[acc * MH + h]), acc_phase ^ 1u, abort_flag, status,
                                       0x20u + acc * MH + h)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    for (int j = 0; j < lead; ++j) {
                        const unsigned s = (it + j) % STAGES, phase = ((it + j) / STAGES) & 1u;
                        if (h == 0) {
                            if (!mtb_mbar_wait(mtb_smem(&bar_full[s]), phase, abort_flag, status, 0x30u + s)) { ok = false; break; }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
                        issue(s, h, j);
                        if (h == MH - 1) mtb_umma_commit_pair(mtb_smem(&bar_empty[s]));
                    }
                }
                if (!ok) break;
                it += lead;
                for (int kb = lead; kb < num_kb - tail; ++kb, ++it) {
                    const unsigned s = it % STAGES, phase = (it / STAGES) & 1u;
                    if (!mtb_mbar_wait(mtb_smem(&bar_full[s]), phase, abort_flag, status, 0x30u + s)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    #pragma unroll
                    for (int h = 0; h < MH; ++h) issue(s, h, kb);
                    mtb_umma_commit_pair(mtb_smem(&bar_empty[s]));       // frees the stage in both CTAs
                }
                if (!ok) break;
                for (int h = 0; h < MH && ok; ++h) {
                    for (int j = 0; j < tail; ++j) {
                        const unsigned s = (it + j) % STAGES, phase = ((it + j) / STAGES) & 1u;
                        if (h == 0) {
                            if (!mtb_mbar_wait(mtb_smem(&bar_full[s]), phase, abort_flag, status, 0x30u + s)) { ok = false; break; }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
                        issue(s, h, num_kb - tail + j);
                        if (h == MH - 1) mtb_umma_commit_pair(mtb_smem(&bar_empty[s]));
                    }
                    // this half of the accumulator is complete: both CTAs' epilogues may read it
                    if (ok) mtb_umma_commit_pair(mtb_smem(&bar_acc_full[acc * MH + h]));
                }
                if (!ok) break;
                it += tail;
            }
        }
    }
'''

PAIR_KERNEL_EPILOGUE = r'''
    if (warp >= 2) {
        // ---------------- epilogue: this CTA's 128 rows, TMEM -> registers -> TMA store ----
        const int quad = warp & 3;
        unsigned local_tile = 0;
        for (int t = pair; t < num_tiles && !*abort_flag; t += num_pairs, ++local_tile) {
            int pm, pn;
            tile_coords(t, pm, pn);
            const unsigned acc = local_tile % ACCS, acc_phase = (local_tile / ACCS) & 1u;
            bool alive = true;
            #pragma unroll 1
            for (int h = 0; h < MH && alive; ++h) {
            if (num_kb > 0) {
                // one lane polls the barrier, the other 31 sleep at the shuffle; every lane then
                // makes its own (immediately successful) wait so that each of them has observed
                // the phase before it reads the accumulator
                unsigned ready = 1u;
                const unsigned bar = mtb_smem(&bar_acc_full[acc * MH + h]);
                if (lane == 0) ready = mtb_mbar_wait(bar, acc_phase, abort_flag, status, 0x40u + acc * MH + h) ? 1u : 0u;
                ready = __shfl_sync(0xffffffffu, ready, 0);
                if (!ready) { alive = false; break; }
                if (lane != 0) mtb_mbar_wait(bar, acc_phase, abort_flag, status, 0x40u + acc * MH + h);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
@EPILOGUE_TILE@
            }
            if (!alive) break;
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    // ---------------- teardown ----------------
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) { }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    mtb_cluster_sync();        // neither CTA leaves (or frees TMEM) while its partner may still use it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}
'''

PAIR_OUT_STAGING_BYTES = 4 * 2 * 32 * 32 * 4


def pair_stage_bytes(bm: int, bn: int, bk: int, elem_bytes: int = 2) -> int:
    return (bm * bk + bk * (bn // 2)) * elem_bytes


def pair_source(prelude: str, substitutions: dict) -> str:
    text = PAIR_KERNEL_HEAD + PAIR_KERNEL_MAINLOOP + PAIR_KERNEL_EPILOGUE
    for key, value in substitutions.items():
        text = text.replace(f"@{key}@", str(value))
    return prelude + PAIR_PRELUDE + text
