// Tensor-core GEMM for sm_100a, wide 2-CTA form: a pair of CTAs computes a 512 x 256
// tile of C; each CTA owns 256 rows of it as TWO 128 x 256 accumulators that together fill its
// tensor memory (512 columns).
//
// Why this shape.  Measured on B200 with the narrower kernels of this library:
//   * a CTA that computes 128 x 256 per K block must pull 48 KB through the L2 -> shared-memory
//     path every 512 tensor cycles; with four stages of shared memory the loads in flight do
//     not cover that path's latency (about 1.3 microseconds) and the MMA thread waits for data
//     about a fifth of the time;
//   * paired MMAs that all accumulate into ONE accumulator cost about 165 cycles each instead
//     of 128; alternated between TWO accumulators they run at 129 cycles each.
// Here a K block of 48 KB per CTA (256 rows of A, half of the 256-row B block) feeds 1024
// tensor cycles: half the fill rate, twice the latency tolerance, and the single issuing thread
// alternates between the two accumulators.  The price: both accumulators fill tensor memory, so
// the epilogue of a tile cannot overlap the next tile's MMAs on the same accumulator; it is
// kept short (eight warps, coalesced stores) and accumulator 0 is released as soon as it is
// drained, so the next tile starts on it while accumulator 1 drains.
//
// Roles per CTA (320 threads); the loops run on whole warps, one elected lane issues:
//   warp 0      producer: TMA loads of A (one 256-row box) and this rank's half of B,
//               completing on the full barrier of rank 0
//   warp 1      allocates tensor memory; on rank 0 issues the paired MMAs: per K block four on
//               accumulator 0 (rows 0..127 of each CTA), four on accumulator 1 (rows 128..255),
//               then one commit delivered to empty[stage] of both ranks
//   warps 2..9  epilogue: two warps per TMEM lane quarter, each draining half of the columns,
//               accumulator 0 then accumulator 1
// Every wait is bounded; both CTAs of a pair meet at a cluster barrier before tensor memory is
// freed.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "umma_common.cuh"

namespace o64 {

constexpr int kWaitWideProducerEmpty = 0x301;
constexpr int kWaitWideMmaFull = 0x302;
constexpr int kWaitWideMmaAccEmpty = 0x303;
constexpr int kWaitWideEpiAccFull = 0x304;
constexpr int kWideTmemMismatch = 0x305;

constexpr int kWideThreads = 320;  // producer, MMA, eight epilogue warps
constexpr int kWideEpiWarps = 8;
constexpr int kWideBlockN = 256;
constexpr int kWideStages = 4;
constexpr int kWideRowsPerCta = 256;
constexpr int kWideABytes = kWideRowsPerCta * kRowBytes;      // 32 KB
constexpr int kWideBBytes = (kWideBlockN / 2) * kRowBytes;    // 16 KB: this rank's half of B
constexpr int kWideStageBytes = kWideABytes + kWideBBytes;    // 48 KB

struct WideSmem {
    static constexpr int kRingBytes = kWideStages * kWideStageBytes;
    static constexpr int kStagingOffset = kRingBytes;
    static constexpr int kBarOffset = kStagingOffset + kWideEpiWarps * kEpiStagingBytesPerWarp;
    // full[S], empty[S], acc_full[2], acc_empty[2]
    static constexpr int kNumBars = 2 * kWideStages + 4;
    static constexpr int kTmemPtrOffset = kBarOffset + 8 * kNumBars;
    static constexpr int kAbortOffset = kTmemPtrOffset + 4;
    static constexpr int kXchgReadyOffset = kAbortOffset + 4;  // fused exchange: "all ranks have arrived"
    static constexpr int kTotal = kXchgReadyOffset + 4;
    static constexpr int kDynamic = kTotal + 1024;
};

template <int KIND, bool B_KN, int EPI, bool HOOK = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kWideThreads, 1)
umma_gemm_wide_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                      const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ CUtensorMap tm_c,
                      const __grid_constant__ PeerMaps tm_peers,
                      const __grid_constant__ UmmaParams p) {
    using L = WideSmem;
    constexpr int STAGES = kWideStages;
    constexpr int BLOCK_N = kWideBlockN;
    constexpr int kElem = (KIND == MMA_F16) ? 2 : 1;
    constexpr int kBlockK = kRowBytes / kElem;
    constexpr int kMmaPerStage = 4;
    constexpr int kHalfN = BLOCK_N / 2;
    constexpr int kOutN = (EPI == EPI_SWIGLU) ? BLOCK_N / 2 : BLOCK_N;
    constexpr int kPairM = 2 * kWideRowsPerCta;  // 512
    constexpr uint32_t kTmemCols = 512;
    static_assert(!B_KN || KIND == MMA_F16, "[K,N] operands are supported for bf16 only");
    static_assert(EPI != EPI_SWIGLU || B_KN, "SwiGLU weights are [K,N]");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + L::kBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int g) { return bar_base + 8u * (2 * STAGES + g); };
    auto acc_empty_bar = [&](int g) { return bar_base + 8u * (2 * STAGES + 2 + g); };
    volatile uint32_t *tmem_ptr_smem =
        reinterpret_cast<volatile uint32_t *>(smem_gen + L::kTmemPtrOffset);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + L::kAbortOffset);
    volatile int *xchg_ready = reinterpret_cast<volatile int *>(smem_gen + L::kXchgReadyOffset);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair_id = (int)cluster_id_x();
    const int num_pairs = (int)num_clusters_x();
    const int num_tiles = p.num_m_tiles * p.num_n_tiles;  // num_m_tiles counts 512-row blocks

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);   // rank 0's arrive.expect_tx covers both CTAs' bytes
            mbar_init(empty_bar(s), 1);  // one commit per phase from rank 0's MMA thread
        }
        for (int g = 0; g < 2; ++g) {
            mbar_init(acc_full_bar(g), 1);
            mbar_init(acc_empty_bar(g), 2 * kWideEpiWarps);  // the epilogue warps of both CTAs
        }
        *abort_flag = 0;
        *xchg_ready = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        if (EPI == EPI_SWIGLU) tma_prefetch_desc(&tm_b2);
    }
    if (warp == 1) {
        // the whole tensor memory of this SM, from empty: both CTAs get base column 0
        tmem_alloc(smem_u32(smem_gen + L::kTmemPtrOffset), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;
    if (threadIdx.x == 0 && (tmem_base & 0xffffu) != 0) {
        atomicCAS(p.status, 0, kWideTmemMismatch);
        *abort_flag = 1;
    }
    if (p.xchg_local && blockIdx.x == 0 && threadIdx.x == 0) xchg_announce_entry(p);

    if (warp == 0) {
        // ------------------------------ TMA producer (both ranks) ---------------------------
        {
            const bool leader = elect_one();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long wait_clk = 0;
            [[maybe_unused]] int issued = 0;  // K blocks this producer has dealt with (test hook)
            const long long t_begin = clock64();
            WorkItem w;
            for (int item = 0; ok && work_item<false>(p, pair_id, num_pairs, item, w); ++item) {
                int mb, nb;
                tile_coords(w.tile, p, mb, nb);
                const int m0 = mb * kPairM + (int)rank * kWideRowsPerCta;
                const int n0 = nb * kOutN;
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    const long long c0 = O64_DBG(p) ? clock64() : 0;
                    ok = mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, p.status,
                                           kWaitWideProducerEmpty, p.wait_ns);
                    ok = __all_sync(0xffffffffu, ok);
                    if (O64_DBG(p)) wait_clk += clock64() - c0;
                    if (!ok) break;
                    const uint32_t a_dst = smem_base + stage * kWideStageBytes;
                    const uint32_t b_dst = a_dst + kWideABytes;
                    const uint32_t full0 = map_to_cta(full_bar(stage), 0);
                    bool withhold = false;  // both CTAs count alike, so both leave the same K block out
                    if constexpr (HOOK) withhold = (issued++ == p.test_withhold);
                    if ((O64_PROBE(p) & 3) == 1) {
                        if (rank == 0 && leader) mbar_arrive(full_bar(stage));
                    } else if (leader && !withhold) {
                        if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * kWideStageBytes);
                        tma_load_2d_pair(a_dst, &tm_a, kb * kBlockK, m0, full0);
                        if constexpr (!B_KN) {
                            tma_load_2d_pair(b_dst, &tm_b, kb * kBlockK, n0 + (int)rank * kHalfN, full0);
                        } else if constexpr (EPI == EPI_SWIGLU) {
                            // rank 0 holds the gate columns, rank 1 the up columns of the same n0
#pragma unroll
                            for (int g = 0; g < kHalfN / 64; ++g)
                                tma_load_2d_pair(b_dst + g * 8192, rank ? &tm_b2 : &tm_b, n0 + g * 64,
                                                 kb * kBlockK, full0);
                        } else {
#pragma unroll
                            for (int g = 0; g < kHalfN / 64; ++g)
                                tma_load_2d_pair(b_dst + g * 8192, &tm_b,
                                                 n0 + (int)rank * kHalfN + g * 64, kb * kBlockK, full0);
                        }
                    }
                    __syncwarp();
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (O64_DBG(p) && leader) {
                O64_DBG(p)[blockIdx.x * 8 + 2] = wait_clk;
                O64_DBG(p)[blockIdx.x * 8 + 3] = clock64() - t_begin;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (rank 0 only) ----------------------------
        if (rank == 0) {
            const bool leader = elect_one();
            constexpr uint32_t d_fmt = (KIND == MMA_I8) ? 2u : 1u;
            constexpr uint32_t ab_fmt = (KIND == MMA_F8F6F4) ? 0u : 1u;
            constexpr uint32_t idesc = make_idesc(d_fmt, ab_fmt, ab_fmt, B_KN ? 1u : 0u, 256, BLOCK_N);
            constexpr uint32_t kBAdvance = B_KN ? (16 * kRowBytes) >> 4 : 32 >> 4;
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            long long wait_clk = 0, acc_wait_clk = 0;
            const long long t_begin = clock64();
            uint32_t ready = mbar_test_wait(full_bar(0), 0);
            WorkItem w;
            for (; ok && work_item<false>(p, pair_id, num_pairs, it, w); ++it) {
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    if (!__all_sync(0xffffffffu, ready)) {
                        const long long c0 = O64_DBG(p) ? clock64() : 0;
                        ok = mbar_wait_bounded(full_bar(stage), phase, abort_flag, p.status, kWaitWideMmaFull, p.wait_ns);
                        ok = __all_sync(0xffffffffu, ok);
                        if (O64_DBG(p)) wait_clk += clock64() - c0;
                        if (!ok) break;
                    }
                    const int next_stage = (stage + 1 == STAGES) ? 0 : stage + 1;
                    const uint32_t next_phase = (stage + 1 == STAGES) ? (phase ^ 1u) : phase;
                    const uint32_t next_ready = mbar_test_wait(full_bar(next_stage), next_phase);
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + stage * kWideStageBytes;
                    const uint32_t b_addr = a_addr + kWideABytes;
                    const uint64_t a_desc0 = make_smem_desc(a_addr, 16, 1024);
                    const uint64_t a_desc1 = make_smem_desc(a_addr + kABytes, 16, 1024);
                    const uint64_t b_desc =
                        B_KN ? make_smem_desc(b_addr, 8192, 1024) : make_smem_desc(b_addr, 16, 1024);
                    if ((O64_PROBE(p) & 3) == 2) {
                        if (leader) {
                            mbar_arrive(empty_bar(stage));
                            mbar_arrive_cluster(map_to_cta(empty_bar(stage), 1));
                        }
                    } else {
                        if (kb == w.kb0) {
                            // the first MMA of a tile overwrites the accumulator: wait until the
                            // epilogue has drained it (accumulator 1 is drained second)
                            const long long a0 = O64_DBG(p) ? clock64() : 0;
                            ok = mbar_wait_bounded(acc_empty_bar(0), (it & 1u) ^ 1u, abort_flag, p.status,
                                                   kWaitWideMmaAccEmpty, p.wait_ns);
                            if (O64_DBG(p)) acc_wait_clk += clock64() - a0;
                            ok = __all_sync(0xffffffffu, ok);
                            if (!ok) break;
                            tc_fence_after();
                        }
                        {
                            if (leader) {
#pragma unroll
                                for (int k = 0; k < kMmaPerStage; ++k)
                                    tc_mma_pair<KIND>(tmem_base, a_desc0 + 2u * k, b_desc + kBAdvance * k, idesc,
                                                      ((kb - w.kb0) | k) != 0 ? 1u : 0u);
                            }
                            if (kb == w.kb0) {
                                __syncwarp();
                                const long long a1 = O64_DBG(p) ? clock64() : 0;
                                ok = mbar_wait_bounded(acc_empty_bar(1), (it & 1u) ^ 1u, abort_flag, p.status,
                                                       kWaitWideMmaAccEmpty, p.wait_ns);
                                if (O64_DBG(p)) acc_wait_clk += clock64() - a1;
                                ok = __all_sync(0xffffffffu, ok);
                                if (!ok) break;
                                tc_fence_after();
                            }
                            if (leader) {
#pragma unroll
                                for (int k = 0; k < kMmaPerStage; ++k)
                                    tc_mma_pair<KIND>(tmem_base + BLOCK_N, a_desc1 + 2u * k, b_desc + kBAdvance * k,
                                                      idesc, ((kb - w.kb0) | k) != 0 ? 1u : 0u);
                            }
                        }
                        if (leader) tc_commit_pair_mask(empty_bar(stage), 3);
                    }
                    __syncwarp();
                    stage = next_stage;
                    phase = next_phase;
                    ready = next_ready;
                }
                if (ok && leader) {
                    tc_commit_pair_mask(acc_full_bar(0), 3);
                    tc_commit_pair_mask(acc_full_bar(1), 3);
                }
                __syncwarp();
            }
            if (O64_DBG(p) && leader) {
                O64_DBG(p)[blockIdx.x * 8 + 0] = wait_clk;
                O64_DBG(p)[blockIdx.x * 8 + 5] = acc_wait_clk;
                O64_DBG(p)[blockIdx.x * 8 + 1] = clock64() - t_begin;
            }
        }
        __syncwarp();
    } else if (warp >= 2) {
        // ------------------------------ epilogue (both ranks) -------------------------------
        // two warps per TMEM lane quarter, each draining half of the columns
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        constexpr int kColsPerWarp = kOutN / 2;
        int it = 0;
        bool ok = true;
        long long epi_clk = 0;
        WorkItem w;
        if (p.xchg_local) ok = xchg_wait_entry(p, abort_flag, xchg_ready, warp == 2);  // no remote store before every rank is here
        for (; ok && work_item<false>(p, pair_id, num_pairs, it, w); ++it) {
            int mb, nb;
            tile_coords(w.tile, p, mb, nb);
#pragma unroll 1
            for (int g = 0; g < 2 && ok; ++g) {
                if (lane == 0)
                    ok = mbar_wait_bounded(acc_full_bar(g), it & 1u, abort_flag, p.status, kWaitWideEpiAccFull, p.wait_ns);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                tc_fence_after();
                const long long row0 = (long long)mb * kPairM + (long long)rank * kWideRowsPerCta +
                                       g * kBlockM + quarter * 32;
                const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + g * BLOCK_N;
                const long long e0 = O64_DBG(p) ? clock64() : 0;
                if (!(O64_PROBE(p) & 4)) {
                    epilogue_tile<EPI, BLOCK_N>(p, row0, nb * kOutN, t_row,
                                                smem_gen + L::kStagingOffset + (warp - 2) * kEpiStagingBytesPerWarp,
                                                half * kColsPerWarp, (half + 1) * kColsPerWarp, p.tma_store ? &tm_c : nullptr, (p.tma_store && p.n_peers > 0) ? &tm_peers : nullptr);
                }
                tc_fence_before();
                __syncwarp();
                if (O64_DBG(p)) epi_clk += clock64() - e0;
                if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty_bar(g), 0));
            }
        }
        if (p.tma_store && lane == 0) bulk_wait_all();  // this lane's bulk stores are complete before the CTA leaves
        if (p.xchg_local) xchg_stores_done();
        if (O64_DBG(p) && warp == 2 && lane == 0) O64_DBG(p)[blockIdx.x * 8 + 4] = epi_clk;
    }

    // ------------------------------ teardown --------------------------------------------
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (p.xchg_local && threadIdx.x == 0) xchg_finish(p, abort_flag);
    if (warp == 1) {
        if (*abort_flag) {
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int KIND, bool B_KN, int EPI, bool HOOK = false>
static int launch_wide_inst(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tb2, const CUtensorMap &tc,
                            const PeerMaps &tp, const UmmaParams &p, int grid, cudaStream_t stream) {
    auto kern = umma_gemm_wide_kernel<KIND, B_KN, EPI, HOOK>;
    static KernelSetup ks;  // per instantiation; one set-up per device
    int max_pairs = 0;
    const int rc = ks.once(
        [&](int *clusters) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WideSmem::kDynamic) !=
                cudaSuccess)
                return (int)O64_ERR_CUDA;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2, 1, 1);
            cfg.blockDim = dim3(kWideThreads, 1, 1);
            cfg.dynamicSmemBytes = WideSmem::kDynamic;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = 2;
            at[0].val.clusterDim.y = 1;
            at[0].val.clusterDim.z = 1;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
                (void)cudaGetLastError();
                n = 0;
            }
            *clusters = n;
            return (int)O64_OK;
        },
        &max_pairs);
    if (rc) return rc;
    if (max_pairs > 0 && grid > 2 * max_pairs) grid = 2 * max_pairs;
    kern<<<grid, kWideThreads, WideSmem::kDynamic, stream>>>(ta, tb, tb2, tc, tp, p);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

// `p.num_m_tiles` counts 512-row blocks; tile_n is 256.
int umma_launch_wide(const UmmaCall &c, const CUtensorMap &ta, const CUtensorMap &tb,
                     const CUtensorMap &tb2, const UmmaParams &p_in) {
    // full slabs of the result leave by TMA store when C's rows allow it
    UmmaParams p = p_in;
    CUtensorMap tc = ta;
    static const bool tma_store_off = [] { const char *e = getenv("O64_TMA_STORE"); return e && atoi(e) == 0; }();
    static PeerMaps tp_init;  // zero-initialised; entries beyond n_peers are never read
    PeerMaps tp = tp_init;
    bool bulk = !tma_store_off && p.vec_ok && encode_c_bytes(&tc, c.C, c.M, p.N, c.ldc, epi_out_bytes(c.epi)) == O64_OK;
    // the fused exchange: one more map per peer copy of the result
    for (int d = 0; d < p.n_peers && bulk; ++d)
        bulk = encode_c_bytes(&tp.m[d], p.peer_c[d], c.M, p.N, c.ldc, epi_out_bytes(c.epi)) == O64_OK;
    if (bulk)
        p.tma_store = 1;
    else
        tc = ta;
    const long long tiles = (long long)p.num_m_tiles * p.num_n_tiles;
    long long pairs = c.plan.num_ctas / 2;
    if (pairs > tiles) pairs = tiles;
    if (pairs < 1) pairs = 1;
    const int grid = (int)(2 * pairs);
    if (c.test_withhold >= 0) {  // the one instantiation with the test hook: bf16, B [N,K]
        if (c.kind != O64_KIND_BF16 || c.epi != EPI_BF16 || c.b_kn) return O64_ERR_DTYPE;
        return launch_wide_inst<MMA_F16, false, EPI_BF16, true>(ta, tb, tb2, tc, tp, p, grid, c.stream);
    }
    if (c.kind == O64_KIND_BF16) {
        if (c.epi == EPI_SWIGLU) return launch_wide_inst<MMA_F16, true, EPI_SWIGLU>(ta, tb, tb2, tc, tp, p, grid, c.stream);
        if (c.epi == EPI_BF16) {
            if (c.b_kn) return launch_wide_inst<MMA_F16, true, EPI_BF16>(ta, tb, tb2, tc, tp, p, grid, c.stream);
            return launch_wide_inst<MMA_F16, false, EPI_BF16>(ta, tb, tb2, tc, tp, p, grid, c.stream);
        }
    } else if (c.kind == O64_KIND_FP8 && c.epi == EPI_SCALED_BF16) {
        return launch_wide_inst<MMA_F8F6F4, false, EPI_SCALED_BF16>(ta, tb, tb2, tc, tp, p, grid, c.stream);
    } else if (c.kind == O64_KIND_S8 && c.epi == EPI_S32) {
        return launch_wide_inst<MMA_I8, false, EPI_S32>(ta, tb, tb2, tc, tp, p, grid, c.stream);
    }
    return O64_ERR_DTYPE;
}

}  // namespace o64
