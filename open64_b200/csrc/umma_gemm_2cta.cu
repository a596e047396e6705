// Tensor-core GEMM for sm_100a, 2-CTA form: a cluster of two CTAs (two SMs of one TPC)
// computes one 256 x BLOCK_N accumulator tile with tcgen05.mma.cta_group::2.
//
// Why pairs: in the 1-CTA kernel every SM pulls a 128-row A block and a whole BLOCK_N-row B
// block through the L2 -> shared-memory path for each K block.  Paired, each CTA loads its own
// 128 rows of A and only HALF of the B block; the tensor cores of both SMs read both halves.
// Shared-memory fill per CTA and K block drops from 48 KB to 32 KB (BLOCK_N = 256), which
// also buys a deeper ring (6 stages instead of 4).
//
// Division of labour inside a pair (rank = %cluster_ctarank):
//   both ranks   producer warp: TMA loads of A[128 rows of this rank] and B[half of this rank],
//                completing on the full barrier OF RANK 0
//                epilogue warps: drain this rank's 128 accumulator rows (its own tensor memory)
//   rank 0 only  MMA warp: waits for full[stage] (bytes of both ranks), issues the paired
//                MMAs, then one commit that arrives on empty[stage] (and, per tile, on
//                acc_full[buf]) of BOTH ranks
// acc_empty[buf] lives in rank 0 and counts the epilogue warps of both ranks.
//
// No load is shared between CTAs: every TMA load writes the issuing CTA's own shared memory.
// Every wait is bounded; on expiry a CTA records a code in the status word and leaves its
// role loops; both CTAs of a pair meet at a cluster barrier before they free tensor memory.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "umma_common.cuh"

namespace o64 {

constexpr int kWaitPairProducerEmpty = 0x201;
constexpr int kWaitPairMmaFull = 0x202;
constexpr int kWaitPairMmaAccEmpty = 0x203;
constexpr int kWaitPairEpiAccFull = 0x204;
constexpr int kPairTmemMismatch = 0x205;

template <int BLOCK_N, int STAGES>
struct PairSmemLayout {
    static constexpr int kBBytes = (BLOCK_N / 2) * kRowBytes;  // this CTA's half of B
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kRingBytes = STAGES * kStageBytes;
    static constexpr int kStagingOffset = kRingBytes;
    static constexpr int kBarOffset = kStagingOffset + kEpiStagingBytes;
    static constexpr int kNumBars = 2 * STAGES + 4;
    static constexpr int kTmemPtrOffset = kBarOffset + 8 * kNumBars;
    static constexpr int kAbortOffset = kTmemPtrOffset + 4;
    static constexpr int kXchgReadyOffset = kAbortOffset + 4;  // fused exchange: "all ranks have arrived"
    static constexpr int kTotal = kXchgReadyOffset + 4;
    static constexpr int kDynamic = kTotal + 1024;
};

template <int KIND, bool B_KN, int EPI, int BLOCK_N, int STAGES, bool HOOK = false, bool TAIL = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
umma_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                      const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ CUtensorMap tm_c,
                      const __grid_constant__ PeerMaps tm_peers,
                      const __grid_constant__ UmmaParams p) {
    using L = PairSmemLayout<BLOCK_N, STAGES>;
    constexpr int kElem = (KIND == MMA_F16) ? 2 : 1;
    constexpr int kBlockK = kRowBytes / kElem;
    constexpr int kMmaPerStage = 4;
    constexpr int kHalfN = BLOCK_N / 2;  // B rows (N) held by each CTA
    // a [K,N] operand (N contiguous) lands in shared memory as groups of 128 bytes of N (64 bf16 or 128
    // one-byte columns) by kBlockK rows of K each; an MMA consumes 32 bytes of K: 16 bf16 or 32 e4m3 rows
    constexpr int kKnCols = kRowBytes / kElem;
    constexpr int kKnGroupBytes = kBlockK * kRowBytes;
    constexpr int kMmaK = 32 / kElem;
    static_assert(!B_KN || kHalfN % kKnCols == 0, "[K,N] operand: each CTA's columns must be whole 128-byte groups");
    constexpr int kOutN = (EPI == EPI_SWIGLU) ? BLOCK_N / 2 : BLOCK_N;
    constexpr int kPairM = 2 * kBlockM;
    constexpr uint32_t kTmemCols = 2 * BLOCK_N;
    static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns");
    static_assert(!B_KN || KIND == MMA_F16 || KIND == MMA_F8F6F4, "[K,N] operands: bf16 and e4m3");
    static_assert(EPI != EPI_SWIGLU || B_KN, "SwiGLU weights are [K,N]");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + L::kBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
    volatile uint32_t *tmem_ptr_smem =
        reinterpret_cast<volatile uint32_t *>(smem_gen + L::kTmemPtrOffset);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + L::kAbortOffset);
    volatile int *xchg_ready = reinterpret_cast<volatile int *>(smem_gen + L::kXchgReadyOffset);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = issues the MMAs
    const int pair_id = (int)cluster_id_x();
    const int num_pairs = (int)num_clusters_x();
    const int num_tiles = p.num_m_tiles * p.num_n_tiles;  // num_m_tiles counts 256-row blocks

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);   // rank 0: one arrive.expect_tx covering both CTAs' bytes
            mbar_init(empty_bar(s), 1);  // one commit per phase, from rank 0's MMA thread
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), 8);  // four epilogue warps in each of the two CTAs
        }
        *abort_flag = 0;
        *xchg_ready = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        if (EPI == EPI_SWIGLU) tma_prefetch_desc(&tm_b2);
    }
    if (warp == 1) {
        // each CTA takes all the columns it needs from its own, otherwise empty, tensor memory:
        // both CTAs of the pair therefore get the same base address, which the paired MMA needs
        tmem_alloc(smem_u32(smem_gen + L::kTmemPtrOffset), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the partner's barriers are initialised before anything remote happens
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;
    if (threadIdx.x == 0 && (tmem_base & 0xffffu) != 0) {
        atomicCAS(p.status, 0, kPairTmemMismatch | (int)((tmem_base & 0xfffu) << 12) | (int)(rank << 24));
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
            for (int item = 0; ok && work_item<TAIL>(p, pair_id, num_pairs, item, w); ++item) {
                int mb, nb;
                tile_coords(w.tile, p, mb, nb);
                const int m0 = mb * kPairM + (int)rank * kBlockM;
                const int n0 = nb * kOutN;
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    const long long c0 = O64_DBG(p) ? clock64() : 0;
                    ok = mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, p.status,
                                           kWaitPairProducerEmpty, p.wait_ns);
                    ok = __all_sync(0xffffffffu, ok);
                    if (O64_DBG(p)) wait_clk += clock64() - c0;
                    if (!ok) break;
                    const uint32_t a_dst = smem_base + stage * L::kStageBytes;
                    const uint32_t b_dst = a_dst + kABytes;
                    const uint32_t full0 = map_to_cta(full_bar(stage), 0);
                    bool withhold = false;  // both CTAs count alike, so both leave the same K block out
                    if constexpr (HOOK) withhold = (issued++ == p.test_withhold);
                    if ((O64_PROBE(p) & 3) == 1) {
                        if (rank == 0 && leader) mbar_arrive(full_bar(stage));
                    } else if (leader && !withhold) {
                        if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * L::kStageBytes);
                        tma_load_2d_pair(a_dst, &tm_a, kb * kBlockK, m0, full0);
                        if constexpr (!B_KN) {
                            tma_load_2d_pair(b_dst, &tm_b, kb * kBlockK, n0 + (int)rank * kHalfN, full0);
                        } else if constexpr (EPI == EPI_SWIGLU) {
                            // rank 0 holds the gate columns, rank 1 the up columns of the same n0
                            constexpr int kGroups = kHalfN / kKnCols;
#pragma unroll
                            for (int g = 0; g < kGroups; ++g)
                                tma_load_2d_pair(b_dst + g * kKnGroupBytes, rank ? &tm_b2 : &tm_b, n0 + g * kKnCols,
                                                 kb * kBlockK, full0);
                        } else {
                            constexpr int kGroups = kHalfN / kKnCols;
#pragma unroll
                            for (int g = 0; g < kGroups; ++g)
                                tma_load_2d_pair(b_dst + g * kKnGroupBytes, &tm_b, n0 + (int)rank * kHalfN + g * kKnCols,
                                                 kb * kBlockK, full0);
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
            constexpr uint32_t idesc = make_idesc(d_fmt, ab_fmt, ab_fmt, B_KN ? 1u : 0u, kPairM, BLOCK_N);
            constexpr uint32_t kBAdvance = B_KN ? (kMmaK * kRowBytes) >> 4 : 32 >> 4;
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            long long wait_clk = 0;
            const long long t_begin = clock64();
            uint32_t ready = mbar_test_wait(full_bar(0), 0);  // see the 1-CTA kernel: probe ahead
            WorkItem w;
            for (; ok && work_item<TAIL>(p, pair_id, num_pairs, it, w); ++it) {
                const int buf = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1u;
                ok = mbar_wait_bounded(acc_empty_bar(buf), acc_phase ^ 1u, abort_flag, p.status,
                                       kWaitPairMmaAccEmpty, p.wait_ns);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BLOCK_N;
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    if (!__all_sync(0xffffffffu, ready)) {
                        const long long c0 = O64_DBG(p) ? clock64() : 0;
                        ok = mbar_wait_bounded(full_bar(stage), phase, abort_flag, p.status, kWaitPairMmaFull, p.wait_ns);
                        ok = __all_sync(0xffffffffu, ok);
                        if (O64_DBG(p)) wait_clk += clock64() - c0;
                        if (!ok) break;
                    }
                    const int next_stage = (stage + 1 == STAGES) ? 0 : stage + 1;
                    const uint32_t next_phase = (stage + 1 == STAGES) ? (phase ^ 1u) : phase;
                    const uint32_t next_ready = mbar_test_wait(full_bar(next_stage), next_phase);
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + stage * L::kStageBytes;
                    const uint32_t b_addr = a_addr + kABytes;
                    const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024);
                    const uint64_t b_desc =
                        B_KN ? make_smem_desc(b_addr, kKnGroupBytes, 1024) : make_smem_desc(b_addr, 16, 1024);
                    if ((O64_PROBE(p) & 3) == 2) {
                        if (leader) {
                            mbar_arrive(empty_bar(stage));
                            mbar_arrive_cluster(map_to_cta(empty_bar(stage), 1));
                        }
                    } else if (leader) {
#pragma unroll
                        for (int k = 0; k < kMmaPerStage; ++k) {
                            tc_mma_pair<KIND>(d_tmem, a_desc + 2u * k, b_desc + kBAdvance * k, idesc,
                                              ((kb - w.kb0) | k) != 0 ? 1u : 0u);
                        }
                        // frees the stage in both CTAs when these MMAs retire: one commit delivered
                        // to the same barrier of both ranks
                        tc_commit_pair_mask(empty_bar(stage), 3);
                    }
                    __syncwarp();
                    stage = next_stage;
                    phase = next_phase;
                    ready = next_ready;
                }
                if (ok && leader) tc_commit_pair_mask(acc_full_bar(buf), 3);
                __syncwarp();
            }
            if (O64_DBG(p) && leader) {
                O64_DBG(p)[blockIdx.x * 8 + 0] = wait_clk;
                O64_DBG(p)[blockIdx.x * 8 + 1] = clock64() - t_begin;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue (both ranks) -------------------------------
        const int quarter = warp & 3;
        int it = 0;
        bool ok = true;
        WorkItem w;
        long long clk_store = 0, clk_flags = 0, clk_fix = 0, clk_accwait = 0;  // O64_TRACE=pipe
        const long long t_begin = clock64();
        if (p.xchg_local) ok = xchg_wait_entry(p, abort_flag, xchg_ready, warp == 2);  // no remote store before every rank is here
        for (; ok && work_item<TAIL>(p, pair_id, num_pairs, it, w); ++it) {
            int mb, nb;
            tile_coords(w.tile, p, mb, nb);
            const int buf = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1u;
            const long long w0 = O64_DBG(p) ? clock64() : 0;
            if (lane == 0)
                ok = mbar_wait_bounded(acc_full_bar(buf), acc_phase, abort_flag, p.status, kWaitPairEpiAccFull, p.wait_ns);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            if (O64_DBG(p)) clk_accwait += clock64() - w0;
            const long long row0 = (long long)mb * kPairM + (long long)rank * kBlockM + quarter * 32;
            const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + buf * BLOCK_N;
            const long long e0 = O64_DBG(p) ? clock64() : 0;
            if (TAIL && w.mode == WORK_PARTIAL_OUT) {
                // this pair stops short of the tile's last K block: the raw sums go to its slot
                tail_store_partial(t_row, tail_unit<BLOCK_N>(p, pair_id, (int)rank, 4, quarter), 0, BLOCK_N);
                tail_publish(tail_flag(p, pair_id, (int)rank, quarter));
                if (O64_DBG(p)) clk_store += clock64() - e0;
            } else if (!(O64_PROBE(p) & 4)) {
                if (TAIL && w.mode == WORK_FIXUP_IN) {
                    TailFix fix;
                    // the tile's earlier K blocks were multiplied by the pairs before this one
                    const int first = tail_first_contributor(p, pair_id, w.tile);
                    for (int q = first; q < pair_id && ok; ++q)
                        ok = tail_wait_flag(tail_flag(p, q, (int)rank, quarter), abort_flag, p.status, p.wait_ns);
                    if (!ok) break;
                    fix.first_unit = reinterpret_cast<const uint8_t *>(tail_unit<BLOCK_N>(p, first, (int)rank, 4, quarter));
                    fix.stride = p.tail_slot_bytes;
                    fix.n = pair_id - first;
                    if (O64_DBG(p)) clk_flags += clock64() - e0;
                    tail_complete<EPI, BLOCK_N>(t_row, 0, kOutN, fix);
                    for (int q = first; q < pair_id; ++q) tail_release(tail_flag(p, q, (int)rank, quarter), 1);
                }
                const long long f0 = O64_DBG(p) ? clock64() : 0;
                epilogue_tile<EPI, BLOCK_N>(p, row0, nb * kOutN, t_row,
                                            smem_gen + L::kStagingOffset + quarter * kEpiStagingBytesPerWarp, 0, kOutN,
                                            p.tma_store ? &tm_c : nullptr, (p.tma_store && p.n_peers > 0) ? &tm_peers : nullptr);
                if (O64_DBG(p)) clk_fix += clock64() - f0;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty_bar(buf), 0));
        }
        if (p.tma_store && lane == 0) bulk_wait_all();  // this lane's bulk stores are complete before the CTA leaves
        if (p.xchg_local) xchg_stores_done();
        if (O64_DBG(p) && warp == 2 && lane == 0) {
            O64_DBG(p)[blockIdx.x * 8 + 4] = clk_fix;                 // epilogues (owned tiles)
            O64_DBG(p)[blockIdx.x * 8 + 5] = clk_flags;               // waiting for contributors
            O64_DBG(p)[blockIdx.x * 8 + 6] = clk_store;               // partial sums stored and published
            O64_DBG(p)[blockIdx.x * 8 + 7] = clock64() - t_begin;     // epilogue warp's whole loop
        }
    }

    // ------------------------------ teardown --------------------------------------------
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while its partner may
                         // still read its shared memory or signal its barriers
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

template <int KIND, bool B_KN, int EPI, int BLOCK_N, int STAGES, bool HOOK = false>
static int launch_pair_inst(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tb2, const CUtensorMap &tc,
                            const PeerMaps &tp, const UmmaParams &p, int grid, cudaStream_t stream) {
    using L = PairSmemLayout<BLOCK_N, STAGES>;
    auto kern = umma_gemm_pair_kernel<KIND, B_KN, EPI, BLOCK_N, STAGES, HOOK>;
    static KernelSetup ks;  // per instantiation; one set-up per device
    int max_pairs = 0;      // pairs the device can hold at once (the tile walk assumes co-residency)
    const int rc = ks.once(
        [&](int *clusters) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) != cudaSuccess)
                return (int)O64_ERR_CUDA;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2, 1, 1);
            cfg.blockDim = dim3(kThreads, 1, 1);
            cfg.dynamicSmemBytes = L::kDynamic;
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
            const char *tr = getenv("O64_TRACE");
            if (tr && strstr(tr, "plan")) fprintf(stderr, "[o64 pair kernel: %d CTA pairs can be resident]\n", n);
            return (int)O64_OK;
        },
        &max_pairs);
    if (rc) return rc;
    if (max_pairs > 0 && grid > 2 * max_pairs) grid = 2 * max_pairs;
    if constexpr (!HOOK) {
        UmmaParams q = p;
        long long cap = q.tail_slot_bytes;  // the capacity, as umma_launch left it
        // all pairs of the grid must be resident at once for one to wait for another's piece
        if (grid / 2 > kTailMaxPairs || max_pairs <= 0) cap = 0;
        plan_tail(q, grid / 2, 2LL * 4 * 32 * BLOCK_N * 4, cap);
        if (q.tail_tiles > 0) {
            // the instantiation that carries the K split of the last wave (its own set-up per device)
            auto kern_tail = umma_gemm_pair_kernel<KIND, B_KN, EPI, BLOCK_N, STAGES, false, true>;
            static KernelSetup ks_tail;
            const int rc_tail = ks_tail.once(
                [&](int *) {
                    return cudaFuncSetAttribute(kern_tail, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) ==
                                   cudaSuccess
                               ? (int)O64_OK
                               : (int)O64_ERR_CUDA;
                },
                nullptr);
            if (rc_tail) return rc_tail;
            kern_tail<<<grid, kThreads, L::kDynamic, stream>>>(ta, tb, tb2, tc, tp, q);
            return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
        }
        // whole tiles only: no more pairs than tiles
        const long long tiles = (long long)p.num_m_tiles * p.num_n_tiles;
        if (grid / 2 > tiles) grid = (int)(2 * tiles);
    }
    kern<<<grid, kThreads, L::kDynamic, stream>>>(ta, tb, tb2, tc, tp, p);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

// `p.num_m_tiles` counts 256-row blocks here; the grid is an even number of CTAs.
int umma_launch_pair(const UmmaCall &c, const CUtensorMap &ta, const CUtensorMap &tb,
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
    // with memory for a K split even fewer tiles than pairs can keep every pair busy
    if (pairs > tiles && !(p.tail_slots && p.tail_flags)) pairs = tiles;
    if (pairs < 1) pairs = 1;
    const int grid = (int)(2 * pairs);
    const int block_n = c.plan.tile_n;

#define O64_PAIR(KIND, BKN, EPI_, BN, ST) \
    return launch_pair_inst<KIND, BKN, EPI_, BN, ST>(ta, tb, tb2, tc, tp, p, grid, c.stream)

    if (c.test_withhold >= 0) {  // the one instantiation with the test hook: bf16, B [N,K], 256 x 256 tiles
        if (c.kind != O64_KIND_BF16 || c.epi != EPI_BF16 || c.b_kn || block_n != 256) return O64_ERR_DTYPE;
        return launch_pair_inst<MMA_F16, false, EPI_BF16, 256, 6, true>(ta, tb, tb2, tc, tp, p, grid, c.stream);
    }
    if (c.kind == O64_KIND_BF16) {
        if (c.epi == EPI_SWIGLU) {
            if (block_n == 256) O64_PAIR(MMA_F16, true, EPI_SWIGLU, 256, 6);
        } else if (c.epi == EPI_BF16) {
            if (c.b_kn) {
                if (block_n == 256) O64_PAIR(MMA_F16, true, EPI_BF16, 256, 6);
                if (block_n == 128) O64_PAIR(MMA_F16, true, EPI_BF16, 128, 8);
            } else {
                if (block_n == 256) O64_PAIR(MMA_F16, false, EPI_BF16, 256, 6);
                if (block_n == 128) O64_PAIR(MMA_F16, false, EPI_BF16, 128, 8);
            }
        }
    } else if (c.kind == O64_KIND_FP8 && c.b_kn) {  // e4m3 weight stored [K,N]: 256-column tiles only
        if (block_n == 256 && c.epi == EPI_SCALED_BF16) O64_PAIR(MMA_F8F6F4, true, EPI_SCALED_BF16, 256, 6);
        if (block_n == 256 && c.epi == EPI_SCALED_E4M3) O64_PAIR(MMA_F8F6F4, true, EPI_SCALED_E4M3, 256, 6);
    } else if (c.kind == O64_KIND_FP8 && c.epi == EPI_SCALED_BF16) {
        if (block_n == 256) O64_PAIR(MMA_F8F6F4, false, EPI_SCALED_BF16, 256, 6);
        if (block_n == 128) O64_PAIR(MMA_F8F6F4, false, EPI_SCALED_BF16, 128, 8);
    } else if (c.kind == O64_KIND_S8 && c.epi == EPI_S32) {
        if (block_n == 256) O64_PAIR(MMA_I8, false, EPI_S32, 256, 6);
        if (block_n == 128) O64_PAIR(MMA_I8, false, EPI_S32, 128, 8);
    } else if (c.kind == O64_KIND_FP8 && c.epi == EPI_SCALED_E4M3) {
        if (block_n == 256) O64_PAIR(MMA_F8F6F4, false, EPI_SCALED_E4M3, 256, 6);
        if (block_n == 128) O64_PAIR(MMA_F8F6F4, false, EPI_SCALED_E4M3, 128, 8);
    } else if (c.kind == O64_KIND_S8 && c.epi == EPI_ISCALED_BF16) {
        if (block_n == 256) O64_PAIR(MMA_I8, false, EPI_ISCALED_BF16, 256, 6);
        if (block_n == 128) O64_PAIR(MMA_I8, false, EPI_ISCALED_BF16, 128, 8);
    } else if (c.kind == O64_KIND_S8 && c.epi == EPI_ISCALED_S8) {
        if (block_n == 256) O64_PAIR(MMA_I8, false, EPI_ISCALED_S8, 256, 6);
        if (block_n == 128) O64_PAIR(MMA_I8, false, EPI_ISCALED_S8, 128, 8);
    }
#undef O64_PAIR
    return O64_ERR_DTYPE;
}

}  // namespace o64
