// Tensor-core GEMM for sm_100a: TMA -> multi-stage shared-memory ring -> tcgen05.mma with
// the accumulator in tensor memory -> fused epilogue.  One persistent CTA per SM walks a
// rasterised list of 128 x BLOCK_N output tiles.
//
// This kernel is the tiled form of the loop nest the reference compiler builds for MATMUL
// (osprey/be/vho/f90_lower.cxx:5149-5169): the K loop is the ring of shared-memory stages
// (the reference's L1 strip, osprey/be/lno/snl_inv.cxx:639-887), the register tile is one
// tcgen05.mma instruction (osprey/be/lno/snl_inv.cxx:904), software prefetch
// (osprey/be/lno/prefetch.cxx:679) is the TMA producer warp running ahead of the MMA warp.
//
// Warp roles (192 threads):
//   warp 0      producer: one lane issues the TMA loads of A and B for each K block
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma and the commits
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator, apply bias / activation /
//               scales, convert and store; overlaps the next tile's main loop because the
//               accumulator is double-buffered in tensor memory
//
// Every wait is bounded (mbar_wait_bounded): on expiry the CTA records a code in the status
// word, leaves all role loops, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>

#include "umma_common.cuh"

namespace o64 {

template <int BLOCK_N, int STAGES>
struct SmemLayout {
    static constexpr int kBBytes = BLOCK_N * kRowBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kRingBytes = STAGES * kStageBytes;
    // after the ring: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2] (8 bytes each),
    // the TMEM base address and the abort flag
    static constexpr int kStagingOffset = kRingBytes;  // epilogue patches, 4 KB per warp
    static constexpr int kBarOffset = kStagingOffset + kEpiStagingBytes;
    static constexpr int kNumBars = 2 * STAGES + 4;
    static constexpr int kTmemPtrOffset = kBarOffset + 8 * kNumBars;
    static constexpr int kAbortOffset = kTmemPtrOffset + 4;
    static constexpr int kXchgReadyOffset = kAbortOffset + 4;  // fused exchange: "all ranks have arrived"
    static constexpr int kTotal = kXchgReadyOffset + 4;
    static constexpr int kDynamic = kTotal + 1024;  // slack to align the ring to 1024 bytes
};

// KIND: MMA_F16 (bf16 operands) / MMA_F8F6F4 (e4m3) / MMA_I8 (s8).
// B_KN: B stored [K,N] (N contiguous) -> MN-major shared-memory descriptor; else [N,K].
template <int KIND, bool B_KN, int EPI, int BLOCK_N, int STAGES, bool HOOK = false>
__global__ void __launch_bounds__(kThreads, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ UmmaParams p) {
    using L = SmemLayout<BLOCK_N, STAGES>;
    constexpr int kElem = (KIND == MMA_F16) ? 2 : 1;
    constexpr int kBlockK = kRowBytes / kElem;  // K elements per stage
    constexpr int kMmaPerStage = 4;             // 32 bytes of K per tcgen05.mma
    constexpr int kOutN = (EPI == EPI_SWIGLU) ? BLOCK_N / 2 : BLOCK_N;
    constexpr uint32_t kTmemCols = 2 * BLOCK_N;  // two accumulator buffers
    static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns");
    static_assert(!B_KN || KIND == MMA_F16, "[K,N] operands are supported for bf16 only");
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
    const int num_tiles = p.num_m_tiles * p.num_n_tiles;
    const int num_work = num_tiles * p.split_k;  // a work item = (tile, slice of its K blocks)

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), 4);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        *xchg_ready = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        if (EPI == EPI_SWIGLU) tma_prefetch_desc(&tm_b2);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(smem_gen + L::kTmemPtrOffset), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;
    if (p.xchg_local && blockIdx.x == 0 && threadIdx.x == 0) xchg_announce_entry(p);

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------------
        {
            const bool leader = elect_one();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long wait_clk = 0;
            [[maybe_unused]] int issued = 0;  // K blocks this producer has dealt with (test hook)
            const long long t_begin = clock64();
            for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
                int mb, nb;
                tile_coords(w / p.split_k, p, mb, nb);
                const int m0 = mb * kBlockM;
                const int n0 = nb * kOutN;
                const int kb_begin = (w % p.split_k) * p.kb_per_split;
                const int kb_end = min(kb_begin + p.kb_per_split, p.num_k_blocks);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    const long long c0 = O64_DBG(p) ? clock64() : 0;
                    ok = mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, p.status,
                                           kWaitProducerEmpty, p.wait_ns);
                    ok = __all_sync(0xffffffffu, ok);
                    if (O64_DBG(p)) wait_clk += clock64() - c0;
                    if (!ok) break;
                    const uint32_t a_dst = smem_base + stage * L::kStageBytes;
                    const uint32_t b_dst = a_dst + kABytes;
                    bool withhold = false;
                    if constexpr (HOOK) withhold = (issued++ == p.test_withhold);
                    if ((O64_PROBE(p) & 3) == 1) {
                        if (leader) mbar_arrive(full_bar(stage));
                    } else if (leader && !withhold) {
                        mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
                        tma_load_2d(a_dst, &tm_a, kb * kBlockK, m0, full_bar(stage));
                        if constexpr (!B_KN) {
                            tma_load_2d(b_dst, &tm_b, kb * kBlockK, n0, full_bar(stage));
                        } else {
                            // [K,N] operand: boxes of 64 N-elements x 64 K-rows (8 KB each)
                            constexpr int kGroups = BLOCK_N / 64;
#pragma unroll
                            for (int g = 0; g < kGroups; ++g) {
                                if constexpr (EPI == EPI_SWIGLU) {
                                    const bool up = g >= kGroups / 2;
                                    const int gg = up ? g - kGroups / 2 : g;
                                    tma_load_2d(b_dst + g * 8192, up ? &tm_b2 : &tm_b, n0 + gg * 64,
                                                kb * kBlockK, full_bar(stage));
                                } else {
                                    tma_load_2d(b_dst + g * 8192, &tm_b, n0 + g * 64, kb * kBlockK,
                                                full_bar(stage));
                                }
                            }
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
        // ------------------------------ MMA issuer --------------------------------------
        {
            const bool leader = elect_one();
            constexpr uint32_t d_fmt = (KIND == MMA_I8) ? 2u : 1u;
            constexpr uint32_t ab_fmt = (KIND == MMA_F8F6F4) ? 0u : 1u;  // bf16 / e4m3 / s8
            constexpr uint32_t idesc =
                make_idesc(d_fmt, ab_fmt, ab_fmt, B_KN ? 1u : 0u, kBlockM, BLOCK_N);
            constexpr uint32_t kBAdvance = B_KN ? (16 * kRowBytes) >> 4 : 32 >> 4;
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            long long wait_clk = 0;
            const long long t_begin = clock64();
            // The thread looks at the NEXT stage's barrier before it issues the current stage's
            // MMAs, so that the probe's latency hides behind the issue instead of opening a gap
            // in the tensor pipe between two K blocks.
            uint32_t ready = mbar_test_wait(full_bar(0), 0);
            for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++it) {
                const int buf = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1u;
                const int kb_begin = (w % p.split_k) * p.kb_per_split;
                const int kb_end = min(kb_begin + p.kb_per_split, p.num_k_blocks);
                ok = mbar_wait_bounded(acc_empty_bar(buf), acc_phase ^ 1u, abort_flag, p.status,
                                       kWaitMmaAccEmpty, p.wait_ns);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BLOCK_N;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!__all_sync(0xffffffffu, ready)) {
                        const long long c0 = O64_DBG(p) ? clock64() : 0;
                        ok = mbar_wait_bounded(full_bar(stage), phase, abort_flag, p.status,
                                               kWaitMmaFull, p.wait_ns);
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
                        B_KN ? make_smem_desc(b_addr, 8192, 1024) : make_smem_desc(b_addr, 16, 1024);
                    if ((O64_PROBE(p) & 3) == 2) {
                        if (leader) mbar_arrive(empty_bar(stage));
                    } else if (leader) {
#pragma unroll
                        for (int k = 0; k < kMmaPerStage; ++k) {
                            tc_mma<KIND>(d_tmem, a_desc + 2u * k, b_desc + kBAdvance * k, idesc,
                                         ((kb - kb_begin) | k) != 0 ? 1u : 0u);
                        }
                        tc_commit(empty_bar(stage));  // frees the stage when these MMAs retire
                    }
                    __syncwarp();
                    stage = next_stage;
                    phase = next_phase;
                    ready = next_ready;
                }
                if (ok && leader) tc_commit(acc_full_bar(buf));
                __syncwarp();
            }
            if (O64_DBG(p) && leader) {
                O64_DBG(p)[blockIdx.x * 8 + 0] = wait_clk;
                O64_DBG(p)[blockIdx.x * 8 + 1] = clock64() - t_begin;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue ----------------------------------------
        const int quarter = warp & 3;  // TMEM lane quarter this warp may read
        int it = 0;
        bool ok = true;
        if (p.xchg_local) ok = xchg_wait_entry(p, abort_flag, xchg_ready, warp == 2);  // no remote store before every rank is here
        for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++it) {
            int mb, nb;
            tile_coords(w / p.split_k, p, mb, nb);
            const int buf = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1u;
            // one lane polls, the warp follows (tcgen05.ld is warp-wide: the warp leaves together)
            if (lane == 0)
                ok = mbar_wait_bounded(acc_full_bar(buf), acc_phase, abort_flag, p.status,
                                       kWaitEpiAccFull, p.wait_ns);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            const long long row0 = (long long)mb * kBlockM + quarter * 32;
            const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + buf * BLOCK_N;
            if (p.split_k > 1) {
                if constexpr (EPI == EPI_S32)
                    epilogue_partial<true>(p, p.C, p.ldc, row0, nb * kOutN, t_row,
                                           smem_gen + L::kStagingOffset + quarter * kEpiStagingBytesPerWarp, BLOCK_N);
                else if constexpr (EPI == EPI_BF16 || EPI == EPI_SCALED_BF16)
                    epilogue_partial<false>(p, p.partial, p.N, row0, nb * kOutN, t_row,
                                            smem_gen + L::kStagingOffset + quarter * kEpiStagingBytesPerWarp, BLOCK_N);
            } else if (!(O64_PROBE(p) & 4))
                epilogue_tile<EPI, BLOCK_N>(p, row0, nb * kOutN, t_row,
                                            smem_gen + L::kStagingOffset + quarter * kEpiStagingBytesPerWarp);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(buf));
        }
        if (p.xchg_local) xchg_stores_done();
    }

    // ------------------------------ teardown --------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (p.xchg_local && threadIdx.x == 0) xchg_finish(p, abort_flag);
    if (warp == 1) {
        if (*abort_flag) {
            // a wait ran out: give copies and MMAs still in flight time to land before the
            // tensor memory goes back (bounded: about 200 microseconds)
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// 2-D row-major tensor [rows, cols] of `elem` bytes with `ld` elements between rows; box of
// box_cols x box_rows; 128-byte swizzle; out-of-range elements read as zero.
int encode_2d(CUtensorMap *tm, int kind, const void *base, int64_t rows, int64_t cols, int64_t ld,
              int box_cols, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return O64_ERR_CUDA;
    const int elem = (kind == O64_KIND_BF16) ? 2 : 1;
    const CUtensorMapDataType dt =
        (kind == O64_KIND_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * elem};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? O64_OK : O64_ERR_CUDA;
}

int encode_c_bytes(CUtensorMap *tm, void *base, int64_t rows, int64_t cols, int64_t ld, int elem) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return O64_ERR_CUDA;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || ((ld * elem) % 16) || cols * elem < 128 || rows < 1) return O64_ERR_ALIGN;
    cuuint64_t dims[2] = {(cuuint64_t)(cols * elem), (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * elem};
    cuuint32_t box[2] = {128, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? O64_OK : O64_ERR_CUDA;
}

static std::atomic<int> g_force_tail{-1};
void force_tail_split(int mode) { g_force_tail.store(mode < 0 ? -1 : (mode ? 1 : 0)); }

// what the last launch of a CTA-pair kernel on this thread decided (read by o64_test_last_tail_split)
static thread_local int g_last_tail_tiles = 0, g_last_tail_pairs = 0;
void last_tail_split(int *tiles, int *pairs) {
    *tiles = g_last_tail_tiles;
    *pairs = g_last_tail_pairs;
}

void plan_tail(UmmaParams &p, int pairs, long long slot_bytes, long long capacity) {
    p.tail_tiles = 0;
    p.tail_pairs = 0;
    g_last_tail_tiles = g_last_tail_pairs = 0;
    p.tail_slot_bytes = slot_bytes;
    if (!p.tail_slots || !p.tail_flags || pairs < 2 || slot_bytes <= 0) return;
    // O64_TAIL_SPLIT=0 turns the split off, =1 takes it whenever a last wave is partly filled;
    // o64_test_force_tail_split overrides the environment
    static const int env_mode = [] {
        const char *e = getenv("O64_TAIL_SPLIT");
        return e ? atoi(e) : -1;
    }();
    const int forced = g_force_tail.load(std::memory_order_relaxed);
    const int mode = forced >= 0 ? forced : env_mode;
    const long long tiles = (long long)p.num_m_tiles * p.num_n_tiles;
    const int rows_per_cta = slot_bytes >= (long long)kTailSlotBytesMax ? 256 : 128;
    tail_model(tiles, pairs, p.num_k_blocks, rows_per_cta, capacity / slot_bytes, mode, &p.tail_tiles, &p.tail_pairs);
    g_last_tail_tiles = p.tail_tiles;
    g_last_tail_pairs = p.tail_pairs;
    const char *tr = getenv("O64_TRACE");
    if (p.tail_tiles && tr && strstr(tr, "plan"))
        fprintf(stderr, "[o64 last wave: %d of %lld tiles cut along K over %d of %d CTA pairs]\n", p.tail_tiles, tiles,
                p.tail_pairs, pairs);
}

template <int KIND, bool B_KN, int EPI, int BLOCK_N, int STAGES, bool HOOK = false>
static int launch_inst(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tb2,
                       const UmmaParams &p, int grid, cudaStream_t stream) {
    using L = SmemLayout<BLOCK_N, STAGES>;
    auto kern = umma_gemm_kernel<KIND, B_KN, EPI, BLOCK_N, STAGES, HOOK>;
    static KernelSetup ks;  // per instantiation; one set-up per device
    const int rc = ks.once(
        [&](int *) {
            return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) == cudaSuccess
                       ? O64_OK
                       : O64_ERR_CUDA;
        },
        nullptr);
    if (rc) return rc;
    kern<<<grid, kThreads, L::kDynamic, stream>>>(ta, tb, tb2, p);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int umma_launch(const UmmaCall &c) {
    const int elem = (c.kind == O64_KIND_BF16) ? 2 : 1;
    if (c.M <= 0 || c.N <= 0 || c.K <= 0) return O64_ERR_RANK;
    if (c.M > INT32_MAX || c.N > INT32_MAX || c.K > INT32_MAX) return O64_ERR_RANK;
    if (c.kind != O64_KIND_BF16 && c.kind != O64_KIND_FP8 && c.kind != O64_KIND_S8)
        return O64_ERR_DTYPE;
    if (c.b_kn && c.kind != O64_KIND_BF16 && c.kind != O64_KIND_FP8) return O64_ERR_DTYPE;
    // an e4m3 weight stored [K,N] is read by the CTA-pair kernel on 256 x 256 tiles only
    if (c.b_kn && c.kind == O64_KIND_FP8 &&
        !(c.plan.cta_group == 2 && c.plan.tile_m == 256 && c.plan.tile_n == 256 && c.plan.split_k == 1))
        return O64_ERR_DTYPE;
    if (c.epi == EPI_SWIGLU && (!c.b_kn || !c.B2)) return O64_ERR_DTYPE;
    // TMA needs 16-byte aligned bases and row pitches
    if (!aligned16(c.A) || !aligned16(c.B) || (c.B2 && !aligned16(c.B2))) return O64_ERR_ALIGN;
    if ((c.lda * elem) % 16 || (c.ldb * elem) % 16) return O64_ERR_ALIGN;
    const int64_t b_cols = c.b_kn ? c.N : c.K;
    if (c.lda < c.K || c.ldb < b_cols || c.ldc < c.N) return O64_ERR_CONFORM;

    const o64_plan_t &pl = c.plan;
    const int block_n = pl.tile_n;
    const int block_k = kRowBytes / elem;
    const int out_n = (c.epi == EPI_SWIGLU) ? block_n / 2 : block_n;

    const bool pair = pl.cta_group == 2;
    const bool wide = pair && pl.tile_m == 512;  // each CTA of the pair owns 256 rows
    if (wide && block_n != 256) return O64_ERR_DTYPE;
    const int tile_m = wide ? 512 : (pair ? 2 * kBlockM : kBlockM);
    UmmaParams p;
    p.M = (int)c.M;
    p.N = (int)c.N;
    p.K = (int)c.K;
    p.C = c.C;
    p.ldc = c.ldc;
    p.bias = c.bias;
    p.scale_a = c.scale_a;
    p.scale_b = c.scale_b;
    p.act = c.act;
    p.num_m_tiles = (int)((c.M + tile_m - 1) / tile_m);
    p.num_n_tiles = (int)((c.N + out_n - 1) / out_n);
    p.group_m = pl.group_m > 0 ? pl.group_m : 8;
    p.raster = pl.raster;
    p.num_k_blocks = (int)((c.K + block_k - 1) / block_k);
    const int out_elem = epi_out_bytes(c.epi);
    p.vec_ok = aligned16(c.C) && ((c.ldc * out_elem) % 16 == 0);
    p.tma_store = 0;
    p.status = c.status_word;
    p.wait_ns = c.wait_ns ? c.wait_ns : kDefaultWaitNs;
    p.test_withhold = c.test_withhold;
    p.split_k = 1;
    p.kb_per_split = p.num_k_blocks;
    p.partial = nullptr;
    if (!pair && c.split_ready && pl.split_k > 1 && (c.epi == EPI_BF16 || c.epi == EPI_SCALED_BF16 || c.epi == EPI_S32) &&
        (c.partial || c.epi == EPI_S32)) {
        const int per = (p.num_k_blocks + pl.split_k - 1) / pl.split_k;
        p.kb_per_split = per;
        p.split_k = (p.num_k_blocks + per - 1) / per;  // every slice non-empty
        p.partial = c.partial;
    }
    p.tail_tiles = 0;
    p.tail_pairs = 0;
    p.tail_slots = c.tail_slots;
    p.tail_flags = c.tail_flags;
    p.tail_slot_bytes = (long long)c.tail_bytes;  // capacity until a launcher has planned the split
    p.n_peers = c.n_peers;
    for (int i = 0; i < 7; ++i) p.peer_c[i] = c.peer_c[i];
    p.xchg_local = c.n_peers > 0 ? c.xchg_local : nullptr;
    p.xchg_rank = c.xchg_rank;
    for (int i = 0; i < 7; ++i) {
        p.xchg_peer[i] = c.xchg_peer[i];
        p.xchg_peer_rank[i] = c.xchg_peer_rank[i];
    }
    if (c.n_peers > 0 && !p.vec_ok) return O64_ERR_ALIGN;  // the fused exchange uses the vector-store path only
    p.sk_a_rows = 0;
    p.sk_stages = 0;
    p.sk_split = 1;
    if (pl.split_k < 0) return umma_launch_skinny(c, p);  // few rows of A: the stream-K kernel

    CUtensorMap ta, tb, tb2;
    int rc = encode_2d(&ta, c.kind, c.A, c.M, c.K, c.lda, block_k, wide ? 256 : kBlockM);
    if (rc) return rc;
    if (!c.b_kn) {
        // a CTA of a pair loads half of the B block
        rc = encode_2d(&tb, c.kind, c.B, c.N, c.K, c.ldb, block_k, pair ? block_n / 2 : block_n);
        tb2 = tb;
    } else {
        const int kn_cols = (c.kind == O64_KIND_BF16) ? 64 : 128;  // 128 bytes of N per shared-memory row
        rc = encode_2d(&tb, c.kind, c.B, c.K, c.N, c.ldb, kn_cols, block_k);
        tb2 = tb;
        if (!rc && c.epi == EPI_SWIGLU) rc = encode_2d(&tb2, c.kind, c.B2, c.K, c.N, c.ldb, kn_cols, block_k);
    }
    if (rc) return rc;

#ifdef O64_TUNING
    {
        const char *pr = getenv("O64_PROBE");  // pipeline probes for tuning; results are invalid
        p.probe = pr ? atoi(pr) : 0;
    }
    // O64_TRACE=pipe: the issuing threads count the cycles they spend waiting; the launch is then
    // synchronous and prints the averages
    static unsigned long long *dbg_bufs[kMaxDevices] = {nullptr};  // one buffer per device
    int dbg_dev = 0;
    if (cudaGetDevice(&dbg_dev) != cudaSuccess || dbg_dev < 0 || dbg_dev >= kMaxDevices) dbg_dev = 0;
    unsigned long long *&dbg_buf = dbg_bufs[dbg_dev];
    const char *tr = getenv("O64_TRACE");
    const bool trace_pipe = tr && strstr(tr, "pipe") && c.may_allocate;
    p.dbg = nullptr;
    if (trace_pipe) {
        if (!dbg_buf && cudaMalloc(&dbg_buf, 8 * 1024 * sizeof(unsigned long long)) != cudaSuccess) dbg_buf = nullptr;
        if (dbg_buf) cudaMemsetAsync(dbg_buf, 0, 8 * 1024 * sizeof(unsigned long long), c.stream);
        p.dbg = dbg_buf;
    }
    auto report = [&](int rc_launch, int ctas) {
        if (!trace_pipe || !dbg_buf || rc_launch) return rc_launch;
        static unsigned long long host[8 * 1024];
        cudaStreamSynchronize(c.stream);
        cudaMemcpy(host, dbg_buf, sizeof(host), cudaMemcpyDeviceToHost);
        double s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int n = 0, n_mma = 0;
        for (int i = 0; i < ctas && i < 1024; ++i) {
            if (!host[8 * i + 1] && !host[8 * i + 3]) continue;
            for (int j = 0; j < 8; ++j) s[j] += (double)host[8 * i + j];
            ++n;
            if (host[8 * i + 1]) ++n_mma;
        }
        if (n && n_mma)
            fprintf(stderr,
                    "[o64 pipe: mma thread %.0f clk, waits for data %.1f%%, for a drained accumulator %.1f%%; "
                    "producer waits %.1f%% of %.0f clk; epilogue busy %.0f clk per CTA; %d CTAs; pair kernels: waiting for "
                    "contributors %.0f, partial sums out %.0f, epilogue warp loop %.0f clk]\n",
                    s[1] / n_mma, 100.0 * s[0] / s[1], 100.0 * s[5] / s[1],
                    100.0 * s[2] / (s[3] > 0 ? s[3] : 1), s[3] / n, s[4] / n, n, s[5] / n, s[6] / n, s[7] / n);
        return rc_launch;
    };
#else
    auto report = [](int rc_launch, int) { return rc_launch; };
#endif
    if (wide) return report(umma_launch_wide(c, ta, tb, tb2, p), pl.num_ctas);
    if (pair) return report(umma_launch_pair(c, ta, tb, tb2, p), pl.num_ctas);
    const long long tiles = (long long)p.num_m_tiles * p.num_n_tiles * p.split_k;
    const int grid = (int)(tiles < pl.num_ctas ? tiles : pl.num_ctas);

#define O64_INST(KIND, BKN, EPI_, BN, ST) \
    return report(launch_inst<KIND, BKN, EPI_, BN, ST>(ta, tb, tb2, p, grid, c.stream), grid)

    // the one instantiation with the test hook: bf16, B [N,K], 128 x 256 tiles
    if (c.test_withhold >= 0) {
        if (c.kind != O64_KIND_BF16 || c.epi != EPI_BF16 || c.b_kn || block_n != 256 || p.split_k != 1) return O64_ERR_DTYPE;
        return launch_inst<MMA_F16, false, EPI_BF16, 256, 4, true>(ta, tb, tb2, p, grid, c.stream);
    }

    if (c.kind == O64_KIND_BF16) {
        if (c.epi == EPI_SWIGLU) {
            if (block_n == 256) O64_INST(MMA_F16, true, EPI_SWIGLU, 256, 4);
            if (block_n == 128) O64_INST(MMA_F16, true, EPI_SWIGLU, 128, 6);
        } else if (c.epi == EPI_BF16) {
            if (c.b_kn) {
                if (block_n == 256) O64_INST(MMA_F16, true, EPI_BF16, 256, 4);
                if (block_n == 128) O64_INST(MMA_F16, true, EPI_BF16, 128, 6);
            } else {
                if (block_n == 256) O64_INST(MMA_F16, false, EPI_BF16, 256, 4);
                if (block_n == 128) O64_INST(MMA_F16, false, EPI_BF16, 128, 6);
            }
        }
    } else if (c.kind == O64_KIND_FP8 && c.epi == EPI_SCALED_BF16) {
        if (block_n == 256) O64_INST(MMA_F8F6F4, false, EPI_SCALED_BF16, 256, 4);
        if (block_n == 128) O64_INST(MMA_F8F6F4, false, EPI_SCALED_BF16, 128, 6);
    } else if (c.kind == O64_KIND_S8 && c.epi == EPI_S32) {
        if (block_n == 256) O64_INST(MMA_I8, false, EPI_S32, 256, 4);
        if (block_n == 128) O64_INST(MMA_I8, false, EPI_S32, 128, 6);
    } else if (c.kind == O64_KIND_FP8 && c.epi == EPI_SCALED_E4M3) {
        if (block_n == 256) O64_INST(MMA_F8F6F4, false, EPI_SCALED_E4M3, 256, 4);
        if (block_n == 128) O64_INST(MMA_F8F6F4, false, EPI_SCALED_E4M3, 128, 6);
    } else if (c.kind == O64_KIND_S8 && c.epi == EPI_ISCALED_BF16) {
        if (block_n == 256) O64_INST(MMA_I8, false, EPI_ISCALED_BF16, 256, 4);
        if (block_n == 128) O64_INST(MMA_I8, false, EPI_ISCALED_BF16, 128, 6);
    } else if (c.kind == O64_KIND_S8 && c.epi == EPI_ISCALED_S8) {
        if (block_n == 256) O64_INST(MMA_I8, false, EPI_ISCALED_S8, 256, 4);
        if (block_n == 128) O64_INST(MMA_I8, false, EPI_ISCALED_S8, 128, 6);
    }
#undef O64_INST
    return O64_ERR_DTYPE;
}

}  // namespace o64
