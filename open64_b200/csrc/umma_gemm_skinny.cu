// Tensor-core GEMM for few rows of A against a large weight (M <= 128): the weight is read
// once, so the kernel is bound by HBM and is built to keep enough loads in flight.
//
// Differences from the 128 x BLOCK_N tile kernel (umma_gemm.cu):
//   * the TMA box of A holds only `a_rows` rows (16 / 32 / 64 / 128, the next size >= M), and a
//     shared-memory stage is that many rows of A plus BN rows of B.  The MMA still runs with
//     M = 128: the accumulator rows beyond a_rows are computed from whatever follows the A box in
//     shared memory and are never read back (row i of the product depends on row i of A only).
//     A 16-row problem thus keeps 6 stages x 32 KB of weight in flight per SM instead of 4.
//   * a 128 x 256 (or 128 x 128: template parameter BN) output tile belongs to a thread-block
//     CLUSTER of S CTAs (S = 1, 2, 4, 8; at most BN / 32), each of which multiplies one slice of
//     K.  The partial sums never touch global memory: after a
//     cluster barrier (every main loop done, so every ring is free) each CTA stores the columns
//     c * BN/S .. of its accumulator into CTA c's idle ring (distributed shared memory), a
//     second cluster barrier follows, and each CTA adds the S slices it received, applies the
//     epilogue and writes its BN/S columns of C.  Measured: partial sums exchanged through L2
//     (atomics, a fence, a completion counter) cost three dependent round trips of about 2 us each
//     at the end of the kernel, while the memory system is still saturated by the other CTAs.
//
// In the reference's terms this is the K loop of the nest (osprey/be/vho/f90_lower.cxx:5155)
// strip-mined once more and its strips run in parallel, the sum being a reduction the compiler
// may reassociate at -O3 (osprey/common/com/config.cxx:1670-1680); integer sums are exact in
// any order.
//
// Warp roles as in umma_gemm.cu (producer, MMA issuer, four epilogue warps) plus two warps that
// only help with the exchange: 256 threads, two warps for each quarter of the TMEM lanes.
// Every mbarrier wait is bounded; on expiry the CTA records a code and leaves its loops, but
// still takes part in both cluster barriers, so that the other CTAs of its cluster return too.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "umma_common.cuh"

namespace o64 {

namespace {

constexpr int kSkMaxStages = 8;
constexpr int kSkThreads = 256;  // producer, MMA issuer, four epilogue warps, two more for the exchange
constexpr int kSkMaxRows = 512;  // up to four 128-row tiles per 256-column block
constexpr int kSkRingBytes = 6 * (256 + 16) * kRowBytes;  // 6 stages of 256 columns at a_rows = 16
constexpr int kSkStagingOffset = kSkRingBytes;                   // epilogue patches, 4 KB per warp
constexpr int kSkBarOffset = kSkStagingOffset + kEpiStagingBytes;
constexpr int kSkNumBars = 2 * kSkMaxStages + 1;  // full[], empty[], accumulator ready
constexpr int kSkTmemPtrOffset = kSkBarOffset + 8 * kSkNumBars;
constexpr int kSkAbortOffset = kSkTmemPtrOffset + 4;
constexpr int kSkTotal = kSkAbortOffset + 4;
constexpr int kSkDynamic = kSkTotal + 1024;  // slack to align the ring to 1024 bytes
static_assert(kSkDynamic <= 227 * 1024, "shared memory");
static_assert(kSkRingBytes - 4 * kEpiStagingBytesPerWarp >= 128 * 1024, "borrowed patches lie beyond the receive area");

__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint4 v) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Sends 32 accumulator rows (this warp's TMEM lane quarter; row0 and `rows` count inside the
// tile), 32-column chunks c_begin .. c_end-1,
// to the CTAs of the cluster: columns c*slice .. of the tile go to CTA c, into slot `rank` of its
// receive area ([S][rows][slice] 4-byte sums at `recv`, the same shared-memory offset in every
// CTA).  Through the swizzled patch, so that a store instruction writes four full 128-byte row
// segments (measured: storing each thread's own row straight from its registers, 32 rows per
// instruction, takes twice as long for 128 rows); the load of the next chunk is in flight while
// this one is sent.
__device__ __forceinline__ void scatter_rows(int rows, int row0, uint32_t t_row, uint8_t *staging, uint32_t recv,
                                             uint8_t *recv_local, int rank, int slice, int c_begin, int c_end) {
    const int lane = threadIdx.x & 31;
    uint4 *patch = reinterpret_cast<uint4 *>(staging);
    const int sw = lane & 7;
    auto send = [&](const uint32_t (&v)[32], int i) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
            patch[lane * 8 + (q ^ sw)] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        __syncwarp();
        const int owner = (32 * i) / slice;          // uniform: slice is a multiple of 32
        const int cin = (32 * i) % slice + (lane & 7) * 4;
        const uint32_t base = map_to_cta(recv, owner);
#pragma unroll
        for (int r4 = 0; r4 < 8; ++r4) {
            const int r = 4 * r4 + (lane >> 3);
            const uint4 val = patch[r * 8 + ((lane & 7) ^ (r & 7))];
            const int grow = row0 + r;
            if (grow < rows) {
                const uint32_t off = (uint32_t)(((rank * rows + grow) * slice + cin) * 4);
                if (owner == rank)  // this CTA's own columns: a plain shared-memory store
                    *reinterpret_cast<uint4 *>(recv_local + off) = val;
                else
                    st_cluster_v4(base + off, val);
            }
        }
        __syncwarp();
    };
    uint32_t va[32], vb[32];
    __syncwarp();
    tmem_ld_32x32(t_row + 32 * c_begin, va);
#pragma unroll 1
    for (int i = c_begin; i < c_end; i += 2) {
        tmem_ld_wait();
        __syncwarp();
        if (i + 1 < c_end) tmem_ld_32x32(t_row + 32 * (i + 1), vb);
        send(va, i);
        if (i + 1 < c_end) {
            tmem_ld_wait();
            __syncwarp();
            if (i + 2 < c_end) tmem_ld_32x32(t_row + 32 * (i + 2), va);
            send(vb, i + 1);
        }
    }
}

// Adds the S slices received for this CTA's columns, applies the epilogue and writes C.
// All threads of the CTA; four columns per thread.
template <int EPI, int ACT>
__device__ __forceinline__ void gather_store(const UmmaParams &p, const uint8_t *recv, int m_base, int rows, int n0,
                                             int rank, int S, int slice, int t) {
    const int tpr = slice / 4;  // threads per row
    const int c4 = (t % tpr) * 4;
    const int col = n0 + rank * slice + c4;
    if (col >= p.N) return;
    const int ncols = min(4, p.N - col);
    float bias[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sb[4] = {1.0f, 1.0f, 1.0f, 1.0f};
    if constexpr (EPI != EPI_S32) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (e < ncols) {
                if (p.bias) bias[e] = __ldg(p.bias + col + e);
                if constexpr (EPI == EPI_SCALED_BF16) {
                    if (p.scale_b) sb[e] = __ldg(p.scale_b + col + e);
                }
            }
        }
    }
    for (int m = t / tpr; m < rows; m += kSkThreads / tpr) {
        const int pitch = slice;
        uint4 acc = *reinterpret_cast<const uint4 *>(recv + (size_t)((m * pitch) + c4) * 4);
        for (int src = 1; src < S; ++src) {
            const uint4 w = *reinterpret_cast<const uint4 *>(recv + (size_t)(((src * rows + m) * pitch) + c4) * 4);
            if constexpr (EPI == EPI_S32) {
                acc.x += w.x; acc.y += w.y; acc.z += w.z; acc.w += w.w;  // two's complement: exact
            } else {
                acc.x = __float_as_uint(__uint_as_float(acc.x) + __uint_as_float(w.x));
                acc.y = __float_as_uint(__uint_as_float(acc.y) + __uint_as_float(w.y));
                acc.z = __float_as_uint(__uint_as_float(acc.z) + __uint_as_float(w.z));
                acc.w = __float_as_uint(__uint_as_float(acc.w) + __uint_as_float(w.w));
            }
        }
        const uint32_t w[4] = {acc.x, acc.y, acc.z, acc.w};
        if constexpr (EPI == EPI_S32) {
            int32_t *dst = reinterpret_cast<int32_t *>(p.C) + (long long)(m_base + m) * p.ldc + col;
            if (ncols == 4 && p.vec_ok) {
                *reinterpret_cast<uint4 *>(dst) = acc;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (e < ncols) dst[e] = (int32_t)w[e];
            }
        } else {
            float x[4];
            float sa = 1.0f;
            if constexpr (EPI == EPI_SCALED_BF16) {
                if (p.scale_a) sa = __ldg(p.scale_a + m_base + m);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                x[e] = __uint_as_float(w[e]);
                if constexpr (EPI == EPI_SCALED_BF16) {
                    // every operation rounded by itself, as in the tile kernels' scaled tail
                    x[e] = act_fixed<ACT>(__fadd_rn(__fmul_rn(x[e], __fmul_rn(sa, sb[e])), bias[e]));
                } else {
                    if (p.bias) x[e] += bias[e];
                    x[e] = act_fixed<ACT>(x[e]);
                }
            }
            __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(p.C) + (long long)(m_base + m) * p.ldc + col;
            if (ncols == 4 && p.vec_ok) {
                *reinterpret_cast<uint2 *>(dst) = make_uint2(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]));
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (e < ncols) dst[e] = __float2bfloat16_rn(x[e]);
            }
        }
    }
}

template <int EPI>
__device__ __forceinline__ void gather_store_dispatch(const UmmaParams &p, const uint8_t *recv, int m_base, int rows,
                                                      int n0, int rank, int S, int slice, int t) {
    if constexpr (EPI == EPI_BF16 || EPI == EPI_SCALED_BF16) {
        switch (p.act) {  // uniform: one branch per tile
        case O64_ACT_RELU: gather_store<EPI, O64_ACT_RELU>(p, recv, m_base, rows, n0, rank, S, slice, t); break;
        case O64_ACT_GELU_TANH: gather_store<EPI, O64_ACT_GELU_TANH>(p, recv, m_base, rows, n0, rank, S, slice, t); break;
        case O64_ACT_GELU_ERF: gather_store<EPI, O64_ACT_GELU_ERF>(p, recv, m_base, rows, n0, rank, S, slice, t); break;
        case O64_ACT_SILU: gather_store<EPI, O64_ACT_SILU>(p, recv, m_base, rows, n0, rank, S, slice, t); break;
        default: gather_store<EPI, O64_ACT_NONE>(p, recv, m_base, rows, n0, rank, S, slice, t); break;
        }
    } else {
        gather_store<EPI, O64_ACT_NONE>(p, recv, m_base, rows, n0, rank, S, slice, t);
    }
}

}  // namespace

// KIND / B_KN / EPI as in umma_gemm_kernel; BN: columns of a tile (256, or 128: half the partial
// sums to exchange per CTA and twice the tiles, for 128 rows or a narrow weight).  Launched with
// clusters of p.sk_split CTAs; CTA r of cluster t multiplies K blocks [r*kbs/S, (r+1)*kbs/S) of tile t.
template <int KIND, bool B_KN, int EPI, int BN, bool HOOK = false>
__global__ void __launch_bounds__(kSkThreads, 1)
umma_gemm_skinny_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                        const UmmaParams p) {
    constexpr int kElem = (KIND == MMA_F16) ? 2 : 1;
    constexpr int kBlockK = kRowBytes / kElem;
    constexpr int kMmaPerStage = 4;
    constexpr uint32_t kTmemCols = BN;  // one accumulator
    constexpr int kBBytes = BN * kRowBytes;  // 32 or 16 KB of weight per stage
    static_assert(!B_KN || KIND == MMA_F16, "[K,N] operands are supported for bf16 only");
    static_assert(EPI != EPI_SWIGLU, "no SwiGLU variant");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + kSkBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kSkMaxStages + s); };
    const uint32_t acc_full_bar = bar_base + 8u * (2 * kSkMaxStages);
    volatile uint32_t *tmem_ptr_smem = reinterpret_cast<volatile uint32_t *>(smem_gen + kSkTmemPtrOffset);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem_gen + kSkAbortOffset);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int stages = p.sk_stages;
    const uint32_t a_bytes = (uint32_t)p.sk_a_rows * kRowBytes;
    const uint32_t stage_bytes = kBBytes + a_bytes;  // B first: the MMA's reads past the A box stay inside the allocation
    const int S = p.sk_split;
    const int rank = (int)cluster_ctarank();
    const int tile = blockIdx.x / S;             // tiles of one 256-column block are neighbours: they share B in L2
    const int mt = tile % p.num_m_tiles;
    const int m_base = mt * kBlockM;
    const int rows = min(kBlockM, p.M - m_base);  // rows of A this tile really has
    const int n0 = (tile / p.num_m_tiles) * BN;
    const int kbs = p.num_k_blocks;
    const int kb_begin = (int)((long long)kbs * rank / S);
    const int kb_end = (int)((long long)kbs * (rank + 1) / S);

    // The next launch of the stream may take the SMs this grid leaves idle, and each SM a CTA of
    // this grid leaves, without waiting for the whole grid to drain: its set-up and an L2 prefetch
    // of its first weights then overlap this grid's tail (it waits below before it reads or writes
    // anything this grid may touch).
    griddep_launch_dependents();
    unsigned long long *dbg = O64_DBG(p) ? O64_DBG(p) + 8 * blockIdx.x : nullptr;  // O64_TRACE=pipe: time stamps (ns)
    if (threadIdx.x == 0) {
        if (dbg) dbg[0] = globaltimer_ns();
        for (int s = 0; s < kSkMaxStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(acc_full_bar, 1);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(smem_gen + kSkTmemPtrOffset), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;
    // Before the dependency wait nothing may be read into the SM or written: an earlier kernel of
    // the stream may still be producing A, B or bias, or reading C.  A prefetch into L2 is safe (L2
    // is where those writes land, so it never holds stale data) and starts the weight's first
    // blocks on their way from HBM.
    if (threadIdx.x == 0) {
        const int ahead = min(stages, kb_end - kb_begin);
        for (int i = 0; i < ahead; ++i) {
            if constexpr (!B_KN) {
                tma_prefetch_l2_2d(&tm_b, (kb_begin + i) * kBlockK, n0);
            } else {
#pragma unroll
                for (int g = 0; g < BN / 64; ++g) tma_prefetch_l2_2d(&tm_b, n0 + g * 64, (kb_begin + i) * kBlockK);
            }
        }
    }
    griddep_wait();
    if (dbg && threadIdx.x == 0) dbg[1] = globaltimer_ns();

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------------
        const bool leader = elect_one();
        const uint64_t stream_once = l2_policy_evict_first();  // the weight: read once, first out of L2
        int stage = 0;
        uint32_t phase = 0;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
            bool ok = mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, p.status, kWaitProducerEmpty, p.wait_ns);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint32_t b_dst = smem_base + stage * stage_bytes;
            const uint32_t a_dst = b_dst + kBBytes;
            bool withhold = false;  // test hook: this K block's loads are left out
            if constexpr (HOOK) withhold = (kb - kb_begin == p.test_withhold);
            if (leader && !withhold) {
                mbar_arrive_expect_tx(full_bar(stage), stage_bytes);
                tma_load_2d(a_dst, &tm_a, kb * kBlockK, m_base, full_bar(stage));
                if constexpr (!B_KN) {
                    tma_load_2d_hint(b_dst, &tm_b, kb * kBlockK, n0, full_bar(stage), stream_once);
                } else {
#pragma unroll
                    for (int g = 0; g < BN / 64; ++g)
                        tma_load_2d_hint(b_dst + g * 8192, &tm_b, n0 + g * 64, kb * kBlockK, full_bar(stage),
                                         stream_once);
                }
            }
            __syncwarp();
            if (++stage == stages) {
                stage = 0;
                phase ^= 1u;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------------
        const bool leader = elect_one();
        constexpr uint32_t d_fmt = (KIND == MMA_I8) ? 2u : 1u;
        constexpr uint32_t ab_fmt = (KIND == MMA_F8F6F4) ? 0u : 1u;
        constexpr uint32_t idesc = make_idesc(d_fmt, ab_fmt, ab_fmt, B_KN ? 1u : 0u, kBlockM, BN);
        constexpr uint32_t kBAdvance = B_KN ? (16 * kRowBytes) >> 4 : 32 >> 4;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
            ok = mbar_wait_bounded(full_bar(stage), phase, abort_flag, p.status, kWaitMmaFull, p.wait_ns);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (dbg && leader && kb == kb_begin) dbg[2] = globaltimer_ns();
            tc_fence_after();
            const uint32_t b_addr = smem_base + stage * stage_bytes;
            const uint32_t a_addr = b_addr + kBBytes;
            const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024);
            const uint64_t b_desc = B_KN ? make_smem_desc(b_addr, 8192, 1024) : make_smem_desc(b_addr, 16, 1024);
            if (leader) {
#pragma unroll
                for (int k = 0; k < kMmaPerStage; ++k)
                    tc_mma<KIND>(tmem_base, a_desc + 2u * k, b_desc + kBAdvance * k, idesc,
                                 ((kb - kb_begin) | k) != 0 ? 1u : 0u);
                tc_commit(empty_bar(stage));
            }
            __syncwarp();
            if (++stage == stages) {
                stage = 0;
                phase ^= 1u;
            }
        }
        if (ok && leader) tc_commit(acc_full_bar);
        if (dbg && leader) dbg[3] = globaltimer_ns();
        __syncwarp();
    } else {
        // ------------------------------ epilogue warps: wait for the accumulator ---------
        bool ok = true;
        if (lane == 0) ok = mbar_wait_bounded(acc_full_bar, 0, abort_flag, p.status, kWaitEpiAccFull, p.wait_ns);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        tc_fence_after();
        if (dbg && warp == 2 && lane == 0) dbg[4] = globaltimer_ns();
        if (S == 1 && ok && warp < 6) {
            const int quarter = warp & 3;
            if (quarter * 32 < rows)
                epilogue_tile<EPI, BN>(p, m_base + quarter * 32, n0, tmem_base + (uint32_t(quarter * 32) << 16),
                                              smem_gen + kSkStagingOffset + quarter * kEpiStagingBytesPerWarp);
        }
        tc_fence_before();
    }

    if (S > 1) {
        // ------------------------------ sum over the cluster ------------------------------
        __syncthreads();
        cluster_sync_all();  // every CTA of the cluster is past its main loop: the rings are free
        if (dbg && threadIdx.x == 64) dbg[5] = globaltimer_ns();
        const bool good = (*abort_flag == 0);
        const int slice = BN / S;  // a multiple of 32: S <= BN / 32
        if (good) {
            // every warp sends: warp w reads TMEM lane quarter w % 4, so each quarter has two warps
            // (w and w + 4), which take four chunks each
            const int quarter = warp & 3;
            const int c_begin = warp >= 4 ? BN / 64 : 0;
            const int c_end = warp < 4 ? BN / 64 : BN / 32;
            // patches: the epilogue warps' own; warps 0, 1, 6 and 7 borrow the end of the (now idle)
            // ring, beyond the receive area (at most 128 KB from its start)
            const int borrowed = warp < 2 ? warp : warp - 4;
            uint8_t *patch = (warp >= 2 && warp < 6)
                                 ? smem_gen + kSkStagingOffset + quarter * kEpiStagingBytesPerWarp
                                 : smem_gen + kSkRingBytes - (borrowed + 1) * kEpiStagingBytesPerWarp;
            tc_fence_after();
            if (quarter * 32 < rows)
                scatter_rows(rows, quarter * 32, tmem_base + (uint32_t(quarter * 32) << 16), patch, smem_base, smem_gen,
                             rank, slice, c_begin, c_end);
            tc_fence_before();
        }
        cluster_sync_all();  // the slices sent to this CTA have arrived
        if (dbg && threadIdx.x == 64) dbg[6] = globaltimer_ns();
        if (good) gather_store_dispatch<EPI>(p, smem_gen, m_base, rows, n0, rank, S, slice, (int)threadIdx.x);
    }
    if (dbg && threadIdx.x == 64) dbg[7] = globaltimer_ns();

    // ------------------------------ teardown --------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (*abort_flag) {
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int KIND, bool B_KN, int EPI, int BN, bool HOOK = false>
static int launch_skinny(const CUtensorMap &ta, const CUtensorMap &tb, UmmaParams p, int tiles, int want_split,
                         cudaStream_t stream, int *split_out) {
    auto kern = umma_gemm_skinny_kernel<KIND, B_KN, EPI, BN, HOOK>;
    static KernelSetup ks;  // per instantiation; one set-up per device
    int max_split = 1;      // largest cluster the device can place with this much shared memory
    const int rc = ks.once(
        [&](int *clusters) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkDynamic) != cudaSuccess)
                return (int)O64_ERR_CUDA;
            *clusters = 1;
            for (int s = 8; s > 1; s /= 2) {
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(s, 1, 1);
                cfg.blockDim = dim3(kSkThreads, 1, 1);
                cfg.dynamicSmemBytes = kSkDynamic;
                cudaLaunchAttribute at[1];
                at[0].id = cudaLaunchAttributeClusterDimension;
                at[0].val.clusterDim.x = s;
                at[0].val.clusterDim.y = 1;
                at[0].val.clusterDim.z = 1;
                cfg.attrs = at;
                cfg.numAttrs = 1;
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n >= 1) {
                    *clusters = s;
                    break;
                }
                (void)cudaGetLastError();
            }
            return (int)O64_OK;
        },
        &max_split);
    if (rc) return rc;
    int split = want_split < max_split ? want_split : max_split;
    if (split < 1) split = 1;
    p.sk_split = split;
    *split_out = split;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * split), 1, 1);
    cfg.blockDim = dim3(kSkThreads, 1, 1);
    cfg.dynamicSmemBytes = kSkDynamic;
    cfg.stream = stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = split;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    // programmatic dependent launch: this grid may be scheduled before the previous kernel of the
    // stream has drained (the kernel waits for it before touching memory); O64_PDL=0 turns it off
    static const bool pdl = [] {
        const char *e = getenv("O64_PDL");
        return !(e && e[0] == '0');
    }();
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 2 : 1;
    if (cudaLaunchKernelEx(&cfg, kern, ta, tb, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return O64_ERR_CUDA;
    }
    return O64_OK;
}

// K slices per tile: the largest cluster size that keeps tiles * S within the CTAs the plan
// allows and leaves every slice at least one K block.  Clusters of 8 only for 8 tiles or fewer:
// measured, sixteen clusters of 8 CTAs with this much shared memory do not all fit at once.
int umma_skinny_split(int64_t M, int64_t N, int64_t K, int elem, int num_ctas, int bn) {
    const int64_t tiles = ((M + kBlockM - 1) / kBlockM) * ((N + bn - 1) / bn);
    const int64_t kbs = (K + kRowBytes / elem - 1) / (kRowBytes / elem);
    int s = tiles <= 8 ? 8 : 4;
    if (s > bn / 32) s = bn / 32;  // every CTA owns at least one 32-column chunk
    while (s > 1 && (tiles * s > num_ctas || s > kbs)) s /= 2;
    return s;
}

int umma_launch_skinny(const UmmaCall &c, UmmaParams p) {
    if (c.M > kSkMaxRows || c.epi == EPI_SWIGLU || c.n_peers > 0) return O64_ERR_DTYPE;
    const int elem = (c.kind == O64_KIND_BF16) ? 2 : 1;
    const int block_k = kRowBytes / elem;
    const int a_rows = c.M <= 16 ? 16 : (c.M <= 32 ? 32 : (c.M <= 64 ? 64 : 128));  // 128 per tile when M > 128
    const int bn = c.plan.tile_n == 128 ? 128 : 256;
    CUtensorMap ta, tb;
    int rc = encode_2d(&ta, c.kind, c.A, c.M, c.K, c.lda, block_k, a_rows);
    if (rc) return rc;
    if (!c.b_kn)
        rc = encode_2d(&tb, c.kind, c.B, c.N, c.K, c.ldb, block_k, bn);
    else
        rc = encode_2d(&tb, c.kind, c.B, c.K, c.N, c.ldb, 64, block_k);
    if (rc) return rc;
    p.num_m_tiles = (int)((c.M + kBlockM - 1) / kBlockM);
    p.num_n_tiles = (int)((c.N + bn - 1) / bn);
    p.split_k = 1;
    p.kb_per_split = p.num_k_blocks;
    p.n_peers = 0;
    p.tma_store = 0;
    p.xchg_local = nullptr;
#ifdef O64_TUNING
    p.probe = 0;
    p.dbg = nullptr;
#endif
    p.sk_a_rows = a_rows;
    const int stage_bytes = (bn + a_rows) * kRowBytes;
    p.sk_stages = kSkRingBytes / stage_bytes;
    if (p.sk_stages > kSkMaxStages) p.sk_stages = kSkMaxStages;
    const int ctas = c.plan.num_ctas > 0 ? c.plan.num_ctas : 148;
    // the plan's split_k is -S; -1 also stands for "choose"
    int want = c.plan.split_k < -1 ? -c.plan.split_k : umma_skinny_split(c.M, c.N, c.K, elem, ctas, bn);
    if (want > bn / 32) want = bn / 32;
    if (want > p.num_k_blocks) want = 1;
    const int tiles = p.num_m_tiles * p.num_n_tiles;

    int split = 1;
#ifdef O64_TUNING
    // O64_TRACE=pipe: every CTA leaves time stamps; the launch is then synchronous and prints where
    // the time went (a tuning aid, off by default)
    static unsigned long long *dbg_bufs[kMaxDevices] = {nullptr};  // one buffer per device
    int dbg_dev = 0;
    if (cudaGetDevice(&dbg_dev) != cudaSuccess || dbg_dev < 0 || dbg_dev >= kMaxDevices) dbg_dev = 0;
    unsigned long long *&dbg_buf = dbg_bufs[dbg_dev];
    constexpr int kDbgCtas = 1024;
    const char *tr = getenv("O64_TRACE");
    const bool trace = tr && strstr(tr, "pipe") && c.may_allocate && tiles * 8 <= kDbgCtas;
    if (trace) {
        if (!dbg_buf && cudaMalloc(&dbg_buf, 8 * kDbgCtas * sizeof(unsigned long long)) != cudaSuccess) dbg_buf = nullptr;
        if (dbg_buf) cudaMemsetAsync(dbg_buf, 0, 8 * kDbgCtas * sizeof(unsigned long long), c.stream);
        p.dbg = dbg_buf;
    }
    auto report = [&](int rc_launch) {
        if (!trace || !dbg_buf || rc_launch) return rc_launch;
        static unsigned long long host[8 * kDbgCtas];
        const int grid = tiles * split;
        cudaStreamSynchronize(c.stream);
        cudaMemcpy(host, dbg_buf, sizeof(host), cudaMemcpyDeviceToHost);
        unsigned long long t0 = ~0ull;
        for (int i = 0; i < grid; ++i)
            if (host[8 * i] && host[8 * i] < t0) t0 = host[8 * i];
        double sum[8] = {0}, mx[8] = {0};
        for (int i = 0; i < grid; ++i)
            for (int j = 0; j < 8; ++j) {
                const double v = host[8 * i + j] ? (double)(host[8 * i + j] - t0) * 1e-3 : 0.0;
                sum[j] += v;
                if (v > mx[j]) mx[j] = v;
            }
        fprintf(stderr,
                "[o64 few-rows timeline, us after the first CTA started, mean/max over %d CTAs (clusters of %d): start "
                "%.1f/%.1f, set up %.1f/%.1f, first data %.1f/%.1f, last MMA issued %.1f/%.1f, accumulator ready "
                "%.1f/%.1f, cluster past its main loops %.1f/%.1f, slices exchanged %.1f/%.1f, done %.1f/%.1f]\n",
                grid, split, sum[0] / grid, mx[0], sum[1] / grid, mx[1], sum[2] / grid, mx[2], sum[3] / grid, mx[3],
                sum[4] / grid, mx[4], sum[5] / grid, mx[5], sum[6] / grid, mx[6], sum[7] / grid, mx[7]);
        return rc_launch;
    };
#else
    auto report = [](int rc_launch) { return rc_launch; };
#endif
#define O64_SK(KIND, BKN, EPI_)                                                                              \
    return report(bn == 128 ? launch_skinny<KIND, BKN, EPI_, 128>(ta, tb, p, tiles, want, c.stream, &split)  \
                            : launch_skinny<KIND, BKN, EPI_, 256>(ta, tb, p, tiles, want, c.stream, &split))
    if (c.test_withhold >= 0) {  // the one instantiation with the test hook: bf16, B [N,K], 256-column tiles
        if (c.kind != O64_KIND_BF16 || c.epi != EPI_BF16 || c.b_kn || bn != 256) return O64_ERR_DTYPE;
        return launch_skinny<MMA_F16, false, EPI_BF16, 256, true>(ta, tb, p, tiles, want, c.stream, &split);
    }
    if (c.kind == O64_KIND_BF16 && c.epi == EPI_BF16) {
        if (c.b_kn) O64_SK(MMA_F16, true, EPI_BF16);
        O64_SK(MMA_F16, false, EPI_BF16);
    } else if (c.kind == O64_KIND_FP8 && c.epi == EPI_SCALED_BF16 && !c.b_kn) {
        O64_SK(MMA_F8F6F4, false, EPI_SCALED_BF16);
    } else if (c.kind == O64_KIND_S8 && c.epi == EPI_S32 && !c.b_kn) {
        O64_SK(MMA_I8, false, EPI_S32);
    }
#undef O64_SK
    return O64_ERR_DTYPE;
}

}  // namespace o64
