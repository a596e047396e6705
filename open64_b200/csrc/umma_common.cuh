// Pieces shared by the 1-CTA and the 2-CTA tcgen05 GEMM kernels: launch parameters, tile
// rasterisation, the fused epilogue.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <mutex>

#include "ptx_sm100.cuh"
#include "umma_gemm.cuh"

namespace o64 {

// Tuning aids exist only in a build with -DO64_TUNING (python -m open64_b200.build --tuning): the
// pipeline probes (O64_PROBE: skip the loads / the MMAs / the epilogue / the stores; results are
// invalid) and the cycle counters behind O64_TRACE=pipe.  In the shipped build both macros are
// constants and every branch on them is removed by the compiler.
#ifdef O64_TUNING
#define O64_PROBE(p) ((p).probe)
#define O64_DBG(p) ((p).dbg)
#else
#define O64_PROBE(p) 0
#define O64_DBG(p) (static_cast<unsigned long long *>(nullptr))
#endif

struct UmmaParams {
    int M, N, K;
    void *C;
    long long ldc;
    const float *bias;
    const float *scale_a;
    const float *scale_b;
    int act;
    int num_m_tiles, num_n_tiles, group_m, raster;
    int num_k_blocks;
    int vec_ok;  // C rows 16-byte aligned: vector stores allowed
    int tma_store;  // kernels that take a tensor map of C: full 32-row x 128-byte slabs leave by TMA store
#ifdef O64_TUNING
    unsigned long long *dbg;  // O64_TRACE=pipe: per-CTA wait/total cycles of the issuing threads
    int probe;   // O64_PROBE: 1 = skip the loads, 2 = skip the MMAs, +4 = skip the epilogue,
                 // +32 = skip the global stores
#endif
    int *status;
    unsigned long long wait_ns;  // budget of every bounded wait, in nanoseconds
    // test hook (kernels instantiated with HOOK = true only, reached through o64_test_*): the
    // producer leaves out the loads of the k-th K block it would issue, so that the stage's "full"
    // barrier never completes and the waits behind it run out; -1 = none
    int test_withhold;
    // split-K: each tile's K blocks are divided over split_k work items whose partial sums are
    // added (fp32 / int32 atomics) into `partial` (fp32 results: a dense [M,N] workspace, finished
    // by a second kernel) or straight into C (int32 results, C zeroed first); 1 = off
    int split_k, kb_per_split;
    void *partial;
    // fused all-gather: the same result tile is also stored into these peer GPUs' copies of C
    // (peer-mapped device pointers to the same element as C); 0 peers = plain GEMM
    int n_peers;
    void *peer_c[7];
    // ... and the rank barriers of that exchange, done by the kernel itself: a block of counters in every
    // rank's memory (xchg_local here, xchg_peer[d] the same block of the rank behind peer_c[d]):
    //   [j]      entry arrivals of rank j: rank j's stream has reached this call, so nothing of it reads
    //            the previous result any more           (first remote store waits for all of them)
    //   [8 + j]  exit arrivals of rank j: all of rank j's stores of this call have been performed
    //            (the kernel does not end before all of them are in)
    //   [16]     calls completed here      [17] CTAs of the running call that have finished storing
    // Counters only grow (compared as signed differences), so a launch replayed from a CUDA graph
    // needs no new parameter.  NULL = the caller orders the ranks itself.
    unsigned *xchg_local;
    unsigned *xchg_peer[7];
    int xchg_rank;
    int xchg_peer_rank[7];
    // the kernel for few rows of A (umma_gemm_skinny.cu): rows in the TMA box of A, stages of its
    // ring, K slices per tile (= CTAs per cluster)
    int sk_a_rows, sk_stages, sk_split;
    // CTA-pair kernels: the first tail_tiles tiles of the walk (the ones a last, partly filled wave
    // of whole tiles would hold) are divided along K over tail_pairs pairs; a pair that does not
    // reach a tile's last K block leaves its partial sums in its slot of tail_slots and sets its
    // words of tail_flags; the pair that does reach it adds them up.  0 tiles = off.
    int tail_tiles, tail_pairs;
    void *tail_slots;
    unsigned *tail_flags;
    long long tail_slot_bytes;  // bytes of one pair's slot
};

// Tensor maps (as bytes, like the map of C the bulk-store epilogue uses) of the peers' copies of the
// result, in the order of UmmaParams::peer_c: the fused exchange then sends a finished slab with one
// bulk-tensor store per peer.
struct PeerMaps {
    CUtensorMap m[7];
};

constexpr int kBlockM = 128;
constexpr int kRowBytes = 128;  // bytes of K (or of N for a [K,N] operand) per shared-memory row
constexpr int kThreads = 192;
constexpr int kABytes = kBlockM * kRowBytes;

// Status-word detail codes: which wait gave up.
constexpr int kWaitProducerEmpty = 0x101;
constexpr int kWaitMmaFull = 0x102;
constexpr int kWaitMmaAccEmpty = 0x103;
constexpr int kWaitEpiAccFull = 0x104;

__device__ __forceinline__ void tile_coords(int t, const UmmaParams &p, int &mb, int &nb) {
    if (p.raster == 0) {
        const int per_group = p.group_m * p.num_n_tiles;
        const int g = t / per_group;
        const int first = g * p.group_m;
        const int gsz = min(p.num_m_tiles - first, p.group_m);
        const int r = t - g * per_group;
        mb = first + r % gsz;
        nb = r / gsz;
    } else {
        const int per_group = p.group_m * p.num_m_tiles;
        const int g = t / per_group;
        const int first = g * p.group_m;
        const int gsz = min(p.num_n_tiles - first, p.group_m);
        const int r = t - g * per_group;
        nb = first + r % gsz;
        mb = r / gsz;
    }
}

__device__ __forceinline__ float act_apply(float x, int act) {
    switch (act) {
    case O64_ACT_RELU: return fmaxf(x, 0.0f);
    case O64_ACT_GELU_TANH: {
        const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
        return 0.5f * x * (1.0f + tanhf(u));
    }
    case O64_ACT_GELU_ERF: return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
    case O64_ACT_SILU: return x / (1.0f + expf(-x));
    default: return x;
    }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}


// ------------------------------------------------------------------------------------------------
// The work list of one CTA pair.  Whole tiles are dealt out pair by pair (pair p takes tiles
// tail_tiles + p, + pairs, + 2 pairs, ...).  When the tile count does not divide by the number of
// pairs, a last wave of whole tiles would leave pairs idle; those tail_tiles tiles come FIRST and are
// cut along K instead: their tail_tiles * num_k_blocks K blocks form one line that is dealt out evenly,
// pair q taking blocks [U q / tail_pairs, U (q + 1) / tail_pairs).  A pair's piece can start inside a
// tile and end inside another:
//   * the piece of its last tile, if it stops short of that tile's last K block, makes the pair a
//     CONTRIBUTOR: it writes the raw partial accumulator into its slot and raises its flags.  This
//     item runs first, so that no contributor ever waits for anybody before it delivers;
//   * every other tile of the range ends at the tile's last K block and is OWNED: if the piece
//     starts inside the tile, the owner adds the slots of the pairs before it (in a fixed order,
//     so results do not depend on timing) before it applies the epilogue.
// This is the blocking of the K strip the reference's cache model applies when a level cannot hold
// a whole strip (osprey/be/lno/cache_model.cxx:6650-6727), used here to level the last wave.
// ------------------------------------------------------------------------------------------------
enum : int { WORK_FULL = 0, WORK_PARTIAL_OUT = 1, WORK_FIXUP_IN = 2 };
struct WorkItem {
    int tile, kb0, kb1, mode;
};
constexpr int kWaitTailFlag = 0x401;

__device__ __forceinline__ long long tail_range_begin(const UmmaParams &p, int pair) {
    return (long long)p.tail_tiles * p.num_k_blocks * pair / p.tail_pairs;
}

// The idx-th item of pair `pair`; false when the list is exhausted.  TAIL = false: the kernel was
// built without the K split (whole tiles only, none of the split's code or registers).
template <bool TAIL>
__device__ __forceinline__ bool work_item(const UmmaParams &p, int pair, int num_pairs, int idx, WorkItem &w) {
    const int kb = p.num_k_blocks;
    const int num_tiles = p.num_m_tiles * p.num_n_tiles;
    int n_tail = 0;
    if (TAIL && p.tail_tiles > 0 && pair < p.tail_pairs) {
        const long long a = tail_range_begin(p, pair), b = tail_range_begin(p, pair + 1);
        if (b > a) {
            const int tf = (int)(a / kb), tl = (int)((b - 1) / kb);
            const int end_in_tile = (int)(b - (long long)tl * kb);  // 1 .. kb
            const int contrib = end_in_tile < kb ? 1 : 0;
            n_tail = tl - tf + 1;  // contributor piece (if any) + owned tiles
            if (idx < n_tail) {
                if (contrib && idx == 0) {
                    const long long t0 = (long long)tl * kb;
                    w.tile = tl;
                    w.kb0 = (int)((a > t0 ? a : t0) - t0);
                    w.kb1 = end_in_tile;
                    w.mode = WORK_PARTIAL_OUT;
                } else {
                    const int t = tf + idx - contrib;
                    const long long t0 = (long long)t * kb;
                    w.tile = t;
                    w.kb0 = a > t0 ? (int)(a - t0) : 0;
                    w.kb1 = kb;
                    w.mode = w.kb0 > 0 ? WORK_FIXUP_IN : WORK_FULL;
                }
                return true;
            }
        }
    }
    const long long t = (TAIL ? (long long)p.tail_tiles : 0LL) + pair + (long long)(idx - n_tail) * num_pairs;
    if (t >= num_tiles) return false;
    w.tile = (int)t;
    w.kb0 = 0;
    w.kb1 = kb;
    w.mode = WORK_FULL;
    return true;
}

// First of the pairs whose pieces of tile `tile` the owner `pair` has to add: pairs first .. pair - 1.
__device__ __forceinline__ int tail_first_contributor(const UmmaParams &p, int pair, int tile) {
    const long long t0 = (long long)tile * p.num_k_blocks;
    int q = pair - 1;
    while (q > 0 && tail_range_begin(p, q) > t0) --q;
    return q;
}

// A pair's slot holds, per CTA and per 32-row unit of its accumulator rows, BLOCK_N raw 32-bit
// columns in the order the epilogue warps hold them in registers: [chunk of 32 columns][group of 4
// columns][lane] as 16-byte words, so that contributor and owner both move 512 contiguous bytes per
// warp instruction and no transposition is needed.
template <int BLOCK_N>
__device__ __forceinline__ uint4 *tail_unit(const UmmaParams &p, int pair, int rank, int units_per_cta, int unit) {
    constexpr long long kUnitBytes = 32LL * BLOCK_N * 4;
    return reinterpret_cast<uint4 *>(static_cast<uint8_t *>(p.tail_slots) + (long long)pair * p.tail_slot_bytes +
                                     ((long long)rank * units_per_cta + unit) * kUnitBytes);
}

__device__ __forceinline__ unsigned *tail_flag(const UmmaParams &p, int pair, int rank, int warp_slot) {
    return p.tail_flags + ((pair * 2 + rank) * 8 + warp_slot);
}

// Contributor: this warp's columns [c_begin, c_end) of the finished partial accumulator go to the slot.
// Two register sets: the next chunk is on its way out of tensor memory while this one is stored.
static __device__ __noinline__ void tail_store_partial(uint32_t t_row, uint4 *unit, int c_begin, int c_end) {
    const int lane = threadIdx.x & 31;
    auto put = [&](const uint32_t (&v)[32], int c) {
        uint4 *dst = unit + (c >> 5) * 256 + lane;
#pragma unroll
        for (int q = 0; q < 8; ++q) dst[q * 32] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    };
    uint32_t va[32], vb[32];
    __syncwarp();
    tmem_ld_32x32(t_row + c_begin, va);
#pragma unroll 1
    for (int c = c_begin; c < c_end; c += 64) {
        tmem_ld_wait();
        __syncwarp();
        if (c + 32 < c_end) tmem_ld_32x32(t_row + c + 32, vb);
        put(va, c);
        if (c + 32 < c_end) {
            tmem_ld_wait();
            __syncwarp();
            if (c + 64 < c_end) tmem_ld_32x32(t_row + c + 64, va);
            put(vb, c + 32);
        }
    }
}

// Flag words start at zero and return to zero by themselves, so that a launch replayed from a CUDA
// graph (whose parameters are frozen) finds them as the first launch did:
//   contributor   stores its partial sums, fences, sets the word to 1;
//   each consumer waits until the word is not zero, reads the slot, then adds 1; the consumer that
//                 brings it to 1 + `consumers` sets it back to zero.
// A launch that ended in a time-out can leave words set; o64_last_status clears them when it
// reports one.
__device__ __forceinline__ void tail_publish(unsigned *flag) {
    __threadfence();
    __syncwarp();
    if ((threadIdx.x & 31) == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(1u) : "memory");
}

// Consumer: waits (bounded) until a contributor's word is set.  Whole-warp call.
__device__ __forceinline__ bool tail_wait_flag(const unsigned *flag, volatile int *abort_flag, int *status_word,
                                               unsigned long long budget_ns) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0) {
        uint64_t t0 = 0;
        uint32_t probes = 0;
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v != 0) break;
            if ((++probes & 63u) == 0) {
                if (*abort_flag) {
                    ok = false;
                    break;
                }
                const uint64_t now = globaltimer_ns();
                if (t0 == 0) {
                    t0 = now;
                } else if (now - t0 > budget_ns) {
                    atomicCAS(status_word, 0, kWaitTailFlag);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
            }
            __nanosleep(64);
        }
    }
    return __shfl_sync(0xffffffffu, ok, 0);
}

// Consumer, after it has read the slot: the last of `consumers` clears the word.  Whole-warp call.
__device__ __forceinline__ void tail_release(unsigned *flag, unsigned consumers) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) {
        if (atomicAdd(flag, 1u) == consumers) atomicExch(flag, 0u);
    }
}

// ---- rank barriers of the fused exchange (see UmmaParams::xchg_local) ------------------------------
constexpr int kWaitXchgEntry = 0x501;
constexpr int kWaitXchgExit = 0x502;

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *ptr) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned *ptr, unsigned v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}

// One thread: waits (bounded) until every peer's counter at `base` has reached `target`.
static __device__ __noinline__ bool xchg_wait_all(const UmmaParams &p, int base, unsigned target, volatile int *abort_flag,
                                              int code) {
    uint64_t t0 = 0;
    uint32_t probes = 0;
    for (int d = 0; d < p.n_peers; ++d) {
        const unsigned *w = p.xchg_local + base + p.xchg_peer_rank[d];
        while ((int)(ld_acquire_sys(w) - target) < 0) {
            if ((++probes & 15u) == 0) {
                if (*abort_flag) return false;
                const uint64_t now = globaltimer_ns();
                if (t0 == 0) {
                    t0 = now;
                } else if (now - t0 > p.wait_ns) {
                    atomicCAS(p.status, 0, code | (p.xchg_peer_rank[d] << 12));
                    *abort_flag = 1;
                    return false;
                }
            }
            __nanosleep(500);
        }
    }
    return true;
}

// Kernel start, one thread of the whole grid: tells every peer that this rank has reached the call.
static __device__ __noinline__ void xchg_announce_entry(const UmmaParams &p) {
    for (int d = 0; d < p.n_peers; ++d) red_release_sys_add(p.xchg_peer[d] + p.xchg_rank, 1u);
}

// Epilogue warps, before their first store of the call (whole-warp call): all ranks have arrived.
// Polling is kept away from the line the peers write: ONE thread of the grid (CTA 0's `leader` warp)
// reads the peers' arrival words and then publishes the call number in a word of its own; one
// warp per CTA polls that word and sets `ready_smem`; the CTA's other epilogue warps watch
// shared memory.  (With every epilogue warp of every CTA polling the arrival words, the peers'
// atomics queued behind thousands of loads on one L2 line: 8 GPUs ran five times slower.)
static __device__ __noinline__ bool xchg_wait_entry(const UmmaParams &p, volatile int *abort_flag, volatile int *ready_smem,
                                                  bool leader) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0) {
        if (leader) {
            // [kXchgCalls] is written only by the last CTA of a call, after every CTA has passed this point
            const unsigned call = p.xchg_local[kXchgCalls] + 1u;
            if (blockIdx.x == 0) {
                ok = xchg_wait_all(p, 0, call, abort_flag, kWaitXchgEntry);
                if (ok) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.xchg_local + kXchgReady), "r"(call) : "memory");
            } else {
                uint64_t t0 = 0;
                uint32_t probes = 0;
                for (;;) {
                    unsigned v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.xchg_local + kXchgReady) : "memory");
                    if ((int)(v - call) >= 0) break;
                    if ((++probes & 15u) == 0) {
                        if (*abort_flag) { ok = false; break; }
                        const uint64_t now = globaltimer_ns();
                        if (t0 == 0) {
                            t0 = now;
                        } else if (now - t0 > p.wait_ns) {
                            atomicCAS(p.status, 0, kWaitXchgEntry | 0x80);
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                    }
                    __nanosleep(1000);
                }
            }
            *ready_smem = ok ? 1 : -1;
        } else {
            uint32_t probes = 0;
            uint64_t t0 = 0;
            int v;
            while ((v = *ready_smem) == 0) {
                if ((++probes & 63u) == 0) {
                    if (*abort_flag) { v = -1; break; }
                    const uint64_t now = globaltimer_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > 2 * p.wait_ns) { v = -1; break; }  // the leader gives up first and says so
                }
                __nanosleep(200);
            }
            ok = v > 0;
        }
    }
    return __shfl_sync(0xffffffffu, ok, 0);
}

// Every thread that stored to a peer, after its last store.
// (Slabs sent by bulk-tensor stores: the issuing lane has waited for its bulk groups before this; the
// proxy fence orders what the TMA unit wrote before the counters this thread's CTA will signal.)
__device__ __forceinline__ void xchg_stores_done() {
    asm volatile("fence.proxy.async;" ::: "memory");
    __threadfence_system();
}

// Teardown, one thread per CTA, after a CTA-wide barrier behind the epilogue: the last CTA of the grid
// tells the peers that this rank's stores are complete and waits for theirs.
static __device__ __noinline__ void xchg_finish(const UmmaParams &p, volatile int *abort_flag) {
    __threadfence();
    const unsigned done = atomicAdd(p.xchg_local + kXchgCtasDone, 1u);
    if (done != gridDim.x - 1) return;
    __threadfence();
    p.xchg_local[kXchgCtasDone] = 0;
    const unsigned call = p.xchg_local[kXchgCalls] + 1u;
    __threadfence_system();
    for (int d = 0; d < p.n_peers; ++d) red_release_sys_add(p.xchg_peer[d] + kXchgExit + p.xchg_rank, 1u);
    (void)xchg_wait_all(p, kXchgExit, call, abort_flag, kWaitXchgExit);
    p.xchg_local[kXchgCalls] = call;
    __threadfence();
}

// What an owner adds to its accumulator before the epilogue: the same unit of every contributor.
// The contributors are consecutive pairs, so their units lie one slot apart.
struct TailFix {
    const uint8_t *first_unit = nullptr;  // this warp's unit in the first contributor's slot
    long long stride = 0;                 // bytes from one pair's slot to the next
    int n = 0;                            // contributors
};

// Owner: adds the contributors' partial sums for columns [c_begin, c_end) INTO the accumulator in
// tensor memory (tcgen05.ld, add, tcgen05.st), one contributor after the other in pair order, so the
// ordinary epilogue then runs on the complete sums.  The slot reads come through L2 from another SM
// at about a microsecond per round trip: each chunk's reads are issued one chunk ahead, so that the
// loop runs at the rate of the loads, not of their latency.
// (Not inlined: a rare path whose two register sets must not cost the ordinary epilogue its registers.)
template <bool INTEGER>
__device__ __noinline__ void tail_reduce(uint32_t t_row, int c_begin, int c_end, const TailFix &fix) {
    const int lane = threadIdx.x & 31;
    auto fetch = [&](uint4 (&x)[8], const uint4 *unit, int c) {
        const uint4 *src = unit + (c >> 5) * 256 + lane;
#pragma unroll
        for (int q = 0; q < 8; ++q) x[q] = __ldcg(src + q * 32);  // written by another SM: read through L2
    };
    auto add = [&](int c, const uint4 (&x)[8]) {
        uint32_t v[32];
        tmem_ld_32x32(t_row + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const uint32_t w[4] = {x[q].x, x[q].y, x[q].z, x[q].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if constexpr (INTEGER)
                    v[4 * q + e] += w[e];
                else
                    v[4 * q + e] = __float_as_uint(__uint_as_float(v[4 * q + e]) + __uint_as_float(w[e]));
            }
        }
        tmem_st_32x32(t_row + c, v);
    };
    for (int f = 0; f < fix.n; ++f) {
        const uint4 *unit = reinterpret_cast<const uint4 *>(fix.first_unit + f * fix.stride);
        uint4 xa[8], xb[8];
        fetch(xa, unit, c_begin);
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 64) {
            if (c + 32 < c_end) fetch(xb, unit, c + 32);
            __syncwarp();
            add(c, xa);
            if (c + 32 < c_end) {
                if (c + 64 < c_end) fetch(xa, unit, c + 64);
                __syncwarp();
                add(c + 32, xb);
            }
        }
        tmem_st_wait();  // the next contributor (or the epilogue) reads what was just written
        __syncwarp();
    }
}

constexpr int kEpiStagingBytesPerWarp = 4096;  // 32 rows x 128 bytes
constexpr int kEpiStagingBytes = 4 * kEpiStagingBytesPerWarp;

// Applies the fused tail to 32 accumulator values of one row (columns col0 .. col0+31).
template <int ACT>
__device__ __forceinline__ float act_fixed(float x) {
    if constexpr (ACT == O64_ACT_RELU) {
        return fmaxf(x, 0.0f);
    } else if constexpr (ACT == O64_ACT_GELU_TANH) {
        const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
        return 0.5f * x * (1.0f + tanhf(u));
    } else if constexpr (ACT == O64_ACT_GELU_ERF) {
        return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
    } else if constexpr (ACT == O64_ACT_SILU) {
        return x / (1.0f + expf(-x));
    } else {
        return x;
    }
}

// 32 consecutive values of a per-column vector (bias, scale_b) starting at column col0, the same for
// every lane: eight 16-byte loads where the vector allows them (a per-element load of the same
// address by all lanes costs the load pipe 64 instructions per chunk instead of 16), else scalar loads
// clamped to the last column.  base == NULL gives `neutral`.
__device__ __forceinline__ void load_column_values(const float *base, int col0, int N, float neutral, float (&out)[32]) {
    if (!base) {
#pragma unroll
        for (int j = 0; j < 32; ++j) out[j] = neutral;
    } else if (col0 + 32 <= N && ((reinterpret_cast<uintptr_t>(base + col0) & 15u) == 0)) {
        const float4 *src = reinterpret_cast<const float4 *>(base + col0);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 x = __ldg(src + q);
            out[4 * q] = x.x, out[4 * q + 1] = x.y, out[4 * q + 2] = x.z, out[4 * q + 3] = x.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) out[j] = __ldg(base + min(col0 + j, N - 1));
    }
}

// The activation is a template parameter: with a run-time switch inside the element loop the
// compiler evaluates every branch (tanhf, erff, expf) for every element, which made the
// epilogue of a 128 x 256 tile as long as its main loop.
template <int EPI, int ACT>
__device__ __forceinline__ void epilogue_math(const UmmaParams &p, const uint32_t (&v)[32],
                                              const uint32_t (&u)[32], int col0, float sa, float (&f)[32]) {
    if constexpr (EPI == EPI_SWIGLU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float x = __uint_as_float(v[j]);
            f[j] = (x / (1.0f + expf(-x))) * __uint_as_float(u[j]);
        }
    } else if constexpr (epi_scaled(EPI)) {
        float sb[32], bias[32];
        load_column_values(p.scale_b, col0, p.N, 1.0f, sb);
        load_column_values(p.bias, col0, p.N, 0.0f, bias);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float acc = epi_int_acc(EPI) ? __int2float_rn((int)v[j]) : __uint_as_float(v[j]);
            // each operation rounded by itself: the CPU restatement computes the same bits
            const float x = __fadd_rn(__fmul_rn(acc, __fmul_rn(sa, sb[j])), bias[j]);
            f[j] = act_fixed<ACT>(x);
        }
    } else {
        if (p.bias) {
            float bias[32];
            load_column_values(p.bias, col0, p.N, 0.0f, bias);
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = act_fixed<ACT>(__uint_as_float(v[j]) + bias[j]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = act_fixed<ACT>(__uint_as_float(v[j]));
        }
    }
}

// Conversions of the requantising tails: round to nearest even, saturating.
__device__ __forceinline__ uint32_t quant_s8(float x) {
    int q = __float2int_rn(x);  // NaN -> 0
    q = max(-128, min(127, q));
    return (uint32_t)q & 0xffu;
}
__device__ __forceinline__ uint32_t quant_e4m3(float x) {
    return (uint32_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
template <int EPI>
__device__ __forceinline__ uint32_t quant4(float a, float b, float c, float d) {
    if constexpr (EPI == EPI_ISCALED_S8)
        return quant_s8(a) | (quant_s8(b) << 8) | (quant_s8(c) << 16) | (quant_s8(d) << 24);
    else
        return quant_e4m3(a) | (quant_e4m3(b) << 8) | (quant_e4m3(c) << 16) | (quant_e4m3(d) << 24);
}

// Drains one finished accumulator buffer: this warp's 32 lanes (TMEM lane quarter) by
// 128-byte-wide column slabs.  tcgen05.ld gives every thread one ROW of the slab; a store
// straight from those registers would have each warp instruction touch 32 rows with 16 bytes
// each (measured: about 50 000 cycles per 128 x 256 tile, slower than the tile's main loop).
// So the slab goes through a warp-private, XOR-swizzled shared-memory patch and comes back
// transposed: each store instruction then writes four full 128-byte row segments.
// Whole-warp call; rows >= M and columns >= N are computed but not stored.
//   row0     global row of lane 0 of this warp      n0   first output column of the tile
//   t_row    TMEM address of (first lane of the quarter, first column of the buffer)
//   staging  this warp's 4 KB patch of shared memory
//   tm_c     NULL, or a tensor map of C as bytes ([M][N * element size], box 128 bytes x 32 rows, 128-byte
//            swizzle - the patch's own layout): a finished slab then leaves with ONE bulk-tensor store
//            issued by one lane instead of eight vector stores per lane.  Measured on stores alone,
//            eight warps per SM: 3.3 TB/s with 16-byte vector stores, 5.2 TB/s with bulk stores.
template <int EPI, int BLOCK_N, int ACT>
__device__ __forceinline__ void epilogue_tile_act(const UmmaParams &p, long long row0, int n0,
                                                  uint32_t t_row, uint8_t *staging, int c_begin, int c_end,
                                                  const CUtensorMap *tm_c = nullptr, const PeerMaps *tm_peers = nullptr) {
    constexpr int kOutN = (EPI == EPI_SWIGLU) ? BLOCK_N / 2 : BLOCK_N;
    constexpr int kOutElem = epi_out_bytes(EPI);
    constexpr int kSlabCols = 128 / kOutElem;  // 128 one-byte, 64 bf16 or 32 int32 columns per 128-byte row
    constexpr int kChunksPerSlab = kSlabCols / 32;
    const int lane = threadIdx.x & 31;
    const long long row = row0 + lane;
    const bool row_ok = row < p.M;
    float sa = 1.0f;
    if constexpr (epi_scaled(EPI)) {
        if (p.scale_a && row_ok) sa = p.scale_a[row];
    }
    uint4 *patch = reinterpret_cast<uint4 *>(staging);
    const int sw = lane & 7;  // XOR swizzle of the 16-byte chunk index, by row


    // 32-column chunks of the accumulator this warp has to drain (uniform over the warp)
    const int cols_avail = min(c_end, p.N - n0) - c_begin;
    if (cols_avail <= 0) return;
    const int nchunks = (cols_avail + 31) >> 5;

    // one chunk: fused tail on 32 values of this thread's row, into the patch or straight out
    auto process = [&](const uint32_t (&v)[32], const uint32_t (&u)[32], int i) {
        const int c = c_begin + 32 * i;          // column inside the tile
        const int slab_c = c_begin + (i / kChunksPerSlab) * kSlabCols;
        const int h = i % kChunksPerSlab;
        const bool coalesced = p.vec_ok && (n0 + slab_c + kSlabCols <= p.N) && !(O64_PROBE(p) & 32);
        if (tm_c && h == 0 && coalesced) {
            // the bulk store of this warp's previous slab has finished reading the patch
            if (lane == 0) bulk_wait_read_all();
            __syncwarp();
        }
        if constexpr (EPI == EPI_S32) {
            if (coalesced) {
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    patch[lane * 8 + (q ^ sw)] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            } else if (row_ok && !(O64_PROBE(p) & 32)) {
                int32_t *dst = reinterpret_cast<int32_t *>(p.C) + row * p.ldc + n0 + c;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (n0 + c + j < p.N) dst[j] = (int32_t)v[j];
            }
        } else if constexpr (kOutElem == 1) {
            float f[32];
            epilogue_math<EPI, ACT>(p, v, u, n0 + c, sa, f);
            if (coalesced) {  // 32 one-byte results: two 16-byte pieces of the row's 128-byte slab
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    patch[lane * 8 + ((h * 2 + q) ^ sw)] =
                        make_uint4(quant4<EPI>(f[16 * q], f[16 * q + 1], f[16 * q + 2], f[16 * q + 3]),
                                   quant4<EPI>(f[16 * q + 4], f[16 * q + 5], f[16 * q + 6], f[16 * q + 7]),
                                   quant4<EPI>(f[16 * q + 8], f[16 * q + 9], f[16 * q + 10], f[16 * q + 11]),
                                   quant4<EPI>(f[16 * q + 12], f[16 * q + 13], f[16 * q + 14], f[16 * q + 15]));
            } else if (row_ok && !(O64_PROBE(p) & 32)) {
                uint8_t *dst = reinterpret_cast<uint8_t *>(p.C) + row * p.ldc + n0 + c;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (n0 + c + j < p.N) dst[j] = (uint8_t)(EPI == EPI_ISCALED_S8 ? quant_s8(f[j]) : quant_e4m3(f[j]));
            }
        } else {
            float f[32];
            epilogue_math<EPI, ACT>(p, v, u, n0 + c, sa, f);
            if (coalesced) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    patch[lane * 8 + ((h * 4 + q) ^ sw)] =
                        make_uint4(pack_bf16x2(f[8 * q], f[8 * q + 1]), pack_bf16x2(f[8 * q + 2], f[8 * q + 3]),
                                   pack_bf16x2(f[8 * q + 4], f[8 * q + 5]), pack_bf16x2(f[8 * q + 6], f[8 * q + 7]));
            } else if (row_ok && !(O64_PROBE(p) & 32)) {
                __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(p.C) + row * p.ldc + n0 + c;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (n0 + c + j < p.N) dst[j] = __float2bfloat16_rn(f[j]);
            }
        }
        // the chunk that completes a slab sends the patch out, transposed: lane -> (row 4*r + lane/8,
        // 16-byte piece lane%8), four full 128-byte row segments per store instruction
        if (h == kChunksPerSlab - 1 && coalesced && tm_c) {
            fence_proxy_async_smem();  // the patch, written through the generic proxy, as the TMA unit will read it
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(tm_c, smem_u32(staging), (n0 + slab_c) * kOutElem, (int)row0);
                // the exchange step of a column-sharded linear, fused: the same slab into every peer's copy of C
                if (tm_peers)
                    for (int d = 0; d < p.n_peers; ++d)
                        tma_store_2d(&tm_peers->m[d], smem_u32(staging), (n0 + slab_c) * kOutElem, (int)row0);
                bulk_commit_group();
            }
        } else if (h == kChunksPerSlab - 1 && coalesced) {
            __syncwarp();
            const int piece = lane & 7;
            uint8_t *cbase = reinterpret_cast<uint8_t *>(p.C) + (size_t)(n0 + slab_c) * kOutElem + piece * 16;
#pragma unroll
            for (int r4 = 0; r4 < 8; ++r4) {
                const int r = 4 * r4 + (lane >> 3);
                const uint4 val = patch[r * 8 + (piece ^ (r & 7))];
                const long long grow = row0 + r;
                if (grow < p.M) {
                    const size_t off = (size_t)(n0 + slab_c) * kOutElem + piece * 16 + (size_t)grow * p.ldc * kOutElem;
                    *reinterpret_cast<uint4 *>(cbase + (size_t)grow * p.ldc * kOutElem) = val;
                    // the exchange step of a column-sharded linear, fused: push the tile over NVLink
                    // into every peer's copy of C while the next tile's MMAs run
                    for (int d = 0; d < p.n_peers; ++d)
                        *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.peer_c[d]) + off) = val;
                }
            }
            __syncwarp();
        }
    };

    if constexpr (EPI == EPI_SWIGLU || ACT != O64_ACT_NONE) {
        // register-hungry tails (two accumulators, or tanhf / erff / expf): plain load -> wait -> use
#pragma unroll 1
        for (int i = 0; i < nchunks; ++i) {
            uint32_t v[32];
            [[maybe_unused]] uint32_t u[32];
            __syncwarp();
            tmem_ld_32x32(t_row + c_begin + 32 * i, v);
            if constexpr (EPI == EPI_SWIGLU) tmem_ld_32x32(t_row + kOutN + c_begin + 32 * i, u);
            tmem_ld_wait();
            if constexpr (EPI == EPI_SWIGLU)
                process(v, u, i);
            else
                process(v, v, i);
        }
    } else {
        // two register sets: the load of the next chunk is in flight while this one is processed
        uint32_t va[32], vb[32];
        __syncwarp();
        tmem_ld_32x32(t_row + c_begin, va);
#pragma unroll 1
        for (int i = 0; i < nchunks; i += 2) {
            tmem_ld_wait();
            __syncwarp();
            if (i + 1 < nchunks) tmem_ld_32x32(t_row + c_begin + 32 * (i + 1), vb);
            process(va, va, i);
            if (i + 1 < nchunks) {
                tmem_ld_wait();
                __syncwarp();
                if (i + 2 < nchunks) tmem_ld_32x32(t_row + c_begin + 32 * (i + 2), va);
                process(vb, vb, i + 1);
            }
        }
    }
}

// c_begin .. c_end: the output columns of the tile this warp drains (the whole tile by default;
// kernels that put two warps on one lane quarter give each half of the columns).
template <int EPI, int BLOCK_N>
__device__ __forceinline__ void epilogue_tile(const UmmaParams &p, long long row0, int n0,
                                              uint32_t t_row, uint8_t *staging, int c_begin = 0,
                                              int c_end = (EPI == EPI_SWIGLU) ? BLOCK_N / 2 : BLOCK_N,
                                              const CUtensorMap *tm_c = nullptr, const PeerMaps *tm_peers = nullptr) {
    if constexpr (EPI == EPI_BF16 || epi_scaled(EPI)) {
        switch (p.act) {  // uniform: one branch per tile, not per element
        case O64_ACT_RELU: epilogue_tile_act<EPI, BLOCK_N, O64_ACT_RELU>(p, row0, n0, t_row, staging, c_begin, c_end, tm_c, tm_peers); break;
        case O64_ACT_GELU_TANH: epilogue_tile_act<EPI, BLOCK_N, O64_ACT_GELU_TANH>(p, row0, n0, t_row, staging, c_begin, c_end, tm_c, tm_peers); break;
        case O64_ACT_GELU_ERF: epilogue_tile_act<EPI, BLOCK_N, O64_ACT_GELU_ERF>(p, row0, n0, t_row, staging, c_begin, c_end, tm_c, tm_peers); break;
        case O64_ACT_SILU: epilogue_tile_act<EPI, BLOCK_N, O64_ACT_SILU>(p, row0, n0, t_row, staging, c_begin, c_end, tm_c, tm_peers); break;
        default: epilogue_tile_act<EPI, BLOCK_N, O64_ACT_NONE>(p, row0, n0, t_row, staging, c_begin, c_end, tm_c, tm_peers); break;
        }
    } else {
        epilogue_tile_act<EPI, BLOCK_N, O64_ACT_NONE>(p, row0, n0, t_row, staging, c_begin, c_end, tm_c, tm_peers);
    }
}

// An owner of a tile cut along K completes the sums of its columns in tensor memory (for the SwiGLU
// epilogue: the gate and the up columns), then the ordinary epilogue runs.
template <int EPI, int BLOCK_N>
__device__ __forceinline__ void tail_complete(uint32_t t_row, int c_begin, int c_end, const TailFix &fix) {
    constexpr int kOutN = (EPI == EPI_SWIGLU) ? BLOCK_N / 2 : BLOCK_N;
    if (fix.n == 0) return;
    tail_reduce<epi_int_acc(EPI)>(t_row, c_begin, c_end, fix);
    if constexpr (EPI == EPI_SWIGLU) tail_reduce<false>(t_row, kOutN + c_begin, kOutN + c_end, fix);
}

// Split-K epilogue: adds this work item's raw partial sums into `dst` ([M, ldd] of 4-byte
// elements) with atomics.  Through the same swizzled patch as the normal epilogue so that a warp
// instruction adds to four full 128-byte row segments.
template <bool INTEGER>
__device__ __forceinline__ void epilogue_partial(const UmmaParams &p, void *dst, long long ldd, long long row0,
                                                 int n0, uint32_t t_row, uint8_t *staging, int ncols) {
    const int lane = threadIdx.x & 31;
    uint4 *patch = reinterpret_cast<uint4 *>(staging);
    const int sw = lane & 7;
    const int cols_avail = min(ncols, p.N - n0);
    const int nchunks = cols_avail > 0 ? (cols_avail + 31) >> 5 : 0;
    // fp32 sums go out four at a time when the rows of dst allow 16-byte accesses
    const bool v4ok = !INTEGER && ((ldd & 3) == 0) && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) && ((n0 & 3) == 0);
#pragma unroll 1
    for (int i = 0; i < nchunks; ++i) {
        uint32_t v[32];
        __syncwarp();
        tmem_ld_32x32(t_row + 32 * i, v);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 8; ++q)
            patch[lane * 8 + (q ^ sw)] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        __syncwarp();
        const int piece = lane & 7;
#pragma unroll
        for (int r4 = 0; r4 < 8; ++r4) {
            const int r = 4 * r4 + (lane >> 3);
            const uint4 val = patch[r * 8 + (piece ^ (r & 7))];
            const long long grow = row0 + r;
            const int col = n0 + 32 * i + piece * 4;
            if (grow < p.M && v4ok && col + 3 < p.N) {
                red_add_v4_f32(reinterpret_cast<float *>(dst) + grow * ldd + col, __uint_as_float(val.x),
                               __uint_as_float(val.y), __uint_as_float(val.z), __uint_as_float(val.w));
            } else if (grow < p.M) {
                const uint32_t w[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (col + e < p.N) {
                        if constexpr (INTEGER)
                            atomicAdd(reinterpret_cast<int *>(dst) + grow * ldd + col + e, (int)w[e]);
                        else
                            atomicAdd(reinterpret_cast<float *>(dst) + grow * ldd + col + e, __uint_as_float(w[e]));
                    }
                }
            }
        }
        __syncwarp();
    }
}

// Per-device set-up of one kernel instantiation.  cudaFuncSetAttribute and the cluster occupancy
// query act on the CURRENT device, so a process that drives several GPUs needs them once per
// (instantiation, device); each launcher keeps one of these in a function-local static.
constexpr int kMaxDevices = 64;
struct KernelSetup {
    std::mutex mu;
    bool done[kMaxDevices] = {};
    int max_clusters[kMaxDevices] = {};
    // Runs `setup(&max_clusters)` (returns an O64 status) the first time this instantiation is
    // launched on the current device; *clusters receives the value it stored.
    template <typename F>
    int once(F setup, int *clusters) {
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
            (void)cudaGetLastError();
            return O64_ERR_CUDA;
        }
        std::lock_guard<std::mutex> lock(mu);
        if (!done[dev]) {
            int n = 0;
            const int rc = setup(&n);
            if (rc) return rc;
            max_clusters[dev] = n;
            done[dev] = true;
        }
        if (clusters) *clusters = max_clusters[dev];
        return O64_OK;
    }
};

// Decides, for a launch on `pairs` CTA pairs, whether the tiles of the last, partly filled wave are
// cut along K (see work_item) and over how many pairs; needs the slot and flag memory in `p`.
// slot_bytes: one pair's slot for this kernel; capacity: bytes behind p.tail_slots.
void plan_tail(UmmaParams &p, int pairs, long long slot_bytes, long long capacity);

// host helpers shared by the launchers (umma_gemm.cu)
// 2-D row-major tensor [rows, cols] with `ld` elements between rows; box of box_cols x box_rows;
// 128-byte swizzle; out-of-range elements read as zero.
int encode_2d(CUtensorMap *tm, int kind, const void *base, int64_t rows, int64_t cols, int64_t ld,
              int box_cols, int box_rows);
// The kernel for M <= 128 (umma_gemm_skinny.cu); `p` carries the fields common to all kernels.
int umma_launch_skinny(const UmmaCall &c, UmmaParams p);
int umma_launch_pair(const UmmaCall &c, const CUtensorMap &ta, const CUtensorMap &tb,
                     const CUtensorMap &tb2, const UmmaParams &p);
// Tensor map of a result matrix as bytes: [rows][cols * elem bytes], pitch ld * elem, box 128 bytes x 32 rows.
int encode_c_bytes(CUtensorMap *tm, void *base, int64_t rows, int64_t cols, int64_t ld, int elem);
int umma_launch_wide(const UmmaCall &c, const CUtensorMap &ta, const CUtensorMap &tb,
                     const CUtensorMap &tb2, const UmmaParams &p);

}  // namespace o64
