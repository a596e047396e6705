// Host-side interface of the tcgen05 GEMM kernels (umma_gemm.cu).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "../../include/o64gemm.h"

namespace o64 {

constexpr int kTailMaxPairs = 80;                 // flag words cover this many CTA pairs
constexpr int kTailFlagWords = kTailMaxPairs * 16;  // [pair][CTA of the pair][8 epilogue warps]
constexpr size_t kTailSlotBytesMax = 512 * 1024;   // a pair's slot in the 512-row kernel
constexpr unsigned long long kDefaultWaitNs = 2000000000ull;  // two seconds

// Fused tails.  The "scaled" ones compute  act( acc * (scale_a[m] * scale_b[n]) + bias[n] )  in fp32 with
// every operation rounded by itself (no fused multiply-add), so that a CPU restatement gives the same
// bits, and then convert: to bf16, or - the requantising forms - to e4m3 / int8, round to nearest
// even, saturating.
enum : int {
    EPI_BF16 = 0,          // fp32 accumulator: act(acc + bias) -> bf16
    EPI_SWIGLU = 1,        // two fp32 accumulators: silu(gate) * up -> bf16
    EPI_SCALED_BF16 = 2,   // fp32 accumulator (fp8 operands), scaled -> bf16
    EPI_S32 = 3,           // int32 accumulator as it is
    EPI_SCALED_E4M3 = 4,   // fp32 accumulator (fp8 operands), scaled -> e4m3
    EPI_ISCALED_BF16 = 5,  // int32 accumulator (int8 operands), scaled -> bf16
    EPI_ISCALED_S8 = 6     // int32 accumulator (int8 operands), scaled -> int8
};
__host__ __device__ constexpr bool epi_scaled(int e) { return e == EPI_SCALED_BF16 || e == EPI_SCALED_E4M3 || e == EPI_ISCALED_BF16 || e == EPI_ISCALED_S8; }
__host__ __device__ constexpr bool epi_int_acc(int e) { return e == EPI_S32 || e == EPI_ISCALED_BF16 || e == EPI_ISCALED_S8; }
__host__ __device__ constexpr int epi_out_bytes(int e) { return e == EPI_S32 ? 4 : ((e == EPI_SCALED_E4M3 || e == EPI_ISCALED_S8) ? 1 : 2); }

// One GEMM on the tensor cores.  A is [M,K] row-major.  B is [N,K] row-major (b_kn == false)
// or [K,N] row-major (b_kn == true, bf16 only).  For EPI_SWIGLU, B and B2 are the gate and up
// weights, both [K,N], and C is [M,N].  Leading dimensions in elements.
struct UmmaCall {
    int kind;  // O64_KIND_BF16 / O64_KIND_FP8 / O64_KIND_S8
    bool b_kn;
    int epi;
    int64_t M, N, K;
    const void *A;
    int64_t lda;
    const void *B;
    const void *B2;
    int64_t ldb;
    void *C;
    int64_t ldc;
    const float *bias;
    const float *scale_a;
    const float *scale_b;
    int act;
    o64_plan_t plan;
    int *status_word;  // device int, 0 = ok
    cudaStream_t stream;
    bool split_ready = false;  // split-K: the caller has zeroed `partial` (or C, for int32 results)
    void *partial = nullptr;   // split-K: zeroed fp32 [M,N] workspace (fp32-accumulating kinds)
    int n_peers = 0;           // fused all-gather: peer copies of C (same element as C), at most 7
    void *peer_c[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    // ... with the rank barriers done by the kernel (UmmaParams::xchg_local); NULL = the caller's business
    unsigned *xchg_local = nullptr;
    unsigned *xchg_peer[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int xchg_rank = 0;
    int xchg_peer_rank[7] = {0, 0, 0, 0, 0, 0, 0};
    bool may_allocate = true;  // false: never allocate (the pipeline trace, which needs a buffer, stays off)
    unsigned long long wait_ns = 0;  // budget of the kernels' bounded waits; 0 = kDefaultWaitNs
    // CTA-pair kernels, K split of the last wave's tiles: slot memory (tail_bytes) and flag words
    // (kTailFlagWords, zero between launches: the kernels leave them so); NULL = no split
    void *tail_slots = nullptr;
    unsigned *tail_flags = nullptr;
    size_t tail_bytes = 0;
    int test_withhold = -1;          // o64_test_* only: K block whose loads the producer leaves out
};

// Layout of the fused exchange's counter block (UmmaParams::xchg_local), in 32-bit words.
// entry [0..7] and exit [8..15] arrivals share the line the peers write; what this GPU's own CTAs
// poll and count lives on the next line
constexpr int kXchgExit = 8, kXchgCalls = 32, kXchgCtasDone = 33, kXchgReady = 34, kXchgWords = 64;

// Validates alignment, encodes the tensor maps and launches.  Returns O64_OK or an error code.
int umma_launch(const UmmaCall &call);

// Model and decision of the K split of a last, partly filled wave (plan.cpp); force: -1 = decide,
// 0 = never, 1 = whenever a last wave is partly filled.
long long tail_model(long long tiles, int pairs, long long kb, int rows_per_cta, long long max_pairs_by_memory,
                     int force, int *tail_tiles, int *tail_pairs);

// Tiles and CTA pairs of the K split the last CTA-pair launch of this thread chose (0, 0: none).
void last_tail_split(int *tiles, int *pairs);
// Test hook: -1 = the model decides (default), 0 = never split, 1 = split whenever a last wave is partly filled.
void force_tail_split(int mode);

// K slices per tile (CTAs per cluster) the kernel for few rows of A uses for a shape.
int umma_skinny_split(int64_t M, int64_t N, int64_t K, int elem, int num_ctas, int bn = 256);

// Fills tile_*, stages, group_m, num_ctas, ... for a shape; applies `pin` (fields != 0) and the
// O64_LNO environment override.  Pure host code.
void plan_choose(int kind, int epi, int64_t M, int64_t N, int64_t K, int num_sms,
                 const o64_plan_t *pin, o64_plan_t *out);

}  // namespace o64
