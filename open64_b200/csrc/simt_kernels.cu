// CUDA-core kernels: the fp32 fused linear / strided GEMM (FFMA), the strided GEMV, the
// one-thread-per-output reference kernels and the slab permute.
//
// The fp32 kernel keeps fp32 arithmetic end to end (no TF32): the fused linear is checked
// against the CPU loop nest to 1e-4 relative, and the compat entry points promise the
// reference runtime's semantics (osprey/libfi/matrix/xgemmx.h:172-236).
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "../../include/o64gemm.h"
#include "simt_kernels.cuh"

namespace o64 {

__device__ __forceinline__ float act_f32(float x, int act) {
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

struct SimtParams {
    long long M, N, K;
    float alpha, beta;
    const float *A;
    long long a1, a2;
    const float *B;
    long long b1, b2;
    float *C;
    long long c1, c2;
    const float *bias;
    int act;
    int a_k_fast;  // A's K index is the contiguous one
    int b_n_fast;  // B's N index is the contiguous one
    int c_n_fast;
};

// BM x BN tile per CTA, BK deep, TM x TN outputs per thread.  The tile loop is the K strip
// of the reference's cache blocking; the TM x TN register block is its unroll-and-jam
// (osprey/be/lno/snl_inv.cxx:639,904).
template <int BM, int BN, int BK, int TM, int TN, bool SKIP_ZERO>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
simt_gemm_kernel(const SimtParams p) {
    constexpr int T = (BM / TM) * (BN / TN);
    constexpr int PAD = 4;
    __shared__ __align__(16) float As[BK][BM + PAD];
    __shared__ __align__(16) float Bs[BK][BN + PAD];

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN);
    const int ty = tid / (BN / TN);
    const long long m0 = (long long)blockIdx.y * BM;
    const long long n0 = (long long)blockIdx.x * BN;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (long long k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
        for (int e = tid; e < BM * BK; e += T) {
            int i, l;
            if (p.a_k_fast) {
                l = e % BK;
                i = e / BK;
            } else {
                i = e % BM;
                l = e / BM;
            }
            const long long gi = m0 + i, gl = k0 + l;
            As[l][i] = (gi < p.M && gl < p.K) ? __ldg(p.A + gi * p.a1 + gl * p.a2) : 0.0f;
        }
#pragma unroll
        for (int e = tid; e < BK * BN; e += T) {
            int l, j;
            if (p.b_n_fast) {
                j = e % BN;
                l = e / BN;
            } else {
                l = e % BK;
                j = e / BK;
            }
            const long long gl = k0 + l, gj = n0 + j;
            Bs[l][j] = (gl < p.K && gj < p.N) ? __ldg(p.B + gl * p.b1 + gj * p.b2) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int l = 0; l < BK; ++l) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[l][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[l][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    if (SKIP_ZERO) {
                        if (b[j] != 0.0f) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    } else {
                        acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    }
                }
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const long long gi = m0 + ty * TM + i;
        if (gi >= p.M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const long long gj = n0 + tx * TN + j;
            if (gj >= p.N) continue;
            float *dst = p.C + gi * p.c1 + gj * p.c2;
            float v = p.alpha * acc[i][j];
            if (p.beta != 0.0f) v += p.beta * *dst;
            if (p.bias) v += __ldg(p.bias + gj);
            *dst = act_f32(v, p.act);
        }
    }
}

// 16-byte asynchronous copy global -> shared; `bytes` = 16 copies, 0 writes zeros (the address
// must still be valid).
__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gmem_src, int bytes) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// The fused linear on dense row-major operands (A [M,K], B [K,N], C [M,N], every pitch and K, N
// multiples of four, 16-byte aligned): the same BM x BN x 16 blocking with a 4 x 4 register
// block, 16-byte accesses throughout, and a four-deep ring of K strips filled by asynchronous
// copies, so that the loads of three strips are in flight while one is multiplied.  At 512^3 the
// kernel with a single strip of look-ahead spent two thirds of its time waiting for global loads.
// KSPLIT = 2 (small problems): twice the threads, each half of them multiplying one half of every
// strip, summed through shared memory at the end: more warps per SM to cover latencies when
// there are too few tiles to fill the GPU.
template <int BM, int BN, int KSPLIT>
__global__ void __launch_bounds__(BM *BN / 16 * KSPLIT)
linear_f32_dense_kernel(const SimtParams p) {
    constexpr int BK = 16;
    constexpr int STAGES = 4;
    constexpr int T = BM * BN / 16 * KSPLIT;
    constexpr int TC = BM * BN / 16;  // threads of one K half
    constexpr int A_QUADS = BM * BK / 4, B_QUADS = BK * BN / 4;  // 16-byte copies per strip
    constexpr int A_LD = (A_QUADS + T - 1) / T;                     // ... per thread
    constexpr int B_LD = (B_QUADS + T - 1) / T;
    constexpr int A_PITCH = BK + 4;          // floats; rows stay 16-byte aligned, banks rotate by row
    constexpr int B_PITCH = BN + 4;
    __shared__ __align__(16) float As[STAGES][BM][A_PITCH];  // As[m][k]
    __shared__ __align__(16) float Bs[STAGES][BK][B_PITCH];  // Bs[k][n]

    const int tid = threadIdx.x;
    const int kpart = tid / TC;
    const int tx = (tid % TC) % (BN / 4);
    const int ty = (tid % TC) / (BN / 4);
    const long long m0 = (long long)blockIdx.y * BM;
    const long long n0 = (long long)blockIdx.x * BN;
    const long long strips = (p.K + BK - 1) / BK;

    auto fetch = [&](long long strip, int buf) {
        const long long k0 = strip * BK;
#pragma unroll
        for (int i = 0; i < A_LD; ++i) {
            const int e = tid + i * T;  // BM rows x 4 quads of K
            if (A_QUADS % T != 0 && e >= A_QUADS) break;
            const int m = e / 4, kq = (e % 4) * 4;
            const long long gm = m0 + m, gk = k0 + kq;
            const bool ok = gm < p.M && gk < p.K;
            cp_async_16(&As[buf][m][kq], ok ? p.A + gm * p.a1 + gk : p.A, ok ? 16 : 0);
        }
#pragma unroll
        for (int i = 0; i < B_LD; ++i) {
            const int e = tid + i * T;  // 16 rows of K x BN/4 quads of N
            if (B_QUADS % T != 0 && e >= B_QUADS) break;
            const int k = e / (BN / 4), nq = (e % (BN / 4)) * 4;
            const long long gk = k0 + k, gn = n0 + nq;
            const bool ok = gk < p.K && gn < p.N;
            cp_async_16(&Bs[buf][k][nq], ok ? p.B + gk * p.b1 + gn : p.B, ok ? 16 : 0);
        }
    };

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < strips) fetch(s, s);
        cp_async_commit();  // a group per strip, empty past the end: the wait below counts groups
    }
    for (long long strip = 0; strip < strips; ++strip) {
        const int buf = (int)(strip % STAGES);
        cp_async_wait<STAGES - 2>();  // this strip's copies (of this thread) have landed
        __syncthreads();              // ... everybody's; and the buffer refilled below is no longer read
        if (strip + STAGES - 1 < strips) fetch(strip + STAGES - 1, (int)((strip + STAGES - 1) % STAGES));
        cp_async_commit();
#pragma unroll
        for (int lq = 0; lq < BK / KSPLIT; lq += 4) {
            const int l = kpart * (BK / KSPLIT) + lq;
            float4 a4[4], b4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a4[i] = *reinterpret_cast<const float4 *>(&As[buf][ty * 4 + i][l]);
#pragma unroll
            for (int d = 0; d < 4; ++d) b4[d] = *reinterpret_cast<const float4 *>(&Bs[buf][l + d][tx * 4]);
#pragma unroll
            for (int d = 0; d < 4; ++d) {  // ascending k, as the loop nest sums
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float a = d == 0 ? a4[i].x : (d == 1 ? a4[i].y : (d == 2 ? a4[i].z : a4[i].w));
                    acc[i][0] = fmaf(a, b4[d].x, acc[i][0]);
                    acc[i][1] = fmaf(a, b4[d].y, acc[i][1]);
                    acc[i][2] = fmaf(a, b4[d].z, acc[i][2]);
                    acc[i][3] = fmaf(a, b4[d].w, acc[i][3]);
                }
            }
        }
    }
    cp_async_wait<0>();
    if constexpr (KSPLIT == 2) {
        // the second half hands its sums over through the (now idle) ring of A strips
        static_assert(STAGES * BM * A_PITCH >= TC * 16, "room for the partial sums");
        float *xchg = &As[0][0][0];
        __syncthreads();
        if (kpart == 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) xchg[(i * 4 + j) * TC + (tid - TC)] = acc[i][j];
        }
        __syncthreads();
        if (kpart == 1) return;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] += xchg[(i * 4 + j) * TC + tid];
    }

    const long long gn = n0 + tx * 4;
    if (gn >= p.N) return;
    float4 bias4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (p.bias) bias4 = __ldg(reinterpret_cast<const float4 *>(p.bias + gn));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long gm = m0 + ty * 4 + i;
        if (gm >= p.M) continue;
        float4 v;
        v.x = act_f32(acc[i][0] + bias4.x, p.act);
        v.y = act_f32(acc[i][1] + bias4.y, p.act);
        v.z = act_f32(acc[i][2] + bias4.z, p.act);
        v.w = act_f32(acc[i][3] + bias4.w, p.act);
        *reinterpret_cast<float4 *>(p.C + gm * p.c1 + gn) = v;
    }
}

// Tile of the dense kernel for a shape: the largest that still gives every SM a CTA.
void simt_dense_tile(int64_t M, int64_t N, int num_sms, int *tile_m, int *tile_n) {
    auto ctas = [&](int bm, int bn) { return ((M + bm - 1) / bm) * ((N + bn - 1) / bn); };
    if (ctas(64, 64) >= 2LL * num_sms) {
        *tile_m = 64, *tile_n = 64;
    } else if (ctas(32, 64) >= num_sms) {
        *tile_m = 32, *tile_n = 64;
    } else {
        *tile_m = 32, *tile_n = 32;
    }
    if (const char *env = getenv("O64_SIMT_TILE")) {  // tuning: "64x64", "32x64" or "32x32"
        int a = 0, b = 0;
        if (sscanf(env, "%dx%d", &a, &b) == 2 && (a == 32 || a == 64) && (b == 32 || b == 64) && !(a == 64 && b == 32))
            *tile_m = a, *tile_n = b;
    }
}

void simt_apply_pin(int pin_m, int pin_n, int *tile_m, int *tile_n) {
    if (pin_m == 32 || pin_m == 64) *tile_m = pin_m;
    if (pin_n == 32 || pin_n == 64) *tile_n = pin_n;
    if (*tile_m == 64 && *tile_n == 32) *tile_n = 64;
}

bool simt_dense_ok(const SimtGemmCall &c) {
    auto al16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    return c.a2 == 1 && c.b2 == 1 && c.c2 == 1 && c.alpha == 1.0f && c.beta == 0.0f && !c.skip_zero_b && c.K > 0 &&
           (c.K % 4) == 0 && (c.N % 4) == 0 && (c.a1 % 4) == 0 && (c.b1 % 4) == 0 && (c.c1 % 4) == 0 && c.a1 >= c.K &&
           c.b1 >= c.N && c.c1 >= c.N && al16(c.A) && al16(c.B) && al16(c.C) && (!c.bias || al16(c.bias));
}

template <int BM, int BN, int KSPLIT>
static int launch_dense(const SimtParams &p, cudaStream_t stream) {
    dim3 grid((unsigned)((p.N + BN - 1) / BN), (unsigned)((p.M + BM - 1) / BM));
    linear_f32_dense_kernel<BM, BN, KSPLIT><<<grid, BM * BN / 16 * KSPLIT, 0, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

template <int BM, int BN, int BK, int TM, int TN>
static int launch_simt(const SimtParams &p, bool skip_zero, cudaStream_t stream) {
    dim3 grid((unsigned)((p.N + BN - 1) / BN), (unsigned)((p.M + BM - 1) / BM));
    constexpr int T = (BM / TM) * (BN / TN);
    if (skip_zero)
        simt_gemm_kernel<BM, BN, BK, TM, TN, true><<<grid, T, 0, stream>>>(p);
    else
        simt_gemm_kernel<BM, BN, BK, TM, TN, false><<<grid, T, 0, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

// sets *flag when any element of the rows x cols matrix (cols contiguous, pitch ld) is an infinity or a NaN
__global__ void nonfinite_f32_kernel(const float *p, long long rows, long long cols, long long ld, int *flag) {
    bool bad = false;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < rows * cols; e += (long long)gridDim.x * blockDim.x) {
        const float v = p[(e / cols) * ld + (e % cols)];
        bad |= !(fabsf(v) <= 3.402823466e38f);
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicExch(flag, 1);
}

// A call that has the shape of the dense kernel - plainly laid out, row-major or column-major (then as
// C' = B' A'), alpha 1, beta 0 - but is not in its form yet.  Where it carries the runtime's rule about zero
// factors of B (the strided kernels behind MATMUL): the rule can only change a result when A holds an
// infinity or a NaN, so A is scanned and, if it is clean, the dense kernel runs.  Synchronises the stream (these
// entry points are synchronous anyway).  Returns true when `*out` is to be used instead of `c`.
static bool dense_form_of_skipping_call(const SimtGemmCall &c, SimtGemmCall *out) {
    if (c.K <= 0 || simt_dense_ok(c)) return false;  // (already in the dense kernel's own form)
    SimtGemmCall d = c;
    long long o_rows, o_cols, o_ld;
    if (c.a2 == 1 && c.b2 == 1 && c.c2 == 1) {
        o_rows = c.M, o_cols = c.K, o_ld = c.a1;
    } else if (c.a1 == 1 && c.b1 == 1 && c.c1 == 1) {
        d.M = c.N, d.N = c.M;
        d.A = c.B, d.a1 = c.b2, d.a2 = 1;
        d.B = c.A, d.b1 = c.a2, d.b2 = 1;
        d.c1 = c.c2, d.c2 = 1;
        o_rows = c.K, o_cols = c.M, o_ld = c.a2;
    } else {
        return false;
    }
    d.skip_zero_b = false;
    if (!simt_dense_ok(d)) return false;
    if (!c.skip_zero_b) {  // no rule to keep: the exchange of roles is all
        *out = d;
        return true;
    }
    static int *flags[64] = {nullptr};  // one word per device
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    std::lock_guard<std::mutex> lock(mu);
    if (!flags[dev] && cudaMalloc(&flags[dev], sizeof(int)) != cudaSuccess) {
        (void)cudaGetLastError();
        flags[dev] = nullptr;
        return false;
    }
    int bad = 1;
    const long long total = o_rows * o_cols;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (cudaMemsetAsync(flags[dev], 0, sizeof(int), c.stream) != cudaSuccess) return false;
    nonfinite_f32_kernel<<<(unsigned)blocks, 256, 0, c.stream>>>(c.A, o_rows, o_cols, o_ld, flags[dev]);
    if (cudaMemcpyAsync(&bad, flags[dev], sizeof(int), cudaMemcpyDeviceToHost, c.stream) != cudaSuccess ||
        cudaStreamSynchronize(c.stream) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    if (bad) return false;
    *out = d;
    return true;
}

int simt_gemm_f32(const SimtGemmCall &c_in) {
    SimtGemmCall c = c_in;
    {
        SimtGemmCall d;
        if (dense_form_of_skipping_call(c_in, &d)) c = d;
    }
    if (c.M < 0 || c.N < 0 || c.K < 0) return O64_ERR_RANK;
    if (c.M == 0 || c.N == 0) return O64_OK;
    if ((c.N + 31) / 32 > 2147483647LL || (c.M + 31) / 32 > 65535LL) return O64_ERR_RANK;
    SimtParams p;
    p.M = c.M; p.N = c.N; p.K = c.K;
    p.alpha = c.alpha; p.beta = c.beta;
    p.A = c.A; p.a1 = c.a1; p.a2 = c.a2;
    p.B = c.B; p.b1 = c.b1; p.b2 = c.b2;
    p.C = c.C; p.c1 = c.c1; p.c2 = c.c2;
    p.bias = c.bias;
    p.act = c.act;
    auto mag = [](int64_t v) { return v < 0 ? -v : v; };
    p.a_k_fast = mag(c.a2) <= mag(c.a1);
    p.b_n_fast = mag(c.b2) <= mag(c.b1);
    p.c_n_fast = mag(c.c2) <= mag(c.c1);
    if (simt_dense_ok(c)) {
        int tm, tn;
        simt_dense_tile(c.M, c.N, c.num_sms, &tm, &tn);
        simt_apply_pin(c.pin_tile_m, c.pin_tile_n, &tm, &tn);
        // measured: the K split inside the CTA gains 5 % at 512^3 (32 x 32 tiles) and loses 15 % at
        // 1024^3 (32 x 64 tiles, already two CTAs per SM)
        if (tm == 64) return launch_dense<64, 64, 1>(p, c.stream);
        if (tn == 64) return launch_dense<32, 64, 1>(p, c.stream);
        return launch_dense<32, 32, 2>(p, c.stream);
    }
    // strided operands: 64 x 64 tiles when there are enough of them, else 32 x 32; a pinned tile_m decides
    const long long big_tiles = ((c.M + 63) / 64) * ((c.N + 63) / 64);
    const bool big = c.pin_tile_m ? c.pin_tile_m == 64 : big_tiles >= 2LL * c.num_sms;
    if (big) return launch_simt<64, 64, 16, 4, 4>(p, c.skip_zero_b, c.stream);
    return launch_simt<32, 32, 16, 2, 2>(p, c.skip_zero_b, c.stream);
}

// ------------------------------------------------------------------------------------------
// GEMV
// ------------------------------------------------------------------------------------------
// One warp per row: lanes stride over the columns, shuffle reduction.
__global__ void gemv_warp_kernel(long long M, long long N, float alpha, const float *A, long long a1,
                                 long long a2, const float *X, long long incx, float beta, float *Y,
                                 long long incy) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= M) return;
    float acc = 0.0f;
    for (long long j = lane; j < N; j += 32) {
        const float x = __ldg(X + j * incx);
        if (x != 0.0f) acc = fmaf(alpha * x, __ldg(A + row * a1 + j * a2), acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        float *y = Y + row * incy;
        *y = (beta == 0.0f ? 0.0f : beta * *y) + acc;
    }
}

// One thread per row: coalesced when consecutive rows are adjacent in memory (column-major A).
__global__ void gemv_thread_kernel(long long M, long long N, float alpha, const float *A,
                                   long long a1, long long a2, const float *X, long long incx,
                                   float beta, float *Y, long long incy) {
    const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= M) return;
    float *y = Y + row * incy;
    float acc = (beta == 0.0f) ? 0.0f : beta * *y;
    for (long long j = 0; j < N; ++j) {
        const float x = __ldg(X + j * incx);
        if (x != 0.0f) acc = fmaf(alpha * x, __ldg(A + row * a1 + j * a2), acc);
    }
    *y = acc;
}

int simt_gemv_f32(int64_t M, int64_t N, float alpha, const float *A, int64_t a1, int64_t a2,
                  const float *X, int64_t incx, float beta, float *Y, int64_t incy,
                  cudaStream_t stream) {
    if (M <= 0) return O64_OK;
    auto mag = [](int64_t v) { return v < 0 ? -v : v; };
    if (mag(a1) <= mag(a2) && M >= 4096) {
        const int T = 128;
        gemv_thread_kernel<<<(unsigned)((M + T - 1) / T), T, 0, stream>>>(M, N, alpha, A, a1, a2, X,
                                                                            incx, beta, Y, incy);
    } else {
        const int T = 128;  // 4 rows per block
        gemv_warp_kernel<<<(unsigned)((M + 3) / 4), T, 0, stream>>>(M, N, alpha, A, a1, a2, X, incx,
                                                                      beta, Y, incy);
    }
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

__global__ void scale_kernel(long long M, long long N, float beta, float *C, long long c1,
                             long long c2, int n_fast) {
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= M * N) return;
    long long i, j;
    if (n_fast) {
        j = e % N;
        i = e / N;
    } else {
        i = e % M;
        j = e / M;
    }
    float *c = C + i * c1 + j * c2;
    *c = (beta == 0.0f) ? 0.0f : beta * *c;
}

int simt_scale_f32(int64_t M, int64_t N, float beta, float *C, int64_t c1, int64_t c2,
                   cudaStream_t stream) {
    if (M <= 0 || N <= 0) return O64_OK;
    auto mag = [](int64_t v) { return v < 0 ? -v : v; };
    const long long total = (long long)M * N;
    scale_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(M, N, beta, C, c1, c2,
                                                                       mag(c2) <= mag(c1));
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

// ------------------------------------------------------------------------------------------
// reference kernels: one thread per output, ascending k, separate multiply and add — the
// compiler's loop nest (osprey/be/vho/f90_lower.cxx:5149-5169) run as is on the device.
// ------------------------------------------------------------------------------------------
template <int KIND>
__device__ __forceinline__ float load_as_f32(const void *base, long long idx) {
    if constexpr (KIND == O64_KIND_F32) {
        return reinterpret_cast<const float *>(base)[idx];
    } else if constexpr (KIND == O64_KIND_BF16) {
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(base)[idx]);
    } else {
        __nv_fp8_e4m3 v;
        v.__x = reinterpret_cast<const unsigned char *>(base)[idx];
        return static_cast<float>(v);
    }
}

template <int KIND>
__global__ void naive_float_kernel(long long M, long long N, long long K, const void *A,
                                   long long lda, const void *B, long long ldb, int transB,
                                   const float *scaleA, const float *scaleB, const float *bias,
                                   int act, float *out, long long ldo) {
    const long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long i = (long long)blockIdx.y * blockDim.y + threadIdx.y;
    if (i >= M || j >= N) return;
    const float sa = scaleA ? scaleA[i] : 1.0f;
    const float sb = scaleB ? scaleB[j] : 1.0f;
    float acc = 0.0f;
    for (long long k = 0; k < K; ++k) {
        float a = load_as_f32<KIND>(A, i * lda + k);
        float b = load_as_f32<KIND>(B, transB ? j * ldb + k : k * ldb + j);
        if (KIND == O64_KIND_FP8) {
            a = __fmul_rn(a, sa);
            b = __fmul_rn(b, sb);
        }
        acc = __fadd_rn(acc, __fmul_rn(a, b));
    }
    if (bias) acc = __fadd_rn(acc, bias[j]);
    out[i * ldo + j] = act_f32(acc, act);
}

__global__ void naive_s8_kernel(long long M, long long N, long long K, const int8_t *A, long long lda,
                                const int8_t *B, long long ldb, int transB, int32_t *out,
                                long long ldo) {
    const long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long i = (long long)blockIdx.y * blockDim.y + threadIdx.y;
    if (i >= M || j >= N) return;
    int32_t acc = 0;
    for (long long k = 0; k < K; ++k)
        acc += (int32_t)A[i * lda + k] * (int32_t)B[transB ? j * ldb + k : k * ldb + j];
    out[i * ldo + j] = acc;
}

int naive_gemm(int kind, int64_t M, int64_t N, int64_t K, const void *A, int64_t lda, const void *B,
               int64_t ldb, int transB, const float *scaleA, const float *scaleB, const float *bias,
               int act, void *out, int64_t ldo, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return O64_OK;
    dim3 block(32, 8);
    dim3 grid((unsigned)((N + 31) / 32), (unsigned)((M + 7) / 8));
    if (grid.y > 65535) return O64_ERR_RANK;
    float *of = reinterpret_cast<float *>(out);
    switch (kind) {
    case O64_KIND_F32:
        naive_float_kernel<O64_KIND_F32><<<grid, block, 0, stream>>>(M, N, K, A, lda, B, ldb, transB,
                                                                      nullptr, nullptr, bias, act, of, ldo);
        break;
    case O64_KIND_BF16:
        naive_float_kernel<O64_KIND_BF16><<<grid, block, 0, stream>>>(M, N, K, A, lda, B, ldb, transB,
                                                                       nullptr, nullptr, bias, act, of, ldo);
        break;
    case O64_KIND_FP8:
        naive_float_kernel<O64_KIND_FP8><<<grid, block, 0, stream>>>(M, N, K, A, lda, B, ldb, transB,
                                                                      scaleA, scaleB, bias, act, of, ldo);
        break;
    case O64_KIND_S8:
        naive_s8_kernel<<<grid, block, 0, stream>>>(M, N, K, reinterpret_cast<const int8_t *>(A), lda,
                                                    reinterpret_cast<const int8_t *>(B), ldb, transB,
                                                    reinterpret_cast<int32_t *>(out), ldo);
        break;
    default: return O64_ERR_DTYPE;
    }
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

__global__ void finalize_partial_kernel(const float *__restrict__ partial, long long M, long long N,
                                        const float *scale_a, const float *scale_b, const float *bias,
                                        int act, __nv_bfloat16 *C, long long ldc, int out_kind) {
    const long long total = M * N;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        const long long i = e / N, j = e % N;
        float x = partial ? partial[e] : 0.0f;  // no partial sums: the empty sum (K == 0)
        if (scale_a || scale_b)  // as the tile kernels' scaled tail: acc * (sa * sb) + bias, nothing fused
            x = __fmul_rn(x, __fmul_rn(scale_a ? scale_a[i] : 1.0f, scale_b ? scale_b[j] : 1.0f));
        if (bias) x = __fadd_rn(x, bias[j]);
        x = act_f32(x, act);
        if (out_kind == 1) {  // int8, round to nearest even, saturating
            int q = __float2int_rn(x);
            q = max(-128, min(127, q));
            reinterpret_cast<int8_t *>(C)[i * ldc + j] = (int8_t)q;
        } else if (out_kind == 2) {  // e4m3, round to nearest even, saturating
            reinterpret_cast<uint8_t *>(C)[i * ldc + j] = (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
        } else {
            C[i * ldc + j] = __float2bfloat16_rn(x);
        }
    }
}

int finalize_partial_bf16(const float *partial, int64_t M, int64_t N, const float *scale_a,
                          const float *scale_b, const float *bias, int act, void *C, int64_t ldc,
                          cudaStream_t stream, int out_kind) {
    if (M <= 0 || N <= 0) return O64_OK;
    long long blocks = ((long long)M * N + 255) / 256;
    if (blocks > 148LL * 8) blocks = 148LL * 8;
    finalize_partial_kernel<<<(unsigned)blocks, 256, 0, stream>>>(partial, M, N, scale_a, scale_b, bias, act,
                                                                  reinterpret_cast<__nv_bfloat16 *>(C), ldc, out_kind);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

// ------------------------------------------------------------------------------------------
// operand pattern for timing runs: pseudo-random finite values (zero-filled operands toggle no
// bits in the tensor cores, draw far less power and run at clocks real data never sees)
// ------------------------------------------------------------------------------------------
__global__ void fill_pattern_kernel(uint32_t *p, size_t words, int kind, uint32_t seed) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t x = (uint32_t)i * 2654435761u + seed;
        x ^= x >> 15;
        x *= 2246822519u;
        x ^= x >> 13;
        x *= 3266489917u;
        x ^= x >> 16;
        if (kind == O64_KIND_BF16) {
            // two bf16 values in [1/128, 1/64) with random sign and mantissa
            x = (x & 0x807f807fu) | 0x3c003c00u;
        } else if (kind == O64_KIND_FP8) {
            x &= 0xf7f7f7f7u;  // e4m3: exponent below the NaN code
        }
        p[i] = x;
    }
}

int fill_pattern(void *p, size_t bytes, int kind, cudaStream_t stream) {
    const size_t words = bytes / 4;
    if (!words) return O64_OK;
    fill_pattern_kernel<<<1184, 256, 0, stream>>>(static_cast<uint32_t *>(p), words, kind, 0x9e3779b9u);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

// ------------------------------------------------------------------------------------------
// slab permute: the all-gather delivers [g][M][N/g]; callers that want row-major [M,N] get it
// through this copy (16-byte vectors when the slab width allows).
// ------------------------------------------------------------------------------------------
__global__ void permute_slabs_kernel(const int32_t *__restrict__ src, int32_t *__restrict__ dst,
                                     long long M, long long ncols, int nslabs, long long ld_dst,
                                     int vec) {
    const long long per_row = ncols / vec;
    const long long total = (long long)nslabs * M * per_row;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        const long long jv = e % per_row;
        const long long rest = e / per_row;
        const long long r = rest % nslabs;  // slab varies fastest after the column: a row of dst stays contiguous
        const long long m = rest / nslabs;
        const int32_t *s = src + (r * M + m) * ncols + jv * vec;
        int32_t *d = dst + m * ld_dst + r * ncols + jv * vec;
        if (vec == 4)
            *reinterpret_cast<int4 *>(d) = *reinterpret_cast<const int4 *>(s);
        else
            *d = *s;
    }
}

// dst[c][r] = src[r][c] for one-byte elements: 64 x 64 tiles through shared memory, so that both the
// loads (along c) and the stores (along r) are contiguous; the padding column keeps the transposed
// reads free of bank conflicts.
__global__ void transpose_bytes_kernel(const uint8_t *__restrict__ src, long long ld_src, uint8_t *__restrict__ dst,
                                       long long ld_dst, long long rows, long long cols) {
    __shared__ uint8_t tile[64][64 + 4];
    const long long tiles_c = (cols + 63) / 64, tiles_r = (rows + 63) / 64;
    for (long long t = blockIdx.x; t < tiles_c * tiles_r; t += gridDim.x) {
        const long long r0 = (t / tiles_c) * 64, c0 = (t % tiles_c) * 64;
        for (int i = threadIdx.x; i < 64 * 64; i += blockDim.x) {
            const int r = i >> 6, c = i & 63;
            tile[r][c] = (r0 + r < rows && c0 + c < cols) ? src[(r0 + r) * ld_src + c0 + c] : (uint8_t)0;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < 64 * 64; i += blockDim.x) {
            const int c = i >> 6, r = i & 63;
            if (c0 + c < cols && r0 + r < rows) dst[(c0 + c) * ld_dst + r0 + r] = tile[r][c];
        }
        __syncthreads();
    }
}

int transpose_bytes(const void *src, int64_t ld_src, void *dst, int64_t ld_dst, int64_t rows, int64_t cols,
                    cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return O64_OK;
    long long tiles = ((rows + 63) / 64) * ((cols + 63) / 64);
    if (tiles > 148LL * 8) tiles = 148LL * 8;
    transpose_bytes_kernel<<<(unsigned)tiles, 256, 0, stream>>>(static_cast<const uint8_t *>(src), ld_src,
                                                               static_cast<uint8_t *>(dst), ld_dst, rows, cols);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

int permute_slabs_s32(const int32_t *src, int32_t *dst, int64_t M, int64_t ncols, int nslabs,
                      int64_t ld_dst, cudaStream_t stream) {
    if (M <= 0 || ncols <= 0 || nslabs <= 0) return O64_OK;
    const bool v4 = (ncols % 4 == 0) && (ld_dst % 4 == 0) &&
                    ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    const int vec = v4 ? 4 : 1;
    const long long total = (long long)nslabs * M * (ncols / vec);
    long long blocks = (total + 255) / 256;
    if (blocks > 148LL * 16) blocks = 148LL * 16;
    permute_slabs_kernel<<<(unsigned)blocks, 256, 0, stream>>>(src, dst, M, ncols, nslabs, ld_dst, vec);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

}  // namespace o64
