// The rest of the runtime's X-interface family on CUDA cores: C = alpha*A*B + beta*C and
// y = alpha*A*x + beta*y for REAL*8, COMPLEX*8 / *16 and the integer kinds (8 to 64 bits, A of the
// same or a narrower kind than B and C), with the semantics of the reference's template
// (osprey/libfi/matrix/xgemmx.h:172-236: element (i,j) of X at X[inc1x*i + inc2x*j], beta == 0
// does not read C, a zero B(l,j) skips its term; integers wrap in the kind of C).
// These kinds have no tensor-core path that keeps their exact arithmetic; the kernel is a plain
// shared-memory tiled loop nest (the L1 strip and register tile of osprey/be/lno/snl_inv.cxx:639,904).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "../../include/o64gemm.h"
#include "simt_kernels.cuh"

namespace o64 {

// A's element in the kind of C: integers are sign-extended, then carried on the unsigned type;
// with a REAL result (the mixed kernels such as _i4s4gemmx__, _s4sgemmx__) A is converted to it.
template <typename T, typename TA> __device__ __forceinline__ T widen(TA a) {
    if constexpr (std::is_same<T, TA>::value) return a;
    else if constexpr (std::is_floating_point<T>::value) return (T)a;  // REAL results: plain conversion
    else return (T)(long long)a;
}
template <typename T> struct IsComplex { static constexpr bool value = false; };
template <typename R> struct IsComplex<Cx<R>> { static constexpr bool value = true; };
template <typename T> __device__ __forceinline__ T conj_if(T x, int) { return x; }
template <typename R> __device__ __forceinline__ Cx<R> conj_if(Cx<R> x, int on) { return on ? Cx<R>(x.re, -x.im) : x; }

// Product in the kind T.  8- and 16-bit operands are multiplied as unsigned 32-bit values: the
// usual promotion to (signed) int would overflow for 16-bit factors.
template <typename T> __device__ __forceinline__ T mul(T a, T b) {
    if constexpr (sizeof(T) < 4) return (T)((unsigned)a * (unsigned)b);
    else return a * b;
}

template <typename TA, typename T>
__global__ void __launch_bounds__(256)
gemmx_generic_kernel(long long M, long long N, long long K, T alpha, const TA *A, long long a1, long long a2,
                     const T *B, long long b1, long long b2, T beta, T *C, long long c1, long long c2,
                     int a_k_fast, int b_n_fast, int conj_a, int conj_b) {
    constexpr int BM = 32, BN = 32, BK = 16, TM = 2, TN = 2;
    __shared__ T As[BK][BM + 1];
    __shared__ T Bs[BK][BN + 1];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const long long m0 = (long long)blockIdx.y * BM, n0 = (long long)blockIdx.x * BN;
    T acc[TM][TN] = {};
    for (long long k0 = 0; k0 < K; k0 += BK) {
        for (int e = tid; e < BM * BK; e += 256) {
            int i, l;
            if (a_k_fast) { l = e % BK; i = e / BK; } else { i = e % BM; l = e / BM; }
            const long long gi = m0 + i, gl = k0 + l;
            As[l][i] = (gi < M && gl < K) ? conj_if(widen<T, TA>(A[gi * a1 + gl * a2]), conj_a) : T(0);
        }
        for (int e = tid; e < BK * BN; e += 256) {
            int l, j;
            if (b_n_fast) { j = e % BN; l = e / BN; } else { l = e % BK; j = e / BK; }
            const long long gl = k0 + l, gj = n0 + j;
            Bs[l][j] = (gl < K && gj < N) ? conj_if(B[gl * b1 + gj * b2], conj_b) : T(0);
        }
        __syncthreads();
#pragma unroll
        for (int l = 0; l < BK; ++l) {
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    const T b = Bs[l][tx * TN + j];
                    // zero B(l,j): term left out (the template of the real and integer kernels; the
                    // complex kernels have no such test, osprey/libfi/matrix/c4gemmx.f:199-212)
                    if (IsComplex<T>::value || b != T(0)) acc[i][j] = (T)(acc[i][j] + mul<T>(As[l][ty * TM + i], b));
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const long long gi = m0 + ty * TM + i;
        if (gi >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const long long gj = n0 + tx * TN + j;
            if (gj >= N) continue;
            T *dst = C + gi * c1 + gj * c2;
            T v = mul<T>(alpha, acc[i][j]);
            if (beta != T(0)) v = (T)(v + mul<T>(beta, *dst));
            *dst = v;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// REAL*8 on plainly laid out operands (what MATMUL on whole REAL*8 arrays and the dgemm_ hook pass):
// Y[Mr,Nr] = alpha * X[Mr,K] * W[K,Nr] + beta * Y, X with K contiguous, W and Y with Nr contiguous.
// A column-major product C = A B is this with X = B', W = A', Y = C' (the caller exchanges the roles).
// 64 x 64 tiles with a 4 x 4 register block per thread; strips of 8 in a four-deep ring of asynchronous
// 16-byte copies (the structure of the REAL*4 linear in simt_kernels.cu).  The template's rule that a
// zero factor in B leaves its term out only changes a result when the other operand holds an
// infinity or a NaN; the launcher checks that operand first and keeps the general kernel for that case.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async_16_g(void *smem_dst, const void *gmem_src, int bytes) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}

template <int TM>  // rows of the register block (4: 64 x 64 tiles)
__global__ void __launch_bounds__(256)
dense_f64_kernel(long long Mr, long long Nr, long long K, double alpha, const double *__restrict__ X, long long ldx,
                 const double *__restrict__ W, long long ldw, double beta, double *__restrict__ Y, long long ldy) {
    constexpr int BM = 16 * TM, BN = 64, BK = 8, STAGES = (TM == 8) ? 3 : 4;
    constexpr int A_PITCH = BK + 2, B_PITCH = BN + 2;  // doubles: rows stay 16-byte aligned, banks rotate by row
    __shared__ __align__(16) double As[STAGES][BM][A_PITCH];
    __shared__ __align__(16) double Bs[STAGES][BK][B_PITCH];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const long long m0 = (long long)blockIdx.y * BM, n0 = (long long)blockIdx.x * BN;
    const long long strips = (K + BK - 1) / BK;

    auto fetch = [&](long long strip, int buf) {
        const long long k0 = strip * BK;
#pragma unroll
        for (int r = 0; r < TM / 4; ++r) {  // X: BM rows x 4 pairs of K, 16-byte copies
            const int e = tid + r * 256;
            const int m = e >> 2, kp = (e & 3) * 2;
            const long long gm = m0 + m, gk = k0 + kp;
            const bool ok = gm < Mr && gk < K;  // K is even: a pair is inside or outside as a whole
            cp_async_16_g(&As[buf][m][kp], ok ? X + gm * ldx + gk : X, ok ? 16 : 0);
        }
        {  // W: 8 rows of K x 32 pairs of Nr
            const int k = tid >> 5, np = (tid & 31) * 2;
            const long long gk = k0 + k, gn = n0 + np;
            const bool ok = gk < K && gn < Nr;
            cp_async_16_g(&Bs[buf][k][np], ok ? W + gk * ldw + gn : W, ok ? 16 : 0);
        }
    };

    double acc[TM][4];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0;
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        if (st < strips) fetch(st, st);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (long long strip = 0; strip < strips; ++strip) {
        const int buf = (int)(strip % STAGES);
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
        __syncthreads();
        if (strip + STAGES - 1 < strips) fetch(strip + STAGES - 1, (int)((strip + STAGES - 1) % STAGES));
        asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
        for (int l = 0; l < BK; ++l) {  // ascending k, as the loop nest sums
            double a[TM];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[buf][ty * TM + i][l];
            // this thread's four columns are tx*2, tx*2+1 and 32 + the same: consecutive threads read
            // consecutive 16-byte words (columns tx*4 .. tx*4+3 would put threads 0 and 4 on one bank)
            const double2 b01 = *reinterpret_cast<const double2 *>(&Bs[buf][l][tx * 2]);
            const double2 b23 = *reinterpret_cast<const double2 *>(&Bs[buf][l][32 + tx * 2]);
#pragma unroll
            for (int i = 0; i < TM; ++i) {
                acc[i][0] = fma(a[i], b01.x, acc[i][0]);
                acc[i][1] = fma(a[i], b01.y, acc[i][1]);
                acc[i][2] = fma(a[i], b23.x, acc[i][2]);
                acc[i][3] = fma(a[i], b23.y, acc[i][3]);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const long long gm = m0 + ty * TM + i;
        if (gm >= Mr) continue;
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
            const long long gn = n0 + (j ? 32 : 0) + tx * 2;
            if (gn >= Nr) continue;  // Nr is even: a pair is inside or outside as a whole
            double *dst = Y + gm * ldy + gn;
            double2 v = make_double2(alpha * acc[i][j], alpha * acc[i][j + 1]);
            if (beta != 0.0) {
                const double2 o = *reinterpret_cast<const double2 *>(dst);
                v.x += beta * o.x;
                v.y += beta * o.y;
            }
            *reinterpret_cast<double2 *>(dst) = v;
        }
    }
}

// The same product on the fp64 tensor path (mma.sync m8n8k4: the only tensor instruction for REAL*8; tcgen05
// has no 64-bit kind).  64 x 64 tiles, eight warps of 32 x 16, strips of 16 in a three-deep ring.  Each
// instruction adds a0 b0 + ... + a3 b3 to its 8 x 8 block: 8 multiply-adds per thread for two values read
// from shared memory, against 16 for 6 in the kernel above.  Shared-memory pitches put the eight rows of an
// A fragment (4 doubles each) and the four rows of a B fragment (8 doubles each) on distinct banks.
constexpr int kF64MmaBK = 16, kF64MmaStages = 3, kF64MmaKPitch = kF64MmaBK + 4, kF64MmaNPitch = 64 + 4;
constexpr int kF64MmaTile = 64 * kF64MmaKPitch;  // doubles per operand tile and stage (>= 16 * kF64MmaNPitch)
constexpr int kF64MmaSmemBytes = kF64MmaStages * 2 * kF64MmaTile * 8;
static_assert(kF64MmaTile >= kF64MmaBK * kF64MmaNPitch, "an operand tile fits either way round");

// X_MFAST: X is stored with its rows (not K) contiguous, X(m,k) at X[k*ldx + m] - a transposed first operand;
// W_KFAST: W is stored with K (not its columns) contiguous, W(k,n) at W[n*ldw + k] - a transposed second one.
// In shared memory a tile keeps the operand's own orientation ([64][K strip] or [K strip][64]); the
// fragments are read accordingly, and both orientations are free of bank conflicts with these pitches.
template <bool X_MFAST, bool W_KFAST>
__global__ void __launch_bounds__(256)
dense_f64_mma_kernel(long long Mr, long long Nr, long long K, double alpha, const double *__restrict__ X, long long ldx,
                     const double *__restrict__ W, long long ldw, double beta, double *__restrict__ Y, long long ldy) {
    constexpr int BM = 64, BN = 64, BK = kF64MmaBK, STAGES = kF64MmaStages, KP = kF64MmaKPitch, NP = kF64MmaNPitch;
    extern __shared__ __align__(16) double smem_f64[];
    double *const xs = smem_f64, *const ws = smem_f64 + STAGES * kF64MmaTile;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 2, wn = warp & 3;     // 2 x 4 warps, 32 x 16 each
    const int fr = lane >> 2, fc = lane & 3;     // fragment coordinates of this lane
    const long long m0 = (long long)blockIdx.y * BM, n0 = (long long)blockIdx.x * BN;
    const long long strips = (K + BK - 1) / BK;

    // a 64 x 16 tile of an operand whose K runs contiguously: [64][KP]; one whose other index does: [16][NP]
    auto fetch_kfast = [&](double *dst, const double *src, long long ld, long long r0, long long rows, long long k0) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int e = tid + r * 256;
            const int m = e >> 3, kp = (e & 7) * 2;
            const long long gm = r0 + m, gk = k0 + kp;
            const bool ok = gm < rows && gk < K;  // K is even: a pair is inside or outside as a whole
            cp_async_16_g(dst + m * KP + kp, ok ? src + gm * ld + gk : src, ok ? 16 : 0);
        }
    };
    auto fetch_other = [&](double *dst, const double *src, long long ld, long long c0, long long cols, long long k0) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int e = tid + r * 256;
            const int k = e >> 5, np = (e & 31) * 2;
            const long long gk = k0 + k, gn = c0 + np;
            const bool ok = gk < K && gn < cols;  // the extent is even
            cp_async_16_g(dst + k * NP + np, ok ? src + gk * ld + gn : src, ok ? 16 : 0);
        }
    };
    auto fetch = [&](long long strip, int buf) {
        const long long k0 = strip * BK;
        if constexpr (X_MFAST) fetch_other(xs + buf * kF64MmaTile, X, ldx, m0, Mr, k0);
        else fetch_kfast(xs + buf * kF64MmaTile, X, ldx, m0, Mr, k0);
        if constexpr (W_KFAST) fetch_kfast(ws + buf * kF64MmaTile, W, ldw, n0, Nr, k0);
        else fetch_other(ws + buf * kF64MmaTile, W, ldw, n0, Nr, k0);
    };

    double acc[4][2][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        if (st < strips) fetch(st, st);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (long long strip = 0; strip < strips; ++strip) {
        const int buf = (int)(strip % STAGES);
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
        __syncthreads();
        if (strip + STAGES - 1 < strips) fetch(strip + STAGES - 1, (int)((strip + STAGES - 1) % STAGES));
        asm volatile("cp.async.commit_group;" ::: "memory");
        const double *xt = xs + buf * kF64MmaTile, *wt = ws + buf * kF64MmaTile;
#pragma unroll
        for (int k4 = 0; k4 < BK; k4 += 4) {  // ascending k, four at a time
            double a[4], b[2];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int m = wm * 32 + i * 8 + fr, k = k4 + fc;
                a[i] = X_MFAST ? xt[k * NP + m] : xt[m * KP + k];
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int n = wn * 16 + j * 8 + fr, k = k4 + fc;
                b[j] = W_KFAST ? wt[n * KP + k] : wt[k * NP + n];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                                 : "+d"(acc[i][j][0]), "+d"(acc[i][j][1])
                                 : "d"(a[i]), "d"(b[j]));
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long gm = m0 + wm * 32 + i * 8 + fr;
        if (gm >= Mr) continue;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const long long gn = n0 + wn * 16 + j * 8 + fc * 2;
            if (gn >= Nr) continue;  // Nr is even: a pair is inside or outside as a whole
            double *dst = Y + gm * ldy + gn;
            double2 v = make_double2(alpha * acc[i][j][0], alpha * acc[i][j][1]);
            if (beta != 0.0) {
                const double2 o = *reinterpret_cast<const double2 *>(dst);
                v.x += beta * o.x;
                v.y += beta * o.y;
            }
            *reinterpret_cast<double2 *>(dst) = v;
        }
    }
}

// sets *flag when any element of the rows x cols matrix (cols contiguous, pitch ld) is an infinity or a NaN
__global__ void nonfinite_f64_kernel(const double *p, long long rows, long long cols, long long ld, int *flag) {
    bool bad = false;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < rows * cols; e += (long long)gridDim.x * blockDim.x) {
        const double v = p[(e / cols) * ld + (e % cols)];
        bad |= !(fabs(v) <= 1.7976931348623157e308);
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicExch(flag, 1);
}

// The dense REAL*8 path, if the call has its shape; *done says whether it ran.  The shape: every matrix
// has one index with unit stride.  The result is taken row-major (its unit-stride index as columns; a
// column-major C = A B is C' = B' A'), the operands may each lie either way round.
static int try_dense_f64(int64_t M, int64_t N, int64_t K, double alpha, const double *A, int64_t a1, int64_t a2, const double *B,
                         int64_t b1, int64_t b2, double beta, double *C, int64_t c1, int64_t c2, cudaStream_t s, bool *done) {
    *done = false;
    if (K <= 0) return O64_OK;
    if ((a1 != 1 && a2 != 1) || (b1 != 1 && b2 != 1) || (c1 != 1 && c2 != 1)) return O64_OK;
    const double *X, *W;
    double *Y = C;
    int64_t Mr, Nr, ldx, ldw, ldy;
    bool x_mfast, w_kfast;
    if (c2 == 1) {  // Y = C: rows i, columns j
        Mr = M, Nr = N, ldy = c1;
        X = A, x_mfast = (a2 != 1), ldx = x_mfast ? a2 : a1;  // X(i,l) = A(i,l)
        W = B, w_kfast = (b2 != 1), ldw = w_kfast ? b2 : b1;  // W(l,j) = B(l,j)
    } else {        // Y = C': rows j, columns i
        Mr = N, Nr = M, ldy = c2;
        X = B, x_mfast = (b1 != 1), ldx = x_mfast ? b1 : b2;  // X(j,l) = B(l,j): K contiguous when b1 == 1
        W = A, w_kfast = (a1 != 1), ldw = w_kfast ? a1 : a2;  // W(l,i) = A(i,l): i contiguous when a1 == 1
    }
    // the operand whose infinities or NaNs a skipped zero term would have hidden: A, as it lies in memory
    const double *other = A;
    const int64_t o_rows = (a2 == 1) ? M : K, o_cols = (a2 == 1) ? K : M, o_ld = (a2 == 1) ? a1 : a2;
    auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    // 16-byte copies: the contiguous extent of every tile is even, pitches are even, bases aligned
    const int64_t x_run = x_mfast ? Mr : K, w_run = w_kfast ? K : Nr;
    if ((K & 1) || (Nr & 1) || (x_run & 1) || (ldx & 1) || (ldw & 1) || (ldy & 1) || ldx < x_run || ldw < w_run || ldy < Nr ||
        !al16(X) || !al16(W) || !al16(Y) || (Mr + 63) / 64 > 65535)
        return O64_OK;
    static int *flags[64] = {nullptr};  // one word per device, allocated on first use
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return O64_OK;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!flags[dev] && cudaMalloc(&flags[dev], sizeof(int)) != cudaSuccess) {
        (void)cudaGetLastError();
        flags[dev] = nullptr;
        return O64_OK;
    }
    int bad = 0;
    if (cudaMemsetAsync(flags[dev], 0, sizeof(int), s) != cudaSuccess) return O64_ERR_CUDA;
    const long long total = (long long)o_rows * o_cols;
    nonfinite_f64_kernel<<<(unsigned)std::min<long long>((total + 255) / 256, 148 * 8), 256, 0, s>>>(other, o_rows, o_cols, o_ld, flags[dev]);
    if (cudaMemcpyAsync(&bad, flags[dev], sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess)
        return O64_ERR_CUDA;
    if (bad) return O64_OK;  // the general kernel keeps the rule about zero factors
    dim3 grid((unsigned)((Nr + 63) / 64), (unsigned)((Mr + 63) / 64));
    static const int mma_env = [] { const char *e = getenv("O64_F64_MMA"); return e ? atoi(e) : 1; }();
    static bool mma_ready[64] = {false};  // the larger dynamic shared memory is allowed per device
    if (mma_env && !mma_ready[dev]) {
        bool ok = true;
        ok &= cudaFuncSetAttribute(dense_f64_mma_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kF64MmaSmemBytes) == cudaSuccess;
        ok &= cudaFuncSetAttribute(dense_f64_mma_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kF64MmaSmemBytes) == cudaSuccess;
        ok &= cudaFuncSetAttribute(dense_f64_mma_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kF64MmaSmemBytes) == cudaSuccess;
        ok &= cudaFuncSetAttribute(dense_f64_mma_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kF64MmaSmemBytes) == cudaSuccess;
        mma_ready[dev] = ok;
        if (!ok) (void)cudaGetLastError();
    }
    if (mma_env && mma_ready[dev]) {
        if (x_mfast && w_kfast)
            dense_f64_mma_kernel<true, true><<<grid, 256, kF64MmaSmemBytes, s>>>(Mr, Nr, K, alpha, X, ldx, W, ldw, beta, Y, ldy);
        else if (x_mfast)
            dense_f64_mma_kernel<true, false><<<grid, 256, kF64MmaSmemBytes, s>>>(Mr, Nr, K, alpha, X, ldx, W, ldw, beta, Y, ldy);
        else if (w_kfast)
            dense_f64_mma_kernel<false, true><<<grid, 256, kF64MmaSmemBytes, s>>>(Mr, Nr, K, alpha, X, ldx, W, ldw, beta, Y, ldy);
        else
            dense_f64_mma_kernel<false, false><<<grid, 256, kF64MmaSmemBytes, s>>>(Mr, Nr, K, alpha, X, ldx, W, ldw, beta, Y, ldy);
    } else if (!x_mfast && !w_kfast) {
        // (128 x 64 tiles with 8 x 4 register blocks were measured too: 16.0 TFLOP/s at 2048^3 against 17.8 for
        // these - fewer CTAs per SM cover the load latency less well)
        dense_f64_kernel<4><<<grid, 256, 0, s>>>(Mr, Nr, K, alpha, X, ldx, W, ldw, beta, Y, ldy);
    } else {
        return O64_OK;  // transposed operands without the tensor path: the general kernel
    }
    *done = true;
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

template <typename T>
__global__ void gemvx_generic_kernel(long long M, long long N, T alpha, const T *A, long long a1, long long a2,
                                     const T *X, long long incx, T beta, T *Y, long long incy, int conj_a) {
    const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= M) return;
    T *y = Y + row * incy;
    T acc = (beta == T(0)) ? T(0) : mul<T>(beta, *y);
    for (long long j = 0; j < N; ++j) {
        const T x = X[j * incx];
        if (x != T(0)) acc = acc + mul<T>(mul<T>(alpha, x), conj_if(A[row * a1 + j * a2], conj_a));
    }
    *y = acc;
}

template <typename T>
__global__ void scale_generic_kernel(long long M, long long N, T beta, T *C, long long c1, long long c2) {
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= M * N) return;
    T *c = C + (e % M) * c1 + (e / M) * c2;
    *c = (beta == T(0)) ? T(0) : mul<T>(beta, *c);
}

template <typename TA, typename T>
int generic_gemmx(int64_t M, int64_t N, int64_t K, T alpha, const TA *A, int64_t a1, int64_t a2, const T *B,
                  int64_t b1, int64_t b2, T beta, T *C, int64_t c1, int64_t c2, cudaStream_t s, int conj_a, int conj_b) {
    if (M <= 0 || N <= 0) return O64_OK;
    if constexpr (std::is_same<T, double>::value && std::is_same<TA, double>::value) {
        if (!conj_a && !conj_b) {
            bool done = false;
            const int rc = try_dense_f64(M, N, K, alpha, A, a1, a2, B, b1, b2, beta, C, c1, c2, s, &done);
            if (rc || done) return rc;
        }
    }
    if ((M + 31) / 32 > 65535) return O64_ERR_RANK;
    auto mag = [](int64_t v) { return v < 0 ? -v : v; };
    dim3 grid((unsigned)((N + 31) / 32), (unsigned)((M + 31) / 32));
    gemmx_generic_kernel<TA, T><<<grid, 256, 0, s>>>(M, N, K, alpha, A, a1, a2, B, b1, b2, beta, C, c1, c2,
                                                 mag(a2) <= mag(a1), mag(b2) <= mag(b1), conj_a, conj_b);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

template <typename T>
int generic_gemvx(int64_t M, int64_t N, T alpha, const T *A, int64_t a1, int64_t a2, const T *X, int64_t incx,
                  T beta, T *Y, int64_t incy, cudaStream_t s, int conj_a) {
    if (M <= 0) return O64_OK;
    gemvx_generic_kernel<T><<<(unsigned)((M + 127) / 128), 128, 0, s>>>(M, N, alpha, A, a1, a2, X, incx, beta, Y, incy, conj_a);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

template <typename T>
int generic_scale(int64_t M, int64_t N, T beta, T *C, int64_t c1, int64_t c2, cudaStream_t s) {
    if (M <= 0 || N <= 0) return O64_OK;
    const long long total = (long long)M * N;
    scale_generic_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, s>>>(M, N, beta, C, c1, c2);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}

// LOGICAL kinds (osprey/libfi/matrix/lgemmx.h): C(i,j) = (beta .AND. C(i,j)) .OR. (alpha .AND. OR over l of
// A(i,l) .AND. B(l,j)); any non-zero value is true, results are stored as 1 / 0.  One thread per
// result element: a logical MATMUL is rare and small.
template <typename TA, typename T>
__global__ void lgemmx_kernel(long long M, long long N, long long K, int alpha, const TA *A, long long a1, long long a2,
                              const T *B, long long b1, long long b2, int beta, T *C, long long c1, long long c2) {
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= M * N) return;
    const long long i = e % M, j = e / M;
    T *c = C + i * c1 + j * c2;
    bool acc = beta && (*c != T(0));
    if (alpha)
        for (long long l = 0; l < K && !acc; ++l) acc = (B[l * b1 + j * b2] != T(0)) && (A[i * a1 + l * a2] != TA(0));
    *c = acc ? T(1) : T(0);
}

template <typename TA, typename T>
int logical_gemmx(int64_t M, int64_t N, int64_t K, int alpha, const TA *A, int64_t a1, int64_t a2, const T *B,
                  int64_t b1, int64_t b2, int beta, T *C, int64_t c1, int64_t c2, cudaStream_t s) {
    if (M <= 0 || N <= 0) return O64_OK;
    const long long total = (long long)M * N;
    lgemmx_kernel<TA, T><<<(unsigned)((total + 255) / 256), 256, 0, s>>>(M, N, K, alpha, A, a1, a2, B, b1, b2, beta, C, c1, c2);
    return cudaGetLastError() == cudaSuccess ? O64_OK : O64_ERR_CUDA;
}
#define O64_INSTANTIATE_LGEMMX(TA, T)                                                                          \
    template int logical_gemmx<TA, T>(int64_t, int64_t, int64_t, int, const TA *, int64_t, int64_t, const T *,    \
                                      int64_t, int64_t, int, T *, int64_t, int64_t, cudaStream_t);
O64_INSTANTIATE_LGEMMX(int8_t, int8_t)
O64_INSTANTIATE_LGEMMX(int8_t, int16_t)
O64_INSTANTIATE_LGEMMX(int8_t, int32_t)
O64_INSTANTIATE_LGEMMX(int8_t, int64_t)
O64_INSTANTIATE_LGEMMX(int16_t, int16_t)
O64_INSTANTIATE_LGEMMX(int16_t, int32_t)
O64_INSTANTIATE_LGEMMX(int16_t, int64_t)
O64_INSTANTIATE_LGEMMX(int32_t, int32_t)
O64_INSTANTIATE_LGEMMX(int32_t, int64_t)
O64_INSTANTIATE_LGEMMX(int64_t, int64_t)
#undef O64_INSTANTIATE_LGEMMX

#define O64_INSTANTIATE_GEMMX(TA, T)                                                                          \
    template int generic_gemmx<TA, T>(int64_t, int64_t, int64_t, T, const TA *, int64_t, int64_t, const T *,     \
                                      int64_t, int64_t, T, T *, int64_t, int64_t, cudaStream_t, int, int);
#define O64_INSTANTIATE_SCALE(T) template int generic_scale<T>(int64_t, int64_t, T, T *, int64_t, int64_t, cudaStream_t);
O64_INSTANTIATE_GEMMX(double, double)
O64_INSTANTIATE_GEMMX(int8_t, uint8_t)
O64_INSTANTIATE_GEMMX(int8_t, uint16_t)
O64_INSTANTIATE_GEMMX(int8_t, uint32_t)
O64_INSTANTIATE_GEMMX(int8_t, uint64_t)
O64_INSTANTIATE_GEMMX(int16_t, uint16_t)
O64_INSTANTIATE_GEMMX(int16_t, uint32_t)
O64_INSTANTIATE_GEMMX(int16_t, uint64_t)
O64_INSTANTIATE_GEMMX(int32_t, uint32_t)
O64_INSTANTIATE_GEMMX(int32_t, uint64_t)
O64_INSTANTIATE_GEMMX(int64_t, uint64_t)
O64_INSTANTIATE_GEMMX(float, double)
O64_INSTANTIATE_GEMMX(int8_t, float)
O64_INSTANTIATE_GEMMX(int16_t, float)
O64_INSTANTIATE_GEMMX(int32_t, float)
O64_INSTANTIATE_GEMMX(int64_t, float)
O64_INSTANTIATE_GEMMX(int8_t, double)
O64_INSTANTIATE_GEMMX(int16_t, double)
O64_INSTANTIATE_GEMMX(int32_t, double)
O64_INSTANTIATE_GEMMX(int64_t, double)
O64_INSTANTIATE_SCALE(float)
O64_INSTANTIATE_SCALE(double)
O64_INSTANTIATE_SCALE(uint8_t)
O64_INSTANTIATE_SCALE(uint16_t)
O64_INSTANTIATE_SCALE(uint32_t)
O64_INSTANTIATE_SCALE(uint64_t)
#define O64_INSTANTIATE_GEMVX(T)                                                                              \
    template int generic_gemvx<T>(int64_t, int64_t, T, const T *, int64_t, int64_t, const T *, int64_t, T, T *,  \
                                  int64_t, cudaStream_t, int);
O64_INSTANTIATE_GEMVX(double)
O64_INSTANTIATE_GEMVX(Cx<float>)
O64_INSTANTIATE_GEMVX(Cx<double>)
O64_INSTANTIATE_GEMMX(Cx<float>, Cx<float>)
O64_INSTANTIATE_GEMMX(Cx<double>, Cx<double>)
O64_INSTANTIATE_SCALE(Cx<float>)
O64_INSTANTIATE_SCALE(Cx<double>)
#undef O64_INSTANTIATE_GEMVX
#undef O64_INSTANTIATE_GEMMX
#undef O64_INSTANTIATE_SCALE

}  // namespace o64
