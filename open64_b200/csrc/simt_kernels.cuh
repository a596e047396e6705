// Host-side interface of the CUDA-core kernels (simt_kernels.cu): the fp32 fused linear /
// strided GEMM, the strided GEMV, the one-thread-per-output reference kernels and the slab
// permute used after the all-gather.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace o64 {

// C(i,j) = act( alpha * sum_l A(i,l)*B(l,j) + beta*C(i,j) + bias[j] ), fp32, with
// X(i,j) at X[i*x1 + j*x2].  skip_zero_b: leave out terms whose B(l,j) == 0, as the
// reference's runtime kernel does (osprey/libfi/matrix/xgemmx.h:227).
struct SimtGemmCall {
    int64_t M, N, K;
    float alpha, beta;
    const float *A;
    int64_t a1, a2;
    const float *B;
    int64_t b1, b2;
    float *C;
    int64_t c1, c2;
    const float *bias;
    int act;
    bool skip_zero_b;
    int num_sms;
    cudaStream_t stream;
    int pin_tile_m = 0, pin_tile_n = 0;  // dense kernel: 0 = choose, else 32 or 64
};
int simt_gemm_f32(const SimtGemmCall &c);
// Dense row-major fast path of simt_gemm_f32: whether a call qualifies, and the CTA tile it gets.
bool simt_dense_ok(const SimtGemmCall &c);
void simt_dense_tile(int64_t M, int64_t N, int num_sms, int *tile_m, int *tile_n);
// Applies a pinned tile (0 = keep the chosen value); the pair 64 x 32 has no kernel and becomes 64 x 64.
void simt_apply_pin(int pin_m, int pin_n, int *tile_m, int *tile_n);

// y(i) = alpha * sum_j A(i,j)*x(j) + beta*y(i); terms with x(j) == 0 are left out
// (osprey/libfi/matrix/s4gemvx.f).
int simt_gemv_f32(int64_t M, int64_t N, float alpha, const float *A, int64_t a1, int64_t a2,
                  const float *X, int64_t incx, float beta, float *Y, int64_t incy,
                  cudaStream_t stream);

// Scales or zeroes C in place: C = beta*C (beta == 0 writes zeros without reading C).
int simt_scale_f32(int64_t M, int64_t N, float beta, float *C, int64_t c1, int64_t c2,
                   cudaStream_t stream);

int naive_gemm(int kind, int64_t M, int64_t N, int64_t K, const void *A, int64_t lda, const void *B,
               int64_t ldb, int transB, const float *scaleA, const float *scaleB, const float *bias,
               int act, void *out, int64_t ldo, cudaStream_t stream);

// Second pass of a split-K GEMM with a 16-bit result: C = bf16(act(partial * sa[m] * sb[n] + bias[n])),
// `partial` a dense fp32 [M,N], or NULL for the empty sum (every partial zero).  scale vectors and bias may be NULL.
// out_kind: 0 = bf16 (ldc in 2-byte elements), 1 = int8, 2 = e4m3 (both round to nearest even, saturating;
// ldc in bytes).
int finalize_partial_bf16(const float *partial, int64_t M, int64_t N, const float *scale_a,
                          const float *scale_b, const float *bias, int act, void *C, int64_t ldc,
                          cudaStream_t stream, int out_kind = 0);

// COMPLEX*8 / COMPLEX*16 element: (re, im) as Fortran stores it.
template <typename R>
struct Cx {
    R re, im;
    Cx() = default;
    __host__ __device__ Cx(R r) : re(r), im(R(0)) {}
    __host__ __device__ Cx(R r, R i) : re(r), im(i) {}
    __host__ __device__ Cx operator+(const Cx &o) const { return Cx(re + o.re, im + o.im); }
    __host__ __device__ Cx operator*(const Cx &o) const { return Cx(re * o.re - im * o.im, re * o.im + im * o.re); }
    __host__ __device__ bool operator==(const Cx &o) const { return re == o.re && im == o.im; }
    __host__ __device__ bool operator!=(const Cx &o) const { return !(*this == o); }
};

// The same strided operations for REAL*8 and the integer kinds (simt_generic.cu).  T is the kind
// of B and C (integers: the unsigned type of that width); TA the kind of A (integers: signed, of
// the same or a smaller width, sign-extended to T).  conj_a / conj_b: use the conjugate of a
// complex operand (the complex kernels of the runtime take these flags, osprey/libfi/matrix/c4gemmx.f:77-85).
template <typename TA, typename T>
int generic_gemmx(int64_t M, int64_t N, int64_t K, T alpha, const TA *A, int64_t a1, int64_t a2, const T *B,
                  int64_t b1, int64_t b2, T beta, T *C, int64_t c1, int64_t c2, cudaStream_t s, int conj_a = 0,
                  int conj_b = 0);
template <typename T>
int generic_gemvx(int64_t M, int64_t N, T alpha, const T *A, int64_t a1, int64_t a2, const T *X, int64_t incx,
                  T beta, T *Y, int64_t incy, cudaStream_t s, int conj_a = 0);
template <typename T>
int generic_scale(int64_t M, int64_t N, T beta, T *C, int64_t c1, int64_t c2, cudaStream_t s);

// DOT_PRODUCT (dotprod.cu): sum over i of x(i) * y(i) with element strides, formed in TR (integers on
// the unsigned type of the result's width); MODE 0 arithmetic, 1 LOGICAL (.OR. of .AND.), 2 COMPLEX with
// x conjugated.  `workspace`: device memory of dot_workspace_bytes(); the result arrives in *host_result
// and the call waits for it.
size_t dot_workspace_bytes();
template <typename TX, typename TY, typename TR, int MODE>
int dot_device(long long n, const TX *x, long long incx, const TY *y, long long incy, void *workspace, TR *host_result,
               cudaStream_t s);

// LOGICAL kinds: C = (beta AND C) OR (alpha AND (A AND B, OR-reduced over K)); non-zero is true.
template <typename TA, typename T>
int logical_gemmx(int64_t M, int64_t N, int64_t K, int alpha, const TA *A, int64_t a1, int64_t a2, const T *B,
                  int64_t b1, int64_t b2, int beta, T *C, int64_t c1, int64_t c2, cudaStream_t s);

// Fills a buffer with pseudo-random finite values of the kind (bf16 / e4m3 / int8): operands for timing runs.
int fill_pattern(void *p, size_t bytes, int kind, cudaStream_t stream);

// dst[c][r] = src[r][c], one-byte elements, leading dimensions in elements.
int transpose_bytes(const void *src, int64_t ld_src, void *dst, int64_t ld_dst, int64_t rows, int64_t cols,
                    cudaStream_t stream);

// dst[m][r*ncols + j] = src[r][m][j] for r < nslabs (int32 elements).
int permute_slabs_s32(const int32_t *src, int32_t *dst, int64_t M, int64_t ncols, int nslabs,
                      int64_t ld_dst, cudaStream_t stream);

}  // namespace o64
