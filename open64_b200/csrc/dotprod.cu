// DOT_PRODUCT on the GPU: the sibling of MATMUL in the reference's runtime
// (osprey/libfi/dotprod/dot90.h:83-86: s = 0; do i: s = s + x(1+(i-1)*incx) * y(1+(i-1)*incy);
// dotc90.h:84-87 conjugates x for COMPLEX; dotl90.h:84-87 is s = s .OR. (x .AND. y)).
// One pass over both vectors, bound by memory: a grid of blocks forms partial sums in a fixed
// order (so the result does not depend on timing), a second one-block kernel adds them.
#include <cuda_runtime.h>

#include "../../include/o64gemm.h"
#include "simt_kernels.cuh"

namespace o64 {

namespace {
constexpr int kDotThreads = 256;
constexpr int kDotMaxBlocks = 592;  // 4 per SM of a B200

template <typename T>
struct DotOps {
    __device__ static T zero() { return T(0); }
    __device__ static T add(T a, T b) { return a + b; }
};

// MODE: 0 = arithmetic (operands converted to TR, integers carried on unsigned types so that they
// wrap), 1 = LOGICAL (non-zero is true; TR holds 0 / 1), 2 = COMPLEX with x conjugated
template <typename TX, typename TY, typename TR, int MODE>
__device__ __forceinline__ TR dot_term(const TX &x, const TY &y) {
    if constexpr (MODE == 1) {
        return (x != TX(0) && y != TY(0)) ? TR(1) : TR(0);
    } else if constexpr (MODE == 2) {
        const TR a(x.re, -x.im), b(y.re, y.im);
        return a * b;
    } else {
        return TR(x) * TR(y);
    }
}

template <typename TR, int MODE>
__device__ __forceinline__ TR dot_join(const TR &a, const TR &b) {
    if constexpr (MODE == 1)
        return (a != TR(0) || b != TR(0)) ? TR(1) : TR(0);
    else
        return a + b;
}

template <typename TR, int MODE>
__device__ __forceinline__ TR block_reduce(TR v, TR *smem) {
    smem[threadIdx.x] = v;
    __syncthreads();
    for (int s = kDotThreads / 2; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) smem[threadIdx.x] = dot_join<TR, MODE>(smem[threadIdx.x], smem[threadIdx.x + s]);
        __syncthreads();
    }
    return smem[0];
}

template <typename TX, typename TY, typename TR, int MODE>
__global__ void dot_partial_kernel(long long n, const TX *x, long long incx, const TY *y, long long incy, TR *partial) {
    __shared__ TR smem[kDotThreads];
    TR acc = TR(0);
    for (long long i = (long long)blockIdx.x * kDotThreads + threadIdx.x; i < n; i += (long long)gridDim.x * kDotThreads)
        acc = dot_join<TR, MODE>(acc, dot_term<TX, TY, TR, MODE>(x[i * incx], y[i * incy]));
    const TR total = block_reduce<TR, MODE>(acc, smem);
    if (threadIdx.x == 0) partial[blockIdx.x] = total;
}

template <typename TR, int MODE>
__global__ void dot_final_kernel(const TR *partial, int nblocks, TR *out) {
    __shared__ TR smem[kDotThreads];
    TR acc = TR(0);
    for (int i = threadIdx.x; i < nblocks; i += kDotThreads) acc = dot_join<TR, MODE>(acc, partial[i]);
    const TR total = block_reduce<TR, MODE>(acc, smem);
    if (threadIdx.x == 0) *out = total;
}
}  // namespace

size_t dot_workspace_bytes() { return (size_t)(kDotMaxBlocks + 1) * 16; }  // partials + the result, 16 bytes each at most

template <typename TX, typename TY, typename TR, int MODE>
int dot_device(long long n, const TX *x, long long incx, const TY *y, long long incy, void *workspace, TR *host_result,
               cudaStream_t s) {
    TR *partial = static_cast<TR *>(workspace);
    TR *out = partial + kDotMaxBlocks;
    long long blocks = (n + kDotThreads - 1) / kDotThreads;
    if (blocks > kDotMaxBlocks) blocks = kDotMaxBlocks;
    if (blocks < 1) blocks = 1;
    dot_partial_kernel<TX, TY, TR, MODE><<<(unsigned)blocks, kDotThreads, 0, s>>>(n, x, incx, y, incy, partial);
    dot_final_kernel<TR, MODE><<<1, kDotThreads, 0, s>>>(partial, (int)blocks, out);
    if (cudaGetLastError() != cudaSuccess) return O64_ERR_CUDA;
    if (cudaMemcpyAsync(host_result, out, sizeof(TR), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        (void)cudaGetLastError();
        return O64_ERR_CUDA;
    }
    return O64_OK;
}

#define O64_DOT_INST(TX, TY, TR, MODE) \
    template int dot_device<TX, TY, TR, MODE>(long long, const TX *, long long, const TY *, long long, void *, TR *, cudaStream_t);
// REAL and INTEGER kinds and their mixed pairs (result: the wider or the real kind)
O64_DOT_INST(float, float, float, 0)
O64_DOT_INST(double, double, double, 0)
O64_DOT_INST(float, double, double, 0)
O64_DOT_INST(double, float, double, 0)
O64_DOT_INST(int32_t, int32_t, uint32_t, 0)
O64_DOT_INST(int64_t, int64_t, uint64_t, 0)
O64_DOT_INST(int32_t, int64_t, uint64_t, 0)
O64_DOT_INST(int64_t, int32_t, uint64_t, 0)
O64_DOT_INST(int32_t, float, float, 0)
O64_DOT_INST(float, int32_t, float, 0)
O64_DOT_INST(int32_t, double, double, 0)
O64_DOT_INST(double, int32_t, double, 0)
O64_DOT_INST(int64_t, float, float, 0)
O64_DOT_INST(float, int64_t, float, 0)
O64_DOT_INST(int64_t, double, double, 0)
O64_DOT_INST(double, int64_t, double, 0)
// LOGICAL kinds
O64_DOT_INST(int32_t, int32_t, int32_t, 1)
O64_DOT_INST(int64_t, int64_t, int64_t, 1)
O64_DOT_INST(int32_t, int64_t, int64_t, 1)
O64_DOT_INST(int64_t, int32_t, int64_t, 1)
// COMPLEX*8 and COMPLEX*16: sum of conjg(x) * y
O64_DOT_INST(Cx<float>, Cx<float>, Cx<float>, 2)
O64_DOT_INST(Cx<double>, Cx<double>, Cx<double>, 2)
#undef O64_DOT_INST

}  // namespace o64
