// o64_gemm_s8s8_s32_static: the int8 GEMM for callers that must not allocate device memory.
//
// Who needs it: host code that runs with a fixed device-memory plan.  A program compiled ahead
// of time may have handed every byte of the device heap to its own arena, or may call the GEMM
// from a section in which cudaMalloc is forbidden because it synchronises the device and can fail
// under memory pressure.  Such a caller cannot use a handle (o64_create allocates the status word,
// and unaligned operands make the handle grow scratch buffers on demand).
//
// This entry point takes no handle and calls no cudaMalloc, cudaFree or allocating library
// routine.  Everything the kernel needs beyond the caller's A, B and C lives in one file-scope
// device array of O64_STATIC_SCRATCH_BYTES that every GPU holding the library keeps until the
// process exits:
//   bytes [0, 256)   the device status word of the bounded waits (cleared by every call)
//   the rest         operands copied to a padded pitch when the caller's base address or row
//                    pitch is not a multiple of 16 bytes (TMA cannot address those directly)
// A call whose padded copies do not fit returns O64_ERR_NOMEM and touches nothing.
//
// The array's name is only a host-side stand-in: the device address comes from
// cudaGetSymbolAddress, once per device, on the first call made with that device current.  Make
// that first call before any stream capture begins.  A, B and C must be memory of the device that
// is current at the call (or managed memory) and `stream` a stream of that device; operands of
// another device are refused with O64_ERR_RANK before anything is launched.
//
// All calls on a device share the array and it keeps the previous call's contents, so two calls
// that overlap on the GPU (different streams, no dependency) race on it; serialise them.  A wait
// that times out inside the kernel still ends the kernel, but this variant has nowhere to report
// it: use the handle-based entry point when you need o64_last_status.
#include <cuda_runtime.h>

#include <cstring>

#include <mutex>

#include "../../include/o64gemm.h"
#include "umma_gemm.cuh"

namespace {

constexpr size_t kScratchBytes = O64_STATIC_SCRATCH_BYTES;
constexpr size_t kStatusBytes = 256;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

struct PerDevice {
    unsigned char *scratch = nullptr;  // device address of g_static_scratch on this device
    int num_sms = 0;
    int index = 0;
    bool ready = false;
};
PerDevice g_devices[kMaxDevices];
std::mutex g_setup_mutex;

// Once per device, with that device current: resolve the array's device address.
int setup_current_device(PerDevice **out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        return O64_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    PerDevice &d = g_devices[dev];
    if (!d.ready) {
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) {
            (void)cudaGetLastError();
            return O64_ERR_CUDA;
        }
        int major = 0, sms = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
            (void)cudaGetLastError();
            return O64_ERR_CUDA;
        }
        if (major != 10) return O64_ERR_DTYPE;  // the kernels are sm_100a only
        d.scratch = static_cast<unsigned char *>(ptr);
        d.num_sms = sms;
        d.index = dev;
        d.ready = true;
    }
    *out = &d;
    return O64_OK;
}

// Device (or managed) memory, and memory of the device this call runs on: the padded copies and
// the tensor maps below are made for the current device, so an operand that lives on another GPU
// would end in a launch failure or in reads over a peer link nobody asked for.
bool is_pointer_of_device(const void *p, int dev) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    if (a.type == cudaMemoryTypeManaged) return true;
    return a.type == cudaMemoryTypeDevice && a.device == dev;
}

bool tma_addressable(const void *p, int64_t ld_bytes) {
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && (ld_bytes % 16) == 0;
}

size_t padded_bytes(int64_t rows, int64_t cols) { return (size_t)rows * (size_t)((cols + 15) / 16 * 16); }

}  // namespace

extern "C" int o64_gemm_s8s8_s32_static(int64_t M, int64_t N, int64_t K, const int8_t *A, int64_t lda,
                                        const int8_t *B, int64_t ldb, int32_t *C, int64_t ldc,
                                        void *stream) {
    if (M < 0 || N < 0 || K < 0) return O64_ERR_RANK;
    if (M == 0 || N == 0) return O64_OK;
    if (K == 0 || !A || !B || !C) return O64_ERR_RANK;
    if (lda < K || ldb < K || ldc < N) return O64_ERR_CONFORM;
    PerDevice *d = nullptr;
    int rc = setup_current_device(&d);
    if (rc) return rc;
    // host operands would need staging, i.e. an allocation; operands of another GPU are refused
    if (!is_pointer_of_device(A, d->index) || !is_pointer_of_device(B, d->index) || !is_pointer_of_device(C, d->index))
        return O64_ERR_RANK;
    cudaStream_t s = (cudaStream_t)stream;

    // operands TMA cannot address are copied to a 16-byte pitch inside the static array
    const bool copy_a = !tma_addressable(A, lda), copy_b = !tma_addressable(B, ldb);
    const size_t bytes_a = copy_a ? (padded_bytes(M, K) + 255) / 256 * 256 : 0;
    const size_t bytes_b = copy_b ? padded_bytes(N, K) : 0;
    if (kStatusBytes + bytes_a + bytes_b > kScratchBytes) return O64_ERR_NOMEM;

    int *status_word = reinterpret_cast<int *>(d->scratch);
    if (cudaMemsetAsync(status_word, 0, sizeof(int), s) != cudaSuccess) {  // must start at zero
        (void)cudaGetLastError();
        return O64_ERR_CUDA;
    }
    const int8_t *a_use = A, *b_use = B;
    int64_t lda_use = lda, ldb_use = ldb;
    if (copy_a) {
        int8_t *dst = reinterpret_cast<int8_t *>(d->scratch + kStatusBytes);
        lda_use = (K + 15) / 16 * 16;
        if (cudaMemcpy2DAsync(dst, (size_t)lda_use, A, (size_t)lda, (size_t)K, (size_t)M,
                              cudaMemcpyDeviceToDevice, s) != cudaSuccess) {
            (void)cudaGetLastError();
            return O64_ERR_CUDA;
        }
        a_use = dst;
    }
    if (copy_b) {
        int8_t *dst = reinterpret_cast<int8_t *>(d->scratch + kStatusBytes + bytes_a);
        ldb_use = (K + 15) / 16 * 16;
        if (cudaMemcpy2DAsync(dst, (size_t)ldb_use, B, (size_t)ldb, (size_t)K, (size_t)N,
                              cudaMemcpyDeviceToDevice, s) != cudaSuccess) {
            (void)cudaGetLastError();
            return O64_ERR_CUDA;
        }
        b_use = dst;
    }

    o64::UmmaCall c;
    c.kind = O64_KIND_S8;
    c.b_kn = false;
    c.epi = o64::EPI_S32;
    c.M = M; c.N = N; c.K = K;
    c.A = a_use; c.lda = lda_use;
    c.B = b_use; c.B2 = nullptr; c.ldb = ldb_use;
    c.C = C; c.ldc = ldc;
    c.bias = nullptr; c.scale_a = nullptr; c.scale_b = nullptr;
    c.act = O64_ACT_NONE;
    o64_plan_t pin;
    memset(&pin, 0, sizeof(pin));
    pin.split_k = 1;  // the tile kernels only: this entry point is specified on their scratch use
    o64::plan_choose(O64_KIND_S8, o64::EPI_S32, M, N, K, d->num_sms, &pin, &c.plan);
    c.status_word = status_word;
    c.stream = s;
    c.may_allocate = false;
    return o64::umma_launch(c);
}
