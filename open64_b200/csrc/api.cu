// The C ABI of libo64gemm.so (include/o64gemm.h): handle management, argument checking in the
// manner of the reference runtime's _premult (osprey/libfi/matrix/matmul.h:135-400, errors as
// return codes instead of aborts), staging of host operands, the compat entry points and the
// column-sharded int8 GEMM with its all-gather.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <array>
#include <initializer_list>
#include <map>
#include <mutex>
#include <new>
#include <string>
#include <type_traits>
#include <vector>

#include "../../include/o64gemm.h"
#include "simt_kernels.cuh"
#include "umma_gemm.cuh"

using namespace o64;

// ---- NCCL, bound at run time --------------------------------------------------------------
// The library is resolved with dlopen so that libo64gemm.so loads (and its symbols can be
// listed) on hosts without NCCL or without a GPU.  Prototypes follow nccl.h.
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId_;
struct NcclApi {
    void *lib = nullptr;
    int (*GetUniqueId)(ncclUniqueId_ *) = nullptr;
    int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId_, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool ok = false;
};
static const int kNcclInt32 = 2;
static const int kNcclBfloat16 = 9;  // ncclBfloat16 in ncclDataType_t
static const int kNcclInt8 = 0;
static const int kNcclSum = 0;

static NcclApi &nccl() {
    static NcclApi api;
    static bool tried = false;
    if (tried) return api;
    tried = true;
    const char *names[] = {getenv("O64_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        if (!n || !*n) continue;
        api.lib = dlopen(n, RTLD_NOW | RTLD_NOLOAD);  // prefer the copy the process already has
        if (!api.lib) api.lib = dlopen(n, RTLD_NOW);
        if (api.lib) break;
    }
    if (!api.lib) return api;
    api.GetUniqueId = (int (*)(ncclUniqueId_ *))dlsym(api.lib, "ncclGetUniqueId");
    api.CommInitRank = (int (*)(ncclComm_t *, int, ncclUniqueId_, int))dlsym(api.lib, "ncclCommInitRank");
    api.CommDestroy = (int (*)(ncclComm_t))dlsym(api.lib, "ncclCommDestroy");
    api.AllGather = (int (*)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t))dlsym(
        api.lib, "ncclAllGather");
    api.AllReduce = (int (*)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t))dlsym(
        api.lib, "ncclAllReduce");
    api.GetErrorString = (const char *(*)(int))dlsym(api.lib, "ncclGetErrorString");
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.AllReduce;
    return api;
}

// ---- handle ---------------------------------------------------------------------------------
static const int kSlots = 10;  // 0-5 host staging, 6-8 repacked operands (A, B, B2), 9 a transposed 8-bit weight
static const int kMaxBlocks = 32;       // row blocks of a pipelined host-operand call
static const int64_t kBlockRows = 1024;  // at least this many rows per block

struct o64_handle_s {
    int device = 0;
    int num_sms = 148;
    int *status_word = nullptr;
    o64_plan_t pins[4];
    bool has_pin[4] = {false, false, false, false};
    void *stage[kSlots] = {nullptr};
    size_t stage_cap[kSlots] = {0};
    void *ws = nullptr;
    size_t ws_cap = 0;
    // plans found by o64_plan_tune, by (kind, SwiGLU?, M, N, K): used when the kind has no pin
    // (key: kind, SwiGLU?, M, N, K, ranks of the communicator; predicted_ms holds the measured time)
    std::map<std::array<int64_t, 6>, o64_plan_t> tuned;
    char device_name[128] = {0};
    // host operands of a large product travel in row blocks on two side streams, so that the
    // copies in both directions overlap the kernels (created on first use)
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t ev_entry = nullptr, ev_done = nullptr;
    cudaEvent_t ev_in[kMaxBlocks] = {nullptr}, ev_mm[kMaxBlocks] = {nullptr};
    ncclComm_t comm = nullptr;
    int rank = 0, nranks = 1;
    // symmetric result buffer for the fused GEMM + all-gather (one allocation per rank, every
    // rank holds peer-mapped pointers to the others')
    void *sym_local = nullptr;
    void *sym_peer[8] = {nullptr};  // indexed by rank; [rank] == sym_local
    size_t sym_bytes = 0;
    // the exchange's counters (kXchgWords words, zeroed): an allocation of their own, mapped into every
    // rank like the result.  (Kept out of the result's allocation on purpose: with 256 bytes of counters
    // behind a 512 MiB result the allocation was no longer a whole number of large pages, and with seven
    // peers' mappings of that kind the remote stores of the fused kernel ran at 96 GB/s instead of 600.)
    void *xchg_local = nullptr;
    void *xchg_peer[8] = {nullptr};
    bool push_nccl_barriers = false;  // O64_PUSH_NCCL_BARRIER=1: order the ranks with two tiny all-reduces instead
    int *barrier_word = nullptr;    // one int, reduced over the ranks as a stream-ordered barrier
    unsigned long long wait_ns = 0;  // budget of the kernels' bounded waits; 0 = the default (two seconds)
    // CTA-pair kernels: slots and flags for the K split of a last, partly filled wave of tiles
    // (allocated on the first launch of such a kernel; the kernels leave the flags at zero)
    void *tail_slots = nullptr;
    unsigned *tail_flags = nullptr;
};

#define CUDA_TRY(x)                          \
    do {                                     \
        if ((x) != cudaSuccess) {            \
            (void)cudaGetLastError();        \
            return O64_ERR_CUDA;             \
        }                                    \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    bool ok;
    explicit DeviceGuard(int dev) {
        ok = cudaGetDevice(&prev) == cudaSuccess;
        if (ok && prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

extern "C" const char *o64_version(void) { return "o64gemm 0.1 (sm_100a)"; }

extern "C" const char *o64_status_string(int s) {
    switch (s) {
    case O64_OK: return "ok";
    case O64_ERR_RANK: return "illegal rank or argument";
    case O64_ERR_CONFORM: return "operands not conformable";
    case O64_ERR_NOMEM: return "out of memory";
    case O64_ERR_ALIGN: return "operand not 16-byte aligned";
    case O64_ERR_DTYPE: return "unsupported element type or layout";
    case O64_ERR_TIMEOUT: return "device-side wait timed out";
    case O64_ERR_CUDA: return "CUDA call failed";
    case O64_ERR_NCCL: return "NCCL call failed or no communicator";
    default: return "unknown status";
    }
}

extern "C" int o64_create(o64_handle_t *out, int device) {
    if (!out) return O64_ERR_RANK;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        (void)cudaGetLastError();
        return O64_ERR_CUDA;
    }
    DeviceGuard g(device);
    if (!g.ok) return O64_ERR_CUDA;
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return O64_ERR_DTYPE;  // the kernels are sm_100a only
    o64_handle_s *h = new (std::nothrow) o64_handle_s();
    if (!h) return O64_ERR_NOMEM;
    h->device = device;
    h->num_sms = prop.multiProcessorCount;
    strncpy(h->device_name, prop.name, sizeof(h->device_name) - 1);
    memset(h->pins, 0, sizeof(h->pins));
    if (const char *wb = getenv("O64_WAIT_BUDGET_US")) {
        const long long us = atoll(wb);
        if (us > 0) h->wait_ns = (unsigned long long)us * 1000ull;
    }
    if (cudaMalloc(&h->status_word, sizeof(int)) != cudaSuccess) {
        delete h;
        return O64_ERR_NOMEM;
    }
    cudaMemset(h->status_word, 0, sizeof(int));
    *out = h;
    if (const char *cache = getenv("O64_PLAN_CACHE")) (void)o64_plan_load(h, cache);  // a missing file is fine
    return O64_OK;
}

static void free_symmetric(o64_handle_t h) {
    for (int i = 0; i < 8; ++i) {
        if (h->sym_peer[i] && i != h->rank) cudaIpcCloseMemHandle(h->sym_peer[i]);
        h->sym_peer[i] = nullptr;
        if (h->xchg_peer[i] && i != h->rank) cudaIpcCloseMemHandle(h->xchg_peer[i]);
        h->xchg_peer[i] = nullptr;
    }
    if (h->xchg_local) cudaFree(h->xchg_local);
    h->xchg_local = nullptr;
    if (h->sym_local) cudaFree(h->sym_local);
    h->sym_local = nullptr;
    h->sym_bytes = 0;
    if (h->barrier_word) cudaFree(h->barrier_word);
    h->barrier_word = nullptr;
    (void)cudaGetLastError();
}

extern "C" int o64_comm_destroy(o64_handle_t h) {
    if (!h) return O64_ERR_RANK;
    free_symmetric(h);
    if (h->comm) {
        if (nccl().ok) nccl().CommDestroy(h->comm);
        h->comm = nullptr;
    }
    h->rank = 0;
    h->nranks = 1;
    return O64_OK;
}

extern "C" int o64_destroy(o64_handle_t h) {
    if (!h) return O64_ERR_RANK;
    DeviceGuard g(h->device);
    o64_comm_destroy(h);
    for (int i = 0; i < kSlots; ++i)
        if (h->stage[i]) cudaFree(h->stage[i]);
    if (h->ws) cudaFree(h->ws);
    if (h->copy_in) cudaStreamDestroy(h->copy_in);
    if (h->copy_out) cudaStreamDestroy(h->copy_out);
    if (h->ev_entry) cudaEventDestroy(h->ev_entry);
    if (h->ev_done) cudaEventDestroy(h->ev_done);
    for (int i = 0; i < kMaxBlocks; ++i) {
        if (h->ev_in[i]) cudaEventDestroy(h->ev_in[i]);
        if (h->ev_mm[i]) cudaEventDestroy(h->ev_mm[i]);
    }
    if (h->tail_slots) cudaFree(h->tail_slots);
    if (h->tail_flags) cudaFree(h->tail_flags);
    if (h->status_word) cudaFree(h->status_word);
    delete h;
    return O64_OK;
}

extern "C" int o64_last_status(o64_handle_t h, void *stream, int *detail) {
    if (!h) return O64_ERR_RANK;
    DeviceGuard g(h->device);
    cudaStream_t s = (cudaStream_t)stream;
    int word = 0;
    CUDA_TRY(cudaMemcpyAsync(&word, h->status_word, sizeof(int), cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaStreamSynchronize(s));
    if (detail) *detail = word;
    if (word != 0) {
        CUDA_TRY(cudaMemsetAsync(h->status_word, 0, sizeof(int), s));
        // a kernel that gave up may have left words of the last-wave K split set
        if (h->tail_flags) CUDA_TRY(cudaMemsetAsync(h->tail_flags, 0, kTailFlagWords * sizeof(unsigned), s));
        return O64_ERR_TIMEOUT;
    }
    return O64_OK;
}

extern "C" int o64_set_wait_budget_us(o64_handle_t h, int64_t microseconds) {
    if (!h || microseconds < 0) return O64_ERR_RANK;
    h->wait_ns = (unsigned long long)microseconds * 1000ull;  // 0: back to the default
    return O64_OK;
}

extern "C" int o64_plan_set(o64_handle_t h, int kind, const o64_plan_t *plan) {
    if (!h || kind < 0 || kind > 3) return O64_ERR_RANK;
    if (!plan) {
        h->has_pin[kind] = false;
        return O64_OK;
    }
    if (kind == O64_KIND_F32) {
        // the CUDA-core kernel: 32 x 32, 32 x 64 or 64 x 64 tiles (tile_k and the rest are fixed)
        const bool m_ok = plan->tile_m == 0 || plan->tile_m == 32 || plan->tile_m == 64;
        const bool n_ok = plan->tile_n == 0 || plan->tile_n == 32 || plan->tile_n == 64;
        if (!m_ok || !n_ok || (plan->tile_m == 64 && plan->tile_n == 32)) return O64_ERR_RANK;
        if (plan->tile_k && plan->tile_k != 16) return O64_ERR_RANK;
        h->pins[kind] = *plan;
        h->has_pin[kind] = true;
        return O64_OK;
    }
    const bool few_rows = plan->split_k < 0;  // the kernel for M <= 128: tile_m = rows of A per stage
    if (few_rows && plan->tile_m && plan->tile_m != 16 && plan->tile_m != 32 && plan->tile_m != 64 && plan->tile_m != 128)
        return O64_ERR_RANK;
    if (few_rows && plan->cta_group == 2) return O64_ERR_RANK;  // tile_n: 256 or 128, checked below
    if (!few_rows && plan->tile_m && plan->tile_m != 128 && plan->tile_m != 256 && plan->tile_m != 512) return O64_ERR_RANK;
    if (plan->tile_n && plan->tile_n != 128 && plan->tile_n != 256) return O64_ERR_RANK;
    if (plan->cta_group && plan->cta_group != 1 && plan->cta_group != 2) return O64_ERR_RANK;
    if (!few_rows && plan->tile_m && plan->cta_group && (plan->cta_group == 1) != (plan->tile_m == 128)) return O64_ERR_RANK;
    if (plan->tile_m == 512 && plan->tile_n && plan->tile_n != 256) return O64_ERR_RANK;
    if (plan->group_m < 0 || plan->num_ctas < 0) return O64_ERR_RANK;
    if (few_rows && plan->split_k != -1 && plan->split_k != -2 && plan->split_k != -4 && plan->split_k != -8) return O64_ERR_RANK;
    h->pins[kind] = *plan;
    h->has_pin[kind] = true;
    return O64_OK;
}

static void choose(o64_handle_t h, int kind, int epi, int64_t M, int64_t N, int64_t K, o64_plan_t *out) {
    const o64_plan_t *pin = h->has_pin[kind] ? &h->pins[kind] : nullptr;
    if (!pin && !h->tuned.empty()) {
        auto it = h->tuned.find({kind, epi == EPI_SWIGLU ? 1 : 0, M, N, K, h->nranks});
        if (it != h->tuned.end()) pin = &it->second;
    }
    plan_choose(kind, epi, M, N, K, h->num_sms, pin, out);
}

extern "C" int o64_plan_get(o64_handle_t h, int kind, int64_t M, int64_t N, int64_t K, o64_plan_t *plan) {
    if (!h || !plan || kind < 0 || kind > 3) return O64_ERR_RANK;
    if (M <= 0 || N <= 0 || K <= 0) return O64_ERR_RANK;
    if (kind == O64_KIND_F32) {
        // the plan of the dense fused linear (operands aligned to 16 bytes; other calls use a
        // scalar-access kernel with 64 x 64 or 32 x 32 tiles)
        memset(plan, 0, sizeof(*plan));
        plan->kind = kind;
        simt_dense_tile(M, N, h->num_sms, &plan->tile_m, &plan->tile_n);
        if (h->has_pin[kind]) simt_apply_pin(h->pins[kind].tile_m, h->pins[kind].tile_n, &plan->tile_m, &plan->tile_n);
        plan->tile_k = 16;
        plan->stages = 2;
        plan->cta_group = 1;
        plan->mma_m = plan->mma_n = 4;
        plan->mma_k = 1;
        plan->split_k = 1;
        plan->num_ctas = (int)(((M + plan->tile_m - 1) / plan->tile_m) * ((N + plan->tile_n - 1) / plan->tile_n));
        return O64_OK;
    }
    choose(h, kind, EPI_BF16, M, N, K, plan);
    return O64_OK;
}

extern "C" int o64_plan_model(int kind, int swiglu, int64_t M, int64_t N, int64_t K, int num_sms,
                              const o64_plan_t *pin, o64_plan_t *plan) {
    if (!plan || kind < O64_KIND_BF16 || kind > O64_KIND_S8) return O64_ERR_RANK;
    if (M <= 0 || N <= 0 || K <= 0 || num_sms <= 0) return O64_ERR_RANK;
    if (swiglu && kind != O64_KIND_BF16) return O64_ERR_DTYPE;
    plan_choose(kind, swiglu ? EPI_SWIGLU : EPI_BF16, M, N, K, num_sms, pin, plan);
    return O64_OK;
}

// ---- host-operand staging ---------------------------------------------------------------------
enum { PTR_DEVICE = 0, PTR_HOST = 1, PTR_OTHER_DEVICE = 2 };

// Where an operand lives, seen from device `dev`: host memory (to be staged), memory the device can
// use in place (its own or managed), or memory of ANOTHER GPU.  The last kind is refused by every
// entry point: kernels, tensor maps and copies are made for the handle's device, and a pointer of
// another GPU would end in an illegal-address fault (no peer access) or in silent peer traffic.
static int ptr_class(const void *p, int dev) {
    if (!p) return PTR_DEVICE;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return PTR_HOST;
    }
    if (a.type == cudaMemoryTypeHost || a.type == cudaMemoryTypeUnregistered) return PTR_HOST;
    if (a.type == cudaMemoryTypeDevice && a.device != dev) return PTR_OTHER_DEVICE;
    return PTR_DEVICE;
}

static bool is_host_ptr(const void *p) {
    if (!p) return false;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return true;
    }
    return a.type == cudaMemoryTypeHost || a.type == cudaMemoryTypeUnregistered;
}

// True when every pointer is host memory, memory of the handle's device, or NULL.
static bool on_handles_device(o64_handle_t h, std::initializer_list<const void *> ptrs) {
    for (const void *p : ptrs)
        if (ptr_class(p, h->device) == PTR_OTHER_DEVICE) return false;
    return true;
}

static int reserve(void **buf, size_t *cap, size_t bytes) {
    if (bytes <= *cap) return O64_OK;
    if (*buf) cudaFree(*buf);
    *buf = nullptr;
    *cap = 0;
    if (cudaMalloc(buf, bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        return O64_ERR_NOMEM;
    }
    *cap = bytes;
    return O64_OK;
}

// Bytes spanned by a row-major [rows, cols] matrix with leading dimension ld.
static size_t span_bytes(int64_t rows, int64_t cols, int64_t ld, int elem) {
    if (rows <= 0 || cols <= 0) return 0;
    return (size_t)((rows - 1) * ld + cols) * (size_t)elem;
}

// Stages a host operand into slot `slot`; returns the device pointer to use (the original
// pointer when it already is device memory).
static int stage_in(o64_handle_t h, int slot, const void *src, size_t bytes, cudaStream_t s,
                    const void **dev) {
    *dev = src;
    const int where = ptr_class(src, h->device);
    if (where == PTR_OTHER_DEVICE) return O64_ERR_RANK;
    if (!src || where != PTR_HOST) return O64_OK;
    int rc = reserve(&h->stage[slot], &h->stage_cap[slot], bytes ? bytes : 16);
    if (rc) return rc;
    if (bytes) CUDA_TRY(cudaMemcpyAsync(h->stage[slot], src, bytes, cudaMemcpyHostToDevice, s));
    *dev = h->stage[slot];
    return O64_OK;
}

struct StagedOut {
    void *host = nullptr;
    void *dev = nullptr;
    size_t bytes = 0;
};

static int stage_out_begin(o64_handle_t h, int slot, void *dst, size_t bytes, bool preload,
                           cudaStream_t s, StagedOut *o) {
    o->host = nullptr;
    o->dev = dst;
    o->bytes = bytes;
    const int where = ptr_class(dst, h->device);
    if (where == PTR_OTHER_DEVICE) return O64_ERR_RANK;
    if (!dst || where != PTR_HOST) return O64_OK;
    int rc = reserve(&h->stage[slot], &h->stage_cap[slot], bytes ? bytes : 16);
    if (rc) return rc;
    o->host = dst;
    o->dev = h->stage[slot];
    // a padded result (ld > cols) or beta != 0 needs the caller's bytes underneath
    if (preload && bytes) CUDA_TRY(cudaMemcpyAsync(o->dev, dst, bytes, cudaMemcpyHostToDevice, s));
    return O64_OK;
}

// Copies a staged result back and waits for it: with a host result the call is synchronous.
static int stage_out_end(const StagedOut &o, cudaStream_t s) {
    if (!o.host) return O64_OK;
    if (o.bytes) CUDA_TRY(cudaMemcpyAsync(o.host, o.dev, o.bytes, cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaStreamSynchronize(s));
    return O64_OK;
}

// TMA needs a 16-byte aligned base and row pitch.  An operand that lacks either is copied once
// into handle-owned scratch with the pitch rounded up (a strided device-to-device copy on the
// caller's stream); aligned operands are used in place.
static bool tma_aligned(const void *ptr, int64_t ld, int elem) {
    return ((reinterpret_cast<uintptr_t>(ptr) & 15u) == 0) && ((ld * elem) % 16 == 0);
}

static int repack_if_unaligned(o64_handle_t h, int slot, const void **ptr, int64_t *ld, int64_t rows,
                               int64_t cols, int elem, cudaStream_t s, bool force = false) {
    if (!*ptr) return O64_OK;
    if (!force && tma_aligned(*ptr, *ld, elem)) return O64_OK;
    const int64_t new_ld = ((cols * elem + 15) / 16) * 16 / elem;
    int rc = reserve(&h->stage[slot], &h->stage_cap[slot], (size_t)rows * new_ld * elem);
    if (rc) return rc;
    CUDA_TRY(cudaMemcpy2DAsync(h->stage[slot], (size_t)new_ld * elem, *ptr, (size_t)*ld * elem,
                               (size_t)cols * elem, (size_t)rows, cudaMemcpyDeviceToDevice, s));
    *ptr = h->stage[slot];
    *ld = new_ld;
    return O64_OK;
}

// ---- native layer ---------------------------------------------------------------------------
extern "C" int o64_linear_f32(o64_handle_t h, int64_t M, int64_t N, int64_t K, const float *A,
                              int64_t lda, const float *B, int64_t ldb, const float *bias, float *Y,
                              int64_t ldy, int act, void *stream) {
    if (!h || M < 0 || N < 0 || K < 0) return O64_ERR_RANK;
    if (act < O64_ACT_NONE || act > O64_ACT_SILU) return O64_ERR_RANK;
    if (M == 0 || N == 0) return O64_OK;
    if (!Y || (K > 0 && (!A || !B))) return O64_ERR_RANK;  // K == 0: the empty sum, Y = act(bias)
    if (lda < K || ldb < N || ldy < N) return O64_ERR_CONFORM;
    DeviceGuard g(h->device);
    cudaStream_t s = (cudaStream_t)stream;
    const void *dA, *dB, *dbias;
    StagedOut out;
    int rc;
    if ((rc = stage_in(h, 0, A, span_bytes(M, K, lda, 4), s, &dA))) return rc;
    if ((rc = stage_in(h, 1, B, span_bytes(K, N, ldb, 4), s, &dB))) return rc;
    if ((rc = stage_in(h, 2, bias, (size_t)N * 4, s, &dbias))) return rc;
    if ((rc = stage_out_begin(h, 3, Y, span_bytes(M, N, ldy, 4), ldy != N, s, &out))) return rc;
    SimtGemmCall c;
    c.M = M; c.N = N; c.K = K;
    c.alpha = 1.0f; c.beta = 0.0f;
    c.A = (const float *)dA; c.a1 = lda; c.a2 = 1;
    c.B = (const float *)dB; c.b1 = ldb; c.b2 = 1;
    c.C = (float *)out.dev; c.c1 = ldy; c.c2 = 1;
    c.bias = (const float *)dbias;
    c.act = act;
    c.skip_zero_b = false;
    c.num_sms = h->num_sms;
    c.stream = s;
    if (h->has_pin[O64_KIND_F32]) {
        c.pin_tile_m = h->pins[O64_KIND_F32].tile_m;
        c.pin_tile_n = h->pins[O64_KIND_F32].tile_n;
    }
    if ((rc = simt_gemm_f32(c))) return rc;
    return stage_out_end(out, s);
}

static int pipeline_resources(o64_handle_t h) {
    if (h->copy_in) return O64_OK;
    cudaStream_t a = nullptr, b = nullptr;
    if (cudaStreamCreateWithFlags(&a, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&b, cudaStreamNonBlocking) != cudaSuccess) {
        (void)cudaGetLastError();
        if (a) cudaStreamDestroy(a);
        return O64_ERR_CUDA;
    }
    bool ok = cudaEventCreateWithFlags(&h->ev_entry, cudaEventDisableTiming) == cudaSuccess &&
              cudaEventCreateWithFlags(&h->ev_done, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; ok && i < kMaxBlocks; ++i)
        ok = cudaEventCreateWithFlags(&h->ev_in[i], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&h->ev_mm[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
        (void)cudaGetLastError();
        cudaStreamDestroy(a);
        cudaStreamDestroy(b);
        return O64_ERR_CUDA;  // events created so far are released with the handle
    }
    h->copy_in = a;
    h->copy_out = b;
    return O64_OK;
}

// Gives a call of a CTA-pair kernel the handle's slot and flag memory for the K split of its last
// wave (allocated once, 40 MB; without it the kernels simply run whole tiles).
static void attach_tail(o64_handle_t h, UmmaCall *c) {
    if (c->plan.cta_group != 2 || c->plan.split_k < 0) return;
    if (!h->tail_slots) {
        void *slots = nullptr, *flags = nullptr;
        if (cudaMalloc(&slots, (size_t)kTailMaxPairs * kTailSlotBytesMax) != cudaSuccess ||
            cudaMalloc(&flags, kTailFlagWords * sizeof(unsigned)) != cudaSuccess ||
            cudaMemset(flags, 0, kTailFlagWords * sizeof(unsigned)) != cudaSuccess) {
            (void)cudaGetLastError();
            if (slots) cudaFree(slots);
            if (flags) cudaFree(flags);
            return;
        }
        h->tail_slots = slots;
        h->tail_flags = static_cast<unsigned *>(flags);
    }
    c->tail_slots = h->tail_slots;
    c->tail_flags = h->tail_flags;
    c->tail_bytes = (size_t)kTailMaxPairs * kTailSlotBytesMax;
}

static int umma_entry(o64_handle_t h, int kind, bool b_kn, int epi, int64_t M, int64_t N, int64_t K,
                      const void *A, int64_t lda, const void *B, const void *B2, int64_t ldb, void *C,
                      int64_t ldc, const float *bias, const float *sa, const float *sb, int act,
                      void *stream, int test_withhold = -1) {
    if (!h || M < 0 || N < 0 || K < 0) return O64_ERR_RANK;
    if (act < O64_ACT_NONE || act > O64_ACT_SILU) return O64_ERR_RANK;
    if (M == 0 || N == 0) return O64_OK;
    if (!C || (K > 0 && (!A || !B))) return O64_ERR_RANK;
    const int elem = (kind == O64_KIND_BF16) ? 2 : 1;
    const int out_elem = epi_out_bytes(epi);
    const int64_t b_rows = b_kn ? K : N, b_cols = b_kn ? N : K;
    if (lda < K || ldb < b_cols || ldc < N) return O64_ERR_CONFORM;
    DeviceGuard g(h->device);  // (operands of another GPU are refused where each is staged, below)
    cudaStream_t s = (cudaStream_t)stream;
    if (K == 0) {
        // the empty sum, as the runtime's kernels treat it (osprey/libfi/matrix/xgemmx.h:185-196 sets
        // C to zero): every accumulator is zero and the fused tail runs on that
        StagedOut o0;
        const void *dbias0;
        int rc0;
        if ((rc0 = stage_in(h, 3, bias, (size_t)N * 4, s, &dbias0))) return rc0;
        if ((rc0 = stage_out_begin(h, 5, C, span_bytes(M, N, ldc, out_elem), ldc != N, s, &o0))) return rc0;
        if (epi == EPI_S32 || epi == EPI_SWIGLU || !dbias0) {
            // act(0) = 0 for every activation of the vocabulary; silu(0) * 0 = 0; zero is all bits clear
            // in every result type
            CUDA_TRY(cudaMemset2DAsync(o0.dev, (size_t)ldc * out_elem, 0, (size_t)N * out_elem, (size_t)M, s));
        } else {
            const int out_kind = epi == EPI_ISCALED_S8 ? 1 : (epi == EPI_SCALED_E4M3 ? 2 : 0);
            if ((rc0 = finalize_partial_bf16(nullptr, M, N, nullptr, nullptr, (const float *)dbias0, act, o0.dev, ldc, s,
                                             out_kind)))
                return rc0;
        }
        return stage_out_end(o0, s);
    }
    const void *dA, *dB, *dB2, *dbias, *dsa, *dsb;
    StagedOut out;
    int rc;
    // Host A and host C of a tall product: rows travel in blocks.  Block i's rows of A are copied on
    // one side stream, multiplied on the caller's stream, and its rows of C copied back on another,
    // so that host->device, kernels and device->host overlap (the link carries both directions at
    // once); the weight is staged whole, first.  Everything else goes the plain way.
    const bool piped = test_withhold < 0 && M >= 2 * kBlockRows && ldc == N && (lda * elem) % 16 == 0 && is_host_ptr(A) && is_host_ptr(C) &&
                       pipeline_resources(h) == O64_OK;
    if (piped) {
        if ((rc = reserve(&h->stage[0], &h->stage_cap[0], span_bytes(M, K, lda, elem)))) return rc;
        dA = h->stage[0];
    } else if ((rc = stage_in(h, 0, A, span_bytes(M, K, lda, elem), s, &dA))) {
        return rc;
    }
    if ((rc = stage_in(h, 1, B, span_bytes(b_rows, b_cols, ldb, elem), s, &dB))) return rc;
    if ((rc = stage_in(h, 2, B2, span_bytes(b_rows, b_cols, ldb, elem), s, &dB2))) return rc;
    if ((rc = stage_in(h, 3, bias, (size_t)N * 4, s, &dbias))) return rc;
    // the two scale vectors share one slot: sa first, sb after it
    dsa = sa;
    dsb = sb;
    const int sa_where = ptr_class(sa, h->device), sb_where = ptr_class(sb, h->device);
    if (sa_where == PTR_OTHER_DEVICE || sb_where == PTR_OTHER_DEVICE) return O64_ERR_RANK;
    if ((sa && sa_where == PTR_HOST) || (sb && sb_where == PTR_HOST)) {
        if ((rc = reserve(&h->stage[4], &h->stage_cap[4], (size_t)(M + N) * 4))) return rc;
        float *base = (float *)h->stage[4];
        if (sa) {
            CUDA_TRY(cudaMemcpyAsync(base, sa, (size_t)M * 4, cudaMemcpyDefault, s));
            dsa = base;
        }
        if (sb) {
            CUDA_TRY(cudaMemcpyAsync(base + M, sb, (size_t)N * 4, cudaMemcpyDefault, s));
            dsb = base + M;
        }
    }
    if ((rc = stage_out_begin(h, 5, C, span_bytes(M, N, ldc, out_elem), ldc != N, s, &out))) return rc;
    int64_t lda_eff = lda, ldb_eff = ldb, ldb2_eff = ldb;
    if (!piped && (rc = repack_if_unaligned(h, 6, &dA, &lda_eff, M, K, elem, s))) return rc;
    // gate and up weights share one pitch: if either needs the copy, both get it
    const bool both = dB2 && (!tma_aligned(dB, ldb, elem) || !tma_aligned(dB2, ldb, elem));
    if ((rc = repack_if_unaligned(h, 7, &dB, &ldb_eff, b_rows, b_cols, elem, s, both))) return rc;
    if ((rc = repack_if_unaligned(h, 8, &dB2, &ldb2_eff, b_rows, b_cols, elem, s, both))) return rc;

    UmmaCall c;
    c.kind = kind;
    c.b_kn = b_kn;
    c.epi = epi;
    c.M = M; c.N = N; c.K = K;
    c.A = dA; c.lda = lda_eff;
    c.B = dB; c.B2 = dB2; c.ldb = ldb_eff;
    c.C = out.dev; c.ldc = ldc;
    c.bias = (const float *)dbias;
    c.scale_a = (const float *)dsa;
    c.scale_b = (const float *)dsb;
    c.act = act;
    c.status_word = h->status_word;
    c.stream = s;
    c.wait_ns = h->wait_ns;
    c.test_withhold = test_withhold;
    if (piped) {
        int64_t rows = (M + kMaxBlocks - 1) / kMaxBlocks;
        if (rows < kBlockRows) rows = kBlockRows;
        rows = (rows + 511) / 512 * 512;  // whole tiles of every kernel
        const int blocks = (int)((M + rows - 1) / rows);
        // the staging buffers may still be read by an earlier call's kernels on the caller's stream
        CUDA_TRY(cudaEventRecord(h->ev_entry, s));
        CUDA_TRY(cudaStreamWaitEvent(h->copy_in, h->ev_entry, 0));
        CUDA_TRY(cudaStreamWaitEvent(h->copy_out, h->ev_entry, 0));
        o64_plan_t pin;
        memset(&pin, 0, sizeof(pin));
        if (h->has_pin[kind]) pin = h->pins[kind];
        if (pin.split_k == 0) pin.split_k = 1;  // no plan that needs zeroed scratch per block
        for (int i = 0; i < blocks; ++i) {
            const int64_t r0 = (int64_t)i * rows;
            const int64_t nr = (M - r0) < rows ? (M - r0) : rows;
            const uint8_t *a_src = static_cast<const uint8_t *>(A) + (size_t)r0 * lda * elem;
            uint8_t *a_dst = static_cast<uint8_t *>(h->stage[0]) + (size_t)r0 * lda * elem;
            CUDA_TRY(cudaMemcpyAsync(a_dst, a_src, span_bytes(nr, K, lda, elem), cudaMemcpyHostToDevice, h->copy_in));
            CUDA_TRY(cudaEventRecord(h->ev_in[i], h->copy_in));
            CUDA_TRY(cudaStreamWaitEvent(s, h->ev_in[i], 0));
            UmmaCall b = c;
            b.M = nr;
            b.A = a_dst;
            b.C = static_cast<uint8_t *>(out.dev) + (size_t)r0 * ldc * out_elem;
            if (b.scale_a) b.scale_a += r0;
            plan_choose(kind, epi, nr, N, K, h->num_sms, &pin, &b.plan);
            if (b.plan.split_k > 1) b.plan.split_k = 1;
            attach_tail(h, &b);
            if ((rc = umma_launch(b))) {
                // leave nothing queued behind the caller's back: the side streams' copies and the
                // waits recorded so far drain before the error is returned
                cudaStreamSynchronize(h->copy_in);
                cudaStreamSynchronize(h->copy_out);
                cudaStreamSynchronize(s);
                (void)cudaGetLastError();
                return rc;
            }
            CUDA_TRY(cudaEventRecord(h->ev_mm[i], s));
            CUDA_TRY(cudaStreamWaitEvent(h->copy_out, h->ev_mm[i], 0));
            CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t *>(out.host) + (size_t)r0 * ldc * out_elem, b.C,
                                     (size_t)nr * ldc * out_elem, cudaMemcpyDeviceToHost, h->copy_out));
        }
        CUDA_TRY(cudaEventRecord(h->ev_done, h->copy_out));
        CUDA_TRY(cudaStreamWaitEvent(s, h->ev_done, 0));
        CUDA_TRY(cudaStreamSynchronize(s));  // with a host result the call is synchronous
        return O64_OK;
    }
    choose(h, kind, epi, M, N, K, &c.plan);
    // split-K (few tiles, long K): partial sums meet in scratch memory; a second small kernel
    // applies the epilogue for 16-bit results, int32 results are summed in place
    const bool split = c.plan.split_k > 1 && c.plan.cta_group == 1 &&
                       (epi == EPI_BF16 || epi == EPI_SCALED_BF16 || epi == EPI_S32);
    if (split) {
        if (epi == EPI_S32) {
            CUDA_TRY(cudaMemset2DAsync(out.dev, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)M, s));
        } else {
            if ((rc = reserve(&h->ws, &h->ws_cap, (size_t)M * N * 4))) return rc;
            CUDA_TRY(cudaMemsetAsync(h->ws, 0, (size_t)M * N * 4, s));
            c.partial = h->ws;
        }
        c.split_ready = true;
    } else if (c.plan.split_k > 1) {
        c.plan.split_k = 1;
    }
    attach_tail(h, &c);
    if ((rc = umma_launch(c))) return rc;
    if (split && epi != EPI_S32) {
        if ((rc = finalize_partial_bf16((const float *)h->ws, M, N, c.scale_a, c.scale_b, c.bias, act, out.dev,
                                        ldc, s)))
            return rc;
    }
    return stage_out_end(out, s);
}

extern "C" int o64_gemm_bf16(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *A, int64_t lda,
                             const void *B, int64_t ldb, int transB, void *C, int64_t ldc,
                             const o64_epilogue_t *epi, void *stream) {
    return umma_entry(h, O64_KIND_BF16, transB == 0, EPI_BF16, M, N, K, A, lda, B, nullptr, ldb, C, ldc,
                      epi ? epi->bias : nullptr, nullptr, nullptr, epi ? epi->act : O64_ACT_NONE, stream);
}

extern "C" int o64_gemm_bf16_swiglu(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *X,
                                    int64_t ldx, const void *Wg, const void *Wu, int64_t ldw, void *H,
                                    int64_t ldh, void *stream) {
    if (!Wu) return O64_ERR_RANK;
    return umma_entry(h, O64_KIND_BF16, true, EPI_SWIGLU, M, N, K, X, ldx, Wg, Wu, ldw, H, ldh, nullptr,
                      nullptr, nullptr, O64_ACT_NONE, stream);
}

extern "C" int o64_gemm_fp8_scaled(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *A8,
                                   int64_t lda, const void *B8, int64_t ldb, const float *scaleA,
                                   const float *scaleB, const float *bias, void *C, int64_t ldc,
                                   void *stream) {
    return umma_entry(h, O64_KIND_FP8, false, EPI_SCALED_BF16, M, N, K, A8, lda, B8, nullptr, ldb, C, ldc,
                      bias, scaleA, scaleB, O64_ACT_NONE, stream);
}

// The scaled products with a choice of result type and an activation after the dequantisation.
extern "C" int o64_gemm_fp8_scaled_ex(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *A8, int64_t lda,
                                      const void *B8, int64_t ldb, const float *scaleA, const float *scaleB,
                                      const float *bias, int act, void *C, int64_t ldc, int out_kind, void *stream) {
    if (out_kind != O64_OUT_BF16 && out_kind != O64_OUT_E4M3) return O64_ERR_DTYPE;
    return umma_entry(h, O64_KIND_FP8, false, out_kind == O64_OUT_E4M3 ? EPI_SCALED_E4M3 : EPI_SCALED_BF16, M, N, K, A8,
                      lda, B8, nullptr, ldb, C, ldc, bias, scaleA, scaleB, act, stream);
}

// The e4m3 product with the weight stored [K,N] (N contiguous).  A weight whose base and pitch are
// multiples of 16 bytes is read in place (below); any other is transposed into scratch the handle owns
// (one extra pass over N*K bytes, on the caller's stream) and the [N,K] kernels run on that.
extern "C" int o64_gemm_fp8_scaled_kn(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *A8, int64_t lda,
                                      const void *B8_kn, int64_t ldb, const float *scaleA, const float *scaleB,
                                      const float *bias, int act, void *C, int64_t ldc, int out_kind, void *stream) {
    if (!h || M < 0 || N < 0 || K < 0) return O64_ERR_RANK;
    if (out_kind != O64_OUT_BF16 && out_kind != O64_OUT_E4M3) return O64_ERR_DTYPE;
    if (K == 0 || N == 0 || M == 0)
        return o64_gemm_fp8_scaled_ex(h, M, N, K, A8, lda, B8_kn, K, scaleA, scaleB, bias, act, C, ldc, out_kind, stream);
    if (!B8_kn) return O64_ERR_RANK;
    if (ldb < N) return O64_ERR_CONFORM;
    if (is_host_ptr(B8_kn)) return O64_ERR_RANK;  // a host weight: transpose it on the host, or copy it over first
    if (!on_handles_device(h, {B8_kn})) return O64_ERR_RANK;
    DeviceGuard g(h->device);
    cudaStream_t s = (cudaStream_t)stream;
    // A weight TMA can address (16-byte aligned base and pitch) is read as it lies: the CTA-pair kernel
    // loads [K,N] boxes and multiplies with an N-major shared-memory descriptor on 256 x 256 tiles.
    static const bool native_off = [] { const char *e = getenv("O64_FP8_KN_NATIVE"); return e && atoi(e) == 0; }();
    if (!native_off && tma_aligned(B8_kn, ldb, 1) && N >= 16) {
        const bool had = h->has_pin[O64_KIND_FP8];
        const o64_plan_t saved = h->pins[O64_KIND_FP8];
        o64_plan_t pin;
        memset(&pin, 0, sizeof(pin));
        pin.kind = O64_KIND_FP8;
        pin.cta_group = 2;
        pin.tile_m = 256;
        pin.tile_n = 256;
        pin.split_k = 1;
        h->pins[O64_KIND_FP8] = pin;
        h->has_pin[O64_KIND_FP8] = true;
        const int rc_native = umma_entry(h, O64_KIND_FP8, true, out_kind == O64_OUT_E4M3 ? EPI_SCALED_E4M3 : EPI_SCALED_BF16, M, N,
                                         K, A8, lda, B8_kn, nullptr, ldb, C, ldc, bias, scaleA, scaleB, act, stream);
        h->pins[O64_KIND_FP8] = saved;
        h->has_pin[O64_KIND_FP8] = had;
        return rc_native;
    }
    const int64_t ld_t = (K + 15) / 16 * 16;
    int rc = reserve(&h->stage[9], &h->stage_cap[9], (size_t)N * ld_t);
    if (rc) return rc;
    if ((rc = transpose_bytes(B8_kn, ldb, h->stage[9], ld_t, K, N, s))) return rc;
    return o64_gemm_fp8_scaled_ex(h, M, N, K, A8, lda, h->stage[9], ld_t, scaleA, scaleB, bias, act, C, ldc, out_kind, stream);
}

extern "C" int o64_gemm_s8_scaled(o64_handle_t h, int64_t M, int64_t N, int64_t K, const int8_t *A, int64_t lda,
                                  const int8_t *B, int64_t ldb, const float *scaleA, const float *scaleB,
                                  const float *bias, int act, void *C, int64_t ldc, int out_kind, void *stream) {
    if (out_kind != O64_OUT_BF16 && out_kind != O64_OUT_S8) return O64_ERR_DTYPE;
    return umma_entry(h, O64_KIND_S8, false, out_kind == O64_OUT_S8 ? EPI_ISCALED_S8 : EPI_ISCALED_BF16, M, N, K, A, lda,
                      B, nullptr, ldb, C, ldc, bias, scaleA, scaleB, act, stream);
}

extern "C" int o64_gemm_s8s8_s32(o64_handle_t h, int64_t M, int64_t N, int64_t K, const int8_t *A,
                                 int64_t lda, const int8_t *B, int64_t ldb, int32_t *C, int64_t ldc,
                                 void *stream) {
    return umma_entry(h, O64_KIND_S8, false, EPI_S32, M, N, K, A, lda, B, nullptr, ldb, C, ldc, nullptr,
                      nullptr, nullptr, O64_ACT_NONE, stream);
}

// Test hook: o64_gemm_bf16 (B [N,K], no epilogue) run by the kernel the handle's pin selects, in an
// instantiation whose producer leaves out the loads of one K block.  The stage's barrier then never
// completes, the waits behind it use up the handle's wait budget, the kernel records which wait gave
// up, frees its tensor memory and returns; o64_last_status reports O64_ERR_TIMEOUT.  Nothing traps or
// spins without a limit.  C's contents are undefined afterwards.
extern "C" int o64_test_gemm_bf16_withheld(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *A, int64_t lda,
                                           const void *B, int64_t ldb, void *C, int64_t ldc, int withhold_kblock,
                                           void *stream) {
    if (withhold_kblock < 0) return O64_ERR_RANK;
    if (is_host_ptr(A) || is_host_ptr(B) || is_host_ptr(C)) return O64_ERR_RANK;
    return umma_entry(h, O64_KIND_BF16, false, EPI_BF16, M, N, K, A, lda, B, nullptr, ldb, C, ldc, nullptr, nullptr,
                      nullptr, O64_ACT_NONE, stream, withhold_kblock);
}

extern "C" int o64_test_force_tail_split(int mode) {
    force_tail_split(mode);
    return O64_OK;
}

extern "C" int o64_test_last_tail_split(int *tiles, int *pairs) {
    if (!tiles || !pairs) return O64_ERR_RANK;
    last_tail_split(tiles, pairs);
    return O64_OK;
}

extern "C" int o64_naive_gemm(o64_handle_t h, int kind, int64_t M, int64_t N, int64_t K, const void *A,
                              int64_t lda, const void *B, int64_t ldb, int transB, const float *scaleA,
                              const float *scaleB, const float *bias, int act, void *out, int64_t ldo,
                              void *stream) {
    if (!h || M < 0 || N < 0 || K < 0) return O64_ERR_RANK;
    if (kind != O64_KIND_FP8 && (scaleA || scaleB)) return O64_ERR_DTYPE;
    if (is_host_ptr(A) || is_host_ptr(B) || is_host_ptr(out)) return O64_ERR_RANK;
    if (!on_handles_device(h, {A, B, out, scaleA, scaleB, bias})) return O64_ERR_RANK;
    DeviceGuard g(h->device);
    return naive_gemm(kind, M, N, K, A, lda, B, ldb, transB, scaleA, scaleB, bias, act, out, ldo,
                      (cudaStream_t)stream);
}

// ---- multi-GPU ------------------------------------------------------------------------------
extern "C" int o64_comm_unique_id(void *id_bytes) {
    if (!id_bytes) return O64_ERR_RANK;
    if (!nccl().ok) return O64_ERR_NCCL;
    ncclUniqueId_ id;
    if (nccl().GetUniqueId(&id) != 0) return O64_ERR_NCCL;
    memcpy(id_bytes, &id, sizeof(id));
    return O64_OK;
}

extern "C" int o64_comm_init(o64_handle_t h, const void *id_bytes, int rank, int nranks) {
    if (!h || !id_bytes || nranks < 1 || rank < 0 || rank >= nranks) return O64_ERR_RANK;
    if (!nccl().ok) return O64_ERR_NCCL;
    DeviceGuard g(h->device);
    o64_comm_destroy(h);
    ncclUniqueId_ id;
    memcpy(&id, id_bytes, sizeof(id));
    if (nccl().CommInitRank(&h->comm, nranks, id, rank) != 0) {
        h->comm = nullptr;
        return O64_ERR_NCCL;
    }
    h->rank = rank;
    h->nranks = nranks;
    return O64_OK;
}

// Stream-ordered barrier over the ranks: a one-int all-reduce.
static int rank_barrier(o64_handle_t h, cudaStream_t s) {
    if (h->nranks == 1) return O64_OK;
    if (!h->comm || !h->barrier_word) return O64_ERR_NCCL;
    return nccl().AllReduce(h->barrier_word, h->barrier_word, 1, kNcclInt32, kNcclSum, h->comm, s) == 0
               ? O64_OK
               : O64_ERR_NCCL;
}

extern "C" int o64_comm_alloc_result(o64_handle_t h, size_t bytes, void **local) {
    if (!h || !local || bytes == 0) return O64_ERR_RANK;
    *local = nullptr;
    const int g = h->nranks;
    if (g > 8) return O64_ERR_RANK;
    if (g > 1 && !h->comm) return O64_ERR_NCCL;
    DeviceGuard guard(h->device);
    free_symmetric(h);
    const size_t kXchgAlloc = 2u << 20;  // a block of its own, so that its handle exports nothing else
    // whole 2 MiB pages (see the note at xchg_local)
    const size_t alloc_bytes = (bytes + (2u << 20) - 1) & ~(size_t)((2u << 20) - 1);
    if (cudaMalloc(&h->sym_local, alloc_bytes) != cudaSuccess || cudaMalloc(&h->barrier_word, sizeof(int)) != cudaSuccess ||
        cudaMalloc(&h->xchg_local, kXchgAlloc) != cudaSuccess) {
        (void)cudaGetLastError();
        free_symmetric(h);
        return O64_ERR_NOMEM;
    }
    cudaMemset(h->barrier_word, 0, sizeof(int));
    cudaMemset(h->xchg_local, 0, kXchgAlloc);  // before any peer can learn the handle
    cudaDeviceSynchronize();
    {
        const char *e = getenv("O64_PUSH_NCCL_BARRIER");
        h->push_nccl_barriers = e && atoi(e) != 0;
    }
    h->sym_bytes = bytes;
    h->sym_peer[h->rank] = h->sym_local;
    h->xchg_peer[h->rank] = h->xchg_local;
    if (g > 1) {
        // exchange the inter-process handles of both allocations with an all-gather of 128-byte records
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
        cudaIpcMemHandle_t mine[2];
        if (cudaIpcGetMemHandle(&mine[0], h->sym_local) != cudaSuccess || cudaIpcGetMemHandle(&mine[1], h->xchg_local) != cudaSuccess) {
            (void)cudaGetLastError();
            free_symmetric(h);
            return O64_ERR_CUDA;
        }
        unsigned char *dev_all = nullptr;
        if (cudaMalloc(&dev_all, 128 * (size_t)g) != cudaSuccess) {
            (void)cudaGetLastError();
            free_symmetric(h);
            return O64_ERR_NOMEM;
        }
        cudaMemcpy(dev_all + 128 * h->rank, mine, 128, cudaMemcpyHostToDevice);
        int rc = nccl().AllGather(dev_all + 128 * h->rank, dev_all, 128, kNcclInt8, h->comm, nullptr);
        cudaIpcMemHandle_t all[16];
        if (rc == 0 && cudaStreamSynchronize(nullptr) == cudaSuccess)
            cudaMemcpy(all, dev_all, 128 * (size_t)g, cudaMemcpyDeviceToHost);
        cudaFree(dev_all);
        if (rc != 0) {
            free_symmetric(h);
            return O64_ERR_NCCL;
        }
        for (int i = 0; i < g; ++i) {
            if (i == h->rank) continue;
            if (cudaIpcOpenMemHandle(&h->sym_peer[i], all[2 * i], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess ||
                cudaIpcOpenMemHandle(&h->xchg_peer[i], all[2 * i + 1], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                (void)cudaGetLastError();
                free_symmetric(h);
                return O64_ERR_CUDA;
            }
        }
    }
    *local = h->sym_local;
    return O64_OK;
}

extern "C" size_t o64_gemm_s8_sharded_workspace(int64_t M, int64_t N, int nranks, int gather) {
    (void)nranks;
    if (gather != O64_GATHER_ROWMAJOR || M <= 0 || N <= 0) return 0;
    return (size_t)M * (size_t)N * sizeof(int32_t);
}

// The fused GEMM + exchange of a column-sharded linear: ONE kernel computes this rank's column
// slab and stores every finished tile into all ranks' copies of C (its own and, over NVLink, the
// peers'), so the exchange overlaps the GEMM tile by tile.  C_full must be the buffer
// o64_comm_alloc_result handed out; bias (or NULL) is the full vector of N values.
static int push_gemm(o64_handle_t h, int kind, int epi, int64_t M, int64_t N, int64_t K, const void *A, int64_t lda,
                     const void *B_slab, int64_t ldb, void *C_full, int out_elem, const float *bias, int act,
                     cudaStream_t s) {
    const int g = h->nranks, r = h->rank;
    const int64_t ns = N / g;
    const int elem = (kind == O64_KIND_BF16) ? 2 : 1;
    if (C_full != h->sym_local || (size_t)M * N * out_elem > h->sym_bytes) return O64_ERR_RANK;
    if ((ns * out_elem) % 128) return O64_ERR_CONFORM;  // whole 128-byte store slabs only
    if (is_host_ptr(A) || is_host_ptr(B_slab) || (bias && is_host_ptr(bias))) return O64_ERR_RANK;
    int rc;
    // nobody may still be reading the previous result when the first remote store lands, and nobody
    // may read this one before every rank's stores are in: the kernel itself exchanges arrival
    // counters with its peers (UmmaParams::xchg_local), so the whole exchange is this one launch
    const bool own_barriers = g > 1 && !h->push_nccl_barriers;
    if (g > 1 && !own_barriers && (rc = rank_barrier(h, s))) return rc;
    const void *dA = A, *dB = B_slab;
    int64_t lda_eff = lda, ldb_eff = ldb;
    if ((rc = repack_if_unaligned(h, 6, &dA, &lda_eff, M, K, elem, s))) return rc;
    if ((rc = repack_if_unaligned(h, 7, &dB, &ldb_eff, ns, K, elem, s))) return rc;
    UmmaCall c;
    c.kind = kind;
    c.b_kn = false;
    c.epi = epi;
    c.M = M; c.N = ns; c.K = K;
    c.A = dA; c.lda = lda_eff;
    c.B = dB; c.B2 = nullptr; c.ldb = ldb_eff;
    c.C = static_cast<uint8_t *>(C_full) + (size_t)r * ns * out_elem; c.ldc = N;
    c.bias = bias ? bias + (int64_t)r * ns : nullptr;
    c.scale_a = nullptr; c.scale_b = nullptr;
    c.act = act;
    {
        // the fused exchange lives in the tile kernels' epilogue
        o64_plan_t pin;
        memset(&pin, 0, sizeof(pin));
        if (h->has_pin[kind]) pin = h->pins[kind];
        if (pin.split_k <= 0) pin.split_k = 1;
        plan_choose(kind, epi, M, ns, K, h->num_sms, &pin, &c.plan);
    }
    c.status_word = h->status_word;
    c.stream = s;
    c.wait_ns = h->wait_ns;
    c.n_peers = 0;
    // peers in ring order from this rank on, so that at any moment the ranks write to different targets
    for (int k = 1; k < g; ++k) {
        const int i = (r + k) % g;
        c.peer_c[c.n_peers] = static_cast<uint8_t *>(h->sym_peer[i]) + (size_t)r * ns * out_elem;
        c.xchg_peer[c.n_peers] = static_cast<unsigned *>(h->xchg_peer[i]);
        c.xchg_peer_rank[c.n_peers] = i;
        ++c.n_peers;
    }
    if (own_barriers) {
        c.xchg_local = static_cast<unsigned *>(h->xchg_local);
        c.xchg_rank = r;
    }
    attach_tail(h, &c);
    if ((rc = umma_launch(c))) return rc;
    if (g > 1 && !own_barriers) {
        // every rank's stores are complete when its kernel is; the barrier tells each rank that all
        // the others got there
        return rank_barrier(h, s);
    }
    return O64_OK;
}

extern "C" int o64_gemm_s8_sharded(o64_handle_t h, int64_t M, int64_t N, int64_t K, const int8_t *A,
                                   int64_t lda, const int8_t *B_slab, int64_t ldb, int32_t *C_full,
                                   int gather, void *workspace, void *stream) {
    if (!h || M <= 0 || N <= 0 || K <= 0 || !A || !B_slab || !C_full) return O64_ERR_RANK;
    const int g = h->nranks, r = h->rank;
    if (N % g) return O64_ERR_CONFORM;
    if (gather < O64_GATHER_NONE || gather > O64_GATHER_PUSH) return O64_ERR_RANK;
    if (gather != O64_GATHER_NONE && g > 1 && !h->comm) return O64_ERR_NCCL;
    if (is_host_ptr(A) || is_host_ptr(B_slab) || is_host_ptr(C_full)) return O64_ERR_RANK;
    if (!on_handles_device(h, {A, B_slab, C_full, workspace})) return O64_ERR_RANK;
    const int64_t ns = N / g;
    DeviceGuard guard(h->device);
    cudaStream_t s = (cudaStream_t)stream;
    int rc;

    if (gather == O64_GATHER_NONE) {
        return o64_gemm_s8s8_s32(h, M, ns, K, A, lda, B_slab, ldb, C_full + (int64_t)r * ns, N, stream);
    }
    if (gather == O64_GATHER_PUSH)
        return push_gemm(h, O64_KIND_S8, EPI_S32, M, N, K, A, lda, B_slab, ldb, C_full, 4, nullptr, O64_ACT_NONE, s);
    int32_t *slabs = C_full;  // [g][M][ns]
    if (gather == O64_GATHER_ROWMAJOR) {
        if (g == 1) return o64_gemm_s8s8_s32(h, M, N, K, A, lda, B_slab, ldb, C_full, N, stream);
        slabs = (int32_t *)workspace;
        if (!slabs) {
            if ((rc = reserve(&h->ws, &h->ws_cap, (size_t)M * N * 4))) return rc;
            slabs = (int32_t *)h->ws;
        }
    }
    int32_t *mine = slabs + (int64_t)r * M * ns;
    if ((rc = o64_gemm_s8s8_s32(h, M, ns, K, A, lda, B_slab, ldb, mine, ns, stream))) return rc;
    if (g > 1) {
        // in place: this rank's slab already sits at its offset of the receive buffer
        if (nccl().AllGather(mine, slabs, (size_t)M * ns, kNcclInt32, h->comm, s) != 0)
            return O64_ERR_NCCL;
    }
    if (gather == O64_GATHER_ROWMAJOR) return permute_slabs_s32(slabs, C_full, M, ns, g, N, s);
    return O64_OK;
}

extern "C" int o64_gemm_bf16_sharded(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *A, int64_t lda,
                                     const void *B_slab, int64_t ldb, void *C_full, int gather,
                                     const o64_epilogue_t *epi, void *stream) {
    if (!h || M <= 0 || N <= 0 || K <= 0 || !A || !B_slab || !C_full) return O64_ERR_RANK;
    const int g = h->nranks, r = h->rank;
    if (N % g) return O64_ERR_CONFORM;
    if (gather != O64_GATHER_NONE && gather != O64_GATHER_SLABS && gather != O64_GATHER_PUSH) return O64_ERR_RANK;
    if (gather != O64_GATHER_NONE && g > 1 && !h->comm) return O64_ERR_NCCL;
    if (is_host_ptr(A) || is_host_ptr(B_slab) || is_host_ptr(C_full)) return O64_ERR_RANK;
    if (!on_handles_device(h, {A, B_slab, C_full, epi ? epi->bias : nullptr})) return O64_ERR_RANK;
    const int64_t ns = N / g;
    const float *bias = epi ? epi->bias : nullptr;
    const int act = epi ? epi->act : O64_ACT_NONE;
    DeviceGuard guard(h->device);
    cudaStream_t s = (cudaStream_t)stream;
    if (gather == O64_GATHER_PUSH)
        return push_gemm(h, O64_KIND_BF16, EPI_BF16, M, N, K, A, lda, B_slab, ldb, C_full, 2, bias, act, s);
    o64_epilogue_t mine;
    mine.bias = bias ? bias + (int64_t)r * ns : nullptr;
    mine.act = act;
    uint16_t *C = static_cast<uint16_t *>(C_full);
    if (gather == O64_GATHER_NONE)  // this rank's columns of the row-major result
        return o64_gemm_bf16(h, M, ns, K, A, lda, B_slab, ldb, 1, C + (int64_t)r * ns, N, &mine, stream);
    uint16_t *slab = C + (int64_t)r * M * ns;  // slab-major [g][M][ns], gathered in place
    int rc = o64_gemm_bf16(h, M, ns, K, A, lda, B_slab, ldb, 1, slab, ns, &mine, stream);
    if (rc) return rc;
    if (g > 1 && nccl().AllGather(slab, C, (size_t)M * ns, kNcclBfloat16, h->comm, s) != 0) return O64_ERR_NCCL;
    return O64_OK;
}

// ---- measured plans -----------------------------------------------------------------------------
// The reference scores its tile candidates with a model only (LOOP_MODEL::Evaluate,
// osprey/be/lno/model.cxx:1289); here the candidates can also be run: every kernel shape that
// exists for the kind is timed on pseudo-random operands of the given extents and the fastest is
// remembered for that shape.
extern "C" int o64_plan_tune(o64_handle_t h, int kind, int swiglu, int64_t M, int64_t N, int64_t K, void *stream,
                             o64_plan_t *best) {
    if (!h || kind < O64_KIND_BF16 || kind > O64_KIND_S8 || M <= 0 || N <= 0 || K <= 0) return O64_ERR_RANK;
    if (swiglu && kind != O64_KIND_BF16) return O64_ERR_DTYPE;
    DeviceGuard g(h->device);
    cudaStream_t s = (cudaStream_t)stream;
    const int elem = (kind == O64_KIND_BF16) ? 2 : 1;
    const int out_elem = (kind == O64_KIND_S8) ? 4 : 2;
    const int epi = swiglu ? EPI_SWIGLU : (kind == O64_KIND_BF16 ? EPI_BF16 : (kind == O64_KIND_FP8 ? EPI_SCALED_BF16 : EPI_S32));
    void *A = nullptr, *B = nullptr, *B2 = nullptr, *C = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    auto release = [&]() {
        if (A) cudaFree(A);
        if (B) cudaFree(B);
        if (B2) cudaFree(B2);
        if (C) cudaFree(C);
        if (e0) cudaEventDestroy(e0);
        if (e1) cudaEventDestroy(e1);
    };
    const size_t a_bytes = (size_t)M * K * elem, b_bytes = (size_t)N * K * elem, c_bytes = (size_t)M * N * out_elem;
    bool ok = cudaMalloc(&A, a_bytes) == cudaSuccess && cudaMalloc(&B, b_bytes) == cudaSuccess &&
              cudaMalloc(&C, c_bytes) == cudaSuccess && (!swiglu || cudaMalloc(&B2, b_bytes) == cudaSuccess);
    if (!ok) {
        (void)cudaGetLastError();
        release();
        return O64_ERR_NOMEM;
    }
    // pseudo-random operands: with zeros the tensor cores toggle no bits, draw far less power and run at
    // clocks real data never sees, which ranks the candidates differently
    ok = fill_pattern(A, a_bytes, kind, s) == O64_OK && fill_pattern(B, b_bytes, kind, s) == O64_OK &&
         (!swiglu || fill_pattern(B2, b_bytes, kind, s) == O64_OK) && cudaEventCreate(&e0) == cudaSuccess &&
         cudaEventCreate(&e1) == cudaSuccess;
    if (!ok) {
        (void)cudaGetLastError();
        release();
        return O64_ERR_CUDA;
    }
    // candidates: every tile kernel, the one-CTA kernel with and without its automatic K split,
    // and for few rows the cluster kernel with every cluster size
    std::vector<o64_plan_t> cand;
    auto add = [&](int cg, int tm, int tn, int sk) {
        o64_plan_t c;
        memset(&c, 0, sizeof(c));
        c.cta_group = cg;
        c.tile_m = tm;
        c.tile_n = tn;
        c.split_k = sk;
        cand.push_back(c);
    };
    add(1, 128, 256, 1);
    add(1, 128, 128, 1);
    add(2, 256, 256, 0);
    if (!swiglu) {
        add(1, 128, 256, 0);
        add(1, 128, 128, 0);
        add(2, 256, 128, 0);
        if (M <= 512)  // few rows: one to four 128-row tiles per column block, K split over a cluster
            for (int sk = -1; sk >= -8; sk *= 2) {
                add(0, 0, 256, sk);
                if (sk >= -4) add(0, 0, 128, sk);  // 128-column tiles: clusters of at most 4
            }
    }
    add(2, 512, 256, 0);
    const bool had_pin = h->has_pin[kind];
    const o64_plan_t saved = h->pins[kind];
    double best_ms = 1e300;
    o64_plan_t best_pin;
    memset(&best_pin, 0, sizeof(best_pin));
    const int64_t ldb = swiglu ? N : K;
    for (const o64_plan_t &c : cand) {
        h->pins[kind] = c;
        h->has_pin[kind] = true;
        int rc = O64_OK;
        float ms = 0.0f;
        for (int it = 0; it < 7 && rc == O64_OK; ++it) {  // two warm-ups, five timed
            if (it == 2 && cudaEventRecord(e0, s) != cudaSuccess) rc = O64_ERR_CUDA;
            if (rc == O64_OK)
                rc = umma_entry(h, kind, swiglu != 0, epi, M, N, K, A, K, B, B2, ldb, C, N, nullptr, nullptr, nullptr,
                                O64_ACT_NONE, stream);
        }
        if (rc == O64_OK && (cudaEventRecord(e1, s) != cudaSuccess || cudaEventSynchronize(e1) != cudaSuccess ||
                             cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess))
            rc = O64_ERR_CUDA;
        (void)cudaGetLastError();
        if (rc == O64_OK && ms / 5.0 < best_ms) {
            best_ms = ms / 5.0;
            best_pin = c;
        }
    }
    h->pins[kind] = saved;
    h->has_pin[kind] = had_pin;
    release();
    if (best_ms == 1e300) return O64_ERR_CUDA;
    best_pin.predicted_ms = best_ms;
    h->tuned[{kind, swiglu ? 1 : 0, M, N, K, h->nranks}] = best_pin;
    if (const char *cache = getenv("O64_PLAN_CACHE")) (void)o64_plan_save(h, cache);
    if (best) {
        plan_choose(kind, epi, M, N, K, h->num_sms, &best_pin, best);
        best->predicted_ms = best_ms;  // measured, not modelled
    }
    return O64_OK;
}

// ---- measured plans on disk ---------------------------------------------------------------------
// The reference writes what a phase decided into the file the next phase reads (the WHIRL file,
// osprey/common/com/ir_bwrite.cxx:1505); the decisions here are the measured plans, one JSON object
// per (kind, epilogue, M, N, K, ranks) with the kernel shape and the time it was measured at, under the
// device they were measured on.
extern "C" int o64_plan_save(o64_handle_t h, const char *path) {
    if (!h || !path || !*path) return O64_ERR_RANK;
    std::string tmp = std::string(path) + ".tmp";
    FILE *f = fopen(tmp.c_str(), "w");
    if (!f) return O64_ERR_NOMEM;
    fprintf(f, "{\"version\": 1, \"device\": \"%s\", \"num_sms\": %d,\n \"plans\": [", h->device_name, h->num_sms);
    bool first = true;
    for (const auto &kv : h->tuned) {
        const auto &k = kv.first;
        const o64_plan_t &p = kv.second;
        fprintf(f,
                "%s\n  {\"kind\": %lld, \"swiglu\": %lld, \"M\": %lld, \"N\": %lld, \"K\": %lld, \"gpus\": %lld, "
                "\"cta_group\": %d, \"tile_m\": %d, \"tile_n\": %d, \"split_k\": %d, \"ms\": %.6f}",
                first ? "" : ",", (long long)k[0], (long long)k[1], (long long)k[2], (long long)k[3], (long long)k[4],
                (long long)k[5], p.cta_group, p.tile_m, p.tile_n, p.split_k, p.predicted_ms);
        first = false;
    }
    fprintf(f, "\n ]}\n");
    if (fclose(f) != 0 || rename(tmp.c_str(), path) != 0) return O64_ERR_NOMEM;
    return O64_OK;
}

// Value of "key": <number> inside one JSON object's text; `missing` when the key is absent.
static double json_number(const std::string &obj, const char *key, double missing) {
    const std::string pat = std::string("\"") + key + "\"";
    size_t at = obj.find(pat);
    if (at == std::string::npos) return missing;
    at = obj.find(':', at + pat.size());
    if (at == std::string::npos) return missing;
    return strtod(obj.c_str() + at + 1, nullptr);
}

extern "C" int o64_plan_load(o64_handle_t h, const char *path) {
    if (!h || !path || !*path) return O64_ERR_RANK;
    FILE *f = fopen(path, "r");
    if (!f) return O64_ERR_RANK;
    std::string text;
    char buf[4096];
    size_t got;
    while ((got = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, got);
    fclose(f);
    // plans measured on another kind of device (or SM count) say nothing about this one
    const size_t dev_at = text.find("\"device\"");
    if (dev_at == std::string::npos || text.find(std::string("\"") + h->device_name + "\"", dev_at) == std::string::npos)
        return O64_ERR_CONFORM;
    if ((int)json_number(text, "num_sms", -1) != h->num_sms) return O64_ERR_CONFORM;
    size_t at = text.find("\"plans\"");
    if (at == std::string::npos) return O64_ERR_DTYPE;
    int loaded = 0;
    while ((at = text.find('{', at)) != std::string::npos) {
        const size_t end = text.find('}', at);
        if (end == std::string::npos) break;
        const std::string obj = text.substr(at, end - at + 1);
        at = end + 1;
        const int kind = (int)json_number(obj, "kind", -1);
        const int64_t M = (int64_t)json_number(obj, "M", 0), N = (int64_t)json_number(obj, "N", 0),
                      K = (int64_t)json_number(obj, "K", 0);
        if (kind < O64_KIND_BF16 || kind > O64_KIND_S8 || M <= 0 || N <= 0 || K <= 0) continue;
        o64_plan_t p;
        memset(&p, 0, sizeof(p));
        p.cta_group = (int)json_number(obj, "cta_group", 0);
        p.tile_m = (int)json_number(obj, "tile_m", 0);
        p.tile_n = (int)json_number(obj, "tile_n", 0);
        p.split_k = (int)json_number(obj, "split_k", 0);
        p.predicted_ms = json_number(obj, "ms", 0.0);
        // the same checks a pin goes through: a damaged file must not select a kernel that does not exist
        o64_plan_t saved = h->pins[kind];
        const bool had = h->has_pin[kind];
        const bool ok = o64_plan_set(h, kind, &p) == O64_OK;
        h->pins[kind] = saved;
        h->has_pin[kind] = had;
        if (!ok) continue;
        h->tuned[{kind, (int64_t)json_number(obj, "swiglu", 0), M, N, K, (int64_t)json_number(obj, "gpus", 1)}] = p;
        ++loaded;
    }
    return loaded > 0 ? O64_OK : O64_ERR_DTYPE;
}

// Number of measured plans the handle holds (tuned here or loaded).
extern "C" int o64_plan_count(o64_handle_t h) { return h ? (int)h->tuned.size() : 0; }

extern "C" int o64_plan_tune_clear(o64_handle_t h) {
    if (!h) return O64_ERR_RANK;
    h->tuned.clear();
    return O64_OK;
}

// ---- compat layer (Fortran ABI) ---------------------------------------------------------------
static thread_local int g_compat_status = O64_OK;
static o64_handle_t g_compat_handle = nullptr;

extern "C" int o64_compat_last_status(void) { return g_compat_status; }

// One engine handle for all Fortran-ABI calls of the process, on the device that is current at the
// first call.  Its creation is guarded; the calls themselves share the handle's staging buffers and
// are not thread-safe (the runtime they replace has no locks either).
static std::mutex g_compat_mutex;

static o64_handle_t compat_handle() {
    std::lock_guard<std::mutex> lock(g_compat_mutex);
    if (!g_compat_handle) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        if (o64_create(&g_compat_handle, dev) != O64_OK) g_compat_handle = nullptr;
    }
    return g_compat_handle;
}

extern "C" o64_handle_t o64_compat_handle(void) { return compat_handle(); }

// Largest element offset touched (plus one) by an extent-(n1,n2) operand with strides (s1,s2).
static size_t strided_span(int64_t n1, int64_t n2, int64_t s1, int64_t s2) {
    if (n1 <= 0 || n2 <= 0) return 0;
    return (size_t)((n1 - 1) * s1 + (n2 - 1) * s2 + 1);
}

// Element type the CUDA-core kernels compute in: the integer kinds run on the unsigned type of
// the same width, whose wrap-around is the two's-complement result the Fortran kernels produce.
typedef Cx<float> c4_t;   // COMPLEX*8: (re, im) single precision
typedef Cx<double> c8_t;  // COMPLEX*16
template <typename T> struct IsCx { static constexpr bool value = false; };
template <typename R> struct IsCx<Cx<R>> { static constexpr bool value = true; };
template <typename T> struct ComputeType { typedef T type; };
template <> struct ComputeType<int8_t> { typedef uint8_t type; };
template <> struct ComputeType<int16_t> { typedef uint16_t type; };
template <> struct ComputeType<int32_t> { typedef uint32_t type; };
template <> struct ComputeType<int64_t> { typedef uint64_t type; };

// TA: element kind of A; T: element kind of B, C, alpha and beta (the same as TA, or wider for
// the mixed integer kernels such as _i1i4gemmx__).
template <typename TA, typename T>
static int xgemmx_impl(int M, int N, int K, T alpha, const TA *A, int64_t a1, int64_t a2, const T *B,
                       int64_t b1, int64_t b2, T beta, T *C, int64_t c1, int64_t c2, bool skip_zero, int conj_a = 0,
                       int conj_b = 0) {
    typedef typename ComputeType<T>::type U;
    // quick returns, in the order of osprey/libfi/matrix/xgemmx.h:172-208
    if (M < 0 || N < 0 || K < 0) return O64_ERR_RANK;
    if (M == 0 || N == 0 || (alpha == T(0) && beta == T(1))) return O64_OK;
    if (a1 < 0 || a2 < 0 || b1 < 0 || b2 < 0 || c1 < 0 || c2 < 0) return O64_ERR_RANK;
    o64_handle_t h = compat_handle();
    if (!h) return O64_ERR_CUDA;
    DeviceGuard g(h->device);
    cudaStream_t s = nullptr;
    const bool only_scale = (K == 0) || (alpha == T(0));
    const T beta_eff = (K == 0) ? T(0) : beta;
    const void *dA = A, *dB = B;
    StagedOut out;
    int rc;
    if (!only_scale) {
        if (!A || !B) return O64_ERR_RANK;
        if ((rc = stage_in(h, 0, A, strided_span(M, K, a1, a2) * sizeof(TA), s, &dA))) return rc;
        if ((rc = stage_in(h, 1, B, strided_span(K, N, b1, b2) * sizeof(T), s, &dB))) return rc;
    }
    if (!C) return O64_ERR_RANK;
    if ((rc = stage_out_begin(h, 3, C, strided_span(M, N, c1, c2) * sizeof(T), true, s, &out))) return rc;
    if constexpr (std::is_same<T, float>::value && std::is_same<TA, float>::value) {
        if (only_scale) {
            rc = simt_scale_f32(M, N, beta_eff, (float *)out.dev, c1, c2, s);
        } else {
            SimtGemmCall c;
            c.M = M; c.N = N; c.K = K;
            c.alpha = alpha; c.beta = beta;
            c.A = (const float *)dA; c.a1 = a1; c.a2 = a2;
            c.B = (const float *)dB; c.b1 = b1; c.b2 = b2;
            c.C = (float *)out.dev; c.c1 = c1; c.c2 = c2;
            c.bias = nullptr;
            c.act = O64_ACT_NONE;
            c.skip_zero_b = skip_zero;
            c.num_sms = h->num_sms;
            c.stream = s;
            if (h->has_pin[O64_KIND_F32]) {  // pins set on o64_compat_handle()
                c.pin_tile_m = h->pins[O64_KIND_F32].tile_m;
                c.pin_tile_n = h->pins[O64_KIND_F32].tile_n;
            }
            rc = simt_gemm_f32(c);
        }
    } else {
        (void)skip_zero;  // a zero factor changes nothing for integers; the REAL*8 kernel always skips
        if (only_scale)
            rc = generic_scale<U>(M, N, (U)beta_eff, (U *)out.dev, c1, c2, s);
        else
            rc = generic_gemmx<TA, U>(M, N, K, (U)alpha, (const TA *)dA, a1, a2, (const U *)dB, b1, b2, (U)beta,
                                  (U *)out.dev, c1, c2, s, conj_a, conj_b);
    }
    if (rc) return rc;
    if ((rc = stage_out_end(out, s))) return rc;
    if (!out.host) CUDA_TRY(cudaStreamSynchronize(s));  // the Fortran interface is synchronous
    return O64_OK;
}

#define O64_XGEMMX_ENTRY(NAME, TA, T)                                                                      \
    extern "C" void NAME(const int *m, const int *n, const int *k, const T *alpha, const TA *a,            \
                         const int *inc1a, const int *inc2a, const T *b, const int *inc1b,                 \
                         const int *inc2b, const T *beta, T *c, const int *inc1c, const int *inc2c) {      \
        g_compat_status = xgemmx_impl<TA, T>(*m, *n, *k, *alpha, a, *inc1a, *inc2a, b, *inc1b, *inc2b,     \
                                             *beta, c, *inc1c, *inc2c, true);                              \
    }
O64_XGEMMX_ENTRY(_s4gemmx__, float, float)
O64_XGEMMX_ENTRY(_sgemmx__, double, double)
O64_XGEMMX_ENTRY(_i1gemmx__, int8_t, int8_t)
O64_XGEMMX_ENTRY(_i1i2gemmx__, int8_t, int16_t)
O64_XGEMMX_ENTRY(_i1i4gemmx__, int8_t, int32_t)
O64_XGEMMX_ENTRY(_i1jgemmx__, int8_t, int64_t)
O64_XGEMMX_ENTRY(_i2gemmx__, int16_t, int16_t)
O64_XGEMMX_ENTRY(_i2i4gemmx__, int16_t, int32_t)
O64_XGEMMX_ENTRY(_i2jgemmx__, int16_t, int64_t)
O64_XGEMMX_ENTRY(_i4gemmx__, int32_t, int32_t)
O64_XGEMMX_ENTRY(_i4jgemmx__, int32_t, int64_t)
O64_XGEMMX_ENTRY(_jgemmx__, int64_t, int64_t)
O64_XGEMMX_ENTRY(_s4sgemmx__, float, double)
O64_XGEMMX_ENTRY(_i1s4gemmx__, int8_t, float)
O64_XGEMMX_ENTRY(_i2s4gemmx__, int16_t, float)
O64_XGEMMX_ENTRY(_i4s4gemmx__, int32_t, float)
O64_XGEMMX_ENTRY(_js4gemmx__, int64_t, float)
O64_XGEMMX_ENTRY(_i1sgemmx__, int8_t, double)
O64_XGEMMX_ENTRY(_i2sgemmx__, int16_t, double)
O64_XGEMMX_ENTRY(_i4sgemmx__, int32_t, double)
O64_XGEMMX_ENTRY(_jsgemmx__, int64_t, double)
#undef O64_XGEMMX_ENTRY

// LOGICAL kinds (osprey/libfi/matrix/lgemmx.h:  quick returns in its order: empty extents; K == 0 clears
// C; alpha false leaves C, or clears it when beta is false too).
template <typename TA, typename T>
static int lgemmx_impl(int M, int N, int K, bool alpha, const TA *A, int64_t a1, int64_t a2, const T *B, int64_t b1,
                       int64_t b2, bool beta, T *C, int64_t c1, int64_t c2) {
    if (M < 0 || N < 0 || K < 0) return O64_ERR_RANK;
    if (M == 0 || N == 0) return O64_OK;
    if (K > 0 && !alpha && beta) return O64_OK;
    if (a1 < 0 || a2 < 0 || b1 < 0 || b2 < 0 || c1 < 0 || c2 < 0) return O64_ERR_RANK;
    o64_handle_t h = compat_handle();
    if (!h) return O64_ERR_CUDA;
    DeviceGuard g(h->device);
    cudaStream_t s = nullptr;
    const bool clear_only = (K == 0) || !alpha;
    const void *dA = A, *dB = B;
    StagedOut out;
    int rc;
    if (!clear_only) {
        if (!A || !B) return O64_ERR_RANK;
        if ((rc = stage_in(h, 0, A, strided_span(M, K, a1, a2) * sizeof(TA), s, &dA))) return rc;
        if ((rc = stage_in(h, 1, B, strided_span(K, N, b1, b2) * sizeof(T), s, &dB))) return rc;
    }
    if (!C) return O64_ERR_RANK;
    if ((rc = stage_out_begin(h, 3, C, strided_span(M, N, c1, c2) * sizeof(T), true, s, &out))) return rc;
    // clearing is the product with alpha and beta false
    rc = logical_gemmx<TA, T>(M, N, clear_only ? 0 : K, clear_only ? 0 : 1, (const TA *)dA, a1, a2, (const T *)dB, b1, b2,
                              clear_only ? 0 : (beta ? 1 : 0), (T *)out.dev, c1, c2, s);
    if (rc) return rc;
    if ((rc = stage_out_end(out, s))) return rc;
    if (!out.host) CUDA_TRY(cudaStreamSynchronize(s));
    return O64_OK;
}

#define O64_LGEMMX_ENTRY(NAME, TA, T)                                                                      \
    extern "C" void NAME(const int *m, const int *n, const int *k, const T *alpha, const TA *a,            \
                         const int *inc1a, const int *inc2a, const T *b, const int *inc1b,                 \
                         const int *inc2b, const T *beta, T *c, const int *inc1c, const int *inc2c) {      \
        g_compat_status = lgemmx_impl<TA, T>(*m, *n, *k, *alpha != 0, a, *inc1a, *inc2a, b, *inc1b, *inc2b, \
                                             *beta != 0, c, *inc1c, *inc2c);                               \
    }
O64_LGEMMX_ENTRY(_l1gemmx__, int8_t, int8_t)
O64_LGEMMX_ENTRY(_l1l2gemmx__, int8_t, int16_t)
O64_LGEMMX_ENTRY(_l1l4gemmx__, int8_t, int32_t)
O64_LGEMMX_ENTRY(_l1lgemmx__, int8_t, int64_t)
O64_LGEMMX_ENTRY(_l2gemmx__, int16_t, int16_t)
O64_LGEMMX_ENTRY(_l2l4gemmx__, int16_t, int32_t)
O64_LGEMMX_ENTRY(_l2lgemmx__, int16_t, int64_t)
O64_LGEMMX_ENTRY(_l4gemmx__, int32_t, int32_t)
O64_LGEMMX_ENTRY(_l4lgemmx__, int32_t, int64_t)
O64_LGEMMX_ENTRY(_lgemmx__, int64_t, int64_t)
#undef O64_LGEMMX_ENTRY

// COMPLEX*8 / COMPLEX*16: the kernels take conjugation flags in front (osprey/libfi/matrix/c4gemmx.f:37-85,
// cgemmx.f); complex values are (re, im) pairs of floats / doubles.
#define O64_CGEMMX_ENTRY(NAME, R)                                                                          \
    extern "C" void NAME(const int *iconja, const int *iconjb, const int *m, const int *n, const int *k,   \
                         const R *alpha, const R *a, const int *inc1a, const int *inc2a, const R *b,       \
                         const int *inc1b, const int *inc2b, const R *beta, R *c, const int *inc1c,        \
                         const int *inc2c) {                                                               \
        typedef Cx<R> T;                                                                                   \
        g_compat_status = xgemmx_impl<T, T>(*m, *n, *k, T(alpha[0], alpha[1]), reinterpret_cast<const T *>(a), \
                                            *inc1a, *inc2a, reinterpret_cast<const T *>(b), *inc1b, *inc2b, \
                                            T(beta[0], beta[1]), reinterpret_cast<T *>(c), *inc1c, *inc2c, \
                                            false, *iconja != 0, *iconjb != 0);                            \
    }
O64_CGEMMX_ENTRY(_c4gemmx__, float)
O64_CGEMMX_ENTRY(_cgemmx__, double)
#undef O64_CGEMMX_ENTRY

template <typename T>
static int blas_gemm_impl(const char *transa, const char *transb, const int *m, const int *n, const int *k,
                          const T *alpha, const T *a, const int *lda, const T *b, const int *ldb,
                          const T *beta, T *c, const int *ldc) {
    auto is_n = [](char ch) { return ch == 'n' || ch == 'N'; };
    auto is_t = [](char ch) { return ch == 't' || ch == 'T' || ch == 'c' || ch == 'C'; };
    const bool na = is_n(*transa), nb = is_n(*transb);
    if ((!na && !is_t(*transa)) || (!nb && !is_t(*transb))) return O64_ERR_RANK;
    const int rows_a = na ? *m : *k, rows_b = nb ? *k : *n;
    if (*lda < (rows_a > 1 ? rows_a : 1) || *ldb < (rows_b > 1 ? rows_b : 1) || *ldc < (*m > 1 ? *m : 1))
        return O64_ERR_CONFORM;
    // column-major: op(A)(i,l) = A[i + l*lda] or A[l + i*lda]
    const int64_t a1 = na ? 1 : *lda, a2 = na ? *lda : 1;
    const int64_t b1 = nb ? 1 : *ldb, b2 = nb ? *ldb : 1;
    return xgemmx_impl<T, T>(*m, *n, *k, *alpha, a, a1, a2, b, b1, b2, *beta, c, 1, *ldc, false);
}

extern "C" void sgemm_(const char *transa, const char *transb, const int *m, const int *n, const int *k,
                       const float *alpha, const float *a, const int *lda, const float *b, const int *ldb,
                       const float *beta, float *c, const int *ldc) {
    g_compat_status = blas_gemm_impl<float>(transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}

extern "C" void dgemm_(const char *transa, const char *transb, const int *m, const int *n, const int *k,
                       const double *alpha, const double *a, const int *lda, const double *b, const int *ldb,
                       const double *beta, double *c, const int *ldc) {
    g_compat_status = blas_gemm_impl<double>(transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}

template <typename T>
static int xgemvx_impl(int M, int N, T alpha, const T *a, int64_t incca, int64_t incra, const T *x,
                       int64_t incx, T beta, T *y, int64_t incy, int conj_a = 0) {
    if (M < 0 || N < 0) return O64_ERR_RANK;
    // quick returns of osprey/libfi/matrix/s4gemvx.f (sgemvx.f is the same text in REAL*8)
    if (M == 0) return O64_OK;
    const bool zero_only = (N == 0);
    if (!zero_only && alpha == T(0) && beta == T(1)) return O64_OK;
    o64_handle_t h = compat_handle();
    if (!h) return O64_ERR_CUDA;
    DeviceGuard g(h->device);
    cudaStream_t s = nullptr;
    const void *dA = a, *dX = x;
    StagedOut out;
    int rc = O64_OK;
    const bool need_ax = !zero_only && alpha != T(0);
    if (need_ax) {
        rc = stage_in(h, 0, a, strided_span(M, N, incca, incra) * sizeof(T), s, &dA);
        if (!rc) rc = stage_in(h, 1, x, strided_span(N, 1, incx, 0) * sizeof(T), s, &dX);
    }
    if (!rc) rc = stage_out_begin(h, 3, y, strided_span(M, 1, incy, 0) * sizeof(T), true, s, &out);
    if (!rc) {
        if constexpr (std::is_same<T, float>::value) {
            if (need_ax)
                rc = simt_gemv_f32(M, N, alpha, (const float *)dA, incca, incra, (const float *)dX, incx, beta,
                                   (float *)out.dev, incy, s);
            else
                rc = simt_scale_f32(M, 1, zero_only ? 0.0f : beta, (float *)out.dev, incy, 0, s);
        } else {
            if (need_ax)
                rc = generic_gemvx<T>(M, N, alpha, (const T *)dA, incca, incra, (const T *)dX, incx, beta,
                                      (T *)out.dev, incy, s, conj_a);
            else
                rc = generic_scale<T>(M, 1, zero_only ? T(0) : beta, (T *)out.dev, incy, 0, s);
        }
    }
    if (!rc) rc = stage_out_end(out, s);
    if (!rc && !out.host && cudaStreamSynchronize(s) != cudaSuccess) rc = O64_ERR_CUDA;
    return rc;
}

extern "C" void _s4gemvx__(const int *m, const int *n, const float *alpha, const float *a,
                           const int *incca, const int *incra, const float *x, const int *incx,
                           const float *beta, float *y, const int *incy) {
    g_compat_status = xgemvx_impl<float>(*m, *n, *alpha, a, *incca, *incra, x, *incx, *beta, y, *incy);
}

extern "C" void _sgemvx__(const int *m, const int *n, const double *alpha, const double *a,
                          const int *incca, const int *incra, const double *x, const int *incx,
                          const double *beta, double *y, const int *incy) {
    g_compat_status = xgemvx_impl<double>(*m, *n, *alpha, a, *incca, *incra, x, *incx, *beta, y, *incy);
}

#define O64_CGEMVX_ENTRY(NAME, R)                                                                          \
    extern "C" void NAME(const int *iconj, const int *m, const int *n, const R *alpha, const R *a,         \
                         const int *incca, const int *incra, const R *x, const int *incx, const R *beta,   \
                         R *y, const int *incy) {                                                          \
        typedef Cx<R> T;                                                                                   \
        g_compat_status = xgemvx_impl<T>(*m, *n, T(alpha[0], alpha[1]), reinterpret_cast<const T *>(a), *incca, \
                                         *incra, reinterpret_cast<const T *>(x), *incx, T(beta[0], beta[1]), \
                                         reinterpret_cast<T *>(y), *incy, *iconj != 0);                    \
    }
O64_CGEMVX_ENTRY(_c4gemvx__, float)
O64_CGEMVX_ENTRY(_cgemvx__, double)
#undef O64_CGEMVX_ENTRY

// BLAS hooks for COMPLEX MATMUL (osprey/libfi/matrix/mmx_dlutil.c:135-136): 'c' is the conjugate transpose.
template <typename R>
static int blas_cgemm_impl(const char *transa, const char *transb, const int *m, const int *n, const int *k,
                           const R *alpha, const R *a, const int *lda, const R *b, const int *ldb, const R *beta,
                           R *c, const int *ldc) {
    typedef Cx<R> T;
    auto kind = [](char ch) { return (ch == 'n' || ch == 'N') ? 0 : (ch == 't' || ch == 'T') ? 1 : (ch == 'c' || ch == 'C') ? 2 : -1; };
    const int ka = kind(*transa), kb = kind(*transb);
    if (ka < 0 || kb < 0) return O64_ERR_RANK;
    const int rows_a = ka == 0 ? *m : *k, rows_b = kb == 0 ? *k : *n;
    if (*lda < (rows_a > 1 ? rows_a : 1) || *ldb < (rows_b > 1 ? rows_b : 1) || *ldc < (*m > 1 ? *m : 1))
        return O64_ERR_CONFORM;
    const int64_t a1 = ka == 0 ? 1 : *lda, a2 = ka == 0 ? *lda : 1;
    const int64_t b1 = kb == 0 ? 1 : *ldb, b2 = kb == 0 ? *ldb : 1;
    return xgemmx_impl<T, T>(*m, *n, *k, T(alpha[0], alpha[1]), reinterpret_cast<const T *>(a), a1, a2,
                             reinterpret_cast<const T *>(b), b1, b2, T(beta[0], beta[1]), reinterpret_cast<T *>(c), 1,
                             *ldc, false, ka == 2, kb == 2);
}

extern "C" void cgemm_(const char *transa, const char *transb, const int *m, const int *n, const int *k,
                       const float *alpha, const float *a, const int *lda, const float *b, const int *ldb,
                       const float *beta, float *c, const int *ldc) {
    g_compat_status = blas_cgemm_impl<float>(transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}

extern "C" void zgemm_(const char *transa, const char *transb, const int *m, const int *n, const int *k,
                       const double *alpha, const double *a, const int *lda, const double *b, const int *ldb,
                       const double *beta, double *c, const int *ldc) {
    g_compat_status = blas_cgemm_impl<double>(transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}

// ---- the MATMUL operator entry point (osprey/libfi/matrix/matmul_s4s4.c:66-112) ----------------
namespace {
struct DvView {
    void *ptr;
    int ndim;
    long n1, n2, inc1, inc2;
};

// Extents and element strides of a dope vector, as _premult reads them
// (osprey/libfi/matrix/matmul.h:145-176): multi-word elements carry a factor in stride_mult.
DvView view_of(const o64_dopevec_t *d) {
    DvView v;
    v.ptr = d->ptr;
    v.ndim = (int)(d->flags1 >> 29);
    const unsigned int_len = (d->type_bits >> 12) & 0xfffu;
    const int shift = int_len == 64 ? 1 : (int_len == 128 ? 2 : (int_len == 256 ? 3 : 0));
    v.n1 = d->dimension[0].extent;
    v.inc1 = d->dimension[0].stride_mult >> shift;
    if (v.ndim == 1) {
        v.n2 = 1;
        v.inc2 = v.inc1;
    } else {
        v.n2 = d->dimension[1].extent;
        v.inc2 = d->dimension[1].stride_mult >> shift;
    }
    return v;
}

struct MatDims {
    DvView a, b, c;
    int m, n, k;
};

// The part of _premult every entry point shares: rank check, allocation of an unassociated
// RESULT (matmul.h:222-266; default_bits is the result's element size where its type word gives
// none), conformance checks and m, n, k (matmul.h:325-363).
int matmul_premult(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B, unsigned default_bits,
                   MatDims *d) {
    if (!RESULT || !MATRIX_A || !MATRIX_B) return O64_ERR_RANK;
    const DvView a = view_of(MATRIX_A), b = view_of(MATRIX_B);
    if (!((a.ndim == 1 && b.ndim == 2) || (a.ndim == 2 && b.ndim == 1) || (a.ndim == 2 && b.ndim == 2)))
        return O64_ERR_RANK;  // FESCIRNK
    if (!(RESULT->flags0 & 1u)) {
        unsigned int_len = (RESULT->type_bits >> 12) & 0xfffu;
        if (int_len == 0) {
            // a RESULT whose type word carries no element length gets the entry point's result kind,
            // written back so that the strides below and their later reading agree
            int_len = default_bits;
            RESULT->type_bits = (RESULT->type_bits & ~(0xfffu << 12)) | ((int_len & 0xfffu) << 12);
        }
        long stride0 = int_len / 32;
        if (stride0 == 0) stride0 = 1;
        RESULT->dimension[0].stride_mult = stride0;
        RESULT->dimension[0].low_bound = 1;
        long nbits;
        if (a.ndim == 1) {
            RESULT->dimension[0].extent = b.n2;
            nbits = b.n2 * (long)int_len;
        } else if (b.ndim == 1) {
            RESULT->dimension[0].extent = a.n1;
            nbits = a.n1 * (long)int_len;
        } else {
            RESULT->dimension[0].extent = a.n1;
            RESULT->dimension[1].low_bound = 1;
            RESULT->dimension[1].extent = b.n2;
            RESULT->dimension[1].stride_mult = a.n1 * stride0;
            nbits = a.n1 * b.n2 * (long)int_len;
        }
        const long nbytes = nbits >> 3;
        void *mem = nullptr;
        if (nbytes != 0) {
            mem = malloc((size_t)nbytes);
            if (!mem) return O64_ERR_NOMEM;  // FENOMEMY
        }
        RESULT->flags0 |= 1u;
        RESULT->ptr = mem;
        RESULT->orig_base = mem;
        RESULT->orig_size = (unsigned long)nbits;
    }
    const DvView c = view_of(RESULT);
    d->a = a, d->b = b, d->c = c;
    if (a.ndim == 2 && b.ndim == 2) {
        if (!(a.n2 == b.n1 && c.n1 == a.n1 && c.n2 == b.n2)) return O64_ERR_CONFORM;  // FESCICNF
        d->m = (int)a.n1, d->n = (int)b.n2, d->k = (int)a.n2;
    } else if (a.ndim == 2) {  // y = A x
        if (!(a.n2 == b.n1 && a.n1 == c.n1)) return O64_ERR_CONFORM;
        d->m = (int)a.n1, d->n = 1, d->k = (int)a.n2;
    } else {  // y = x B
        if (!(a.n1 == b.n1 && c.n1 == b.n2)) return O64_ERR_CONFORM;
        d->m = 1, d->n = (int)b.n2, d->k = (int)b.n1;
    }
    return O64_OK;
}

// One MATMUL entry point of the runtime: parse the dope vectors and allocate an unassociated
// RESULT as _premult does (matmul.h:135-400), then call the strided kernels the way the entry
// point of that type does.  TN: the narrower (or equal) operand kind, T: the kind of the other
// operand and of the result.
//   use_gemv: the real kinds send the rank-1 cases to the matrix-vector kernel
//     (matmul_s4s4.c:86-104, matmul_ss@.c:100-117); the integer kinds send all three cases to the
//     matrix kernel with m, n, k of matmul.h:325-363 (matmul_i4i4.c:84-86).
//   swapped: MATRIX_A is the wider kind, so the product is formed as C' = B'A' with every pair of
//     increments exchanged (matmul_i2i1.c:82-84, matmul_i4i1.c:83-85, matmul_ji4.c).
template <typename TN, typename T, bool LOGICAL = false>
int matmul_impl(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B, bool use_gemv,
                bool swapped) {
    MatDims d;
    const int rc_dims = matmul_premult(RESULT, MATRIX_A, MATRIX_B, 8 * sizeof(T), &d);
    if (rc_dims) return rc_dims;
    const DvView &a = d.a, &b = d.b, &c = d.c;
    T *C = static_cast<T *>(c.ptr);
    const T one = T(1), zero = T(0);
    const int m = d.m, n = d.n, k = d.k;
    if constexpr (std::is_floating_point<T>::value || IsCx<T>::value) {
        if (use_gemv && a.ndim == 2 && b.ndim == 1)  // y = A x
            return xgemvx_impl<T>((int)a.n1, (int)a.n2, one, static_cast<const T *>(a.ptr), a.inc1, a.inc2,
                                  static_cast<const T *>(b.ptr), b.inc1, zero, C, c.inc1);
        if (use_gemv && a.ndim == 1)  // y = x B, i.e. y' = B' x'
            return xgemvx_impl<T>((int)b.n2, (int)b.n1, one, static_cast<const T *>(b.ptr), b.inc2, b.inc1,
                                  static_cast<const T *>(a.ptr), a.inc1, zero, C, c.inc1);
    }
    if constexpr (LOGICAL) {  // alpha = .TRUE., beta = .FALSE. (matmul_ll@.c:92-94)
        if (swapped)
            return lgemmx_impl<TN, T>(n, m, k, true, static_cast<const TN *>(b.ptr), b.inc2, b.inc1,
                                      static_cast<const T *>(a.ptr), a.inc2, a.inc1, false, C, c.inc2, c.inc1);
        return lgemmx_impl<TN, T>(m, n, k, true, static_cast<const TN *>(a.ptr), a.inc1, a.inc2,
                                  static_cast<const T *>(b.ptr), b.inc1, b.inc2, false, C, c.inc1, c.inc2);
    }
    if (swapped)
        return xgemmx_impl<TN, T>(n, m, k, one, static_cast<const TN *>(b.ptr), b.inc2, b.inc1,
                                  static_cast<const T *>(a.ptr), a.inc2, a.inc1, zero, C, c.inc2, c.inc1, true);
    return xgemmx_impl<TN, T>(m, n, k, one, static_cast<const TN *>(a.ptr), a.inc1, a.inc2,
                              static_cast<const T *>(b.ptr), b.inc1, b.inc2, zero, C, c.inc1, c.inc2, true);
}
}  // namespace

#define O64_MATMUL_ENTRY(NAME, TN, T, GEMV, SWAPPED)                                                      \
    extern "C" void NAME(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B) {       \
        g_compat_status = matmul_impl<TN, T>(RESULT, MATRIX_A, MATRIX_B, GEMV, SWAPPED);                  \
    }
O64_MATMUL_ENTRY(_MATMUL_S4S4, float, float, true, false)
O64_MATMUL_ENTRY(_MATMUL_SS, double, double, true, false)
O64_MATMUL_ENTRY(_MATMUL_C4C4, c4_t, c4_t, true, false)
O64_MATMUL_ENTRY(_MATMUL_CC, c8_t, c8_t, true, false)
O64_MATMUL_ENTRY(_MATMUL_I1I1, int8_t, int8_t, false, false)
O64_MATMUL_ENTRY(_MATMUL_I1I2, int8_t, int16_t, false, false)
O64_MATMUL_ENTRY(_MATMUL_I1I4, int8_t, int32_t, false, false)
O64_MATMUL_ENTRY(_MATMUL_I1J, int8_t, int64_t, false, false)
O64_MATMUL_ENTRY(_MATMUL_I2I1, int8_t, int16_t, false, true)
O64_MATMUL_ENTRY(_MATMUL_I2I2, int16_t, int16_t, false, false)
O64_MATMUL_ENTRY(_MATMUL_I2I4, int16_t, int32_t, false, false)
O64_MATMUL_ENTRY(_MATMUL_I2J, int16_t, int64_t, false, false)
O64_MATMUL_ENTRY(_MATMUL_I4I1, int8_t, int32_t, false, true)
O64_MATMUL_ENTRY(_MATMUL_I4I2, int16_t, int32_t, false, true)
O64_MATMUL_ENTRY(_MATMUL_I4I4, int32_t, int32_t, false, false)
O64_MATMUL_ENTRY(_MATMUL_I4J, int32_t, int64_t, false, false)
O64_MATMUL_ENTRY(_MATMUL_JI1, int8_t, int64_t, false, true)
O64_MATMUL_ENTRY(_MATMUL_JI2, int16_t, int64_t, false, true)
O64_MATMUL_ENTRY(_MATMUL_JI4, int32_t, int64_t, false, true)
O64_MATMUL_ENTRY(_MATMUL_JJ, int64_t, int64_t, false, false)
// mixed kinds with a REAL result: the narrower or integer operand is the kernel's A
O64_MATMUL_ENTRY(_MATMUL_S4S, float, double, false, false)
O64_MATMUL_ENTRY(_MATMUL_SS4, float, double, false, true)
O64_MATMUL_ENTRY(_MATMUL_I1S4, int8_t, float, false, false)
O64_MATMUL_ENTRY(_MATMUL_S4I1, int8_t, float, false, true)
O64_MATMUL_ENTRY(_MATMUL_I1S, int8_t, double, false, false)
O64_MATMUL_ENTRY(_MATMUL_SI1, int8_t, double, false, true)
O64_MATMUL_ENTRY(_MATMUL_I2S4, int16_t, float, false, false)
O64_MATMUL_ENTRY(_MATMUL_S4I2, int16_t, float, false, true)
O64_MATMUL_ENTRY(_MATMUL_I2S, int16_t, double, false, false)
O64_MATMUL_ENTRY(_MATMUL_SI2, int16_t, double, false, true)
O64_MATMUL_ENTRY(_MATMUL_I4S4, int32_t, float, false, false)
O64_MATMUL_ENTRY(_MATMUL_S4I4, int32_t, float, false, true)
O64_MATMUL_ENTRY(_MATMUL_I4S, int32_t, double, false, false)
O64_MATMUL_ENTRY(_MATMUL_SI4, int32_t, double, false, true)
O64_MATMUL_ENTRY(_MATMUL_JS4, int64_t, float, false, false)
O64_MATMUL_ENTRY(_MATMUL_S4J, int64_t, float, false, true)
O64_MATMUL_ENTRY(_MATMUL_JS, int64_t, double, false, false)
O64_MATMUL_ENTRY(_MATMUL_SJ, int64_t, double, false, true)
#undef O64_MATMUL_ENTRY
// LOGICAL arrays: every pair of the four kinds, result of the wider kind (matmul_l1l1.c ... matmul_ll@.c)
// COMPLEX with a REAL or INTEGER operand, or with COMPLEX of the other width: real and imaginary
// parts are separate products of the REAL kernel for the pair of component kinds, every increment
// of a COMPLEX array doubled (osprey/libfi/matrix/matmul_c4s4.c:84-108, matmul_i1c4.c,
// matmul_c4c.c:88-128).  TA / T: the kernel's first operand kind and its second operand / result
// kind.  swapped: the kernel's first operand is MATRIX_B, so the product is formed as C' = B'A'
// (matmul_c4i1.c:95-106, matmul_cs4.c, matmul_sc4.c, matmul_cc4.c).
namespace {
template <typename TA, typename T>
int matmul_cx_impl(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B, bool a_cx, bool b_cx,
                   bool swapped) {
    MatDims d;
    int rc = matmul_premult(RESULT, MATRIX_A, MATRIX_B, 16 * sizeof(T), &d);
    if (rc) return rc;
    const long fa = a_cx ? 2 : 1, fb = b_cx ? 2 : 1;
    const long a1 = d.a.inc1 * fa, a2 = d.a.inc2 * fa, b1 = d.b.inc1 * fb, b2 = d.b.inc2 * fb;
    const long c1 = d.c.inc1 * 2, c2 = d.c.inc2 * 2;
    T *Cr = static_cast<T *>(d.c.ptr);
    // part 0 / 1 of an operand: real / imaginary (a REAL or INTEGER operand has part 0 only)
    auto mul = [&](T alpha, int part_a, int part_b, T beta, T *C) {
        if (!swapped) {
            const TA *A = static_cast<const TA *>(d.a.ptr);
            const T *B = static_cast<const T *>(d.b.ptr);
            return xgemmx_impl<TA, T>(d.m, d.n, d.k, alpha, A ? A + part_a : A, a1, a2, B ? B + part_b : B, b1, b2, beta,
                                      C, c1, c2, true);
        }
        const TA *B = static_cast<const TA *>(d.b.ptr);
        const T *A = static_cast<const T *>(d.a.ptr);
        return xgemmx_impl<TA, T>(d.n, d.m, d.k, alpha, B ? B + part_b : B, b2, b1, A ? A + part_a : A, a2, a1, beta, C,
                                  c2, c1, true);
    };
    T *Ci = Cr ? Cr + 1 : Cr;
    if (a_cx && b_cx) {  // (Ar Br - Ai Bi) + (Ar Bi + Ai Br) i
        if ((rc = mul(T(1), 0, 0, T(0), Cr))) return rc;
        if ((rc = mul(T(-1), 1, 1, T(1), Cr))) return rc;
        if ((rc = mul(T(1), 0, 1, T(0), Ci))) return rc;
        return mul(T(1), 1, 0, T(1), Ci);
    }
    if ((rc = mul(T(1), 0, 0, T(0), Cr))) return rc;
    return mul(T(1), a_cx ? 1 : 0, b_cx ? 1 : 0, T(0), Ci);
}
}  // namespace

#define O64_CXMATMUL_ENTRY(NAME, TA, T, A_CX, B_CX, SWAPPED)                                              \
    extern "C" void NAME(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B) {       \
        g_compat_status = matmul_cx_impl<TA, T>(RESULT, MATRIX_A, MATRIX_B, A_CX, B_CX, SWAPPED);         \
    }
O64_CXMATMUL_ENTRY(_MATMUL_C4S4, float, float, true, false, false)
O64_CXMATMUL_ENTRY(_MATMUL_S4C4, float, float, false, true, false)
O64_CXMATMUL_ENTRY(_MATMUL_C4S, float, double, true, false, false)
O64_CXMATMUL_ENTRY(_MATMUL_SC4, float, double, false, true, true)
O64_CXMATMUL_ENTRY(_MATMUL_CS4, float, double, true, false, true)
O64_CXMATMUL_ENTRY(_MATMUL_S4C, float, double, false, true, false)
O64_CXMATMUL_ENTRY(_MATMUL_CS, double, double, true, false, false)
O64_CXMATMUL_ENTRY(_MATMUL_SC, double, double, false, true, false)
O64_CXMATMUL_ENTRY(_MATMUL_C4C, float, double, true, true, false)
O64_CXMATMUL_ENTRY(_MATMUL_CC4, float, double, true, true, true)
O64_CXMATMUL_ENTRY(_MATMUL_C4I1, int8_t, float, true, false, true)
O64_CXMATMUL_ENTRY(_MATMUL_C4I2, int16_t, float, true, false, true)
O64_CXMATMUL_ENTRY(_MATMUL_C4I4, int32_t, float, true, false, true)
O64_CXMATMUL_ENTRY(_MATMUL_C4J, int64_t, float, true, false, true)
O64_CXMATMUL_ENTRY(_MATMUL_I1C4, int8_t, float, false, true, false)
O64_CXMATMUL_ENTRY(_MATMUL_I2C4, int16_t, float, false, true, false)
O64_CXMATMUL_ENTRY(_MATMUL_I4C4, int32_t, float, false, true, false)
O64_CXMATMUL_ENTRY(_MATMUL_JC4, int64_t, float, false, true, false)
O64_CXMATMUL_ENTRY(_MATMUL_CI1, int8_t, double, true, false, true)
O64_CXMATMUL_ENTRY(_MATMUL_CI2, int16_t, double, true, false, true)
O64_CXMATMUL_ENTRY(_MATMUL_CI4, int32_t, double, true, false, true)
O64_CXMATMUL_ENTRY(_MATMUL_CJ, int64_t, double, true, false, true)
O64_CXMATMUL_ENTRY(_MATMUL_I1C, int8_t, double, false, true, false)
O64_CXMATMUL_ENTRY(_MATMUL_I2C, int16_t, double, false, true, false)
O64_CXMATMUL_ENTRY(_MATMUL_I4C, int32_t, double, false, true, false)
O64_CXMATMUL_ENTRY(_MATMUL_JC, int64_t, double, false, true, false)
#undef O64_CXMATMUL_ENTRY

#define O64_LMATMUL_ENTRY(NAME, TN, T, SWAPPED)                                                           \
    extern "C" void NAME(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B) {       \
        g_compat_status = matmul_impl<TN, T, true>(RESULT, MATRIX_A, MATRIX_B, false, SWAPPED);           \
    }
O64_LMATMUL_ENTRY(_MATMUL_L1L1, int8_t, int8_t, false)
O64_LMATMUL_ENTRY(_MATMUL_L1L2, int8_t, int16_t, false)
O64_LMATMUL_ENTRY(_MATMUL_L1L4, int8_t, int32_t, false)
O64_LMATMUL_ENTRY(_MATMUL_L1L, int8_t, int64_t, false)
O64_LMATMUL_ENTRY(_MATMUL_L2L1, int8_t, int16_t, true)
O64_LMATMUL_ENTRY(_MATMUL_L2L2, int16_t, int16_t, false)
O64_LMATMUL_ENTRY(_MATMUL_L2L4, int16_t, int32_t, false)
O64_LMATMUL_ENTRY(_MATMUL_L2L, int16_t, int64_t, false)
O64_LMATMUL_ENTRY(_MATMUL_L4L1, int8_t, int32_t, true)
O64_LMATMUL_ENTRY(_MATMUL_L4L2, int16_t, int32_t, true)
O64_LMATMUL_ENTRY(_MATMUL_L4L4, int32_t, int32_t, false)
O64_LMATMUL_ENTRY(_MATMUL_L4L, int32_t, int64_t, false)
O64_LMATMUL_ENTRY(_MATMUL_LL1, int8_t, int64_t, true)
O64_LMATMUL_ENTRY(_MATMUL_LL2, int16_t, int64_t, true)
O64_LMATMUL_ENTRY(_MATMUL_LL4, int32_t, int64_t, true)
O64_LMATMUL_ENTRY(_MATMUL_LL, int64_t, int64_t, false)
#undef O64_LMATMUL_ENTRY

// ---- DOT_PRODUCT over dope vectors (osprey/libfi/dotprod) ----------------------------------------
// _DOT_<A><B>(VECTOR_A, VECTOR_B): the vectors' addresses, length and element strides are read as the
// runtime's _PREDOT reads them (osprey/libfi/dotprod/predot@.c:52-93: the length is VECTOR_A's extent,
// strides of 64- and 128-bit elements are divided down from 32-bit words), then one pass on the GPU
// (dotprod.cu) forms the sum of dot90.h / dotc90.h / dotl90.h.  Host vectors are staged.  Unlike the
// reference a VECTOR_B shorter than VECTOR_A is reported (O64_ERR_CONFORM, result 0) instead of read
// past its end.
namespace {
template <typename TX, typename TY, typename TR, int MODE>
TR dot_impl(const o64_dopevec_t *X, const o64_dopevec_t *Y) {
    TR result = TR(0);
    g_compat_status = O64_OK;
    if (!X || !Y) {
        g_compat_status = O64_ERR_RANK;
        return result;
    }
    const DvView x = view_of(X), y = view_of(Y);
    if (x.ndim != 1 || y.ndim != 1) {
        g_compat_status = O64_ERR_RANK;
        return result;
    }
    const long n = x.n1;
    if (n <= 0) return result;
    if (y.n1 < n) {
        g_compat_status = O64_ERR_CONFORM;
        return result;
    }
    if (!x.ptr || !y.ptr || x.inc1 < 0 || y.inc1 < 0) {
        g_compat_status = O64_ERR_RANK;
        return result;
    }
    o64_handle_t h = compat_handle();
    if (!h) {
        g_compat_status = O64_ERR_CUDA;
        return result;
    }
    DeviceGuard g(h->device);
    cudaStream_t s = nullptr;
    const void *dx, *dy;
    int rc = stage_in(h, 0, x.ptr, strided_span(n, 1, x.inc1, 0) * sizeof(TX), s, &dx);
    if (!rc) rc = stage_in(h, 1, y.ptr, strided_span(n, 1, y.inc1, 0) * sizeof(TY), s, &dy);
    if (!rc) rc = reserve(&h->ws, &h->ws_cap, dot_workspace_bytes());
    if (!rc)
        rc = dot_device<TX, TY, TR, MODE>(n, static_cast<const TX *>(dx), x.inc1, static_cast<const TY *>(dy), y.inc1, h->ws,
                                          &result, s);
    g_compat_status = rc;
    return rc ? TR(0) : result;
}
}  // namespace

#define O64_DOT_ENTRY(NAME, RET, TX, TY, TR, MODE)                                       \
    extern "C" RET NAME(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B) {  \
        const TR r = dot_impl<TX, TY, TR, MODE>(VECTOR_A, VECTOR_B);                     \
        RET out;                                                                         \
        static_assert(sizeof(out) == sizeof(r), "result size");                          \
        memcpy(&out, &r, sizeof(out));                                                   \
        return out;                                                                      \
    }
O64_DOT_ENTRY(_DOT_S4S4, float, float, float, float, 0)
O64_DOT_ENTRY(_DOT_SS, double, double, double, double, 0)
O64_DOT_ENTRY(_DOT_S4S, double, float, double, double, 0)
O64_DOT_ENTRY(_DOT_SS4, double, double, float, double, 0)
O64_DOT_ENTRY(_DOT_I4I4, int32_t, int32_t, int32_t, uint32_t, 0)
O64_DOT_ENTRY(_DOT_JJ, int64_t, int64_t, int64_t, uint64_t, 0)
O64_DOT_ENTRY(_DOT_I4J, int64_t, int32_t, int64_t, uint64_t, 0)
O64_DOT_ENTRY(_DOT_JI4, int64_t, int64_t, int32_t, uint64_t, 0)
O64_DOT_ENTRY(_DOT_I4S4, float, int32_t, float, float, 0)
O64_DOT_ENTRY(_DOT_S4I4, float, float, int32_t, float, 0)
O64_DOT_ENTRY(_DOT_I4S, double, int32_t, double, double, 0)
O64_DOT_ENTRY(_DOT_SI4, double, double, int32_t, double, 0)
O64_DOT_ENTRY(_DOT_JS4, float, int64_t, float, float, 0)
O64_DOT_ENTRY(_DOT_S4J, float, float, int64_t, float, 0)
O64_DOT_ENTRY(_DOT_JS, double, int64_t, double, double, 0)
O64_DOT_ENTRY(_DOT_SJ, double, double, int64_t, double, 0)
O64_DOT_ENTRY(_DOT_L4L4, int32_t, int32_t, int32_t, int32_t, 1)
O64_DOT_ENTRY(_DOT_LL, int64_t, int64_t, int64_t, int64_t, 1)
O64_DOT_ENTRY(_DOT_L4L, int64_t, int32_t, int64_t, int64_t, 1)
O64_DOT_ENTRY(_DOT_LL4, int64_t, int64_t, int32_t, int64_t, 1)
O64_DOT_ENTRY(_DOT_C4C4, o64_complex8_t, c4_t, c4_t, c4_t, 2)
O64_DOT_ENTRY(_DOT_CC, o64_complex16_t, c8_t, c8_t, c8_t, 2)
#undef O64_DOT_ENTRY
