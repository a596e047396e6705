/*
 * o64gemm.h — C ABI of libo64gemm.so, a B200 (sm_100a) dense GEMM / fused-linear engine
 * that sits behind the matrix-multiply boundary of the Open64 compiler's runtime.
 *
 * Two layers:
 *
 *   compat layer  — the symbols the reference's own callers already bind:
 *       sgemm_        the BLAS hook resolved by dlsym when F90_MATMUL_BLAS is set
 *                     (osprey/libfi/matrix/mmx_dlutil.c:75-136, called as
 *                     ('n','n',m,n,k,alpha,A,m,B,k,beta,R,m), mmx_fort.h:94-95)
 *       _s4gemmx__    the strided "X interface" kernel behind _MATMUL_S4S4
 *                     (osprey/libfi/matrix/s4gemmx.f:37-199, template xgemmx.h:156-236,
 *                     call site matmul_s4s4.c:107-109)
 *       _s4gemvx__    its matrix-vector sibling (osprey/libfi/matrix/s4gemvx.f,
 *                     call sites matmul_s4s4.c:91-101)
 *       the same three for
 *       REAL*8 (dgemm_, _sgemmx__, _sgemvx__, _MATMUL_SS), COMPLEX*8 / *16 (cgemm_, zgemm_,
 *       _c4gemmx__, _cgemmx__, _MATMUL_C4C4, _MATMUL_CC), every pair of integer kinds
 *       (_MATMUL_I1I1 ... _MATMUL_JJ over _i1gemmx__ ... _jgemmx__) and the real x real / integer x
 *       real pairs (_MATMUL_S4S, _MATMUL_I4S4, ...), and COMPLEX with any of those or with the
 *       other COMPLEX width (_MATMUL_C4S4, _MATMUL_I1C4, _MATMUL_C4C, ...); in the runtime's naming "S" is the 64-bit
 *       real, "S4" the 32-bit one, "J" the 64-bit integer, "C" / "C4" the complex kinds
 *     Fortran ABI: every scalar by reference, synchronous, void.  Host or device
 *     pointers are accepted (host operands are staged through device memory).
 *
 *   native layer  — o64_* functions: device pointers (host pointers are staged when
 *     detected), asynchronous on the caller's CUDA stream, int status returned, never
 *     abort.  These are what host code lowered from a tiled loop nest calls.
 *
 * Error codes mirror the runtime's abort codes (osprey/libfi/matrix/matmul.h:217,258,
 * 333-369; osprey/clibinc/liberrno.h:326,442-443): FESCIRNK -> O64_ERR_RANK,
 * FESCICNF -> O64_ERR_CONFORM, FENOMEMY -> O64_ERR_NOMEM.  An operand that is device memory of a GPU
 * other than the one the call runs on is refused with O64_ERR_RANK before anything is launched.
 * K == 0 is the empty sum: the result is the epilogue applied to zero (osprey/libfi/matrix/xgemmx.h:185-196
 * sets C to zero); only the no-allocation entry point rejects it.
 *
 * No C++ or torch types cross this boundary.  cudaStream_t is passed as void*.
 */
#ifndef O64GEMM_H
#define O64GEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct o64_handle_s *o64_handle_t;

/* ---- status codes ------------------------------------------------------------------- */
enum {
    O64_OK = 0,
    O64_ERR_RANK = -1,    /* illegal rank / bad argument          (FESCIRNK) */
    O64_ERR_CONFORM = -2, /* operands not conformable             (FESCICNF) */
    O64_ERR_NOMEM = -3,   /* allocation failed                    (FENOMEMY) */
    O64_ERR_ALIGN = -4,   /* pointer or leading dimension not 16-byte aligned */
    O64_ERR_DTYPE = -5,   /* unsupported element type / layout combination */
    O64_ERR_TIMEOUT = -6, /* a bounded device-side wait ran out (read by o64_last_status) */
    O64_ERR_CUDA = -7,    /* a CUDA runtime or driver call failed */
    O64_ERR_NCCL = -8     /* an NCCL call failed or no communicator is bound */
};

/* ---- epilogue vocabulary --------------------------------------------------------------
 * The elementwise tail of a fused linear: what OPR_MAX and the exp/tanh intrinsics express
 * in the reference's IR (osprey/be/cg/x8664/expand.cxx:4517,
 * osprey/common/com/intrn_entry.def:915,1346). */
enum {
    O64_ACT_NONE = 0,
    O64_ACT_RELU = 1,
    O64_ACT_GELU_TANH = 2,
    O64_ACT_GELU_ERF = 3,
    O64_ACT_SILU = 4
};

typedef struct {
    const float *bias; /* [N] fp32, device pointer, may be NULL */
    int act;           /* O64_ACT_* */
} o64_epilogue_t;

/* ---- element kinds (plan queries, naive reference kernels) ---------------------------- */
enum {
    O64_KIND_F32 = 0,  /* fp32 SIMT */
    O64_KIND_BF16 = 1, /* bf16 x bf16 -> fp32 accumulate */
    O64_KIND_FP8 = 2,  /* e4m3 x e4m3 -> fp32 accumulate */
    O64_KIND_S8 = 3    /* s8 x s8 -> s32 accumulate */
};

/* ---- the tile plan ----------------------------------------------------------------------
 * Carries the vocabulary of the reference's tile decision (LOOP_MODEL results,
 * osprey/be/lno/model.h:57-118, handed on as SNL_TILE_INFO, osprey/be/lno/snl_utils.h:388)
 * onto the B200 memory hierarchy:
 *   Block_Number (register tile)      -> mma_m x mma_n x mma_k of one tensor-core instruction
 *   Stripsz at level 1 (L1 block)     -> tile_m x tile_n x tile_k staged in shared memory
 *   number of in-flight L1 blocks     -> stages of the shared-memory ring
 *   Stripsz at level 2 (L2 block)     -> group_m: rows of tiles rasterised together in L2
 *   New_Order (loop permutation)      -> raster: 0 = tiles walk M fastest inside a group,
 *                                                1 = N fastest
 * cta_group = 1 or 2 CTAs cooperating on one accumulator tile. */
typedef struct {
    int kind;      /* O64_KIND_* */
    int tile_m;    /* rows of C per CTA tile (per CTA pair when cta_group == 2); with split_k < 0:
                      rows of A loaded per stage (16, 32, 64 or 128, the next size >= M) */
    int tile_n;    /* accumulator columns per tile */
    int tile_k;    /* K elements per shared-memory stage */
    int stages;    /* depth of the TMA -> MMA ring */
    int cta_group; /* 1 or 2 */
    int group_m;   /* L2 rasterisation group, in tiles */
    int raster;    /* 0 = M fastest, 1 = N fastest */
    int mma_m, mma_n, mma_k;
    int num_ctas;        /* persistent grid size */
    int split_k;         /* > 1: K slices on separate CTAs, reduced through scratch memory; 1: none;
                            < 0: the kernel for M <= 128 - every 128 x tile_n tile (tile_n = 256 or 128)
                            is split along K over a thread-block cluster of -split_k CTAs (1, 2, 4, 8;
                            at most tile_n / 32) whose partial sums meet in distributed shared memory.  In a pin, -1 asks for that kernel and lets the
                            library choose the cluster size; >= 1 rules it out */
    double predicted_ms; /* model estimate, compare with the measured time */
} o64_plan_t;

/* ---- handle ------------------------------------------------------------------------- */
/* A handle is bound to one device and is not thread-safe; distinct handles are independent.
 * It owns the device status word, staging buffers for host operands and the NCCL
 * communicator (if one is bound). */
int o64_create(o64_handle_t *out, int device);
int o64_destroy(o64_handle_t h);
/* Synchronises `stream`, reads and clears the device status word: O64_OK or
 * O64_ERR_TIMEOUT.  `detail`, if not NULL, receives the raw word (which wait gave up). */
int o64_last_status(o64_handle_t h, void *stream, int *detail);
/* Budget of the kernels' bounded device-side waits for later calls on this handle, in microseconds
 * (0 = the default, two seconds; the environment variable O64_WAIT_BUDGET_US sets the default of new
 * handles).  A wait that outlasts it ends its kernel in the ordinary way - tensor memory freed, no
 * trap - with O64_ERR_TIMEOUT left for o64_last_status: the runtime this library replaces names the
 * failing phase and aborts (osprey/common/util/errors.cxx:343-417); here the code names the wait. */
int o64_set_wait_budget_us(o64_handle_t h, int64_t microseconds);
const char *o64_status_string(int status);
const char *o64_version(void);

/* Plan query / override.  o64_plan_get fills the plan the engine would use for this shape.
 * o64_plan_set pins fields for later calls of `kind` (fields set to 0 stay automatic);
 * plan == NULL clears the override.  The environment variable O64_LNO
 * ("blocking_size=128x256x64:stages=4:cta_group=1:group_m=8", after the reference's
 * -LNO:blocking_size / pragma BLOCKING SIZE vocabulary, osprey/common/com/config_lno.cxx:128-129,
 * osprey/common/com/wn_pragmas.h:143-151) does the same for every handle. */
int o64_plan_get(o64_handle_t h, int kind, int64_t M, int64_t N, int64_t K, o64_plan_t *plan);
int o64_plan_set(o64_handle_t h, int kind, const o64_plan_t *plan);
/* The chooser itself, without a device: the plan for a machine of `num_sms` SMs, with `pin`
 * (may be NULL) and O64_LNO applied.  `swiglu` != 0 scores the fused gate/up GEMM. */
int o64_plan_model(int kind, int swiglu, int64_t M, int64_t N, int64_t K, int num_sms,
                   const o64_plan_t *pin, o64_plan_t *plan);
/* Measures instead of modelling: runs every kernel shape that exists for `kind` on pseudo-random
 * scratch operands of these extents (A [M,K], B [N,K]; SwiGLU: two [K,N] weights), remembers the
 * fastest for (kind, swiglu, M, N, K) and uses it from then on whenever the kind has no pin.
 * Allocates and frees its scratch, synchronises `stream`; *best (may be NULL) receives the plan
 * with predicted_ms = the measured time.  o64_plan_tune_clear forgets every measured plan. */
int o64_plan_tune(o64_handle_t h, int kind, int swiglu, int64_t M, int64_t N, int64_t K, void *stream,
                  o64_plan_t *best);
int o64_plan_tune_clear(o64_handle_t h);
/* Measured plans outlive the handle in a JSON file: one object per (kind, epilogue, M, N, K, ranks of the
 * communicator) with the kernel shape and the time it was measured at, under the device name and SM
 * count they were measured on (the reference hands each phase's decisions to the next through the WHIRL
 * file it writes, osprey/common/com/ir_bwrite.cxx:1505).  o64_plan_load merges a file into the handle:
 * O64_ERR_RANK if it cannot be read, O64_ERR_CONFORM if it was measured on another device type,
 * O64_ERR_DTYPE if it holds no usable plan; entries that name no existing kernel are skipped.  With
 * O64_PLAN_CACHE=<path> in the environment o64_create loads that file and o64_plan_tune rewrites it. */
int o64_plan_save(o64_handle_t h, const char *path);
int o64_plan_load(o64_handle_t h, const char *path);
int o64_plan_count(o64_handle_t h);

/* ---- native layer -------------------------------------------------------------------
 * Row-major operands; ld* in elements.  A is [M,K].  B is [K,N] when transB == 0 and
 * [N,K] when transB != 0.  `stream` is a cudaStream_t (NULL = default stream). */

/* Y = act(A*B + bias), fp32, B [K,N].  Replaces the loop nest the compiler builds for
 * MATMUL plus its elementwise tail (osprey/be/vho/f90_lower.cxx:5116-5178). */
int o64_linear_f32(o64_handle_t h, int64_t M, int64_t N, int64_t K, const float *A, int64_t lda,
                   const float *B, int64_t ldb, const float *bias, float *Y, int64_t ldy, int act,
                   void *stream);

/* C = act(A*op(B) + bias): bf16 operands, fp32 accumulate, bf16 result.  Same nest on a
 * 16-bit element type the reference's IR lacks (osprey/common/com/mtypes.h:81-143). */
int o64_gemm_bf16(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *A, int64_t lda,
                  const void *B, int64_t ldb, int transB, void *C, int64_t ldc,
                  const o64_epilogue_t *epi, void *stream);

/* H = silu(X*Wg) (.) (X*Wu): X [M,K], Wg and Wu [K,N] (ldw), H [M,N], all bf16; both
 * products accumulate side by side and the SiLU-multiply runs in the epilogue. */
int o64_gemm_bf16_swiglu(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *X,
                         int64_t ldx, const void *Wg, const void *Wu, int64_t ldw, void *H,
                         int64_t ldh, void *stream);

/* C = bf16( (A8*B8^T) * scaleA[m] * scaleB[n] + bias[n] ): e4m3 operands, A8 [M,K], B8 [N,K],
 * fp32 accumulate.  scaleA, scaleB, bias are fp32 device vectors and may be NULL. */
int o64_gemm_fp8_scaled(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *A8,
                        int64_t lda, const void *B8, int64_t ldb, const float *scaleA,
                        const float *scaleB, const float *bias, void *C, int64_t ldc,
                        void *stream);

/* The same e4m3 product with the weight stored [K,N] row-major (N contiguous, ldb >= N; device
 * memory).  A weight whose base address and ldb are multiples of 16 is read in place (same speed
 * and the same bits as the [N,K] entry point on the transposed weight); any other is first
 * transposed into handle-owned scratch on the caller's stream (one extra pass over N*K bytes). */
int o64_gemm_fp8_scaled_kn(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *A8, int64_t lda,
                           const void *B8_kn, int64_t ldb, const float *scaleA, const float *scaleB,
                           const float *bias, int act, void *C, int64_t ldc, int out_kind, void *stream);

/* The scaled products with a fused activation and a choice of result type ("requantisation"):
 *   C = convert( act( acc * (scaleA[m] * scaleB[n]) + bias[n] ) )
 * acc: the fp32 (e4m3 operands) or int32 (int8 operands, converted to fp32) accumulator; every fp32
 * operation is rounded by itself (nothing is fused), so the value is reproducible bit for bit on a
 * CPU; scaleA, scaleB, bias may be NULL (1, 1, 0).  out_kind: O64_OUT_BF16 (ldc in 2-byte elements),
 * or the operands' own 8-bit type - O64_OUT_E4M3 for the fp8 product, O64_OUT_S8 for the int8 product,
 * ldc in bytes - rounded to nearest even and saturated (e4m3: +-448, int8: -128 ... 127), which is
 * what feeds the next 8-bit layer without a pass over a wide intermediate.  The narrow integer result
 * has a relative in the reference's MATMUL of INTEGER*1 arrays, which returns INTEGER*1
 * (osprey/crayf90/fe90/intrin.h:4294, osprey/libfi/matrix/i1gemmx.f) - there by wrap-around, here by
 * scaling and saturation; the elementwise vocabulary is the one of O64_ACT_*. */
enum { O64_OUT_BF16 = 0, O64_OUT_S8 = 1, O64_OUT_E4M3 = 2 };
int o64_gemm_fp8_scaled_ex(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *A8, int64_t lda,
                           const void *B8, int64_t ldb, const float *scaleA, const float *scaleB,
                           const float *bias, int act, void *C, int64_t ldc, int out_kind, void *stream);
int o64_gemm_s8_scaled(o64_handle_t h, int64_t M, int64_t N, int64_t K, const int8_t *A, int64_t lda,
                       const int8_t *B, int64_t ldb, const float *scaleA, const float *scaleB,
                       const float *bias, int act, void *C, int64_t ldc, int out_kind, void *stream);

/* C = A*B^T: int8 operands, A [M,K], B [N,K], int32 accumulate and result, exact.  The
 * reference's integer kernels are instances of the same template
 * (osprey/libfi/matrix/i1i4gemmx.f; front-end table osprey/crayf90/fe90/intrin.h:4276-4303). */
int o64_gemm_s8s8_s32(o64_handle_t h, int64_t M, int64_t N, int64_t K, const int8_t *A,
                      int64_t lda, const int8_t *B, int64_t ldb, int32_t *C, int64_t ldc,
                      void *stream);

/* The same product for callers that must not allocate device memory (no counterpart in the
 * reference: its runtime mallocs freely, osprey/libfi/matrix/matmul.h:222-266).  No handle, no
 * cudaMalloc / cudaFree anywhere on the path: the status word of the bounded waits and the padded
 * copies of operands whose base or row pitch is not a multiple of 16 bytes live in one static device
 * array of O64_STATIC_SCRATCH_BYTES per GPU.  Device pointers only, of the device that is current at
 * the call (`stream` too); anything else is O64_ERR_RANK.  Returns O64_ERR_NOMEM, and does
 * nothing, when the padded copies (M*ceil16(K) for A plus N*ceil16(K) for B, each only if needed)
 * exceed the array.  The first call on a device resolves the array's address; make it before any
 * stream capture.  Calls on one device share the array: calls that overlap on the GPU race. */
#define O64_STATIC_SCRATCH_BYTES (16u << 20)
int o64_gemm_s8s8_s32_static(int64_t M, int64_t N, int64_t K, const int8_t *A, int64_t lda,
                             const int8_t *B, int64_t ldb, int32_t *C, int64_t ldc, void *stream);

/* Test hook for the failure path (no counterpart in the reference): o64_gemm_bf16 with B [N,K] and no
 * epilogue, run by the kernel the handle's plan pin selects in an instantiation whose loader leaves
 * out the loads of its `withhold_kblock`-th K block.  The kernel's waits then run out of the handle's
 * wait budget and it returns; o64_last_status gives O64_ERR_TIMEOUT and which wait gave up.  Device
 * pointers only; C is undefined afterwards.  Shipped kernels carry no such branch. */
int o64_test_gemm_bf16_withheld(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *A, int64_t lda,
                                const void *B, int64_t ldb, void *C, int64_t ldc, int withhold_kblock,
                                void *stream);

/* Test hook: what the last launch of a CTA-pair kernel made from this thread did about a partly
 * filled last wave of tiles - how many tiles it cut along K and over how many CTA pairs (0, 0: it ran
 * whole tiles only).  No counterpart in the reference. */
int o64_test_last_tail_split(int *tiles, int *pairs);
/* Test hook, process-wide: 1 = cut the last wave's tiles along K whenever that wave is partly filled
 * (also where the model expects no gain), 0 = never, -1 = back to the model's decision. */
int o64_test_force_tail_split(int mode);

/* One-thread-per-output reference kernels: an independent device implementation of the same
 * contracts, used to compare full matrices where a CPU check would take minutes.
 * out_f32: fp32 result [M,N] (s32 for O64_KIND_S8).  For O64_KIND_FP8 the scales and bias
 * apply; for the others `bias`/`act` apply and the scales must be NULL. */
int o64_naive_gemm(o64_handle_t h, int kind, int64_t M, int64_t N, int64_t K, const void *A,
                   int64_t lda, const void *B, int64_t ldb, int transB, const float *scaleA,
                   const float *scaleB, const float *bias, int act, void *out, int64_t ldo,
                   void *stream);

/* ---- multi-GPU: output columns sharded over the ranks of one node ----------------------
 * Rank r of g owns B[r*N/g : (r+1)*N/g, :] and produces C[:, r*N/g : (r+1)*N/g]; no
 * reduction.  The only exchange is an all-gather of the column slabs when every rank wants
 * the whole C. */
#define O64_UNIQUE_ID_BYTES 128
/* Rank 0 creates the id, the caller distributes the bytes, every rank calls o64_comm_init. */
int o64_comm_unique_id(void *id_bytes);
int o64_comm_init(o64_handle_t h, const void *id_bytes, int rank, int nranks);
int o64_comm_destroy(o64_handle_t h);

enum {
    O64_GATHER_NONE = 0,      /* write only this rank's slab into C_full[:, r*N/g ...] */
    O64_GATHER_ROWMAJOR = 1,  /* all-gather, then permute into row-major C_full [M,N] */
    O64_GATHER_SLABS = 2,     /* all-gather only: C_full is [g][M][N/g] (slab-major) */
    O64_GATHER_PUSH = 3       /* fused: the GEMM kernel stores each finished tile into every rank's
                                 row-major C_full over NVLink peer memory and exchanges arrival
                                 counters with its peers itself: one launch, no separate collective.
                                 C_full must come from o64_comm_alloc_result; N/g a multiple of 32 */
};
/* Ordering of O64_GATHER_PUSH: work queued on `stream` before the call on ANY
 * rank is complete before the first byte lands in that rank's C_full, and when the call's work
 * on `stream` is complete every rank's columns are in this rank's C_full.  All waits are bounded
 * by the handle's wait budget; after O64_ERR_TIMEOUT from such a call (a rank that never made
 * it) the ranks' counters may disagree: allocate the result again (o64_comm_alloc_result is
 * collective and starts them afresh). */
/* Allocates `bytes` of device memory on every rank (collective over the communicator) and maps
 * every rank's allocation into every other rank's address space; returns this rank's pointer.
 * The handle owns the memory (freed by o64_comm_destroy / o64_destroy / the next call). */
int o64_comm_alloc_result(o64_handle_t h, size_t bytes, void **local);
/* A [M,K] replicated, B_slab [N/g,K] local, C_full [M,N] int32 (ldc = N) on every rank.
 * workspace: device scratch of at least o64_gemm_s8_sharded_workspace(...) bytes, or NULL to
 * let the handle grow its own. */
size_t o64_gemm_s8_sharded_workspace(int64_t M, int64_t N, int nranks, int gather);
int o64_gemm_s8_sharded(o64_handle_t h, int64_t M, int64_t N, int64_t K, const int8_t *A,
                        int64_t lda, const int8_t *B_slab, int64_t ldb, int32_t *C_full,
                        int gather, void *workspace, void *stream);

/* The same column-sharded linear for bf16 (C = act(A * B^T + bias), fp32 accumulate, bf16 result):
 * A [M,K] replicated, B_slab [N/g,K] local, bias (epilogue->bias, or NULL) the full vector of N
 * values on every rank.  gather: O64_GATHER_NONE (this rank's columns of the row-major C_full),
 * O64_GATHER_SLABS (slab-major [g][M][N/g], NCCL all-gather in place) or O64_GATHER_PUSH (fused,
 * row-major on every rank; C_full from o64_comm_alloc_result; N/g a multiple of 64). */
int o64_gemm_bf16_sharded(o64_handle_t h, int64_t M, int64_t N, int64_t K, const void *A, int64_t lda,
                          const void *B_slab, int64_t ldb, void *C_full, int gather,
                          const o64_epilogue_t *epilogue, void *stream);

/* ---- compat layer (Fortran ABI) -------------------------------------------------------- */
/* Column-major BLAS sgemm: C = alpha*op(A)*op(B) + beta*C. */
void sgemm_(const char *transa, const char *transb, const int *m, const int *n, const int *k,
            const float *alpha, const float *a, const int *lda, const float *b, const int *ldb,
            const float *beta, float *c, const int *ldc);
/* C = alpha*A*B + beta*C, element (i,j) of X at X[inc1x*i + inc2x*j]; quick returns and the
 * skip of zero B(l,j) follow osprey/libfi/matrix/xgemmx.h:172-236. */
void _s4gemmx__(const int *m, const int *n, const int *k, const float *alpha, const float *a,
                const int *inc1a, const int *inc2a, const float *b, const int *inc1b,
                const int *inc2b, const float *beta, float *c, const int *inc1c,
                const int *inc2c);
/* y = alpha*A*x + beta*y (osprey/libfi/matrix/s4gemvx.f). */
void _s4gemvx__(const int *m, const int *n, const float *alpha, const float *a,
                const int *incca, const int *incra, const float *x, const int *incx,
                const float *beta, float *y, const int *incy);
/* The operator entry point the reference's Fortran front end emits for MATMUL on REAL*4 operands
 * (osprey/libfi/matrix/matmul_s4s4.c:66-112; argument parsing osprey/libfi/matrix/matmul.h:135-400).
 * o64_dopevec_t is the x86-64 little-endian layout of DopeVectorType
 * (osprey/clibinc/cray/dopevec.h:212-334) with the bit-fields written out as words:
 *   flags0: bit 0 assoc, bit 1 ptr_alloc, bits 2-3 p_or_a, bit 4 a_contig, bit 5 alloc_cpnt
 *   flags1: bits 29-31 n_dim
 *   type_bits: bits 0-7 type (3 = REAL), bit 8 dpflag, bits 9-11 kind_or_star, bits 12-23 int_len
 *              (element length in bits), bits 24-31 dec_len
 * stride_mult is in elements for 32-bit elements.  As in the reference: rank combinations other
 * than (2,2), (2,1), (1,2) are an error (FESCIRNK), extents must conform (FESCICNF), and a RESULT
 * that is not associated is allocated with malloc and handed to the caller (FENOMEMY on failure);
 * unlike the reference nothing aborts: the code is left in o64_compat_last_status(). */
typedef struct {
    void *ptr;             /* base address (host or device) */
    unsigned long el_len;  /* element length in bits */
    uint32_t flags0, flags1;
    uint32_t type_pad, type_bits;
    void *orig_base;
    unsigned long orig_size;
    struct {
        long low_bound, extent, stride_mult;
    } dimension[7];
} o64_dopevec_t;
/* the sizes and offsets the reference's compiler gives DopeVectorType on x86-64 */
#if defined(__cplusplus)
static_assert(sizeof(o64_dopevec_t) == 216 && offsetof(o64_dopevec_t, flags0) == 16 &&
                  offsetof(o64_dopevec_t, type_bits) == 28 && offsetof(o64_dopevec_t, orig_base) == 32 &&
                  offsetof(o64_dopevec_t, dimension) == 48,
              "o64_dopevec_t does not match DopeVectorType");
#elif defined(__STDC_VERSION__) && __STDC_VERSION__ >= 201112L
_Static_assert(sizeof(o64_dopevec_t) == 216 && offsetof(o64_dopevec_t, flags0) == 16 &&
                   offsetof(o64_dopevec_t, type_bits) == 28 && offsetof(o64_dopevec_t, orig_base) == 32 &&
                   offsetof(o64_dopevec_t, dimension) == 48,
               "o64_dopevec_t does not match DopeVectorType");
#endif
void _MATMUL_S4S4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);

/* ---- the same family for REAL*8 and the integer kinds ------------------------------------
 * Exact arithmetic of the element kind on CUDA cores (fp64 FMA; integers wrap in the kind of C
 * as the Fortran kernels do), same quick returns and increments as the REAL*4 entry points.
 * For 64-bit elements the dope vector's stride_mult counts 32-bit words (matmul.h:145-176); for
 * 8-, 16- and 32-bit elements it counts elements. */
/* BLAS hook for REAL*8 MATMUL (osprey/libfi/matrix/MATMUL_SSdispatch.c:43, mmx_dlutil.c:46,133). */
void dgemm_(const char *transa, const char *transb, const int *m, const int *n, const int *k,
            const double *alpha, const double *a, const int *lda, const double *b, const int *ldb,
            const double *beta, double *c, const int *ldc);
/* osprey/libfi/matrix/sgemmx.f (REAL(KIND=8); call site matmul_ss@.c:120-122). */
void _sgemmx__(const int *m, const int *n, const int *k, const double *alpha, const double *a,
               const int *inc1a, const int *inc2a, const double *b, const int *inc1b,
               const int *inc2b, const double *beta, double *c, const int *inc1c, const int *inc2c);
/* osprey/libfi/matrix/sgemvx.f (call sites matmul_ss@.c:104-114). */
void _sgemvx__(const int *m, const int *n, const double *alpha, const double *a, const int *incca,
               const int *incra, const double *x, const int *incx, const double *beta, double *y,
               const int *incy);
/* The integer instances of the template osprey/libfi/matrix/xgemmx.h: i1gemmx.f, i2gemmx.f,
 * i4gemmx.f, jgemmx.f (one kind throughout) and i1i2gemmx.f, i1i4gemmx.f, i1jgemmx.f, i2i4gemmx.f,
 * i2jgemmx.f, i4jgemmx.f (A of the narrower kind; B, C, alpha and beta of the wider one). */
void _i1gemmx__(const int *m, const int *n, const int *k, const int8_t *alpha, const int8_t *a,
                const int *inc1a, const int *inc2a, const int8_t *b, const int *inc1b, const int *inc2b,
                const int8_t *beta, int8_t *c, const int *inc1c, const int *inc2c);
void _i1i2gemmx__(const int *m, const int *n, const int *k, const int16_t *alpha, const int8_t *a,
                  const int *inc1a, const int *inc2a, const int16_t *b, const int *inc1b, const int *inc2b,
                  const int16_t *beta, int16_t *c, const int *inc1c, const int *inc2c);
void _i1i4gemmx__(const int *m, const int *n, const int *k, const int32_t *alpha, const int8_t *a,
                  const int *inc1a, const int *inc2a, const int32_t *b, const int *inc1b, const int *inc2b,
                  const int32_t *beta, int32_t *c, const int *inc1c, const int *inc2c);
void _i1jgemmx__(const int *m, const int *n, const int *k, const int64_t *alpha, const int8_t *a,
                 const int *inc1a, const int *inc2a, const int64_t *b, const int *inc1b, const int *inc2b,
                 const int64_t *beta, int64_t *c, const int *inc1c, const int *inc2c);
void _i2gemmx__(const int *m, const int *n, const int *k, const int16_t *alpha, const int16_t *a,
                const int *inc1a, const int *inc2a, const int16_t *b, const int *inc1b, const int *inc2b,
                const int16_t *beta, int16_t *c, const int *inc1c, const int *inc2c);
void _i2i4gemmx__(const int *m, const int *n, const int *k, const int32_t *alpha, const int16_t *a,
                  const int *inc1a, const int *inc2a, const int32_t *b, const int *inc1b, const int *inc2b,
                  const int32_t *beta, int32_t *c, const int *inc1c, const int *inc2c);
void _i2jgemmx__(const int *m, const int *n, const int *k, const int64_t *alpha, const int16_t *a,
                 const int *inc1a, const int *inc2a, const int64_t *b, const int *inc1b, const int *inc2b,
                 const int64_t *beta, int64_t *c, const int *inc1c, const int *inc2c);
void _i4gemmx__(const int *m, const int *n, const int *k, const int32_t *alpha, const int32_t *a,
                const int *inc1a, const int *inc2a, const int32_t *b, const int *inc1b, const int *inc2b,
                const int32_t *beta, int32_t *c, const int *inc1c, const int *inc2c);
void _i4jgemmx__(const int *m, const int *n, const int *k, const int64_t *alpha, const int32_t *a,
                 const int *inc1a, const int *inc2a, const int64_t *b, const int *inc1b, const int *inc2b,
                 const int64_t *beta, int64_t *c, const int *inc1c, const int *inc2c);
void _jgemmx__(const int *m, const int *n, const int *k, const int64_t *alpha, const int64_t *a,
               const int *inc1a, const int *inc2a, const int64_t *b, const int *inc1b, const int *inc2b,
               const int64_t *beta, int64_t *c, const int *inc1c, const int *inc2c);
/* The mixed instances with a REAL result (s4sgemmx.f; i1s4gemmx.f ... js4gemmx.f; i1sgemmx.f ... jsgemmx.f):
 * A of the narrower real or of an integer kind, converted to the kind of B, C, alpha and beta. */
void _s4sgemmx__(const int *m, const int *n, const int *k, const double *alpha, const float *a,
                 const int *inc1a, const int *inc2a, const double *b, const int *inc1b, const int *inc2b,
                 const double *beta, double *c, const int *inc1c, const int *inc2c);
void _i1s4gemmx__(const int *m, const int *n, const int *k, const float *alpha, const int8_t *a,
                  const int *inc1a, const int *inc2a, const float *b, const int *inc1b, const int *inc2b,
                  const float *beta, float *c, const int *inc1c, const int *inc2c);
void _i2s4gemmx__(const int *m, const int *n, const int *k, const float *alpha, const int16_t *a,
                  const int *inc1a, const int *inc2a, const float *b, const int *inc1b, const int *inc2b,
                  const float *beta, float *c, const int *inc1c, const int *inc2c);
void _i4s4gemmx__(const int *m, const int *n, const int *k, const float *alpha, const int32_t *a,
                  const int *inc1a, const int *inc2a, const float *b, const int *inc1b, const int *inc2b,
                  const float *beta, float *c, const int *inc1c, const int *inc2c);
void _js4gemmx__(const int *m, const int *n, const int *k, const float *alpha, const int64_t *a,
                 const int *inc1a, const int *inc2a, const float *b, const int *inc1b, const int *inc2b,
                 const float *beta, float *c, const int *inc1c, const int *inc2c);
void _i1sgemmx__(const int *m, const int *n, const int *k, const double *alpha, const int8_t *a,
                 const int *inc1a, const int *inc2a, const double *b, const int *inc1b, const int *inc2b,
                 const double *beta, double *c, const int *inc1c, const int *inc2c);
void _i2sgemmx__(const int *m, const int *n, const int *k, const double *alpha, const int16_t *a,
                 const int *inc1a, const int *inc2a, const double *b, const int *inc1b, const int *inc2b,
                 const double *beta, double *c, const int *inc1c, const int *inc2c);
void _i4sgemmx__(const int *m, const int *n, const int *k, const double *alpha, const int32_t *a,
                 const int *inc1a, const int *inc2a, const double *b, const int *inc1b, const int *inc2b,
                 const double *beta, double *c, const int *inc1c, const int *inc2c);
void _jsgemmx__(const int *m, const int *n, const int *k, const double *alpha, const int64_t *a,
                const int *inc1a, const int *inc2a, const double *b, const int *inc1b, const int *inc2b,
                const double *beta, double *c, const int *inc1c, const int *inc2c);
/* MATMUL on REAL*8 arrays (matmul_ss@.c:78-125) and on every pair of integer kinds
 * (matmul_i1i1.c ... matmul_jj@.c; result kind = the wider operand kind).  The integer entry
 * points send rank-1 operands through the matrix kernel with (m,n,k) = (n1a,1,n2a) or
 * (1,n2b,n1b) (matmul.h:343-363, matmul_i4i4.c:84-86); when MATRIX_A is the wider kind they form
 * C' = B'A' with exchanged increments (matmul_i2i1.c:82-84, matmul_i4i1.c:83-85). */
void _MATMUL_SS(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I1I1(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I1I2(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I1I4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I1J(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I2I1(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I2I2(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I2I4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I2J(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I4I1(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I4I2(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I4I4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I4J(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_JI1(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_JI2(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_JI4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_JJ(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
/* MATMUL of a REAL*4 by a REAL*8 array and of integer by real arrays, either way round (matmul_s4s.c,
 * matmul_ss4.c, matmul_i4s4.c, matmul_s4i4.c, ...): result of the real (wider) kind; when MATRIX_B is the
 * integer or narrower operand the product is formed as C' = B'A' (matmul_ss4.c:87-89, matmul_s4i4.c:85-87). */
void _MATMUL_S4S(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_SS4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I1S4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_S4I1(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I1S(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_SI1(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I2S4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_S4I2(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I2S(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_SI2(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I4S4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_S4I4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I4S(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_SI4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_JS4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_S4J(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_JS(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_SJ(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);

/* ---- COMPLEX*8 and COMPLEX*16 ------------------------------------------------------------
 * Complex values are (re, im) pairs of floats / doubles, increments count complex elements, and
 * the kernels take conjugation flags in front (0 = as is, 1 = conjugate), as
 * osprey/libfi/matrix/c4gemmx.f:37-85, cgemmx.f, c4gemvx.f and cgemvx.f do.  Unlike the real and
 * integer kernels the matrix kernel has no test for zero elements of B (c4gemmx.f:199-212). */
void _c4gemmx__(const int *iconja, const int *iconjb, const int *m, const int *n, const int *k,
                const float *alpha, const float *a, const int *inc1a, const int *inc2a, const float *b,
                const int *inc1b, const int *inc2b, const float *beta, float *c, const int *inc1c,
                const int *inc2c);
void _cgemmx__(const int *iconja, const int *iconjb, const int *m, const int *n, const int *k,
               const double *alpha, const double *a, const int *inc1a, const int *inc2a, const double *b,
               const int *inc1b, const int *inc2b, const double *beta, double *c, const int *inc1c,
               const int *inc2c);
void _c4gemvx__(const int *iconj, const int *m, const int *n, const float *alpha, const float *a,
                const int *incca, const int *incra, const float *x, const int *incx, const float *beta,
                float *y, const int *incy);
void _cgemvx__(const int *iconj, const int *m, const int *n, const double *alpha, const double *a,
               const int *incca, const int *incra, const double *x, const int *incx, const double *beta,
               double *y, const int *incy);
/* BLAS hooks for complex MATMUL (mmx_dlutil.c:135-136); trans 'c' is the conjugate transpose. */
void cgemm_(const char *transa, const char *transb, const int *m, const int *n, const int *k,
            const float *alpha, const float *a, const int *lda, const float *b, const int *ldb,
            const float *beta, float *c, const int *ldc);
void zgemm_(const char *transa, const char *transb, const int *m, const int *n, const int *k,
            const double *alpha, const double *a, const int *lda, const double *b, const int *ldb,
            const double *beta, double *c, const int *ldc);
/* MATMUL on COMPLEX*8 (matmul_c4c4.c:76-134) and COMPLEX*16 (matmul_cc@.c) arrays; rank-1 operands go
 * to the matrix-vector kernels, nothing is conjugated. */
void _MATMUL_C4C4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_CC(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);

/* COMPLEX with a REAL or INTEGER operand, or with COMPLEX of the other width: the 26 entry points
 * osprey/libfi/matrix/matmul_c4s4.c, matmul_s4c4.c, matmul_c4i1.c ... matmul_jc@.c, matmul_c4c.c and
 * matmul_cc4.c.  The result is COMPLEX*8 when both operands are 4 bytes per component or INTEGER
 * with COMPLEX*8, COMPLEX*16 otherwise.  As in the reference the real and imaginary parts are
 * separate products of the REAL kernel for the pair of component kinds (_s4gemmx__, _s4sgemmx__,
 * _sgemmx__, _i1s4gemmx__ ... _jsgemmx__) with the increments of the COMPLEX arrays doubled; four
 * products when both operands are COMPLEX (matmul_c4c.c:88-128). */
void _MATMUL_C4S4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_S4C4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_C4S(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_SC4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_CS4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_S4C(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_CS(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_SC(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_C4C(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_CC4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_C4I1(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_C4I2(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_C4I4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_C4J(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I1C4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I2C4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I4C4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_JC4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_CI1(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_CI2(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_CI4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_CJ(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I1C(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I2C(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_I4C(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_JC(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);

/* ---- LOGICAL kinds ------------------------------------------------------------------------
 * C(i,j) = (beta .AND. C(i,j)) .OR. (alpha .AND. OR over l of A(i,l) .AND. B(l,j)), the template
 * osprey/libfi/matrix/lgemmx.h instantiated by l1gemmx.f, l1l2gemmx.f, ... lgemmx.f: A of the same or
 * a narrower kind than B, C, alpha and beta; 1-, 2-, 4- and 8-byte logicals are carried as integers of
 * that width, any non-zero value is true, results are 1 or 0.  K == 0 clears C. */
void _l1gemmx__(const int *m, const int *n, const int *k, const int8_t *alpha, const int8_t *a,
                const int *inc1a, const int *inc2a, const int8_t *b, const int *inc1b, const int *inc2b,
                const int8_t *beta, int8_t *c, const int *inc1c, const int *inc2c);
void _l1l2gemmx__(const int *m, const int *n, const int *k, const int16_t *alpha, const int8_t *a,
                  const int *inc1a, const int *inc2a, const int16_t *b, const int *inc1b, const int *inc2b,
                  const int16_t *beta, int16_t *c, const int *inc1c, const int *inc2c);
void _l1l4gemmx__(const int *m, const int *n, const int *k, const int32_t *alpha, const int8_t *a,
                  const int *inc1a, const int *inc2a, const int32_t *b, const int *inc1b, const int *inc2b,
                  const int32_t *beta, int32_t *c, const int *inc1c, const int *inc2c);
void _l1lgemmx__(const int *m, const int *n, const int *k, const int64_t *alpha, const int8_t *a,
                 const int *inc1a, const int *inc2a, const int64_t *b, const int *inc1b, const int *inc2b,
                 const int64_t *beta, int64_t *c, const int *inc1c, const int *inc2c);
void _l2gemmx__(const int *m, const int *n, const int *k, const int16_t *alpha, const int16_t *a,
                const int *inc1a, const int *inc2a, const int16_t *b, const int *inc1b, const int *inc2b,
                const int16_t *beta, int16_t *c, const int *inc1c, const int *inc2c);
void _l2l4gemmx__(const int *m, const int *n, const int *k, const int32_t *alpha, const int16_t *a,
                  const int *inc1a, const int *inc2a, const int32_t *b, const int *inc1b, const int *inc2b,
                  const int32_t *beta, int32_t *c, const int *inc1c, const int *inc2c);
void _l2lgemmx__(const int *m, const int *n, const int *k, const int64_t *alpha, const int16_t *a,
                 const int *inc1a, const int *inc2a, const int64_t *b, const int *inc1b, const int *inc2b,
                 const int64_t *beta, int64_t *c, const int *inc1c, const int *inc2c);
void _l4gemmx__(const int *m, const int *n, const int *k, const int32_t *alpha, const int32_t *a,
                const int *inc1a, const int *inc2a, const int32_t *b, const int *inc1b, const int *inc2b,
                const int32_t *beta, int32_t *c, const int *inc1c, const int *inc2c);
void _l4lgemmx__(const int *m, const int *n, const int *k, const int64_t *alpha, const int32_t *a,
                 const int *inc1a, const int *inc2a, const int64_t *b, const int *inc1b, const int *inc2b,
                 const int64_t *beta, int64_t *c, const int *inc1c, const int *inc2c);
void _lgemmx__(const int *m, const int *n, const int *k, const int64_t *alpha, const int64_t *a,
               const int *inc1a, const int *inc2a, const int64_t *b, const int *inc1b, const int *inc2b,
               const int64_t *beta, int64_t *c, const int *inc1c, const int *inc2c);
/* MATMUL on LOGICAL arrays (matmul_l1l1.c ... matmul_ll@.c): alpha = .TRUE., beta = .FALSE.; the wider
 * operand first means C' = B'A' as for the integer kinds. */
void _MATMUL_L1L1(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_L1L2(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_L1L4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_L1L(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_L2L1(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_L2L2(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_L2L4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_L2L(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_L4L1(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_L4L2(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_L4L4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_L4L(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_LL1(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_LL2(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_LL4(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);
void _MATMUL_LL(o64_dopevec_t *RESULT, o64_dopevec_t *MATRIX_A, o64_dopevec_t *MATRIX_B);

/* ---- DOT_PRODUCT ------------------------------------------------------------------------------
 * MATMUL's rank-1 sibling in the same runtime: _DOT_<A><B>(VECTOR_A, VECTOR_B) over two rank-1 dope
 * vectors (osprey/libfi/dotprod/dot_s4s4.f ... dot_ll.f; argument parsing predot@.c:52-93; the sums
 * dot90.h:83-86, dotc90.h:84-87 - COMPLEX conjugates VECTOR_A -, dotl90.h:84-87 - LOGICAL is the .OR. of
 * the .AND.s).  The result has the wider (or the REAL) kind of the two; integers wrap; a LOGICAL result
 * is 1 or 0.  COMPLEX results come back as a (re, im) structure, which the x86-64 ABI returns in the
 * registers a C99 _Complex value uses.  The kinds with a REAL*16 / COMPLEX*32 operand and the Cray
 * default-integer names are not provided.  Errors are left in o64_compat_last_status() and give 0. */
typedef struct { float re, im; } o64_complex8_t;
typedef struct { double re, im; } o64_complex16_t;
float _DOT_S4S4(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
double _DOT_SS(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
double _DOT_S4S(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
double _DOT_SS4(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
int32_t _DOT_I4I4(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
int64_t _DOT_JJ(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
int64_t _DOT_I4J(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
int64_t _DOT_JI4(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
float _DOT_I4S4(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
float _DOT_S4I4(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
double _DOT_I4S(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
double _DOT_SI4(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
float _DOT_JS4(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
float _DOT_S4J(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
double _DOT_JS(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
double _DOT_SJ(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
int32_t _DOT_L4L4(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
int64_t _DOT_LL(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
int64_t _DOT_L4L(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
int64_t _DOT_LL4(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
o64_complex8_t _DOT_C4C4(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);
o64_complex16_t _DOT_CC(const o64_dopevec_t *VECTOR_A, const o64_dopevec_t *VECTOR_B);

/* The handle behind the Fortran-ABI entry points (one per process, on the device current at the first
 * call; created here if need be; NULL without a usable GPU): for o64_plan_set / o64_set_wait_budget_us /
 * o64_last_status on the calls that take no handle.  Do not destroy it. */
o64_handle_t o64_compat_handle(void);
/* Status of the last compat call on this thread (the Fortran entry points return void). */
int o64_compat_last_status(void);

#ifdef __cplusplus
}
#endif
#endif /* O64GEMM_H */
