/*
 * What the reference's C front half of MATMUL needs around it in order to run in a test
 * process.  TEST INFRASTRUCTURE ONLY: built by ref_front.mk into oracle/_ref/ together with the
 * reference's own, unmodified C sources (osprey/libfi/matrix/matmul_*.c, MATMUL_*dispatch.c,
 * mmx_dlutil.c, compiled where they lie); the shipped library never links or loads it.
 *
 *   _lerror              the runtime's abort routine (osprey/clibinc/liberrno.h:127).  The real one
 *                        prints and ends the process; this one records the code and jumps back to
 *                        o64front_call, which returns it.
 *   o64front_call        calls one MATMUL entry point of the reference under that guard.
 *   o64front_dv_probe    sets one field of a real DopeVectorType (osprey/clibinc/cray/dopevec.h:212-334)
 *                        and hands back its bytes, so that a test can hold the engine's plain-word
 *                        view of the structure against the compiler's own bit-field layout.
 *   _MM_ / _MV_ / _VM_MATMUL_<A><B>
 *                        the three Fortran subroutines each MATMUL_<A><B>.F90 is compiled to
 *                        (template osprey/libfi/matrix/mmx_fort.h:38-229), restated in C because no
 *                        Fortran compiler exists here: allocate R, copy an operand whose kind differs
 *                        from the result's (CONVERTT1 / CONVERTT2), then either call the BLAS routine
 *                        the reference's mmx_dlutil.c resolved, as
 *                        ('n','n',m,k,n,alpha,A,m,B,n,beta,R,m) (mmx_fort.h:94-95), or run the
 *                        dot-product loops j > i > kk (mmx_fort.h:102-116).  Operands arrive as
 *                        assumed-shape arrays, i.e. dope vectors; a strided one is made contiguous
 *                        before the BLAS call, as a Fortran compiler's copy-in does.
 */
#include <complex.h>
#include <setjmp.h>
#include <stdlib.h>
#include <string.h>

#include <cray/dopevec.h>
#include <liberrno.h>

/* ---- the abort routine, made returnable -------------------------------------------------- */
static __thread jmp_buf *g_jump = NULL;
static __thread int g_code = 0;

void _lerror(int level, int code, ...) {
    (void)level;
    g_code = code;
    if (g_jump) longjmp(*g_jump, 1);
    abort(); /* outside o64front_call: behave like the runtime */
}

int o64front_call(void (*entry)(DopeVectorType *, DopeVectorType *, DopeVectorType *), DopeVectorType *R,
                  DopeVectorType *A, DopeVectorType *B) {
    jmp_buf jb;
    g_code = 0;
    g_jump = &jb;
    if (setjmp(jb) == 0) entry(R, A, B);
    g_jump = NULL;
    return g_code;
}

int o64front_code(int which) { return which == 0 ? FESCIRNK : (which == 1 ? FESCICNF : FENOMEMY); }

/* ---- layout of the real dope vector -------------------------------------------------------- */
long o64front_dv_sizeof(void) { return (long)sizeof(DopeVectorType); }

/* which: 0 assoc, 1 ptr_alloc, 2 p_or_a (all ones), 3 a_contig, 4 n_dim (all ones), 5 type (all ones),
 * 6 dpflag, 7 kind_or_star (all ones), 8 int_len (all ones), 9 dec_len (all ones), 10 base pointer,
 * 11 el_len, 12 orig_base, 13 orig_size, 14 dimension[1].low_bound, 15 dimension[1].extent,
 * 16 dimension[1].stride_mult, 17 dimension[6].stride_mult.  Returns 0, or -1 for an unknown field. */
int o64front_dv_probe(int which, unsigned char *out) {
    DopeVectorType d;
    memset(&d, 0, sizeof(d));
    switch (which) {
    case 0: d.assoc = 1; break;
    case 1: d.ptr_alloc = 1; break;
    case 2: d.p_or_a = 3; break;
    case 3: d.a_contig = 1; break;
    case 4: d.n_dim = 7; break;
    case 5: d.type_lens.type = 0xff; break;
    case 6: d.type_lens.dpflag = 1; break;
    case 7: d.type_lens.kind_or_star = 7; break;
    case 8: d.type_lens.int_len = 0xfff; break;
    case 9: d.type_lens.dec_len = 0xff; break;
    case 10: d.base_addr.a.ptr = (void *)~0ul; break;
    case 11: d.base_addr.a.el_len = ~0ul; break;
    case 12: d.orig_base = (void *)~0ul; break;
    case 13: d.orig_size = ~0ul; break;
    case 14: d.dimension[1].low_bound = -1; break;
    case 15: d.dimension[1].extent = -1; break;
    case 16: d.dimension[1].stride_mult = -1; break;
    case 17: d.dimension[6].stride_mult = -1; break;
    default: return -1;
    }
    memcpy(out, &d, sizeof(d));
    return 0;
}

/* ---- MATMUL_<A><B>.F90 in C ------------------------------------------------------------------ */
typedef float _Complex c4_t;
typedef double _Complex c8_t;

typedef void (*blas_fn)(const char *, const char *, const int *, const int *, const int *, const void *,
                        const void *, const int *, const void *, const int *, const void *, void *,
                        const int *, int, int);

/* stride of dimension d in elements: stride_mult counts 32-bit words for elements of 64 bits and
 * more (osprey/libfi/matrix/matmul.h:145-176 divides the same way) */
static long elem_stride(const DopeVectorType *v, int d) {
    long s = v->dimension[d].stride_mult;
    const unsigned len = v->type_lens.int_len;
    if (len >= 64) s /= (long)(len / 32);
    return s;
}

/* `allocate(R(...))` on a Fortran pointer: fresh contiguous storage, dope vector filled in */
static void *allocate_result(DopeVectorType *R, int rank, long n1, long n2, size_t elem_bytes) {
    const long words = (long)(elem_bytes >= 8 ? elem_bytes / 4 : 1);
    const long count = n1 * (rank == 2 ? n2 : 1);
    void *mem = malloc(count > 0 ? (size_t)count * elem_bytes : 1);
    if (!mem) {
        _lerror(_LELVL_ABORT, FENOMEMY);
        return NULL;
    }
    R->base_addr.a.ptr = mem;
    R->base_addr.a.el_len = elem_bytes * 8;
    R->assoc = 1;
    R->ptr_alloc = 1;
    R->p_or_a = POINTTR;
    R->a_contig = 1;
    R->n_dim = rank;
    R->orig_base = mem;
    R->orig_size = (unsigned long)count * elem_bytes * 8;
    R->dimension[0].low_bound = 1;
    R->dimension[0].extent = n1;
    R->dimension[0].stride_mult = words;
    if (rank == 2) {
        R->dimension[1].low_bound = 1;
        R->dimension[1].extent = n2;
        R->dimension[1].stride_mult = words * n1;
    }
    return mem;
}

extern void _F90_MMULT_ERROR(void);

#define O64FRONT_MATMUL(SUFFIX, T1, T2, T3)                                                               \
    void _MM_MATMUL_##SUFFIX(DopeVectorType *r, DopeVectorType *a, DopeVectorType *b, void *blasroutine) { \
        const int m = (int)a->dimension[0].extent, n = (int)a->dimension[1].extent;                       \
        const int k = (int)b->dimension[1].extent, n1 = (int)b->dimension[0].extent;                      \
        if (n1 != n) _F90_MMULT_ERROR();                                                                  \
        T3 *R = (T3 *)allocate_result(r, 2, m, k, sizeof(T3));                                            \
        if (!R) return;                                                                                   \
        if (m == 0 || n == 0 || k == 0) {                                                                 \
            for (long i = 0; i < (long)m * k; ++i) R[i] = 0;                                              \
            return;                                                                                       \
        }                                                                                                 \
        const T1 *A = (const T1 *)a->base_addr.a.ptr;                                                     \
        const T2 *B = (const T2 *)b->base_addr.a.ptr;                                                     \
        const long a1 = elem_stride(a, 0), a2 = elem_stride(a, 1);                                        \
        const long b1 = elem_stride(b, 0), b2 = elem_stride(b, 1);                                        \
        T3 *AA = (T3 *)malloc((size_t)m * n * sizeof(T3));                                                \
        T3 *BB = (T3 *)malloc((size_t)n * k * sizeof(T3));                                                \
        if (!AA || !BB) {                                                                                 \
            free(AA);                                                                                     \
            free(BB);                                                                                     \
            _lerror(_LELVL_ABORT, FENOMEMY);                                                              \
            return;                                                                                       \
        }                                                                                                 \
        for (long j = 0; j < n; ++j)                                                                      \
            for (long i = 0; i < m; ++i) AA[i + j * (long)m] = (T3)A[i * a1 + j * a2];                    \
        for (long j = 0; j < k; ++j)                                                                      \
            for (long i = 0; i < n; ++i) BB[i + j * (long)n] = (T3)B[i * b1 + j * b2];                    \
        if (blasroutine) {                                                                                \
            const T3 alpha = 1, beta = 0;                                                                 \
            ((blas_fn)blasroutine)("n", "n", &m, &k, &n, &alpha, AA, &m, BB, &n, &beta, R, &m, 1, 1);     \
        } else {                                                                                          \
            for (long i = 0; i < (long)m * k; ++i) R[i] = 0;                                              \
            for (long j = 0; j < k; ++j)                                                                  \
                for (long i = 0; i < m; ++i)                                                              \
                    for (long kk = 0; kk < n; ++kk)                                                       \
                        R[i + j * (long)m] = R[i + j * (long)m] + AA[i + kk * (long)m] * BB[kk + j * (long)n]; \
        }                                                                                                 \
        free(AA);                                                                                         \
        free(BB);                                                                                         \
    }                                                                                                     \
    void _MV_MATMUL_##SUFFIX(DopeVectorType *r, DopeVectorType *a, DopeVectorType *b) {                   \
        const int m = (int)a->dimension[0].extent, n = (int)a->dimension[1].extent;                       \
        const int n1 = (int)b->dimension[0].extent;                                                       \
        if (n1 != n) _F90_MMULT_ERROR();                                                                  \
        T3 *R = (T3 *)allocate_result(r, 1, m, 1, sizeof(T3));                                            \
        if (!R) return;                                                                                   \
        const T1 *A = (const T1 *)a->base_addr.a.ptr;                                                     \
        const T2 *B = (const T2 *)b->base_addr.a.ptr;                                                     \
        const long a1 = elem_stride(a, 0), a2 = elem_stride(a, 1), b1 = elem_stride(b, 0);                \
        for (long i = 0; i < m; ++i) {                                                                    \
            R[i] = 0;                                                                                     \
            for (long kk = 0; kk < n; ++kk) R[i] = R[i] + A[i * a1 + kk * a2] * (T3)B[kk * b1];           \
        }                                                                                                 \
    }                                                                                                     \
    void _VM_MATMUL_##SUFFIX(DopeVectorType *r, DopeVectorType *a, DopeVectorType *b) {                   \
        const int n = (int)a->dimension[0].extent, n1 = (int)b->dimension[0].extent;                      \
        const int m = (int)b->dimension[1].extent;                                                        \
        if (n1 != n) _F90_MMULT_ERROR();                                                                  \
        T3 *R = (T3 *)allocate_result(r, 1, m, 1, sizeof(T3));                                            \
        if (!R) return;                                                                                   \
        const T1 *A = (const T1 *)a->base_addr.a.ptr;                                                     \
        const T2 *B = (const T2 *)b->base_addr.a.ptr;                                                     \
        const long a1 = elem_stride(a, 0), b1 = elem_stride(b, 0), b2 = elem_stride(b, 1);                \
        for (long i = 0; i < m; ++i) {                                                                    \
            R[i] = 0;                                                                                     \
            for (long kk = 0; kk < n; ++kk) R[i] = R[i] + (T3)A[kk * a1] * B[kk * b1 + i * b2];           \
        }                                                                                                 \
    }

O64FRONT_MATMUL(S4S4, float, float, float)
O64FRONT_MATMUL(S4S, float, double, double)
O64FRONT_MATMUL(SS4, double, float, double)
O64FRONT_MATMUL(SS, double, double, double)
O64FRONT_MATMUL(C4C4, c4_t, c4_t, c4_t)
O64FRONT_MATMUL(C4C, c4_t, c8_t, c8_t)
O64FRONT_MATMUL(CC4, c8_t, c4_t, c8_t)
O64FRONT_MATMUL(CC, c8_t, c8_t, c8_t)
O64FRONT_MATMUL(C4S4, c4_t, float, c4_t)
O64FRONT_MATMUL(S4C4, float, c4_t, c4_t)
O64FRONT_MATMUL(C4S, c4_t, double, c8_t)
O64FRONT_MATMUL(SC4, double, c4_t, c8_t)
O64FRONT_MATMUL(CS4, c8_t, float, c8_t)
O64FRONT_MATMUL(S4C, float, c8_t, c8_t)
O64FRONT_MATMUL(CS, c8_t, double, c8_t)
O64FRONT_MATMUL(SC, double, c8_t, c8_t)
