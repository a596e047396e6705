/*
 * The Fortran-ABI names of the runtime's strided kernels (_s4gemmx__, _i1i4gemmx__, _lgemmx__,
 * _c4gemvx__, ...: every scalar by reference, osprey/libfi/matrix/xgemmx.h:49-53, call sites
 * matmul_s4s4.c:91-109) forwarded to the CPU oracle's restatements in gemm_ref.c.
 *
 * TEST INFRASTRUCTURE ONLY.  Linked with the reference's own C wrappers into
 * oracle/_ref/libfi_front_oracle.so, it gives a CPU-only MATMUL whose front half (dope-vector
 * parsing, RESULT allocation, conformance checks, operand exchange for mixed kinds) is the
 * reference's code and whose arithmetic is the oracle's.  The shipped library never sees it.
 */
#include <stdint.h>

#define XIFACE(NAME, ORACLE, TA, T)                                                                       \
    extern void ORACLE(int, int, int, T, const TA *, int, int, const T *, int, int, T, T *, int, int);    \
    void NAME(const int *m, const int *n, const int *k, const T *alpha, const TA *a, const int *inc1a,    \
              const int *inc2a, const T *b, const int *inc1b, const int *inc2b, const T *beta, T *c,      \
              const int *inc1c, const int *inc2c) {                                                       \
        ORACLE(*m, *n, *k, *alpha, a, *inc1a, *inc2a, b, *inc1b, *inc2b, *beta, c, *inc1c, *inc2c);       \
    }

XIFACE(_s4gemmx__, o64ref_s4gemmx, float, float)
XIFACE(_sgemmx__, o64ref_sgemmx_f64, double, double)
XIFACE(_s4sgemmx__, o64ref_s4sgemmx, float, double)
XIFACE(_i1s4gemmx__, o64ref_i1s4gemmx, int8_t, float)
XIFACE(_i2s4gemmx__, o64ref_i2s4gemmx, int16_t, float)
XIFACE(_i4s4gemmx__, o64ref_i4s4gemmx, int32_t, float)
XIFACE(_js4gemmx__, o64ref_js4gemmx, int64_t, float)
XIFACE(_i1sgemmx__, o64ref_i1sgemmx, int8_t, double)
XIFACE(_i2sgemmx__, o64ref_i2sgemmx, int16_t, double)
XIFACE(_i4sgemmx__, o64ref_i4sgemmx, int32_t, double)
XIFACE(_jsgemmx__, o64ref_jsgemmx, int64_t, double)
/* the oracle carries integers on the unsigned twin of the result kind (wrap-around is then defined) */
XIFACE(_i1gemmx__, o64ref_i1gemmx, int8_t, uint8_t)
XIFACE(_i1i2gemmx__, o64ref_i1i2gemmx, int8_t, uint16_t)
XIFACE(_i1i4gemmx__, o64ref_i1i4gemmx, int8_t, uint32_t)
XIFACE(_i1jgemmx__, o64ref_i1jgemmx, int8_t, uint64_t)
XIFACE(_i2gemmx__, o64ref_i2gemmx, int16_t, uint16_t)
XIFACE(_i2i4gemmx__, o64ref_i2i4gemmx, int16_t, uint32_t)
XIFACE(_i2jgemmx__, o64ref_i2jgemmx, int16_t, uint64_t)
XIFACE(_i4gemmx__, o64ref_i4gemmx, int32_t, uint32_t)
XIFACE(_i4jgemmx__, o64ref_i4jgemmx, int32_t, uint64_t)
XIFACE(_jgemmx__, o64ref_jgemmx, int64_t, uint64_t)
#undef XIFACE

/* LOGICAL kinds: alpha and beta are logicals of the result kind (lgemmx.h); the oracle takes ints */
#define LIFACE(NAME, ORACLE, TA, T)                                                                       \
    extern void ORACLE(int, int, int, int, const TA *, int, int, const T *, int, int, int, T *, int, int); \
    void NAME(const int *m, const int *n, const int *k, const T *alpha, const TA *a, const int *inc1a,    \
              const int *inc2a, const T *b, const int *inc1b, const int *inc2b, const T *beta, T *c,      \
              const int *inc1c, const int *inc2c) {                                                       \
        ORACLE(*m, *n, *k, *alpha != 0, a, *inc1a, *inc2a, b, *inc1b, *inc2b, *beta != 0, c, *inc1c,      \
               *inc2c);                                                                                   \
    }
LIFACE(_l1gemmx__, o64ref_l1gemmx, int8_t, int8_t)
LIFACE(_l1l2gemmx__, o64ref_l1l2gemmx, int8_t, int16_t)
LIFACE(_l1l4gemmx__, o64ref_l1l4gemmx, int8_t, int32_t)
LIFACE(_l1lgemmx__, o64ref_l1lgemmx, int8_t, int64_t)
LIFACE(_l2gemmx__, o64ref_l2gemmx, int16_t, int16_t)
LIFACE(_l2l4gemmx__, o64ref_l2l4gemmx, int16_t, int32_t)
LIFACE(_l2lgemmx__, o64ref_l2lgemmx, int16_t, int64_t)
LIFACE(_l4gemmx__, o64ref_l4gemmx, int32_t, int32_t)
LIFACE(_l4lgemmx__, o64ref_l4lgemmx, int32_t, int64_t)
LIFACE(_lgemmx__, o64ref_lgemmx, int64_t, int64_t)
#undef LIFACE

/* matrix-vector kernels (s4gemvx.f, sgemvx.f) */
extern void o64ref_s4gemvx(int, int, float, const float *, int, int, const float *, int, float, float *, int);
extern void o64ref_sgemvx_f64(int, int, double, const double *, int, int, const double *, int, double, double *, int);
void _s4gemvx__(const int *m, const int *n, const float *alpha, const float *a, const int *incca, const int *incra,
                const float *x, const int *incx, const float *beta, float *y, const int *incy) {
    o64ref_s4gemvx(*m, *n, *alpha, a, *incca, *incra, x, *incx, *beta, y, *incy);
}
void _sgemvx__(const int *m, const int *n, const double *alpha, const double *a, const int *incca, const int *incra,
               const double *x, const int *incx, const double *beta, double *y, const int *incy) {
    o64ref_sgemvx_f64(*m, *n, *alpha, a, *incca, *incra, x, *incx, *beta, y, *incy);
}

/* complex kernels: conjugation flags in front (c4gemmx.f:37-85) */
#define CIFACE(NAME, NAMEV, ORACLE, ORACLEV, R)                                                           \
    extern void ORACLE(int, int, int, int, int, const R *, const R *, int, int, const R *, int, int, const R *, R *, \
                       int, int);                                                                         \
    extern void ORACLEV(int, int, int, const R *, const R *, int, int, const R *, int, const R *, R *, int); \
    void NAME(const int *ca, const int *cb, const int *m, const int *n, const int *k, const R *alpha, const R *a, \
              const int *inc1a, const int *inc2a, const R *b, const int *inc1b, const int *inc2b, const R *beta, \
              R *c, const int *inc1c, const int *inc2c) {                                                 \
        ORACLE(*ca, *cb, *m, *n, *k, alpha, a, *inc1a, *inc2a, b, *inc1b, *inc2b, beta, c, *inc1c, *inc2c); \
    }                                                                                                     \
    void NAMEV(const int *cj, const int *m, const int *n, const R *alpha, const R *a, const int *incca,   \
               const int *incra, const R *x, const int *incx, const R *beta, R *y, const int *incy) {     \
        ORACLEV(*cj, *m, *n, alpha, a, *incca, *incra, x, *incx, beta, y, *incy);                         \
    }
CIFACE(_c4gemmx__, _c4gemvx__, o64ref_c4gemmx, o64ref_c4gemvx, float)
CIFACE(_cgemmx__, _cgemvx__, o64ref_cgemmx, o64ref_cgemvx, double)
#undef CIFACE
