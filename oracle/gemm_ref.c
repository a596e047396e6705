/*
 * CPU oracle for the dense GEMM / fused-linear path.  TEST INFRASTRUCTURE ONLY:
 * the shipped library never links, loads or calls anything in this file; only
 * the tests, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * PARITY UNPINNED: the reference (open64-compiler/open64) holds no golden
 * vector, known-answer test or fixture for a matrix product, and its own
 * arithmetic kernels (libfi/matrix Fortran sources) cannot be compiled without a Fortran
 * compiler.  This file therefore restates the reference's algorithms from its sources:
 *
 *   - the loop nest the compiler builds for MATMUL
 *       osprey/be/vho/f90_lower.cxx:5149-5169   (lower_mm_matmul: accumulator
 *       zeroed, one loop over the inner extent in ascending order,
 *       acc = acc + a*b with a separate multiply and add)
 *   - the strided alpha/beta runtime kernel
 *       osprey/libfi/matrix/xgemmx.h:172-236    (quick returns, loop order
 *       J > L > I, axpy skipped when B(L,J) == 0)
 *       osprey/libfi/matrix/s4gemmx.f:151-196   (the REAL*4 instance)
 *   - the dot-product form used behind the BLAS hook
 *       osprey/libfi/matrix/mmx_fort.h:102-116  (internal_mm: j > i > kk)
 *   - the matrix-vector sibling  osprey/libfi/matrix/s4gemvx.f
 *
 * Compile with -ffp-contract=off and without -ffast-math so that multiply and
 * add stay separate, as the reference emits them when the target has no FMA
 * (osprey/be/cg/x8664/expand.cxx:5732-5743).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- element conversions --------------------------------------------------------- */

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even fp32 -> bf16, NaN kept quiet */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* OCP e4m3 (fn variant: no infinity, 0x7f/0xff are NaN, max finite 448) */
static inline float e4m3_to_f32(uint8_t v) {
    int s = v >> 7, e = (v >> 3) & 0xf, m = v & 7;
    float r;
    if (e == 0) r = ldexpf((float)m, -9);              /* subnormal: m/8 * 2^-6 */
    else if (e == 15 && m == 7) r = NAN;
    else r = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return s ? -r : r;
}

/* saturating RNE fp32 -> e4m3 */
static inline uint8_t f32_to_e4m3(float f) {
    uint8_t s = signbit(f) ? 0x80 : 0;
    float a = fabsf(f);
    if (isnan(a)) return s | 0x7f;
    if (a >= 448.0f) return s | 0x7e;
    if (a < ldexpf(1.0f, -10)) return s;                /* below half the least subnormal */
    int e;
    frexpf(a, &e);                                      /* a = m * 2^e, m in [0.5,1) */
    int ue = e - 1;                                     /* unbiased exponent of a */
    if (ue < -6) ue = -6;                               /* subnormal range shares 2^-6 */
    float q = ldexpf(a, 3 - ue);                        /* in units of the last place */
    float r = nearbyintf(q);                            /* RNE under the default rounding mode */
    int qi = (int)r;
    if (ue == -6 && qi < 8) return s | (uint8_t)qi;     /* subnormal */
    if (qi == 16) { qi = 8; ue += 1; }
    int be = ue + 7;
    if (be > 15 || (be == 15 && qi - 8 > 6)) return s | 0x7e;
    return s | (uint8_t)((be << 3) | (qi - 8));
}

void o64ref_bf16_to_f32(long n, const uint16_t *in, float *out) {
    for (long i = 0; i < n; ++i) out[i] = bf16_to_f32(in[i]);
}
void o64ref_f32_to_bf16(long n, const float *in, uint16_t *out) {
    for (long i = 0; i < n; ++i) out[i] = f32_to_bf16(in[i]);
}
void o64ref_e4m3_to_f32(long n, const uint8_t *in, float *out) {
    for (long i = 0; i < n; ++i) out[i] = e4m3_to_f32(in[i]);
}
void o64ref_f32_to_e4m3(long n, const float *in, uint8_t *out) {
    for (long i = 0; i < n; ++i) out[i] = f32_to_e4m3(in[i]);
}

/* ---- epilogue vocabulary ------------------------------------------------------------
 * What max(x,0), x/(1+exp(-x)) and the two GELU forms compile to on the CPU:
 * OPR_MAX (osprey/be/cg/x8664/expand.cxx:4517), INTRN_F4EXP / INTRN_F4TANH
 * (osprey/common/com/intrn_entry.def:915,1346).  Codes match include/o64gemm.h. */
enum { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU_TANH = 2, ACT_GELU_ERF = 3, ACT_SILU = 4 };

static inline float apply_act(float x, int act) {
    switch (act) {
    case ACT_RELU: return x > 0.0f ? x : 0.0f;
    case ACT_GELU_TANH: {
        float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
        return 0.5f * x * (1.0f + tanhf(u));
    }
    case ACT_GELU_ERF: return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f));
    case ACT_SILU: return x / (1.0f + expf(-x));
    default: return x;
    }
}

/* ---- the compiler's loop nest (f90_lower.cxx:5149-5169) ------------------------------
 * Y[i][j] = act( sum_k A[i][k]*B(k,j) + bias[j] ), fp32, ascending k, accumulator in a
 * scalar.  B(k,j) = B[k*ldb + j] when transB == 0 ([K,N] row-major) and B[j*ldb + k] when
 * transB != 0 ([N,K] row-major).  bias may be NULL. */
void o64ref_linear_f32(long M, long N, long K, const float *A, long lda, const float *B,
                       long ldb, int transB, const float *bias, float *Y, long ldy, int act) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M; ++i) {
        const float *a = A + i * lda;
        for (long j = 0; j < N; ++j) {
            float acc = 0.0f;
            if (transB) {
                const float *b = B + j * ldb;
                for (long k = 0; k < K; ++k) acc = acc + a[k] * b[k];
            } else {
                for (long k = 0; k < K; ++k) acc = acc + a[k] * B[k * ldb + j];
            }
            if (bias) acc = acc + bias[j];
            Y[i * ldy + j] = apply_act(acc, act);
        }
    }
}

/* Same nest with a double accumulator: used to measure how far any legal re-association
 * of the fp32 sum (licensed at -O3: osprey/common/com/config.cxx:1670-1680) can move the
 * answer.  Output still fp32. */
void o64ref_linear_f32_acc64(long M, long N, long K, const float *A, long lda, const float *B,
                             long ldb, int transB, const float *bias, float *Y, long ldy,
                             int act) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M; ++i) {
        const float *a = A + i * lda;
        for (long j = 0; j < N; ++j) {
            double acc = 0.0;
            for (long k = 0; k < K; ++k)
                acc += (double)a[k] * (double)(transB ? B[j * ldb + k] : B[k * ldb + j]);
            if (bias) acc += (double)bias[j];
            Y[i * ldy + j] = apply_act((float)acc, act);
        }
    }
}

/* bf16 operands upcast to fp32, the fp32 nest, fp32 result (the caller compares a bf16
 * device result against it with a relative-to-max tolerance). */
void o64ref_gemm_bf16(long M, long N, long K, const uint16_t *A, long lda, const uint16_t *B,
                      long ldb, int transB, const float *bias, float *C, long ldc, int act) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M; ++i) {
        const uint16_t *a = A + i * lda;
        for (long j = 0; j < N; ++j) {
            float acc = 0.0f;
            if (transB) {
                const uint16_t *b = B + j * ldb;
                for (long k = 0; k < K; ++k) acc = acc + bf16_to_f32(a[k]) * bf16_to_f32(b[k]);
            } else {
                for (long k = 0; k < K; ++k)
                    acc = acc + bf16_to_f32(a[k]) * bf16_to_f32(B[k * ldb + j]);
            }
            if (bias) acc = acc + bias[j];
            C[i * ldc + j] = apply_act(acc, act);
        }
    }
}

/* H = silu(X*Wg) (.) (X*Wu); X [M,K] bf16, Wg/Wu [K,N] bf16 row-major (ldw); the product is
 * rounded to bf16 because the second GEMM of the MLP consumes it as bf16. */
void o64ref_swiglu_bf16(long M, long N, long K, const uint16_t *X, long ldx, const uint16_t *Wg,
                        const uint16_t *Wu, long ldw, uint16_t *H, long ldh) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M; ++i) {
        const uint16_t *x = X + i * ldx;
        for (long j = 0; j < N; ++j) {
            float g = 0.0f, u = 0.0f;
            for (long k = 0; k < K; ++k) {
                float xv = bf16_to_f32(x[k]);
                g = g + xv * bf16_to_f32(Wg[k * ldw + j]);
                u = u + xv * bf16_to_f32(Wu[k * ldw + j]);
            }
            H[i * ldh + j] = f32_to_bf16(apply_act(g, ACT_SILU) * u);
        }
    }
}

/* fp8 e4m3 scaled GEMM: operands dequantised (q * scale) to fp32 first, then the fp32 nest,
 * plus bias; fp32 result.  A8 [M,K], B8 [N,K]. */
void o64ref_gemm_fp8_scaled(long M, long N, long K, const uint8_t *A8, long lda,
                            const uint8_t *B8, long ldb, const float *scaleA,
                            const float *scaleB, const float *bias, float *C, long ldc) {
    float lut[256];
    for (int v = 0; v < 256; ++v) lut[v] = e4m3_to_f32((uint8_t)v);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M; ++i) {
        const uint8_t *a = A8 + i * lda;
        const float sa = scaleA ? scaleA[i] : 1.0f;
        for (long j = 0; j < N; ++j) {
            const uint8_t *b = B8 + j * ldb;
            const float sb = scaleB ? scaleB[j] : 1.0f;
            float acc = 0.0f;
            for (long k = 0; k < K; ++k) acc = acc + (lut[a[k]] * sa) * (lut[b[k]] * sb);
            if (bias) acc = acc + bias[j];
            C[i * ldc + j] = acc;
        }
    }
}

/* int8 x int8 -> int32, A [M,K], B [N,K]; integer sums are order independent, so any
 * correct device kernel must match this bit for bit.  The reference's integer kernels are the
 * same template with integer types (osprey/libfi/matrix/i1i4gemmx.f); it has no s8*s8->s32
 * instance, the nearest being _MATMUL_I1I4 (osprey/crayf90/fe90/intrin.h:4300). */
void o64ref_gemm_s8s8_s32(long M, long N, long K, const int8_t *A, long lda, const int8_t *B,
                          long ldb, int32_t *C, long ldc) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M; ++i) {
        const int8_t *a = A + i * lda;
        for (long j = 0; j < N; ++j) {
            const int8_t *b = B + j * ldb;
            int32_t acc = 0;
            for (long k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
            C[i * ldc + j] = acc;
        }
    }
}

/* ---- the scaled ("requantising") tails -------------------------------------------------
 * out = convert( act( acc * (scaleA[m] * scaleB[n]) + bias[n] ) ), every fp32 operation rounded by
 * itself (this file is compiled with -ffp-contract=off), as the device kernels' scaled tail does.
 * out_kind: 0 = fp32 (the value before any conversion, for tolerance checks), 1 = int8 (nearest even,
 * saturating at -128 / 127), 2 = e4m3 (nearest even, saturating at +-448), 3 = bf16 bits.
 * The reference has no scaled product; its narrow integer MATMUL (INTEGER*1 in, INTEGER*1 out,
 * osprey/libfi/matrix/i1gemmx.f) wraps instead of scaling.  The tail's vocabulary is apply_act's. */
static inline void store_scaled(float x, int out_kind, void *C, long idx) {
    if (out_kind == 1) {
        float r = nearbyintf(x);
        if (isnan(r)) r = 0.0f;
        if (r < -128.0f) r = -128.0f;
        if (r > 127.0f) r = 127.0f;
        ((int8_t *)C)[idx] = (int8_t)r;
    } else if (out_kind == 2) {
        ((uint8_t *)C)[idx] = f32_to_e4m3(x);
    } else if (out_kind == 3) {
        ((uint16_t *)C)[idx] = f32_to_bf16(x);
    } else {
        ((float *)C)[idx] = x;
    }
}

/* int8 operands: the accumulator is the exact int32 sum, so the whole result is reproducible bit for
 * bit wherever act is exact (none, ReLU). */
void o64ref_gemm_s8_scaled(long M, long N, long K, const int8_t *A, long lda, const int8_t *B, long ldb,
                           const float *scaleA, const float *scaleB, const float *bias, int act, int out_kind,
                           void *C, long ldc) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M; ++i) {
        const int8_t *a = A + i * lda;
        const float sa = scaleA ? scaleA[i] : 1.0f;
        for (long j = 0; j < N; ++j) {
            const int8_t *b = B + j * ldb;
            int32_t acc = 0;
            for (long k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
            const float s = sa * (scaleB ? scaleB[j] : 1.0f);
            float x = (float)acc * s;
            x = x + (bias ? bias[j] : 0.0f);
            store_scaled(apply_act(x, act), out_kind, C, i * ldc + j);
        }
    }
}

/* e4m3 operands: fp32 nest on the unscaled values (what the tensor cores accumulate), then the tail. */
void o64ref_gemm_fp8_scaled_ex(long M, long N, long K, const uint8_t *A8, long lda, const uint8_t *B8, long ldb,
                               const float *scaleA, const float *scaleB, const float *bias, int act, int out_kind,
                               void *C, long ldc) {
    float lut[256];
    for (int v = 0; v < 256; ++v) lut[v] = e4m3_to_f32((uint8_t)v);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M; ++i) {
        const uint8_t *a = A8 + i * lda;
        const float sa = scaleA ? scaleA[i] : 1.0f;
        for (long j = 0; j < N; ++j) {
            const uint8_t *b = B8 + j * ldb;
            float acc = 0.0f;
            for (long k = 0; k < K; ++k) acc = acc + lut[a[k]] * lut[b[k]];
            const float s = sa * (scaleB ? scaleB[j] : 1.0f);
            float x = acc * s;
            x = x + (bias ? bias[j] : 0.0f);
            store_scaled(apply_act(x, act), out_kind, C, i * ldc + j);
        }
    }
}

/* ---- the runtime's strided kernel (xgemmx.h:172-236, s4gemmx.f:151-196) ---------------
 * C = alpha*A*B + beta*C with element(i,j) of X at X[inc1x*i + inc2x*j] (0-based).
 * Loop order J > L > I; the axpy over a column of C is skipped when B(L,J) == 0. */
void o64ref_s4gemmx(int M, int N, int K, float alpha, const float *A, int inc1a, int inc2a,
                    const float *B, int inc1b, int inc2b, float beta, float *C, int inc1c,
                    int inc2c) {
    if (M == 0 || N == 0 || (alpha == 0.0f && beta == 1.0f)) return;
    if (K == 0) {
        for (long j = 0; j < N; ++j)
            for (long i = 0; i < M; ++i) C[(long)inc2c * j + (long)inc1c * i] = 0.0f;
        return;
    }
    if (alpha == 0.0f) {
        for (long j = 0; j < N; ++j)
            for (long i = 0; i < M; ++i) {
                long ic = (long)inc2c * j + (long)inc1c * i;
                C[ic] = (beta == 0.0f) ? 0.0f : beta * C[ic];
            }
        return;
    }
    for (long j = 0; j < N; ++j) {
        if (beta == 0.0f) {
            for (long i = 0; i < M; ++i) C[(long)inc2c * j + (long)inc1c * i] = 0.0f;
        } else if (beta != 1.0f) {
            for (long i = 0; i < M; ++i) {
                long ic = (long)inc2c * j + (long)inc1c * i;
                C[ic] = beta * C[ic];
            }
        }
        for (long l = 0; l < K; ++l) {
            float b = B[(long)inc2b * j + (long)inc1b * l];
            if (b != 0.0f) {
                float temp = alpha * b;
                for (long i = 0; i < M; ++i) {
                    long ic = (long)inc2c * j + (long)inc1c * i;
                    C[ic] = C[ic] + temp * A[(long)inc2a * l + (long)inc1a * i];
                }
            }
        }
    }
}

/* The dot-product form behind the BLAS hook (mmx_fort.h:102-116): contiguous column-major
 * operands, R(M,N) zeroed, loops j > i > kk.  Called as sgemm('n','n',m,n,k,...) with
 * lda = m, ldb = k, ldc = m (mmx_fort.h:94-95). */
void o64ref_internal_mm_f32(int M, int N, int K, const float *A, const float *B, float *R) {
    for (long j = 0; j < N; ++j)
        for (long i = 0; i < M; ++i) {
            float r = 0.0f;
            for (long kk = 0; kk < K; ++kk) r = r + A[i + kk * (long)M] * B[kk + j * (long)K];
            R[i + j * (long)M] = r;
        }
}

/* y = alpha*A*x + beta*y, the matrix-vector sibling (osprey/libfi/matrix/s4gemvx.f):
 * column sweep, a column's axpy skipped when x(j) == 0.  A(i,j) at A[inc1a*i + inc2a*j]. */
void o64ref_s4gemvx(int M, int N, float alpha, const float *A, int inc1a, int inc2a,
                    const float *X, int incx, float beta, float *Y, int incy) {
    if (M != 0 && N == 0) {                         /* s4gemvx.f: empty sum zeroes Y */
        for (long i = 0; i < M; ++i) Y[(long)incy * i] = 0.0f;
        return;
    }
    if (M == 0 || N == 0 || (alpha == 0.0f && beta == 1.0f)) return;
    if (beta == 0.0f) {
        for (long i = 0; i < M; ++i) Y[(long)incy * i] = 0.0f;
    } else if (beta != 1.0f) {
        for (long i = 0; i < M; ++i) Y[(long)incy * i] = beta * Y[(long)incy * i];
    }
    if (alpha == 0.0f) return;
    for (long j = 0; j < N; ++j) {
        float x = X[(long)incx * j];
        if (x != 0.0f) {
            float temp = alpha * x;
            for (long i = 0; i < M; ++i)
                Y[(long)incy * i] = Y[(long)incy * i] + temp * A[(long)inc1a * i + (long)inc2a * j];
        }
    }
}

/* ---- the same two kernels for the other element kinds ------------------------------------
 * sgemmx.f / sgemvx.f are the REAL*4 texts with REAL(KIND=8) declarations.  The integer
 * kernels instantiate the xgemmx.h template: i1gemmx.f, i2gemmx.f, i4gemmx.f, jgemmx.f with one
 * kind throughout, and i1i2 / i1i4 / i1j / i2i4 / i2j / i4j gemmx.f with A of the narrower kind
 * and B, C, alpha, beta, temp of the wider one (A's element is converted, i.e. sign-extended,
 * in `temp*a(i,l)`).  Integers are computed on unsigned types (TS: signed kind of C, T: its
 * unsigned twin, W: the unsigned type products are formed in, at least 32 bits so that C's
 * integer promotion cannot overflow): the wrap-around is the two's-complement result of the
 * Fortran code without C's signed-overflow caveat. */
#define O64REF_GEMMX(NAME, TA, TS, T, W)                                                        \
    void NAME(int M, int N, int K, T alpha, const TA *A, int inc1a, int inc2a, const T *B,      \
              int inc1b, int inc2b, T beta, T *C, int inc1c, int inc2c) {                       \
        if (M == 0 || N == 0 || (alpha == (T)0 && beta == (T)1)) return;                        \
        if (K == 0) {                                                                           \
            for (long j = 0; j < N; ++j)                                                        \
                for (long i = 0; i < M; ++i) C[(long)inc2c * j + (long)inc1c * i] = (T)0;       \
            return;                                                                             \
        }                                                                                       \
        if (alpha == (T)0) {                                                                    \
            for (long j = 0; j < N; ++j)                                                        \
                for (long i = 0; i < M; ++i) {                                                  \
                    long ic = (long)inc2c * j + (long)inc1c * i;                                \
                    C[ic] = (beta == (T)0) ? (T)0 : (T)((W)beta * (W)C[ic]);                    \
                }                                                                               \
            return;                                                                             \
        }                                                                                       \
        for (long j = 0; j < N; ++j) {                                                          \
            if (beta == (T)0) {                                                                 \
                for (long i = 0; i < M; ++i) C[(long)inc2c * j + (long)inc1c * i] = (T)0;       \
            } else if (beta != (T)1) {                                                          \
                for (long i = 0; i < M; ++i) {                                                  \
                    long ic = (long)inc2c * j + (long)inc1c * i;                                \
                    C[ic] = (T)((W)beta * (W)C[ic]);                                            \
                }                                                                               \
            }                                                                                   \
            for (long l = 0; l < K; ++l) {                                                      \
                T b = B[(long)inc2b * j + (long)inc1b * l];                                     \
                if (b != (T)0) {                                                                \
                    T temp = (T)((W)alpha * (W)b);                                              \
                    for (long i = 0; i < M; ++i) {                                              \
                        long ic = (long)inc2c * j + (long)inc1c * i;                            \
                        T a = (T)(TS)A[(long)inc2a * l + (long)inc1a * i];                      \
                        C[ic] = (T)((W)C[ic] + (W)temp * (W)a);                                 \
                    }                                                                           \
                }                                                                               \
            }                                                                                   \
        }                                                                                       \
    }
O64REF_GEMMX(o64ref_sgemmx_f64, double, double, double, double)
O64REF_GEMMX(o64ref_i1gemmx, int8_t, int8_t, uint8_t, uint32_t)
O64REF_GEMMX(o64ref_i1i2gemmx, int8_t, int16_t, uint16_t, uint32_t)
O64REF_GEMMX(o64ref_i1i4gemmx, int8_t, int32_t, uint32_t, uint32_t)
O64REF_GEMMX(o64ref_i1jgemmx, int8_t, int64_t, uint64_t, uint64_t)
O64REF_GEMMX(o64ref_i2gemmx, int16_t, int16_t, uint16_t, uint32_t)
O64REF_GEMMX(o64ref_i2i4gemmx, int16_t, int32_t, uint32_t, uint32_t)
O64REF_GEMMX(o64ref_i2jgemmx, int16_t, int64_t, uint64_t, uint64_t)
O64REF_GEMMX(o64ref_i4gemmx, int32_t, int32_t, uint32_t, uint32_t)
O64REF_GEMMX(o64ref_i4jgemmx, int32_t, int64_t, uint64_t, uint64_t)
O64REF_GEMMX(o64ref_jgemmx, int64_t, int64_t, uint64_t, uint64_t)
/* mixed kinds with a REAL result: A converted to the kind of B and C (s4sgemmx.f, i4s4gemmx.f, jsgemmx.f, ...) */
O64REF_GEMMX(o64ref_s4sgemmx, float, double, double, double)
O64REF_GEMMX(o64ref_i1s4gemmx, int8_t, float, float, float)
O64REF_GEMMX(o64ref_i2s4gemmx, int16_t, float, float, float)
O64REF_GEMMX(o64ref_i4s4gemmx, int32_t, float, float, float)
O64REF_GEMMX(o64ref_js4gemmx, int64_t, float, float, float)
O64REF_GEMMX(o64ref_i1sgemmx, int8_t, double, double, double)
O64REF_GEMMX(o64ref_i2sgemmx, int16_t, double, double, double)
O64REF_GEMMX(o64ref_i4sgemmx, int32_t, double, double, double)
O64REF_GEMMX(o64ref_jsgemmx, int64_t, double, double, double)
#undef O64REF_GEMMX

void o64ref_sgemvx_f64(int M, int N, double alpha, const double *A, int inc1a, int inc2a,
                       const double *X, int incx, double beta, double *Y, int incy) {
    if (M != 0 && N == 0) {
        for (long i = 0; i < M; ++i) Y[(long)incy * i] = 0.0;
        return;
    }
    if (M == 0 || N == 0 || (alpha == 0.0 && beta == 1.0)) return;
    if (beta == 0.0) {
        for (long i = 0; i < M; ++i) Y[(long)incy * i] = 0.0;
    } else if (beta != 1.0) {
        for (long i = 0; i < M; ++i) Y[(long)incy * i] = beta * Y[(long)incy * i];
    }
    if (alpha == 0.0) return;
    for (long j = 0; j < N; ++j) {
        double x = X[(long)incx * j];
        if (x != 0.0) {
            double temp = alpha * x;
            for (long i = 0; i < M; ++i)
                Y[(long)incy * i] = Y[(long)incy * i] + temp * A[(long)inc1a * i + (long)inc2a * j];
        }
    }
}

/* ---- LOGICAL kinds (lgemmx.h): non-zero is true, results are 1 / 0 ------------------------------ */
#define O64REF_LGEMMX(NAME, TA, T)                                                               \
    void NAME(int M, int N, int K, int alpha, const TA *A, int inc1a, int inc2a, const T *B,     \
              int inc1b, int inc2b, int beta, T *C, int inc1c, int inc2c) {                      \
        if (M == 0 || N == 0) return;                                                            \
        if (K == 0 || (!alpha && !beta)) {                                                       \
            for (long j = 0; j < N; ++j)                                                         \
                for (long i = 0; i < M; ++i) C[(long)inc2c * j + (long)inc1c * i] = 0;           \
            return;                                                                              \
        }                                                                                        \
        if (!alpha) return;                                                                      \
        for (long j = 0; j < N; ++j) {                                                           \
            for (long i = 0; i < M; ++i) {                                                       \
                T *c = C + (long)inc2c * j + (long)inc1c * i;                                    \
                *c = (beta && *c != 0) ? 1 : 0;                                                  \
            }                                                                                    \
            for (long l = 0; l < K; ++l) {                                                       \
                if (B[(long)inc2b * j + (long)inc1b * l] == 0) continue;                         \
                for (long i = 0; i < M; ++i)                                                     \
                    if (A[(long)inc2a * l + (long)inc1a * i] != 0) C[(long)inc2c * j + (long)inc1c * i] = 1; \
            }                                                                                    \
        }                                                                                        \
    }
O64REF_LGEMMX(o64ref_l1gemmx, int8_t, int8_t)
O64REF_LGEMMX(o64ref_l1l2gemmx, int8_t, int16_t)
O64REF_LGEMMX(o64ref_l1l4gemmx, int8_t, int32_t)
O64REF_LGEMMX(o64ref_l1lgemmx, int8_t, int64_t)
O64REF_LGEMMX(o64ref_l2gemmx, int16_t, int16_t)
O64REF_LGEMMX(o64ref_l2l4gemmx, int16_t, int32_t)
O64REF_LGEMMX(o64ref_l2lgemmx, int16_t, int64_t)
O64REF_LGEMMX(o64ref_l4gemmx, int32_t, int32_t)
O64REF_LGEMMX(o64ref_l4lgemmx, int32_t, int64_t)
O64REF_LGEMMX(o64ref_lgemmx, int64_t, int64_t)
#undef O64REF_LGEMMX

/* ---- COMPLEX*8 / COMPLEX*16 (c4gemmx.f:156-244, cgemmx.f; c4gemvx.f, cgemvx.f) -------------
 * Values are (re, im) pairs; increments count complex elements.  The matrix kernel applies the
 * conjugation flags and, unlike the real template, does not test B for zeros; the vector kernel
 * skips a column when x(j) == 0. */
#define O64REF_CGEMMX(NAME, NAMEV, R)                                                            \
    void NAME(int conja, int conjb, int M, int N, int K, const R *alpha, const R *A, int inc1a,   \
              int inc2a, const R *B, int inc1b, int inc2b, const R *beta, R *C, int inc1c,       \
              int inc2c) {                                                                       \
        const R ar = alpha[0], ai = alpha[1], br = beta[0], bi = beta[1];                        \
        const int a_zero = (ar == 0 && ai == 0), b_one = (br == 1 && bi == 0);                   \
        const int b_zero = (br == 0 && bi == 0);                                                 \
        if (M == 0 || N == 0 || (a_zero && b_one)) return;                                       \
        for (long j = 0; j < N; ++j) {                                                           \
            for (long i = 0; i < M; ++i) {                                                       \
                R *c = C + 2 * ((long)inc2c * j + (long)inc1c * i);                              \
                if (b_zero || K == 0) { /* K == 0: the result is set to zero (c4gemmx.f:164-172) */ \
                    c[0] = 0, c[1] = 0;                                                          \
                    continue;                                                                    \
                }                                                                                \
                if (b_zero) {                                                                    \
                    c[0] = 0, c[1] = 0;                                                          \
                } else if (!b_one) {                                                             \
                    const R cr = c[0], ci = c[1];                                                \
                    c[0] = br * cr - bi * ci, c[1] = br * ci + bi * cr;                          \
                }                                                                                \
            }                                                                                    \
            if (a_zero) continue;                                                                \
            for (long l = 0; l < K; ++l) {                                                       \
                const R *b = B + 2 * ((long)inc2b * j + (long)inc1b * l);                        \
                const R xr = b[0], xi = conjb ? -b[1] : b[1];                                    \
                const R tr = ar * xr - ai * xi, ti = ar * xi + ai * xr;                          \
                for (long i = 0; i < M; ++i) {                                                   \
                    const R *a = A + 2 * ((long)inc2a * l + (long)inc1a * i);                    \
                    const R yr = a[0], yi = conja ? -a[1] : a[1];                                \
                    R *c = C + 2 * ((long)inc2c * j + (long)inc1c * i);                          \
                    c[0] = c[0] + (tr * yr - ti * yi);                                           \
                    c[1] = c[1] + (tr * yi + ti * yr);                                           \
                }                                                                                \
            }                                                                                    \
        }                                                                                        \
    }                                                                                            \
    void NAMEV(int conj, int M, int N, const R *alpha, const R *A, int inc1a, int inc2a,         \
               const R *X, int incx, const R *beta, R *Y, int incy) {                            \
        const R ar = alpha[0], ai = alpha[1], br = beta[0], bi = beta[1];                        \
        if (M != 0 && N == 0) {                                                                  \
            for (long i = 0; i < M; ++i) Y[2 * (long)incy * i] = 0, Y[2 * (long)incy * i + 1] = 0; \
            return;                                                                              \
        }                                                                                        \
        if (M == 0 || N == 0 || (ar == 0 && ai == 0 && br == 1 && bi == 0)) return;              \
        for (long i = 0; i < M; ++i) {                                                           \
            R *y = Y + 2 * (long)incy * i;                                                       \
            if (br == 0 && bi == 0) {                                                            \
                y[0] = 0, y[1] = 0;                                                              \
            } else if (!(br == 1 && bi == 0)) {                                                  \
                const R yr = y[0], yi = y[1];                                                    \
                y[0] = br * yr - bi * yi, y[1] = br * yi + bi * yr;                              \
            }                                                                                    \
        }                                                                                        \
        if (ar == 0 && ai == 0) return;                                                          \
        for (long j = 0; j < N; ++j) {                                                           \
            const R xr = X[2 * (long)incx * j], xi = X[2 * (long)incx * j + 1];                  \
            if (xr == 0 && xi == 0) continue;                                                    \
            const R tr = ar * xr - ai * xi, ti = ar * xi + ai * xr;                              \
            for (long i = 0; i < M; ++i) {                                                       \
                const R *a = A + 2 * ((long)inc1a * i + (long)inc2a * j);                        \
                const R zr = a[0], zi = conj ? -a[1] : a[1];                                     \
                R *y = Y + 2 * (long)incy * i;                                                   \
                y[0] = y[0] + (tr * zr - ti * zi);                                               \
                y[1] = y[1] + (tr * zi + ti * zr);                                               \
            }                                                                                    \
        }                                                                                        \
    }
O64REF_CGEMMX(o64ref_c4gemmx, o64ref_c4gemvx, float)
O64REF_CGEMMX(o64ref_cgemmx, o64ref_cgemvx, double)
#undef O64REF_CGEMMX

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the CPU baseline asks for the cores back. */
void o64ref_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int o64ref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
