/* Product nests over SECTIONS of arrays: loops that do not start at zero (the form the reference's
 * front end leaves for A(3:, 2:) = MATMUL(...) style code after lowering, and what whirl2c prints for
 * DO loops with a non-trivial first value), untouched elements around them, and one nest whose bounds
 * depend on an outer loop variable, which must be left alone.  Input of o64nest in the tests: `main`
 * fills the operands with seeded values, runs every nest and writes the results to the file named on
 * the command line. */
#include <stdio.h>
#include <stdlib.h>

#define M 140
#define N 96
#define K 80

float A[M][K], B[K][N], Y[M][N], T[M][N], bias[N];
double P[50 * 30], Q[30 * 20], R[50 * 20];
int Ai[40][24], Bi[24][56], Ci[40][56];

/* fused linear on the lower right part of Y: constant first values, `<=` on one loop, ReLU as a conditional */
void section_linear(void) {
  int i, j, k;
  for (i = 2; i < M; i++)
    for (j = 3; j <= N - 2; j++) {
      float acc = 0;
      for (k = 1; k < K; k++) acc = acc + A[i][k] * B[k][j];
      Y[i][j] = acc + bias[j] > 0 ? acc + bias[j] : 0;
    }
}

/* REAL*8, flattened subscripts, first values that are variables and expressions */
void section_flat(int lo, int hi) {
  int i, j, k;
  for (i = lo; i < hi; i = i + 1)
    for (j = 4; j < 20; j++) {
      R[i * 20 + j] = 0;
      for (k = lo + 1; k < 30; k++) R[i * 20 + j] = R[i * 20 + j] + P[i * 30 + k] * Q[k * 20 + j];
    }
}

/* integers, the second operand read transposed */
void section_int(void) {
  int i, j, k;
  for (i = 5; i <= 39; i = i + 1)
    for (j = 7; j <= 50; j = j + 1) {
      Ci[i][j] = 0;
      for (k = 2; k <= 22; k = k + 1) Ci[i][j] = Ci[i][j] + Ai[i][k] * Bi[k][j];
    }
}

/* not a rectangle: j starts at i.  Must pass through unchanged. */
void triangle(void) {
  int i, j, k;
  for (i = 0; i < N; i++)
    for (j = i; j < N; j++) {
      float acc = 0;
      for (k = 0; k < K; k++) acc += A[i][k] * B[k][j];
      T[i][j] = acc;
    }
}

static unsigned long long seed = 0x9E3779B97F4A7C15ull;
static float frand(void) {
  seed = seed * 6364136223846793005ull + 1442695040888963407ull;
  return (float)((seed >> 40) & 0xFFFF) / 32768.0f - 1.0f;
}

int main(int argc, char **argv) {
  if (argc < 2) return 2;
  for (int i = 0; i < M; i++) for (int k = 0; k < K; k++) A[i][k] = frand();
  for (int k = 0; k < K; k++) for (int j = 0; j < N; j++) B[k][j] = frand();
  for (int j = 0; j < N; j++) bias[j] = frand();
  for (int i = 0; i < M; i++) for (int j = 0; j < N; j++) { Y[i][j] = -5.0f; T[i][j] = -6.0f; }
  for (int i = 0; i < 50 * 30; i++) P[i] = frand();
  for (int i = 0; i < 30 * 20; i++) Q[i] = frand();
  for (int i = 0; i < 50 * 20; i++) R[i] = -7.0;
  for (int i = 0; i < 40; i++) for (int k = 0; k < 24; k++) Ai[i][k] = (int)(frand() * 2000000.0f);
  for (int k = 0; k < 24; k++) for (int j = 0; j < 56; j++) Bi[k][j] = (int)(frand() * 2000000.0f);
  for (int i = 0; i < 40; i++) for (int j = 0; j < 56; j++) Ci[i][j] = -8;
  section_linear();
  section_flat(3, 47);
  section_int();
  triangle();
  FILE *f = fopen(argv[1], "wb");
  if (!f) return 3;
  fwrite(Y, sizeof(Y), 1, f);
  fwrite(R, sizeof(R), 1, f);
  fwrite(Ci, sizeof(Ci), 1, f);
  fwrite(T, sizeof(T), 1, f);
  fclose(f);
  return 0;
}
