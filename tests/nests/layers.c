/* Loop nests in the form the reference's C back-translator prints them, plus hand-written
 * variants; input of o64nest in the tests.  `main` fills the operands with seeded values, runs
 * every nest and writes the results to the file named on the command line. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#define MM 192
#define NN 160
#define KK 224

float A[MM][KK], B[KK][NN], Y[MM][NN], bias[NN];
double Ad[100][60], Bd[60][80], Cd[100][80];
int Ai[64][32], Bi[48][32], Ci[64][48];
long long Aj[40][24], Bj[24][56], Cj[40][56];
float Yplain[MM][NN];

void fused_linear(void) {
  int i, j, k;
  float acc;
#pragma blocking size (32, 128)
  for(i = 0; i <= 191; i = i + 1)
  {
#pragma blocking size (64)
    for(j = 0; j <= 159; j = j + 1)
    {
      acc = 0.0F;
      for(k = 0; k <= 223; k = k + 1)
      {
        acc = acc + (A[i][k] * B[k][j]);
      }
      Y[i][j] = fmaxf(acc + bias[j], 0.0F);
    }
  }
}

void plain_product(void) {
  for (int i = 0; i < MM; i++)
    for (int j = 0; j < NN; j++) {
      float acc = 0;
      for (int k = 0; k < KK; k++)
        acc += A[i][k] * B[k][j];
      Yplain[i][j] = acc;
    }
}

void double_in_place(void) {
  for (int i = 0; i < 100; i++)
    for (int j = 0; j < 80; ++j) {
      Cd[i][j] = 0;
      for (int k = 0; k < 60; k += 1)
        Cd[i][j] += Ad[i][k] * Bd[k][j];
    }
}

void int_times_transposed(void) {   /* Bi is stored [N][K]: Ci = Ai * Bi^T */
  for (int i = 0; i < 64; i++)
    for (int j = 0; j < 48; j++) {
      int s = 0;
      for (int k = 0; k < 32; k++)
        s = s + Ai[i][k] * Bi[j][k];
      Ci[i][j] = s;
    }
}

void int64_product(void) {
  for (int i = 0; i < 40; i++)
    for (int j = 0; j < 56; j++) {
      Cj[i][j] = 0;
      for (int k = 0; k < 24; k++)
        Cj[i][j] = Cj[i][j] + Aj[i][k] * Bj[k][j];
    }
}

void flattened(const float *X, const float *W, float *O, int m, int n, int kk) {
  for (int i = 0; i < m; i++)
    for (int j = 0; j < n; j++) {
      float acc = 0;
      for (int k = 0; k < kk; k++)
        acc += X[i*kk + k] * W[k*n + j];
      O[i*n + j] = acc;
    }
}

float not_a_product(void) {   /* same shape of nest, but a sum: must stay as it is */
  float t = 0;
  for (int i = 0; i < 10; i++)
    for (int j = 0; j < 10; j++) {
      Y[i][j] = 0;
      for (int k = 0; k < 10; k++)
        Y[i][j] = Y[i][j] + A[i][k] + B[k][j];
      t += Y[i][j];
    }
  return t;
}

static unsigned rng_state = 12345u;
static float frand(void) {
  rng_state = rng_state * 1664525u + 1013904223u;
  return (float)((rng_state >> 8) & 0xffff) / 65536.0f - 0.5f;
}

int main(int argc, char **argv) {
  if (argc < 2) return 2;
  for (int i = 0; i < MM; i++) for (int k = 0; k < KK; k++) A[i][k] = frand();
  for (int k = 0; k < KK; k++) for (int j = 0; j < NN; j++) B[k][j] = frand();
  for (int j = 0; j < NN; j++) bias[j] = frand();
  for (int i = 0; i < 100; i++) for (int k = 0; k < 60; k++) Ad[i][k] = frand();
  for (int k = 0; k < 60; k++) for (int j = 0; j < 80; j++) Bd[k][j] = frand();
  for (int i = 0; i < 64; i++) for (int k = 0; k < 32; k++) Ai[i][k] = (int)(frand() * 2000000.0f);
  for (int j = 0; j < 48; j++) for (int k = 0; k < 32; k++) Bi[j][k] = (int)(frand() * 2000000.0f);
  for (int i = 0; i < 40; i++) for (int k = 0; k < 24; k++) Aj[i][k] = (long long)(frand() * 4.0e9f);
  for (int k = 0; k < 24; k++) for (int j = 0; j < 56; j++) Bj[k][j] = (long long)(frand() * 4.0e9f);
  static float O[MM * NN];
  not_a_product();
  fused_linear();
  plain_product();
  double_in_place();
  int_times_transposed();
  int64_product();
  flattened(&A[0][0], &B[0][0], O, MM, NN, KK);
  FILE *f = fopen(argv[1], "wb");
  if (!f) return 3;
  fwrite(Y, sizeof(Y), 1, f);
  fwrite(Yplain, sizeof(Yplain), 1, f);
  fwrite(Cd, sizeof(Cd), 1, f);
  fwrite(Ci, sizeof(Ci), 1, f);
  fwrite(Cj, sizeof(Cj), 1, f);
  fwrite(O, sizeof(O), 1, f);
  fclose(f);
  return 0;
}
