/* Nests in the shapes the reference leaves them in AFTER its loop-nest optimiser has run, hand-derived
 * from the transformation itself (SNL_INV_Cache_Block, osprey/be/lno/snl_inv.cxx:774-805: a strip loop
 * stepping by the block size outside, the blocked loop running from the strip variable to
 * min(strip + B - 1, upper bound); the accumulator scalar-expanded and the zeroing distributed into a
 * nest of its own, snl_test.cxx:1036-1040) and printed the way whirl2c prints DO loops and OPR_MIN
 * (wn2c.cxx:4078-4118, 658), plus GELU / SiLU tails on the untiled fused linear.  Input of o64nest in the
 * tests: `main` fills the operands with seeded values, runs every nest and writes the results to the
 * file named on the command line. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#define _I4MIN(v1, v2) ((v1) < (v2)? (v1) : (v2))

float A[300][200], B[200][260], C1[300][260], C2[300][260], C3[300][260], bias[260];
float G1[300][260], G2[300][260], G3[300][260];
double Ad[90][70], Bd[70][50], Cd[90][50];
int Ai[40][24], Bi[24][56], Ci[40][56];

/* L1 blocking of i (64) and k (16), j left whole; loop order it, kt, j, i, k */
void blocked_i_k(void) {
  int i, j, k, it, kt;
  for(i = 0; i <= 299; i = i + 1)
    for(j = 0; j <= 259; j = j + 1)
      C1[i][j] = 0.0F;
  for(it = 0; it <= 299; it = it + 64)
    for(kt = 0; kt <= 199; kt = kt + 16)
      for(j = 0; j <= 259; j = j + 1)
        for(i = it; i <= _I4MIN(it + 63, 299); i = i + 1)
          for(k = kt; k <= _I4MIN(kt + 15, 199); k = k + 1)
            C1[i][j] = C1[i][j] + (A[i][k] * B[k][j]);
}

/* all three loops blocked, the j strip outermost (the optimiser interchanged i and j), a block size
 * that divides the extent exactly printed without the minimum */
void blocked_all_interchanged(void) {
  int i, j, k, it, jt, kt;
  for(i = 0; i <= 299; i = i + 1)
    for(j = 0; j <= 259; j = j + 1)
      C2[i][j] = 0.0F;
  for(jt = 0; jt <= 259; jt = jt + 32)
  {
    for(it = 0; it <= 299; it = it + 100)
    {
      for(kt = 0; kt <= 199; kt = kt + 64)
      {
        for(i = it; i <= it + 99; i = i + 1)
        {
          for(j = jt; j <= _I4MIN(jt + 31, 259); j = j + 1)
          {
            for(k = kt; k <= _I4MIN(kt + 63, 199); k = k + 1)
            {
              C2[i][j] = C2[i][j] + (A[i][k] * B[k][j]);
            }
          }
        }
      }
    }
  }
}

/* hand-written tiling: exclusive bounds, a ternary minimum, += */
void blocked_by_hand(void) {
  for (int i = 0; i < 300; i++)
    for (int j = 0; j < 260; j++) C3[i][j] = 0;
  for (int kt = 0; kt < 200; kt += 40)
    for (int i = 0; i < 300; i++)
      for (int j = 0; j < 260; j++)
        for (int k = kt; k < (kt + 40 < 200 ? kt + 40 : 200); k++)
          C3[i][j] += A[i][k] * B[k][j];
}

/* REAL*8, blocked on i only; the accumulation adds to what the array holds */
void blocked_double(void) {
  int i, j, k, it;
  for(it = 0; it <= 89; it = it + 32)
    for(i = it; i <= _I4MIN(it + 31, 89); i = i + 1)
      for(k = 0; k <= 69; k = k + 1)
        for(j = 0; j <= 49; j = j + 1)
          Cd[i][j] = Cd[i][j] + (Ad[i][k] * Bd[k][j]);
}

/* integers, the plain perfect accumulating nest (no blocking at all) */
void perfect_int(void) {
  for (int i = 0; i < 40; i++)
    for (int k = 0; k < 24; k++)
      for (int j = 0; j < 56; j++)
        Ci[i][j] = Ci[i][j] + Ai[i][k] * Bi[k][j];
}

/* the fused linear with the tails the exp / tanh intrinsics give */
void linear_silu(void) {
  for (int i = 0; i < 300; i++)
    for (int j = 0; j < 260; j++) {
      float acc = 0;
      for (int k = 0; k < 200; k++) acc += A[i][k] * B[k][j];
      float t = acc + bias[j];
      G1[i][j] = t / (1.0f + expf(-t));
    }
}

void linear_gelu_tanh(void) {
  for (int i = 0; i < 300; i++)
    for (int j = 0; j < 260; j++) {
      float acc = 0;
      for (int k = 0; k < 200; k++) acc += A[i][k] * B[k][j];
      float t = acc + bias[j];
      G2[i][j] = 0.5f * t * (1.0f + tanhf(0.7978845608f * (t + 0.044715f * t * t * t)));
    }
}

void linear_gelu_erf(void) {
  for (int i = 0; i < 300; i++)
    for (int j = 0; j < 260; j++) {
      float acc = 0;
      for (int k = 0; k < 200; k++) acc += A[i][k] * B[k][j];
      G3[i][j] = 0.5f * acc * (1.0f + erff(acc * 0.70710678f));
    }
}

/* not blocked consistently: the blocked loop runs past its strip (64 against a step of 32); stays as it is */
float inconsistent(void) {
  float s = 0;
  for (int it = 0; it < 64; it += 32)
    for (int i = it; i < it + 64; i++)
      for (int j = 0; j < 8; j++)
        for (int k = 0; k < 8; k++)
          G3[i][j] = G3[i][j] + A[i][k] * B[k][j];
  for (int i = 0; i < 128; i++) s += G3[i][0];
  return s;
}

static unsigned rng_state = 2468u;
static float frand(void) {
  rng_state = rng_state * 1664525u + 1013904223u;
  return (float)((rng_state >> 8) & 0xffff) / 65536.0f - 0.5f;
}

int main(int argc, char **argv) {
  if (argc < 2) return 2;
  for (int i = 0; i < 300; i++) for (int k = 0; k < 200; k++) A[i][k] = frand();
  for (int k = 0; k < 200; k++) for (int j = 0; j < 260; j++) B[k][j] = frand();
  for (int j = 0; j < 260; j++) bias[j] = frand();
  for (int i = 0; i < 90; i++) for (int k = 0; k < 70; k++) Ad[i][k] = frand();
  for (int k = 0; k < 70; k++) for (int j = 0; j < 50; j++) Bd[k][j] = frand();
  for (int i = 0; i < 90; i++) for (int j = 0; j < 50; j++) Cd[i][j] = frand();
  for (int i = 0; i < 40; i++) for (int k = 0; k < 24; k++) Ai[i][k] = (int)(frand() * 2000000.0f);
  for (int k = 0; k < 24; k++) for (int j = 0; j < 56; j++) Bi[k][j] = (int)(frand() * 2000000.0f);
  for (int i = 0; i < 40; i++) for (int j = 0; j < 56; j++) Ci[i][j] = (int)(frand() * 1000.0f);
  blocked_i_k();
  blocked_all_interchanged();
  blocked_by_hand();
  blocked_double();
  perfect_int();
  linear_silu();
  linear_gelu_tanh();
  linear_gelu_erf();
  FILE *f = fopen(argv[1], "wb");
  if (!f) return 3;
  fwrite(C1, sizeof(C1), 1, f);
  fwrite(C2, sizeof(C2), 1, f);
  fwrite(C3, sizeof(C3), 1, f);
  fwrite(Cd, sizeof(Cd), 1, f);
  fwrite(Ci, sizeof(Ci), 1, f);
  fwrite(G1, sizeof(G1), 1, f);
  fwrite(G2, sizeof(G2), 1, f);
  fwrite(G3, sizeof(G3), 1, f);
  fclose(f);
  return 0;
}
