/* Host check of the integer state pass's arithmetic (the device code is pass_rows_fx and its helpers in
 * statequant_b200/csrc/pass_rows.cuh; this file restates them in plain C).
 *
 * A read-out vector x[128] is scaled by a power of two into (-2^23, 2^23], rounded to integers, cut into three byte
 * slices (top signed, the others unsigned); a lane chunk of 16 codes meets the slices in byte dot products; the three
 * slice sums are recombined in float.  Checked here, for int8 codes and for int4 nibbles (offset 8, carried by the
 * start value of the slice sums), over vectors of many magnitudes:
 *   1. slices recombine to the fixed-point integer exactly, and the fixed-point integer fits 24 bits;
 *   2. the float recombination differs from the exact integer sum by at most two roundings (2^-23 of the sum, plus
 *      8 units of the fixed-point grid for the rounding of the two low slices' sum);
 *   3. the whole chunk sum, scaled back, is within 16 * qmax * 2^-23 * max|x| of the dot product in double precision
 *      (the rounding of the vector to the fixed-point grid), with some slack for the recombination.
 * Prints "failures 0" when all hold. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static void fx_scale(float amax, float* mult, float* inv) {
  const int e = (int)((f2u(amax) >> 23) & 0xFFu) - 127;
  *mult = 0.f;
  *inv = 0.f;
  if (e >= -104) {
    *mult = u2f((uint32_t)(22 - e + 127) << 23);
    *inv = u2f((uint32_t)(e - 22 + 127) << 23);
  }
}
static int fx_fixed(float x, float mult) {
  const int v = (int)rintf(x * mult);
  return v < 8388607 ? v : 8388607;
}

static uint64_t rng = 88172645463325252ull;
static uint32_t rnd(void) { rng ^= rng << 13; rng ^= rng >> 7; rng ^= rng << 17; return (uint32_t)(rng >> 16); }
static float rndu(void) { return (float)(rnd() & 0xFFFFFF) / 8388608.0f - 1.0f; }

int main(void) {
  long failures = 0, cases = 0;
  double worst_rel = 0.0;
  const float mags[] = {1.0f, 0.0883f, 3.7e-5f, 1e-20f, 2.0f, 0.5f, 4096.0f, 7.3e12f, 1.0e-30f};
  for (unsigned mi = 0; mi < sizeof(mags) / sizeof(mags[0]); mi++) {
    for (int trial = 0; trial < 4000; trial++) {
      float x[128];
      float amax = 0.f;
      for (int j = 0; j < 128; j++) {
        x[j] = rndu() * mags[mi];
        if ((trial & 7) == 0 && j == 5) x[j] = (trial & 8) ? -mags[mi] : mags[mi];      /* exact powers of two and extremes */
        if ((trial & 15) == 1) x[j] = (j & 1) ? 0.f : x[j];
        amax = fmaxf(amax, fabsf(x[j]));
      }
      float mult, inv;
      fx_scale(amax, &mult, &inv);
      int qf[128];
      for (int j = 0; j < 128; j++) {
        qf[j] = fx_fixed(x[j], mult);
        const int s0 = (int8_t)((qf[j] >> 16) & 0xFF), s1 = (qf[j] >> 8) & 0xFF, s2 = qf[j] & 0xFF;
        if (qf[j] < -8388608 || qf[j] > 8388607 || s0 * 65536 + s1 * 256 + s2 != qf[j]) failures++;
      }
      for (int bits = 4; bits <= 8; bits += 4) {
        const int qmax = bits == 4 ? 7 : 127;
        for (int c = 0; c < 8; c++) {                       /* the 8 lane chunks of a row */
          int code[16];
          int64_t exact = 0;
          double ref = 0.0;
          for (int j = 0; j < 16; j++) {
            code[j] = (int)(rnd() % (2 * qmax + 1)) - qmax;
            if ((trial & 3) == 2) code[j] = (j & 1) ? qmax : -qmax;
            exact += (int64_t)code[j] * qf[c * 16 + j];
            ref += (double)code[j] * (double)x[c * 16 + j];
          }
          /* slice sums as the device forms them: int8 from the codes, int4 from the nibbles u = code + 8 with the
             start value -8 * (sum of the slice's bytes) */
          int a[3];
          for (int s = 0; s < 3; s++) {
            int acc = 0, colsum = 0;
            for (int j = 0; j < 16; j++) {
              const int q = qf[c * 16 + j];
              const int byte = s == 0 ? (int8_t)((q >> 16) & 0xFF) : (s == 1 ? (q >> 8) & 0xFF : q & 0xFF);
              colsum += byte;
              acc += (bits == 4 ? code[j] + 8 : code[j]) * byte;
            }
            a[s] = bits == 4 ? acc - 8 * colsum : acc;
          }
          if ((int64_t)a[0] * 65536 + (int64_t)a[1] * 256 + a[2] != exact) failures++;
          const float comb = fmaf((float)a[0], 65536.0f, (float)(a[1] * 256 + a[2]));
          if (fabs((double)comb - (double)exact) > ldexp(fabs((double)exact), -23) + 8.0) failures++;
          const double got = (double)comb * (double)inv;
          const double bound = 16.0 * qmax * ldexp((double)amax, -23) * 1.01 + 8.0 * (double)inv + ldexp(fabs(ref), -22);
          if (mult != 0.f && fabs(got - ref) > bound) failures++;
          if (mult != 0.f && ref != 0.0) {
            const double rel = fabs(got - ref) / (16.0 * qmax * (double)amax);
            if (rel > worst_rel) worst_rel = rel;
          }
          cases++;
        }
      }
    }
  }
  printf("cases %ld, worst error / (16 qmax max|x|) %.3g, failures %ld\n", cases, worst_rel, failures);
  return failures != 0;
}
