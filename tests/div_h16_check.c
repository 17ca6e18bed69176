#include <stdio.h>
#include <stdint.h>
#include <string.h>
#include <math.h>
#include <stdlib.h>
/* Check behind div_h16() in statequant_b200/csrc/gga.cuh: for EVERY positive fp16 divisor r (subnormals included,
   2^-24 .. 65504) and 20 000 pseudo-random dividends x of either sign with exponents in [2^-100, 2^82] each,
   fma(fma(-r, x rr, x), rr, x rr) with rr = RN(1 / r) equals the IEEE quotient x / r.  Returns the mismatch count. */
static float h2f(uint16_t h) { // positive only
  int e = (h >> 10) & 31, m = h & 1023;
  if (e == 0) return ldexpf((float)m, -24);
  return ldexpf((float)(1024 + m), e - 25);
}
int main(void) {
  long long bad = 0, tested = 0, badrange = 0;
  #pragma omp parallel for reduction(+:bad,tested,badrange) schedule(dynamic, 64)
  for (int h = 1; h < 0x7C00; h++) {
    const float r = h2f((uint16_t)h);
    const float rr = 1.0f / r;
    uint64_t s = 0x9E3779B97F4A7C15ull * (uint64_t)(h + 1);
    for (int it = 0; it < 20000; it++) {
      s ^= s << 13; s ^= s >> 7; s ^= s << 17;
      uint32_t u = (uint32_t)(s >> 32);
      // exponent range limited so that the quotient stays normal: x in [2^-60, 2^40]
      uint32_t ex = 27 + (u >> 23) % 183;   // x in [2^-100, 2^82]
      uint32_t bits = (u & 0x807FFFFFu) | (ex << 23);
      float x; memcpy(&x, &bits, 4);
      const float q = x / r;
      const float q0 = x * rr;
      const float q1 = fmaf(fmaf(-r, q0, x), rr, q0);
      tested++;
      if (q != q1) { bad++; if (fabsf(q) < 1e-37f || fabsf(q) > 1e37f) badrange++; }
    }
  }
  printf("tested %lld mismatches %lld (of which out of normal range %lld)\n", tested, bad, badrange);
  return bad != 0;
}
