/* Exhaustive check behind div_qmax() in statequant_b200/csrc/common.cuh: for every float x in [1e-8, 3e38] and
   c in {127, 7}, fma(fma(-c, x r, x), r, x r) with r = RN(1 / c) equals the IEEE quotient x / c.  Prints the number
   of mismatches per constant (0 expected) and returns it. */
#include <stdio.h>
#include <stdint.h>
#include <string.h>
#include <math.h>
int main(void) {
  const float cs[2] = {127.0f, 7.0f};
  long long total_bad = 0;
  for (int ci = 0; ci < 2; ci++) {
    const float c = cs[ci];
    const float r = 1.0f / c;
    long long bad = 0, tested = 0;
    uint32_t lo, hi; float flo = 1e-8f, fhi = 3.0e38f;
    memcpy(&lo, &flo, 4); memcpy(&hi, &fhi, 4);
    #pragma omp parallel for reduction(+:bad,tested) schedule(static)
    for (long long u = lo; u <= (long long)hi; u++) {
      uint32_t uu = (uint32_t)u; float x; memcpy(&x, &uu, 4);
      const float q = x / c;
      const float q0 = x * r;
      const float e = fmaf(-c, q0, x);
      const float q1 = fmaf(e, r, q0);
      tested++;
      if (q != q1) bad++;
    }
    printf("c=%g r=%a tested %lld mismatches %lld\n", c, r, tested, bad);
    total_bad += bad;
  }
  return total_bad != 0;
}
