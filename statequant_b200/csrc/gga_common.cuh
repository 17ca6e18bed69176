// What the GGA / STEP kernels share: the argument block, fp16 factor clamping, the E4M3 codec of the window.
#pragma once
#include "common.cuh"

namespace sqb {

struct GgaArgs {
  uint8_t* blob; long long stride;
  const int* offs; const int* bits; const float* w;
  long long qoff; int qsz;
  int HV, HK, DK, DV, M, pw, group, rows;
  const int* idx;
  const uint8_t *q, *k, *v, *a, *b, *A_log, *dt_bias;
  long long sq, sk, sv, sa, sb;
  uint8_t* out; long long so;
  int dt_qk, dt_v, dt_ab, dt_alog, dt_dtb, dt_out;
  float scale;
  // store / load / fit
  const float* X; float* Y; long long P;
  int* status;        // device health word: [0] counts CTAs whose bounded wait ran out
  unsigned long long wait_ns;   // register-tile kernel: how long the wait for its bulk copies may take
  int test_extra_tx;  // test hook: bytes its barrier expects beyond what is copied (so that its wait runs out)
  int skip_packed;    // gga_step_kernel: leave the heads of width 4 / 6 / 8 to the register-tile kernel (gga_reg.cuh)
};

__device__ __forceinline__ float halfc(float x) { return h2f(f2h(fminf(fmaxf(x, FP16_TINY), 65504.0f))); }

// |y| <= 448 rounded to the E4M3 grid, nearest even (spacing 2^(e-3) for exponent e >= -6)
__device__ __forceinline__ float e4m3_round(float y) {
  int e = static_cast<int>((__float_as_uint(y) >> 23) & 255u) - 127;
  e = max(e, -6);
  const float ulp = __uint_as_float(static_cast<uint32_t>(e - 3 + 127) << 23);
  const float inv = __uint_as_float(static_cast<uint32_t>(3 - e + 127) << 23);     // 1 / ulp, a power of two: exact
  return rintf(y * inv) * ulp;
}
__device__ __forceinline__ uint8_t e4m3_byte(float y) {          // y on the grid, |y| <= 448
  const uint32_t u = __float_as_uint(y);
  const uint8_t s = static_cast<uint8_t>((u >> 24) & 0x80u);
  const float a = fabsf(y);
  if (a == 0.f) return s;
  const int e = static_cast<int>((u >> 23) & 255u) - 127;
  if (e < -6) return s | static_cast<uint8_t>(__float2int_rn(a * 512.0f));
  return s | static_cast<uint8_t>(((e + 7) << 3) | ((u >> 20) & 7u));
}
__device__ __forceinline__ float e4m3_val(uint8_t b) {
  const int e = (b >> 3) & 15, m = b & 7;
  const float v = e == 0 ? static_cast<float>(m) * 0.001953125f
                         : __uint_as_float((static_cast<uint32_t>(e - 7 + 127) << 23) | (static_cast<uint32_t>(m) << 20));
  return (b & 0x80) ? -v : v;
}

}  // namespace sqb
