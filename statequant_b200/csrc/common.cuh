// Shared device helpers of the packed-state decode kernels (sm_100a).
//
// Numerics contract (what "the same bytes as the reference" rests on):
//   * scales:   s = fp16_rn(max(amax, 1e-8) / qmax) clamped below at 2^-24, IEEE division
//   * payloads: code = clamp(rint(x / s)), IEEE division, round half to even
//   * no fast-math; this file is compiled with --fmad=false, so every fused multiply-add below is written
//     explicitly (fmaf / __ffma2_rn) and every separately rounded product stays separate.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sqb {

constexpr int NT = 128;  // threads per CTA
constexpr int NW = 4;    // warps per CTA
constexpr float FP16_TINY = 5.960464477539063e-08f;   // 2^-24
constexpr float FP16_MIN_NORMAL = 6.103515625e-05f;   // 2^-14
constexpr float MAGIC = 12582912.0f;                  // 1.5 * 2^23: adding it rounds to an integer (half-even)

enum { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2 };
enum { K_GDN = 0, K_M2 = 1, K_KDA = 2 };

__device__ __forceinline__ float ldf(const void* p, int dt, long long i) {
  if (dt == DT_F32) return reinterpret_cast<const float*>(p)[i];
  if (dt == DT_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void stf(void* p, int dt, long long i, float v) {
  if (dt == DT_F32) reinterpret_cast<float*>(p)[i] = v;
  else if (dt == DT_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}
__host__ __device__ __forceinline__ int dt_size(int dt) { return dt == DT_F32 ? 4 : 2; }

// Activation loads in two steps, so that a group of loads is in flight together: the raw bits first (nothing waits
// for them), the conversion to fp32 where the values are needed.  (ldf converts at once, which makes every load of a
// sequence wait for the one before.)
__device__ __forceinline__ uint32_t ld1_raw(const void* p, int dt, long long i) {
  if (dt == DT_F32) return reinterpret_cast<const uint32_t*>(p)[i];
  return reinterpret_cast<const unsigned short*>(p)[i];
}
__device__ __forceinline__ float cvt_raw(uint32_t w, int dt) {
  if (dt == DT_F32) return __uint_as_float(w);
  if (dt == DT_BF16) return __uint_as_float(w << 16);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(w)));
}
// Elements i .. i + 3 (i a multiple of 4) as loaded, untouched: unpacking a loaded word is already a use that waits
// for the load, so it is left to cvt4_raw.  vec: the row is read by one 8- or 16-byte load (the address allows it).
struct Raw4 { uint4 v; bool vec; };
__device__ __forceinline__ Raw4 ld4_raw(const uint8_t* p, int dt, long long i) {
  Raw4 r;
  r.v = make_uint4(0u, 0u, 0u, 0u);
  if (dt == DT_F32) {
    const uint8_t* q = p + 4 * i;
    r.vec = (reinterpret_cast<uintptr_t>(q) & 15) == 0;
    if (r.vec) {
      r.v = *reinterpret_cast<const uint4*>(q);
    } else {
      r.v.x = reinterpret_cast<const uint32_t*>(q)[0]; r.v.y = reinterpret_cast<const uint32_t*>(q)[1];
      r.v.z = reinterpret_cast<const uint32_t*>(q)[2]; r.v.w = reinterpret_cast<const uint32_t*>(q)[3];
    }
  } else {
    const uint8_t* q = p + 2 * i;
    r.vec = (reinterpret_cast<uintptr_t>(q) & 7) == 0;
    if (r.vec) {
      const uint2 t = *reinterpret_cast<const uint2*>(q);
      r.v.x = t.x; r.v.y = t.y;
    } else {
      r.v.x = reinterpret_cast<const unsigned short*>(q)[0]; r.v.y = reinterpret_cast<const unsigned short*>(q)[1];
      r.v.z = reinterpret_cast<const unsigned short*>(q)[2]; r.v.w = reinterpret_cast<const unsigned short*>(q)[3];
    }
  }
  return r;
}
__device__ __forceinline__ void cvt4_raw(const Raw4& r, int dt, float (&f)[4]) {
  if (dt == DT_F32 || !r.vec) {
    f[0] = cvt_raw(r.v.x, dt); f[1] = cvt_raw(r.v.y, dt); f[2] = cvt_raw(r.v.z, dt); f[3] = cvt_raw(r.v.w, dt);
  } else {
    f[0] = cvt_raw(r.v.x & 0xFFFFu, dt); f[1] = cvt_raw(r.v.x >> 16, dt);
    f[2] = cvt_raw(r.v.y & 0xFFFFu, dt); f[3] = cvt_raw(r.v.y >> 16, dt);
  }
}

__device__ __forceinline__ float h2f(unsigned short h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ unsigned short f2h(float f) { return __half_as_ushort(__float2half_rn(f)); }
__device__ __forceinline__ float bf2f(unsigned short b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
__device__ __forceinline__ unsigned short f2bf(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }

// Quantizer scale of a group with absolute maximum amax (see the contract above).
// x / qmax for the two code ranges in use, without the division: with r = RN(1 / qmax), q0 = RN(x r),
// q = fma(fma(-qmax, q0, x), r, q0) equals div_rn(x, qmax) for EVERY finite float x in [1e-8, 3e38] when qmax is 127
// or 7 (checked exhaustively on the host, tests/div_const_check.c); anything else takes the IEEE division.
__device__ __forceinline__ float div_qmax(float x, float qmax) {
  if ((qmax == 127.0f || qmax == 7.0f) && x <= 3.0e38f) {
    const float r = qmax == 127.0f ? 0x1.020408p-7f : 0x1.24924ap-3f;
    const float q0 = __fmul_rn(x, r);
    return __fmaf_rn(__fmaf_rn(-qmax, q0, x), r, q0);
  }
  return __fdiv_rn(x, qmax);
}
__device__ __forceinline__ float fp16_scale(float amax, float qmax) {
  float s = div_qmax(fmaxf(amax, 1e-8f), qmax);
  s = h2f(f2h(s));
  return fmaxf(s, FP16_TINY);
}
// 1 / s to within a few ulp (one MUFU instruction); enough wherever the result is verified afterwards (round_fast)
__device__ __forceinline__ float rcp_approx(float s) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(s));
  return r;
}
// clamp(rint(x / s), +-qmax), exact
__device__ __forceinline__ float rq_exact(float x, float s, float qmax) {
  return fminf(fmaxf(rintf(__fdiv_rn(x, s)), -qmax), qmax);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- int8 -> fp32 through the mantissa (no integer->float conversion instruction) --------------------------------
// wx = word ^ 0x80808080 holds the four codes as unsigned bytes c + 128; byte i lands in the mantissa of 2^23.
template <int I>
__device__ __forceinline__ float byte_to_f(uint32_t wx) {
  return __uint_as_float(__byte_perm(wx, 0x4B000000u, 0x7540 | I)) - 8388736.0f;   // 2^23 + 128
}

// ---- int4 -> fp32, eight codes of one 32-bit word ----------------------------------------------------------------
// Nibble i (bits 4i..4i+3, key column i of the word) is masked in place into the mantissa of 2^23, which yields
// (u - 8) * 16^e exactly after the bias is subtracted, with e = i for i <= 4 and e = i - 5 for i = 5, 6, 7 (those
// three come from the word shifted down by 20).  The factor 16^-e is a power of two, so it is folded exactly into
// whatever the code is multiplied with (the read-out vector, or the scale).  Pair p holds columns 2p, 2p+1.
// (w & mask) | k as ONE lop3 (the mask is the immediate, k comes in a register; written as two C operators the
// compiler spends an AND and an OR with two immediates)
template <uint32_t MASK>
__device__ __forceinline__ float nib_f(uint32_t w, uint32_t k) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w), "n"(MASK), "r"(k));
  return __uint_as_float(r);
}
__device__ __forceinline__ void unpack_nib8(uint32_t w, float2 f[4]) {
  const uint32_t w2 = w >> 20;
  uint32_t K = 0x4B000000u;
  asm volatile("" : "+r"(K));                 // keep the constant in a register
  float2 t;
  t.x = nib_f<0x0000000Fu>(w, K);
  t.y = nib_f<0x000000F0u>(w, K);
  f[0] = __fadd2_rn(t, make_float2(-8388616.0f, -8388736.0f));     // 2^23 + 8, 2^23 + 8*16
  t.x = nib_f<0x00000F00u>(w, K);
  t.y = nib_f<0x0000F000u>(w, K);
  f[1] = __fadd2_rn(t, make_float2(-8390656.0f, -8421376.0f));     // + 8*16^2, + 8*16^3
  t.x = nib_f<0x000F0000u>(w, K);
  t.y = nib_f<0x0000000Fu>(w2, K);
  f[2] = __fadd2_rn(t, make_float2(-8912896.0f, -8388616.0f));     // + 8*16^4, + 8
  t.x = nib_f<0x000000F0u>(w2, K);
  t.y = nib_f<0x00000F00u>(w2, K);
  f[3] = __fadd2_rn(t, make_float2(-8388736.0f, -8390656.0f));
}

// 16^-e of column j (0..7) of a word, matching unpack_nib8
__device__ __forceinline__ float nib_prescale(int j) {
  const int e = j <= 4 ? j : j - 5;
  return __uint_as_float(static_cast<uint32_t>(127 - 4 * e) << 23);
}

// floats per row of the fold's value-major L tile (M coefficients, padded so that rows fall on distinct banks)
__host__ __device__ inline int fold_lm(int M) { return (M < 4 ? 4 : M) + 4; }

}  // namespace sqb
