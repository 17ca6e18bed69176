// The state pass of one value head of the staged kernel: the dot products of LPR row
// passes with the read-out vectors, reduced so that lane c of a row group ends up with the finished sums of pass
// p0 + c (the row it then owns in the epilogue).
//
// The passes are taken PU at a time (PU unrolled, the groups in a loop): the PU partial sums of a group are reduced by
// a transposing butterfly over PU lanes (PU - 1 shuffles per vector) followed by plain xor rounds over the remaining
// lanes of the row.  PU = LPR is the cheapest in shuffles; a smaller PU keeps the loop body short enough to stay in
// the instruction cache, which matters more.
#pragma once
#include "common.cuh"

namespace sqb {

#ifndef SQB_PASS_UNROLL
#define SQB_PASS_UNROLL 4
#endif

template <int PU>
__device__ __forceinline__ float transpose_reduce_n(float (&v)[PU], int c) {
#pragma unroll
  for (int h = PU / 2; h >= 1; h >>= 1) {
    const bool up = (c & h) != 0;
#pragma unroll
    for (int j = 0; j < h; j++) {
      const float send = up ? v[j] : v[j + h];
      const float keep = up ? v[j + h] : v[j];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, send, h);
    }
  }
  return v[0];
}

// scs: the head's scales; for axis-v states load_slice(gv) reloads vq / vk with group gv's scales folded in.
// CHECK: (axis-v states) look at every pass whether its rows belong to a new scale group
template <int BITS, bool AXK, bool TWO, int LPR, bool CHECK = true, class Slice>
__device__ __forceinline__ void pass_rows(const uint8_t* codes, const unsigned short* scs, const float2 (&vq)[8],
                                          const float2 (&vk)[8], int p0, int npass, int row_base, int G, int NG, int gl,
                                          int c, int rl, int& cur_gv, Slice load_slice, float& tq, float& tk) {
  constexpr int DK = LPR * 16;
  constexpr int RPP = 32 / LPR;
  constexpr int CB = 16 * BITS / 8;
  constexpr int ROWB = DK * BITS / 8;
  constexpr int PU = SQB_PASS_UNROLL < LPR ? SQB_PASS_UNROLL : LPR;
  tq = 0.f;
  tk = 0.f;
  for (int g = 0; g < LPR / PU; g++) {
    if (p0 + g * PU >= npass) break;                       // uniform
    float pq[PU], pk[PU];
#pragma unroll
    for (int p = 0; p < PU; p++) {
      pq[p] = 0.f;
      pk[p] = 0.f;
      const int pass = p0 + g * PU + p;
      if (pass < npass) {                                  // uniform
        const int row = row_base + pass * RPP + rl;
        if constexpr (!AXK && CHECK) {
          const int gv = (row_base + pass * RPP) / G;      // uniform over the warp: G is a multiple of RPP
          if (gv != cur_gv) { cur_gv = gv; load_slice(gv); }
        }
        float2 f[8];
        decode16<BITS>(codes + row * ROWB + c * CB, f);
        float2 aq0 = make_float2(0.f, 0.f), aq1 = aq0, ak0 = aq0, ak1 = aq0;
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          aq0 = __ffma2_rn(f[j], vq[j], aq0);
          aq1 = __ffma2_rn(f[j + 1], vq[j + 1], aq1);
          if constexpr (TWO) {
            ak0 = __ffma2_rn(f[j], vk[j], ak0);
            ak1 = __ffma2_rn(f[j + 1], vk[j + 1], ak1);
          }
        }
        float sq_ = (aq0.x + aq0.y) + (aq1.x + aq1.y);
        float sk_ = (ak0.x + ak0.y) + (ak1.x + ak1.y);
        if constexpr (AXK) {
          const float sc = h2f(scs[row * NG + gl]);
          sq_ = sq_ * sc;
          sk_ = sk_ * sc;
        }
        pq[p] = sq_;
        pk[p] = sk_;
      }
    }
    float sq = transpose_reduce_n<PU>(pq, c);
    float sk = TWO ? transpose_reduce_n<PU>(pk, c) : 0.f;
#pragma unroll
    for (int o = PU; o < LPR; o <<= 1) {
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if constexpr (TWO) sk += __shfl_xor_sync(0xffffffffu, sk, o);
    }
    if (c / PU == g) { tq = sq; tk = sk; }                 // this lane owns pass p0 + c = p0 + g PU + c % PU
  }
}


// ---- fixed-point variant (states scaled along k, head dim 128) -------------------------------------------------------
// The read-out vectors are held as 24-bit fixed-point numbers with one power-of-two scale per vector, cut into three
// byte slices (top slice signed, the other two unsigned), four columns per 32-bit word.  The codes then meet them in
// integer dot products (dp4a): no int -> float conversion of the codes at all, and every partial sum is exact.  The
// rounding of a vector element to 2^-23 of the vector's largest one is of the size of the roundings of an fp32
// accumulation of the same sums (and it is the only rounding before the scale is applied).
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Power-of-two multiplier that brings a vector of largest magnitude amax into (-2^23, 2^23], and its inverse.
// Vectors below 2^-104 count as zero; a non-finite amax poisons the inverse so that the outputs are NaN.
__device__ __forceinline__ void fx_scale(float amax, float& mult, float& inv) {
  const int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xFFu) - 127;
  mult = 0.f;
  inv = 0.f;
  if (e >= -104) {
    mult = __uint_as_float(static_cast<uint32_t>(22 - e + 127) << 23);
    inv = __uint_as_float(static_cast<uint32_t>(e - 22 + 127) << 23);
  }
  if (!(amax <= 3.0e38f)) inv = __uint_as_float(0x7FC00000u);
}
__device__ __forceinline__ int fx_fixed(float x, float mult) {
  return min(__float2int_rn(x * mult), 8388607);
}
// byte B of x0..x3 -> one word in the order (x0, x1, x2, x3), or (x0, x2, x1, x3) for nibble-packed codes
template <int B, bool SWZ>
__device__ __forceinline__ uint32_t fx_slice_word(int x0, int x1, int x2, int x3) {
  const uint32_t sel = 0x0040u + B * 0x11u;              // (a.byte B, b.byte B)
  const uint32_t lo = __byte_perm(x0, SWZ ? x2 : x1, sel);
  const uint32_t hi = __byte_perm(SWZ ? x1 : x2, x3, sel);
  return __byte_perm(lo, hi, 0x5410);
}

// One lane's four columns (4 lane .. 4 lane + 3) of a vector -> its word of each of the three slices; slice i lies at
// fxw + 32 i.  For nibble-packed codes the words of a lane pair are re-paired so that word 2t holds the even and word
// 2t + 1 the odd columns of columns 8t .. 8t + 7, the order in which code_words<4> delivers the codes.
template <int BITS>
__device__ __forceinline__ void put_fx_slices(uint32_t* fxw, int lane, int x0, int x1, int x2, int x3) {
  constexpr bool SWZ = BITS == 4;
  uint32_t w[3] = {fx_slice_word<2, SWZ>(x0, x1, x2, x3), fx_slice_word<1, SWZ>(x0, x1, x2, x3),
                   fx_slice_word<0, SWZ>(x0, x1, x2, x3)};
#pragma unroll
  for (int i = 0; i < 3; i++) {
    if constexpr (SWZ) {
      const uint32_t o = __shfl_xor_sync(0xffffffffu, w[i], 1);
      w[i] = (lane & 1) ? __byte_perm(o, w[i], 0x7632) : __byte_perm(w[i], o, 0x5410);
    }
    fxw[i * 32 + lane] = w[i];
  }
}

// 16 codes of a lane chunk as four words of bytes (4-bit: unsigned nibbles, even columns of each 8 first)
template <int BITS>
__device__ __forceinline__ void code_words(const uint8_t* p, uint32_t (&b)[4]) {
  if constexpr (BITS == 4) {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
    b[0] = w.x & 0x0F0F0F0Fu; b[1] = (w.x >> 4) & 0x0F0F0F0Fu;
    b[2] = w.y & 0x0F0F0F0Fu; b[3] = (w.y >> 4) & 0x0F0F0F0Fu;
  } else {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    b[0] = w.x; b[1] = w.y; b[2] = w.z; b[3] = w.w;
  }
}
// sum over the chunk of code * fixed-point vector element, as a float; i0: start values of the three slice sums
// (-8 * the slice's column sum for 4-bit codes, whose nibbles carry an offset of 8; 0 for 8-bit codes)
__device__ __forceinline__ float fx_dot16(const uint32_t (&b)[4], const uint32_t (&s)[3][4], const int (&i0)[3]) {
  int a0 = i0[0], a1 = i0[1], a2 = i0[2];
#pragma unroll
  for (int w = 0; w < 4; w++) {
    a0 = dp4a_ss(b[w], s[0][w], a0);
    a1 = dp4a_su(b[w], s[1][w], a1);
    a2 = dp4a_su(b[w], s[2][w], a2);
  }
  return fmaf(static_cast<float>(a0), 65536.0f, static_cast<float>(a1 * 256 + a2));
}

template <int BITS, bool TWO, int LPR, int PUX = SQB_PASS_UNROLL>
__device__ __forceinline__ void pass_rows_fx(const uint8_t* codes, const unsigned short* scs,
                                             const uint32_t (&fq)[3][4], const uint32_t (&fk)[3][4],
                                             const int (&iq)[3], const int (&ik)[3], int p0, int npass, int row_base,
                                             int NG, int gl, int c, int rl, float& tq, float& tk) {
  constexpr int DK = LPR * 16;
  constexpr int RPP = 32 / LPR;
  constexpr int CB = 16 * BITS / 8;
  constexpr int ROWB = DK * BITS / 8;
  constexpr int PU = PUX < LPR ? PUX : LPR;
  tq = 0.f;
  tk = 0.f;
  for (int g = 0; g < LPR / PU; g++) {
    if (p0 + g * PU >= npass) break;                       // uniform
    float pq[PU], pk[PU];
#pragma unroll
    for (int p = 0; p < PU; p++) {
      pq[p] = 0.f;
      pk[p] = 0.f;
      const int pass = p0 + g * PU + p;
      if (pass < npass) {                                  // uniform
        const int row = row_base + pass * RPP + rl;
        uint32_t b[4];
        code_words<BITS>(codes + row * ROWB + c * CB, b);
        const float sc = h2f(scs[row * NG + gl]);
        pq[p] = fx_dot16(b, fq, iq) * sc;
        if constexpr (TWO) pk[p] = fx_dot16(b, fk, ik) * sc;
      }
    }
    float sq = transpose_reduce_n<PU>(pq, c);
    float sk = TWO ? transpose_reduce_n<PU>(pk, c) : 0.f;
#pragma unroll
    for (int o = PU; o < LPR; o <<= 1) {
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if constexpr (TWO) sk += __shfl_xor_sync(0xffffffffu, sk, o);
    }
    if (c / PU == g) { tq = sq; tk = sk; }
  }
}

}  // namespace sqb
