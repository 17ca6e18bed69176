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

}  // namespace sqb
