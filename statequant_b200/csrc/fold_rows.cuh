// The fold of one value head (used by the fold kernel):
//     S[v][k] = decay * (code[v][k] * scale) + sum_i L[v][i] * R[i][k]      (slot order, one fma.rn per term)
// re-rounded to codes with fresh scales and written back in place.
//
// Shared-memory operands: codes / scs are the head's stored state (a stage buffer); R[i][.] is slot i's key in the
// lane-chunk layout (16 columns + 4 floats of padding per lane, so 128-bit reads of the LPR chunks of a row hit
// distinct banks); L is value-major, L[v * LM + i] = decayed buffered value of slot i at row v, LM = fold_lm(M), so
// a row's M coefficients are one or two 128-bit reads.  A lane owns 16 columns of two rows at a time; the slot
// loop is unrolled for the usual buffer length 8 (immediate offsets, no loop control in the hot part).
#pragma once
#include "common.cuh"

namespace sqb {

#ifndef SQB_FOLD_UNROLL8
#define SQB_FOLD_UNROLL8 1
#endif

template <int LPR, int MC>
__device__ __forceinline__ void fold_mac(float2 (&a0)[8], float2 (&a1)[8], const float* Rc, const float* l0p,
                                         const float* l1p, int M) {
  constexpr int RDK = LPR * 20;
  if constexpr (MC == 8) {
    const float4 x0 = *reinterpret_cast<const float4*>(l0p), x1 = *reinterpret_cast<const float4*>(l0p + 4);
    const float4 y0 = *reinterpret_cast<const float4*>(l1p), y1 = *reinterpret_cast<const float4*>(l1p + 4);
    const float l0[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    const float l1[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float4* rrow = reinterpret_cast<const float4*>(Rc + i * RDK);
      const float2 la = make_float2(l0[i], l0[i]), lb = make_float2(l1[i], l1[i]);
#pragma unroll
      for (int j4 = 0; j4 < 4; j4++) {
        const float4 k4 = rrow[j4];
        const float2 ka = make_float2(k4.x, k4.y), kb = make_float2(k4.z, k4.w);
        a0[2 * j4] = __ffma2_rn(la, ka, a0[2 * j4]);
        a0[2 * j4 + 1] = __ffma2_rn(la, kb, a0[2 * j4 + 1]);
        a1[2 * j4] = __ffma2_rn(lb, ka, a1[2 * j4]);
        a1[2 * j4 + 1] = __ffma2_rn(lb, kb, a1[2 * j4 + 1]);
      }
    }
  } else {
    for (int i = 0; i < M; i++) {
      const float4* rrow = reinterpret_cast<const float4*>(Rc + i * RDK);
      const float2 la = make_float2(l0p[i], l0p[i]), lb = make_float2(l1p[i], l1p[i]);
#pragma unroll
      for (int j4 = 0; j4 < 4; j4++) {
        const float4 k4 = rrow[j4];
        const float2 ka = make_float2(k4.x, k4.y), kb = make_float2(k4.z, k4.w);
        a0[2 * j4] = __ffma2_rn(la, ka, a0[2 * j4]);
        a0[2 * j4 + 1] = __ffma2_rn(la, kb, a0[2 * j4 + 1]);
        a1[2 * j4] = __ffma2_rn(lb, ka, a1[2 * j4]);
        a1[2 * j4 + 1] = __ffma2_rn(lb, kb, a1[2 * j4 + 1]);
      }
    }
  }
}

// code * scale (* 16^-e of the 4-bit unpacking), then * decay: two roundings, as the reference does them
template <int BITS, bool VDEC>
__device__ __forceinline__ void fold_dequant(float2 (&a)[8], float sc, float alphan, const float* aec) {
#pragma unroll
  for (int p = 0; p < 8; p++) {
    float2 s2;
    if constexpr (BITS == 4) s2 = make_float2(sc * nib_prescale((2 * p) & 7), sc * nib_prescale((2 * p + 1) & 7));
    else s2 = make_float2(sc, sc);
    a[p] = __fmul2_rn(a[p], s2);
    float2 d2 = make_float2(alphan, alphan);
    if constexpr (VDEC) d2 = make_float2(aec[2 * p], aec[2 * p + 1]);
    a[p] = __fmul2_rn(a[p], d2);
  }
}

// The verified candidates of round_fast, clamped to the code range.  A scale that is subnormal in fp16 can be far
// enough below absmax / qmax for the largest quotients to round beyond qmax; the candidate is then still the right
// unclamped integer, and clamping it is what clamp(rint(div_rn(x, s))) does.  A normal fp16 scale is within 2^-11 of
// absmax / qmax, so no quotient exceeds qmax (1 + 2^-10) and none rounds beyond qmax: callers skip the clamp then.
template <int BITS>
__device__ __forceinline__ float2 (&clamp_codes(float2 (&t)[8]))[8] {
  constexpr float QMAX = BITS == 4 ? 7.0f : 127.0f;
  constexpr float MB = BITS == 4 ? MAGIC + 8.0f : MAGIC;
#pragma unroll
  for (int p = 0; p < 8; p++) {
    t[p].x = fminf(fmaxf(t[p].x, MB - QMAX), MB + QMAX);
    t[p].y = fminf(fmaxf(t[p].y, MB - QMAX), MB + QMAX);
  }
  return t;
}

__device__ __forceinline__ void fold_store_f32(float* p, const float2 (&a)[8]) {
#pragma unroll
  for (int j = 0; j < 4; j++)
    reinterpret_cast<float4*>(p)[j] = make_float4(a[2 * j].x, a[2 * j].y, a[2 * j + 1].x, a[2 * j + 1].y);
}

// round_fast with one scale (sc[j]) and approximate reciprocal (rc[j]) per column: the same test, per element;
// smin: the smallest of the 16 scales (the caller clamps the candidates only if one of them is subnormal in fp16)
__device__ __forceinline__ bool round_fast_cols(const float2 (&x)[8], const float* sc, const float* rc, float mb,
                                                float2 (&t)[8], float& smin) {
  const float2 m2 = make_float2(mb, mb), nm2 = make_float2(-mb, -mb), h2 = make_float2(0.49998474f, 0.49998474f);
  float worst = -1.0f;                                   // max over elements of |rem| - thr; the chunk passes if < 0
  smin = 1.0f;
#pragma unroll
  for (int p = 0; p < 8; p++) {
    const float2 s2 = *reinterpret_cast<const float2*>(sc + 2 * p), r2 = *reinterpret_cast<const float2*>(rc + 2 * p);
    smin = fminf(smin, fminf(s2.x, s2.y));
    t[p] = __ffma2_rn(x[p], r2, m2);
    const float2 c = __fadd2_rn(t[p], nm2);
    const float2 rem = __ffma2_rn(make_float2(-c.x, -c.y), s2, x[p]);
    const float2 thr = __fmul2_rn(s2, h2);
    worst = fmaxf(worst, fmaxf(fabsf(rem.x) - thr.x, fabsf(rem.y) - thr.y));
  }
  return worst < 0.f;
}

// sync(): barrier among the 128 threads that fold (returns false if the CTA is aborting).  Returns false on abort.
// PAD: the codes lie in the padded pieces of the tensor-core kernel (16 bytes after every 16 rows, mma_pass.cuh)
template <int BITS, bool AXK, int LPR, bool VDEC, bool PAD = false, class Sync>
__device__ __forceinline__ bool fold_rows(const uint8_t* codes, const unsigned short* scs, const float* R,
                                          const float* L, const float* ae, float alphan, int DV, int G, int M,
                                          float* cmax, uint8_t* Sh, unsigned short* SCh, int warp, int lane, int tid,
                                          Sync sync, float* Yout = nullptr) {
  constexpr int DK = LPR * 16;
  constexpr int RPP = 32 / LPR;
  constexpr int CB = 16 * BITS / 8;
  constexpr int ROWB = DK * BITS / 8;
  constexpr int PPW = 2;
  constexpr float QMAX = BITS == 4 ? 7.0f : 127.0f;
  [[maybe_unused]] constexpr float MB = BITS == 4 ? MAGIC + 8.0f : MAGIC;
  const int c = lane & (LPR - 1), rl = lane / LPR;
  const int LM = fold_lm(M);
  const float* Rc = R + c * 20;
  const float* aec = VDEC ? ae + c * 16 : nullptr;

  if constexpr (AXK) {
    const int NG = DK / G;
    const int gl = (c * 16) / G;
    const int lpg = G / 16;
    constexpr int BR = NW * PPW * RPP;
    const int niter = (DV + BR - 1) / BR;
    for (int it = 0; it < niter; it++) {
      const int row0 = it * BR + warp * (PPW * RPP) + rl, row1 = row0 + RPP;
      const bool v0 = row0 < DV, v1 = row1 < DV;
      const int r0 = v0 ? row0 : 0, r1 = v1 ? row1 : 0;
      float2 a0[8], a1[8];
      decode16<BITS>(codes + r0 * ROWB + (PAD ? (r0 >> 4) * 16 : 0) + c * CB, a0);
      decode16<BITS>(codes + r1 * ROWB + (PAD ? (r1 >> 4) * 16 : 0) + c * CB, a1);
      fold_dequant<BITS, VDEC>(a0, h2f(scs[r0 * NG + gl]), alphan, aec);
      fold_dequant<BITS, VDEC>(a1, h2f(scs[r1 * NG + gl]), alphan, aec);
      if (SQB_FOLD_UNROLL8 && M == 8) fold_mac<LPR, 8>(a0, a1, Rc, L + r0 * LM, L + r1 * LM, M);
      else fold_mac<LPR, 0>(a0, a1, Rc, L + r0 * LM, L + r1 * LM, M);
      if (Yout != nullptr) {                          // read-out mode: the advanced state as fp32, nothing re-rounded
        if (v0) fold_store_f32(Yout + (long long)r0 * DK + c * 16, a0);
        if (v1) fold_store_f32(Yout + (long long)r1 * DK + c * 16, a1);
        continue;
      }
      // fresh scales: absmax over the group's lanes
      float am0 = 0.f, am1 = 0.f;
#pragma unroll
      for (int p = 0; p < 8; p++) {
        am0 = fmaxf(am0, fmaxf(fabsf(a0[p].x), fabsf(a0[p].y)));
        am1 = fmaxf(am1, fmaxf(fabsf(a1[p].x), fabsf(a1[p].y)));
      }
      for (int o = 1; o < lpg; o <<= 1) {
        am0 = fmaxf(am0, __shfl_xor_sync(0xffffffffu, am0, o));
        am1 = fmaxf(am1, __shfl_xor_sync(0xffffffffu, am1, o));
      }
      const float sc0 = fp16_scale(am0, QMAX), sc1 = fp16_scale(am1, QMAX);
      const bool lead = (c & (lpg - 1)) == 0;
      float2 tt[8];
      if (v0) {
        if (lead) SCh[r0 * NG + gl] = f2h(sc0);
        uint4 pk;
        if (round_fast<8>(a0, sc0, rcp_approx(sc0), MB, tt)) {
          if (sc0 < FP16_MIN_NORMAL) clamp_codes<BITS>(tt);     // only a subnormal scale lets a quotient pass qmax
          pk = pack_codes16<BITS>(tt);
        }
        else pk = round_exact_pack<BITS>(a0[0], a0[1], a0[2], a0[3], a0[4], a0[5], a0[6], a0[7], sc0);
        store_packed16<BITS>(Sh + (long long)r0 * ROWB + c * CB, pk);
      }
      if (v1) {
        if (lead) SCh[r1 * NG + gl] = f2h(sc1);
        uint4 pk;
        if (round_fast<8>(a1, sc1, rcp_approx(sc1), MB, tt)) {
          if (sc1 < FP16_MIN_NORMAL) clamp_codes<BITS>(tt);     // only a subnormal scale lets a quotient pass qmax
          pk = pack_codes16<BITS>(tt);
        }
        else pk = round_exact_pack<BITS>(a1[0], a1[1], a1[2], a1[3], a1[4], a1[5], a1[6], a1[7], sc1);
        store_packed16<BITS>(Sh + (long long)r1 * ROWB + c * CB, pk);
      }
    }
    return true;
  } else {
    // scale groups run along d_v: a group of G rows shares one scale per column
    const int wpg = min(NW, G / RPP);               // warps that share a group
    const int ppw = G / (RPP * wpg);                // rows per lane (1 or 2)
    const int gpi = NW / wpg;                       // groups in flight
    const int BR = gpi * G;
    const int niter = (DV + BR - 1) / BR;
    constexpr int CDK = LPR * 20;                   // floats per row of the padded column tables
    for (int it = 0; it < niter; it++) {
      const int gvrow = it * gpi + warp / wpg;
      const bool gvalid = gvrow * G < DV;
      const int row0 = gvrow * G + (warp % wpg) * (ppw * RPP) + rl, row1 = row0 + RPP;
      const bool v0 = row0 < DV, v1 = ppw > 1 && row1 < DV;
      const int r0 = v0 ? row0 : 0, r1 = v1 ? row1 : 0;
      float2 a0[8], a1[8];
      decode16<BITS>(codes + r0 * ROWB + c * CB, a0);
      decode16<BITS>(codes + r1 * ROWB + c * CB, a1);
      uint32_t sw[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};     // the lane's 16 column scales (fp16 pairs), two 128-bit reads
      if (gvalid) {
        const uint4* sp = reinterpret_cast<const uint4*>(scs + gvrow * DK + c * 16);
        const uint4 u0 = sp[0], u1 = sp[1];
        sw[0] = u0.x; sw[1] = u0.y; sw[2] = u0.z; sw[3] = u0.w; sw[4] = u1.x; sw[5] = u1.y; sw[6] = u1.z; sw[7] = u1.w;
      }
#pragma unroll
      for (int p = 0; p < 8; p++) {
        const float s0 = h2f(static_cast<unsigned short>(sw[p] & 0xFFFFu)), s1 = h2f(static_cast<unsigned short>(sw[p] >> 16));
        float2 s2 = make_float2(s0, s1);
        if constexpr (BITS == 4) s2 = make_float2(s0 * nib_prescale((2 * p) & 7), s1 * nib_prescale((2 * p + 1) & 7));
        float2 d2 = make_float2(alphan, alphan);
        if constexpr (VDEC) d2 = make_float2(aec[2 * p], aec[2 * p + 1]);
        a0[p] = __fmul2_rn(__fmul2_rn(a0[p], s2), d2);
        a1[p] = __fmul2_rn(__fmul2_rn(a1[p], s2), d2);
      }
      if (SQB_FOLD_UNROLL8 && M == 8) fold_mac<LPR, 8>(a0, a1, Rc, L + r0 * LM, L + r1 * LM, M);
      else fold_mac<LPR, 0>(a0, a1, Rc, L + r0 * LM, L + r1 * LM, M);
      if (Yout != nullptr) {
        if (v0) fold_store_f32(Yout + (long long)r0 * DK + c * 16, a0);
        if (v1) fold_store_f32(Yout + (long long)r1 * DK + c * 16, a1);
        continue;
      }
      // column maxima over the group's rows: this lane's rows, the lanes of other rows, the other warps
      float cm[16];
#pragma unroll
      for (int p = 0; p < 8; p++) {
        float m0 = 0.f, m1 = 0.f;
        if (v0) { m0 = fabsf(a0[p].x); m1 = fabsf(a0[p].y); }
        if (v1) { m0 = fmaxf(m0, fabsf(a1[p].x)); m1 = fmaxf(m1, fabsf(a1[p].y)); }
        for (int o = LPR; o < 32; o <<= 1) {
          m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
          m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
        }
        cm[2 * p] = m0;
        cm[2 * p + 1] = m1;
      }
      if (!sync()) return false;                      // cmax free (the previous iteration's readers are done)
      if (rl == 0) {
#pragma unroll
        for (int j = 0; j < 16; j++) cmax[warp * CDK + c * 20 + j] = cm[j];
      }
      if (!sync()) return false;
      float* ssc = cmax + NW * CDK;                   // scale of every column of every group in flight
      float* rsc = ssc + NW * CDK;                    // and its approximate reciprocal
      for (int e = tid; e < gpi * DK; e += NT) {
        const int gi = e / DK, k = e - gi * DK;
        const int pk_ = (k >> 4) * 20 + (k & 15);       // lane-chunk layout: 16 columns + 4 floats of padding
        float am = 0.f;
        for (int w = 0; w < wpg; w++) am = fmaxf(am, cmax[(gi * wpg + w) * CDK + pk_]);
        const float sc = fp16_scale(am, QMAX);
        ssc[gi * CDK + pk_] = sc;
        rsc[gi * CDK + pk_] = rcp_approx(sc);
        const int gvr = it * gpi + gi;
        if (gvr * G < DV) SCh[gvr * DK + k] = f2h(sc);
      }
      if (!sync()) return false;
      const float* myssc = ssc + (warp / wpg) * CDK + c * 20;
      const float* myrsc = rsc + (warp / wpg) * CDK + c * 20;
      float2 tt[8];
      if (v0) {
        uint4 pk;
        float smin;
        if (round_fast_cols(a0, myssc, myrsc, MB, tt, smin)) {
          if (smin < FP16_MIN_NORMAL) clamp_codes<BITS>(tt);
          pk = pack_codes16<BITS>(tt);
        }
        else pk = round_exact_pack_cols<BITS>(a0[0], a0[1], a0[2], a0[3], a0[4], a0[5], a0[6], a0[7], myssc);
        store_packed16<BITS>(Sh + (long long)r0 * ROWB + c * CB, pk);
      }
      if (v1) {
        uint4 pk;
        float smin;
        if (round_fast_cols(a1, myssc, myrsc, MB, tt, smin)) {
          if (smin < FP16_MIN_NORMAL) clamp_codes<BITS>(tt);
          pk = pack_codes16<BITS>(tt);
        }
        else pk = round_exact_pack_cols<BITS>(a1[0], a1[1], a1[2], a1[3], a1[4], a1[5], a1[6], a1[7], myssc);
        store_packed16<BITS>(Sh + (long long)r1 * ROWB + c * CB, pk);
      }
    }
    return true;
  }
}

}  // namespace sqb
