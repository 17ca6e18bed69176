// The prefill boundary of a slot table on the device: packing canonical fp32 states into slots.
// (Reading a slot back -- the stored state advanced across its pending buffer -- is the fold kernel run in its
// read-out mode, fold_kernel.cuh.)
//
// slot_write_kernel: one CTA per (row, value head).  S [rows, HV, d_v, d_k] fp32 -> codes and scales of slot idx[row],
// bit for bit what the reference's torch packer writes (kernels/fold.py:111-147 via kernels/slots.py:236-252):
// scale = max(fp16(max(absmax, 1e-8) / qmax), 2^-24) per group, code = clamp(rint(div_rn(x, scale))), 4-bit codes
// two per byte, low nibble first, biased by 8.  The slot's buffer is emptied (counters and running decay zeroed).
#pragma once
#include "step_tma.cuh"

namespace sqb {

struct WriteArgs {
  uint8_t *S, *SC, *GCUR, *NPTR;
  long long sS, sSC, sGC, sN;
  const int* idx;
  const float* X;            // [rows, HV, d_v, d_k]
  int group, HV, DV, rows, nptr, gc_width;   // nptr: counters per slot; gc_width: floats of GCUR per head (1, KDA: d_k)
};

template <int BITS, bool AXK, int LPR>
__global__ void __launch_bounds__(NT) slot_write_kernel(const __grid_constant__ WriteArgs A) {
  constexpr int DK = LPR * 16;
  constexpr int RPP = 32 / LPR;
  constexpr int CB = 16 * BITS / 8;
  constexpr int ROWB = DK * BITS / 8;
  constexpr float QMAX = BITS == 4 ? 7.0f : 127.0f;
  constexpr float MB = BITS == 4 ? MAGIC + 8.0f : MAGIC;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int HV = A.HV, DV = A.DV, G = A.group;
  const int bh = blockIdx.x, b = bh / HV, h = bh - b * HV;
  const long long seq = A.idx != nullptr ? static_cast<long long>(A.idx[b]) : static_cast<long long>(b);
  if (A.idx != nullptr && seq <= 0) return;
  const int c = lane & (LPR - 1), rl = lane / LPR;
  const float* X = A.X + (long long)bh * DV * DK;
  const int NG = AXK ? DK / G : 1;
  const int scn = AXK ? DV * NG : (DV / G) * DK;
  uint8_t* Sh = A.S + seq * A.sS + (long long)h * DV * ROWB;
  unsigned short* SCh = reinterpret_cast<unsigned short*>(A.SC + seq * A.sSC) + (long long)h * scn;

  auto load16 = [&](int row, float2 (&x)[8]) {
    const float4* p = reinterpret_cast<const float4*>(X + (long long)row * DK + c * 16);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float4 v = p[j];
      x[2 * j] = make_float2(v.x, v.y);
      x[2 * j + 1] = make_float2(v.z, v.w);
    }
  };
  if constexpr (AXK) {
    const int lpg = G / 16, gl = (c * 16) / G;
    for (int row = warp * RPP + rl; row < DV; row += NW * RPP) {
      float2 x[8];
      load16(row, x);
      float am = 0.f;
#pragma unroll
      for (int p = 0; p < 8; p++) am = fmaxf(am, fmaxf(fabsf(x[p].x), fabsf(x[p].y)));
      for (int o = 1; o < lpg; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
      const float sc = fp16_scale(am, QMAX);
      if ((c & (lpg - 1)) == 0) SCh[row * NG + gl] = f2h(sc);
      store_packed16<BITS>(Sh + (long long)row * ROWB + c * CB,
                           round_exact_pack<BITS>(x[0], x[1], x[2], x[3], x[4], x[5], x[6], x[7], sc));
    }
  } else {
    // groups of G rows share one scale per column: a warp takes whole groups
    __shared__ float ssc[NW][LPR * 16];
    for (int g0 = warp; g0 * G < DV; g0 += NW) {
      float cm[16];
#pragma unroll
      for (int j = 0; j < 16; j++) cm[j] = 0.f;
      for (int r = rl; r < G; r += RPP) {
        float2 x[8];
        load16(g0 * G + r, x);
#pragma unroll
        for (int p = 0; p < 8; p++) { cm[2 * p] = fmaxf(cm[2 * p], fabsf(x[p].x)); cm[2 * p + 1] = fmaxf(cm[2 * p + 1], fabsf(x[p].y)); }
      }
#pragma unroll
      for (int j = 0; j < 16; j++) {
        for (int o = LPR; o < 32; o <<= 1) cm[j] = fmaxf(cm[j], __shfl_xor_sync(0xffffffffu, cm[j], o));
      }
      __syncwarp();
      if (rl == 0) {
#pragma unroll
        for (int j = 0; j < 16; j++) {
          const float sc = fp16_scale(cm[j], QMAX);
          ssc[warp][c * 16 + j] = sc;
          SCh[g0 * DK + c * 16 + j] = f2h(sc);
        }
      }
      __syncwarp();
      for (int r = rl; r < G; r += RPP) {
        float2 x[8];
        const int row = g0 * G + r;
        load16(row, x);
        store_packed16<BITS>(Sh + (long long)row * ROWB + c * CB,
                             round_exact_pack_cols<BITS>(x[0], x[1], x[2], x[3], x[4], x[5], x[6], x[7], &ssc[warp][c * 16]));
      }
      __syncwarp();
    }
  }
  // empty buffer: counters (all copies, by the CTA of head 0) and this head's running decay
  if (h == 0) {
    int* np = reinterpret_cast<int*>(A.NPTR + seq * A.sN);
    for (int i = tid; i < A.nptr; i += NT) np[i] = 0;
  }
  float* gc = reinterpret_cast<float*>(A.GCUR + seq * A.sGC) + (long long)h * A.gc_width;
  for (int i = tid; i < A.gc_width; i += NT) gc[i] = 0.f;
  (void)MB;
}

}  // namespace sqb
