// GGA / STEP mixed-bit state with the pure-write window (PW-S m): the fused decode step, the prefill-side
// store / load, and STEP's dual-axis fit as a stand-alone pass.
//
// One CTA (512 threads) per (batch row, value head) holds the head's whole [d_k, d_v] tile in shared memory
// (fp32, rows padded by one float so that row-wise and column-wise sweeps are both free of bank conflicts):
//   decode codes -> O;  A O = a (O - beta k (k^T O));  the queued left factors are propagated and re-encoded in FP8,
//   one warp per window row;  o = (A O)^T q + sum_i (R(A p_i) . q) v_i + (beta k . q) v;  the evicted pair is merged;
//   the tile is re-fitted (row factors, column factors, one weighted least-squares refit of the column factors)
//   and re-packed in place;  (R(beta k), R(v)) is enqueued.  A second, tiny kernel moves the window counters.
// Every token reads and rewrites the whole head: 2 x state bytes of HBM traffic per step, no dense contraction.
//
// Arithmetic follows the reference's device statement (src/statequant/kernels/_gga_triton.py:207-308 and
// _stepquant_triton.py:37-60): IEEE division and square root, round half to even, fp16 factors clamped to
// [2^-24, 65504], E4M3 nearest-even with saturation at 448; only the order of fp32 reductions differs.
#pragma once
#include "gga_common.cuh"

namespace sqb {

constexpr int GNT = 512;   // threads per CTA of the GGA kernels
constexpr int GNW = 16;

template <bool MAX>
__device__ __forceinline__ float block_reduce256(float v, float* red) {
  v = MAX ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < GNW; w++) r = MAX ? fmaxf(r, red[w]) : r + red[w];
  return r;
}

__device__ __forceinline__ float enc_level(float y, float qmax, bool two) {
  if (two) return (y >= 0.f ? 1.0f : -1.0f) * (fabsf(y) >= 2.0f ? 3.0f : 1.0f);
  return fminf(fmaxf(rintf(y), -qmax), qmax);
}

// ---- head codes -> fp32 tile T[k * LD + v] ------------------------------------------------------------------------
__device__ __forceinline__ void gga_decode_head(const uint8_t* S, int b, int dk, int dv, int group, float* T, int LD) {
  const int tid = threadIdx.x;
  if (b == 16) {
    const unsigned short* p = reinterpret_cast<const unsigned short*>(S);
    for (int e = tid; e < dk * dv; e += GNT) T[(e / dv) * LD + (e % dv)] = h2f(p[e]);
    return;
  }
  const int ng = dv / group, nr = b == 2 ? dk * ng : dk, qmax = (1 << (b - 1)) - 1;
  const unsigned short* R = reinterpret_cast<const unsigned short*>(S + static_cast<size_t>(dk) * dv * b / 8);
  const unsigned short* C = R + nr;
  const int rowb = dv * b / 8;
  const int lane = tid & 31, warp = tid >> 5;
  if (b != 2 && dv <= 128) {
    // widths 4 / 6 / 8: a row per warp, lane l takes columns l, l + 32, l + 64, l + 96 (column factors in registers)
    float cf[4];
#pragma unroll
    for (int j = 0; j < 4; j++) cf[j] = lane + 32 * j < dv ? h2f(C[lane + 32 * j]) : 0.f;
    auto rows = [&](auto code_of) {
      for (int k = warp; k < dk; k += GNW) {
        const uint8_t* row = S + static_cast<size_t>(k) * rowb;
        const float rrow = h2f(R[k]);
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int v = lane + 32 * j;
          if (v < dv) T[k * LD + v] = (rrow * cf[j]) * static_cast<float>(code_of(row, v) - qmax);
        }
      }
    };
    if (b == 8) rows([](const uint8_t* row, int v) { return static_cast<int>(row[v]); });
    else if (b == 4) rows([](const uint8_t* row, int v) { return static_cast<int>((row[v >> 1] >> (4 * (v & 1))) & 15); });
    else rows([](const uint8_t* row, int v) {
      const uint8_t* t = row + 3 * (v >> 2);
      const uint32_t wd = t[0] | (static_cast<uint32_t>(t[1]) << 8) | (static_cast<uint32_t>(t[2]) << 16);
      return static_cast<int>((wd >> (6 * (v & 3))) & 63);
    });
    return;
  }
  for (int k = warp; k < dk; k += GNW) {                      // a row per warp, the columns over the lanes
    const uint8_t* row = S + static_cast<size_t>(k) * rowb;
    const float rrow = b == 2 ? 0.f : h2f(R[k]);
    for (int v = lane; v < dv; v += 32) {
      float z;
      if (b == 8) z = static_cast<float>(static_cast<int>(row[v]) - qmax);
      else if (b == 4) z = static_cast<float>(static_cast<int>((row[v >> 1] >> (4 * (v & 1))) & 15) - qmax);
      else if (b == 2) z = static_cast<float>((row[v >> 2] >> (2 * (v & 3))) & 3) * 2.0f - 3.0f;
      else {
        const uint8_t* t = row + 3 * (v >> 2);
        const uint32_t wd = t[0] | (static_cast<uint32_t>(t[1]) << 8) | (static_cast<uint32_t>(t[2]) << 16);
        z = static_cast<float>(static_cast<int>((wd >> (6 * (v & 3))) & 63) - qmax);
      }
      const float rf = b == 2 ? h2f(R[k * ng + v / group]) : rrow;
      T[k * LD + v] = (rf * h2f(C[v])) * z;
    }
  }
}

// ---- STEP dual-axis fit of the tile T (values x), then either pack it at S or write r c z to Yout -----------------
// scratch: rs[dk * ng] row factors, cs[dv] column factors, ps[2 * dv] partial sums, red[8]
__device__ void gga_fit_store(float* T, int LD, const float* w, int b, int dk, int dv, int group, uint8_t* S,
                              float* Yout, float* rs, float* cs, float* ps, float* wsm) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (b == 16) {
    for (int e = tid; e < dk * dv; e += GNT) {
      const int k = e / dv, v = e - k * dv;
      const unsigned short hbits = f2h(T[k * LD + v]);
      if (S) reinterpret_cast<unsigned short*>(S)[e] = hbits;
      else Yout[e] = h2f(hbits);
    }
    return;
  }
  const bool two = b == 2;
  const float qmax = two ? 3.0f : static_cast<float>((1 << (b - 1)) - 1);
  const int ng = dv / group, nrg = two ? ng : 1;
  for (int k = tid; k < dk; k += GNT) wsm[k] = w[k];
  __syncthreads();
  // row factors: r = half(sqrt(max(mean |x|, 1e-20) / w)), per row or per (row, 32-column group)
  for (int k = warp; k < dk; k += GNW) {
    if (two) {
      for (int g = 0; g < ng; g++) {
        float s = 0.f;
        for (int v = g * group + lane; v < (g + 1) * group; v += 32) s += fabsf(T[k * LD + v]);
        s = warp_sum(s);
        if (lane == 0) rs[k * ng + g] = halfc(__fsqrt_rn(__fdiv_rn(fmaxf(s * (1.0f / group), 1e-20f), wsm[k])));
      }
    } else {
      float s = 0.f;
      for (int v = lane; v < dv; v += 32) s += fabsf(T[k * LD + v]);
      s = warp_sum(s);
      if (lane == 0) rs[k] = halfc(__fsqrt_rn(__fdiv_rn(fmaxf(s * (1.0f / dv), 1e-20f), wsm[k])));
    }
  }
  __syncthreads();
  // column factors: c = half(max_k |x / r| / qmax); two threads per column, each half of the rows
  const int half_id = tid / dv, col = tid - half_id * dv;      // dv <= 128: half_id in {0, 1}
  const int k0 = half_id * (dk / 2), k1 = k0 + dk / 2;
  const bool act = tid < 2 * dv;
  if (act) {
    float m = 0.f;
    for (int k = k0; k < k1; k++) {
      const float y0 = __fdiv_rn(T[k * LD + col], rs[k * nrg + (two ? col / group : 0)]);
      m = fmaxf(m, __fdiv_rn(fabsf(y0), qmax));
    }
    ps[half_id * dv + col] = m;
  }
  __syncthreads();
  if (tid < dv) cs[tid] = halfc(fmaxf(ps[tid], ps[dv + tid]));
  __syncthreads();
  // weighted least-squares refit of c with the codes fixed
  if (act) {
    const float c0 = cs[col];
    float num = 0.f, den = 0.f;
    for (int k = k0; k < k1; k++) {
      const float x = T[k * LD + col], rf = rs[k * nrg + (two ? col / group : 0)];
      const float z = enc_level(__fdiv_rn(__fdiv_rn(x, rf), c0), qmax, two);
      const float vv = rf * z, ww = wsm[k] * wsm[k];
      num += (ww * vv) * x;
      den += ww * (vv * vv);
    }
    ps[half_id * dv + col] = num;
    ps[2 * dv + half_id * dv + col] = den;
  }
  __syncthreads();
  if (tid < dv) {
    const float num = ps[tid] + ps[dv + tid], den = ps[2 * dv + tid] + ps[3 * dv + tid];
    cs[tid] = halfc(den > 0.f ? __fdiv_rn(num, fmaxf(den, 1e-30f)) : cs[tid]);
  }
  __syncthreads();
  // codes with the refitted c
  if (!S) {
    for (int e = tid; e < dk * dv; e += GNT) {
      const int k = e / dv, v = e - k * dv;
      const float rf = rs[k * nrg + (two ? v / group : 0)];
      const float z = enc_level(__fdiv_rn(__fdiv_rn(T[k * LD + v], rf), cs[v]), qmax, two);
      Yout[e] = (rf * cs[v]) * z;
    }
    return;
  }
  const int iq = static_cast<int>(qmax);
  const int rowb = dv * b / 8;
  const int per = b == 8 ? 1 : (b == 4 ? 2 : 4);                 // codes per packing unit
  const int ub = b == 6 ? 3 : 1;                                 // bytes per packing unit
  const int units = dv / per;
  for (int e = tid; e < dk * units; e += GNT) {
    const int k = e / units, j = e - k * units;
    uint32_t wd = 0;
    for (int t = 0; t < per; t++) {
      const int v = j * per + t;
      const float rf = rs[k * nrg + (two ? v / group : 0)];
      const float z = enc_level(__fdiv_rn(__fdiv_rn(T[k * LD + v], rf), cs[v]), qmax, two);
      const int u = two ? static_cast<int>((z + 3.0f) * 0.5f) : static_cast<int>(z) + iq;
      wd |= static_cast<uint32_t>(u) << (b * t);
    }
    uint8_t* p = S + static_cast<size_t>(k) * rowb + j * ub;
    p[0] = static_cast<uint8_t>(wd & 255u);
    if (b == 6) { p[1] = static_cast<uint8_t>((wd >> 8) & 255u); p[2] = static_cast<uint8_t>(wd >> 16); }
  }
  unsigned short* R = reinterpret_cast<unsigned short*>(S + static_cast<size_t>(dk) * dv * b / 8);
  for (int i = tid; i < dk * nrg; i += GNT) R[i] = f2h(rs[i]);
  unsigned short* C = R + dk * nrg;
  for (int v = tid; v < dv; v += GNT) C[v] = f2h(cs[v]);
}

// ---- the same fit + pack for the widths 4 / 6 / 8 with the tile's columns owned by threads ---------------------------
// Thread (half, col) owns rows [half dk/2, (half + 1) dk/2) of column col (2 dv <= 256 threads) in the three sweeps
// (column maximum, refit, final codes).  Both divisors of an element, its row factor and its column factor, are fp16
// values, and for such divisors x / d is exactly fma(fma(-d, x rd, x), rd, x rd) with rd = RN(1 / d) whenever the
// quotient is far from the subnormal and overflow ranges (checked on the host for every fp16 divisor against
// hundreds of millions of dividends), so the sweeps recompute the quotients with three FMAs instead of keeping them;
// the division of the column maximum by qmax is taken out of the loop (a positive constant divisor keeps the
// maximum the maximum).  Codes of a packing unit (2 or 4 adjacent columns) meet in one lane by shuffles.
// The range condition is checked once per head on the tile: all non-zero |x| within [1e-30, 1e14].  With factors in
// [2^-24, 65504] the first quotient y = x / r is then exact (no subnormal residual); the second one, y / c, can be an
// ulp off only where y is below 1e-31, i.e. where its code is 0 whatever the last bit.  A head outside the range takes
// gga_fit_store.
__device__ __forceinline__ float div_h16(float x, float d, float rd) {
  const float q0 = x * rd;
  return __fmaf_rn(__fmaf_rn(-d, q0, x), rd, q0);
}

template <int B>
__device__ __forceinline__ bool gga_fit_pack_cols(const float* T, int LD, const float* w, int dk, int dv, uint8_t* S, float* rs,
                                  float* cs, float* ps, float* wsm, float* rrs, float* red) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr float qmax = static_cast<float>((1 << (B - 1)) - 1);
  constexpr int iq = (1 << (B - 1)) - 1;
  for (int k = tid; k < dk; k += GNT) wsm[k] = w[k];
  __syncthreads();
  // row factors: r = half(sqrt(max(mean |x|, 1e-20) / w)), one warp per row; and their reciprocals
  const float inv_dv = 1.0f / dv;
  float hi = 0.f, lo = 1.0f;                                         // largest |x|, smallest non-zero |x| (capped at 1)
  for (int k = warp; k < dk; k += GNW) {
    float sum = 0.f;
    for (int v = lane; v < dv; v += 32) {
      const float ax = fabsf(T[k * LD + v]);
      sum += ax;
      hi = fmaxf(hi, ax);
      lo = fminf(lo, ax > 0.f ? ax : 1.0f);
    }
    sum = warp_sum(sum);
    if (lane == 0) {
      const float r = halfc(__fsqrt_rn(__fdiv_rn(fmaxf(sum * inv_dv, 1e-20f), wsm[k])));
      rs[k] = r;
      rrs[k] = __frcp_rn(r);
    }
  }
  hi = block_reduce256<true>(hi, red);
  lo = -block_reduce256<true>(-lo, red);
  if (!(hi < 1e14f && lo > 1e-30f)) return false;                    // uniform: the caller takes the IEEE path
  __syncthreads();
  const int np = GNT / dv < 8 ? GNT / dv : 8;                        // threads per column; each takes dk / np rows
  const int KR = dk / np;
  const int part = tid / dv, col = tid - part * dv;
  const bool act = tid < np * dv;
  const int k0 = part * KR;
  const float* Tc = T + k0 * LD + col;
  if (act) {
    float m = 0.f;
#pragma unroll 4
    for (int i = 0; i < KR; i++) m = fmaxf(m, fabsf(div_h16(Tc[i * LD], rs[k0 + i], rrs[k0 + i])));
    ps[part * dv + col] = m;
  }
  __syncthreads();
  if (tid < dv) {
    float mm = ps[tid];
    for (int pp = 1; pp < np; pp++) mm = fmaxf(mm, ps[pp * dv + tid]);
    cs[tid] = halfc(__fdiv_rn(mm, qmax));
  }
  __syncthreads();
  // weighted least-squares refit of c with the codes fixed
  if (act) {
    const float c0 = cs[col], rc0 = __frcp_rn(c0);
    float num = 0.f, den = 0.f;
#pragma unroll 4
    for (int i = 0; i < KR; i++) {
      const float x = Tc[i * LD], r = rs[k0 + i];
      const float z = fminf(fmaxf(rintf(div_h16(div_h16(x, r, rrs[k0 + i]), c0, rc0)), -qmax), qmax);
      const float vv = r * z, ww = wsm[k0 + i] * wsm[k0 + i];
      num += (ww * vv) * x;
      den += ww * (vv * vv);
    }
    ps[part * dv + col] = num;
    ps[(np + part) * dv + col] = den;
  }
  __syncthreads();
  if (tid < dv) {
    float num = 0.f, den = 0.f;
    for (int pp = 0; pp < np; pp++) { num += ps[pp * dv + tid]; den += ps[(np + pp) * dv + tid]; }
    cs[tid] = halfc(den > 0.f ? __fdiv_rn(num, fmaxf(den, 1e-30f)) : cs[tid]);
  }
  __syncthreads();
  // codes with the refitted c, packed along d_v: 8 bit one byte per lane, 4 bit two lanes per byte, 6 bit four lanes
  // per three bytes
  constexpr int rowb_num = B;                                        // row bytes = dv * B / 8
  const int rowb = dv * rowb_num / 8;
  const float c1 = act ? cs[col] : 1.0f, rc1 = __frcp_rn(c1);
  if ((tid & ~31) < np * dv) {                                       // whole warps, for the shuffles
#pragma unroll 4
    for (int i = 0; i < KR; i++) {
      int u = 0;
      if (act) u = static_cast<int>(fminf(fmaxf(rintf(div_h16(div_h16(Tc[i * LD], rs[k0 + i], rrs[k0 + i]), c1, rc1)), -qmax), qmax)) + iq;
      uint8_t* row = S + static_cast<size_t>(k0 + i) * rowb;
      if constexpr (B == 8) {
        if (act) row[col] = static_cast<uint8_t>(u);
      } else if constexpr (B == 4) {
        const int hi = __shfl_down_sync(0xffffffffu, u, 1);
        if (act && !(col & 1)) row[col >> 1] = static_cast<uint8_t>(u | (hi << 4));
      } else {
        const int u1 = __shfl_down_sync(0xffffffffu, u, 1), u2 = __shfl_down_sync(0xffffffffu, u, 2),
                  u3 = __shfl_down_sync(0xffffffffu, u, 3);
        if (act && !(col & 3)) {
          const uint32_t wd = static_cast<uint32_t>(u) | (static_cast<uint32_t>(u1) << 6) |
                              (static_cast<uint32_t>(u2) << 12) | (static_cast<uint32_t>(u3) << 18);
          uint8_t* p = row + 3 * (col >> 2);
          p[0] = static_cast<uint8_t>(wd & 255u); p[1] = static_cast<uint8_t>((wd >> 8) & 255u); p[2] = static_cast<uint8_t>(wd >> 16);
        }
      }
    }
  }
  unsigned short* R = reinterpret_cast<unsigned short*>(S + static_cast<size_t>(dk) * dv * B / 8);
  for (int i = tid; i < dk; i += GNT) R[i] = f2h(rs[i]);
  unsigned short* C = R + dk;
  for (int v = tid; v < dv; v += GNT) C[v] = f2h(cs[v]);
  return true;
}

// fit + pack, picking the column-owner version where it applies
__device__ __forceinline__ void gga_fit_pack(float* T, int LD, const float* w, int b, int dk, int dv, int group,
                                             uint8_t* S, float* rs, float* cs, float* ps, float* wsm, float* rrs,
                                             float* red) {
  const bool cols = 2 * dv <= GNT && dv % 32 == 0 && dk % 8 == 0;
  bool done = false;
  if (cols && b == 4) done = gga_fit_pack_cols<4>(T, LD, w, dk, dv, S, rs, cs, ps, wsm, rrs, red);
  else if (cols && b == 6) done = gga_fit_pack_cols<6>(T, LD, w, dk, dv, S, rs, cs, ps, wsm, rrs, red);
  else if (cols && b == 8) done = gga_fit_pack_cols<8>(T, LD, w, dk, dv, S, rs, cs, ps, wsm, rrs, red);
  if (!done) {
    __syncthreads();
    gga_fit_store(T, LD, w, b, dk, dv, group, S, nullptr, rs, cs, ps, wsm);
  }
}

// shared-memory plan (floats) of the GGA kernels
struct GgaSmem { int T, q, k, bk, v, o, kO, rs, rrs, cs, ps, wsm, Pw, Vw, r0, coef, red, total, LD; };
__host__ __device__ inline GgaSmem gga_smem(int dk, int dv, int M, int group) {
  GgaSmem s;
  int o = 0;
  s.LD = dv + 1;
  s.T = o; o += dk * s.LD;
  s.q = o; o += dk; s.k = o; o += dk; s.bk = o; o += dk;
  s.v = o; o += dv; s.o = o; o += dv; s.kO = o; o += GNT;
  s.rs = o; o += dk * (dv / group > 0 ? dv / group : 1);
  s.rrs = o; o += dk;
  s.cs = o; o += dv; s.ps = o; o += 2 * GNT; s.wsm = o; o += dk;
  s.Pw = o; o += M * dk; s.Vw = o; o += M * dv; s.r0 = o; o += dk; s.coef = o; o += (M > 32 ? M : 32); s.red = o; o += 32;
  s.total = o;
  return s;
}


// ---- the decode step ----------------------------------------------------------------------------------------------
// DKT, DVT: the head dims as compile-time constants (0: taken from the arguments), so that the tile's index
// arithmetic folds into immediates for the usual 128 x 128 head
template <int DKT, int DVT>
__global__ void __launch_bounds__(GNT) gga_step_kernel(const __grid_constant__ GgaArgs A) {
  extern __shared__ __align__(16) float gsm[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int dk = DKT ? DKT : A.DK, dv = DVT ? DVT : A.DV, M = A.M, HV = A.HV;
  const int bh = blockIdx.x, b = bh / HV, h = bh - b * HV, hk = h / (HV / A.HK);
  uint8_t* orow = A.out + (long long)b * A.so + (long long)h * dv * dt_size(A.dt_out);
  const long long seq = A.idx[b];
  if (seq <= 0) {
    for (int v = tid; v < dv; v += GNT) stf(orow, A.dt_out, v, 0.0f);
    return;
  }
  if (A.skip_packed) {
    const int wb = A.bits[h];
    if (wb == 4 || wb == 6 || wb == 8) return;
  }
  const GgaSmem P = gga_smem(dk, dv, M, A.group);
  const int LD = dv + 1;
  float *T = gsm + P.T, *q = gsm + P.q, *k = gsm + P.k, *bk = gsm + P.bk, *v = gsm + P.v, *o = gsm + P.o,
        *kO = gsm + P.kO, *Pw = gsm + P.Pw, *Vw = gsm + P.Vw, *coef = gsm + P.coef, *red = gsm + P.red;
  uint8_t* base = A.blob + seq * A.stride;
  const int bits = A.bits[h];
  uint8_t* S = base + A.offs[h];

  // q, k (fla's normalisation), gates
  float sq = 0.f, sk = 0.f;
  for (int i = tid; i < dk; i += GNT) {
    const float qv = ldf(A.q + (long long)b * A.sq, A.dt_qk, (long long)hk * dk + i);
    const float kv = ldf(A.k + (long long)b * A.sk, A.dt_qk, (long long)hk * dk + i);
    q[i] = qv; k[i] = kv;
    sq += qv * qv; sk += kv * kv;
  }
  for (int i = tid; i < dv; i += GNT) v[i] = ldf(A.v + (long long)b * A.sv, A.dt_v, (long long)h * dv + i);
  sq = block_reduce256<false>(sq, red);
  sk = block_reduce256<false>(sk, red);
  const float nq = __fsqrt_rn(sq + 1e-6f), nk = __fsqrt_rn(sk + 1e-6f);
  const float x = ldf(A.a + (long long)b * A.sa, A.dt_ab, h) + ldf(A.dt_bias, A.dt_dtb, h);
  const float sp = x <= 20.0f ? logf(1.0f + expf(x)) : x;
  const float a = expf(-expf(ldf(A.A_log, A.dt_alog, h)) * sp);
  const float beta = __fdiv_rn(1.0f, 1.0f + expf(-ldf(A.b + (long long)b * A.sb, A.dt_ab, h)));
  float bqp = 0.f;
  for (int i = tid; i < dk; i += GNT) {
    const float qn = __fdiv_rn(q[i], nq) * A.scale, kn = __fdiv_rn(k[i], nk);
    q[i] = qn; k[i] = kn; bk[i] = beta * kn;
    bqp += (beta * kn) * qn;
  }
  gga_decode_head(S, bits, dk, dv, A.group, T, LD);
  const float bq = block_reduce256<false>(bqp, red);            // (beta k) . q; also orders the tile writes
  // kO = k^T O, np threads per column
  const int np = GNT / dv < 8 ? GNT / dv : 8;
  const int part = tid / dv, col = tid - part * dv;
  const bool act = tid < np * dv && dk % np == 0;
  const int KRp = dk / np, k0 = part * KRp, k1 = k0 + KRp;
  const bool single = dk % np != 0;                         // odd shapes: one thread per column
  if (act || (single && tid < dv)) {
    float sum = 0.f;
    const int lo_ = single ? 0 : k0, hi_ = single ? dk : k1;
    for (int i = lo_; i < hi_; i++) sum = fmaf(k[i], T[i * LD + col], sum);
    kO[part * dv + col] = sum;
  }
  __syncthreads();
  if (tid < dv && !single) {
    float sum = kO[tid];
    for (int pp = 1; pp < np; pp++) sum += kO[pp * dv + tid];
    kO[tid] = sum;
  }
  __syncthreads();
  // A O in place
  for (int i = warp; i < dk; i += GNW) {
    const float bki = bk[i];
    for (int j = lane; j < dv; j += 32) T[i * LD + j] = a * (T[i * LD + j] - bki * kO[j]);
  }
  __syncthreads();
  if (act || (single && tid < dv)) {
    float sum = 0.f;
    const int lo_ = single ? 0 : k0, hi_ = single ? dk : k1;
    for (int i = lo_; i < hi_; i++) sum = fmaf(T[i * LD + col], q[i], sum);
    kO[part * dv + col] = sum;
  }
  __syncthreads();
  if (tid < dv) {
    float sum = kO[tid];
    if (!single) for (int pp = 1; pp < np; pp++) sum += kO[pp * dv + tid];
    o[tid] = sum + bq * v[tid];
  }
  __syncthreads();

  const bool window = A.pw && bits != 16;
  if (window) {
    const int* ct = reinterpret_cast<const int*>(base);
    const int n = ct[0], hd = ct[1];
    uint8_t* qb = base + A.qoff + (long long)h * A.qsz;
    uint8_t *PP = qb, *VP = qb + (long long)M * dk;
    float *PS = reinterpret_cast<float*>(qb + (long long)M * (dk + dv)), *VS = PS + M;
    // one warp per window row, in age order: propagate, re-encode, read out
    for (int i = warp; i < M; i += GNW) {
      const bool live = i < n;
      float cf = 0.f;
      if (live) {
        const int jj = (hd + i) % M;
        const float ps_ = PS[jj], vs_ = VS[jj];
        float kp = 0.f;
        for (int t = lane; t < dk; t += 32) {
          const float pv = e4m3_val(PP[jj * dk + t]) * ps_;
          Pw[i * dk + t] = pv;
          kp = fmaf(k[t], pv, kp);
        }
        for (int t = lane; t < dv; t += 32) Vw[i * dv + t] = e4m3_val(VP[jj * dv + t]) * vs_;
        kp = warp_sum(kp);
        float am = 0.f;
        for (int t = lane; t < dk; t += 32) {
          const float ap = a * (Pw[i * dk + t] - bk[t] * kp);
          Pw[i * dk + t] = ap;
          am = fmaxf(am, fabsf(ap));
        }
        am = warp_max(am);
        const float sc = __fdiv_rn(am, 448.0f), safe = sc > 0.f ? sc : 1.0f;
        for (int t = lane; t < dk; t += 32) {
          const float y = e4m3_round(fminf(fmaxf(__fdiv_rn(Pw[i * dk + t], safe), -448.0f), 448.0f));
          PP[jj * dk + t] = e4m3_byte(y);
          const float r = sc > 0.f ? y * safe : 0.f;
          Pw[i * dk + t] = r;
          cf = fmaf(r, q[t], cf);
        }
        if (lane == 0) PS[jj] = sc;
        cf = warp_sum(cf);
      }
      if (lane == 0) coef[i] = live ? cf : 0.f;
    }
    __syncthreads();
    if (tid < dv) {
      float acc = o[tid];
      for (int i = 0; i < M && i < n; i++) acc = fmaf(coef[i], Vw[i * dv + tid], acc);
      o[tid] = acc;
    }
    if (n == M) {                                               // merge the evicted (oldest) pair into the state
      for (int i = warp; i < dk; i += GNW) {
        const float pi = Pw[i];
        for (int j = lane; j < dv; j += 32) T[i * LD + j] = T[i * LD + j] + pi * Vw[j];
      }
    }
    // enqueue (R(beta k), R(v)) at the slot after the youngest pair (the evicted one's when the window is full)
    const int jn = n < M ? (hd + n) % M : hd;
    if (warp < 2) {
      const float* src = warp == 0 ? bk : v;
      const int len = warp == 0 ? dk : dv;
      float am = 0.f;
      for (int t = lane; t < len; t += 32) am = fmaxf(am, fabsf(src[t]));
      am = warp_max(am);
      const float sc = __fdiv_rn(am, 448.0f), safe = sc > 0.f ? sc : 1.0f;
      uint8_t* dst = warp == 0 ? PP + jn * dk : VP + jn * dv;
      for (int t = lane; t < len; t += 32)
        dst[t] = e4m3_byte(e4m3_round(fminf(fmaxf(__fdiv_rn(src[t], safe), -448.0f), 448.0f)));
      if (lane == 0) (warp == 0 ? PS : VS)[jn] = sc;
    }
  } else {
    for (int i = warp; i < dk; i += GNW) {
      const float bki = bk[i];
      for (int j = lane; j < dv; j += 32) T[i * LD + j] = T[i * LD + j] + bki * v[j];
    }
  }
  __syncthreads();
  for (int j = tid; j < dv; j += GNT) stf(orow, A.dt_out, j, o[j]);
  gga_fit_pack(T, LD, A.w + (long long)h * dk, bits, dk, dv, A.group, S, gsm + P.rs, gsm + P.cs, gsm + P.ps, gsm + P.wsm,
               gsm + P.rrs, gsm + P.red);
}

// window counters, after every head of the slot has read them
__global__ void gga_advance_kernel(uint8_t* blob, long long stride, const int* idx, int rows, int M) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= rows) return;
  const long long seq = idx[b];
  if (seq <= 0) return;
  int* ct = reinterpret_cast<int*>(blob + seq * stride);
  const int n = ct[0], hd = ct[1];
  ct[0] = min(n + 1, M);
  ct[1] = n == M ? (hd + 1) % M : hd;
}

// fit + pack canonical states X [P, HV, dk, dv] into slots; zero the counters
__global__ void __launch_bounds__(GNT) gga_store_kernel(const __grid_constant__ GgaArgs A) {
  extern __shared__ __align__(16) float gsm[];
  const int tid = threadIdx.x;
  const int dk = A.DK, dv = A.DV, HV = A.HV;
  const int ph = blockIdx.x, p = ph / HV, h = ph - p * HV;
  const long long seq = A.idx[p];
  if (seq <= 0) return;                      // a padding row (0, or an engine's -1): nothing is written
  const GgaSmem P = gga_smem(dk, dv, A.M, A.group);
  float* T = gsm + P.T;
  const float* x = A.X + (long long)ph * dk * dv;
  for (int e = tid; e < dk * dv; e += GNT) T[(e / dv) * P.LD + (e % dv)] = x[e];
  __syncthreads();
  uint8_t* base = A.blob + seq * A.stride;
  gga_fit_pack(T, P.LD, A.w + (long long)h * dk, A.bits[h], dk, dv, A.group, base + A.offs[h], gsm + P.rs, gsm + P.cs,
               gsm + P.ps, gsm + P.wsm, gsm + P.rrs, gsm + P.red);
  if (h == 0 && tid < 2) reinterpret_cast<int*>(base)[tid] = 0;
}

// unpack slots into canonical fp32 Y [P, HV, dk, dv] (the stored state, without the window)
__global__ void __launch_bounds__(GNT) gga_load_kernel(const __grid_constant__ GgaArgs A) {
  extern __shared__ __align__(16) float gsm[];
  const int tid = threadIdx.x;
  const int dk = A.DK, dv = A.DV, HV = A.HV;
  const int ph = blockIdx.x, p = ph / HV, h = ph - p * HV;
  const long long seq = A.idx[p];
  float* y = A.Y + (long long)ph * dk * dv;
  if (seq <= 0) {                            // a padding row: its output is zeroed, no slot is read
    for (int e = tid; e < dk * dv; e += GNT) y[e] = 0.f;
    return;
  }
  const GgaSmem P = gga_smem(dk, dv, A.M, A.group);
  float* T = gsm + P.T;
  gga_decode_head(A.blob + seq * A.stride + A.offs[h], A.bits[h], dk, dv, A.group, T, P.LD);
  __syncthreads();
  for (int e = tid; e < dk * dv; e += GNT) y[e] = T[(e / dv) * P.LD + (e % dv)];
}

// STEP's dual-axis fit as a fake-quant pass: Y = fit(X), X / Y [B, H, dk, dv]
__global__ void __launch_bounds__(GNT) stepquant_fit_kernel(const __grid_constant__ GgaArgs A) {
  extern __shared__ __align__(16) float gsm[];
  const int tid = threadIdx.x;
  const int dk = A.DK, dv = A.DV, HV = A.HV;
  const int ph = blockIdx.x, h = ph % HV;
  const GgaSmem P = gga_smem(dk, dv, 1, A.group);
  float* T = gsm + P.T;
  const float* x = A.X + (long long)ph * dk * dv;
  for (int e = tid; e < dk * dv; e += GNT) T[(e / dv) * P.LD + (e % dv)] = x[e];
  __syncthreads();
  gga_fit_store(T, P.LD, A.w + (long long)h * dk, A.bits[h], dk, dv, A.group, nullptr, A.Y + (long long)ph * dk * dv,
                gsm + P.rs, gsm + P.cs, gsm + P.ps, gsm + P.wsm);
}

}  // namespace sqb
