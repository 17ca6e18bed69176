// The GGA / STEP decode step with the head's tile held in REGISTERS (heads of 128 x 128 at widths 4, 6 or 8 bits).
//
// One CTA of 256 threads per (batch row, value head).  Warp w owns rows 16 w .. 16 w + 15 of the [d_k, d_v] tile, lane l
// the four adjacent columns 4 l .. 4 l + 3: 64 elements per thread, which never leave the register file between the
// decode and the re-pack.  A packing unit along d_v (2 codes per byte, 4 codes per 3 bytes, 1 code per byte) lies inside
// one lane, so decode and pack need no exchange.  The head's bytes (codes, row factors, column factors: one
// contiguous chunk) and the window's (one contiguous chunk) come in by one bulk copy each and leave the same way.
// Row-wise reductions stay inside a warp (a transposing butterfly: 16 shuffles for 16 rows); column-wise ones go
// through 8 x 128 partial sums in shared memory.  The element-wise sweeps work on column pairs with the packed
// f32x2 instructions.
//
// Arithmetic is that of the tile kernel (gga.cuh: gga_step_kernel with gga_fit_pack_cols): the same operations per element, the same
// exact-quotient scheme for the two fp16 divisors (div_h16); only the order of the fp32 sums differs.  A head whose
// values leave the range in which div_h16 is exact takes the IEEE divisions instead (the cold path below).
// Heads of other widths (2-bit, fp16 pivots) are left to gga_step_kernel: this kernel's CTA returns at once for them.
#pragma once
#include <cuda_fp8.h>
#include "gga_common.cuh"
#include "step_tma.cuh"
#include "fold_mma.cuh"

namespace sqb {

#ifndef SQB_GGA_RPW
#define SQB_GGA_RPW 16
#endif
constexpr int RD = 128;            // d_k = d_v
constexpr int RPW = SQB_GGA_RPW;   // tile rows per warp: 16 (256 threads, 64 elements per thread) or 8 (512 threads, 32)
constexpr int RNW = RD / RPW;
constexpr int RNT = 32 * RNW;      // threads per CTA
static_assert(RPW == 16 || RPW == 8, "rows per warp");

// shared-memory plan (bytes)
struct GgaRegSmem { int bar, raw, win, f0, total; int q, k, bk, v, o, w, rs, rrs, cs, rcs, pa, pb, Pw, Vw, coef, red; };
__host__ __device__ inline GgaRegSmem gga_reg_smem(int M, int qsz) {
  GgaRegSmem s;
  int o = 0;
  s.bar = o; o += 16;
  s.raw = o; o += RD * RD + 4 * RD;                       // the widest head: 8-bit codes + fp16 row and column factors
  s.win = o; o += (qsz + 15) & ~15;
  s.f0 = o;
  int f = 0;
  s.q = f; f += RD; s.k = f; f += RD; s.bk = f; f += RD; s.v = f; f += RD; s.o = f; f += RD; s.w = f; f += RD;
  s.rs = f; f += RD; s.rrs = f; f += RD; s.cs = f; f += RD; s.rcs = f; f += RD;
  s.pa = f; f += RNW * RD; s.pb = f; f += RNW * RD;
  s.Pw = f; f += M * RD; s.Vw = f; f += M * RD;
  s.coef = f; f += 32; s.red = f; f += 32;
  s.total = s.f0 + f * 4;
  return s;
}

// RPW per-lane values -> their sums over the warp, one row per group of lanes: the rounds halve the number of values a
// lane carries (it keeps one half and sends the other to its partner), so RPW - 1 shuffles do the job, plus one per
// remaining level for the lanes that end up with the same row.  On return lane l holds the total of row
// transpose_row(l).
__device__ __forceinline__ float transpose_sum(float (&v)[RPW], int lane) {
  int n = RPW, bit = 16;
#pragma unroll
  for (int level = 0; level < (RPW == 16 ? 4 : 3); level++) {
    n >>= 1;
#pragma unroll
    for (int j = 0; j < RPW / 2; j++) {
      if (j < n) {
        const bool up = lane & bit;
        const float send = up ? v[j] : v[j + n], keep = up ? v[j + n] : v[j];
        v[j] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
      }
    }
    bit >>= 1;
  }
  float t = v[0];
#pragma unroll
  for (int o = RPW == 16 ? 1 : 2; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}
__device__ __forceinline__ int transpose_row(int lane) {
  if (RPW == 16) return ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
  return ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
}
constexpr int ROW_LANES = RPW == 16 ? 2 : 4;       // lanes that end up with the same row's total

// E4M3 through the conversion instructions (round to nearest even, saturating at 448, subnormals down to 2^-9: what
// e4m3_round / e4m3_byte / e4m3_val of gga_common.cuh spell out), two values at a time
__device__ __forceinline__ float2 e4m3x2_val(uint32_t b0, uint32_t b1) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(b0 | (b1 << 8)), __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
__device__ __forceinline__ uint32_t e4m3x2_byte(float a, float b) {
  return __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
}

// x / d for a pair, d an fp16 value with rd = RN(1 / d) (see div_h16)
__device__ __forceinline__ float2 div_h16x2(float2 x, float2 d, float2 nd, float2 rd) {
  const float2 q0 = __fmul2_rn(x, rd);
  return __ffma2_rn(__ffma2_rn(nd, q0, x), rd, q0);
}
// clamp(rint(y), +-qmax) for a pair (|y| < 2^22)
__device__ __forceinline__ float2 rint_clamp2(float2 y, float qmax) {
  const float2 mg = make_float2(MAGIC, MAGIC), nmg = make_float2(-MAGIC, -MAGIC);
  const float2 z = __fadd2_rn(__fadd2_rn(y, mg), nmg);
  return make_float2(fminf(fmaxf(z.x, -qmax), qmax), fminf(fmaxf(z.y, -qmax), qmax));
}

// The rare head outside div_h16's range: the three sweeps of the fit with IEEE divisions, on a copy of the tile in
// local memory (kept out of line; the hot path's registers are untouched).  Writes the column factors to cs / rcs and
// the final codes (offset by qmax) to u.
template <int B>
__device__ __noinline__ void gga_reg_fit_cold(const float* x, uint8_t* u, const float* rs, const float* wsm, float* cs,
                                              float* pa, float* pb, int warp, int lane) {
  constexpr float qmax = static_cast<float>((1 << (B - 1)) - 1);
  const int tid = warp * 32 + lane;
  float m[4] = {0.f, 0.f, 0.f, 0.f};
  for (int r = 0; r < RPW; r++)
    for (int c = 0; c < 4; c++) m[c] = fmaxf(m[c], fabsf(__fdiv_rn(x[r * 4 + c], rs[RPW * warp + r])));
  for (int c = 0; c < 4; c++) pa[warp * RD + 4 * lane + c] = m[c];
  __syncthreads();
  if (tid < RD) {
    float mm = pa[tid];
    for (int w = 1; w < RNW; w++) mm = fmaxf(mm, pa[w * RD + tid]);
    cs[tid] = halfc(__fdiv_rn(mm, qmax));
  }
  __syncthreads();
  float num[4] = {0.f, 0.f, 0.f, 0.f}, den[4] = {0.f, 0.f, 0.f, 0.f};
  for (int r = 0; r < RPW; r++) {
    const float rf = rs[RPW * warp + r], ww = wsm[RPW * warp + r] * wsm[RPW * warp + r];
    for (int c = 0; c < 4; c++) {
      const float xv = x[r * 4 + c];
      const float z = fminf(fmaxf(rintf(__fdiv_rn(__fdiv_rn(xv, rf), cs[4 * lane + c])), -qmax), qmax);
      const float vv = rf * z;
      num[c] += (ww * vv) * xv;
      den[c] += ww * (vv * vv);
    }
  }
  for (int c = 0; c < 4; c++) { pa[warp * RD + 4 * lane + c] = num[c]; pb[warp * RD + 4 * lane + c] = den[c]; }
  __syncthreads();
  if (tid < RD) {
    float n = 0.f, d = 0.f;
    for (int w = 0; w < RNW; w++) { n += pa[w * RD + tid]; d += pb[w * RD + tid]; }
    cs[tid] = halfc(d > 0.f ? __fdiv_rn(n, fmaxf(d, 1e-30f)) : cs[tid]);
  }
  __syncthreads();
  for (int r = 0; r < RPW; r++)
    for (int c = 0; c < 4; c++) {
      const float z = fminf(fmaxf(rintf(__fdiv_rn(__fdiv_rn(x[r * 4 + c], rs[RPW * warp + r]), cs[4 * lane + c])), -qmax), qmax);
      u[r * 4 + c] = static_cast<uint8_t>(static_cast<int>(z) + static_cast<int>(qmax));
    }
}

// the four codes of a lane in row `row` of the raw head bytes (offset by qmax, as stored)
template <int B>
__device__ __forceinline__ void gga_reg_codes(const uint8_t* raw, int row, int lane, uint32_t (&u)[4]) {
  if constexpr (B == 8) {
    const uint32_t wd = *reinterpret_cast<const uint32_t*>(raw + row * 128 + 4 * lane);
    u[0] = wd & 255u; u[1] = (wd >> 8) & 255u; u[2] = (wd >> 16) & 255u; u[3] = wd >> 24;
  } else if constexpr (B == 4) {
    const uint32_t wd = *reinterpret_cast<const unsigned short*>(raw + row * 64 + 2 * lane);
    u[0] = wd & 15u; u[1] = (wd >> 4) & 15u; u[2] = (wd >> 8) & 15u; u[3] = wd >> 12;
  } else {
    const uint8_t* t = raw + row * 96 + 3 * lane;
    const uint32_t wd = t[0] | (static_cast<uint32_t>(t[1]) << 8) | (static_cast<uint32_t>(t[2]) << 16);
    u[0] = wd & 63u; u[1] = (wd >> 6) & 63u; u[2] = (wd >> 12) & 63u; u[3] = wd >> 18;
  }
}
template <int B>
__device__ __forceinline__ void gga_reg_put(uint8_t* raw, int row, int lane, uint32_t u0, uint32_t u1, uint32_t u2, uint32_t u3) {
  if constexpr (B == 8) {
    *reinterpret_cast<uint32_t*>(raw + row * 128 + 4 * lane) = u0 | (u1 << 8) | (u2 << 16) | (u3 << 24);
  } else if constexpr (B == 4) {
    *reinterpret_cast<unsigned short*>(raw + row * 64 + 2 * lane) = static_cast<unsigned short>(u0 | (u1 << 4) | (u2 << 8) | (u3 << 12));
  } else {
    const uint32_t wd = u0 | (u1 << 6) | (u2 << 12) | (u3 << 18);
    uint8_t* t = raw + row * 96 + 3 * lane;
    t[0] = static_cast<uint8_t>(wd & 255u); t[1] = static_cast<uint8_t>((wd >> 8) & 255u); t[2] = static_cast<uint8_t>(wd >> 16);
  }
}

struct GgaRegCtx {
  uint8_t *raw, *win;                 // shared: the head's bytes, the window's bytes
  float *q, *k, *bk, *v, *o, *w, *rs, *rrs, *cs, *rcs, *pa, *pb, *Pw, *Vw, *coef;
  float a, bq;                        // decay, (beta k) . q
  int n, hd, M;                       // window: live pairs, ring head, length
  bool window;
  uint8_t* orow; int dt_out;
};

// q, k (fla's normalisation) and the gates of one head: gga_step_kernel's arithmetic on ONE warp (four channels per
// lane, sums by shuffles), while the other warps bring in v and w.  Results in shared memory: C.q, C.k, C.bk, C.v, C.w
// and sc = (a, (beta k) . q, window count, ring head); a block barrier must follow before anybody reads them.
__device__ __forceinline__ void gga_reg_prologue(const GgaArgs& A, const GgaRegCtx& C, float* sc, int b, int h, int hk,
                                                 const uint8_t* base, bool window, int warp, int lane) {
  const int tid = warp * 32 + lane;
  if (warp == 0) {
    const Raw4 rq = ld4_raw(A.q + (long long)b * A.sq, A.dt_qk, (long long)hk * RD + 4 * lane);
    const Raw4 rk = ld4_raw(A.k + (long long)b * A.sk, A.dt_qk, (long long)hk * RD + 4 * lane);
    const uint32_t ra = ld1_raw(A.a + (long long)b * A.sa, A.dt_ab, h), rdb = ld1_raw(A.dt_bias, A.dt_dtb, h);
    const uint32_t ral = ld1_raw(A.A_log, A.dt_alog, h), rb = ld1_raw(A.b + (long long)b * A.sb, A.dt_ab, h);
    int n = 0, hd = 0;
    if (window && lane == 0) { const int* ct = reinterpret_cast<const int*>(base); n = ct[0]; hd = ct[1]; }
    float qv[4], kv[4];
    cvt4_raw(rq, A.dt_qk, qv);
    cvt4_raw(rk, A.dt_qk, kv);
    float sq = (qv[0] * qv[0] + qv[1] * qv[1]) + (qv[2] * qv[2] + qv[3] * qv[3]);
    float sk = (kv[0] * kv[0] + kv[1] * kv[1]) + (kv[2] * kv[2] + kv[3] * kv[3]);
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float nq = __fsqrt_rn(sq + 1e-6f), nk = __fsqrt_rn(sk + 1e-6f);
    const float xg = cvt_raw(ra, A.dt_ab) + cvt_raw(rdb, A.dt_dtb);
    const float sp = xg <= 20.0f ? logf(1.0f + expf(xg)) : xg;
    const float a = expf(-expf(cvt_raw(ral, A.dt_alog)) * sp);
    const float beta = __fdiv_rn(1.0f, 1.0f + expf(-cvt_raw(rb, A.dt_ab)));
    float qn[4], kn[4], bkv[4], bqp = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      qn[j] = __fdiv_rn(qv[j], nq) * A.scale;
      kn[j] = __fdiv_rn(kv[j], nk);
      bkv[j] = beta * kn[j];
      bqp += bkv[j] * qn[j];
    }
    bqp = warp_sum(bqp);
    *reinterpret_cast<float4*>(C.q + 4 * lane) = make_float4(qn[0], qn[1], qn[2], qn[3]);
    *reinterpret_cast<float4*>(C.k + 4 * lane) = make_float4(kn[0], kn[1], kn[2], kn[3]);
    *reinterpret_cast<float4*>(C.bk + 4 * lane) = make_float4(bkv[0], bkv[1], bkv[2], bkv[3]);
    if (lane == 0) { sc[0] = a; sc[1] = bqp; sc[2] = __int_as_float(n); sc[3] = __int_as_float(hd); }
  } else {
    for (int i = tid - 32; i < RD; i += RNT - 32) {
      C.v[i] = ldf(A.v + (long long)b * A.sv, A.dt_v, (long long)h * RD + i);
      C.w[i] = A.w[(long long)h * RD + i];
    }
  }
}

// Everything between the arrival of the head's bytes and their departure, for width B.
// Returns false if the wait for the head's bytes ran out (the verdict of the whole CTA): nothing has been written then.
template <int B>
__device__ __forceinline__ bool gga_reg_head(GgaRegCtx& C, const GgaArgs& A, float* sc, uint64_t* bar, int b, int h, int hk,
                                             const uint8_t* base, int warp, int lane) {
  constexpr float qmax = static_cast<float>((1 << (B - 1)) - 1);
  constexpr int iq = (1 << (B - 1)) - 1;
  constexpr int ROWB = RD * B / 8;
  const int tid = warp * 32 + lane, M = C.M;
  const int row0 = RPW * warp, col0 = 4 * lane;
  const unsigned short* Rf = reinterpret_cast<const unsigned short*>(C.raw + RD * ROWB);
  const unsigned short* Cf = Rf + RD;

  // ---- the head's prologue on warp 0; meanwhile the other warps fetch v and w and, once the head's bytes have landed,
  // decode their part of the tile (which needs nothing of the prologue): warp 0 follows when it is done ----
  gga_reg_prologue(A, C, sc, b, h, hk, base, C.window, warp, lane);
  const bool landed = mbar_wait(bar, 0, A.wait_ns);
  // ---- decode: x = (r c) (code - qmax), pairs (columns 0,1) and (2,3) ----
  float2 x[RPW][2];
  {
    const uint2 cw = *reinterpret_cast<const uint2*>(Cf + col0);
    const float2 c01 = __half22float2(*reinterpret_cast<const __half2*>(&cw.x)), c23 = __half22float2(*reinterpret_cast<const __half2*>(&cw.y));
    const float2 off = make_float2(-(8388608.0f + qmax), -(8388608.0f + qmax));
#pragma unroll
    for (int r = 0; r < RPW; r++) {
      uint32_t u[4];
      gga_reg_codes<B>(C.raw, row0 + r, lane, u);
      const float rr = h2f(Rf[row0 + r]);
      const float2 z01 = __fadd2_rn(make_float2(__uint_as_float(u[0] | 0x4B000000u), __uint_as_float(u[1] | 0x4B000000u)), off);
      const float2 z23 = __fadd2_rn(make_float2(__uint_as_float(u[2] | 0x4B000000u), __uint_as_float(u[3] | 0x4B000000u)), off);
      x[r][0] = __fmul2_rn(__fmul2_rn(make_float2(rr, rr), c01), z01);
      x[r][1] = __fmul2_rn(__fmul2_rn(make_float2(rr, rr), c23), z23);
    }
  }
  // (a bounded wait: the verdict is taken by the whole CTA together, since threads poll on their own clocks; the barrier
  // also publishes the prologue's results)
  if (__syncthreads_or(!landed)) return false;
  C.a = sc[0]; C.bq = sc[1]; C.n = __float_as_int(sc[2]); C.hd = __float_as_int(sc[3]);
  // ---- kO = k^T O: this warp's 16 rows, then the 8 warps ----
  {
    float2 s0 = make_float2(0.f, 0.f), s1 = s0;
#pragma unroll
    for (int r = 0; r < RPW; r++) {
      const float kv = C.k[row0 + r];
      s0 = __ffma2_rn(make_float2(kv, kv), x[r][0], s0);
      s1 = __ffma2_rn(make_float2(kv, kv), x[r][1], s1);
    }
    *reinterpret_cast<float4*>(C.pa + warp * RD + col0) = make_float4(s0.x, s0.y, s1.x, s1.y);
  }
  __syncthreads();
  {
    float4 t = *reinterpret_cast<const float4*>(C.pa + col0);
#pragma unroll
    for (int w = 1; w < RNW; w++) {
      const float4 p = *reinterpret_cast<const float4*>(C.pa + w * RD + col0);
      t.x += p.x; t.y += p.y; t.z += p.z; t.w += p.w;
    }
    // ---- A O = a (O - (beta k) kO) in place, and its read-out against q ----
    const float2 a2 = make_float2(C.a, C.a);
    float2 o0 = make_float2(0.f, 0.f), o1 = o0;
#pragma unroll
    for (int r = 0; r < RPW; r++) {
      const float nb = -C.bk[row0 + r], qv = C.q[row0 + r];
      // O - bk kO as O + (-(bk kO)): the product is rounded first, as in the tile kernel
      x[r][0] = __fmul2_rn(a2, __fadd2_rn(x[r][0], __fmul2_rn(make_float2(nb, nb), make_float2(t.x, t.y))));
      x[r][1] = __fmul2_rn(a2, __fadd2_rn(x[r][1], __fmul2_rn(make_float2(nb, nb), make_float2(t.z, t.w))));
      o0 = __ffma2_rn(x[r][0], make_float2(qv, qv), o0);
      o1 = __ffma2_rn(x[r][1], make_float2(qv, qv), o1);
    }
    *reinterpret_cast<float4*>(C.pb + warp * RD + col0) = make_float4(o0.x, o0.y, o1.x, o1.y);
  }
  // ---- the window: one warp per queued pair, in age order: propagate, re-encode in FP8, read out ----
  uint8_t *PP = C.win, *VP = C.win + M * RD;
  float *PS = reinterpret_cast<float*>(C.win + 2 * M * RD), *VS = PS + M;
  if (C.window) {
    for (int i = warp; i < M; i += RNW) {
      const bool live = i < C.n;
      float cf = 0.f;
      if (live) {
        const int jj = (C.hd + i) % M;
        const float ps_ = PS[jj], vs_ = VS[jj];
        uint8_t *pp = PP + jj * RD, *vp = VP + jj * RD;
        float* pw = C.Pw + i * RD;
        // this lane's channels: lane, lane + 32, lane + 64, lane + 96
        const float2 p01 = e4m3x2_val(pp[lane], pp[lane + 32]), p23 = e4m3x2_val(pp[lane + 64], pp[lane + 96]);
        const float2 v01 = e4m3x2_val(vp[lane], vp[lane + 32]), v23 = e4m3x2_val(vp[lane + 64], vp[lane + 96]);
        float pv[4] = {p01.x * ps_, p01.y * ps_, p23.x * ps_, p23.y * ps_};
        C.Vw[i * RD + lane] = v01.x * vs_; C.Vw[i * RD + lane + 32] = v01.y * vs_;
        C.Vw[i * RD + lane + 64] = v23.x * vs_; C.Vw[i * RD + lane + 96] = v23.y * vs_;
        float kp = 0.f;
#pragma unroll
        for (int j = 0; j < 4; j++) kp = fmaf(C.k[lane + 32 * j], pv[j], kp);
        kp = warp_sum(kp);
        float am = 0.f;
#pragma unroll
        for (int j = 0; j < 4; j++) {
          pv[j] = C.a * (pv[j] - C.bk[lane + 32 * j] * kp);
          am = fmaxf(am, fabsf(pv[j]));
        }
        am = warp_max(am);
        const float sc = __fdiv_rn(am, 448.0f), safe = sc > 0.f ? sc : 1.0f;
        const uint32_t e01 = e4m3x2_byte(__fdiv_rn(pv[0], safe), __fdiv_rn(pv[1], safe));
        const uint32_t e23 = e4m3x2_byte(__fdiv_rn(pv[2], safe), __fdiv_rn(pv[3], safe));
        pp[lane] = static_cast<uint8_t>(e01 & 255u); pp[lane + 32] = static_cast<uint8_t>(e01 >> 8);
        pp[lane + 64] = static_cast<uint8_t>(e23 & 255u); pp[lane + 96] = static_cast<uint8_t>(e23 >> 8);
        const float2 y01 = e4m3x2_val(e01 & 255u, e01 >> 8), y23 = e4m3x2_val(e23 & 255u, e23 >> 8);
        const float yv[4] = {y01.x, y01.y, y23.x, y23.y};
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const float r = sc > 0.f ? yv[j] * safe : 0.f;
          pw[lane + 32 * j] = r;
          cf = fmaf(r, C.q[lane + 32 * j], cf);
        }
        if (lane == 0) PS[jj] = sc;
        cf = warp_sum(cf);
      }
      if (lane == 0) C.coef[i] = live ? cf : 0.f;
    }
  }
  __syncthreads();
  if (tid < RD) {
    float sum = C.pb[tid];
#pragma unroll
    for (int w = 1; w < RNW; w++) sum += C.pb[w * RD + tid];
    float acc = sum + C.bq * C.v[tid];
    if (C.window)
      for (int i = 0; i < M && i < C.n; i++) acc = fmaf(C.coef[i], C.Vw[i * RD + tid], acc);
    stf(C.orow, C.dt_out, tid, acc);
  }
  // ---- the rank-one write: the evicted (oldest) pair when the window is full; (beta k, v) itself without a window ----
  if (!C.window || C.n == M) {
    const float* lf = C.window ? C.Pw : C.bk;
    const float4 rv = *reinterpret_cast<const float4*>((C.window ? C.Vw : C.v) + col0);
#pragma unroll
    for (int r = 0; r < RPW; r++) {
      const float pi = lf[row0 + r];
      x[r][0] = __fadd2_rn(x[r][0], __fmul2_rn(make_float2(pi, pi), make_float2(rv.x, rv.y)));
      x[r][1] = __fadd2_rn(x[r][1], __fmul2_rn(make_float2(pi, pi), make_float2(rv.z, rv.w)));
    }
  }
  // enqueue (R(beta k), R(v)) at the slot after the youngest pair (the evicted one's when the window is full)
  if (C.window && warp < 2) {
    const int jn = C.n < M ? (C.hd + C.n) % M : C.hd;
    const float* src = warp == 0 ? C.bk : C.v;
    float am = 0.f;
    for (int t = lane; t < RD; t += 32) am = fmaxf(am, fabsf(src[t]));
    am = warp_max(am);
    const float sc = __fdiv_rn(am, 448.0f), safe = sc > 0.f ? sc : 1.0f;
    uint8_t* dst = (warp == 0 ? PP : VP) + jn * RD;
    const uint32_t e01 = e4m3x2_byte(__fdiv_rn(src[lane], safe), __fdiv_rn(src[lane + 32], safe));
    const uint32_t e23 = e4m3x2_byte(__fdiv_rn(src[lane + 64], safe), __fdiv_rn(src[lane + 96], safe));
    dst[lane] = static_cast<uint8_t>(e01 & 255u); dst[lane + 32] = static_cast<uint8_t>(e01 >> 8);
    dst[lane + 64] = static_cast<uint8_t>(e23 & 255u); dst[lane + 96] = static_cast<uint8_t>(e23 >> 8);
    if (lane == 0) (warp == 0 ? PS : VS)[jn] = sc;
  }
  // ---- the fit: row factors r = half(sqrt(max(mean |x|, 1e-20) / w)) ----
  // Range check for div_h16 on the way: every row sum below 1e14 (so every |x| is).  No lower bound is needed here: a
  // quotient x / r that is an ulp off can only come from |x| < 1e-30, and such an element weighs nothing in what
  // follows: its code is 0 whatever the last bit (|x / r / c| < 1e-15 with factors of at least 2^-24), it adds zero to
  // the refit's sums, and a column whose maximum it is gets the smallest factor 2^-24 either way.
  bool bad;
  {
    float s[RPW];
#pragma unroll
    for (int r = 0; r < RPW; r++) s[r] = (fabsf(x[r][0].x) + fabsf(x[r][0].y)) + (fabsf(x[r][1].x) + fabsf(x[r][1].y));
    const float tot = transpose_sum(s, lane);
    const int rr_ = row0 + transpose_row(lane);
    const float rf = halfc(__fsqrt_rn(__fdiv_rn(fmaxf(tot * (1.0f / RD), 1e-20f), C.w[rr_])));
    if (!(lane & (ROW_LANES - 1))) { C.rs[rr_] = rf; C.rrs[rr_] = __frcp_rn(rf); }
    bad = !(tot < 1e14f);
  }
  bad = __syncthreads_or(bad);
  if (!bad) {
    // ---- column factors c = half(max |x / r| / qmax) ----
    {
      float m0 = 0.f, m1 = 0.f, m2 = 0.f, m3 = 0.f;
#pragma unroll
      for (int r = 0; r < RPW; r++) {
        const float rv = C.rs[row0 + r], ri = C.rrs[row0 + r];
        const float2 d = make_float2(rv, rv), nd = make_float2(-rv, -rv), rd = make_float2(ri, ri);
        const float2 y0 = div_h16x2(x[r][0], d, nd, rd), y1 = div_h16x2(x[r][1], d, nd, rd);
        m0 = fmaxf(m0, fabsf(y0.x)); m1 = fmaxf(m1, fabsf(y0.y)); m2 = fmaxf(m2, fabsf(y1.x)); m3 = fmaxf(m3, fabsf(y1.y));
      }
      *reinterpret_cast<float4*>(C.pa + warp * RD + col0) = make_float4(m0, m1, m2, m3);
    }
    __syncthreads();
    bool big = false;
    if (tid < RD) {
      float mm = C.pa[tid];
#pragma unroll
      for (int w = 1; w < RNW; w++) mm = fmaxf(mm, C.pa[w * RD + tid]);
      const float cq = __fdiv_rn(mm, qmax);
      const float c0 = halfc(cq);
      C.cs[tid] = c0;
      C.rcs[tid] = __frcp_rn(c0);
      big = !(cq <= 65504.0f);                         // the factor is cut at fp16's largest value: quotients pass qmax
    }
    // Unless a column factor was cut, |x / r / c| <= qmax (1 + 2^-10) for every element and the refit's codes need no clamp.
    bad = __syncthreads_or(big);
  }
  if (!bad) {
    // ---- one weighted least-squares refit of c with the codes fixed; x / r replaces x on the way ----
    {
      const float4 c4 = *reinterpret_cast<const float4*>(C.cs + col0), rc4 = *reinterpret_cast<const float4*>(C.rcs + col0);
      const float2 ca = make_float2(c4.x, c4.y), cb = make_float2(c4.z, c4.w), nca = make_float2(-c4.x, -c4.y),
                   ncb = make_float2(-c4.z, -c4.w), rca = make_float2(rc4.x, rc4.y), rcb = make_float2(rc4.z, rc4.w);
      const float2 mg = make_float2(MAGIC, MAGIC), nmg = make_float2(-MAGIC, -MAGIC);
      float2 n0 = make_float2(0.f, 0.f), n1 = n0, d0 = n0, d1 = n0;
#pragma unroll
      for (int r = 0; r < RPW; r++) {
        const float rv = C.rs[row0 + r], ri = C.rrs[row0 + r], wv = C.w[row0 + r];
        const float ww = wv * wv;
        const float2 d = make_float2(rv, rv), nd = make_float2(-rv, -rv), rd = make_float2(ri, ri), w2 = make_float2(ww, ww);
        const float2 y0 = div_h16x2(x[r][0], d, nd, rd), y1 = div_h16x2(x[r][1], d, nd, rd);
        const float2 z0 = __fadd2_rn(__fadd2_rn(div_h16x2(y0, ca, nca, rca), mg), nmg);      // rint
        const float2 z1 = __fadd2_rn(__fadd2_rn(div_h16x2(y1, cb, ncb, rcb), mg), nmg);
        const float2 v0 = __fmul2_rn(d, z0), v1 = __fmul2_rn(d, z1);
        n0 = __fadd2_rn(n0, __fmul2_rn(__fmul2_rn(w2, v0), x[r][0]));
        n1 = __fadd2_rn(n1, __fmul2_rn(__fmul2_rn(w2, v1), x[r][1]));
        d0 = __fadd2_rn(d0, __fmul2_rn(w2, __fmul2_rn(v0, v0)));
        d1 = __fadd2_rn(d1, __fmul2_rn(w2, __fmul2_rn(v1, v1)));
        x[r][0] = y0;
        x[r][1] = y1;
      }
      *reinterpret_cast<float4*>(C.pa + warp * RD + col0) = make_float4(n0.x, n0.y, n1.x, n1.y);
      *reinterpret_cast<float4*>(C.pb + warp * RD + col0) = make_float4(d0.x, d0.y, d1.x, d1.y);
    }
    __syncthreads();
    if (tid < RD) {
      float num = 0.f, den = 0.f;
#pragma unroll
      for (int w = 0; w < RNW; w++) { num += C.pa[w * RD + tid]; den += C.pb[w * RD + tid]; }
      const float c1 = halfc(den > 0.f ? __fdiv_rn(num, fmaxf(den, 1e-30f)) : C.cs[tid]);
      C.cs[tid] = c1;
      C.rcs[tid] = __frcp_rn(c1);
    }
    __syncthreads();
    // ---- the codes with the refitted c: clamp, then round by adding 1.5 * 2^23 + 2^(B-1) (an even constant, so
    // ties still go to even codes): the sum's low B bits are code + qmax + 1, the bits above them up to bit 15 clear.
    // They go straight into the head's bytes (every thread is long past reading them). ----
    {
      const float4 c4 = *reinterpret_cast<const float4*>(C.cs + col0), rc4 = *reinterpret_cast<const float4*>(C.rcs + col0);
      const float2 ca = make_float2(c4.x, c4.y), cb = make_float2(c4.z, c4.w), nca = make_float2(-c4.x, -c4.y),
                   ncb = make_float2(-c4.z, -c4.w), rca = make_float2(rc4.x, rc4.y), rcb = make_float2(rc4.z, rc4.w);
      constexpr float MG = MAGIC + static_cast<float>(iq + 1);
      const float2 mg = make_float2(MG, MG);
#pragma unroll
      for (int r = 0; r < RPW; r++) {
        float2 y0 = div_h16x2(x[r][0], ca, nca, rca), y1 = div_h16x2(x[r][1], cb, ncb, rcb);     // x holds x / r by now
        y0 = make_float2(fminf(fmaxf(y0.x, -qmax), qmax), fminf(fmaxf(y0.y, -qmax), qmax));
        y1 = make_float2(fminf(fmaxf(y1.x, -qmax), qmax), fminf(fmaxf(y1.y, -qmax), qmax));
        const float2 t0 = __fadd2_rn(y0, mg), t1 = __fadd2_rn(y1, mg);
        const uint32_t b0 = __float_as_uint(t0.x), b1 = __float_as_uint(t0.y), b2 = __float_as_uint(t1.x), b3 = __float_as_uint(t1.y);
        if constexpr (B == 8) {
          *reinterpret_cast<uint32_t*>(C.raw + (row0 + r) * 128 + 4 * lane) =
              __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410) - 0x01010101u;
        } else if constexpr (B == 4) {
          *reinterpret_cast<unsigned short*>(C.raw + (row0 + r) * 64 + 2 * lane) =
              static_cast<unsigned short>((b0 + (b1 << 4) + (b2 << 8) + (b3 << 12)) - 0x1111u);
        } else {
          const uint32_t wd = ((b0 & 0xFFFFu) + (b1 << 6) + (b2 << 12) + (b3 << 18)) - 0x41041u;
          uint8_t* t = C.raw + (row0 + r) * 96 + 3 * lane;
          t[0] = static_cast<uint8_t>(wd & 255u); t[1] = static_cast<uint8_t>((wd >> 8) & 255u); t[2] = static_cast<uint8_t>((wd >> 16) & 255u);
        }
      }
    }
  } else {
    float xc[4 * RPW];
    uint8_t uc[4 * RPW];
#pragma unroll
    for (int r = 0; r < RPW; r++) { xc[4 * r] = x[r][0].x; xc[4 * r + 1] = x[r][0].y; xc[4 * r + 2] = x[r][1].x; xc[4 * r + 3] = x[r][1].y; }
    gga_reg_fit_cold<B>(xc, uc, C.rs, C.w, C.cs, C.pa, C.pb, warp, lane);
    for (int r = 0; r < RPW; r++) gga_reg_put<B>(C.raw, row0 + r, lane, uc[4 * r], uc[4 * r + 1], uc[4 * r + 2], uc[4 * r + 3]);
  }
  unsigned short* Rw = reinterpret_cast<unsigned short*>(C.raw + RD * ROWB);
  if (tid < RD) { Rw[tid] = f2h(C.rs[tid]); Rw[RD + tid] = f2h(C.cs[tid]); }
  return true;
}

#ifndef SQB_GGA_REG_MINB
#define SQB_GGA_REG_MINB 2
#endif
__global__ void __launch_bounds__(RNT, SQB_GGA_REG_MINB) gga_step_reg_kernel(const __grid_constant__ GgaArgs A) {
  extern __shared__ __align__(128) uint8_t rsm[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int HV = A.HV, M = A.M;
  const int bh = blockIdx.x, b = bh / HV, h = bh - b * HV, hk = h / (HV / A.HK);
  const int bits = A.bits[h];
  if (bits != 4 && bits != 6 && bits != 8) return;          // 2-bit heads and fp16 pivots: the tile kernel's
  uint8_t* orow = A.out + (long long)b * A.so + (long long)h * RD * dt_size(A.dt_out);
  const long long seq = A.idx[b];
  if (seq <= 0) {
    for (int v = tid; v < RD; v += RNT) stf(orow, A.dt_out, v, 0.0f);
    return;
  }
  const GgaRegSmem P = gga_reg_smem(M, A.qsz);
  uint64_t* bar = reinterpret_cast<uint64_t*>(rsm + P.bar);
  float* fs = reinterpret_cast<float*>(rsm + P.f0);
  uint8_t* base = A.blob + seq * A.stride;
  uint8_t* S = base + A.offs[h];
  const bool window = A.pw != 0;
  uint8_t* qb = base + A.qoff + (long long)h * A.qsz;
  const uint32_t head_bytes = RD * RD * bits / 8 + 4 * RD;
  if (tid == 0) {
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(bar, head_bytes + (window ? A.qsz : 0) + A.test_extra_tx);
    bulk_g2s(rsm + P.raw, S, head_bytes, bar);
    if (window) bulk_g2s(rsm + P.win, qb, A.qsz, bar);
  }
  GgaRegCtx C;
  C.raw = rsm + P.raw; C.win = rsm + P.win;
  C.q = fs + P.q; C.k = fs + P.k; C.bk = fs + P.bk; C.v = fs + P.v; C.o = fs + P.o; C.w = fs + P.w;
  C.rs = fs + P.rs; C.rrs = fs + P.rrs; C.cs = fs + P.cs; C.rcs = fs + P.rcs; C.pa = fs + P.pa; C.pb = fs + P.pb;
  C.Pw = fs + P.Pw; C.Vw = fs + P.Vw; C.coef = fs + P.coef;
  C.M = M; C.window = window; C.orow = orow; C.dt_out = A.dt_out;
  __syncthreads();                                          // nobody looks at the barrier before thread 0 has set it up
  float* sc = fs + P.red;                                   // a, (beta k) . q, window count, ring head
  bool done;
  if (bits == 4) done = gga_reg_head<4>(C, A, sc, bar, b, h, hk, base, warp, lane);
  else if (bits == 6) done = gga_reg_head<6>(C, A, sc, bar, b, h, hk, base, warp, lane);
  else done = gga_reg_head<8>(C, A, sc, bar, b, h, hk, base, warp, lane);
  if (!done) {
    // both copies complete on the one barrier, so after a wait that ran out there is nothing further to drain
    for (int v = tid; v < RD; v += RNT) stf(orow, A.dt_out, v, 0.0f);
    if (tid == 0 && A.status) atomicAdd(&A.status[0], 1);
    return;
  }
  // back to the slot
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if (tid == 0) {
    bulk_s2g(S, rsm + P.raw, head_bytes);
    if (window) bulk_s2g(qb, rsm + P.win, A.qsz);
    bulk_commit();
    bulk_wait_read();
  }
}

}  // namespace sqb
