// The fused packed-state decode step: one token of recurrence for one (batch row, value head) per CTA.
//
// Covers the three recurrences of the path with one kernel template (KIND):
//   Gated DeltaNet   S <- a S + k u^T,  u = beta (v - a S^T k),  o = a S^T q + (k.q) u        (scalar decay a)
//   Mamba2 / SSD     S <- a S + B u^T,  u = dt x,                y = a S^T C + (B.C) u + D x
//   KDA              S <- diag(a) S + k u^T, u = beta (v - (diag(a) S)^T k), o = (diag(a) S)^T q + (k.q) u
// against a state S_0 that is stored rounded (int4 / int8 codes with fp16 group scales, or bf16 / fp32) and only
// rewritten every m tokens.  In between, tokens sit in a buffer of (cumulative log decay G_i, key k_i, value u_i);
// a step reads the stored state once and the buffer once; when the buffer fills the state is folded,
// S = alpha_m S_0 + sum_i (alpha_m / alpha_i) k_i u_i^T, and re-rounded in place.
//
// Work decomposition (128 threads):
//   * the head's codes are [d_v rows][d_k cols], d_k contiguous.  A row is split into 16-byte chunks, one per lane:
//     LPR = d_k * bits / 128 lanes per row, 32 / LPR rows per warp pass; warp w owns rows [w d_v/4, (w+1) d_v/4).
//     Every global access to codes is a 128-bit load or store and a warp's access is one contiguous span.
//   * a lane keeps its slice of the read-out vectors (q, k) in registers for all its rows, so the inner loop is
//     unpack + packed fp32 FMA (fma.rn.f32x2) with no shared-memory operand; S^T q and S^T k are finished by
//     log2(LPR) warp shuffles per row.
//   * the buffer (a few KB) is staged dequantised in shared memory; dead slots (i >= n, possibly garbage) are
//     discarded by selection, never multiplied away.
//   * fold: the same lane <-> chunk mapping, 64 accumulators per lane, scale groups resolved by shuffles
//     (key axis) or a shuffle + shared-memory exchange (value axis); rounding is a reciprocal multiply that is
//     verified by an exact FMA residual and falls back to the IEEE division near ties, so codes are exactly
//     clamp(rint(div_rn(x, s))).
//
// Mirrors the arithmetic of the reference's Triton kernels (src/statequant/kernels/_fused_triton.py:56-190,
// 240-267, 279-394; _mamba2_triton.py:56-197, 214-332; _kda_triton.py:45-149, 218-316); only the order of fp32
// reductions differs.
#pragma once
#include "common.cuh"

namespace sqb {

struct StepArgs {
  // state tables, byte pointers / byte strides per sequence
  uint8_t *S, *SC, *KB, *KBS, *UB, *UBS, *GB, *GCUR, *NPTR;
  long long sS, sSC, sKB, sKBS, sUB, sUBS, sGB, sGC, sN;
  int group, qbuf, M, HV, HK, DK, DV, rows;
  int lpr_log2;              // log2(lanes per row)
  int state_f32;             // BITS == 16 instantiation holds fp32 values instead of bf16 (never set: own template)
  const int* idx;
  // inputs.  GDN / KDA: q, k, v, g, beta (+ a, b, A_log, dt_bias when gate).  Mamba2: q = C, k = B, v = x, g = dt,
  // A_log = A, beta = D (may be null), dt_bias (may be null).
  const uint8_t *q, *k, *v, *g, *beta, *a, *b, *A_log, *dt_bias;
  long long sq, sk, sv, sg, sbeta, sa, sb;
  uint8_t* out;
  long long so;
  int dt_qk, dt_v, dt_g, dt_beta, dt_ab, dt_alog, dt_dtb, dt_out;
  int per_key_head, gate, dt_softplus, dt_clamp;
  float scale, dt_min, dt_max;
  int* status;               // device health word: [0] counts CTAs whose bounded wait ran out
  unsigned long long wait_ns;   // how long a wait for a bulk copy may take before the CTA gives up
  int hpc;                   // tensor-core kernels: value heads a CTA takes (divides hv / hk)
  int m_log2, gqa_full;      // tensor-core kernels: log2(m), value heads per key head
  int test_extra_tx;         // test hook: bytes a stage barrier expects beyond what is copied (so its wait runs out)
  int axv;                   // tensor-core kernels: the scale groups run along d_v (32 rows per group)
};

// shared-memory plan (floats)
struct Smem {
  int xq, xk, kx, ga, ae, vin, us, R, L, cq, ck, dec, red, cmax, total;
  int rdk, ldv;   // padded row lengths of R and L
};
__host__ __device__ inline Smem smem_plan(int kind, int DK, int DV, int M, int cpl, int lpr) {
  Smem s;
  int o = 0;
  s.rdk = lpr * (cpl + 4);          // each lane chunk padded by 4 floats: conflict-free 128-bit reads
  s.ldv = DV + 32 / lpr;            // row stride that spreads (slot, row) pairs over the banks
  s.xq = o; o += DK;
  s.xk = o; o += DK;
  s.kx = o; o += DK;
  s.ga = o; o += (kind == K_KDA ? DK : 0);
  s.ae = o; o += (kind == K_KDA ? DK : 0);
  s.vin = o; o += DV;
  s.us = o; o += DV;
  s.R = o; o += M * s.rdk;
  s.L = o; o += M * s.ldv;
  s.cq = o; o += 32;
  s.ck = o; o += 32;
  s.dec = o; o += 32;
  s.red = o; o += 32;
  s.cmax = o; o += NW * DK;
  s.total = o;
  return s;
}

// ---- block reductions over NV values -------------------------------------------------------------------------------
template <int NV, bool MAX>
__device__ __forceinline__ void block_reduce(float (&v)[NV], float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < NV; i++) v[i] = MAX ? warp_max(v[i]) : warp_sum(v[i]);
  __syncthreads();   // red may still be read from an earlier reduction
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < NV; i++) red[warp * NV + i] = v[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < NV; i++) {
    float r = red[i];
#pragma unroll
    for (int w = 1; w < NW; w++) r = MAX ? fmaxf(r, red[w * NV + i]) : r + red[w * NV + i];
    v[i] = r;
  }
}

// ---- per-format chunk decoding ------------------------------------------------------------------------------------
// A chunk is 16 bytes = CPL columns.  decode() yields CPL/2 float2 pairs; for 4-bit codes the values carry the
// factor 16^e of unpack_nib8, which prescale() folds into the vector they are multiplied with.
template <int BITS> struct Fmt;
template <> struct Fmt<4> {
  static constexpr int CPL = 32;
  __device__ static __forceinline__ void decode(const uint4& c, float2 (&f)[16]) {
    float2 t[4];
    unpack_nib8(c.x, t); f[0] = t[0]; f[1] = t[1]; f[2] = t[2]; f[3] = t[3];
    unpack_nib8(c.y, t); f[4] = t[0]; f[5] = t[1]; f[6] = t[2]; f[7] = t[3];
    unpack_nib8(c.z, t); f[8] = t[0]; f[9] = t[1]; f[10] = t[2]; f[11] = t[3];
    unpack_nib8(c.w, t); f[12] = t[0]; f[13] = t[1]; f[14] = t[2]; f[15] = t[3];
  }
  __device__ static __forceinline__ float prescale(int j) { return nib_prescale(j & 7); }
};
template <> struct Fmt<8> {
  static constexpr int CPL = 16;
  __device__ static __forceinline__ void word(uint32_t w, float2* f) {
    const uint32_t wx = w ^ 0x80808080u;
    f[0] = make_float2(byte_to_f<0>(wx), byte_to_f<1>(wx));
    f[1] = make_float2(byte_to_f<2>(wx), byte_to_f<3>(wx));
  }
  __device__ static __forceinline__ void decode(const uint4& c, float2 (&f)[8]) {
    word(c.x, f); word(c.y, f + 2); word(c.z, f + 4); word(c.w, f + 6);
  }
  __device__ static __forceinline__ float prescale(int) { return 1.0f; }
};
template <> struct Fmt<16> {   // bf16 values
  static constexpr int CPL = 8;
  __device__ static __forceinline__ void decode(const uint4& c, float2 (&f)[4]) {
    f[0] = make_float2(__uint_as_float(c.x << 16), __uint_as_float(c.x & 0xFFFF0000u));
    f[1] = make_float2(__uint_as_float(c.y << 16), __uint_as_float(c.y & 0xFFFF0000u));
    f[2] = make_float2(__uint_as_float(c.z << 16), __uint_as_float(c.z & 0xFFFF0000u));
    f[3] = make_float2(__uint_as_float(c.w << 16), __uint_as_float(c.w & 0xFFFF0000u));
  }
  __device__ static __forceinline__ float prescale(int) { return 1.0f; }
};
template <> struct Fmt<32> {   // fp32 values
  static constexpr int CPL = 4;
  __device__ static __forceinline__ void decode(const uint4& c, float2 (&f)[2]) {
    f[0] = make_float2(__uint_as_float(c.x), __uint_as_float(c.y));
    f[1] = make_float2(__uint_as_float(c.z), __uint_as_float(c.w));
  }
  __device__ static __forceinline__ float prescale(int) { return 1.0f; }
};

// ---- rounding of one chunk ----------------------------------------------------------------------------------------
// t[j] = fma(x, r, MAGIC + bias) has the rounded quotient in its low mantissa bits; c = t - (MAGIC + bias) is the
// candidate code, rem = x - c s is exact, and the candidate equals rint(div_rn(x, s)) whenever |rem| stays clear
// of s/2 -- whatever the error of r (a wrong candidate is off by at least one step, so its |rem| exceeds s/2), which
// is why r may be an approximate reciprocal.  Returns true if every element of the chunk passed that test.
template <int NP>
__device__ __forceinline__ bool round_fast(const float2 (&x)[NP], float s, float r, float mb, float2 (&t)[NP]) {
  const float thr = s * 0.49998474f;   // s * (1/2 - 2^-16)
  const float2 r2 = make_float2(r, r), m2 = make_float2(mb, mb), nm2 = make_float2(-mb, -mb), ns2 = make_float2(-s, -s);
  float worst = 0.f;
#pragma unroll
  for (int p = 0; p < NP; p++) {
    t[p] = __ffma2_rn(x[p], r2, m2);
    const float2 c = __fadd2_rn(t[p], nm2);
    const float2 rem = __ffma2_rn(c, ns2, x[p]);
    worst = fmaxf(worst, fmaxf(fabsf(rem.x), fabsf(rem.y)));
  }
  return worst < thr;
}

template <int KIND, int BITS, bool AXK>
__global__ void __launch_bounds__(NT) delta_step_kernel(const __grid_constant__ StepArgs A) {
  using F = Fmt<BITS>;
  constexpr int CPL = F::CPL;            // columns per lane chunk
  constexpr int NP = CPL / 2;            // float2 pairs per chunk
  constexpr bool QUANT = BITS <= 8;
  constexpr int EB = BITS;               // bits per stored element
  constexpr int NPF = (BITS == 4) ? 4 : 8;   // row passes whose loads are in flight together
  constexpr int PPW = 64 / CPL;          // fold: rows a lane accumulates at a time
  constexpr bool TWO = KIND != K_M2;     // two read-out vectors (q and k); Mamba2 reads the state against C only
  constexpr float QMAX = BITS == 4 ? 7.0f : 127.0f;

  extern __shared__ __align__(16) float sm[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int DK = A.DK, DV = A.DV, M = A.M, HV = A.HV;
  const int bh = blockIdx.x;
  const int b = bh / HV, h = bh - b * HV;
  const int gqa = HV / A.HK, hk = h / gqa;
  uint8_t* orow = A.out + (long long)b * A.so + (long long)h * DV * dt_size(A.dt_out);

  long long seq = b;
  if (A.idx != nullptr) {
    seq = A.idx[b];
    if (seq <= 0) {   // padding row: zero the output, touch nothing else
      for (int v = tid; v < DV; v += NT) stf(orow, A.dt_out, v, 0.0f);
      return;
    }
  }
  // LPR: lanes per row rounded up to a power of two; a d_k that is not a power of two (96, 192) leaves the last lanes
  // of every row without columns: such a lane (lv false) loads nothing, reads the state against zeros and stores
  // nothing, but takes part in every shuffle
  const int LPR = 1 << A.lpr_log2, RPP = 32 >> A.lpr_log2;
  const int c = lane & (LPR - 1), rl = lane >> A.lpr_log2;
  const bool lv = c * CPL < DK;
  const Smem P = smem_plan(KIND, DK, DV, M, CPL, LPR);
  float *xq = sm + P.xq, *xk = sm + P.xk, *kxs = sm + P.kx, *ga = sm + P.ga, *ae = sm + P.ae, *vin = sm + P.vin,
        *us = sm + P.us, *R = sm + P.R, *L = sm + P.L, *cq = sm + P.cq, *ck = sm + P.ck, *dec = sm + P.dec,
        *red = sm + P.red, *cmax = sm + P.cmax;
  const int RDK = P.rdk, LDV = P.ldv;

  const int rowbytes = DK * EB / 8;
  uint8_t* Sh = A.S + seq * A.sS + (long long)h * DV * rowbytes;
  const int G = A.group;
  const int NG = QUANT && AXK ? (DK + G - 1) / G : 1;            // key-axis groups per row (the last one may be short)
  unsigned short* SCh = nullptr;
  if (QUANT) SCh = reinterpret_cast<unsigned short*>(A.SC + seq * A.sSC) + (long long)h * (AXK ? DV * NG : (DV / G) * DK);
  const int gl = QUANT && AXK ? (c * CPL) / G : 0;               // this lane's key group
  const int bsz = A.qbuf ? 1 : 2;
  uint8_t* KBh = A.KB + seq * A.sKB + (long long)hk * M * DK * bsz;
  uint8_t* UBh = A.UB + seq * A.sUB + (long long)h * M * DV * bsz;
  unsigned short* KBSh = A.qbuf ? reinterpret_cast<unsigned short*>(A.KBS + seq * A.sKBS) + hk * M : nullptr;
  unsigned short* UBSh = A.qbuf ? reinterpret_cast<unsigned short*>(A.UBS + seq * A.sUBS) + h * M : nullptr;
  constexpr bool VDEC = KIND == K_KDA;                           // decay per key channel
  float* GBh = reinterpret_cast<float*>(A.GB + seq * A.sGB) + (long long)h * M * (VDEC ? DK : 1);
  float* GCh = reinterpret_cast<float*>(A.GCUR + seq * A.sGC) + (long long)h * (VDEC ? DK : 1);
  int* NPh = reinterpret_cast<int*>(A.NPTR + seq * A.sN) + h;

  // ---- read pass: rows of this lane, first batch of code chunks in flight before anything else -----------------
  const int RW = DV / NW;                      // rows per warp
  const int npass = (RW + RPP - 1) / RPP;
  uint4 cw[NPF];
  unsigned short scw[NPF];
#pragma unroll
  for (int p = 0; p < NPF; p++) {
    const int rr = p * RPP + rl;
    cw[p] = make_uint4(0, 0, 0, 0);
    scw[p] = 0;
    if (p < npass && rr < RW && lv) {
      const int row = warp * RW + rr;
      cw[p] = *reinterpret_cast<const uint4*>(Sh + (long long)row * rowbytes + c * 16);
      if (QUANT && AXK) scw[p] = SCh[row * NG + gl];
    }
  }
  const int n = *NPh & (M - 1);

  // ---- prologue: vectors, gates ------------------------------------------------------------------------------
  float g = 0.f, beta = 0.f, dtv = 0.f, Dv = 0.f, gcur = 0.f;
  if (KIND == K_GDN) {
    if (A.gate) {
      const float x = ldf(A.a + (long long)b * A.sa, A.dt_ab, h) + ldf(A.dt_bias, A.dt_dtb, h);
      const float sp = x <= 20.0f ? logf(1.0f + expf(x)) : x;
      g = -expf(ldf(A.A_log, A.dt_alog, h)) * sp;
      beta = __fdiv_rn(1.0f, 1.0f + expf(-ldf(A.b + (long long)b * A.sb, A.dt_ab, h)));
    } else {
      g = ldf(A.g + (long long)b * A.sg, A.dt_g, h);
      beta = ldf(A.beta + (long long)b * A.sbeta, A.dt_g, h);
    }
  } else if (KIND == K_M2) {
    dtv = ldf(A.g + (long long)b * A.sg, A.dt_g, h);
    if (A.dt_bias) dtv = dtv + ldf(A.dt_bias, A.dt_dtb, h);
    if (A.dt_softplus) dtv = dtv <= 20.0f ? logf(1.0f + expf(dtv)) : dtv;
    if (A.dt_clamp) dtv = fminf(fmaxf(dtv, A.dt_min), A.dt_max);
    g = __fmul_rn(ldf(A.A_log, A.dt_alog, h), dtv);
    if (A.beta) Dv = ldf(A.beta, A.dt_beta, h);
  } else {
    beta = ldf(A.beta + (long long)b * A.sbeta, A.dt_beta, h);
  }
  if (!VDEC) gcur = *GCh;

  const int hq = (KIND == K_GDN && !A.per_key_head) ? h : hk;
  const uint8_t* qrow = A.q + (long long)b * A.sq;
  const uint8_t* krow = A.k + (long long)b * A.sk;
  const bool own_kx = KIND == K_GDN && !A.per_key_head && gqa > 1;   // buffered key = first head of the group
  float kq, kmax;
  {
    float s3[3] = {0.f, 0.f, 0.f};
    for (int t = tid; t < DK; t += NT) {
      const float qv = ldf(qrow, A.dt_qk, (long long)hq * DK + t);
      const float kv = ldf(krow, A.dt_qk, (long long)hq * DK + t);
      xq[t] = qv;
      xk[t] = kv;
      if (KIND != K_M2) {
        s3[0] += qv * qv;
        s3[1] += kv * kv;
      }
      if (own_kx) {
        const float kf = ldf(krow, A.dt_qk, (long long)(hk * gqa) * DK + t);
        kxs[t] = kf;
        s3[2] += kf * kf;
      }
      if (VDEC) {
        const float gn = GCh[t] + ldf(A.g + (long long)b * A.sg, A.dt_g, (long long)h * DK + t);
        ga[t] = gn;
        ae[t] = expf(gn);
      }
    }
    for (int v = tid; v < DV; v += NT) vin[v] = ldf(A.v + (long long)b * A.sv, A.dt_v, (long long)h * DV + v);
    if (KIND != K_M2) {
      block_reduce<3, false>(s3, red);
      const float nq = __fsqrt_rn(s3[0] + 1e-6f), nk = __fsqrt_rn(s3[1] + 1e-6f), nx = __fsqrt_rn(s3[2] + 1e-6f);
      for (int t = tid; t < DK; t += NT) {
        xq[t] = __fdiv_rn(xq[t], nq) * A.scale;
        xk[t] = __fdiv_rn(xk[t], nk);
        if (own_kx) kxs[t] = __fdiv_rn(kxs[t], nx);
      }
    }
    float d1[1] = {0.f}, m1[1] = {0.f};
    for (int t = tid; t < DK; t += NT) {
      d1[0] += xk[t] * xq[t];
      m1[0] = fmaxf(m1[0], fabsf(own_kx ? kxs[t] : xk[t]));
    }
    block_reduce<1, false>(d1, red);
    block_reduce<1, true>(m1, red);
    kq = d1[0];
    kmax = m1[0];
  }
  const float* kxp = own_kx ? kxs : xk;      // the key that goes into the buffer (Mamba2: B, held in xk)
  const float alpha = VDEC ? 1.0f : expf(gcur);
  const float a = VDEC ? 1.0f : expf(g);
  const float gnew = gcur + g;

  // ---- stage the buffer: R[i][k] = key_i (KDA: times its decay ratio), L[i][v] = u_i; dead slots -> 0 ----------
  auto rcol = [&](int k) { return (k / CPL) * (CPL + 4) + (k % CPL); };
  for (int e = tid; e < M * DK / 4; e += NT) {
    const int i = (e * 4) / DK, k0 = (e * 4) % DK;
    float f[4];
    if (A.qbuf) {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(KBh + (long long)i * DK + k0);
      const uint32_t wx = w ^ 0x80808080u;
      const float s = h2f(KBSh[i]);
      f[0] = byte_to_f<0>(wx) * s; f[1] = byte_to_f<1>(wx) * s; f[2] = byte_to_f<2>(wx) * s; f[3] = byte_to_f<3>(wx) * s;
    } else {
      const uint2 w = *reinterpret_cast<const uint2*>(KBh + ((long long)i * DK + k0) * 2);
      f[0] = __uint_as_float(w.x << 16); f[1] = __uint_as_float(w.x & 0xFFFF0000u);
      f[2] = __uint_as_float(w.y << 16); f[3] = __uint_as_float(w.y & 0xFFFF0000u);
    }
    const bool live = i < n;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float val = 0.f;
      if (live) {
        val = f[j];
        if (VDEC) val = val * expf(ga[k0 + j] - GBh[(long long)i * DK + k0 + j]);
      }
      R[i * RDK + rcol(k0 + j)] = val;
    }
  }
  for (int e = tid; e < M * DV / 4; e += NT) {
    const int i = (e * 4) / DV, v0 = (e * 4) % DV;
    float f[4];
    if (A.qbuf) {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(UBh + (long long)i * DV + v0);
      const uint32_t wx = w ^ 0x80808080u;
      const float s = h2f(UBSh[i]);
      f[0] = byte_to_f<0>(wx) * s; f[1] = byte_to_f<1>(wx) * s; f[2] = byte_to_f<2>(wx) * s; f[3] = byte_to_f<3>(wx) * s;
    } else {
      const uint2 w = *reinterpret_cast<const uint2*>(UBh + ((long long)i * DV + v0) * 2);
      f[0] = __uint_as_float(w.x << 16); f[1] = __uint_as_float(w.x & 0xFFFF0000u);
      f[2] = __uint_as_float(w.y << 16); f[3] = __uint_as_float(w.y & 0xFFFF0000u);
    }
    const bool live = i < n;
#pragma unroll
    for (int j = 0; j < 4; j++) L[i * LDV + v0 + j] = live ? f[j] : 0.f;
  }
  __syncthreads();
  // buffer coefficients c_q[i] = (a_n / a_i) k_i . q (and c_k), one warp per slot
  for (int i = warp; i < M; i += NW) {
    float sq_ = 0.f, sk_ = 0.f;
    for (int k = lane; k < DK; k += 32) {
      const float kv = R[i * RDK + rcol(k)];
      sq_ = fmaf(kv, xq[k], sq_);
      if (TWO) sk_ = fmaf(kv, xk[k], sk_);
    }
    sq_ = warp_sum(sq_);
    sk_ = warp_sum(sk_);
    if (lane == 0) {
      float d = 1.0f;
      const bool live = i < n;
      if (!VDEC && live) d = expf(gcur - GBh[i]);
      cq[i] = live ? d * sq_ : 0.f;
      ck[i] = live ? d * sk_ : 0.f;
    }
  }
  __syncthreads();

  // ---- state pass ----------------------------------------------------------------------------------------------
  // lane slice of the read-out vectors (KDA: times A = exp(G_n)); 4-bit: prescaled by 16^-e (see unpack_nib8)
  float2 vq[NP], vk[NP];
  auto load_slice = [&](const unsigned short* scrow) {
#pragma unroll
    for (int p = 0; p < NP; p++) {
      if (!lv) {
        vq[p] = make_float2(0.f, 0.f);
        vk[p] = make_float2(0.f, 0.f);
        continue;
      }
      const int k0 = c * CPL + 2 * p;
      float q0 = xq[k0], q1 = xq[k0 + 1], k0v = 0.f, k1v = 0.f;
      if (TWO) { k0v = xk[k0]; k1v = xk[k0 + 1]; }
      if (VDEC) { q0 = ae[k0] * q0; q1 = ae[k0 + 1] * q1; k0v = ae[k0] * k0v; k1v = ae[k0 + 1] * k1v; }
      if (QUANT && !AXK) {   // value-axis scales: folded into the vectors, per row group
        const float s0 = h2f(scrow[k0]), s1 = h2f(scrow[k0 + 1]);
        q0 = q0 * s0; q1 = q1 * s1; k0v = k0v * s0; k1v = k1v * s1;
      }
      const float p0 = F::prescale(2 * p), p1 = F::prescale(2 * p + 1);
      vq[p] = make_float2(q0 * p0, q1 * p1);
      vk[p] = make_float2(k0v * p0, k1v * p1);
    }
  };
  if (!(QUANT && !AXK)) load_slice(nullptr);
  int cur_gv = -1;
  for (int p0 = 0; p0 < npass; p0 += NPF) {
    if (p0 > 0) {
#pragma unroll
      for (int p = 0; p < NPF; p++) {
        const int rr = (p0 + p) * RPP + rl;
        cw[p] = make_uint4(0, 0, 0, 0);
        scw[p] = 0;
        if (p0 + p < npass && rr < RW && lv) {
          const int row = warp * RW + rr;
          cw[p] = *reinterpret_cast<const uint4*>(Sh + (long long)row * rowbytes + c * 16);
          if (QUANT && AXK) scw[p] = SCh[row * NG + gl];
        }
      }
    }
#pragma unroll
    for (int p = 0; p < NPF; p++) {
      if (p0 + p >= npass) break;                       // uniform
      const int rr = (p0 + p) * RPP + rl;
      const bool valid = rr < RW;
      const int row = valid ? warp * RW + rr : warp * RW;
      if (QUANT && !AXK) {
        const int gv = (warp * RW + (p0 + p) * RPP) / G;   // uniform over the warp: G is a multiple of RPP
        if (gv != cur_gv) {
          cur_gv = gv;
          load_slice(SCh + gv * DK);
        }
      }
      float2 f[NP];
      F::decode(cw[p], f);
      float2 aq0 = make_float2(0.f, 0.f), aq1 = aq0, ak0 = aq0, ak1 = aq0;
#pragma unroll
      for (int j = 0; j < NP; j += 2) {
        aq0 = __ffma2_rn(f[j], vq[j], aq0);
        aq1 = __ffma2_rn(f[j + 1], vq[j + 1], aq1);
        if (TWO) {
          ak0 = __ffma2_rn(f[j], vk[j], ak0);
          ak1 = __ffma2_rn(f[j + 1], vk[j + 1], ak1);
        }
      }
      float pq = (aq0.x + aq0.y) + (aq1.x + aq1.y);
      float pk = (ak0.x + ak0.y) + (ak1.x + ak1.y);
      if (QUANT && AXK) {
        const float s = h2f(scw[p]);
        pq = pq * s;
        pk = pk * s;
      }
      if (!VDEC) {
        pq = alpha * pq;
        pk = alpha * pk;
      }
      // this lane's share of the buffer term: slots c, c + LPR, ...
      for (int i = c; i < M; i += LPR) {
        const float ub = L[i * LDV + row];
        pq = fmaf(ub, cq[i], pq);
        if (TWO) pk = fmaf(ub, ck[i], pk);
      }
      for (int o = 1; o < LPR; o <<= 1) {
        pq += __shfl_xor_sync(0xffffffffu, pq, o);
        if (TWO) pk += __shfl_xor_sync(0xffffffffu, pk, o);
      }
      if (valid && c == 0) {
        const float vt = vin[row];
        float u, o;
        if (KIND == K_GDN) {
          u = beta * fmaf(-a, pk, vt);
          o = fmaf(kq, u, a * pq);
        } else if (KIND == K_KDA) {
          u = beta * (vt - pk);
          o = fmaf(kq, u, pq);
        } else {
          u = dtv * vt;
          o = fmaf(kq, u, a * pq);
          if (A.beta) o = fmaf(Dv, vt, o);
        }
        us[row] = u;
        stf(orow, A.dt_out, row, o);
      }
    }
  }
  __syncthreads();

  // ---- append at slot n ----------------------------------------------------------------------------------------
  const bool full = n == M - 1;
  float usc = 1.0f, ksc = 1.0f;
  {
    float m1[1] = {0.f};
    for (int v = tid; v < DV; v += NT) m1[0] = fmaxf(m1[0], fabsf(us[v]));
    if (A.qbuf) {
      block_reduce<1, true>(m1, red);
      usc = fp16_scale(m1[0], 127.0f);
      ksc = fp16_scale(kmax, 127.0f);
    }
  }
  const bool wkey = KIND == K_KDA || (h % gqa) == 0;
  if (A.qbuf) {
    for (int e = tid; e < DV / 4; e += NT) {
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float cc = rq_exact(us[4 * e + j], usc, 127.0f);
        w |= (static_cast<uint32_t>(static_cast<int>(cc)) & 0xFFu) << (8 * j);
        if (full) L[n * LDV + 4 * e + j] = cc * usc;
      }
      *reinterpret_cast<uint32_t*>(UBh + (long long)n * DV + 4 * e) = w;
    }
    for (int e = tid; e < DK / 4; e += NT) {
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float cc = rq_exact(kxp[4 * e + j], ksc, 127.0f);
        w |= (static_cast<uint32_t>(static_cast<int>(cc)) & 0xFFu) << (8 * j);
        if (full) R[n * RDK + rcol(4 * e + j)] = cc * ksc;
      }
      if (wkey) *reinterpret_cast<uint32_t*>(KBh + (long long)n * DK + 4 * e) = w;
    }
    if (tid == 0) {
      UBSh[n] = f2h(usc);
      if (wkey) KBSh[n] = f2h(ksc);
    }
  } else {
    for (int e = tid; e < DV / 2; e += NT) {
      const unsigned short b0 = f2bf(us[2 * e]), b1 = f2bf(us[2 * e + 1]);
      if (full) { L[n * LDV + 2 * e] = bf2f(b0); L[n * LDV + 2 * e + 1] = bf2f(b1); }
      *reinterpret_cast<uint32_t*>(UBh + ((long long)n * DV + 2 * e) * 2) = b0 | (static_cast<uint32_t>(b1) << 16);
    }
    for (int e = tid; e < DK / 2; e += NT) {
      const unsigned short b0 = f2bf(kxp[2 * e]), b1 = f2bf(kxp[2 * e + 1]);
      if (full) { R[n * RDK + rcol(2 * e)] = bf2f(b0); R[n * RDK + rcol(2 * e + 1)] = bf2f(b1); }
      if (wkey) *reinterpret_cast<uint32_t*>(KBh + ((long long)n * DK + 2 * e) * 2) = b0 | (static_cast<uint32_t>(b1) << 16);
    }
  }
  if (VDEC) {
    for (int t = tid; t < DK; t += NT) {
      GBh[(long long)n * DK + t] = ga[t];
      GCh[t] = full ? 0.f : ga[t];
    }
  } else if (tid == 0) {
    GBh[n] = gnew;
    *GCh = full ? 0.f : gnew;
  }
  if (tid == 0) *NPh = full ? 0 : n + 1;
  if (!full) return;

  // ---- fold (this sequence's buffer is full): S = decay * S_0 + sum_i L_i R_i^T in slot order, re-rounded -------
  const float alphan = VDEC ? 1.0f : expf(gnew);
  if (!VDEC) {
    if (tid < M - 1) dec[tid] = expf(gnew - GBh[tid]);      // slots 0 .. M-2 (slot M-1: exp(0) = 1)
    __syncthreads();
    for (int e = tid; e < (M - 1) * DV; e += NT) {
      const int i = e / DV, v = e - i * DV;
      L[i * LDV + v] = dec[i] * L[i * LDV + v];
    }
  }
  __syncthreads();

  // fold row mapping: an iteration covers BR rows; warp w takes ppw passes of RPP rows inside it.  Value-axis
  // formats make an iteration a whole number of scale groups (all warps of a group exchange column maxima).
  int wpg = NW, ppw = PPW, gpi = 1;           // warps per group, passes per warp, groups per iteration
  if (QUANT && !AXK) {
    wpg = min(NW, G / RPP);
    ppw = G / (RPP * wpg);
    gpi = NW / wpg;
  }
  const int BR = (QUANT && !AXK) ? gpi * G : NW * PPW * RPP;
  const int niter = (DV + BR - 1) / BR;
  for (int it = 0; it < niter; it++) {
    int rows[PPW];
    bool rv[PPW];
    float2 acc[PPW][NP];
    int gvrow = 0;
    if (QUANT && !AXK) gvrow = it * gpi + warp / wpg;
    // base: decay * (code * scale)
#pragma unroll
    for (int pp = 0; pp < PPW; pp++) {
      int row;
      if (QUANT && !AXK) row = gvrow * G + (warp % wpg) * (ppw * RPP) + pp * RPP + rl;
      else row = it * BR + warp * (PPW * RPP) + pp * RPP + rl;
      rv[pp] = pp < ppw && row < DV;
      rows[pp] = rv[pp] ? row : 0;
      uint4 cwv = make_uint4(0, 0, 0, 0);
      if (rv[pp] && lv) cwv = *reinterpret_cast<const uint4*>(Sh + (long long)rows[pp] * rowbytes + c * 16);
      F::decode(cwv, acc[pp]);
      if (QUANT && AXK) {
        const float s = rv[pp] && lv ? h2f(SCh[rows[pp] * NG + gl]) : 0.f;
#pragma unroll
        for (int p = 0; p < NP; p++) {
          const float2 s2 = make_float2(s * F::prescale(2 * p), s * F::prescale(2 * p + 1));
          acc[pp][p] = __fmul2_rn(acc[pp][p], s2);
        }
      }
    }
    if (QUANT && !AXK) {
      const bool gvalid = gvrow * G < DV && lv;
#pragma unroll
      for (int p = 0; p < NP; p++) {
        const int k0 = c * CPL + 2 * p;
        const float s0 = gvalid ? h2f(SCh[gvrow * DK + k0]) : 0.f, s1 = gvalid ? h2f(SCh[gvrow * DK + k0 + 1]) : 0.f;
        const float2 s2 = make_float2(s0 * F::prescale(2 * p), s1 * F::prescale(2 * p + 1));
#pragma unroll
        for (int pp = 0; pp < PPW; pp++) acc[pp][p] = __fmul2_rn(acc[pp][p], s2);
      }
    }
#pragma unroll
    for (int p = 0; p < NP; p++) {
      float2 d2 = make_float2(alphan, alphan);
      if (VDEC && lv) d2 = make_float2(ae[c * CPL + 2 * p], ae[c * CPL + 2 * p + 1]);
#pragma unroll
      for (int pp = 0; pp < PPW; pp++) acc[pp][p] = __fmul2_rn(acc[pp][p], d2);
    }
    // slots in order
    for (int i = 0; i < M; i++) {
      float2 l2[PPW];
#pragma unroll
      for (int pp = 0; pp < PPW; pp++) {
        const float l = L[i * LDV + rows[pp]];
        l2[pp] = make_float2(l, l);
      }
      const float4* rrow = reinterpret_cast<const float4*>(R + i * RDK + c * (CPL + 4));
#pragma unroll
      for (int j4 = 0; j4 < CPL / 4; j4++) {
        const float4 kr = rrow[j4];
        const float2 ka = make_float2(kr.x, kr.y), kb = make_float2(kr.z, kr.w);
#pragma unroll
        for (int pp = 0; pp < PPW; pp++) {
          acc[pp][2 * j4] = __ffma2_rn(l2[pp], ka, acc[pp][2 * j4]);
          acc[pp][2 * j4 + 1] = __ffma2_rn(l2[pp], kb, acc[pp][2 * j4 + 1]);
        }
      }
    }
    // ---- re-round and store ----
    if constexpr (!QUANT) {
#pragma unroll
      for (int pp = 0; pp < PPW; pp++) {
        if (!rv[pp] || !lv) continue;
        uint4 o;
        if constexpr (BITS == 16) {
          o.x = f2bf(acc[pp][0].x) | (static_cast<uint32_t>(f2bf(acc[pp][0].y)) << 16);
          o.y = f2bf(acc[pp][1].x) | (static_cast<uint32_t>(f2bf(acc[pp][1].y)) << 16);
          o.z = f2bf(acc[pp][2].x) | (static_cast<uint32_t>(f2bf(acc[pp][2].y)) << 16);
          o.w = f2bf(acc[pp][3].x) | (static_cast<uint32_t>(f2bf(acc[pp][3].y)) << 16);
        } else {
          o.x = __float_as_uint(acc[pp][0].x); o.y = __float_as_uint(acc[pp][0].y);
          o.z = __float_as_uint(acc[pp][1].x); o.w = __float_as_uint(acc[pp][1].y);
        }
        *reinterpret_cast<uint4*>(Sh + (long long)rows[pp] * rowbytes + c * 16) = o;
      }
    } else {
      // scales
      float sc[AXK ? PPW : CPL];
      if constexpr (AXK) {
        const int lpg = G / CPL;                 // lanes per key group
#pragma unroll
        for (int pp = 0; pp < PPW; pp++) {
          float am = 0.f;
#pragma unroll
          for (int p = 0; p < NP; p++) am = fmaxf(am, fmaxf(fabsf(acc[pp][p].x), fabsf(acc[pp][p].y)));
          if (!lv) am = 0.f;                     // a short last group: its missing lanes hold nothing
          for (int o = 1; o < lpg; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
          sc[pp] = fp16_scale(am, QMAX);
          if (rv[pp] && lv && (c & (lpg - 1)) == 0) SCh[rows[pp] * NG + gl] = f2h(sc[pp]);
        }
      } else {
        // column maxima over the group's rows: this lane's passes, then the lanes of other rows, then other warps
#pragma unroll
        for (int p = 0; p < NP; p++) {
          float m0 = 0.f, m1 = 0.f;
#pragma unroll
          for (int pp = 0; pp < PPW; pp++) {
            if (rv[pp]) { m0 = fmaxf(m0, fabsf(acc[pp][p].x)); m1 = fmaxf(m1, fabsf(acc[pp][p].y)); }
          }
          for (int o = LPR; o < 32; o <<= 1) {
            m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
            m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
          }
          sc[2 * p] = m0;
          sc[2 * p + 1] = m1;
        }
        __syncthreads();      // cmax free (previous iteration's readers are done)
        if (rl == 0 && lv) {
#pragma unroll
          for (int j = 0; j < CPL; j++) cmax[warp * DK + c * CPL + j] = sc[j];
        }
        __syncthreads();
        const int w0 = (warp / wpg) * wpg;
        const bool gvalid = gvrow * G < DV && lv;
#pragma unroll
        for (int j = 0; j < CPL; j++) {
          float am = 0.f;
          if (lv)
            for (int w = 0; w < wpg; w++) am = fmaxf(am, cmax[(w0 + w) * DK + c * CPL + j]);
          sc[j] = fp16_scale(am, QMAX);
          if (gvalid && rl == 0 && warp == w0) SCh[gvrow * DK + c * CPL + j] = f2h(sc[j]);
        }
      }
      // codes
#pragma unroll
      for (int pp = 0; pp < PPW; pp++) {
        if (!rv[pp] || !lv) continue;
        float2 t[NP];
        constexpr float MB = BITS == 4 ? MAGIC + 8.0f : MAGIC;
        bool ok;
        if constexpr (AXK) {
          const float s = sc[pp];
          ok = s >= FP16_MIN_NORMAL && round_fast<NP>(acc[pp], s, rcp_approx(s), MB, t);
          if (!ok) {
#pragma unroll
            for (int p = 0; p < NP; p++) {
              t[p].x = rq_exact(acc[pp][p].x, s, QMAX) + MB;
              t[p].y = rq_exact(acc[pp][p].y, s, QMAX) + MB;
            }
          }
        } else {
#pragma unroll
          for (int p = 0; p < NP; p++) {
            t[p].x = rq_exact(acc[pp][p].x, sc[2 * p], QMAX) + MB;
            t[p].y = rq_exact(acc[pp][p].y, sc[2 * p + 1], QMAX) + MB;
          }
        }
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
        if constexpr (BITS == 4) {
#pragma unroll
          for (int w = 0; w < 4; w++) {
            uint32_t x = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
              x |= (__float_as_uint(t[4 * w + j].x) & 0xFu) << (8 * j);
              x |= (__float_as_uint(t[4 * w + j].y) & 0xFu) << (8 * j + 4);
            }
            ow[w] = x;
          }
        } else {
#pragma unroll
          for (int w = 0; w < 4; w++) {
            const uint32_t lo = __byte_perm(__float_as_uint(t[2 * w].x), __float_as_uint(t[2 * w].y), 0x0040);
            const uint32_t hi = __byte_perm(__float_as_uint(t[2 * w + 1].x), __float_as_uint(t[2 * w + 1].y), 0x0040);
            ow[w] = __byte_perm(lo, hi, 0x5410);
          }
        }
        *reinterpret_cast<uint4*>(Sh + (long long)rows[pp] * rowbytes + c * 16) = o;
      }
    }
  }
}

}  // namespace sqb
