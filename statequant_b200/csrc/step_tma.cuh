// The fused packed-state decode step for integer states, staged through shared memory by bulk async copies.
//
// One CTA per (batch row, KEY head); it walks the value heads that share the key head (GQA group: 2 for Qwen GDN,
// 16 for Nemotron-H Mamba2, 1 for KDA).  What depends on the key head only -- normalising q and k, the buffered
// keys and their dot products with q and k, the key appended to the buffer -- is done once per CTA; the heads'
// codes, scales and buffered values arrive through a ring of shared-memory stages filled by cp.async.bulk
// (one elected thread issues the copies, an mbarrier per stage counts the bytes), so all of a CTA's state traffic
// is in flight from its first instructions on, whatever the occupancy.
//
// Thread mapping (128 threads): a state row (d_k codes) is cut into 16-column chunks, one per lane: LPR = d_k / 16
// lanes per row (8 bytes of int4 or 16 bytes of int8 per lane), 32 / LPR rows per warp pass, warp w owns rows
// [w d_v/4, (w+1) d_v/4).  A lane keeps its 16 columns of the read-out vectors in registers, so the inner loop is
// unpack + fma.rn.f32x2.  The partial dot products of LPR passes are reduced by a transposing butterfly (LPR-1
// shuffles per vector instead of LPR log2 LPR), after which every lane owns one finished row and does that row's
// buffer term, u and o.
//
// Arithmetic is that of the generic kernel in delta_step.cuh (same rounding of scales, payloads and buffer
// entries; only the order of fp32 reductions differs).
#pragma once
#include "delta_step.cuh"

namespace sqb {

__device__ int g_step_status[4];   // [0]: number of CTAs whose copy-completion wait ran out (0 in a healthy run)

// ---- mbarrier / bulk-copy wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: gives up after about a second, records it and lets the caller bail out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (int it = 0; it < (1 << 22); it++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 64) __nanosleep(200);
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// shared-memory plan of the staged kernel (byte offsets)
struct Smem2 {
  int bars, stage0, stage_bytes, codes_b, scales_b, ub_b, kb, gbt, f0, total;
  int xq, xk, ga, ae, us, R, L, Dq, Dk, cq, ck, dec, red, ubs, cmax, rdk, ldv;   // float offsets from f0
};
__host__ __device__ inline int al16i(int x) { return (x + 15) & ~15; }
__host__ __device__ inline Smem2 smem2_plan(int kind, int bits, int axk, int group, int DK, int DV, int M, int qbuf, int nst) {
  Smem2 s;
  const int bsz = qbuf ? 1 : 2;
  s.codes_b = DV * DK * bits / 8;
  s.scales_b = al16i((axk ? DV * (DK / group) : (DV / group) * DK) * 2);
  s.ub_b = al16i(M * DV * bsz);
  s.stage_bytes = s.codes_b + s.scales_b + s.ub_b;
  int o = 0;
  s.bars = o; o += 64;
  s.stage0 = o; o += nst * s.stage_bytes;
  s.kb = o; o += al16i(M * DK * bsz);
  s.gbt = o; o += (kind == K_KDA ? M * DK * 4 : 0);
  s.f0 = o;
  const int lpr = DK / 16;
  s.rdk = lpr * 20;                 // 16 columns + 4 floats of padding per lane chunk
  s.ldv = DV + 32 / lpr;
  int f = 0;
  s.xq = f; f += DK;
  s.xk = f; f += DK;
  s.ga = f; f += (kind == K_KDA ? DK : 0);
  s.ae = f; f += (kind == K_KDA ? DK : 0);
  s.us = f; f += DV;
  s.R = f; f += M * s.rdk;
  s.L = f; f += M * s.ldv;
  s.Dq = f; f += 32;
  s.Dk = f; f += 32;
  s.cq = f; f += 32;
  s.ck = f; f += 32;
  s.dec = f; f += 32;
  s.ubs = f; f += 32;
  s.red = f; f += 16;
  s.cmax = f; f += (axk ? 0 : 2 * NW * DK);
  s.total = s.f0 + f * 4;
  return s;
}

// 16 codes of one lane chunk -> 8 float2 pairs (4-bit: carrying the 16^e factors of unpack_nib8)
template <int BITS>
__device__ __forceinline__ void decode16(const uint8_t* p, float2 (&f)[8]) {
  if constexpr (BITS == 4) {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
    float2 t[4];
    unpack_nib8(w.x, t); f[0] = t[0]; f[1] = t[1]; f[2] = t[2]; f[3] = t[3];
    unpack_nib8(w.y, t); f[4] = t[0]; f[5] = t[1]; f[6] = t[2]; f[7] = t[3];
  } else {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    const float2 bias = make_float2(-8388736.0f, -8388736.0f);
    const uint32_t ws[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float2 a, b;
      a.x = __uint_as_float(__byte_perm(ws[i], 0x4B000000u, 0x7540));
      a.y = __uint_as_float(__byte_perm(ws[i], 0x4B000000u, 0x7541));
      b.x = __uint_as_float(__byte_perm(ws[i], 0x4B000000u, 0x7542));
      b.y = __uint_as_float(__byte_perm(ws[i], 0x4B000000u, 0x7543));
      f[2 * i] = __fadd2_rn(a, bias);
      f[2 * i + 1] = __fadd2_rn(b, bias);
    }
  }
}
template <int BITS>
__device__ __forceinline__ float presc(int j) {
  if constexpr (BITS == 4) return nib_prescale(j & 7);
  return 1.0f;
}

// 16 rounded codes, held as the low mantissa bits of t (see round_fast), packed and stored: 8 bytes of int4 or 16
// bytes of int8.
template <int BITS>
__device__ __forceinline__ void store_codes16(uint8_t* p, const float2 (&t)[8]) {
  if constexpr (BITS == 4) {
    uint2 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int w = 0; w < 2; w++) {
      uint32_t x = 0;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        x |= (__float_as_uint(t[4 * w + j].x) & 0xFu) << (8 * j);
        x |= (__float_as_uint(t[4 * w + j].y) & 0xFu) << (8 * j + 4);
      }
      ow[w] = x;
    }
    *reinterpret_cast<uint2*>(p) = o;
  } else {
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int w = 0; w < 4; w++) {
      const uint32_t lo = __byte_perm(__float_as_uint(t[2 * w].x), __float_as_uint(t[2 * w].y), 0x0040);
      const uint32_t hi = __byte_perm(__float_as_uint(t[2 * w + 1].x), __float_as_uint(t[2 * w + 1].y), 0x0040);
      ow[w] = __byte_perm(lo, hi, 0x5410);
    }
    *reinterpret_cast<uint4*>(p) = o;
  }
}

// Transposing butterfly over the LPR lanes of a row group: in v[j] = this lane's partial for pass j; out: the full
// sum of pass (lane % LPR).
template <int LPR>
__device__ __forceinline__ float transpose_reduce(float (&v)[LPR], int c) {
#pragma unroll
  for (int h = LPR / 2; h >= 1; h >>= 1) {
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

template <int KIND, int BITS, bool AXK, int LPR>
__global__ void __launch_bounds__(NT) step_tma_kernel(const __grid_constant__ StepArgs A, const int nst) {
  constexpr int DK = LPR * 16;
  constexpr int RPP = 32 / LPR;                  // rows per warp pass
  constexpr int CB = 16 * BITS / 8;              // bytes of a lane chunk
  constexpr int ROWB = DK * BITS / 8;
  constexpr int CW = DK / 32;                    // columns per lane in the prologue
  constexpr bool TWO = KIND != K_M2;
  constexpr bool VDEC = KIND == K_KDA;
  constexpr float QMAX = BITS == 4 ? 7.0f : 127.0f;
  constexpr int PPW = 2;                         // fold: rows a lane accumulates at a time

  extern __shared__ __align__(128) uint8_t smraw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int DV = A.DV, M = A.M, HV = A.HV, G = A.group;
  const int gqa = HV / A.HK;
  const int b = blockIdx.x / A.HK, hk = blockIdx.x - b * A.HK;
  const int h0 = hk * gqa;
  const int osz = dt_size(A.dt_out);

  long long seq = b;
  if (A.idx != nullptr) {
    seq = A.idx[b];
    if (seq <= 0) {
      uint8_t* orow = A.out + (long long)b * A.so + (long long)h0 * DV * osz;
      for (int v = tid; v < gqa * DV; v += NT) stf(orow, A.dt_out, v, 0.0f);
      return;
    }
  }
  const Smem2 P = smem2_plan(KIND, BITS, AXK, G, DK, DV, M, A.qbuf, nst);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smraw + P.bars);
  uint8_t* kbt = smraw + P.kb;
  float* fsm = reinterpret_cast<float*>(smraw + P.f0);
  float *xq = fsm + P.xq, *xk = fsm + P.xk, *ga = fsm + P.ga, *ae = fsm + P.ae, *us = fsm + P.us, *R = fsm + P.R,
        *L = fsm + P.L, *Dq = fsm + P.Dq, *Dk = fsm + P.Dk, *cq = fsm + P.cq, *ck = fsm + P.ck, *dec = fsm + P.dec,
        *red = fsm + P.red, *ubsf = fsm + P.ubs, *cmax = fsm + P.cmax;
  const float* gbt = reinterpret_cast<const float*>(smraw + P.gbt);
  const int RDK = P.rdk, LDV = P.ldv;
  const int bsz = A.qbuf ? 1 : 2;
  const int NG = AXK ? DK / G : 1;
  const int scn = AXK ? DV * NG : (DV / G) * DK;         // scales per head
  const int c = lane & (LPR - 1), rl = lane / LPR;
  const int gl = AXK ? (c * 16) / G : 0;

  uint8_t* Sseq = A.S + seq * A.sS;
  unsigned short* SCseq = reinterpret_cast<unsigned short*>(A.SC + seq * A.sSC);
  uint8_t* KBh = A.KB + seq * A.sKB + (long long)hk * M * DK * bsz;
  uint8_t* UBseq = A.UB + seq * A.sUB;
  unsigned short* KBSh = A.qbuf ? reinterpret_cast<unsigned short*>(A.KBS + seq * A.sKBS) + hk * M : nullptr;
  unsigned short* UBSseq = A.qbuf ? reinterpret_cast<unsigned short*>(A.UBS + seq * A.sUBS) : nullptr;
  float* GBseq = reinterpret_cast<float*>(A.GB + seq * A.sGB);
  float* GCseq = reinterpret_cast<float*>(A.GCUR + seq * A.sGC);
  int* NPseq = reinterpret_cast<int*>(A.NPTR + seq * A.sN);

  // ---- producer: barriers, the key tile, the first stages ------------------------------------------------------
  auto issue_stage = [&](int s, int h) {
    uint8_t* st = smraw + P.stage0 + s * P.stage_bytes;
    mbar_expect_tx(&bars[s], P.codes_b + scn * 2 + M * DV * bsz);
    bulk_g2s(st, Sseq + (long long)h * P.codes_b, P.codes_b, &bars[s]);
    bulk_g2s(st + P.codes_b, SCseq + (long long)h * scn, scn * 2, &bars[s]);
    bulk_g2s(st + P.codes_b + P.scales_b, UBseq + (long long)h * M * DV * bsz, M * DV * bsz, &bars[s]);
  };
  if (tid == 0) {
    for (int s = 0; s <= nst; s++) mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    uint32_t kbytes = M * DK * bsz + (VDEC ? M * DK * 4 : 0);
    mbar_expect_tx(&bars[nst], kbytes);
    bulk_g2s(kbt, KBh, M * DK * bsz, &bars[nst]);
    if (VDEC) bulk_g2s(smraw + P.gbt, GBseq + (long long)h0 * M * DK, M * DK * 4, &bars[nst]);
    for (int s = 0; s < nst && s < gqa; s++) issue_stage(s, h0 + s);
  }
  __syncthreads();     // barriers initialised before anyone polls them

  // ---- key-head prologue: each warp normalises q and k redundantly (shuffles only); lane holds CW columns -------
  const bool per_head_qk = KIND == K_GDN && !A.per_key_head;     // q, k given per value head: prologue per head
  float qr[CW], kr[CW], gnr[CW];     // normalised q (scaled), normalised k (Mamba2: C, B), KDA: running decay incl. this token
  float kq = 0.f, kmax = 0.f;
  auto prologue = [&](int hq) {
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < CW; j++) {
      qr[j] = ldf(A.q + (long long)b * A.sq, A.dt_qk, (long long)hq * DK + lane * CW + j);
      kr[j] = ldf(A.k + (long long)b * A.sk, A.dt_qk, (long long)hq * DK + lane * CW + j);
      s0 += qr[j] * qr[j];
      s1 += kr[j] * kr[j];
    }
    if (KIND != K_M2) {
      s0 = warp_sum(s0);
      s1 = warp_sum(s1);
      const float nq = __fsqrt_rn(s0 + 1e-6f), nk = __fsqrt_rn(s1 + 1e-6f);
#pragma unroll
      for (int j = 0; j < CW; j++) {
        qr[j] = __fdiv_rn(qr[j], nq) * A.scale;
        kr[j] = __fdiv_rn(kr[j], nk);
      }
    }
    float d = 0.f, mx = 0.f;
#pragma unroll
    for (int j = 0; j < CW; j++) {
      d += kr[j] * qr[j];
      mx = fmaxf(mx, fabsf(kr[j]));
    }
    kq = warp_sum(d);
    kmax = warp_max(mx);
  };
  prologue(per_head_qk ? h0 : hk);
  // the key that goes into the buffer is the group's first head's (identical to every head's when q, k are per key head)
  float kxr[CW];
#pragma unroll
  for (int j = 0; j < CW; j++) kxr[j] = kr[j];
  const float ksc = A.qbuf ? fp16_scale(kmax, 127.0f) : 1.0f;
  if (VDEC) {
#pragma unroll
    for (int j = 0; j < CW; j++) {
      const int k = lane * CW + j;
      gnr[j] = GCseq[(long long)h0 * DK + k] + ldf(A.g + (long long)b * A.sg, A.dt_g, (long long)h0 * DK + k);
    }
  }
  auto publish_qk = [&]() {     // warp 0's copy goes to shared memory for the lane slices of the state pass
    if (warp == 0) {
#pragma unroll
      for (int j = 0; j < CW; j++) {
        xq[lane * CW + j] = qr[j];
        xk[lane * CW + j] = kr[j];
        if (VDEC) { ga[lane * CW + j] = gnr[j]; ae[lane * CW + j] = expf(gnr[j]); }
      }
    }
  };
  publish_qk();

  // ---- buffered keys: dot products with q and k per slot (warp w: slots w, w + 4, ...) --------------------------
  bool alive = mbar_wait(&bars[nst], 0);
  const int n0 = NPseq[h0] & (M - 1);       // the heads of a slot advance together; each still reads its own copy below
  auto key_of = [&](int i, int j) -> float {        // buffered key i, column lane*CW + j, dequantised
    const int k = lane * CW + j;
    if (A.qbuf) return static_cast<float>(reinterpret_cast<const int8_t*>(kbt)[i * DK + k]) * h2f(KBSh[i]);
    return bf2f(reinterpret_cast<const unsigned short*>(kbt)[i * DK + k]);
  };
  auto key_dots = [&]() {
    for (int i = warp; i < M; i += NW) {
      float dq = 0.f, dk = 0.f;
      if (i < n0) {
#pragma unroll
        for (int j = 0; j < CW; j++) {
          float kv = key_of(i, j);
          if (VDEC) kv = kv * expf(gnr[j] - gbt[i * DK + lane * CW + j]);
          dq = fmaf(kv, qr[j], dq);
          if (TWO) dk = fmaf(kv, kr[j], dk);
        }
      }
      dq = warp_sum(dq);
      dk = warp_sum(dk);
      if (lane == 0) { Dq[i] = dq; Dk[i] = dk; }
    }
  };
  key_dots();
  // append the key at slot n (first head's counter); int8: one fp16 absmax scale per vector
  if (warp == 0) {
    const int n = n0;
    if (A.qbuf) {
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < CW; j++) w |= (static_cast<uint32_t>(static_cast<int>(rq_exact(kxr[j], ksc, 127.0f))) & 0xFFu) << (8 * j);
      if (CW == 4) *reinterpret_cast<uint32_t*>(KBh + (long long)n * DK + lane * 4) = w;
      else *reinterpret_cast<unsigned short*>(KBh + (long long)n * DK + lane * 2) = static_cast<unsigned short>(w);
      if (lane == 0) KBSh[n] = f2h(ksc);
    } else {
#pragma unroll
      for (int j = 0; j < CW; j++)
        reinterpret_cast<unsigned short*>(KBh)[(long long)n * DK + lane * CW + j] = f2bf(kxr[j]);
    }
  }
  alive = __syncthreads_and(alive) != 0;    // xq, xk, Dq, Dk visible; the decision to go on is CTA-wide
  if (!alive) {
    if (tid == 0) atomicAdd(&g_step_status[0], 1);
    return;
  }

  // ---- the value heads of this key head ---------------------------------------------------------------------------
  bool r_built = false;
  for (int hi = 0; hi < gqa; hi++) {
    const int h = h0 + hi;
    const int s = hi % nst;
    const uint32_t parity = (hi / nst) & 1;
    uint8_t* st = smraw + P.stage0 + s * P.stage_bytes;
    const uint8_t* codes = st;
    const unsigned short* scs = reinterpret_cast<const unsigned short*>(st + P.codes_b);
    const uint8_t* ubt = st + P.codes_b + P.scales_b;
    uint8_t* orow = A.out + (long long)b * A.so + (long long)h * DV * osz;
    unsigned short* UBSh = A.qbuf ? UBSseq + h * M : nullptr;
    float* GBh = GBseq + (long long)h * M * (VDEC ? DK : 1);
    float* GCh = GCseq + (long long)h * (VDEC ? DK : 1);
    int* NPh = NPseq + h;
    const int n = *NPh & (M - 1);

    if (per_head_qk && hi > 0) {       // q, k of this value head
      __syncthreads();
      prologue(h);
      publish_qk();
      key_dots();
      __syncthreads();
    }
    // gates
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
    const float alpha = VDEC ? 1.0f : expf(gcur);
    const float a = VDEC ? 1.0f : expf(g);
    const float gnew = gcur + g;
    // buffer coefficients of this head: c_q[i] = (a_n / a_i) (k_i . q) for live slots; buffered value scales
    if (tid < M) {
      const bool live = tid < n;
      float d = 1.0f;
      if (!VDEC && live) d = expf(gcur - GBh[tid]);
      cq[tid] = live ? d * Dq[tid] : 0.f;
      ck[tid] = live ? d * Dk[tid] : 0.f;
      ubsf[tid] = (live && A.qbuf) ? h2f(UBSh[tid]) : (live ? 1.0f : 0.f);
    }
    alive = __syncthreads_and(mbar_wait(&bars[s], parity)) != 0;
    if (!alive) break;

    // ---- state pass ----
    const int RW = DV / NW;
    const int npass = RW / RPP;
    float2 vq[8], vk[8];
    auto load_slice = [&](const unsigned short* scrow) {
#pragma unroll
      for (int p = 0; p < 8; p++) {
        const int k0 = c * 16 + 2 * p;
        float q0 = xq[k0], q1 = xq[k0 + 1], k0v = 0.f, k1v = 0.f;
        if (TWO) { k0v = xk[k0]; k1v = xk[k0 + 1]; }
        if (VDEC) { q0 = ae[k0] * q0; q1 = ae[k0 + 1] * q1; k0v = ae[k0] * k0v; k1v = ae[k0 + 1] * k1v; }
        if (!AXK) {
          const float s0 = h2f(scrow[k0]), s1 = h2f(scrow[k0 + 1]);
          q0 = q0 * s0; q1 = q1 * s1; k0v = k0v * s0; k1v = k1v * s1;
        }
        const float p0 = presc<BITS>(2 * p), p1 = presc<BITS>(2 * p + 1);
        vq[p] = make_float2(q0 * p0, q1 * p1);
        vk[p] = make_float2(k0v * p0, k1v * p1);
      }
    };
    if (AXK) load_slice(nullptr);
    int cur_gv = -1;
    float umax = 0.f;
    for (int p0 = 0; p0 < npass; p0 += LPR) {
      float pq[LPR], pk[LPR];
      const bool own = p0 + c < npass;                         // this lane finishes the row of pass p0 + c
      const int orow_i = warp * RW + (own ? p0 + c : 0) * RPP + rl;
      const float vt = ldf(A.v + (long long)b * A.sv, A.dt_v, (long long)h * DV + orow_i);
#pragma unroll
      for (int p = 0; p < LPR; p++) {
        pq[p] = 0.f;
        pk[p] = 0.f;
        if (p0 + p < npass) {                                  // uniform
          const int row = warp * RW + (p0 + p) * RPP + rl;
          if (!AXK) {
            const int gv = (warp * RW + (p0 + p) * RPP) / G;   // uniform over the warp: G is a multiple of RPP
            if (gv != cur_gv) { cur_gv = gv; load_slice(scs + gv * DK); }
          }
          float2 f[8];
          decode16<BITS>(codes + row * ROWB + c * CB, f);
          float2 aq0 = make_float2(0.f, 0.f), aq1 = aq0, ak0 = aq0, ak1 = aq0;
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            aq0 = __ffma2_rn(f[j], vq[j], aq0);
            aq1 = __ffma2_rn(f[j + 1], vq[j + 1], aq1);
            if (TWO) {
              ak0 = __ffma2_rn(f[j], vk[j], ak0);
              ak1 = __ffma2_rn(f[j + 1], vk[j + 1], ak1);
            }
          }
          float sq_ = (aq0.x + aq0.y) + (aq1.x + aq1.y);
          float sk_ = (ak0.x + ak0.y) + (ak1.x + ak1.y);
          if (AXK) {
            const float sc = h2f(scs[row * NG + gl]);
            sq_ = sq_ * sc;
            sk_ = sk_ * sc;
          }
          pq[p] = sq_;
          pk[p] = sk_;
        }
      }
      float tq = transpose_reduce<LPR>(pq, c);
      float tk = TWO ? transpose_reduce<LPR>(pk, c) : 0.f;
      if (own) {
        const int row = orow_i;
        if (!VDEC) { tq = alpha * tq; tk = alpha * tk; }
        for (int i = 0; i < M; i++) {
          float ub;
          if (A.qbuf) ub = static_cast<float>(reinterpret_cast<const int8_t*>(ubt)[i * DV + row]) * ubsf[i];
          else ub = bf2f(reinterpret_cast<const unsigned short*>(ubt)[i * DV + row]);
          ub = i < n ? ub : 0.f;
          tq = fmaf(ub, cq[i], tq);
          if (TWO) tk = fmaf(ub, ck[i], tk);
        }
        float u, o;
        if (KIND == K_GDN) {
          u = beta * fmaf(-a, tk, vt);
          o = fmaf(kq, u, a * tq);
        } else if (KIND == K_KDA) {
          u = beta * (vt - tk);
          o = fmaf(kq, u, tq);
        } else {
          u = dtv * vt;
          o = fmaf(kq, u, a * tq);
          if (A.beta) o = fmaf(Dv, vt, o);
        }
        us[row] = u;
        umax = fmaxf(umax, fabsf(u));
        stf(orow, A.dt_out, row, o);
      }
    }
    // ---- append the value at slot n: one absmax scale over the whole row ----
    umax = warp_max(umax);
    if (lane == 0) red[warp] = umax;
    __syncthreads();
    const bool full = n == M - 1;
    float usc = 1.0f;
    if (A.qbuf) usc = fp16_scale(fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3])), 127.0f);
    uint8_t* UBh = UBseq + (long long)h * M * DV * bsz;
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
      if (tid == 0) UBSh[n] = f2h(usc);
    } else {
      for (int e = tid; e < DV / 2; e += NT) {
        const unsigned short b0 = f2bf(us[2 * e]), b1 = f2bf(us[2 * e + 1]);
        if (full) { L[n * LDV + 2 * e] = bf2f(b0); L[n * LDV + 2 * e + 1] = bf2f(b1); }
        *reinterpret_cast<uint32_t*>(UBh + ((long long)n * DV + 2 * e) * 2) = b0 | (static_cast<uint32_t>(b1) << 16);
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

    // ---- fold ----
    if (full) {
      const float alphan = VDEC ? 1.0f : expf(gnew);
      // R: the keys of all slots (KDA: times their decay ratio), once per key head; slot M-1 from registers
      if (!r_built) {
        for (int i = warp; i < M - 1; i += NW) {
#pragma unroll
          for (int j = 0; j < CW; j++) {
            const int k = lane * CW + j;
            float kv = key_of(i, j);
            if (VDEC) kv = kv * expf(gnr[j] - gbt[i * DK + k]);
            R[i * RDK + (k / 16) * 20 + (k % 16)] = kv;
          }
        }
        if (warp == 0) {
#pragma unroll
          for (int j = 0; j < CW; j++) {
            const int k = lane * CW + j;
            const float kv = A.qbuf ? rq_exact(kxr[j], ksc, 127.0f) * ksc : bf2f(f2bf(kxr[j]));
            R[(M - 1) * RDK + (k / 16) * 20 + (k % 16)] = kv;
          }
        }
        r_built = true;
      }
      // L: the buffered values of slots 0..M-2 times their decay (GDN, Mamba2); slot M-1 was written above
      if (!VDEC && tid < M - 1) dec[tid] = expf(gnew - GBh[tid]);
      __syncthreads();
      for (int e = tid; e < (M - 1) * DV; e += NT) {
        const int i = e / DV, v = e - i * DV;
        float ub;
        if (A.qbuf) ub = static_cast<float>(reinterpret_cast<const int8_t*>(ubt)[i * DV + v]) * ubsf[i];
        else ub = bf2f(reinterpret_cast<const unsigned short*>(ubt)[i * DV + v]);
        L[i * LDV + v] = VDEC ? ub : dec[i] * ub;
      }
      __syncthreads();

      int wpg = NW, ppw = PPW, gpi = 1;
      if (!AXK) {
        wpg = min(NW, G / RPP);
        ppw = G / (RPP * wpg);
        gpi = NW / wpg;
      }
      const int BR = AXK ? NW * PPW * RPP : gpi * G;
      const int niter = (DV + BR - 1) / BR;
      unsigned short* SCh = SCseq + (long long)h * scn;
      uint8_t* Sh = Sseq + (long long)h * P.codes_b;
      for (int it = 0; it < niter; it++) {
        int rows[PPW];
        bool rv[PPW];
        float2 acc[PPW][8];
        const int gvrow = AXK ? 0 : it * gpi + warp / wpg;
#pragma unroll
        for (int pp = 0; pp < PPW; pp++) {
          int row;
          if (AXK) row = it * BR + warp * (PPW * RPP) + pp * RPP + rl;
          else row = gvrow * G + (warp % wpg) * (ppw * RPP) + pp * RPP + rl;
          rv[pp] = pp < ppw && row < DV;
          rows[pp] = rv[pp] ? row : 0;
          decode16<BITS>(codes + rows[pp] * ROWB + c * CB, acc[pp]);
          if (AXK) {
            const float sc = h2f(scs[rows[pp] * NG + gl]);
#pragma unroll
            for (int p = 0; p < 8; p++)
              acc[pp][p] = __fmul2_rn(acc[pp][p], make_float2(sc * presc<BITS>(2 * p), sc * presc<BITS>(2 * p + 1)));
          }
        }
        if (!AXK) {
          const bool gvalid = gvrow * G < DV;
#pragma unroll
          for (int p = 0; p < 8; p++) {
            const int k0 = c * 16 + 2 * p;
            const float s0 = gvalid ? h2f(scs[gvrow * DK + k0]) : 0.f, s1 = gvalid ? h2f(scs[gvrow * DK + k0 + 1]) : 0.f;
            const float2 s2 = make_float2(s0 * presc<BITS>(2 * p), s1 * presc<BITS>(2 * p + 1));
#pragma unroll
            for (int pp = 0; pp < PPW; pp++) acc[pp][p] = __fmul2_rn(acc[pp][p], s2);
          }
        }
#pragma unroll
        for (int p = 0; p < 8; p++) {
          float2 d2 = make_float2(alphan, alphan);
          if (VDEC) d2 = make_float2(ae[c * 16 + 2 * p], ae[c * 16 + 2 * p + 1]);
#pragma unroll
          for (int pp = 0; pp < PPW; pp++) acc[pp][p] = __fmul2_rn(acc[pp][p], d2);
        }
        for (int i = 0; i < M; i++) {
          float2 l2[PPW];
#pragma unroll
          for (int pp = 0; pp < PPW; pp++) {
            const float l = L[i * LDV + rows[pp]];
            l2[pp] = make_float2(l, l);
          }
          const float4* rrow = reinterpret_cast<const float4*>(R + i * RDK + c * 20);
#pragma unroll
          for (int j4 = 0; j4 < 4; j4++) {
            const float4 kr4 = rrow[j4];
            const float2 ka = make_float2(kr4.x, kr4.y), kb2 = make_float2(kr4.z, kr4.w);
#pragma unroll
            for (int pp = 0; pp < PPW; pp++) {
              acc[pp][2 * j4] = __ffma2_rn(l2[pp], ka, acc[pp][2 * j4]);
              acc[pp][2 * j4 + 1] = __ffma2_rn(l2[pp], kb2, acc[pp][2 * j4 + 1]);
            }
          }
        }
        // re-round
        constexpr float MB = BITS == 4 ? MAGIC + 8.0f : MAGIC;
        if constexpr (AXK) {
          const int lpg = G / 16;
#pragma unroll
          for (int pp = 0; pp < PPW; pp++) {
            float am = 0.f;
#pragma unroll
            for (int p = 0; p < 8; p++) am = fmaxf(am, fmaxf(fabsf(acc[pp][p].x), fabsf(acc[pp][p].y)));
            for (int o = 1; o < lpg; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
            const float sc = fp16_scale(am, QMAX);
            if (!rv[pp]) continue;
            if ((c & (lpg - 1)) == 0) SCh[rows[pp] * NG + gl] = f2h(sc);
            float2 t[8];
            bool ok = sc >= FP16_MIN_NORMAL && round_fast<8>(acc[pp], sc, __fdiv_rn(1.0f, sc), MB, t);
            if (!ok) {
#pragma unroll
              for (int p = 0; p < 8; p++) {
                t[p].x = rq_exact(acc[pp][p].x, sc, QMAX) + MB;
                t[p].y = rq_exact(acc[pp][p].y, sc, QMAX) + MB;
              }
            }
            store_codes16<BITS>(Sh + (long long)rows[pp] * ROWB + c * CB, t);
          }
        } else {
          // column maxima over the group's rows: this lane's passes, the lanes of other rows, the other warps
          float cm[16];
#pragma unroll
          for (int p = 0; p < 8; p++) {
            float m0 = 0.f, m1 = 0.f;
#pragma unroll
            for (int pp = 0; pp < PPW; pp++) {
              if (rv[pp]) { m0 = fmaxf(m0, fabsf(acc[pp][p].x)); m1 = fmaxf(m1, fabsf(acc[pp][p].y)); }
            }
            for (int o = LPR; o < 32; o <<= 1) {
              m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
              m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
            }
            cm[2 * p] = m0;
            cm[2 * p + 1] = m1;
          }
          __syncthreads();
          if (rl == 0) {
#pragma unroll
            for (int j = 0; j < 16; j++) cmax[warp * DK + c * 16 + j] = cm[j];
          }
          __syncthreads();
          // scale and reciprocal of every column of every group in flight, one column per thread
          float* ssc = cmax + NW * DK;          // [gpi][DK] scales, reciprocal flag packed alongside
          for (int e = tid; e < gpi * DK; e += NT) {
            const int gi = e / DK, k = e - gi * DK;
            float am = 0.f;
            for (int w = 0; w < wpg; w++) am = fmaxf(am, cmax[(gi * wpg + w) * DK + k]);
            const float sc = fp16_scale(am, QMAX);
            ssc[gi * DK + k] = sc;
            const int gvr = it * gpi + gi;
            if (gvr * G < DV) SCh[gvr * DK + k] = f2h(sc);
          }
          __syncthreads();
          const float* myssc = ssc + (warp / wpg) * DK + c * 16;
#pragma unroll
          for (int pp = 0; pp < PPW; pp++) {
            if (!rv[pp]) continue;
            float2 t[8];
#pragma unroll
            for (int p = 0; p < 8; p++) {
              t[p].x = rq_exact(acc[pp][p].x, myssc[2 * p], QMAX) + MB;
              t[p].y = rq_exact(acc[pp][p].y, myssc[2 * p + 1], QMAX) + MB;
            }
            store_codes16<BITS>(Sh + (long long)rows[pp] * ROWB + c * CB, t);
          }
        }
      }
    }
    // ---- this stage is free: refill it with the head nst further on ----
    __syncthreads();
    if (tid == 0 && hi + nst < gqa) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      issue_stage(s, h + nst);
    }
  }
  if (!alive) {
    // a copy never completed: record it and leave without touching the state further.  Nothing else of this CTA is
    // in flight except copies into its own shared memory, which the hardware retires with the CTA.
    if (tid == 0) atomicAdd(&g_step_status[0], 1);
  }
}

}  // namespace sqb
