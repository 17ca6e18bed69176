// The fused packed-state decode step for integer states, staged through shared memory by bulk async copies.
//
// One CTA per (batch row, KEY head); it walks the value heads that share the key head (GQA group: 2 for Qwen GDN,
// 16 for Nemotron-H Mamba2, 1 for KDA).  What depends on the key head only -- normalising q and k, the buffered
// keys and their dot products with q and k, the key appended to the buffer -- is done once per CTA; the heads'
// codes, scales and buffered values arrive through a ring of shared-memory stages filled by cp.async.bulk
// (the lanes of the first warp issue the copies, an mbarrier per stage counts the bytes), so all of a CTA's state
// traffic is in flight from its first instructions on, whatever the occupancy.  On a slot's m-th token the kernel
// only appends (the head's counter is left at m); the fold launch that follows (fold_kernel.cuh) rewrites the state.
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
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {       // never blocks
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
constexpr unsigned long long WAIT_LIMIT_NS = 1000000000ull;     // a wait gives up after one second
// Bounded wait: gives up after about limit_ns (try_wait itself may block for a hardware-defined time, so the bound is on
// a clock, not on the iteration count: the SM's cycle counter, taken as 2 cycles per nanosecond, which is cheap to read),
// records nothing itself and lets the caller bail out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long limit_ns = WAIT_LIMIT_NS) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  const long long limit = static_cast<long long>(limit_ns) * 2;
  for (int it = 0;; it++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 256) __nanosleep(64);
    if ((it & 15) == 15 && clock64() - t0 > limit) return false;
  }
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// shared-memory plan of the staged kernel (byte offsets; float offsets from f0)
struct Smem2 {
  int bars, stage0, stage_bytes, codes_b, scales_b, ub_b, kb, gbt, f0, total;
  int xq, xk, ga, ae, wq, wk, wg, fx, us, Dq, Dk, hd, decf, ubs, red, misc;
};
constexpr int HD_W = 8;     // per-head scalars: g, beta | dt, gcur, alpha, a, gnew, D, n
__host__ __device__ inline int al16i(int x) { return (x + 15) & ~15; }
__host__ __device__ inline Smem2 smem2_plan(int kind, int bits, int axk, int group, int DK, int DV, int M, int qbuf,
                                            int nst, int gqa) {
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
  int f = 0;
  s.xq = f; f += DK;
  s.xk = f; f += DK;
  s.ga = f; f += (kind == K_KDA ? DK : 0);
  s.ae = f; f += (kind == K_KDA ? DK : 0);
  s.wq = f; f += DK;                // the dot-product warp's own copy of the normalised q, k (KDA: log decay)
  s.wk = f; f += DK;
  s.wg = f; f += (kind == K_KDA ? DK : 0);
  s.fx = f; f += (axk && DK == 128 ? 6 * DK / 4 : 0);   // byte slices of the fixed-point q and k (pass_rows_fx)
  s.us = f; f += gqa * DV;
  s.Dq = f; f += 32;
  s.Dk = f; f += 32;
  s.hd = f; f += gqa * HD_W;
  s.decf = f; f += gqa * M;
  s.ubs = f; f += gqa * M;
  s.red = f; f += gqa * NW;
  s.misc = f; f += 8;
  s.total = s.f0 + ((f + 3) & ~3) * 4;
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

// 16 rounded codes, held as the low mantissa bits of t (see round_fast), packed: 8 bytes of int4 (x, y of the result)
// or 16 bytes of int8.
template <int BITS>
__device__ __forceinline__ uint4 pack_codes16(const float2 (&t)[8]) {
  uint4 o = make_uint4(0u, 0u, 0u, 0u);
  uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
  if constexpr (BITS == 4) {
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
  } else {
#pragma unroll
    for (int w = 0; w < 4; w++) {
      const uint32_t lo = __byte_perm(__float_as_uint(t[2 * w].x), __float_as_uint(t[2 * w].y), 0x0040);
      const uint32_t hi = __byte_perm(__float_as_uint(t[2 * w + 1].x), __float_as_uint(t[2 * w + 1].y), 0x0040);
      ow[w] = __byte_perm(lo, hi, 0x5410);
    }
  }
  return o;
}
template <int BITS>
__device__ __forceinline__ void store_packed16(uint8_t* p, const uint4& o) {
  if constexpr (BITS == 4) *reinterpret_cast<uint2*>(p) = make_uint2(o.x, o.y);
  else *reinterpret_cast<uint4*>(p) = o;
}
template <int BITS>
__device__ __forceinline__ void store_codes16(uint8_t* p, const float2 (&t)[8]) {
  store_packed16<BITS>(p, pack_codes16<BITS>(t));
}
// The exact path of the rounding, out of line (it is rare where round_fast applies, and long): sixteen values against
// one scale, or against sixteen scales in shared memory.
template <int BITS>
__device__ __noinline__ uint4 round_exact_pack(float2 a0, float2 a1, float2 a2, float2 a3, float2 a4, float2 a5,
                                               float2 a6, float2 a7, float sc) {
  constexpr float QMAX = BITS == 4 ? 7.0f : 127.0f;
  constexpr float MB = BITS == 4 ? MAGIC + 8.0f : MAGIC;
  const float2 a[8] = {a0, a1, a2, a3, a4, a5, a6, a7};
  float2 t[8];
#pragma unroll
  for (int p = 0; p < 8; p++) {
    t[p].x = rq_exact(a[p].x, sc, QMAX) + MB;
    t[p].y = rq_exact(a[p].y, sc, QMAX) + MB;
  }
  return pack_codes16<BITS>(t);
}
template <int BITS>
__device__ __noinline__ uint4 round_exact_pack_cols(float2 a0, float2 a1, float2 a2, float2 a3, float2 a4, float2 a5,
                                                    float2 a6, float2 a7, const float* sc) {
  constexpr float QMAX = BITS == 4 ? 7.0f : 127.0f;
  constexpr float MB = BITS == 4 ? MAGIC + 8.0f : MAGIC;
  const float2 a[8] = {a0, a1, a2, a3, a4, a5, a6, a7};
  float2 t[8];
#pragma unroll
  for (int p = 0; p < 8; p++) {
    t[p].x = rq_exact(a[p].x, sc[2 * p], QMAX) + MB;
    t[p].y = rq_exact(a[p].y, sc[2 * p + 1], QMAX) + MB;
  }
  return pack_codes16<BITS>(t);
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

// Rounds four entries of a value vector against scale s: code = clamp(rint(div_rn(x, s)), +-127), by a reciprocal
// multiply checked with an exact residual (see round_fast); returns the four codes as bytes of a word and their
// dequantised values.
__device__ __forceinline__ uint32_t round4_i8(const float* x, float s, float r, bool fast_ok, float (&deq)[4]) {
  float2 t[2];
  const float2 xv[2] = {make_float2(x[0], x[1]), make_float2(x[2], x[3])};
  bool ok = fast_ok && round_fast<2>(xv, s, r, MAGIC, t);
  if (!ok) {
    t[0].x = rq_exact(x[0], s, 127.0f) + MAGIC; t[0].y = rq_exact(x[1], s, 127.0f) + MAGIC;
    t[1].x = rq_exact(x[2], s, 127.0f) + MAGIC; t[1].y = rq_exact(x[3], s, 127.0f) + MAGIC;
  }
  deq[0] = (t[0].x - MAGIC) * s; deq[1] = (t[0].y - MAGIC) * s;
  deq[2] = (t[1].x - MAGIC) * s; deq[3] = (t[1].y - MAGIC) * s;
  const uint32_t lo = __byte_perm(__float_as_uint(t[0].x), __float_as_uint(t[0].y), 0x0040);
  const uint32_t hi = __byte_perm(__float_as_uint(t[1].x), __float_as_uint(t[1].y), 0x0040);
  return __byte_perm(lo, hi, 0x5410);
}

}  // namespace sqb
#include "fold_rows.cuh"
#include "pass_rows.cuh"
namespace sqb {

// resident CTAs per SM the register allocation aims at: states scaled along k run the integer pass in 64 registers
// with a few spilled words (measured faster than 72 registers and 7 CTAs for GDN and KDA; Mamba2, whose CTAs walk 16
// heads, is faster at 7); states scaled along v keep their scale slices in registers and stay at 4
#ifndef SQB_MINB
#define SQB_MINB 4
#endif
#ifndef SQB_MINB_K
#define SQB_MINB_K 8
#endif
#ifndef SQB_MINB_K_M2
#define SQB_MINB_K_M2 7
#endif
template <int KIND, int BITS, bool AXK, int LPR>
__global__ void __launch_bounds__(NT, AXK ? (KIND == K_M2 ? SQB_MINB_K_M2 : SQB_MINB_K) : SQB_MINB) step_tma_kernel(const __grid_constant__ StepArgs A, const __grid_constant__ Smem2 P,
                                                                const int nst) {
  constexpr int DK = LPR * 16;
  constexpr int RPP = 32 / LPR;                  // rows per warp pass
  constexpr int CW = DK / 32;                    // columns per lane in the prologue
  constexpr int QD = DK / 4;                     // columns per lane in the buffered-key dot products
  constexpr bool TWO = KIND != K_M2;
  constexpr bool VDEC = KIND == K_KDA;
  constexpr bool FX = AXK && LPR == 8;            // integer dot products against fixed-point q, k

  extern __shared__ __align__(128) uint8_t smraw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int DV = A.DV, M = A.M, HV = A.HV, G = A.group;
  const int gqa = HV / A.HK;
  const int b = blockIdx.x / A.HK, hk = blockIdx.x - b * A.HK;
  const int h0 = hk * gqa;
  const int osz = dt_size(A.dt_out);

  // ---- activation loads that do not depend on the slot: issued before anything else ----------------------------
  float qr[CW], kr[CW], g4[4];
  if (warp == 0 || warp == 3) {
#pragma unroll
    for (int j = 0; j < CW; j++) {
      qr[j] = ldf(A.q + (long long)b * A.sq, A.dt_qk, (long long)hk * DK + lane * CW + j);
      kr[j] = ldf(A.k + (long long)b * A.sk, A.dt_qk, (long long)hk * DK + lane * CW + j);
    }
  } else if (warp == 1) {
    g4[0] = g4[1] = g4[2] = g4[3] = 0.f;
    if (lane < gqa) {                                  // heads beyond 32 per key head are loaded in the loop below
      const int h = h0 + lane;
      if (KIND == K_GDN) {
        if (A.gate) {
          g4[0] = ldf(A.a + (long long)b * A.sa, A.dt_ab, h); g4[1] = ldf(A.dt_bias, A.dt_dtb, h);
          g4[2] = ldf(A.A_log, A.dt_alog, h);                 g4[3] = ldf(A.b + (long long)b * A.sb, A.dt_ab, h);
        } else {
          g4[0] = ldf(A.g + (long long)b * A.sg, A.dt_g, h);  g4[1] = ldf(A.beta + (long long)b * A.sbeta, A.dt_g, h);
        }
      } else if (KIND == K_M2) {
        g4[0] = ldf(A.g + (long long)b * A.sg, A.dt_g, h);
        if (A.dt_bias) g4[1] = ldf(A.dt_bias, A.dt_dtb, h);
        g4[2] = ldf(A.A_log, A.dt_alog, h);
        if (A.beta) g4[3] = ldf(A.beta, A.dt_beta, h);
      } else {
        g4[0] = ldf(A.beta + (long long)b * A.sbeta, A.dt_beta, h);
      }
    }
  }

  long long seq = b;
  if (A.idx != nullptr) {
    seq = A.idx[b];
    if (seq <= 0) {
      uint8_t* orow = A.out + (long long)b * A.so + (long long)h0 * DV * osz;
      for (int v = tid; v < gqa * DV; v += NT) stf(orow, A.dt_out, v, 0.0f);
      return;
    }
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smraw + P.bars);
  uint8_t* kbt = smraw + P.kb;
  float* fsm = reinterpret_cast<float*>(smraw + P.f0);
  float *xq = fsm + P.xq, *xk = fsm + P.xk, *ga = fsm + P.ga, *ae = fsm + P.ae, *us = fsm + P.us,
        *Dq = fsm + P.Dq, *Dk = fsm + P.Dk, *hd = fsm + P.hd, *decf = fsm + P.decf, *ubsf = fsm + P.ubs,
        *red = fsm + P.red, *misc = fsm + P.misc, *wq = fsm + P.wq, *wk = fsm + P.wk, *wg = fsm + P.wg;
  const float* gbt = reinterpret_cast<const float*>(smraw + P.gbt);
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
  const uint32_t stage_tx = P.codes_b + scn * 2 + M * DV * bsz;

  auto issue_stage = [&](int s, int h) {                 // one thread issues a whole stage (refills)
    uint8_t* st = smraw + P.stage0 + s * P.stage_bytes;
    mbar_expect_tx(&bars[s], stage_tx);
    bulk_g2s(st, Sseq + (long long)h * P.codes_b, P.codes_b, &bars[s]);
    bulk_g2s(st + P.codes_b, SCseq + (long long)h * scn, scn * 2, &bars[s]);
    bulk_g2s(st + P.codes_b + P.scales_b, UBseq + (long long)h * M * DV * bsz, M * DV * bsz, &bars[s]);
  };

  // ---- prologue, by role ----------------------------------------------------------------------------------------
  if (warp == 0) {
    // producer: the stage barriers, then stage 0, one copy per lane (the key tile belongs to warp 3)
    if (lane == 0) {
      for (int s = 0; s < nst; s++) mbar_init(&bars[s], 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      misc[2] = 0.f;                                      // "a copy never arrived" flag
    }
    __syncwarp();
    if (lane == 2) {
      mbar_expect_tx(&bars[0], stage_tx);
      bulk_g2s(smraw + P.stage0, Sseq + (long long)h0 * P.codes_b, P.codes_b, &bars[0]);
    } else if (lane == 3) {
      bulk_g2s(smraw + P.stage0 + P.codes_b, SCseq + (long long)h0 * scn, scn * 2, &bars[0]);
    } else if (lane == 4) {
      bulk_g2s(smraw + P.stage0 + P.codes_b + P.scales_b, UBseq + (long long)h0 * M * DV * bsz, M * DV * bsz, &bars[0]);
    }
    // the key head: its counter first (the latency overlaps the normalisation)
    const int n0 = NPseq[h0] & (M - 1);       // the heads of a slot advance together
    float gnr[CW];
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < CW; j++) {
      s0 += qr[j] * qr[j];
      s1 += kr[j] * kr[j];
      if (VDEC) gnr[j] = GCseq[(long long)h0 * DK + lane * CW + j] +
                         ldf(A.g + (long long)b * A.sg, A.dt_g, (long long)h0 * DK + lane * CW + j);
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
    float eq[CW], ek[CW], mq = 0.f, mk = 0.f;              // the vectors the state is read against
#pragma unroll
    for (int j = 0; j < CW; j++) {
      d += kr[j] * qr[j];
      mx = fmaxf(mx, fabsf(kr[j]));
      xq[lane * CW + j] = qr[j];
      xk[lane * CW + j] = kr[j];
      eq[j] = qr[j];
      ek[j] = kr[j];
      if (VDEC) {
        const float av = expf(gnr[j]);
        ga[lane * CW + j] = gnr[j];
        ae[lane * CW + j] = av;
        eq[j] = av * qr[j];
        ek[j] = av * kr[j];
      }
      mq = fmaxf(mq, fabsf(eq[j]));
      mk = fmaxf(mk, fabsf(ek[j]));
    }
    // the remaining stages
    if (lane == 0) {
      for (int s = 1; s < nst && s < gqa; s++) issue_stage(s, h0 + s);
    }
    d = warp_sum(d);
    mx = warp_max(mx);
    if (lane == 0) { misc[0] = d; misc[1] = __int_as_float(n0); }
    if constexpr (FX) {
      // q and k as 24-bit fixed point, byte slices of four columns per word (this lane's four columns)
      uint32_t* fxw = reinterpret_cast<uint32_t*>(fsm + P.fx);
      mq = warp_max(mq);
      if (TWO) mk = VDEC ? warp_max(mk) : mx;
      float mult, inv;
      fx_scale(mq, mult, inv);
      if (lane == 0) misc[4] = inv;
      put_fx_slices<BITS>(fxw, lane, fx_fixed(eq[0], mult), fx_fixed(eq[CW > 1 ? 1 : 0], mult),
                          fx_fixed(eq[CW > 2 ? 2 : 0], mult), fx_fixed(eq[CW > 3 ? 3 : 0], mult));
      if (TWO) {
        fx_scale(mk, mult, inv);
        if (lane == 0) misc[5] = inv;
        put_fx_slices<BITS>(fxw + 3 * (DK / 4), lane, fx_fixed(ek[0], mult), fx_fixed(ek[CW > 1 ? 1 : 0], mult),
                            fx_fixed(ek[CW > 2 ? 2 : 0], mult), fx_fixed(ek[CW > 3 ? 3 : 0], mult));
      }
    }
    // append the key at slot n0; its rounded value is what the fold uses for slot M-1
    if (A.qbuf) {
      const float ksc = fp16_scale(mx, 127.0f);
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < CW; j++) {
        const float cc = rq_exact(kr[j], ksc, 127.0f);
        w |= (static_cast<uint32_t>(static_cast<int>(cc)) & 0xFFu) << (8 * j);
      }
      if (CW == 4) *reinterpret_cast<uint32_t*>(KBh + (long long)n0 * DK + lane * 4) = w;
      else *reinterpret_cast<unsigned short*>(KBh + (long long)n0 * DK + lane * 2) = static_cast<unsigned short>(w);
      if (lane == 0) KBSh[n0] = f2h(ksc);
    } else {
#pragma unroll
      for (int j = 0; j < CW; j++) {
        const unsigned short bb = f2bf(kr[j]);
        reinterpret_cast<unsigned short*>(KBh)[(long long)n0 * DK + lane * CW + j] = bb;
      }
    }
  } else if (warp == 3) {
    // the buffered keys: this warp owns the key tile (barrier, copy) and takes its dot products with q and k, from
    // its own copy of the normalised vectors (same arithmetic as warp 0, so the same bits)
    if (lane == 0) {
      mbar_init(&bars[nst], 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      mbar_expect_tx(&bars[nst], M * DK * bsz + (VDEC ? M * DK * 4 : 0));
      bulk_g2s(kbt, KBh, M * DK * bsz, &bars[nst]);
      if (VDEC) bulk_g2s(smraw + P.gbt, GBseq + (long long)h0 * M * DK, M * DK * 4, &bars[nst]);
    }
    const int n0 = NPseq[h0] & (M - 1);
    float ksv = 0.f;                          // scale of buffered key `lane`
    if (A.qbuf && lane < M) ksv = h2f(KBSh[lane]);
    float gnr[CW];
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < CW; j++) {
      s0 += qr[j] * qr[j];
      s1 += kr[j] * kr[j];
      if (VDEC) gnr[j] = GCseq[(long long)h0 * DK + lane * CW + j] +
                         ldf(A.g + (long long)b * A.sg, A.dt_g, (long long)h0 * DK + lane * CW + j);
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
#pragma unroll
    for (int j = 0; j < CW; j++) {
      wq[lane * CW + j] = qr[j];
      wk[lane * CW + j] = kr[j];
      if (VDEC) wg[lane * CW + j] = gnr[j];
    }
    __syncwarp();
    if (!mbar_wait(&bars[nst], 0) && lane == 0) misc[2] = 1.f;
    // dot products of the buffered keys with q and k: lane = (slot, quarter of d_k), 8 slots per round
    for (int i0 = 0; i0 < M; i0 += 8) {
      const int i = i0 + (lane >> 2), part = lane & 3;
      const float ks_i = __shfl_sync(0xffffffffu, ksv, i & 31);
      float dq = 0.f, dk = 0.f;
      if (i < n0) {
#pragma unroll
        for (int j0 = 0; j0 < QD; j0 += 4) {
          const int k = part * QD + j0;
          float kv[4];
          if (A.qbuf) {
            const uint32_t wx = *reinterpret_cast<const uint32_t*>(kbt + i * DK + k) ^ 0x80808080u;
            kv[0] = byte_to_f<0>(wx) * ks_i; kv[1] = byte_to_f<1>(wx) * ks_i;
            kv[2] = byte_to_f<2>(wx) * ks_i; kv[3] = byte_to_f<3>(wx) * ks_i;
          } else {
            const uint2 w2 = *reinterpret_cast<const uint2*>(kbt + (i * DK + k) * 2);
            kv[0] = __uint_as_float(w2.x << 16); kv[1] = __uint_as_float(w2.x & 0xFFFF0000u);
            kv[2] = __uint_as_float(w2.y << 16); kv[3] = __uint_as_float(w2.y & 0xFFFF0000u);
          }
          const float4 q4 = *reinterpret_cast<const float4*>(wq + k);
          const float4 k4 = *reinterpret_cast<const float4*>(wk + k);
          if (VDEC) {
            const float4 g4v = *reinterpret_cast<const float4*>(wg + k);
            const float4 b4 = *reinterpret_cast<const float4*>(gbt + i * DK + k);
            kv[0] = kv[0] * expf(g4v.x - b4.x); kv[1] = kv[1] * expf(g4v.y - b4.y);
            kv[2] = kv[2] * expf(g4v.z - b4.z); kv[3] = kv[3] * expf(g4v.w - b4.w);
          }
          dq = fmaf(kv[0], q4.x, dq); dq = fmaf(kv[1], q4.y, dq); dq = fmaf(kv[2], q4.z, dq); dq = fmaf(kv[3], q4.w, dq);
          if (TWO) { dk = fmaf(kv[0], k4.x, dk); dk = fmaf(kv[1], k4.y, dk); dk = fmaf(kv[2], k4.z, dk); dk = fmaf(kv[3], k4.w, dk); }
        }
      }
      dq += __shfl_xor_sync(0xffffffffu, dq, 1); dq += __shfl_xor_sync(0xffffffffu, dq, 2);
      dk += __shfl_xor_sync(0xffffffffu, dk, 1); dk += __shfl_xor_sync(0xffffffffu, dk, 2);
      if (part == 0 && i < M) { Dq[i] = dq; Dk[i] = dk; }
    }
  } else if (warp == 1) {
    // per value head: gates and the scalars derived from them
    for (int hi = lane; hi < gqa; hi += 32) {
      const int h = h0 + hi;
      if (hi >= 32) {                                    // more than 32 heads per key head: load here
        g4[0] = g4[1] = g4[2] = g4[3] = 0.f;
        if (KIND == K_GDN) {
          if (A.gate) {
            g4[0] = ldf(A.a + (long long)b * A.sa, A.dt_ab, h); g4[1] = ldf(A.dt_bias, A.dt_dtb, h);
            g4[2] = ldf(A.A_log, A.dt_alog, h);                 g4[3] = ldf(A.b + (long long)b * A.sb, A.dt_ab, h);
          } else {
            g4[0] = ldf(A.g + (long long)b * A.sg, A.dt_g, h);  g4[1] = ldf(A.beta + (long long)b * A.sbeta, A.dt_g, h);
          }
        } else if (KIND == K_M2) {
          g4[0] = ldf(A.g + (long long)b * A.sg, A.dt_g, h);
          if (A.dt_bias) g4[1] = ldf(A.dt_bias, A.dt_dtb, h);
          g4[2] = ldf(A.A_log, A.dt_alog, h);
          if (A.beta) g4[3] = ldf(A.beta, A.dt_beta, h);
        } else {
          g4[0] = ldf(A.beta + (long long)b * A.sbeta, A.dt_beta, h);
        }
      }
      const float gcur = VDEC ? 0.f : GCseq[h];
      float g = 0.f, bt = 0.f, Dv = 0.f;
      if (KIND == K_GDN) {
        if (A.gate) {
          const float x = g4[0] + g4[1];
          const float sp = x <= 20.0f ? logf(1.0f + expf(x)) : x;
          g = -expf(g4[2]) * sp;
          bt = __fdiv_rn(1.0f, 1.0f + expf(-g4[3]));
        } else {
          g = g4[0];
          bt = g4[1];
        }
      } else if (KIND == K_M2) {
        float dtv = g4[0];
        if (A.dt_bias) dtv = dtv + g4[1];
        if (A.dt_softplus) dtv = dtv <= 20.0f ? logf(1.0f + expf(dtv)) : dtv;
        if (A.dt_clamp) dtv = fminf(fmaxf(dtv, A.dt_min), A.dt_max);
        g = __fmul_rn(g4[2], dtv);
        bt = dtv;
        Dv = g4[3];
      } else {
        bt = g4[0];
      }
      float* o = hd + hi * HD_W;
      o[0] = g; o[1] = bt; o[2] = gcur; o[3] = VDEC ? 1.0f : expf(gcur); o[4] = VDEC ? 1.0f : expf(g);
      o[5] = gcur + g; o[6] = Dv;
    }
  } else if (warp == 2) {
    // per (value head, buffer slot): counters, decay factors of the live slots and their value scales
    for (int e = lane; e < gqa * M; e += 32) {
      const int hi = e / M, i = e - hi * M, h = h0 + hi;
      const int n = NPseq[h] & (M - 1);
      const bool live = i < n;
      float dcy = 0.f, us_i = 0.f;
      if (live) {
        dcy = VDEC ? 1.0f : expf(GCseq[h] - GBseq[(long long)h * M + i]);
        us_i = A.qbuf ? h2f(UBSseq[h * M + i]) : 1.0f;
      }
      decf[e] = dcy;
      ubsf[e] = us_i;
      if (i == 0) hd[hi * HD_W + 7] = __int_as_float(n);
    }
  }
  __syncthreads();
  if (misc[2] != 0.f) {
    if (tid == 0) atomicAdd(&A.status[0], 1);
    return;
  }
  const float kq = misc[0];

  // ---- the value heads of this key head ---------------------------------------------------------------------------
  const int RW = DV / NW;
  const int npass = RW / RPP;
  const bool one_group = !AXK && RW <= G && (warp * RW) % G + RW <= G;
  float2 vq[8], vk[8];
  auto load_slice = [&](const unsigned short* scrow) {      // this lane's 16 columns of q and k, as 128-bit reads
    const float* sq = xq + c * 16;
    const float* sk = xk + c * 16;
    const float* sa = ae + c * 16;
#pragma unroll
    for (int p4 = 0; p4 < 4; p4++) {
      const float4 q4 = *reinterpret_cast<const float4*>(sq + 4 * p4);
      float4 k4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (TWO) k4 = *reinterpret_cast<const float4*>(sk + 4 * p4);
      float qv[4] = {q4.x, q4.y, q4.z, q4.w}, kv[4] = {k4.x, k4.y, k4.z, k4.w};
      if (VDEC) {
        const float4 a4 = *reinterpret_cast<const float4*>(sa + 4 * p4);
        const float av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
        for (int e = 0; e < 4; e++) { qv[e] = av[e] * qv[e]; kv[e] = av[e] * kv[e]; }
      }
      if (!AXK) {
        const uint2 sw = reinterpret_cast<const uint2*>(scrow + c * 16)[p4];          // four fp16 scales
        const float sc4[4] = {h2f(static_cast<unsigned short>(sw.x & 0xFFFFu)), h2f(static_cast<unsigned short>(sw.x >> 16)),
                              h2f(static_cast<unsigned short>(sw.y & 0xFFFFu)), h2f(static_cast<unsigned short>(sw.y >> 16))};
#pragma unroll
        for (int e = 0; e < 4; e++) { qv[e] = qv[e] * sc4[e]; kv[e] = kv[e] * sc4[e]; }
      }
#pragma unroll
      for (int e = 0; e < 4; e += 2) {
        const int p = 2 * p4 + e / 2;
        const float p0 = presc<BITS>(2 * p), p1 = presc<BITS>(2 * p + 1);
        vq[p] = make_float2(qv[e] * p0, qv[e + 1] * p1);
        vk[p] = make_float2(kv[e] * p0, kv[e + 1] * p1);
      }
    }
  };
  uint32_t fq[3][4], fk[3][4];
  int iq[3] = {0, 0, 0}, ik[3] = {0, 0, 0};
  float invq = 1.f, invk = 1.f;
  if constexpr (FX) {
    const uint4* fxv = reinterpret_cast<const uint4*>(fsm + P.fx);
#pragma unroll
    for (int i = 0; i < 3; i++) {
      const uint4 a4 = fxv[i * 8 + c];
      fq[i][0] = a4.x; fq[i][1] = a4.y; fq[i][2] = a4.z; fq[i][3] = a4.w;
      if (TWO) {
        const uint4 b4 = fxv[(3 + i) * 8 + c];
        fk[i][0] = b4.x; fk[i][1] = b4.y; fk[i][2] = b4.z; fk[i][3] = b4.w;
      } else {
        fk[i][0] = fk[i][1] = fk[i][2] = fk[i][3] = 0u;
      }
      if (BITS == 4) {                                     // nibbles carry an offset of 8
        int sq_ = 0, sk_ = 0;
#pragma unroll
        for (int w = 0; w < 4; w++) {
          sq_ = i == 0 ? dp4a_ss(fq[i][w], 0x01010101u, sq_) : static_cast<int>(__dp4a(fq[i][w], 0x01010101u, static_cast<unsigned>(sq_)));
          sk_ = i == 0 ? dp4a_ss(fk[i][w], 0x01010101u, sk_) : static_cast<int>(__dp4a(fk[i][w], 0x01010101u, static_cast<unsigned>(sk_)));
        }
        iq[i] = -8 * sq_;
        ik[i] = -8 * sk_;
      }
    }
    invq = misc[4];
    if (TWO) invk = misc[5];
  } else if (AXK) {
    load_slice(nullptr);
  }
  for (int hi = 0; hi < gqa; hi++) {
    const int h = h0 + hi;
    const int s = hi % nst;
    const uint32_t parity = (hi / nst) & 1;
    uint8_t* st = smraw + P.stage0 + s * P.stage_bytes;
    const uint8_t* codes = st;
    const unsigned short* scs = reinterpret_cast<const unsigned short*>(st + P.codes_b);
    const uint8_t* ubt = st + P.codes_b + P.scales_b;
    uint8_t* orow = A.out + (long long)b * A.so + (long long)h * DV * osz;
    const float* hdv = hd + hi * HD_W;
    const float beta = hdv[1], alpha = hdv[3], a = hdv[4], Dv = hdv[6];
    const int n = __float_as_int(hdv[7]);
    const float* dcf = decf + hi * M;
    const float* usf = ubsf + hi * M;
    float* usb = us + hi * DV;

    if (!mbar_wait(&bars[s], parity)) misc[2] = 1.f;      // checked CTA-wide after the pass

    // ---- state pass ----
    int cur_gv = -1;
    float umax = 0.f;
    if (!AXK && one_group) load_slice(scs + ((warp * RW) / G) * DK);     // this warp's rows lie in one scale group
    for (int p0 = 0; p0 < npass; p0 += LPR) {
      const bool own = p0 + c < npass;                         // this lane finishes the row of pass p0 + c
      const int orow_i = warp * RW + (own ? p0 + c : 0) * RPP + rl;
      const float vt = ldf(A.v + (long long)b * A.sv, A.dt_v, (long long)h * DV + orow_i);
      float tq, tk;
      if constexpr (FX)
        pass_rows_fx<BITS, TWO, LPR, (KIND == K_M2 ? 4 : 8)>(codes, scs, fq, fk, iq, ik, p0, npass, warp * RW, NG, gl, c, rl, tq, tk);
      else if (AXK || one_group)
        pass_rows<BITS, AXK, TWO, LPR, false>(codes, scs, vq, vk, p0, npass, warp * RW, G, NG, gl, c, rl, cur_gv,
                                              [&](int) {}, tq, tk);
      else
        pass_rows<BITS, AXK, TWO, LPR, true>(codes, scs, vq, vk, p0, npass, warp * RW, G, NG, gl, c, rl, cur_gv,
                                             [&](int gv) { load_slice(scs + gv * DK); }, tq, tk);
      if (own) {
        const int row = orow_i;
        if (FX) { tq = invq * tq; tk = invk * tk; }             // powers of two: exact
        if (!VDEC) { tq = alpha * tq; tk = alpha * tk; }
        for (int i = 0; i < n; i++) {                          // live slots only; dead ones may hold garbage
          float ub;
          if (A.qbuf) ub = static_cast<float>(reinterpret_cast<const int8_t*>(ubt)[i * DV + row]) * usf[i];
          else ub = bf2f(reinterpret_cast<const unsigned short*>(ubt)[i * DV + row]);
          tq = fmaf(ub, dcf[i] * Dq[i], tq);
          if (TWO) tk = fmaf(ub, dcf[i] * Dk[i], tk);
        }
        float u, o;
        if (KIND == K_GDN) {
          u = beta * fmaf(-a, tk, vt);
          o = fmaf(kq, u, a * tq);
        } else if (KIND == K_KDA) {
          u = beta * (vt - tk);
          o = fmaf(kq, u, tq);
        } else {
          u = beta * vt;                                       // beta holds dt
          o = fmaf(kq, u, a * tq);
          if (A.beta) o = fmaf(Dv, vt, o);
        }
        usb[row] = u;
        umax = fmaxf(umax, fabsf(u));
        stf(orow, A.dt_out, row, o);
      }
    }
    umax = warp_max(umax);
    if (lane == 0) red[hi * NW + warp] = umax;
    // appends are done after the last head; a stage that is needed again is refilled once every warp has read it
    if (hi + nst < gqa) {
      __syncthreads();
      if (tid == 0) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue_stage(s, h + nst);
      }
    }
  }
  {
    // ---- append the values of all heads at their slot n: warp w takes heads w, w + 4, ... ----
    __syncthreads();
    if (misc[2] == 0.f) {
      for (int hi = warp; hi < gqa; hi += NW) {
        const int h = h0 + hi;
        const int n = __float_as_int(hd[hi * HD_W + 7]);
        const float gnew = hd[hi * HD_W + 5];
        const float* usb = us + hi * DV;
        uint8_t* UBh = UBseq + (long long)h * M * DV * bsz;
        if (A.qbuf) {
          const float usc = fp16_scale(fmaxf(fmaxf(red[hi * NW], red[hi * NW + 1]), fmaxf(red[hi * NW + 2], red[hi * NW + 3])), 127.0f);
          const bool fast_ok = usc >= FP16_MIN_NORMAL;
          const float r = rcp_approx(usc);
          for (int e = lane; e < DV / 4; e += 32) {
            float dq4[4];
            *reinterpret_cast<uint32_t*>(UBh + (long long)n * DV + 4 * e) = round4_i8(usb + 4 * e, usc, r, fast_ok, dq4);
          }
          if (lane == 0) UBSseq[h * M + n] = f2h(usc);
        } else {
          for (int e = lane; e < DV / 2; e += 32)
            *reinterpret_cast<uint32_t*>(UBh + ((long long)n * DV + 2 * e) * 2) =
                f2bf(usb[2 * e]) | (static_cast<uint32_t>(f2bf(usb[2 * e + 1])) << 16);
        }
        if (VDEC) {
          float* GBh = GBseq + (long long)h * M * DK;
          float* GCh = GCseq + (long long)h * DK;
          for (int t = lane; t < DK; t += 32) {
            GBh[(long long)n * DK + t] = ga[t];
            GCh[t] = ga[t];
          }
        } else if (lane == 0) {
          GBseq[(long long)h * M + n] = gnew;
          GCseq[h] = gnew;
        }
        if (lane == 0) NPseq[h] = n + 1;
      }
    }
  }
  if (misc[2] != 0.f && tid == 0) atomicAdd(&A.status[0], 1);   // a copy never completed (see mbar_wait)
}

}  // namespace sqb
