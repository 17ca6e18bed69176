// The fused packed-state decode step as a persistent, warp-specialised pipeline.
//
// A CTA is four consumer warps and one producer warp, and stays on its SM for the whole launch, walking the tiles
// (batch row, key head) bid, bid + grid, ...  The producer warp runs ahead of the consumers:
//   * it keeps a ring of shared-memory stages full -- one stage is one value head's codes, scales and buffered
//     values, fetched by cp.async.bulk and counted by the stage's "full" mbarrier; the consumers hand a stage back
//     through its "empty" mbarrier;
//   * it does everything of a tile that depends on the key head only (normalising q and k, appending the key to the
//     buffer, the buffered keys' dot products with q and k, the gates and decay factors of the value heads) into a
//     ring of prologue buffers, again handed over by full / empty mbarriers.
// So the dependent global loads at the head of a tile (slot index -> counters and scales -> key tile) and the
// single-warp arithmetic of the prologue overlap the consumers' state passes of the tiles before, and a stage's
// refill is in flight while the other stages are being read.  The consumers' work per head is the state pass of the
// staged kernel (step_tma.cuh: 16-column lane chunks, fma.rn.f32x2, transposing butterfly) and, on a slot's m-th
// token, the fold of that head; they synchronise among themselves with a named barrier that leaves the producer out.
//
// Every wait is bounded; a wait that runs out raises the CTA's abort flag, all roles leave their loops, the producer
// waits (bounded) for the copies it still has in flight, and the launch counts it in the device health word (StepArgs::status).
#pragma once
#include "step_tma.cuh"

namespace sqb {

constexpr int NTP = NT + 32;          // consumer threads + the producer warp
constexpr int MAXST = 6;              // most stages of the ring
constexpr int MAXPB = 3;              // most prologue buffers

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Bounded wait (see mbar_wait) that also gives up when another role of the CTA has raised the abort flag.
__device__ __forceinline__ bool mbar_wait_ab(uint64_t* bar, uint32_t parity, volatile int* abortf) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (int it = 0;; it++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 64) __nanosleep(100);
    if ((it & 15) == 15) {
      if (*abortf) return false;
      if (global_ns() - t0 > WAIT_LIMIT_NS) { *abortf = 1; return false; }
    }
  }
}

// Shared-memory plan (byte offsets; float offsets inside a prologue buffer from p_f, inside the consumers' region
// from c0).
struct Smem3 {
  int bars, abortf, stage0, stage_bytes, codes_b, scales_b, ub_b;
  int pb0, pb_bytes, p_kb, p_gbt, p_v, p_f;
  int xq, xk, ga, ae, krnd, Dq, Dk, ksf, hd, cq, ck, ubs, gbv, misc;
  int c0, us, red, R, L, cmax, us_n, red_n;
  int rdk, ldv, total;
};
__host__ __device__ inline Smem3 smem3_plan(int kind, int bits, int axk, int group, int DK, int DV, int M, int qbuf,
                                            int nst, int npb, int gqa, int vsz) {
  Smem3 s;
  const int bsz = qbuf ? 1 : 2;
  const int lpr = DK / 16;
  s.rdk = lpr * 20;
  s.ldv = fold_lm(M);
  s.codes_b = DV * DK * bits / 8;
  s.scales_b = al16i((axk ? DV * (DK / group) : (DV / group) * DK) * 2);
  s.ub_b = al16i(M * DV * bsz);
  s.stage_bytes = s.codes_b + s.scales_b + s.ub_b;
  int o = 0;
  s.bars = o; o += (2 * MAXST + 3 * MAXPB + 1) * 8;
  s.abortf = o; o += 16;
  o = (o + 127) & ~127;
  s.stage0 = o; o += nst * s.stage_bytes;
  // one prologue buffer
  int p = 0;
  s.p_kb = p; p += al16i(M * DK * bsz);
  s.p_gbt = p; p += (kind == K_KDA ? M * DK * 4 : 0);
  s.p_v = p; p += al16i(gqa * DV * vsz);
  s.p_f = p;
  int f = 0;
  s.xq = f; f += DK;
  s.xk = f; f += DK;
  s.ga = f; f += (kind == K_KDA ? DK : 0);
  s.ae = f; f += (kind == K_KDA ? DK : 0);
  s.krnd = f;
  s.Dq = f; f += 32;
  s.Dk = f; f += 32;
  s.ksf = f;
  s.hd = f; f += gqa * HD_W;
  s.cq = f; f += gqa * M;
  s.ck = f; f += gqa * M;
  s.ubs = f; f += gqa * M;
  s.gbv = f;
  f = (f + 3) & ~3;                         // misc holds a 64-bit slot number
  s.misc = f; f += 8;
  s.pb_bytes = al16i(s.p_f + f * 4);
  s.pb0 = o; o += npb * s.pb_bytes;
  // the consumers' own region
  s.c0 = o;
  f = 0;
  s.us_n = gqa * DV;
  s.red_n = gqa * NW;
  s.us = f; f += 2 * s.us_n;
  s.red = f; f += 2 * s.red_n;
  s.R = s.L = s.cmax = f;
  s.total = s.c0 + ((f + 3) & ~3) * 4;
  return s;
}

struct PipeCfg {
  int nst, npb, grid, ntiles, v_bulk;
};

template <int KIND, int BITS, bool AXK, int LPR>
__global__ void __launch_bounds__(NTP, 3) step_pipe_kernel(const __grid_constant__ StepArgs A,
                                                           const __grid_constant__ Smem3 P,
                                                           const __grid_constant__ PipeCfg C) {
  constexpr int DK = LPR * 16;
  constexpr int RPP = 32 / LPR;
  constexpr int CB = 16 * BITS / 8;
  constexpr int ROWB = DK * BITS / 8;
  constexpr int CW = DK / 32;
  constexpr int QD = DK / 4;
  constexpr bool TWO = KIND != K_M2;
  constexpr bool VDEC = KIND == K_KDA;

  extern __shared__ __align__(128) uint8_t smraw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int DV = A.DV, M = A.M, HV = A.HV, HK = A.HK, G = A.group;
  const int gqa = HV / HK;
  const int nst = C.nst, npb = C.npb;
  const int bsz = A.qbuf ? 1 : 2;
  const int vsz = dt_size(A.dt_v), osz = dt_size(A.dt_out);
  const int NG = AXK ? DK / G : 1;
  const int scn = AXK ? DV * NG : (DV / G) * DK;
  const uint32_t stage_tx = P.codes_b + scn * 2 + M * DV * bsz;

  uint64_t* sfull = reinterpret_cast<uint64_t*>(smraw + P.bars);
  uint64_t* sempty = sfull + MAXST;
  uint64_t* pfull = sempty + MAXST;
  uint64_t* pempty = pfull + MAXPB;
  uint64_t* kbfull = pempty + MAXPB;
  uint64_t* cbar = kbfull + MAXPB;          // the consumers' own barrier (bounded, unlike bar.sync)
  volatile int* abortf = reinterpret_cast<volatile int*>(smraw + P.abortf);

  if (tid == 0) {
    for (int s = 0; s < nst; s++) { mbar_init(&sfull[s], 1); mbar_init(&sempty[s], NW); }
    for (int s = 0; s < npb; s++) { mbar_init(&pfull[s], 1); mbar_init(&pempty[s], NW); mbar_init(&kbfull[s], 1); }
    mbar_init(cbar, NW);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    *abortf = 0;
  }
  __syncthreads();

  const int bid = blockIdx.x, grid = C.grid;
  const int nt_cta = bid < C.ntiles ? (C.ntiles - bid + grid - 1) / grid : 0;
  auto seq_of = [&](int j) -> long long {                  // slot of this CTA's j-th tile (0 / negative: padding)
    const int b = (bid + j * grid) / HK;
    return A.idx != nullptr ? static_cast<long long>(A.idx[b]) : static_cast<long long>(b) + 1;
  };
  // lockstep launches (no index) number their sequences from 0; seq_of returns slot + 1 for them
  const long long seq_bias = A.idx != nullptr ? 0 : 1;

  if (warp == NW) {
    // =============================== producer warp ==================================================================
    int ij = 0, ih = 0, icnt = 0;          // stage issue cursor: tile, head inside it, stages issued so far
    int pj = 0;                            // prologue cursor
    long long seq_i = 0, seq_p = 0;        // slots of 32 tiles at a time, one per lane
    int base_i = -1, base_p = -1;
    int idle = 0;
    int kpar = 0;                          // phase parity of each prologue buffer's copy barrier (bit pb)
    unsigned long long idle_t0 = 0;
    bool dead = false;
    while (!dead && (ij < nt_cta || pj < nt_cta)) {
      // ---- 1. refill a free stage -----------------------------------------------------------------------------------
      if (ij < nt_cta) {
        if ((ij & ~31) != base_i) { base_i = ij & ~31; seq_i = (base_i + lane < nt_cta) ? seq_of(base_i + lane) : 0; }
        const long long seq = __shfl_sync(0xffffffffu, seq_i, ij & 31) - seq_bias;
        if (seq + seq_bias <= 0) { ij++; ih = 0; continue; }
        const int s = icnt % nst, use = icnt / nst;
        if (use == 0 || mbar_test_wait(&sempty[s], (use - 1) & 1)) {
          const int t = bid + ij * grid;
          const int h = (t % HK) * gqa + ih;
          uint8_t* st = smraw + P.stage0 + s * P.stage_bytes;
          if (lane == 0) {
            mbar_expect_tx(&sfull[s], stage_tx);
            bulk_g2s(st, A.S + seq * A.sS + (long long)h * P.codes_b, P.codes_b, &sfull[s]);
          } else if (lane == 1) {
            bulk_g2s(st + P.codes_b, A.SC + seq * A.sSC + (long long)h * scn * 2, scn * 2, &sfull[s]);
          } else if (lane == 2) {
            bulk_g2s(st + P.codes_b + P.scales_b, A.UB + seq * A.sUB + (long long)h * M * DV * bsz, M * DV * bsz, &sfull[s]);
          }
          icnt++;
          if (++ih == gqa) { ih = 0; ij++; }
          idle = 0;
          continue;
        }
      }
      // ---- 2. the prologue of the next tile -------------------------------------------------------------------------
      if (pj < nt_cta) {
        const int pb = pj % npb, use = pj / npb;
        if (use == 0 || mbar_test_wait(&pempty[pb], (use - 1) & 1)) {
          if ((pj & ~31) != base_p) { base_p = pj & ~31; seq_p = (base_p + lane < nt_cta) ? seq_of(base_p + lane) : 0; }
          const long long seq = __shfl_sync(0xffffffffu, seq_p, pj & 31) - seq_bias;
          const int t = bid + pj * grid;
          const int b = t / HK, hk = t - b * HK, h0 = hk * gqa;
          uint8_t* pbb = smraw + P.pb0 + pb * P.pb_bytes;
          float* pf = reinterpret_cast<float*>(pbb + P.p_f);
          float *xq = pf + P.xq, *xk = pf + P.xk, *ga = pf + P.ga, *ae = pf + P.ae,
                *Dq = pf + P.Dq, *Dk = pf + P.Dk, *hd = pf + P.hd, *cq = pf + P.cq, *ck = pf + P.ck,
                *ubsf = pf + P.ubs, *misc = pf + P.misc;
          pj++;
          idle = 0;
          if (seq + seq_bias <= 0) {
            if (lane == 0) { misc[2] = 1.f; mbar_arrive(&pfull[pb]); }
            continue;
          }
          uint8_t* kbt = pbb + P.p_kb;
          const float* gbt = reinterpret_cast<const float*>(pbb + P.p_gbt);
          uint8_t* KBh = A.KB + seq * A.sKB + (long long)hk * M * DK * bsz;
          unsigned short* KBSh = A.qbuf ? reinterpret_cast<unsigned short*>(A.KBS + seq * A.sKBS) + hk * M : nullptr;
          const unsigned short* UBSseq = A.qbuf ? reinterpret_cast<const unsigned short*>(A.UBS + seq * A.sUBS) : nullptr;
          const float* GBseq = reinterpret_cast<const float*>(A.GB + seq * A.sGB);
          const float* GCseq = reinterpret_cast<const float*>(A.GCUR + seq * A.sGC);
          const int* NPseq = reinterpret_cast<const int*>(A.NPTR + seq * A.sN);
          // copies: the key tile, the value rows of the tile's heads, (KDA) the decay tile
          const uint8_t* vsrc = A.v + (long long)b * A.sv + (long long)h0 * DV * vsz;
          const uint32_t vbytes = gqa * DV * vsz;
          const bool vb = C.v_bulk != 0;
          if (lane == 0) {
            mbar_expect_tx(&kbfull[pb], M * DK * bsz + (vb ? vbytes : 0) + (VDEC ? M * DK * 4 : 0));
            bulk_g2s(kbt, KBh, M * DK * bsz, &kbfull[pb]);
          } else if (lane == 1) {
            if (vb) bulk_g2s(pbb + P.p_v, vsrc, vbytes, &kbfull[pb]);
          } else if (lane == 2) {
            if (VDEC) bulk_g2s(pbb + P.p_gbt, GBseq + (long long)h0 * M * DK, M * DK * 4, &kbfull[pb]);
          }
          // loads
          float qr[CW], kr[CW], gnr[CW];
#pragma unroll
          for (int j = 0; j < CW; j++) {
            qr[j] = ldf(A.q + (long long)b * A.sq, A.dt_qk, (long long)hk * DK + lane * CW + j);
            kr[j] = ldf(A.k + (long long)b * A.sk, A.dt_qk, (long long)hk * DK + lane * CW + j);
            if (VDEC) gnr[j] = GCseq[(long long)h0 * DK + lane * CW + j] +
                               ldf(A.g + (long long)b * A.sg, A.dt_g, (long long)h0 * DK + lane * CW + j);
          }
          const int n0 = NPseq[h0] & (M - 1);
          float ksv = 0.f;
          if (A.qbuf && lane < M) ksv = h2f(KBSh[lane]);
          // ---- q, k: normalise, k . q, append the key ----
          float s0 = 0.f, s1 = 0.f;
#pragma unroll
          for (int j = 0; j < CW; j++) { s0 += qr[j] * qr[j]; s1 += kr[j] * kr[j]; }
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
            xq[lane * CW + j] = qr[j];
            xk[lane * CW + j] = kr[j];
            if (VDEC) { ga[lane * CW + j] = gnr[j]; ae[lane * CW + j] = expf(gnr[j]); }
          }
          d = warp_sum(d);
          mx = warp_max(mx);
          if (lane == 0) {
            misc[0] = d; misc[1] = __int_as_float(n0); misc[2] = 0.f;
            *reinterpret_cast<long long*>(misc + 4) = seq;
          }
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
          // ---- per value head: gates and the scalars derived from them ----
          for (int hi = lane; hi < gqa; hi += 32) {
            const int h = h0 + hi;
            float g4[4] = {0.f, 0.f, 0.f, 0.f};
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
          // ---- per (value head, buffer slot): decay factor, value scale, stored log decay ----
          for (int e = lane; e < gqa * M; e += 32) {
            const int hi = e / M, i = e - hi * M, h = h0 + hi;
            const int n = NPseq[h] & (M - 1);
            float dcy = 0.f, us_i = 0.f, gb = 0.f;
            if (i < n) {
              if (!VDEC) { gb = GBseq[(long long)h * M + i]; dcy = expf(GCseq[h] - gb); } else dcy = 1.0f;
              us_i = A.qbuf ? h2f(UBSseq[h * M + i]) : 1.0f;
            }
            cq[e] = dcy;
            ubsf[e] = us_i;
            if (i == 0) hd[hi * HD_W + 7] = __int_as_float(n);
          }
          __syncwarp();
          // ---- dot products of the buffered keys with q and k: lane = (slot, quarter of d_k) ----
          if (!mbar_wait_ab(&kbfull[pb], (kpar >> pb) & 1, abortf)) { dead = true; break; }
          kpar ^= 1 << pb;
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
                const float4 q4 = *reinterpret_cast<const float4*>(xq + k);
                const float4 k4 = *reinterpret_cast<const float4*>(xk + k);
                if (VDEC) {
                  const float4 g4v = *reinterpret_cast<const float4*>(ga + k);
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
          __syncwarp();
          for (int e = lane; e < gqa * M; e += 32) {
            const int i = e & (M - 1);
            const float dcy = cq[e];
            cq[e] = dcy * Dq[i];
            ck[e] = dcy * Dk[i];
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&pfull[pb]);
          continue;
        }
      }
      // ---- nothing could be done: both rings are full ----
      if (idle++ == 0) idle_t0 = global_ns();
      if (idle > 16) __nanosleep(64);
      if ((idle & 63) == 63) {
        if (*abortf) dead = true;
        else if (global_ns() - idle_t0 > WAIT_LIMIT_NS) { *abortf = 1; dead = true; }
      }
    }
    if (dead || *abortf) {
      // leave no copy in flight: wait (bounded) for the latest copy of every stage and prologue buffer
      for (int s = 0; s < nst && s < icnt; s++) {
        const int last = (icnt - 1 - s) / nst;
        for (int it = 0; it < (1 << 16) && !mbar_test_wait(&sfull[s], last & 1); it++) __nanosleep(200);
      }
      for (int s = 0; s < npb; s++) {                       // kpar: parity of the next phase; the latest armed one is the other
        for (int it = 0; it < (1 << 16) && !mbar_test_wait(&kbfull[s], ((kpar >> s) & 1) ^ 1); it++) __nanosleep(200);
        for (int it = 0; it < (1 << 14) && !mbar_test_wait(&kbfull[s], (kpar >> s) & 1); it++) __nanosleep(200);
      }
    }
  } else {
    // =============================== consumer warps =================================================================
    float* cf = reinterpret_cast<float*>(smraw + P.c0);
    const int c = lane & (LPR - 1), rl = lane / LPR;
    const int gl = AXK ? (c * 16) / G : 0;
    const int RW = DV / NW;
    const int npass = RW / RPP;
    int ccnt = 0;                                  // stages consumed so far
    int csn = 0;                                   // consumer barrier phases so far
    int ubuf = 0;                                  // which copy of us / red this tile writes
    int kpar = 0;                                  // phase parity of each prologue buffer's copy barrier (bit pb)
    auto csync = [&]() -> bool {                   // barrier among the consumer warps; false: the CTA is aborting
      __syncwarp();
      if (lane == 0) mbar_arrive(cbar);
      const bool ok = mbar_wait_ab(cbar, csn & 1, abortf);
      csn++;
      return ok;
    };
    for (int j = 0; j < nt_cta; j++) {
      const int pb = j % npb, puse = j / npb;
      const int t = bid + j * grid;
      const int b = t / HK, hk = t - b * HK, h0 = hk * gqa;
      uint8_t* pbb = smraw + P.pb0 + pb * P.pb_bytes;
      const float* pf = reinterpret_cast<const float*>(pbb + P.p_f);
      const float *xq = pf + P.xq, *xk = pf + P.xk, *ga = pf + P.ga, *ae = pf + P.ae, *hd = pf + P.hd,
                  *cqf = pf + P.cq, *ckf = pf + P.ck, *ubsf = pf + P.ubs, *misc = pf + P.misc;
      float* us = cf + P.us + ubuf * P.us_n;
      float* red = cf + P.red + ubuf * P.red_n;
      if (!mbar_wait_ab(&pfull[pb], puse & 1, abortf)) goto consumer_exit;
      if (misc[2] != 0.f) {                                      // padding row: zero its outputs
        uint8_t* orow = A.out + (long long)b * A.so + (long long)h0 * DV * osz;
        for (int v = tid; v < gqa * DV; v += NT) stf(orow, A.dt_out, v, 0.0f);
        __syncwarp();
        if (lane == 0) mbar_arrive(&pempty[pb]);
        continue;
      }
      mbar_test_wait(&kbfull[pb], (kpar >> pb) & 1);             // complete since before the producer's arrival; orders the copies
      kpar ^= 1 << pb;
      const long long seq = *reinterpret_cast<const long long*>(misc + 4);
      const float kq = misc[0];
      uint8_t* Sseq = A.S + seq * A.sS;
      unsigned short* SCseq = reinterpret_cast<unsigned short*>(A.SC + seq * A.sSC);
      uint8_t* UBseq = A.UB + seq * A.sUB;
      unsigned short* UBSseq = A.qbuf ? reinterpret_cast<unsigned short*>(A.UBS + seq * A.sUBS) : nullptr;
      float* GBseq = reinterpret_cast<float*>(A.GB + seq * A.sGB);
      float* GCseq = reinterpret_cast<float*>(A.GCUR + seq * A.sGC);
      int* NPseq = reinterpret_cast<int*>(A.NPTR + seq * A.sN);
      const uint8_t* vrow = C.v_bulk ? pbb + P.p_v : A.v + (long long)b * A.sv + (long long)h0 * DV * vsz;

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
      for (int hi = 0; hi < gqa; hi++, ccnt++) {
        const int h = h0 + hi;
        const int s = ccnt % nst;
        uint8_t* st = smraw + P.stage0 + s * P.stage_bytes;
        const uint8_t* codes = st;
        const unsigned short* scs = reinterpret_cast<const unsigned short*>(st + P.codes_b);
        const uint8_t* ubt = st + P.codes_b + P.scales_b;
        uint8_t* orow = A.out + (long long)b * A.so + (long long)h * DV * osz;
        const float* hdv = hd + hi * HD_W;
        const float beta = hdv[1], alpha = hdv[3], a = hdv[4], gnew = hdv[5], Dv = hdv[6];
        const int n = __float_as_int(hdv[7]);
        const float* cqh = cqf + hi * M;
        const float* ckh = ckf + hi * M;
        const float* usf = ubsf + hi * M;
        float* usb = us + hi * DV;

        if (!mbar_wait_ab(&sfull[s], (ccnt / nst) & 1, abortf)) goto consumer_exit;

        // ---- state pass ----
        int cur_gv = -1;
        float umax = 0.f;
        for (int p0 = 0; p0 < npass; p0 += LPR) {
          const bool own = p0 + c < npass;
          const int orow_i = warp * RW + (own ? p0 + c : 0) * RPP + rl;
          const float vt = ldf(vrow, A.dt_v, hi * DV + orow_i);
          float tq, tk;
          pass_rows<BITS, AXK, TWO, LPR>(codes, scs, vq, vk, p0, npass, warp * RW, G, NG, gl, c, rl, cur_gv,
                                         [&](int gv) { load_slice(scs + gv * DK); }, tq, tk);
          if (own) {
            const int row = orow_i;
            if (!VDEC) { tq = alpha * tq; tk = alpha * tk; }
            for (int i = 0; i < n; i++) {
              float ub;
              if (A.qbuf) ub = static_cast<float>(reinterpret_cast<const int8_t*>(ubt)[i * DV + row]) * usf[i];
              else ub = bf2f(reinterpret_cast<const unsigned short*>(ubt)[i * DV + row]);
              tq = fmaf(ub, cqh[i], tq);
              if (TWO) tk = fmaf(ub, ckh[i], tk);
            }
            float u, o;
            if (KIND == K_GDN) {
              u = beta * fmaf(-a, tk, vt);
              o = fmaf(kq, u, a * tq);
            } else if (KIND == K_KDA) {
              u = beta * (vt - tk);
              o = fmaf(kq, u, tq);
            } else {
              u = beta * vt;
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
        __syncwarp();
        if (lane == 0) mbar_arrive(&sempty[s]);                  // this warp is done with the stage
      }
      {
        // ---- append the values of all heads at their slot n: warp w takes heads w, w + 4, ... ----
        if (!csync()) goto consumer_exit;
        for (int hi = warp; hi < gqa; hi += NW) {
          const int h = h0 + hi;
          const int n = __float_as_int(hd[hi * HD_W + 7]);
          const float gnew = hd[hi * HD_W + 5];
          const float* usb = us + hi * DV;
          uint8_t* UBh = UBseq + (long long)h * M * DV * bsz;
          if (A.qbuf) {
            const float usc = fp16_scale(fmaxf(fmaxf(red[hi * NW], red[hi * NW + 1]), fmaxf(red[hi * NW + 2], red[hi * NW + 3])), 127.0f);
            const bool fast_ok = usc >= FP16_MIN_NORMAL;
            const float r = __fdiv_rn(1.0f, usc);
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
            for (int tt = lane; tt < DK; tt += 32) {
              GBh[(long long)n * DK + tt] = ga[tt];
              GCh[tt] = ga[tt];
            }
          } else if (lane == 0) {
            GBseq[(long long)h * M + n] = gnew;
            GCseq[h] = gnew;
          }
          if (lane == 0) NPseq[h] = n + 1;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&pempty[pb]);                   // this warp is done with the prologue buffer
      ubuf ^= 1;
    }
  consumer_exit:;
  }
  __syncthreads();
  if (tid == 0 && *abortf) atomicAdd(&A.status[0], 1);
}

}  // namespace sqb
