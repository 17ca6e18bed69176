// The fold as its own launch, right after the step kernel of the same call.
//
// On a slot's m-th token the staged step kernel only appends: it leaves the head's counter at m
// (a value that never survives the call), the running log decay in GCUR and the buffer complete.  This kernel then
// rewrites the stored state of exactly those heads,
//     S = exp(gcur) S_0 + sum_i (exp(gcur - G_i) u_i) k_i^T      (KDA: the decay ratio sits on the key, per channel)
// re-rounds it, and resets the counter and GCUR to 0 -- the same arithmetic, on the same rounded buffer entries, as
// the fused fold of the reference (kernels/_fused_triton.py:279-394), so the bytes after the call are identical.
//
// It is persistent: a CTA takes every gridDim.x-th of the (batch row, value head) pairs, its threads test 128 pairs
// at a time (slot index -> counter, two dependent loads, all in flight together), and the heads found are folded one
// after the other with the next head's codes, scales and buffer tiles already on their way (two stages of bulk
// async copies).  A launch in which no head is due costs one such scan.
#pragma once
#include "step_tma.cuh"
#include "fold_mma.cuh"

namespace sqb {

struct SmemF {
  int bars, list, stage0, stage_bytes, codes_b, scales_b, ub_b, kb_b, gb_b, gc_b, o_sc, o_ub, o_kb, o_gb, o_gc;
  int f0, R, L, ae, ksf, cmax, rdk, lm, total;
};
__host__ __device__ inline SmemF smemf_plan(bool vdec, int bits, int axk, int group, int DK, int DV, int M, int qbuf) {
  SmemF s;
  const int bsz = qbuf ? 1 : 2;
  const int lpr = DK / 16;
  s.rdk = lpr * 20;
  s.lm = fold_lm(M);
  s.codes_b = DV * DK * bits / 8;
  s.scales_b = al16i((axk ? DV * (DK / group) : (DV / group) * DK) * 2);
  s.ub_b = al16i(M * DV * bsz);
  s.kb_b = al16i(M * DK * bsz);
  s.gb_b = vdec ? M * DK * 4 : 0;
  s.gc_b = vdec ? DK * 4 : 0;
  s.o_sc = s.codes_b + 128;                 // (room for the padded-piece layout of the tensor-pipe fold)
  s.o_ub = s.o_sc + s.scales_b;
  s.o_kb = s.o_ub + s.ub_b;
  s.o_gb = s.o_kb + s.kb_b;
  s.o_gc = s.o_gb + s.gb_b;
  s.stage_bytes = s.o_gc + s.gc_b;
  int o = 0;
  s.bars = o; o += 64;
  s.list = o; o += 128 * 4 + 64;            // pairs found in one scan round (+ counters)
  o = (o + 127) & ~127;
  s.stage0 = o; o += 2 * s.stage_bytes;
  s.f0 = o;
  int f = 0;
  s.R = f; f += M * s.rdk;
  s.L = f; f += DV * s.lm;
  s.ae = f; f += vdec ? DK : 32;            // KDA: exp(gcur) per key channel; else: the slots' decay factors
  s.ksf = f; f += 64;                       // buffer scales of the slots: keys, then values
  s.cmax = f; f += (axk ? 0 : 3 * NW * s.rdk);      // axis v: column maxima, then scales and their reciprocals (padded)
  s.total = s.f0 + ((f + 3) & ~3) * 4;
  return s;
}

struct FoldArgs {
  uint8_t *S, *SC, *KB, *KBS, *UB, *UBS, *GB, *GCUR, *NPTR;
  long long sS, sSC, sKB, sKBS, sUB, sUBS, sGB, sGC, sN;
  const int* idx;
  int group, qbuf, M, HV, HK, DV, rows;
  int* status;
  int tens;                  // the fold on the tensor pipe (fold_mma.cuh): Gated DeltaNet / Mamba2 heads of 128 x 128, buffer of 8
  float* out;                // read mode: fp32 [rows, HV, d_v, d_k], the state advanced across its pending buffer
};

template <bool VDEC, int BITS, bool AXK, int LPR>
__global__ void __launch_bounds__(NT, 4) fold_kernel(const __grid_constant__ FoldArgs A, const __grid_constant__ SmemF P) {
  constexpr int DK = LPR * 16;
  constexpr bool TENS_OK = !VDEC && AXK && LPR == 8;       // instantiations that carry the tensor-pipe fold
  extern __shared__ __align__(128) uint8_t smraw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int DV = A.DV, M = A.M, HV = A.HV, G = A.group;
  const int gqa = HV / A.HK;
  const int bsz = A.qbuf ? 1 : 2;
  const int NG = AXK ? DK / G : 1;
  const int scn = AXK ? DV * NG : (DV / G) * DK;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smraw + P.bars);
  int* list = reinterpret_cast<int*>(smraw + P.list);
  int* lcount = list + 128;
  float* fsm = reinterpret_cast<float*>(smraw + P.f0);
  float *R = fsm + P.R, *L = fsm + P.L, *ae = fsm + P.ae, *cmax = fsm + P.cmax;
  float* dec = ae;
  float *ksf = fsm + P.ksf, *usf = ksf + 32;
  const int RDK = P.rdk, LM = P.lm;
  const uint32_t stage_tx = P.codes_b + scn * 2 + M * DV * bsz + M * DK * bsz + (VDEC ? M * DK * 4 + DK * 4 : 0);

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // pair q of this CTA is pair q * gridDim.x + blockIdx.x of the launch: the heads of one batch row go to as many
  // CTAs, so that a launch in which only some rows are due (slots at different buffer positions) is still balanced
  const long long pairs = static_cast<long long>(A.rows) * HV;
  const long long per_cta = (pairs + gridDim.x - 1) / gridDim.x;
  uint32_t phases = 0;                         // bit s: parity of the next phase of stage s's barrier
  bool failed = false;

  auto slot_of = [&](int pair) -> long long {  // pair = index relative to nothing: absolute (row, head)
    const int b = pair / HV;
    return A.idx != nullptr ? static_cast<long long>(A.idx[b]) : static_cast<long long>(b);
  };
  auto issue = [&](int s, int pair) {          // one thread: the copies of one head into stage s
    const int b = pair / HV, h = pair - b * HV, hk = h / gqa;
    const long long seq = slot_of(pair);
    uint8_t* st = smraw + P.stage0 + s * P.stage_bytes;
    mbar_expect_tx(&bars[s], stage_tx);
    if (TENS_OK && A.tens) {                   // eight pieces of 16 rows, 16 bytes apart (mma_pass.cuh)
      constexpr int PB = 16 * (DK * BITS / 8);
      for (int l = 0; l < 8; l++) bulk_g2s(st + l * (PB + 16), A.S + seq * A.sS + (long long)h * P.codes_b + l * PB, PB, &bars[s]);
    } else {
      bulk_g2s(st, A.S + seq * A.sS + (long long)h * P.codes_b, P.codes_b, &bars[s]);
    }
    bulk_g2s(st + P.o_sc, A.SC + seq * A.sSC + (long long)h * scn * 2, scn * 2, &bars[s]);
    bulk_g2s(st + P.o_ub, A.UB + seq * A.sUB + (long long)h * M * DV * bsz, M * DV * bsz, &bars[s]);
    bulk_g2s(st + P.o_kb, A.KB + seq * A.sKB + (long long)hk * M * DK * bsz, M * DK * bsz, &bars[s]);
    if (VDEC) {
      bulk_g2s(st + P.o_gb, A.GB + seq * A.sGB + (long long)h * M * DK * 4, M * DK * 4, &bars[s]);
      bulk_g2s(st + P.o_gc, A.GCUR + seq * A.sGC + (long long)h * DK * 4, DK * 4, &bars[s]);
    }
  };

  for (long long base = 0; base < per_cta && !failed; base += NT) {
    // ---- scan 128 pairs: which heads have a full buffer? ----
    __syncthreads();                           // the list of the previous round is no longer read
    if (tid == 0) *lcount = 0;
    __syncthreads();
    const long long pr = (base + tid) * gridDim.x + blockIdx.x;
    bool due = false;
    if (base + tid < per_cta && pr < pairs) {
      const int b = static_cast<int>(pr / HV), h = static_cast<int>(pr - (long long)b * HV);
      long long seq = b;
      bool live = true;
      if (A.idx != nullptr) { seq = A.idx[b]; live = seq > 0; }
      if (live) due = A.out != nullptr || reinterpret_cast<const int*>(A.NPTR + seq * A.sN)[h] == M;
    }
    const unsigned bal = __ballot_sync(0xffffffffu, due);
    int wbase = 0;
    if (lane == 0 && bal) wbase = atomicAdd(lcount, __popc(bal));
    wbase = __shfl_sync(0xffffffffu, wbase, 0);
    if (due) list[wbase + __popc(bal & ((1u << lane) - 1))] = static_cast<int>(pr);
    __syncthreads();
    const int cnt = *lcount;
    if (cnt == 0) continue;
    // ---- fold the heads found, two stages deep ----
    if (tid == 0) {
      issue(0, list[0]);
      if (cnt > 1) issue(1, list[1]);
    }
    for (int e = 0; e < cnt; e++) {
      const int s = e & 1;
      const int pair = list[e];
      const int b = pair / HV, h = pair - b * HV, hk = h / gqa;
      const long long seq = slot_of(pair);
      uint8_t* st = smraw + P.stage0 + s * P.stage_bytes;
      const uint8_t* codes = st;
      const unsigned short* scs = reinterpret_cast<const unsigned short*>(st + P.o_sc);
      const uint8_t* ubt = st + P.o_ub;
      const uint8_t* kbt = st + P.o_kb;
      const float* gbt = reinterpret_cast<const float*>(st + P.o_gb);
      const float* gct = reinterpret_cast<const float*>(st + P.o_gc);
      float* GBh = reinterpret_cast<float*>(A.GB + seq * A.sGB) + (long long)h * M * (VDEC ? DK : 1);
      float* GCh = reinterpret_cast<float*>(A.GCUR + seq * A.sGC) + (long long)h * (VDEC ? DK : 1);
      const unsigned short* KBSh = A.qbuf ? reinterpret_cast<const unsigned short*>(A.KBS + seq * A.sKBS) + hk * M : nullptr;
      const unsigned short* UBSh = A.qbuf ? reinterpret_cast<const unsigned short*>(A.UBS + seq * A.sUBS) + h * M : nullptr;
      // small per-head scalars straight from global memory while the copies land
      float gnew = 0.f;
      if (!VDEC) gnew = *GCh;
      const bool reading = A.out != nullptr;
      const int nlive = reading ? (reinterpret_cast<const int*>(A.NPTR + seq * A.sN)[h] & (M - 1)) : M;   // buffer entries in use
      const bool landed = mbar_wait(&bars[s], (phases >> s) & 1);
      phases ^= 1u << s;
      if (!__syncthreads_and(landed)) {          // uniform: every thread leaves, or none
        if (e + 1 < cnt) mbar_wait(&bars[s ^ 1], (phases >> (s ^ 1)) & 1);   // leave no copy in flight
        failed = true;
        break;
      }
      if constexpr (TENS_OK) {
        if (A.tens) {
          // ---- the fold on the tensor pipe, from the stage as padded pieces, written back by bulk copies ----
          constexpr int UPG = BITS == 8 ? 1 : 2, ROWB = DK * BITS / 8, PITCH = 16 * ROWB + 16;
          float* tab = R;                              // dec_i, value scales, alpha (R and L are free in this mode)
          uint32_t* KBf = reinterpret_cast<uint32_t*>(R + 32);
          float* udq = L;
          if (reading) {
            // the state advanced across the nlive <= 7 pending slots; dead slots (any bytes) count as zero
            if (tid < 8) {
              const bool lv = tid < nlive;
              tab[tid] = lv ? expf(gnew - GBh[tid]) : 0.f;
              tab[8 + tid] = lv ? h2f(UBSh[tid]) : 0.f;
              ksf[tid] = lv ? h2f(KBSh[tid]) : 0.f;
              if (tid == 0) tab[16] = expf(gnew);
            }
            udq[tid] = 0.f;
            build_key_frags<BITS>(KBf, reinterpret_cast<const int8_t*>(kbt), reinterpret_cast<const int8_t*>(kbt) + 7 * DK, tid);
            __syncthreads();
            fold_stage_mma<BITS, UPG, 128, false, true>(smem_u32(st), reinterpret_cast<unsigned short*>(st + P.o_sc),
                                                        reinterpret_cast<const int8_t*>(ubt), udq, tab, ksf, KBf, warp, lane, nullptr,
                                                        A.out + (long long)pair * DV * DK);
            __syncthreads();                           // the stage, the tables and the fragments are free
            if (tid == 0 && e + 2 < cnt) {
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              issue(s, list[e + 2]);
            }
            continue;
          }
          if (tid < 8) {
            tab[tid] = tid == 7 ? 1.0f : expf(gnew - GBh[tid]);
            tab[8 + tid] = h2f(UBSh[tid]);
            ksf[tid] = h2f(KBSh[tid]);
            if (tid == 0) tab[16] = expf(gnew);
          }
          udq[tid] = static_cast<float>(reinterpret_cast<const int8_t*>(ubt)[7 * DV + tid]) * h2f(UBSh[7]);   // d_v = 128 = NT
          build_key_frags<BITS>(KBf, reinterpret_cast<const int8_t*>(kbt), reinterpret_cast<const int8_t*>(kbt) + 7 * DK, tid);
          __syncthreads();
          fold_stage_mma<BITS, UPG, 128, false>(smem_u32(st), reinterpret_cast<unsigned short*>(st + P.o_sc),
                                                reinterpret_cast<const int8_t*>(ubt), udq, tab, ksf, KBf, warp, lane);
          if (tid == 0) { *GCh = 0.f; reinterpret_cast<int*>(A.NPTR + seq * A.sN)[h] = 0; }
          __syncthreads();
          if (warp == 0) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            uint8_t* Sg = A.S + seq * A.sS + (long long)h * P.codes_b;
            if (lane < 8) bulk_s2g(Sg + lane * 16 * ROWB, st + lane * PITCH, 16 * ROWB);
            else if (lane == 8) bulk_s2g(A.SC + seq * A.sSC + (long long)h * scn * 2, st + P.o_sc, scn * 2);
            bulk_commit();
            bulk_wait_read();                          // the stage may be refilled, and the CTA may leave
            __syncwarp();
            if (lane == 0 && e + 2 < cnt) issue(s, list[e + 2]);
          }
          continue;
        }
      }
      if (tid < M) {
        if (!VDEC) dec[tid] = tid >= nlive ? 0.f : (!reading && tid == M - 1 ? 1.0f : expf(gnew - GBh[tid]));
        ksf[tid] = A.qbuf ? h2f(KBSh[tid]) : 1.0f;
        usf[tid] = A.qbuf ? h2f(UBSh[tid]) : 1.0f;
      }
      __syncthreads();
      // R: the keys of all slots (KDA: times their decay ratio); L: the buffered values times their decay
      for (int x = tid; x < M * DK; x += NT) {
        const int i = x / DK, k = x - i * DK;
        float kv;
        if (A.qbuf) kv = static_cast<float>(reinterpret_cast<const int8_t*>(kbt)[x]) * ksf[i];
        else kv = bf2f(reinterpret_cast<const unsigned short*>(kbt)[x]);
        if (VDEC && (reading || i != M - 1)) kv = i < nlive ? kv * expf(gct[k] - gbt[x]) : 0.f;
        if (i >= nlive) kv = 0.f;
        R[i * RDK + (k / 16) * 20 + (k % 16)] = kv;
      }
      if (VDEC) {
        for (int k = tid; k < DK; k += NT) ae[k] = expf(gct[k]);
      }
      if ((M & 3) == 0) {
        // four slots of a row at a time: one 128-bit store each, rows over consecutive threads (conflict-free)
        for (int x = tid; x < (M / 4) * DV; x += NT) {
          const int i0 = (x / DV) * 4, v = x - (x / DV) * DV;
          float ub4[4];
#pragma unroll
          for (int t = 0; t < 4; t++) {
            const int i = i0 + t;
            float ub;
            if (A.qbuf) ub = static_cast<float>(reinterpret_cast<const int8_t*>(ubt)[i * DV + v]) * usf[i];
            else ub = bf2f(reinterpret_cast<const unsigned short*>(ubt)[i * DV + v]);
            if (!VDEC && (reading || i != M - 1)) ub = dec[i] * ub;
            if (i >= nlive) ub = 0.f;
            ub4[t] = ub;
          }
          *reinterpret_cast<float4*>(L + v * LM + i0) = make_float4(ub4[0], ub4[1], ub4[2], ub4[3]);
        }
      } else {
        for (int x = tid; x < M * DV; x += NT) {
          const int i = x / DV, v = x - i * DV;
          float ub;
          if (A.qbuf) ub = static_cast<float>(reinterpret_cast<const int8_t*>(ubt)[x]) * usf[i];
          else ub = bf2f(reinterpret_cast<const unsigned short*>(ubt)[x]);
          if (!VDEC && (reading || i != M - 1)) ub = dec[i] * ub;
          if (i >= nlive) ub = 0.f;
          L[v * LM + i] = ub;
        }
      }
      __syncthreads();
      const float alphan = VDEC ? 1.0f : expf(gnew);
      fold_rows<BITS, AXK, LPR, VDEC>(codes, scs, R, L, ae, alphan, DV, G, M, cmax,
                                      A.S + seq * A.sS + (long long)h * P.codes_b,
                                      reinterpret_cast<unsigned short*>(A.SC + seq * A.sSC) + (long long)h * scn, warp,
                                      lane, tid, [] { __syncthreads(); return true; },
                                      reading ? A.out + (long long)pair * DV * DK : nullptr);
      if (!reading) {
        // counters back to 0: the buffer is empty again
        if (VDEC) {
          for (int k = tid; k < DK; k += NT) GCh[k] = 0.f;
        } else if (tid == 0) {
          *GCh = 0.f;
        }
        if (tid == 0) reinterpret_cast<int*>(A.NPTR + seq * A.sN)[h] = 0;
      }
      __syncthreads();                         // the stage, R and L are free
      if (tid == 0 && e + 2 < cnt) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue(s, list[e + 2]);
      }
    }
  }
  if (failed && tid == 0) atomicAdd(&A.status[0], 1);
}

}  // namespace sqb
