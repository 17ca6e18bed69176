// The fused packed-state decode step with the state pass on the tensor pipe (mma_pass.cuh): 4- and 8-bit states scaled
// along k in groups of 32, 64 or 128 (and 4- / 8-bit states scaled along v in groups of 32 rows), head dim d_k = 128,
// d_v 64 or 128, int8 decode buffer.
//
// One CTA (128 threads) per (batch row, KEY head, part of its value heads) walks its value heads in STAGES of 128
// state rows (one head of d_v 128, two heads of d_v 64).  A stage -- codes as 8 padded pieces, scales, buffered
// values -- arrives by bulk async copies on one mbarrier; the copies of the first stages and of the key tile are
// issued by the lanes of warps 2 and 1 in the CTA's first instructions.  Per stage each warp takes a tile of 32 rows
// through the tensor-core pass and finishes one row per lane (buffer term, u, o).  A CTA with exactly two stages takes
// both at once on a token that does not fold: two independent chains per warp instead of one after the other.
//
// MODE 0: every token is stepped and appended (after the last stage); on a slot's m-th token the head's counter is
//         left at m for the fold launch that follows (fold_kernel.cuh).
// MODE 3: the same, and a slot on its m-th token is folded right here from the staged tile (the stored state is read
//         once per token, fold or not): per stage the append and the fold of the stage's heads follow the read-out
//         (on the tensor pipe, fold_mma.cuh, where the format allows; else in fp32, fold_rows.cuh).
//         Nothing a CTA fetches depends on the slot's counter, so every copy and every scalar load leaves in the
//         CTA's first instructions.
//
// Prologue by role: warp 0 normalises q and k, builds the fixed-point B fragments and (GDN, Mamba2) takes the
// buffered keys' dot products on the tensor pipe; warp 1 the gates; warp 2 issues the copies and computes decay
// factors and value scales of every (head, slot); warp 3 rounds the key that goes into the buffer (KDA: prepares the
// normalised vectors and log decays for the buffered keys' products, which all four warps take in fp32 after the
// block barrier, their decay ratios being per channel; warp 0 rounds the key).
//
// Arithmetic is that of delta_step.cuh (same rounding of scales, payloads and buffer entries); only the order of the
// reductions differs, and the read-out vectors pass through 30-bit fixed point (mma_pass.cuh).
#pragma once
#include "step_tma.cuh"
#include "mma_pass.cuh"
#include "fold_mma.cuh"

namespace sqb {

#ifdef SQB_TRACE
// debug builds only: per-warp cycle stamps of sampled CTAs (never compiled into the shipped library)
__device__ long long g_mma_trace[64 * 4 * 16];
#define SQB_STAMP(k) do { if ((blockIdx.x & 63) == 5 && lane == 0) g_mma_trace[((blockIdx.x >> 6) * 4 + warp) * 16 + (k)] = clock64() - t_start; } while (0)
#else
#define SQB_STAMP(k) do { } while (0)
#endif

struct SmemM {
  int bars, stage0, stage_bytes, sc_off, ub_off, kb, gbt, bf, bfv, kbf, kcur, f0, total;
  int hd, dcu, gbs, dqk, ksv, us, red, misc, ga, ae, wq, wk, wg, tab, R, L, fdec, ksf;     // float offsets from f0
};
// The fold of the m-th token runs on the tensor pipe (fold_mma.cuh) for decays per head, a buffer of 8 and one scale
// group per 32-byte span of a row; otherwise in fp32 (fold_rows.cuh), which needs the R / L tiles.
// (axv: 4-bit codes scaled along v in groups of 32 rows, fold_stage_mma_v4.)
__host__ __device__ inline bool fold_on_tensor_pipe(int kind, int bits, int upg, int M, bool axv = false) {
  if (axv) return kind != K_KDA && M == 8 && (bits == 4 || bits == 8);
  return M == 8 && ((bits == 8 && upg == 1) || (bits == 4 && upg == 2));
}
__host__ __device__ inline SmemM smemm_plan(int kind, int bits, int upg, int DV, int M, int nst, int gqa, bool fold,
                                            bool axv = false) {
  const bool simt = fold && !fold_on_tensor_pipe(kind, bits, upg, M, axv), tens = fold && !simt;
  SmemM s;
  const int rowb = 128 * bits / 8, ng = 4 / upg;
  const bool v8 = axv && bits == 8;                  // 8-bit codes scaled along v: 32 pieces of 4 rows (mma_pass.cuh)
  const int pitch = v8 ? V8_PITCH : 16 * rowb + 16;
  s.sc_off = (v8 ? 32 : 8) * pitch;
  s.ub_off = s.sc_off + 128 * ng * 2;
  s.stage_bytes = s.ub_off + al16i(M * 128);
  int o = 0;
  s.bars = o; o += 128;
  s.stage0 = o; o += nst * s.stage_bytes;
  s.kb = o; o += al16i(M * 128);
  s.gbt = o; o += (kind == K_KDA ? M * 128 * 4 : 0);
  s.bf = o; o += (bits == 4 && kind != K_KDA) ? 2048 : 1024;   // B fragments: the state's layout (+ the byte layout for the key tile)
  s.bfv = o; o += axv ? 4096 : 0;    // states scaled along v: every warp's own B fragments
  s.kbf = o; o += tens ? (kind == K_KDA ? 3 * 2048 : 2048) : 0;   // the fold's key fragments (KDA: three bf16 planes)
  s.kcur = o; o += tens ? 128 : 0;   // the codes of the key appended by this token
  s.f0 = o;
  int f = 0;
  s.hd = f; f += gqa * HD_W;
  s.dcu = f; f += (2 * gqa * M + 3) & ~3;
  s.gbs = f; f += fold ? (gqa * M + 3) & ~3 : 0;       // cumulative log decays of the buffered tokens, as stored
  s.dqk = f; f += 2 * (M < 16 ? 16 : M);
  s.ksv = f; f += 32;                                  // scales of the buffered keys
  s.us = f; f += gqa * DV;
  s.red = f; f += gqa * NW;
  s.misc = f; f += 16;
  s.ga = f; f += (kind == K_KDA ? 128 : 0);
  s.ae = f; f += (kind == K_KDA ? 128 : 0);
  s.wq = f; f += (kind == K_KDA || axv ? 128 : 0);
  s.wk = f; f += (kind == K_KDA || axv ? 128 : 0);
  s.wg = f; f += (kind == K_KDA ? 128 : 0);
  f = (f + 3) & ~3;
  s.tab = f; f += tens ? 2 * 20 : 0;
  s.R = f; f += simt ? M * 160 : 0;
  s.L = f; f += simt ? DV * fold_lm(M) : 0;
  s.fdec = f; f += simt ? 32 : 0;
  s.ksf = f; f += fold ? 64 : 0;
  s.total = s.f0 + ((f + 3) & ~3) * 4;
  return s;
}

#ifndef SQB_MMA_MINB8
#define SQB_MMA_MINB8 5
#endif
#ifndef SQB_MMA_MINB4
#define SQB_MMA_MINB4 6
#endif

#ifndef SQB_MMA_MINB_FOLD
#define SQB_MMA_MINB_FOLD 4
#endif
#ifndef SQB_MMA_MINB_TFOLD
#define SQB_MMA_MINB_TFOLD 5
#endif
#ifndef SQB_MMA_MINB_AXV
#define SQB_MMA_MINB_AXV 5
#endif

// Cold paths kept out of line (they are never taken in a healthy run, and inlined at every use they were an eighth of
// the kernel's code): the zero fill of a CTA's output rows, and the exit of a CTA whose copy never completed.
// clamp(rint(x / s), +-127) by the IEEE division: the rare exact path of a buffer entry's rounding
static __device__ __noinline__ float rq_exact_cold(float x, float s) { return rq_exact(x, s, 127.0f); }
static __device__ __noinline__ void zero_out_rows(uint8_t* orow, int dt, int n) {
  for (int v = threadIdx.x; v < n; v += NT) stf(orow, dt, v, 0.0f);
}
static __device__ __noinline__ void mma_bail(uint8_t* orow, int dt, int n, uint64_t* bars, int narmed, int nst,
                                             unsigned long long wait_ns, int* status) {
  zero_out_rows(orow, dt, n);
  if (threadIdx.x == 0) {       // wait (bounded) for what may still be in flight, count it, leave
    for (int s = 0; s < narmed; s++) mbar_wait(&bars[s], 0, wait_ns);
    mbar_wait(&bars[nst], 0, wait_ns);
    atomicAdd(&status[0], 1);
  }
}

// BIO: q / k / v and the output are bf16 (what a serving engine passes): the element types of the activation loads and
// stores are then compile-time constants instead of three-way run-time dispatches at every access.
template <int KIND, int BITS, int UPG, int DV, int MODE, bool AXV = false, bool BIO = false>
__global__ void __launch_bounds__(NT, MODE == 3 ? (AXV ? SQB_MMA_MINB_AXV : (((BITS == 8 && UPG == 1) || (BITS == 4 && UPG == 2)) ? SQB_MMA_MINB_TFOLD : SQB_MMA_MINB_FOLD))
                                               : (BITS == 4 ? SQB_MMA_MINB4 : SQB_MMA_MINB8))
    step_mma_kernel(const __grid_constant__ StepArgs A, const __grid_constant__ SmemM P, const int nst) {
  constexpr int DK = 128, NG = 4 / UPG, G = 32 * UPG;
  constexpr bool V8 = AXV && BITS == 8;          // 32 pieces of 4 rows instead of 8 pieces of 16
  constexpr int ROWB = DK * BITS / 8, PROWS = V8 ? V8_PIECE_ROWS : 16, PITCH = PROWS * ROWB + 16;
  constexpr int HPS = 128 / DV;                  // heads per stage
  constexpr int CW = 4;                          // columns per lane in the prologue
  constexpr bool TWO = KIND != K_M2, VDEC = KIND == K_KDA, CANFOLD = MODE == 3;
  constexpr bool TFMT = AXV || (BITS == 8 && UPG == 1) || (BITS == 4 && UPG == 2);
  static_assert(DV == 64 || DV == 128, "a stage is 128 rows: one or two heads");
  static_assert(!AXV || (UPG == 1 && !VDEC), "scales along v: groups of 32 rows (the stage's scales are [4][128], as many bytes as UPG = 1)");

  extern __shared__ __align__(128) uint8_t smraw[];
  const int dt_qk = BIO ? static_cast<int>(DT_BF16) : A.dt_qk, dt_v = BIO ? static_cast<int>(DT_BF16) : A.dt_v,
            dt_out = BIO ? static_cast<int>(DT_BF16) : A.dt_out;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // the buffer length: 8 in the kernels whose fold is the tensor-pipe one (the host sends no other there)
  const int M = (MODE == 3 && TFMT) ? 8 : A.M;
  // grid: x = batch row, y = (key head, part of its value heads); no division on the way to the first fetch
  const int gqa = A.hpc;                          // value heads of this CTA: all heads of a key head, or a part of them
  const int gqf = A.gqa_full;                     // value heads per key head
  const int NSH = gqa / HPS;
  const int b = blockIdx.x;
  int hk = blockIdx.y, part = 0;
  if (gqa != gqf) { const int cpk = gqf / gqa; hk = blockIdx.y / cpk; part = blockIdx.y - hk * cpk; }
  const int h0 = hk * gqf + part * gqa;
  const bool first = part == 0;                   // the CTA that appends the key head's key
  const int osz = dt_size(dt_out);
  // the fold, when it comes, runs on the tensor pipe for the formats it takes (the host sends these here only with a
  // buffer of 8, cf. mma_fold_inside), else in fp32
  constexpr bool TFOLD = TFMT;

#ifdef SQB_TRACE
  const long long t_start = clock64();
#endif
  // ---- fetches --------------------------------------------------------------------------------------------------------
  // Under load a global load takes well over a microsecond here, so every fetch of the CTA leaves as early as its
  // address is known, as raw bits (a loaded register is first touched where its value is needed: the conversion of
  // a loaded word already waits for it), and a wait never sits in front of fetches that do not depend on it:
  //   warps 0 and 3 need q and k first and the slot only later: their q / k loads leave before the slot index;
  //   warps 1 and 2 issue the bulk copies, which need nothing but the slot index: they load it alone.
  const int rho = AXV ? tile_row_v<BITS>(warp, lane) : (lane >> 2) * 16 + 4 * warp + (lane & 3);     // this lane's row within a stage
  const int hh = rho / DV, rv = rho % DV;                        // head within the stage, row within the head
  Raw4 rq, rk;
  rq.v = make_uint4(0u, 0u, 0u, 0u); rk.v = rq.v; rq.vec = false; rk.vec = false;
  if (warp == 0 || warp == 3) {
    rq = ld4_raw(A.q + (long long)b * A.sq, dt_qk, (long long)hk * DK + lane * CW);
    rk = ld4_raw(A.k + (long long)b * A.sk, dt_qk, (long long)hk * DK + lane * CW);
  }
  long long seq = b;
  if (A.idx != nullptr) {
    seq = A.idx[b];
    if (seq <= 0) {
      zero_out_rows(A.out + (long long)b * A.so + (long long)h0 * DV * osz, dt_out, gqa * DV);
      return;
    }
  }
  int* NPseq = reinterpret_cast<int*>(A.NPTR + seq * A.sN);
  SQB_STAMP(0);

  uint64_t* bars = reinterpret_cast<uint64_t*>(smraw + P.bars);
  uint8_t* kbt = smraw + P.kb;
  uint32_t* Bfw = reinterpret_cast<uint32_t*>(smraw + P.bf);
  float* fsm = reinterpret_cast<float*>(smraw + P.f0);
  float *hd = fsm + P.hd, *us = fsm + P.us, *red = fsm + P.red, *misc = fsm + P.misc, *ga = fsm + P.ga, *ae = fsm + P.ae,
        *wq = fsm + P.wq, *wk = fsm + P.wk, *wg = fsm + P.wg, *ksv = fsm + P.ksv;
  float2* dcu = reinterpret_cast<float2*>(fsm + P.dcu);    // (decay factor, value scale) of every (head, slot)
  float2* dqk = reinterpret_cast<float2*>(fsm + P.dqk);    // dot products of the buffered keys with q and k
  const float* gbt = reinterpret_cast<const float*>(smraw + P.gbt);
  [[maybe_unused]] float* Rf = fsm + P.R;

  uint8_t* Sseq = A.S + seq * A.sS;
  uint8_t* SCseq = A.SC + seq * A.sSC;
  uint8_t* KBh = A.KB + seq * A.sKB + (long long)hk * M * DK;
  uint8_t* UBseq = A.UB + seq * A.sUB;
  unsigned short* KBSh = reinterpret_cast<unsigned short*>(A.KBS + seq * A.sKBS) + hk * M;
  unsigned short* UBSseq = reinterpret_cast<unsigned short*>(A.UBS + seq * A.sUBS);
  float* GBseq = reinterpret_cast<float*>(A.GB + seq * A.sGB);
  float* GCseq = reinterpret_cast<float*>(A.GCUR + seq * A.sGC);
  const uint32_t stage_tx = 128 * ROWB + 128 * NG * 2 + M * 128 + A.test_extra_tx;
  // KDA: this token's log decays and the slot's running ones, the lane's four channels (warps 0 and 3), as raw bits
  Raw4 rgk;
  rgk.v = make_uint4(0u, 0u, 0u, 0u); rgk.vec = false;
  float4 gck = make_float4(0.f, 0.f, 0.f, 0.f);
  if (VDEC && (warp == 0 || warp == 3)) {
    rgk = ld4_raw(A.g + (long long)b * A.sg, A.dt_g, (long long)h0 * DK + lane * CW);
    gck = *reinterpret_cast<const float4*>(GCseq + (long long)h0 * DK + lane * CW);
  }

  // the copies of stage `sh` into ring position s, one per lane (lanes 0..9 of the calling warp)
  auto issue_stage = [&](int s, int sh, int l) {
    uint8_t* st = smraw + P.stage0 + s * P.stage_bytes;
    const long long row0 = (long long)h0 * DV + sh * 128;
    if constexpr (V8) {                                      // 32 pieces take every lane: two of them copy twice
      bulk_g2s(st + l * PITCH, Sseq + (row0 + l * PROWS) * ROWB, PROWS * ROWB, &bars[s]);
      if (l == 0) bulk_g2s(st + P.sc_off, SCseq + row0 * NG * 2, 128 * NG * 2, &bars[s]);
      else if (l == 1) bulk_g2s(st + P.ub_off, UBseq + (long long)(h0 + sh * HPS) * M * DV, M * 128, &bars[s]);
    } else {
      if (l < 8) bulk_g2s(st + l * PITCH, Sseq + (row0 + l * 16) * ROWB, 16 * ROWB, &bars[s]);
      else if (l == 8) bulk_g2s(st + P.sc_off, SCseq + row0 * NG * 2, 128 * NG * 2, &bars[s]);
      else if (l == 9) bulk_g2s(st + P.ub_off, UBseq + (long long)(h0 + sh * HPS) * M * DV, M * 128, &bars[s]);
    }
  };
  // A stage barrier of the first fill is initialised, armed and its copies issued by ONE warp (a warp's copies leave
  // one after the other, so the stages are spread over warps 2 and 1); everybody else meets it after the block barrier.
  auto start_stage = [&](int s) {
    if (s < nst && s < NSH) {
      if (lane == 0) {
        mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(&bars[s], stage_tx);
      }
      __syncwarp();
      issue_stage(s, s, lane);
    }
  };
  // this lane's value-vector entries of the first two stages (needed after the first pass): each role issues these
  // loads once its urgent fetches are out
  uint32_t rvt[2];
  auto load_v = [&]() {
    rvt[0] = ld1_raw(A.v + (long long)b * A.sv, dt_v, (long long)(h0 + hh) * DV + rv);
    rvt[1] = ld1_raw(A.v + (long long)b * A.sv, dt_v, (long long)(h0 + (NSH > 1 ? HPS : 0) + hh) * DV + rv);
  };
  // The key tile (and KDA's decay tile) is fetched by warp 2; the warp that takes the buffered keys' dot products
  // (warp 0; KDA: warp 3) meets warp 2 at named barrier 1 (64 threads) before it waits for the tile, so that its wait
  // can never meet a barrier that is not initialised yet; by then the key scales and the slot's counter are published.
  constexpr int KEY_WARP = VDEC ? 0 : 3;
  // the key as it goes into the buffer, rounded by KEY_WARP before the block barrier and stored after it
  uint32_t kword = 0;
  float kscale = 0.f;
  float kdeq[CW] = {0.f, 0.f, 0.f, 0.f};
  auto round_key = [&](const float (&kr)[CW], float mx) {
    kscale = fp16_scale(mx, 127.0f);
#pragma unroll
    for (int j = 0; j < CW; j++) {
      const float cc = rq_exact(kr[j], kscale, 127.0f);
      kword |= (static_cast<uint32_t>(static_cast<int>(cc)) & 0xFFu) << (8 * j);
      kdeq[j] = cc * kscale;
    }
  };

  // ---- prologue, by role ----------------------------------------------------------------------------------------
  if (warp == 2) {
    // the slot's small fields first (raw), then the copies
    const int nraw = NPseq[h0];                              // the heads of a slot advance together
    unsigned short ks_raw = 0;
    if (lane < M) ks_raw = KBSh[lane];
    const int e0 = lane;                                     // first (head, slot) pair of this lane
    float gb0 = 0.f, gc0 = 0.f;
    unsigned short us0 = 0;
    if (e0 < gqa * M) {
      const int h = h0 + (e0 >> A.m_log2);
      if (!VDEC) { gb0 = GBseq[(long long)h0 * M + e0]; gc0 = GCseq[h]; }
      us0 = UBSseq[h0 * M + e0];
    }
    SQB_STAMP(1);
    start_stage(0);
    if (lane == 0) {
      mbar_init(&bars[nst], 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      mbar_expect_tx(&bars[nst], M * DK + (VDEC ? M * DK * 4 : 0));
      bulk_g2s(kbt, KBh, M * DK, &bars[nst]);
      if (VDEC) bulk_g2s(smraw + P.gbt, GBseq + (long long)h0 * M * DK, M * DK * 4, &bars[nst]);
    }
    start_stage(3);
    SQB_STAMP(2);
    load_v();
    const int n0 = nraw & (M - 1);
    if (lane < 32) ksv[lane] = lane < M ? h2f(ks_raw) : 0.f;
    if (lane == 0) misc[1] = __int_as_float(n0);
    __syncwarp();
    asm volatile("bar.arrive 1, 64;" ::: "memory");
    // per (value head, buffer slot): decay factors of the live slots and their value scales.  Loaded whether the slot is
    // live or not (dead entries may hold anything; they are selected away), so that the loads do not wait for the counter.
    for (int e = lane; e < gqa * M; e += 32) {
      const int hi = e >> A.m_log2, i = e - hi * M, h = h0 + hi;
      float gb = gb0, gc = gc0;
      unsigned short usr = us0;
      if (e != e0) {
        if (!VDEC) { gb = GBseq[(long long)h * M + i]; gc = GCseq[h]; }
        usr = UBSseq[h * M + i];
      }
      const float dcy = VDEC ? 1.0f : expf(gc - gb);
      dcu[e] = i < n0 ? make_float2(dcy, h2f(usr)) : make_float2(0.f, 0.f);
      if (CANFOLD) fsm[P.gbs + e] = gb;
    }
  } else if (warp == 1) {
    // the gate inputs of this warp's heads (one lane per value head, at most 32 per key head), then stages 1 and 2
    uint32_t rg[4] = {0u, 0u, 0u, 0u};
    float gcur = 0.f;
    const int hi = lane, h = h0 + hi;
    if (lane < gqa) {
      if (KIND == K_GDN) {
        if (A.gate) {
          rg[0] = ld1_raw(A.a + (long long)b * A.sa, A.dt_ab, h); rg[1] = ld1_raw(A.dt_bias, A.dt_dtb, h);
          rg[2] = ld1_raw(A.A_log, A.dt_alog, h);                 rg[3] = ld1_raw(A.b + (long long)b * A.sb, A.dt_ab, h);
        } else {
          rg[0] = ld1_raw(A.g + (long long)b * A.sg, A.dt_g, h);  rg[1] = ld1_raw(A.beta + (long long)b * A.sbeta, A.dt_g, h);
        }
      } else if (KIND == K_M2) {
        rg[0] = ld1_raw(A.g + (long long)b * A.sg, A.dt_g, h);
        if (A.dt_bias) rg[1] = ld1_raw(A.dt_bias, A.dt_dtb, h);
        rg[2] = ld1_raw(A.A_log, A.dt_alog, h);
        if (A.beta) rg[3] = ld1_raw(A.beta, A.dt_beta, h);
      } else {
        rg[0] = ld1_raw(A.beta + (long long)b * A.sbeta, A.dt_beta, h);
      }
      if (!VDEC) gcur = GCseq[h];
    }
    start_stage(1);
    start_stage(2);
    load_v();
    if (lane < gqa) {
      float g4[4];
      if (KIND == K_GDN) {
        if (A.gate) {
          g4[0] = cvt_raw(rg[0], A.dt_ab); g4[1] = cvt_raw(rg[1], A.dt_dtb); g4[2] = cvt_raw(rg[2], A.dt_alog); g4[3] = cvt_raw(rg[3], A.dt_ab);
        } else {
          g4[0] = cvt_raw(rg[0], A.dt_g); g4[1] = cvt_raw(rg[1], A.dt_g); g4[2] = g4[3] = 0.f;
        }
      } else if (KIND == K_M2) {
        g4[0] = cvt_raw(rg[0], A.dt_g); g4[1] = A.dt_bias ? cvt_raw(rg[1], A.dt_dtb) : 0.f;
        g4[2] = cvt_raw(rg[2], A.dt_alog); g4[3] = A.beta ? cvt_raw(rg[3], A.dt_beta) : 0.f;
      } else {
        g4[0] = cvt_raw(rg[0], A.dt_beta); g4[1] = g4[2] = g4[3] = 0.f;
      }
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
  } else if (warp == 0) {
    // q and k: normalised, in fixed point, as B fragments; GDN / Mamba2: the buffered keys' dot products on the tensor
    // pipe; KDA: the key that goes into the buffer
    load_v();
    float qr[CW], kr[CW];
    cvt4_raw(rq, dt_qk, qr);
    cvt4_raw(rk, dt_qk, kr);
    float gnr[CW] = {0.f, 0.f, 0.f, 0.f};
    float s0 = 0.f, s1 = 0.f;
    if constexpr (VDEC) {
      float gin[CW];
      cvt4_raw(rgk, A.dt_g, gin);
      gnr[0] = gck.x + gin[0]; gnr[1] = gck.y + gin[1]; gnr[2] = gck.z + gin[2]; gnr[3] = gck.w + gin[3];
    }
#pragma unroll
    for (int j = 0; j < CW; j++) {
      s0 += qr[j] * qr[j];
      s1 += kr[j] * kr[j];
    }
    SQB_STAMP(1);
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
    // maxima of non-negative floats: their bit patterns order like integers (one reduction instruction each)
    mq = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(mq)));
    if (TWO && VDEC) mk = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(mk)));
    if (TWO && !VDEC) { mx = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(mx))); mk = mx; }
    const FxScale fq = fx30_scale(mq), fk = fx30_scale(mk);
    uint32_t yq[CW], yk[CW];
#pragma unroll
    for (int j = 0; j < CW; j++) { yq[j] = fx30_digits(eq[j], fq); yk[j] = TWO ? fx30_digits(ek[j], fk) : 0u; }
    if constexpr (AXV) {                    // every warp scales the vectors by its group's column scales, per stage
      *reinterpret_cast<float4*>(wq + lane * CW) = make_float4(eq[0], eq[1], eq[2], eq[3]);
      *reinterpret_cast<float4*>(wk + lane * CW) = make_float4(ek[0], ek[1], ek[2], ek[3]);
      if (lane == 0) misc[9] = __uint_as_float(0x3C003C00u);      // the fp16 pair (1, 1): the blocks carry no scale
      if (BITS == 8) {                      // the key tile's product still takes the plain vectors, in the byte layout
        put_b_words<8>(Bfw, lane, 0, yq[0], yq[1], yq[2], yq[3]);
        put_b_words<8>(Bfw, lane, 1, yk[0], yk[1], yk[2], yk[3]);
      }
    } else {
      put_b_words<BITS>(Bfw, lane, 0, yq[0], yq[1], yq[2], yq[3]);
      put_b_words<BITS>(Bfw, lane, 1, yk[0], yk[1], yk[2], yk[3]);
    }
    if (BITS == 4 && !VDEC) {               // the key tile holds bytes: its product takes the byte layout
      put_b_words<8>(Bfw + 256, lane, 0, yq[0], yq[1], yq[2], yq[3]);
      put_b_words<8>(Bfw + 256, lane, 1, yk[0], yk[1], yk[2], yk[3]);
    }
    d = warp_sum(d);
    if (lane == 0) {
      misc[0] = d;
      misc[4] = fq.i1; misc[5] = fq.i2; misc[6] = fk.i1; misc[7] = fk.i2;
    }
    if constexpr (VDEC) {
      mx = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(mx)));
      round_key(kr, mx);
    } else {
      // the buffered keys' dot products with q and k: the key tile [M, 128] int8 is the A operand (rows = slots),
      // the B fragments are those of the state pass (the 8-bit layout: the key tile holds bytes)
      __syncwarp();
      uint32_t bf8[8];
#pragma unroll
      for (int r = 0; r < 8; r++) bf8[r] = Bfw[(BITS == 8 ? 0 : 256) + r * 32 + lane];
      SQB_STAMP(2);
      asm volatile("bar.sync 1, 64;" ::: "memory");           // warp 2 has armed the key tile's barrier
      const bool landed = mbar_wait(&bars[nst], 0, A.wait_ns);
      SQB_STAMP(15);
      if (lane == 0) misc[2] = landed ? 0.f : 1.f;          // "a copy never arrived" flag
      const float ksl = ksv[lane];                          // scale of buffered key `lane`
      const float iq1 = fq.i1, iq2 = fq.i2, ik1 = fk.i1, ik2 = fk.i2;
      for (int sb = 0; sb < M; sb += 16) {
        int acc[4] = {MAGIC_I, MAGIC_I, MAGIC_I, MAGIC_I};
        int srow = sb + ((lane >> 3) & 1) * 8 + (lane & 7);       // slot whose row this lane addresses
        srow &= (M - 1);                                          // rows past the buffer: any valid row (ignored)
        const uint32_t arow = smem_u32(kbt) + srow * DK + (lane >> 4) * 16;
#pragma unroll
        for (int j = 0; j < 4; j++) {
          uint32_t m[4];
          ldsm_x4(m, arow + 32 * j);
          mma_i8<false>(acc, m[0], m[1], m[2], m[3], bf8[2 * j], bf8[2 * j + 1]);
        }
        const int i8 = lane >> 2, t = lane & 3;
        const float k0s = __shfl_sync(0xffffffffu, ksl, (sb + i8) & 31), k1s = __shfl_sync(0xffffffffu, ksl, (sb + i8 + 8) & 31);
        float p[4] = {(__int_as_float(acc[0]) - 12582912.0f) * k0s, (__int_as_float(acc[1]) - 12582912.0f) * k0s,
                      (__int_as_float(acc[2]) - 12582912.0f) * k1s, (__int_as_float(acc[3]) - 12582912.0f) * k1s};
        float T = join_digits(p, t);          // t = 0: q, slot sb + i8; t = 1: q, slot sb + i8 + 8; t = 2, 3: k
        T = t < 2 ? (T * iq1) * iq2 : (T * ik1) * ik2;
        const int slot = sb + i8 + (t & 1) * 8;
        if (slot < M) {
          if (t < 2) dqk[slot].x = T;
          else dqk[slot].y = T;
        }
      }
    }
  } else {
    // warp 3
    load_v();
    float qr[CW], kr[CW];
    cvt4_raw(rq, dt_qk, qr);
    cvt4_raw(rk, dt_qk, kr);
    if constexpr (!VDEC) {
      // the key that goes into the buffer, rounded: its normalisation is redone here (the arithmetic of warp 0, so
      // the same bits)
      float s1 = 0.f;
#pragma unroll
      for (int j = 0; j < CW; j++) s1 += kr[j] * kr[j];
      if (KIND != K_M2) {
        s1 = warp_sum(s1);
        const float nk = __fsqrt_rn(s1 + 1e-6f);
#pragma unroll
        for (int j = 0; j < CW; j++) kr[j] = __fdiv_rn(kr[j], nk);
      }
      float mx = 0.f;
#pragma unroll
      for (int j = 0; j < CW; j++) mx = fmaxf(mx, fabsf(kr[j]));
      mx = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(mx)));
      round_key(kr, mx);
    } else {
      // KDA: dot products of the buffered keys (times their per-channel decay ratios) with q and k, in fp32, from
      // this warp's own copy of the normalised vectors (same arithmetic as warp 0, so the same bits)
      float gnr[CW], gin[CW];
      cvt4_raw(rgk, A.dt_g, gin);
      const float gcu[CW] = {gck.x, gck.y, gck.z, gck.w};
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int j = 0; j < CW; j++) {
        s0 += qr[j] * qr[j];
        s1 += kr[j] * kr[j];
        gnr[j] = gcu[j] + gin[j];
      }
      s0 = warp_sum(s0);
      s1 = warp_sum(s1);
      const float nq = __fsqrt_rn(s0 + 1e-6f), nk = __fsqrt_rn(s1 + 1e-6f);
#pragma unroll
      for (int j = 0; j < CW; j++) {
        wq[lane * CW + j] = __fdiv_rn(qr[j], nq) * A.scale;
        wk[lane * CW + j] = __fdiv_rn(kr[j], nk);
        wg[lane * CW + j] = gnr[j];
      }
      __syncwarp();
      asm volatile("bar.sync 1, 64;" ::: "memory");           // pairs with warp 2's arrival
      if (lane == 0) misc[2] = 0.f;                          // (the key tile's wait follows the block barrier)
    }
  }
  SQB_STAMP(3);
  __syncthreads();
  SQB_STAMP(4);
  // a copy that never completed: wait (bounded) for what may still be in flight, count it, leave
  auto bail = [&]() {
    mma_bail(A.out + (long long)b * A.so + (long long)h0 * DV * osz, dt_out, gqa * DV, bars, min(nst, NSH), nst, A.wait_ns,
             A.status);
  };
  if (misc[2] != 0.f) { bail(); return; }
  if constexpr (VDEC) {
    // KDA: dot products of the buffered keys (times their per-channel decay ratios) with q and k, in fp32: two slots
    // per warp and pass, sixteen lanes per slot, eight channels per lane
    constexpr int QD = 8;
    const bool landed = mbar_wait(&bars[nst], 0, A.wait_ns);
    const int nlive = __float_as_int(misc[1]);
    for (int i0 = 0; i0 < M; i0 += 8) {
      const int i = i0 + 2 * warp + (lane >> 4), k = (lane & 15) * QD;
      float dq = 0.f, dk = 0.f;
      if (landed && i < nlive) {
        const float ks_i = ksv[i];
        const uint2 cw = *reinterpret_cast<const uint2*>(kbt + i * DK + k);
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
          const uint32_t wx = (hf ? cw.y : cw.x) ^ 0x80808080u;
          float kv[4] = {byte_to_f<0>(wx) * ks_i, byte_to_f<1>(wx) * ks_i, byte_to_f<2>(wx) * ks_i, byte_to_f<3>(wx) * ks_i};
          const float4 q4 = *reinterpret_cast<const float4*>(wq + k + 4 * hf);
          const float4 k4 = *reinterpret_cast<const float4*>(wk + k + 4 * hf);
          const float4 g4v = *reinterpret_cast<const float4*>(wg + k + 4 * hf);
          const float4 b4 = *reinterpret_cast<const float4*>(gbt + i * DK + k + 4 * hf);
          kv[0] = kv[0] * expf(g4v.x - b4.x); kv[1] = kv[1] * expf(g4v.y - b4.y);
          kv[2] = kv[2] * expf(g4v.z - b4.z); kv[3] = kv[3] * expf(g4v.w - b4.w);
          dq = fmaf(kv[0], q4.x, dq); dq = fmaf(kv[1], q4.y, dq); dq = fmaf(kv[2], q4.z, dq); dq = fmaf(kv[3], q4.w, dq);
          dk = fmaf(kv[0], k4.x, dk); dk = fmaf(kv[1], k4.y, dk); dk = fmaf(kv[2], k4.z, dk); dk = fmaf(kv[3], k4.w, dk);
        }
      }
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) {
        dq += __shfl_xor_sync(0xffffffffu, dq, o);
        dk += __shfl_xor_sync(0xffffffffu, dk, o);
      }
      if ((lane & 15) == 0 && i < M) dqk[i] = make_float2(dq, dk);
    }
    if (__syncthreads_or(!landed)) { bail(); return; }
  }

  // ---- the stages of this key head ----------------------------------------------------------------------------------
  uint32_t bf[8];
  int ci[NG][2];
  if constexpr (!AXV) {
#pragma unroll
    for (int r = 0; r < 8; r++) bf[r] = Bfw[r * 32 + lane];
    acc_start<BITS, UPG>(bf, ci);
  }
  const float kq = misc[0];
  const int n0 = __float_as_int(misc[1]);                       // live buffer entries of this slot
  const bool FOLD = CANFOLD && n0 == M - 1;                     // this token fills the buffer: fold after the read-out
  if (warp == KEY_WARP) {
    // the key goes into the buffer at slot n0 (one CTA per key head stores it); its rounded value is what the fold
    // uses for slot M - 1
    if (first) {
      *reinterpret_cast<uint32_t*>(KBh + (long long)n0 * DK + lane * 4) = kword;
      if (lane == 0) KBSh[n0] = f2h(kscale);
    }
    if (FOLD) {
      if constexpr (TFOLD) {                  // the tensor-pipe fold takes the codes and the scale
        *reinterpret_cast<uint32_t*>(smraw + P.kcur + lane * 4) = kword;
        if (lane == 0) misc[8] = kscale;
      } else {
#pragma unroll
        for (int j = 0; j < CW; j++) Rf[(M - 1) * 160 + ((lane * CW + j) >> 4) * 20 + ((lane * CW + j) & 15)] = kdeq[j];
      }
    }
  }
  const float iq1 = misc[4], iq2 = misc[5], ik1 = misc[6], ik2 = misc[7];
  const float2 dq01 = dqk[0];
  bool lost = false;

  // rounds the u of this lane's row of stage sh and appends it; returns the dequantised rounded value
  auto append_row = [&](int sh) -> float {
    const int hi = sh * HPS + hh, h = h0 + hi;
    const float u = us[hi * DV + rv];
    const float4 r4 = *reinterpret_cast<const float4*>(red + hi * NW);
    const float usc = fp16_scale(fmaxf(fmaxf(r4.x, r4.y), fmaxf(r4.z, r4.w)), 127.0f);
    const float tt = fmaf(u, rcp_approx(usc), MAGIC);
    float cc = tt - MAGIC;
    const float rem = fmaf(-cc, usc, u);
    if (!(fabsf(rem) < usc * 0.49998474f) || usc < FP16_MIN_NORMAL) cc = rq_exact(u, usc, 127.0f);
    UBseq[((long long)h * M + n0) * DV + rv] = static_cast<uint8_t>(static_cast<int>(cc));
    if (rv == 0) {
      UBSseq[h * M + n0] = f2h(usc);
      if (!VDEC) {
        const float gnew = hd[hi * HD_W + 5];
        GBseq[(long long)h * M + n0] = gnew;
        GCseq[h] = FOLD ? 0.f : gnew;
      }
      NPseq[h] = FOLD ? 0 : n0 + 1;
    }
    return cc * usc;
  };

  if (!FOLD && NSH == 2 && nst >= 2) {
    // ---- a token that does not fold, two stages: both at once -----------------------------------------------------------
    // Both stages were requested in the CTA's first instructions; once both have landed, the two tile passes, the two
    // buffer terms and the two read-outs are independent chains in the same basic blocks, and the instruction scheduler
    // interleaves them (a warp issues in order: one chain alone leaves it waiting on every tensor-core and
    // shared-memory result).
    {
      const int hiA = hh, hiB = HPS + hh;
      uint8_t* stA = smraw + P.stage0;
      uint8_t* stB = stA + P.stage_bytes;
      const float vtA = cvt_raw(rvt[0], dt_v), vtB = cvt_raw(rvt[1], dt_v);
      const float4 hdaA = *reinterpret_cast<const float4*>(hd + hiA * HD_W), hdbA = *reinterpret_cast<const float4*>(hd + hiA * HD_W + 4);
      const float4 hdaB = *reinterpret_cast<const float4*>(hd + hiB * HD_W), hdbB = *reinterpret_cast<const float4*>(hd + hiB * HD_W + 4);
      if (!mbar_wait(&bars[0], 0, A.wait_ns)) lost = true;
      if (!mbar_wait(&bars[1], 0, A.wait_ns)) lost = true;
      float tqA, tkA, tqB, tkB;
      if constexpr (AXV) {
        // every warp scales the vectors by its group's column scales, per stage (the fragment area is reused)
        uint32_t bfB[8];
        FxScale fqA, fkA, fqB, fkB;
        uint32_t* area = reinterpret_cast<uint32_t*>(smraw + P.bfv) + warp * 256;
        const unsigned short* one = reinterpret_cast<const unsigned short*>(misc + 9);
        build_b_v<BITS, TWO>(area, reinterpret_cast<const unsigned short*>(stA + P.sc_off) + warp * 128, wq, wk, lane, bf, fqA, fkA);
        build_b_v<BITS, TWO>(area, reinterpret_cast<const unsigned short*>(stB + P.sc_off) + warp * 128, wq, wk, lane, bfB, fqB, fkB);
        tile_pass_v<BITS>(smem_u32(stA), one, bf, warp, lane, tqA, tkA);
        tile_pass_v<BITS>(smem_u32(stB), one, bfB, warp, lane, tqB, tkB);
        tqA = (tqA * fqA.i1) * fqA.i2; tqB = (tqB * fqB.i1) * fqB.i2;
        if (TWO) { tkA = (tkA * fkA.i1) * fkA.i2; tkB = (tkB * fkB.i1) * fkB.i2; }
      } else {
        tile_pass<BITS, UPG, 16>(smem_u32(stA), reinterpret_cast<const unsigned short*>(stA + P.sc_off), bf, ci, warp, lane, tqA, tkA);
        tile_pass<BITS, UPG, 16>(smem_u32(stB), reinterpret_cast<const unsigned short*>(stB + P.sc_off), bf, ci, warp, lane, tqB, tkB);
        tqA = (tqA * iq1) * iq2; tqB = (tqB * iq1) * iq2;       // powers of two: exact
        if (TWO) { tkA = (tkA * ik1) * ik2; tkB = (tkB * ik1) * ik2; }
      }
      if (!VDEC) { tqA = hdaA.w * tqA; tkA = hdaA.w * tkA; tqB = hdaB.w * tqB; tkB = hdaB.w * tkB; }
      const int8_t* ubA = reinterpret_cast<const int8_t*>(stA + P.ub_off) + hh * M * DV + rv;
      const int8_t* ubB = reinterpret_cast<const int8_t*>(stB + P.ub_off) + hh * M * DV + rv;
      const float2 *dcA = dcu + hiA * M, *dcB = dcu + hiB * M;
      for (int i = 0; i < n0; i++) {                           // live slots only; dead ones may hold garbage
        const float2 dd = i == 0 ? dq01 : dqk[i];
        const float2 duA = dcA[i], duB = dcB[i];
        const float xA = static_cast<float>(ubA[i * DV]) * duA.y, xB = static_cast<float>(ubB[i * DV]) * duB.y;
        tqA = fmaf(xA, duA.x * dd.x, tqA);
        tqB = fmaf(xB, duB.x * dd.x, tqB);
        if (TWO) { tkA = fmaf(xA, duA.x * dd.y, tkA); tkB = fmaf(xB, duB.x * dd.y, tkB); }
      }
      float uA, oA, uB, oB;
      if (KIND == K_GDN) {
        uA = hdaA.y * fmaf(-hdbA.x, tkA, vtA); oA = fmaf(kq, uA, hdbA.x * tqA);
        uB = hdaB.y * fmaf(-hdbB.x, tkB, vtB); oB = fmaf(kq, uB, hdbB.x * tqB);
      } else if (KIND == K_KDA) {
        uA = hdaA.y * (vtA - tkA); oA = fmaf(kq, uA, tqA);
        uB = hdaB.y * (vtB - tkB); oB = fmaf(kq, uB, tqB);
      } else {
        uA = hdaA.y * vtA; oA = fmaf(kq, uA, hdbA.x * tqA);      // beta holds dt
        uB = hdaB.y * vtB; oB = fmaf(kq, uB, hdbB.x * tqB);
        if (A.beta) { oA = fmaf(hdbA.z, vtA, oA); oB = fmaf(hdbB.z, vtB, oB); }
      }
      us[hiA * DV + rv] = uA;
      us[hiB * DV + rv] = uB;
      uint8_t* orow = A.out + (long long)b * A.so + (long long)(h0 + hiA) * DV * osz;
      stf(orow, dt_out, rv, oA);
      stf(orow + (long long)HPS * DV * osz, dt_out, rv, oB);
      const uint32_t umask = HPS == 1 ? 0xffffffffu : (lane < 16 ? 0x0000ffffu : 0xffff0000u);
      const float mA = __uint_as_float(__reduce_max_sync(umask, __float_as_uint(fabsf(uA))));
      const float mB = __uint_as_float(__reduce_max_sync(umask, __float_as_uint(fabsf(uB))));
      if ((lane & (HPS == 1 ? 31 : 15)) == 0) { red[hiA * NW + warp] = mA; red[hiB * NW + warp] = mB; }
    }
  } else
  for (int sh = 0; sh < NSH; sh++) {
    const int s = sh % nst;
    const uint32_t parity = (sh / nst) & 1;
    const int hi = sh * HPS + hh, h = h0 + hi;
    uint8_t* st = smraw + P.stage0 + s * P.stage_bytes;
    const unsigned short* scs = reinterpret_cast<const unsigned short*>(st + P.sc_off);
    const int8_t* ubt = reinterpret_cast<const int8_t*>(st + P.ub_off) + hh * M * DV;
    const float vt = sh < 2 ? cvt_raw(rvt[sh], dt_v) : ldf(A.v + (long long)b * A.sv, dt_v, (long long)h * DV + rv);
    const float4 hda = *reinterpret_cast<const float4*>(hd + hi * HD_W);          // g, beta | dt, gcur, alpha
    const float4 hdb = *reinterpret_cast<const float4*>(hd + hi * HD_W + 4);      // a, gnew, D, -
    const float beta = hda.y, alpha = hda.w, a = hdb.x, Dv = hdb.z;
    const float2* dcf = dcu + hi * M;

    if (!mbar_wait(&bars[s], parity, A.wait_ns)) lost = true;
    SQB_STAMP(5 + 3 * (sh & 1));

    float tq, tk;
    if constexpr (AXV) {
      FxScale fq, fk;
      build_b_v<BITS, TWO>(reinterpret_cast<uint32_t*>(smraw + P.bfv) + warp * 256, scs + warp * 128, wq, wk, lane, bf, fq, fk);
      tile_pass_v<BITS>(smem_u32(st), reinterpret_cast<const unsigned short*>(misc + 9), bf, warp, lane, tq, tk);
      tq = (tq * fq.i1) * fq.i2;
      if (TWO) tk = (tk * fk.i1) * fk.i2;
    } else {
      tile_pass<BITS, UPG, 16>(smem_u32(st), scs, bf, ci, warp, lane, tq, tk);
      tq = (tq * iq1) * iq2;                                  // powers of two: exact
      if (TWO) tk = (tk * ik1) * ik2;
    }
    SQB_STAMP(6 + 3 * (sh & 1));
    if (!VDEC) { tq = alpha * tq; tk = alpha * tk; }
    for (int i = 0; i < n0; i++) {                             // live slots only; dead ones may hold garbage
      const float2 du = dcf[i];
      const float2 dd = i == 0 ? dq01 : dqk[i];
      const float ub = static_cast<float>(ubt[i * DV + rv]) * du.y;
      tq = fmaf(ub, du.x * dd.x, tq);
      if (TWO) tk = fmaf(ub, du.x * dd.y, tk);
    }
    float u, o;
    if (KIND == K_GDN) {
      u = beta * fmaf(-a, tk, vt);
      o = fmaf(kq, u, a * tq);
    } else if (KIND == K_KDA) {
      u = beta * (vt - tk);
      o = fmaf(kq, u, tq);
    } else {
      u = beta * vt;                                           // beta holds dt
      o = fmaf(kq, u, a * tq);
      if (A.beta) o = fmaf(Dv, vt, o);
    }
    us[hi * DV + rv] = u;
    stf(A.out + (long long)b * A.so + (long long)h * DV * osz, dt_out, rv, o);
    // largest |u| of the head's rows in this warp: non-negative floats order like their bit patterns (a NaN ends up
    // as the maximum, as it should)
    const uint32_t umask = HPS == 1 ? 0xffffffffu : (lane < 16 ? 0x0000ffffu : 0xffff0000u);
    const float umax = __uint_as_float(__reduce_max_sync(umask, __float_as_uint(fabsf(u))));
    if ((lane & (HPS == 1 ? 31 : 15)) == 0) red[hi * NW + warp] = umax;
    SQB_STAMP(7 + 3 * (sh & 1));

    if (CANFOLD && FOLD) {
      // append and fold the heads of this stage from the staged tile, then hand the stage back
      float* ksf = fsm + P.ksf;
      if (__syncthreads_or(lost)) { bail(); return; }         // (a barrier: u and its maxima are complete)
      const float udq = append_row(sh);
      if (VDEC) {
        GBseq[((long long)h * M + n0) * DK + tid] = ga[tid];
        GCseq[(long long)h * DK + tid] = 0.f;
      }
      if constexpr (TFMT) {
        {
          // ---- the fold on the tensor pipe (fold_mma.cuh) ----
          uint32_t* KBf = reinterpret_cast<uint32_t*>(smraw + P.kbf);
          float* tab = fsm + P.tab;
          us[hi * DV + rv] = udq;                               // this token's values as stored
          if (sh == 0) {
            mbar_wait(&bars[nst], 0, A.wait_ns);                // the key tile has landed (warp 0 saw it before)
            if (tid < 7) ksf[tid] = h2f(KBSh[tid]);
            if (tid == 7) ksf[7] = misc[8];
            if constexpr (VDEC) {
              __syncthreads();                                  // the key scales (and ga, ae of the prologue) for everybody
              build_key_frags_kda<BITS>(KBf, reinterpret_cast<const int8_t*>(kbt), reinterpret_cast<const int8_t*>(smraw + P.kcur),
                                        gbt, ga, ksf, tid);
            } else {
              build_key_frags<BITS>(KBf, reinterpret_cast<const int8_t*>(kbt), reinterpret_cast<const int8_t*>(smraw + P.kcur), tid);
            }
          }
          if (tid < HPS * 8) {                                  // per head of the stage: decays and value scales of the slots
            const int hq = tid >> 3, i = tid & 7, hf = sh * HPS + hq;
            const float gnew = hd[hf * HD_W + 5];
            tab[hq * 20 + i] = (VDEC || i == 7) ? 1.0f : expf(gnew - fsm[P.gbs + hf * 8 + i]);
            tab[hq * 20 + 8 + i] = dcu[hf * 8 + i].y;
            if (i == 0) tab[hq * 20 + 16] = expf(gnew);
          }
          __syncthreads();
          if constexpr (AXV && BITS == 8)
            fold_stage_mma_v8<DV>(smem_u32(st), reinterpret_cast<unsigned short*>(st + P.sc_off),
                                  reinterpret_cast<const int8_t*>(st + P.ub_off), us + sh * HPS * DV, tab, ksf, KBf, warp, lane);
          else if constexpr (AXV)
            fold_stage_mma_v4<DV>(smem_u32(st), reinterpret_cast<unsigned short*>(st + P.sc_off),
                                  reinterpret_cast<const int8_t*>(st + P.ub_off), us + sh * HPS * DV, tab, ksf, KBf, warp, lane);
          else
            fold_stage_mma<BITS, UPG, DV, VDEC>(smem_u32(st), reinterpret_cast<unsigned short*>(st + P.sc_off),
                                                reinterpret_cast<const int8_t*>(st + P.ub_off), us + sh * HPS * DV, tab, ksf, KBf,
                                                warp, lane, ae);
          __syncthreads();
          if (warp == 0) {
            // the stage goes back to the slot: eight pieces of codes and the scales, as bulk copies
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            const long long row0 = (long long)h0 * DV + sh * 128;
            if constexpr (V8) {
              bulk_s2g(Sseq + (row0 + lane * PROWS) * ROWB, st + lane * PITCH, PROWS * ROWB);
              if (lane == 0) bulk_s2g(SCseq + row0 * NG * 2, st + P.sc_off, 128 * NG * 2);
            } else {
              if (lane < 8) bulk_s2g(Sseq + (row0 + lane * 16) * ROWB, st + lane * PITCH, 16 * ROWB);
              else if (lane == 8) bulk_s2g(SCseq + row0 * NG * 2, st + P.sc_off, 128 * NG * 2);
            }
            bulk_commit();
            if (sh + nst < NSH || sh + 1 == NSH) bulk_wait_read();   // before the stage is refilled, and before leaving
          }
        }
      } else {
      float* Lf = fsm + P.L;
      float* fdec = fsm + P.fdec;
      const int LM = fold_lm(M);
      if (sh == 0) {
        // R: the keys of slots 0 .. M - 2 (KDA: times their decay ratio); row M - 1 was written by the key append
        if (tid < M) ksf[tid] = h2f(KBSh[tid]);
        mbar_wait(&bars[nst], 0, A.wait_ns);                  // the key tile has landed (warp 0 or 3 saw it before)
        __syncthreads();
        for (int x = tid; x < (M - 1) * DK; x += NT) {
          const int i = x / DK, k = x - i * DK;
          float kv = static_cast<float>(reinterpret_cast<const int8_t*>(kbt)[x]) * ksf[i];
          if (VDEC) kv = kv * expf(ga[k] - gbt[x]);
          Rf[i * 160 + (k >> 4) * 20 + (k & 15)] = kv;
        }
      }
      for (int hq = 0; hq < HPS; hq++) {
        const int hf = sh * HPS + hq, hg = h0 + hf;
        const float gnew = hd[hf * HD_W + 5];
        __syncthreads();                                       // L, fdec free (previous head folded); R complete
        if (tid < M) {
          fdec[tid] = (VDEC || tid == M - 1) ? 1.0f : expf(gnew - GBseq[(long long)hg * M + tid]);
          ksf[32 + tid] = h2f(UBSseq[hg * M + tid]);
        }
        if (hh == hq) Lf[rv * LM + M - 1] = udq;               // the value appended just now, as stored
        __syncthreads();
        const int8_t* ubh = reinterpret_cast<const int8_t*>(st + P.ub_off) + hq * M * DV;
        for (int x = tid; x < (M - 1) * DV; x += NT) {
          const int i = x / DV, v = x - i * DV;
          float ub = static_cast<float>(ubh[x]) * ksf[32 + i];
          if (!VDEC) ub = fdec[i] * ub;
          Lf[v * LM + i] = ub;
        }
        __syncthreads();
        const float alphan = VDEC ? 1.0f : expf(gnew);
        fold_rows<BITS, true, 8, VDEC, true>(st + hq * (DV / 16) * PITCH,
                                             reinterpret_cast<const unsigned short*>(st + P.sc_off) + hq * DV * NG, Rf, Lf, ae,
                                             alphan, DV, G, M, nullptr, Sseq + (long long)hg * DV * ROWB,
                                             reinterpret_cast<unsigned short*>(SCseq) + (long long)hg * DV * NG, warp, lane, tid,
                                             [] { __syncthreads(); return true; });
      }
      }
      if (sh + nst < NSH) {
        __syncthreads();
        if (warp == 0) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          if (lane == 0) mbar_expect_tx(&bars[s], stage_tx);
          __syncwarp();
          issue_stage(s, sh + nst, lane);
        }
      }
    } else {
      // a stage that is needed again is refilled once every warp has read it
      if (sh + nst < NSH) {
        __syncthreads();
        if (warp == 0) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          if (lane == 0) mbar_expect_tx(&bars[s], stage_tx);
          __syncwarp();
          issue_stage(s, sh + nst, lane);
        }
      }
    }
  }
  if (!FOLD) {
    // ---- append the values of all heads at slot n0, every lane its own rows ----
    if (__syncthreads_or(lost)) { bail(); return; }
    SQB_STAMP(11);
    if (NSH == 2) {
      // the two stages' rows of this lane at once: one address computation, packed arithmetic, the exact rounding of a
      // near-tie or of a subnormal scale out of line
      const int hiA = hh, hiB = HPS + hh;
      const float2 uu = make_float2(us[hiA * DV + rv], us[hiB * DV + rv]);
      const float4 rA = *reinterpret_cast<const float4*>(red + hiA * NW), rB = *reinterpret_cast<const float4*>(red + hiB * NW);
      const float2 ss = make_float2(fp16_scale(fmaxf(fmaxf(rA.x, rA.y), fmaxf(rA.z, rA.w)), 127.0f),
                                    fp16_scale(fmaxf(fmaxf(rB.x, rB.y), fmaxf(rB.z, rB.w)), 127.0f));
      const float2 mg = make_float2(MAGIC, MAGIC);
      const float2 tt = __ffma2_rn(uu, make_float2(rcp_approx(ss.x), rcp_approx(ss.y)), mg);
      float2 cc = __fadd2_rn(tt, make_float2(-MAGIC, -MAGIC));
      const float2 rem = __ffma2_rn(cc, make_float2(-ss.x, -ss.y), uu);
      const float2 lim = __fmul2_rn(ss, make_float2(0.49998474f, 0.49998474f));
      if (!(fabsf(rem.x) < lim.x) || !(fabsf(rem.y) < lim.y) || fminf(ss.x, ss.y) < FP16_MIN_NORMAL) {
        cc.x = rq_exact_cold(uu.x, ss.x);
        cc.y = rq_exact_cold(uu.y, ss.y);
      }
      uint8_t* ub = UBseq + ((long long)(h0 + hiA) * M + n0) * DV + rv;
      ub[0] = static_cast<uint8_t>(static_cast<int>(cc.x));
      ub[(long long)HPS * M * DV] = static_cast<uint8_t>(static_cast<int>(cc.y));
      if (tid < gqa) {                                        // the heads' scalars: one lane per head
        const int h = h0 + tid;
        const float4 r4 = *reinterpret_cast<const float4*>(red + tid * NW);
        UBSseq[h * M + n0] = f2h(fp16_scale(fmaxf(fmaxf(r4.x, r4.y), fmaxf(r4.z, r4.w)), 127.0f));
        if (!VDEC) {
          const float gnew = hd[tid * HD_W + 5];
          GBseq[(long long)h * M + n0] = gnew;
          GCseq[h] = gnew;
        }
        NPseq[h] = n0 + 1;
      }
    } else {
      for (int sh = 0; sh < NSH; sh++) append_row(sh);
    }
    SQB_STAMP(12);
    if (VDEC) {
      GBseq[((long long)h0 * M + n0) * DK + tid] = ga[tid];
      GCseq[(long long)h0 * DK + tid] = ga[tid];
    }
  }
}

}  // namespace sqb
