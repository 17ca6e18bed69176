// The fold of a stage (128 state rows) on the tensor pipe, for the tensor-core decode kernel (step_mma.cuh), buffer
// length 8, decays per head (Gated DeltaNet, Mamba2):
//     S[v][k] = alpha (code[v][k] scale) + sum_i L_i[v] key_i[k],     L_i[v] = (dec_i u_i[v]) ks_i,  key_i = int8 codes
// The sum over the 8 buffer slots is a K = 8 contraction.  L is fp32: it is cut into three bf16 pieces (8 + 8 + 8
// mantissa bits: exact), the int8 key codes are exact in bf16, so every product of an mma.m16n8k16 (bf16 x bf16 -> fp32)
// is exact and only the accumulation (fp32, in the tensor core's order) rounds.  K index = piece * 8 + slot: k-block 0
// holds pieces 0 and 1, k-block 1 piece 2 and eight zero rows.  The stored state enters as the start value of the
// accumulators, rounded twice as the reference does (code * scale, then * alpha).
//
// The codes never leave the ldmatrix fragment layout of the state pass (mma_pass.cuh): a span = 16 rows x 32 bytes is
// one ldmatrix.x4; its values are the C fragments of 4 (8-bit) or 8 (4-bit) N-blocks whose column order is chosen to
// match (a thread's bytes are its accumulator columns), re-rounded in registers and put back with stmatrix.x4.  The
// stage is then written to the slot by bulk copies (shared -> global).
#pragma once
#include "mma_pass.cuh"

namespace sqb {

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void stsm_x4(uint32_t saddr, const uint32_t (&r)[4]) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};"
               ::"r"(saddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the bulk stores of this thread have read their shared-memory source (which may then be reused or released)
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

__device__ __forceinline__ uint32_t bf2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// x = p1 + p2 + p3 exactly, each a bf16 (x finite; pieces that underflow are dropped, far below the rounding of the sum)
__device__ __forceinline__ void split3(float x, float& p1, float& p2, float& p3) {
  p1 = __bfloat162float(__float2bfloat16_rn(x));
  const float r1 = x - p1;
  p2 = __bfloat162float(__float2bfloat16_rn(r1));
  p3 = __bfloat162float(__float2bfloat16_rn(r1 - p2));
}

// rint(x / s) + mb by the IEEE division: the rare path of the fold's rounding, kept out of line so that the hot loop
// stays small in the instruction cache
static __device__ __noinline__ float div_round_cold(float x, float s, float mb) { return rintf(__fdiv_rn(x, s)) + mb; }

// Column of the head that accumulator column n (0..7) of N-block q of span j stands for.
template <int BITS>
__host__ __device__ __forceinline__ int fold_col(int j, int q, int n) {
  const int tq = n >> 1, e = n & 1;
  if (BITS == 8) return 32 * j + (q >> 1) * 16 + 4 * tq + (q & 1) * 2 + e;        // 4 N-blocks per span of 32 columns
  return 64 * j + (q >> 2) * 32 + 8 * tq + 2 * (q & 3) + e;                        // 8 N-blocks per span of 64 columns
}

// The B operand of the fold: for every (span, N-block) the thread's register: the key codes of slots (2t, 2t + 1) at the
// column of fold_col, as a bf16 pair.  KBf[(j * NQ + q) * 32 + lane]; built by all 128 threads.
// kbt: buffered keys [8][128] int8 (slots 0..6 valid), kcur: the key appended by this token (its rounded codes).
template <int BITS>
__device__ __forceinline__ void build_key_frags(uint32_t* KBf, const int8_t* kbt, const int8_t* kcur, int tid) {
  constexpr int NQ = BITS == 8 ? 4 : 8, NSPAN = BITS == 8 ? 4 : 2;
  for (int x = tid; x < NSPAN * NQ * 32; x += NT) {
    const int l = x & 31, q = (x >> 5) % NQ, j = x / (32 * NQ);
    const int col = fold_col<BITS>(j, q, l >> 2), s0 = 2 * (l & 3);
    const float k0 = static_cast<float>(kbt[s0 * 128 + col]);
    const float k1 = s0 + 1 == 7 ? static_cast<float>(kcur[col]) : static_cast<float>(kbt[(s0 + 1) * 128 + col]);
    KBf[x] = bf2(k0, k1);
  }
}


// KDA: the fold's right factor is the buffered key times its per-channel decay ratio, an fp32 value:
//     Kd_i[k] = (code_i[k] ks_i) exp(gnew[k] - G_i[k])          (slot 7: this token's key, ratio 1)
// cut into three bf16 pieces like L.  Three planes of fragments, KBf[p * NSPAN * NQ * 32 + x], x as in build_key_frags.
// gbt: the slot's buffered log decays [8][128] fp32; ga: gnew [128]; ksf: key scales of slots 0..6, [7] = this token's.
template <int BITS>
__device__ __forceinline__ void build_key_frags_kda(uint32_t* KBf, const int8_t* kbt, const int8_t* kcur, const float* gbt,
                                                    const float* ga, const float* ksf, int tid) {
  constexpr int NQ = BITS == 8 ? 4 : 8, NSPAN = BITS == 8 ? 4 : 2, PLANE = NSPAN * NQ * 32;
  for (int x = tid; x < PLANE; x += NT) {
    const int l = x & 31, q = (x >> 5) % NQ, j = x / (32 * NQ);
    const int col = fold_col<BITS>(j, q, l >> 2), s0 = 2 * (l & 3);
    const float g = ga[col];
    const float k0 = (static_cast<float>(kbt[s0 * 128 + col]) * ksf[s0]) * expf(g - gbt[s0 * 128 + col]);
    const float k1 = s0 + 1 == 7 ? static_cast<float>(kcur[col]) * ksf[7]
                                 : (static_cast<float>(kbt[(s0 + 1) * 128 + col]) * ksf[s0 + 1]) * expf(g - gbt[(s0 + 1) * 128 + col]);
    float a1, a2, a3, b1, b2, b3;
    split3(k0, a1, a2, a3);
    split3(k1, b1, b2, b3);
    KBf[x] = bf2(a1, b1);
    KBf[PLANE + x] = bf2(a2, b2);
    KBf[2 * PLANE + x] = bf2(a3, b3);
  }
}

// Folds the 32 rows of warp w (row blocks 2w and 2w + 1) of a stage.  HPS heads of d_v = 128 / HPS rows per stage.
//   st_addr / scs: the stage's codes (padded pieces) and scales [row][NG] in shared memory, both rewritten in place
//   ubt: the stage's buffered values [HPS][8][DV] int8 (slots 0..6); udq: this token's rounded values [HPS][DV]
//   tab: per head of the stage 8 floats dec_i (dec_7 unused), 8 floats value scales, then alpha; ksf: key scales [8]
// VDEC (KDA): decays per key channel: the start value is (code scale) ae[k], ae = exp(gnew); L carries no decay and no
// key scale (both are in the key fragments, three bf16 planes: build_key_frags_kda), and a product L Kd is taken as
// p1 r1 + p1 r2 + p2 r1 + p1 r3 + p2 r2 + p3 r1 (the three terms left out are below 2^-24 of it).
// READ: nothing is rounded or written back; the accumulators, i.e. the state advanced across the buffer, go to
// out [128 stage rows][128] fp32 instead (a thread's four adjacent columns of a row as one 16-byte store).
template <int BITS, int UPG, int DV, bool VDEC = false, bool READ = false>
__device__ __forceinline__ void fold_stage_mma(uint32_t st_addr, unsigned short* scs, const int8_t* ubt, const float* udq,
                                               const float* tab, const float* ksf, const uint32_t* KBf, int w, int lane,
                                               const float* ae = nullptr, float* out = nullptr) {
  constexpr int NG = 4 / UPG, ROWB = 128 * BITS / 8, PITCH = 16 * ROWB + 16;
  constexpr int NQ = BITS == 8 ? 4 : 8, NSPAN = BITS == 8 ? 4 : 2, TABW = 20;
  constexpr float QMAX = BITS == 4 ? 7.0f : 127.0f, MB = BITS == 4 ? MAGIC + 8.0f : MAGIC;
  static_assert((BITS == 8 && UPG == 1) || (BITS == 4 && UPG == 2), "one scale group per span");
  const int g = lane >> 2, t = lane & 3;
  const uint32_t lrow = st_addr + (lane & 7) * PITCH + ((lane >> 3) & 1) * ROWB + (lane >> 4) * 16;
  const int hh = (g * 16) / DV;                       // head of this thread's rows within the stage
  const float* tb = tab + hh * TABW;
  const float alphan = tb[16];
#pragma unroll 1
  for (int bb = 0; bb < 2; bb++) {
    const int b = 2 * w + bb;
    const int row0 = g * 16 + 2 * b;                   // stage rows row0, row0 + 1
    const int rv0 = row0 % DV;
    // ---- A fragments: L of rows row0, row0 + 1 at slots 2t, 2t + 1, in three bf16 pieces ----
    uint32_t A1[2], A2[2], A3[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      float p1[2], p2[2], p3[2];
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int s = 2 * t + e;
        float L;
        if (s < 7) L = tb[s] * (static_cast<float>(ubt[(hh * 8 + s) * DV + rv0 + r]) * tb[8 + s]);
        else L = udq[hh * DV + rv0 + r];
        split3(VDEC ? L : L * ksf[s], p1[e], p2[e], p3[e]);
      }
      A1[r] = bf2(p1[0], p1[1]); A2[r] = bf2(p2[0], p2[1]); A3[r] = bf2(p3[0], p3[1]);
    }
#pragma unroll 1
    for (int j = 0; j < NSPAN; j++) {
      uint32_t m[4];
      const uint32_t addr = lrow + 2 * b * ROWB + 32 * j;
      ldsm_x4(m, addr);
      const int gi = BITS == 8 ? j : j;                // scale group of the span (one group per span)
      const float sc0 = h2f(scs[row0 * NG + gi]), sc1 = h2f(scs[(row0 + 1) * NG + gi]);
      float acc[NQ][4];
      // ---- start values: (code * scale) * alpha; code * scale is exact in fp32, so this rounds once, as the
      // reference's two multiplications do ----
      const float2 al2 = make_float2(alphan, alphan);
      // the decay of N-block q's column pair: per head, or (KDA) per key channel
      auto decay_of = [&](int q) -> float2 {
        if constexpr (VDEC) return *reinterpret_cast<const float2*>(ae + fold_col<BITS>(j, q, 2 * t));
        else return al2;
      };
      if constexpr (BITS == 8) {
        // byte u = code + 128 lands in bits 8..15 of 2^23's mantissa: the float is 2^23 + 256 u, and
        // fma(that, scale / 256, -(2^23 + 2^15) scale / 256) is code * scale with every intermediate exact
        const float q0 = sc0 * 0.00390625f, q1 = sc1 * 0.00390625f;
        const float2 m0 = make_float2(q0, q0), m1 = make_float2(q1, q1);
        const float2 c0 = make_float2(-8421376.0f * q0, -8421376.0f * q0), c1 = make_float2(-8421376.0f * q1, -8421376.0f * q1);
        const uint32_t x[4] = {m[0] ^ 0x80808080u, m[1] ^ 0x80808080u, m[2] ^ 0x80808080u, m[3] ^ 0x80808080u};
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const uint32_t wa = x[2 * (q >> 1)], wb = x[2 * (q >> 1) + 1];
          float2 a, c;
          if (q & 1) {
            a = make_float2(__uint_as_float(__byte_perm(wa, 0x4B000000u, 0x7424)), __uint_as_float(__byte_perm(wa, 0x4B000000u, 0x7434)));
            c = make_float2(__uint_as_float(__byte_perm(wb, 0x4B000000u, 0x7424)), __uint_as_float(__byte_perm(wb, 0x4B000000u, 0x7434)));
          } else {
            a = make_float2(__uint_as_float(__byte_perm(wa, 0x4B000000u, 0x7404)), __uint_as_float(__byte_perm(wa, 0x4B000000u, 0x7414)));
            c = make_float2(__uint_as_float(__byte_perm(wb, 0x4B000000u, 0x7404)), __uint_as_float(__byte_perm(wb, 0x4B000000u, 0x7414)));
          }
          a = __fmul2_rn(__ffma2_rn(a, m0, c0), decay_of(q));
          c = __fmul2_rn(__ffma2_rn(c, m1, c1), decay_of(q));
          acc[q][0] = a.x; acc[q][1] = a.y; acc[q][2] = c.x; acc[q][3] = c.y;
        }
      } else {
        // nibble n of a word is masked IN PLACE into 2^23's mantissa (n <= 4; nibbles 5, 6, 7 from the word shifted down
        // by 20): the float is 2^23 + u 16^e, minus (2^23 + 8 16^e) gives (u - 8) 16^e exactly, and the power of
        // sixteen goes into the scale.  Byte i of a word holds the pair (e, e') = (0,1), (2,3), (4,0), (1,2).
        constexpr float E0[4] = {1.0f, 256.0f, 65536.0f, 16.0f}, E1[4] = {16.0f, 4096.0f, 1.0f, 256.0f};
        float2 f0[4], f1[4], bias[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
          f0[i] = make_float2(sc0 / E0[i], sc0 / E1[i]);             // divisions by constants: powers of two, exact
          f1[i] = make_float2(sc1 / E0[i], sc1 / E1[i]);
          bias[i] = make_float2(-(8388608.0f + 8.0f * E0[i]), -(8388608.0f + 8.0f * E1[i]));
        }
#pragma unroll
        for (int hx = 0; hx < 2; hx++) {
          const uint32_t w0 = m[2 * hx], w1 = m[2 * hx + 1], w0s = w0 >> 20, w1s = w1 >> 20;
          const uint32_t K = 0x4B000000u;
          float2 a[4], c[4];
          a[0] = make_float2(nib_f<0x0000000Fu>(w0, K), nib_f<0x000000F0u>(w0, K));
          a[1] = make_float2(nib_f<0x00000F00u>(w0, K), nib_f<0x0000F000u>(w0, K));
          a[2] = make_float2(nib_f<0x000F0000u>(w0, K), nib_f<0x0000000Fu>(w0s, K));
          a[3] = make_float2(nib_f<0x000000F0u>(w0s, K), nib_f<0x00000F00u>(w0s, K));
          c[0] = make_float2(nib_f<0x0000000Fu>(w1, K), nib_f<0x000000F0u>(w1, K));
          c[1] = make_float2(nib_f<0x00000F00u>(w1, K), nib_f<0x0000F000u>(w1, K));
          c[2] = make_float2(nib_f<0x000F0000u>(w1, K), nib_f<0x0000000Fu>(w1s, K));
          c[3] = make_float2(nib_f<0x000000F0u>(w1s, K), nib_f<0x00000F00u>(w1s, K));
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const int q = hx * 4 + i;
            const float2 av = __fmul2_rn(__fmul2_rn(__fadd2_rn(a[i], bias[i]), f0[i]), decay_of(q));
            const float2 cv = __fmul2_rn(__fmul2_rn(__fadd2_rn(c[i], bias[i]), f1[i]), decay_of(q));
            acc[q][0] = av.x; acc[q][1] = av.y; acc[q][2] = cv.x; acc[q][3] = cv.y;
          }
        }
      }
      // ---- the eight buffer slots ----
#pragma unroll
      for (int q = 0; q < NQ; q++) {
        if constexpr (VDEC) {
          constexpr int PLANE = NSPAN * NQ * 32;
          const uint32_t r1 = KBf[(j * NQ + q) * 32 + lane], r2 = KBf[PLANE + (j * NQ + q) * 32 + lane],
                         r3 = KBf[2 * PLANE + (j * NQ + q) * 32 + lane];
          mma_bf16(acc[q], A1[0], A1[1], A1[0], A1[1], r1, r2);      // p1 r1 + p1 r2
          mma_bf16(acc[q], A2[0], A2[1], A1[0], A1[1], r1, r3);      // p2 r1 + p1 r3
          mma_bf16(acc[q], A2[0], A2[1], A3[0], A3[1], r2, r1);      // p2 r2 + p3 r1
        } else {
          const uint32_t kw = KBf[(j * NQ + q) * 32 + lane];
          mma_bf16(acc[q], A1[0], A1[1], A2[0], A2[1], kw, kw);
          mma_bf16(acc[q], A3[0], A3[1], 0u, 0u, kw, kw);
        }
      }
      if constexpr (READ) {
        float* o0 = out + (long long)row0 * 128 + (BITS == 8 ? 32 * j + 4 * t : 64 * j + 8 * t);
#pragma unroll
        for (int hx = 0; hx < 2; hx++) {
          if constexpr (BITS == 8) {
            float* p = o0 + 16 * hx;
            *reinterpret_cast<float4*>(p) = make_float4(acc[2 * hx][0], acc[2 * hx][1], acc[2 * hx + 1][0], acc[2 * hx + 1][1]);
            *reinterpret_cast<float4*>(p + 128) = make_float4(acc[2 * hx][2], acc[2 * hx][3], acc[2 * hx + 1][2], acc[2 * hx + 1][3]);
          } else {
            float* p = o0 + 32 * hx;
            const int q = 4 * hx;
            *reinterpret_cast<float4*>(p) = make_float4(acc[q][0], acc[q][1], acc[q + 1][0], acc[q + 1][1]);
            *reinterpret_cast<float4*>(p + 4) = make_float4(acc[q + 2][0], acc[q + 2][1], acc[q + 3][0], acc[q + 3][1]);
            *reinterpret_cast<float4*>(p + 128) = make_float4(acc[q][2], acc[q][3], acc[q + 1][2], acc[q + 1][3]);
            *reinterpret_cast<float4*>(p + 132) = make_float4(acc[q + 2][2], acc[q + 2][3], acc[q + 3][2], acc[q + 3][3]);
          }
        }
        continue;
      }
      // ---- fresh scales: absmax over the group = this span, over the quad ----
      float am0 = 0.f, am1 = 0.f;
#pragma unroll
      for (int q = 0; q < NQ; q++) {
        am0 = fmaxf(am0, fmaxf(fabsf(acc[q][0]), fabsf(acc[q][1])));
        am1 = fmaxf(am1, fmaxf(fabsf(acc[q][2]), fabsf(acc[q][3])));
      }
      am0 = fmaxf(am0, __shfl_xor_sync(0xffffffffu, am0, 1)); am1 = fmaxf(am1, __shfl_xor_sync(0xffffffffu, am1, 1));
      am0 = fmaxf(am0, __shfl_xor_sync(0xffffffffu, am0, 2)); am1 = fmaxf(am1, __shfl_xor_sync(0xffffffffu, am1, 2));
      const float s0 = fp16_scale(am0, QMAX), s1 = fp16_scale(am1, QMAX);
      // ---- round: rint(x / s) lies between the roundings of x r- and x r+ for any r- < 1 / s < r+ (rounding is
      // monotone, and so is the division's own rounding, which moves the quotient by 2^-24 of itself, well inside
      // the bracket).  r+- = r (1 +- 2^-22) around the approximate reciprocal r (error below 2^-23 of itself).
      // Where the two agree, that is the answer; where they differ (the quotient within 1e-4 of a tie) divide. ----
      const float ra0 = rcp_approx(s0), ra1 = rcp_approx(s1);
      const float2 lo0 = make_float2(fmaf(-ra0, 0x1p-22f, ra0), fmaf(-ra0, 0x1p-22f, ra0));
      const float2 hi0 = make_float2(fmaf(ra0, 0x1p-22f, ra0), fmaf(ra0, 0x1p-22f, ra0));
      const float2 lo1 = make_float2(fmaf(-ra1, 0x1p-22f, ra1), fmaf(-ra1, 0x1p-22f, ra1));
      const float2 hi1 = make_float2(fmaf(ra1, 0x1p-22f, ra1), fmaf(ra1, 0x1p-22f, ra1));
      const float2 mb2 = make_float2(MB, MB);
      float tv[NQ][4];
      uint32_t differ = 0;
#pragma unroll
      for (int q = 0; q < NQ; q++) {
        const float2 xa = make_float2(acc[q][0], acc[q][1]), xc = make_float2(acc[q][2], acc[q][3]);
        const float2 la = __ffma2_rn(xa, lo0, mb2), ha = __ffma2_rn(xa, hi0, mb2);
        const float2 lc = __ffma2_rn(xc, lo1, mb2), hc = __ffma2_rn(xc, hi1, mb2);
        tv[q][0] = la.x; tv[q][1] = la.y; tv[q][2] = lc.x; tv[q][3] = lc.y;
        differ |= (__float_as_uint(la.x) ^ __float_as_uint(ha.x)) | (__float_as_uint(la.y) ^ __float_as_uint(ha.y));
        differ |= (__float_as_uint(lc.x) ^ __float_as_uint(hc.x)) | (__float_as_uint(lc.y) ^ __float_as_uint(hc.y));
      }
      if (differ != 0) {                              // rare: some element of this thread is close to a tie
#pragma unroll
        for (int q = 0; q < NQ; q++) {
#pragma unroll
          for (int e = 0; e < 2; e++) {
            tv[q][e] = div_round_cold(acc[q][e], s0, MB);
            tv[q][2 + e] = div_round_cold(acc[q][2 + e], s1, MB);
          }
        }
      }
      // The candidate is the right UNCLAMPED integer whatever the scale; only a scale in fp16's subnormal range
      // (rounded far from absmax / qmax) lets a quotient pass qmax, and then clamping the candidate is what
      // clamp(rint(div_rn(x, s))) does.
      if (s0 < FP16_MIN_NORMAL || s1 < FP16_MIN_NORMAL) {
#pragma unroll
        for (int q = 0; q < NQ; q++) {
#pragma unroll
          for (int e = 0; e < 4; e++) tv[q][e] = fminf(fmaxf(tv[q][e], MB - QMAX), MB + QMAX);
        }
      }
      // ---- repack into the fragment registers ----
      uint32_t o[4];
      auto two = [](uint32_t a, uint32_t c) { return __byte_perm(a, c, 0x0040); };   // bytes (a, c)
      if constexpr (BITS == 8) {
        auto u = [](float f) { return __float_as_uint(f); };
        o[0] = __byte_perm(two(u(tv[0][0]), u(tv[0][1])), two(u(tv[1][0]), u(tv[1][1])), 0x5410);
        o[1] = __byte_perm(two(u(tv[0][2]), u(tv[0][3])), two(u(tv[1][2]), u(tv[1][3])), 0x5410);
        o[2] = __byte_perm(two(u(tv[2][0]), u(tv[2][1])), two(u(tv[3][0]), u(tv[3][1])), 0x5410);
        o[3] = __byte_perm(two(u(tv[2][2]), u(tv[2][3])), two(u(tv[3][2]), u(tv[3][3])), 0x5410);
      } else {
        // a candidate's low 4 bits are code + 8 and the next 4 are zero, so lo + 16 hi has the packed byte at the bottom
        auto by = [](float lo, float hi) { return __float_as_uint(lo) + (__float_as_uint(hi) << 4); };
#pragma unroll
        for (int hx = 0; hx < 2; hx++) {
          const int q = hx * 4;
          o[2 * hx] = __byte_perm(two(by(tv[q][0], tv[q][1]), by(tv[q + 1][0], tv[q + 1][1])),
                                  two(by(tv[q + 2][0], tv[q + 2][1]), by(tv[q + 3][0], tv[q + 3][1])), 0x5410);
          o[2 * hx + 1] = __byte_perm(two(by(tv[q][2], tv[q][3]), by(tv[q + 1][2], tv[q + 1][3])),
                                      two(by(tv[q + 2][2], tv[q + 2][3]), by(tv[q + 3][2], tv[q + 3][3])), 0x5410);
        }
      }
      __syncwarp();                                     // every lane has read the span's codes and old scales
      stsm_x4(addr, o);
      if (t == 0) {
        scs[row0 * NG + gi] = f2h(s0);
        scs[(row0 + 1) * NG + gi] = f2h(s1);
      }
    }
  }
}

__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(saddr));
}
__device__ __forceinline__ void stsm_x2(uint32_t saddr, uint32_t r0, uint32_t r1) {
  asm volatile("stmatrix.sync.aligned.m8n8.x2.shared.b16 [%0], {%1, %2};" ::"r"(saddr), "r"(r0), "r"(r1) : "memory");
}

// The same fold for 4-bit codes scaled along v in groups of 32 rows (one scale per column and group).  Warp w owns
// group w of the stage (the rows of tile_pass_v, mma_pass.cuh), so a column's absolute maximum over the group is a
// reduction inside the warp.  The row is walked in four chunks of 32 columns (16 bytes: one ldmatrix.x2 per 16-row
// block); a thread holds 8 columns of 4 rows per chunk.  After the reduction lane (i, t) computes the fresh scale of
// ONE column (the i-th of the quad's eight) and the quad's lanes exchange them.
//   scs: the stage's scales [4][128] fp16, rewritten in place; the other arguments as fold_stage_mma.
template <int DV>
__device__ __forceinline__ void fold_stage_mma_v4(uint32_t st_addr, unsigned short* scs, const int8_t* ubt, const float* udq,
                                                  const float* tab, const float* ksf, const uint32_t* KBf, int w, int lane) {
  constexpr int ROWB = 64, PITCH = 16 * ROWB + 16, TABW = 20;
  constexpr float QMAX = 7.0f, MB = MAGIC + 8.0f;
  const int i = lane >> 2, t = lane & 3;
  const uint32_t lrow = st_addr + (2 * w + (lane & 1)) * PITCH + (((lane & 7) >> 1) + 4 * ((lane >> 3) & 1)) * ROWB;
  const int hh = (32 * w) / DV;                        // the warp's 32 rows lie in one head
  const float* tb = tab + hh * TABW;
  const float2 al2 = make_float2(tb[16], tb[16]);
  // ---- A fragments: L of the thread's four rows (fragment rows i, i + 8 of blocks 0, 1) at slots 2t, 2t + 1 ----
  uint32_t A1[2][2], A2[2][2], A3[2][2];
#pragma unroll
  for (int bb = 0; bb < 2; bb++) {
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const int rv0 = (32 * w + 16 * (i & 1) + (i >> 1) + 4 * r + 8 * bb) % DV;
      float p1[2], p2[2], p3[2];
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int sl = 2 * t + e;
        float L;
        if (sl < 7) L = tb[sl] * (static_cast<float>(ubt[(hh * 8 + sl) * DV + rv0]) * tb[8 + sl]);
        else L = udq[hh * DV + rv0];
        split3(L * ksf[sl], p1[e], p2[e], p3[e]);
      }
      A1[bb][r] = bf2(p1[0], p1[1]); A2[bb][r] = bf2(p2[0], p2[1]); A3[bb][r] = bf2(p3[0], p3[1]);
    }
  }
  constexpr float E0[4] = {1.0f, 256.0f, 65536.0f, 16.0f}, E1[4] = {16.0f, 4096.0f, 1.0f, 256.0f};   // see fold_stage_mma
#pragma unroll 1
  for (int c4 = 0; c4 < 4; c4++) {
    uint32_t wd[2][2];                                 // [block][fragment row i / i + 8]: 8 nibbles = this thread's 8 columns
    ldsm_x2(wd[0], lrow + 16 * c4);
    ldsm_x2(wd[1], lrow + 8 * ROWB + 16 * c4);
    unsigned short* scol = scs + w * 128 + 32 * c4 + 8 * t;                  // the thread's 8 column scales
    const uint4 sw = *reinterpret_cast<const uint4*>(scol);
    const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sw.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&sw.y));
    const float2 s45 = __half22float2(*reinterpret_cast<const __half2*>(&sw.z)), s67 = __half22float2(*reinterpret_cast<const __half2*>(&sw.w));
    const float2 so[4] = {s01, s23, s45, s67};
    float acc[2][4][4];
    // ---- start values: (code * scale) * alpha ----
#pragma unroll
    for (int bb = 0; bb < 2; bb++) {
      const uint32_t w0 = wd[bb][0], w1 = wd[bb][1], w0s = w0 >> 20, w1s = w1 >> 20;
      const uint32_t K = 0x4B000000u;
      float2 a[4], c[4];
      a[0] = make_float2(nib_f<0x0000000Fu>(w0, K), nib_f<0x000000F0u>(w0, K));
      a[1] = make_float2(nib_f<0x00000F00u>(w0, K), nib_f<0x0000F000u>(w0, K));
      a[2] = make_float2(nib_f<0x000F0000u>(w0, K), nib_f<0x0000000Fu>(w0s, K));
      a[3] = make_float2(nib_f<0x000000F0u>(w0s, K), nib_f<0x00000F00u>(w0s, K));
      c[0] = make_float2(nib_f<0x0000000Fu>(w1, K), nib_f<0x000000F0u>(w1, K));
      c[1] = make_float2(nib_f<0x00000F00u>(w1, K), nib_f<0x0000F000u>(w1, K));
      c[2] = make_float2(nib_f<0x000F0000u>(w1, K), nib_f<0x0000000Fu>(w1s, K));
      c[3] = make_float2(nib_f<0x000000F0u>(w1s, K), nib_f<0x00000F00u>(w1s, K));
#pragma unroll
      for (int b4 = 0; b4 < 4; b4++) {
        const float2 f = make_float2(so[b4].x / E0[b4], so[b4].y / E1[b4]);     // powers of two: exact
        const float2 bias = make_float2(-(8388608.0f + 8.0f * E0[b4]), -(8388608.0f + 8.0f * E1[b4]));
        const float2 av = __fmul2_rn(__fmul2_rn(__fadd2_rn(a[b4], bias), f), al2);
        const float2 cv = __fmul2_rn(__fmul2_rn(__fadd2_rn(c[b4], bias), f), al2);
        acc[bb][b4][0] = av.x; acc[bb][b4][1] = av.y; acc[bb][b4][2] = cv.x; acc[bb][b4][3] = cv.y;
      }
    }
    // ---- the eight buffer slots ----
#pragma unroll
    for (int b4 = 0; b4 < 4; b4++) {
      const uint32_t kw = KBf[(c4 * 4 + b4) * 32 + lane];
#pragma unroll
      for (int bb = 0; bb < 2; bb++) {
        mma_bf16(acc[bb][b4], A1[bb][0], A1[bb][1], A2[bb][0], A2[bb][1], kw, kw);
        mma_bf16(acc[bb][b4], A3[bb][0], A3[bb][1], 0u, 0u, kw, kw);
      }
    }
    // ---- fresh scales: a column's absolute maximum over the group's 32 rows ----
    float cm[8];
#pragma unroll
    for (int b4 = 0; b4 < 4; b4++) {
#pragma unroll
      for (int e = 0; e < 2; e++) {
        float m = fmaxf(fmaxf(fabsf(acc[0][b4][e]), fabsf(acc[0][b4][2 + e])), fmaxf(fabsf(acc[1][b4][e]), fabsf(acc[1][b4][2 + e])));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
        cm[2 * b4 + e] = m;
      }
    }
    float mine = (i & 4) ? ((i & 2) ? ((i & 1) ? cm[7] : cm[6]) : ((i & 1) ? cm[5] : cm[4]))
                         : ((i & 2) ? ((i & 1) ? cm[3] : cm[2]) : ((i & 1) ? cm[1] : cm[0]));
    const float sc_mine = fp16_scale(mine, QMAX), rc_mine = rcp_approx(sc_mine);
    __syncwarp();                                      // every lane has read the chunk's old scales
    scol[i] = f2h(sc_mine);
    float sn[8], rn[8];
    float smin = 1.0f;
#pragma unroll
    for (int x = 0; x < 8; x++) {
      sn[x] = __shfl_sync(0xffffffffu, sc_mine, 4 * x + t);
      rn[x] = __shfl_sync(0xffffffffu, rc_mine, 4 * x + t);
      smin = fminf(smin, sn[x]);
    }
    // ---- round (the bracket of fold_stage_mma, one reciprocal per column) and repack ----
    uint32_t o[2][2];
#pragma unroll
    for (int bb = 0; bb < 2; bb++) {
      float tv[4][4];
      uint32_t differ = 0;
#pragma unroll
      for (int b4 = 0; b4 < 4; b4++) {
        const float2 lo = make_float2(fmaf(-rn[2 * b4], 0x1p-22f, rn[2 * b4]), fmaf(-rn[2 * b4 + 1], 0x1p-22f, rn[2 * b4 + 1]));
        const float2 hi = make_float2(fmaf(rn[2 * b4], 0x1p-22f, rn[2 * b4]), fmaf(rn[2 * b4 + 1], 0x1p-22f, rn[2 * b4 + 1]));
        const float2 mb2 = make_float2(MB, MB);
        const float2 xa = make_float2(acc[bb][b4][0], acc[bb][b4][1]), xc = make_float2(acc[bb][b4][2], acc[bb][b4][3]);
        const float2 la = __ffma2_rn(xa, lo, mb2), ha = __ffma2_rn(xa, hi, mb2);
        const float2 lc = __ffma2_rn(xc, lo, mb2), hc = __ffma2_rn(xc, hi, mb2);
        tv[b4][0] = la.x; tv[b4][1] = la.y; tv[b4][2] = lc.x; tv[b4][3] = lc.y;
        differ |= (__float_as_uint(la.x) ^ __float_as_uint(ha.x)) | (__float_as_uint(la.y) ^ __float_as_uint(ha.y));
        differ |= (__float_as_uint(lc.x) ^ __float_as_uint(hc.x)) | (__float_as_uint(lc.y) ^ __float_as_uint(hc.y));
      }
      if (differ != 0) {                               // rare: some element of this thread is close to a tie
#pragma unroll
        for (int b4 = 0; b4 < 4; b4++) {
#pragma unroll
          for (int e = 0; e < 2; e++) {
            tv[b4][e] = div_round_cold(acc[bb][b4][e], sn[2 * b4 + e], MB);
            tv[b4][2 + e] = div_round_cold(acc[bb][b4][2 + e], sn[2 * b4 + e], MB);
          }
        }
      }
      if (smin < FP16_MIN_NORMAL) {                    // only a scale in fp16's subnormal range lets a quotient pass qmax
#pragma unroll
        for (int b4 = 0; b4 < 4; b4++) {
#pragma unroll
          for (int e = 0; e < 4; e++) tv[b4][e] = fminf(fmaxf(tv[b4][e], MB - QMAX), MB + QMAX);
        }
      }
      auto two = [](uint32_t a, uint32_t c) { return __byte_perm(a, c, 0x0040); };
      auto by = [](float lo, float hi) { return __float_as_uint(lo) + (__float_as_uint(hi) << 4); };
      o[bb][0] = __byte_perm(two(by(tv[0][0], tv[0][1]), by(tv[1][0], tv[1][1])), two(by(tv[2][0], tv[2][1]), by(tv[3][0], tv[3][1])), 0x5410);
      o[bb][1] = __byte_perm(two(by(tv[0][2], tv[0][3]), by(tv[1][2], tv[1][3])), two(by(tv[2][2], tv[2][3]), by(tv[3][2], tv[3][3])), 0x5410);
    }
    __syncwarp();                                      // every lane has read the chunk's codes
    stsm_x2(lrow + 16 * c4, o[0][0], o[0][1]);
    stsm_x2(lrow + 8 * ROWB + 16 * c4, o[1][0], o[1][1]);
  }
}

// The same for 8-bit codes scaled along v (pieces of four rows, see tile_row_v<8>): a chunk is 32 columns = 32 bytes of
// a row, one ldmatrix.x4 per 16-row block; a thread holds columns 4t .. 4t + 3 and 16 + 4t .. 16 + 4t + 3 of the chunk
// (N-block q: half q >> 1, byte pair q & 1) of four rows.
template <int DV>
__device__ __forceinline__ void fold_stage_mma_v8(uint32_t st_addr, unsigned short* scs, const int8_t* ubt, const float* udq,
                                                  const float* tab, const float* ksf, const uint32_t* KBf, int w, int lane) {
  constexpr int TABW = 20;
  constexpr float QMAX = 127.0f, MB = MAGIC;
  const int i = lane >> 2, t = lane & 3;
  const int hh = (32 * w) / DV;
  const float* tb = tab + hh * TABW;
  const float2 al2 = make_float2(tb[16], tb[16]);
  uint32_t A1[2][2], A2[2][2], A3[2][2];
#pragma unroll
  for (int bb = 0; bb < 2; bb++) {
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const int rv0 = (32 * w + 4 * i + 2 * bb + r) % DV;
      float p1[2], p2[2], p3[2];
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int sl = 2 * t + e;
        float L;
        if (sl < 7) L = tb[sl] * (static_cast<float>(ubt[(hh * 8 + sl) * DV + rv0]) * tb[8 + sl]);
        else L = udq[hh * DV + rv0];
        split3(L * ksf[sl], p1[e], p2[e], p3[e]);
      }
      A1[bb][r] = bf2(p1[0], p1[1]); A2[bb][r] = bf2(p2[0], p2[1]); A3[bb][r] = bf2(p3[0], p3[1]);
    }
  }
#pragma unroll 1
  for (int c4 = 0; c4 < 4; c4++) {
    uint32_t m[2][4];
    ldsm_x4(m[0], tile_lrow_v<8>(st_addr, w, lane, 0) + 32 * c4);
    ldsm_x4(m[1], tile_lrow_v<8>(st_addr, w, lane, 1) + 32 * c4);
    // the thread's 8 column scales: columns 4t .. 4t + 3 and 16 + 4t .. 16 + 4t + 3 of the chunk
    unsigned short* scol = scs + w * 128 + 32 * c4 + 4 * t;
    const uint2 swa = *reinterpret_cast<const uint2*>(scol), swb = *reinterpret_cast<const uint2*>(scol + 16);
    const float2 so[4] = {__half22float2(*reinterpret_cast<const __half2*>(&swa.x)), __half22float2(*reinterpret_cast<const __half2*>(&swa.y)),
                          __half22float2(*reinterpret_cast<const __half2*>(&swb.x)), __half22float2(*reinterpret_cast<const __half2*>(&swb.y))};
    float acc[2][4][4];
    // ---- start values: (code * scale) * alpha (fold_stage_mma's exact byte-in-mantissa product, one scale per column) ----
#pragma unroll
    for (int q = 0; q < 4; q++) {
      const float2 mq = make_float2(so[q].x * 0.00390625f, so[q].y * 0.00390625f);
      const float2 cq = make_float2(-8421376.0f * mq.x, -8421376.0f * mq.y);
#pragma unroll
      for (int bb = 0; bb < 2; bb++) {
        const uint32_t wa = m[bb][2 * (q >> 1)] ^ 0x80808080u, wb = m[bb][2 * (q >> 1) + 1] ^ 0x80808080u;
        float2 a, c;
        if (q & 1) {
          a = make_float2(__uint_as_float(__byte_perm(wa, 0x4B000000u, 0x7424)), __uint_as_float(__byte_perm(wa, 0x4B000000u, 0x7434)));
          c = make_float2(__uint_as_float(__byte_perm(wb, 0x4B000000u, 0x7424)), __uint_as_float(__byte_perm(wb, 0x4B000000u, 0x7434)));
        } else {
          a = make_float2(__uint_as_float(__byte_perm(wa, 0x4B000000u, 0x7404)), __uint_as_float(__byte_perm(wa, 0x4B000000u, 0x7414)));
          c = make_float2(__uint_as_float(__byte_perm(wb, 0x4B000000u, 0x7404)), __uint_as_float(__byte_perm(wb, 0x4B000000u, 0x7414)));
        }
        a = __fmul2_rn(__ffma2_rn(a, mq, cq), al2);
        c = __fmul2_rn(__ffma2_rn(c, mq, cq), al2);
        acc[bb][q][0] = a.x; acc[bb][q][1] = a.y; acc[bb][q][2] = c.x; acc[bb][q][3] = c.y;
      }
    }
    // ---- the eight buffer slots ----
#pragma unroll
    for (int q = 0; q < 4; q++) {
      const uint32_t kw = KBf[(c4 * 4 + q) * 32 + lane];
#pragma unroll
      for (int bb = 0; bb < 2; bb++) {
        mma_bf16(acc[bb][q], A1[bb][0], A1[bb][1], A2[bb][0], A2[bb][1], kw, kw);
        mma_bf16(acc[bb][q], A3[bb][0], A3[bb][1], 0u, 0u, kw, kw);
      }
    }
    // ---- fresh scales: a column's absolute maximum over the group's 32 rows ----
    float cm[8];
#pragma unroll
    for (int q = 0; q < 4; q++) {
#pragma unroll
      for (int e = 0; e < 2; e++) {
        float mx = fmaxf(fmaxf(fabsf(acc[0][q][e]), fabsf(acc[0][q][2 + e])), fmaxf(fabsf(acc[1][q][e]), fabsf(acc[1][q][2 + e])));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        cm[2 * q + e] = mx;
      }
    }
    float mine = (i & 4) ? ((i & 2) ? ((i & 1) ? cm[7] : cm[6]) : ((i & 1) ? cm[5] : cm[4]))
                         : ((i & 2) ? ((i & 1) ? cm[3] : cm[2]) : ((i & 1) ? cm[1] : cm[0]));
    const float sc_mine = fp16_scale(mine, QMAX), rc_mine = rcp_approx(sc_mine);
    __syncwarp();                                      // every lane has read the chunk's old scales
    scol[(i >> 2) * 16 + (i & 3)] = f2h(sc_mine);      // column i of the thread's eight: (q, e) = (i >> 1, i & 1)
    float sn[8], rn[8];
    float smin = 1.0f;
#pragma unroll
    for (int x = 0; x < 8; x++) {
      sn[x] = __shfl_sync(0xffffffffu, sc_mine, 4 * x + t);
      rn[x] = __shfl_sync(0xffffffffu, rc_mine, 4 * x + t);
      smin = fminf(smin, sn[x]);
    }
    // ---- round (the bracket of fold_stage_mma, one reciprocal per column) and repack ----
#pragma unroll
    for (int bb = 0; bb < 2; bb++) {
      float tv[4][4];
      uint32_t differ = 0;
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const float2 lo = make_float2(fmaf(-rn[2 * q], 0x1p-22f, rn[2 * q]), fmaf(-rn[2 * q + 1], 0x1p-22f, rn[2 * q + 1]));
        const float2 hi = make_float2(fmaf(rn[2 * q], 0x1p-22f, rn[2 * q]), fmaf(rn[2 * q + 1], 0x1p-22f, rn[2 * q + 1]));
        const float2 mb2 = make_float2(MB, MB);
        const float2 xa = make_float2(acc[bb][q][0], acc[bb][q][1]), xc = make_float2(acc[bb][q][2], acc[bb][q][3]);
        const float2 la = __ffma2_rn(xa, lo, mb2), ha = __ffma2_rn(xa, hi, mb2);
        const float2 lc = __ffma2_rn(xc, lo, mb2), hc = __ffma2_rn(xc, hi, mb2);
        tv[q][0] = la.x; tv[q][1] = la.y; tv[q][2] = lc.x; tv[q][3] = lc.y;
        differ |= (__float_as_uint(la.x) ^ __float_as_uint(ha.x)) | (__float_as_uint(la.y) ^ __float_as_uint(ha.y));
        differ |= (__float_as_uint(lc.x) ^ __float_as_uint(hc.x)) | (__float_as_uint(lc.y) ^ __float_as_uint(hc.y));
      }
      if (differ != 0) {                               // rare: some element of this thread is close to a tie
#pragma unroll
        for (int q = 0; q < 4; q++) {
#pragma unroll
          for (int e = 0; e < 2; e++) {
            tv[q][e] = div_round_cold(acc[bb][q][e], sn[2 * q + e], MB);
            tv[q][2 + e] = div_round_cold(acc[bb][q][2 + e], sn[2 * q + e], MB);
          }
        }
      }
      if (smin < FP16_MIN_NORMAL) {                    // only a scale in fp16's subnormal range lets a quotient pass qmax
#pragma unroll
        for (int q = 0; q < 4; q++) {
#pragma unroll
          for (int e = 0; e < 4; e++) tv[q][e] = fminf(fmaxf(tv[q][e], MB - QMAX), MB + QMAX);
        }
      }
      auto two = [](uint32_t a, uint32_t c) { return __byte_perm(a, c, 0x0040); };
      auto u = [](float f) { return __float_as_uint(f); };
      uint32_t o[4];
      o[0] = __byte_perm(two(u(tv[0][0]), u(tv[0][1])), two(u(tv[1][0]), u(tv[1][1])), 0x5410);
      o[1] = __byte_perm(two(u(tv[0][2]), u(tv[0][3])), two(u(tv[1][2]), u(tv[1][3])), 0x5410);
      o[2] = __byte_perm(two(u(tv[2][0]), u(tv[2][1])), two(u(tv[3][0]), u(tv[3][1])), 0x5410);
      o[3] = __byte_perm(two(u(tv[2][2]), u(tv[2][3])), two(u(tv[3][2]), u(tv[3][3])), 0x5410);
      __syncwarp();                                    // every lane has read the block's codes of this chunk
      stsm_x4(tile_lrow_v<8>(st_addr, w, lane, bb) + 32 * c4, o);
    }
  }
}

}  // namespace sqb
