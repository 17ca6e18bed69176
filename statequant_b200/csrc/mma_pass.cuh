// The state pass of the decode step on the tensor pipe (states scaled along k, head dim 128).
//
// The read-out vectors q and k are held as 30-bit fixed point with one power-of-two scale per vector and cut into four
// BALANCED byte digits (each in [-128, 127]: x = d3 2^24 + d2 2^16 + d1 2^8 + d0).  The eight digit vectors are the
// eight columns of the B operand of an integer tensor-core product
//     D[row][n] = sum_k code[row][k] * digit_n[k]          (mma.sync m16n8k32, int8 x int8 -> int32, exact)
// taken per 32-column unit; the units of one scale group accumulate in the same registers, the group's fp16 scale is
// applied to the exact integer sums, and the four digits of a vector are recombined with powers of two.  No code is
// ever converted to floating point.  A fixed-point element is exact when it lies within 2^-6 of the vector's largest
// one and is otherwise rounded to 2^-30 of it, so the pass is at least as accurate as an fp32 accumulation.
//
// Shared-memory layout of a head's codes ("pieces"): the d_v rows are cut into 8 pieces of R = d_v / 8 consecutive
// rows, piece p starting at p * (R * ROWB + 16) bytes.  The 16 bytes of padding make the eight row addresses of an
// ldmatrix 8x8 tile (one row out of each piece) fall on distinct banks; each piece is one bulk copy.
// Fragment rows: block b (16 rows) = rows 2b and 2b + 1 of every piece; fragment row i < 8 is row 2b of piece i,
// fragment row 8 + i is row 2b + 1 of piece i.  A warp takes blocks 2w and 2w + 1 (a tile of 32 rows) and ends up
// with one finished row per lane: lane (i = lane / 4, t = lane % 4) owns row i * R + 4 w + t.
//
// Column n of B: vector n / 4 (0: q, 1: k), digit 3 - n % 4, so that a thread's two accumulator columns (2t, 2t + 1)
// are the upper digit pair (t even) or the lower digit pair (t odd) of one vector.
// Units: 8-bit codes: unit j = columns 32 j .. 32 j + 31, k index = column - 32 j.  4-bit codes: unit j = the same
// columns = 16 bytes; the low nibbles (even columns) are k 0..15, the high nibbles (odd columns) k 16..31; nibbles
// carry an offset of 8, which the start value of the accumulators takes off (8 * column sum of the digits, itself
// computed by a product with an all-ones A operand).
#pragma once
#include "common.cuh"

namespace sqb {

constexpr int MAGIC_I = 0x4B400000;      // bit pattern of 1.5 * 2^23: an int32 accumulator started here reads, as a
                                          // float, 1.5 * 2^23 + sum (exact while |sum| < 2^22)

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
// D += A B: A 16 x 32 bytes (unsigned if AU), B 32 x 8 signed bytes, int32 accumulators
template <bool AU>
__device__ __forceinline__ void mma_i8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  if constexpr (AU)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- fixed point ----------------------------------------------------------------------------------------------------
// Multipliers m1 m2 = 2^(29 - e) (e: exponent of the vector's largest magnitude) as two factors that are both normal
// floats over the whole float range, and their inverses.  A non-finite amax poisons the inverse (outputs become NaN).
struct FxScale { float m1, m2, i1, i2; };
__device__ __forceinline__ FxScale fx30_scale(float amax) {
  int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xFFu) - 127;
  e = max(e, -126);
  const int sh = 29 - e;
  const int h2 = sh >> 1, h1 = sh - h2;
  FxScale s;
  s.m1 = __uint_as_float(static_cast<uint32_t>(127 + h1) << 23);
  s.m2 = __uint_as_float(static_cast<uint32_t>(127 + h2) << 23);
  s.i1 = __uint_as_float(static_cast<uint32_t>(127 - h1) << 23);
  s.i2 = __uint_as_float(static_cast<uint32_t>(127 - h2) << 23);
  if (!(amax <= 3.0e38f)) { s.m1 = 0.f; s.m2 = 0.f; s.i1 = __uint_as_float(0x7FC00000u); }
  return s;
}
// the four balanced digits of x (|x| <= 2^30) as the bytes of the result, lowest digit in byte 0
__device__ __forceinline__ uint32_t fx30_digits(float v, const FxScale& s) {
  const int x = __float2int_rn((v * s.m1) * s.m2);
  return (static_cast<uint32_t>(x) + 0x80808080u) ^ 0x80808080u;
}

// One lane's four consecutive columns (4 lane .. 4 lane + 3) of vector `vec` -> its words of the B fragments in
// shared memory, Bf[(unit * 2 + reg) * 32 + n * 4 + t].  All 32 lanes call this together.
template <int BITS>
__device__ __forceinline__ void put_b_words(uint32_t* Bf, int lane, int vec, uint32_t y0, uint32_t y1, uint32_t y2,
                                            uint32_t y3) {
  const uint32_t t0 = __byte_perm(y0, y1, 0x5140), t1 = __byte_perm(y2, y3, 0x5140);
  const uint32_t t2 = __byte_perm(y0, y1, 0x7362), t3 = __byte_perm(y2, y3, 0x7362);
  uint32_t W[4] = {__byte_perm(t0, t1, 0x5410), __byte_perm(t0, t1, 0x7632), __byte_perm(t2, t3, 0x5410),
                   __byte_perm(t2, t3, 0x7632)};                 // W[s]: digit s of the four columns
#pragma unroll
  for (int s = 0; s < 4; s++) {
    const int n = vec * 4 + (3 - s);
    if constexpr (BITS == 8) {
      Bf[(lane >> 2) * 32 + n * 4 + (lane & 3)] = W[s];           // unit lane / 8, reg (lane / 4) & 1, t lane % 4
    } else {
      const uint32_t o = __shfl_xor_sync(0xffffffffu, W[s], 1);
      const uint32_t w = (lane & 1) ? __byte_perm(o, W[s], 0x7531) : __byte_perm(W[s], o, 0x6420);
      const int p = lane >> 1;                                   // span of 8 columns; unit p / 4, t p % 4
      Bf[((p >> 2) * 2 + (lane & 1)) * 32 + n * 4 + (p & 3)] = w;
    }
  }
}

// Start values of the accumulators of scale group g (two columns per thread): the magic integer, minus 8 * the column
// sums of the digits over the group's units for nibble codes.
template <int BITS, int UPG>
__device__ __forceinline__ void acc_start(const uint32_t (&bf)[8], int (&ci)[4 / UPG][2]) {
  constexpr int NG = 4 / UPG;
#pragma unroll
  for (int g = 0; g < NG; g++) {
    if constexpr (BITS == 4) {
      int d[4] = {0, 0, 0, 0};
#pragma unroll
      for (int u = 0; u < UPG; u++) {
        const int j = g * UPG + u;
        mma_i8<true>(d, 0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u, bf[2 * j], bf[2 * j + 1]);
      }
      ci[g][0] = MAGIC_I - 8 * d[0];
      ci[g][1] = MAGIC_I - 8 * d[1];
    } else {
      ci[g][0] = MAGIC_I;
      ci[g][1] = MAGIC_I;
    }
  }
}

// One 16-row block against all units: p[0..3] += scale * sums for (row0, col 2t), (row0, col 2t + 1), (row1, ...).
// a_addr: this lane's ldmatrix row address for the block's first 32 bytes; sc: the 2 NG scales of rows row0, row0 + 1.
template <int BITS, int UPG>
__device__ __forceinline__ void block_pass(uint32_t a_addr, const unsigned short* sc, const uint32_t (&bf)[8],
                                           const int (&ci)[4 / UPG][2], float (&p)[4]) {
  constexpr int NG = 4 / UPG;
  float s0[NG], s1[NG];
  if constexpr (NG == 4) {
    const uint4 w = *reinterpret_cast<const uint4*>(sc);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
    const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&w.z)), d = __half22float2(*reinterpret_cast<const __half2*>(&w.w));
    s0[0] = a.x; s0[1] = a.y; s0[2] = b.x; s0[3] = b.y; s1[0] = c.x; s1[1] = c.y; s1[2] = d.x; s1[3] = d.y;
  } else if constexpr (NG == 2) {
    const uint2 w = *reinterpret_cast<const uint2*>(sc);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
    s0[0] = a.x; s0[1] = a.y; s1[0] = b.x; s1[1] = b.y;
  } else {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(sc);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w));
    s0[0] = a.x; s1[0] = a.y;
  }
  int acc[NG][4];
#pragma unroll
  for (int g = 0; g < NG; g++) { acc[g][0] = ci[g][0]; acc[g][1] = ci[g][1]; acc[g][2] = ci[g][0]; acc[g][3] = ci[g][1]; }
  if constexpr (BITS == 8) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      uint32_t m[4];
      ldsm_x4(m, a_addr + 32 * j);
      mma_i8<false>(acc[j / UPG], m[0], m[1], m[2], m[3], bf[2 * j], bf[2 * j + 1]);
    }
  } else {
#pragma unroll
    for (int J = 0; J < 2; J++) {
      uint32_t m[4];
      ldsm_x4(m, a_addr + 32 * J);
      const uint32_t l0 = m[0] & 0x0F0F0F0Fu, l1 = m[1] & 0x0F0F0F0Fu, l2 = m[2] & 0x0F0F0F0Fu, l3 = m[3] & 0x0F0F0F0Fu;
      const uint32_t h0 = (m[0] >> 4) & 0x0F0F0F0Fu, h1 = (m[1] >> 4) & 0x0F0F0F0Fu, h2 = (m[2] >> 4) & 0x0F0F0F0Fu,
                     h3 = (m[3] >> 4) & 0x0F0F0F0Fu;
      mma_i8<true>(acc[(2 * J) / UPG], l0, l1, h0, h1, bf[4 * J], bf[4 * J + 1]);
      mma_i8<true>(acc[(2 * J + 1) / UPG], l2, l3, h2, h3, bf[4 * J + 2], bf[4 * J + 3]);
    }
  }
  // (the accumulators of a row are a register pair: packed f32x2 arithmetic, same roundings)
  float2 p01 = make_float2(p[0], p[1]), p23 = make_float2(p[2], p[3]);
  const float2 nm = make_float2(-12582912.0f, -12582912.0f);
#pragma unroll
  for (int g = 0; g < NG; g++) {
    const float2 a01 = __fadd2_rn(make_float2(__int_as_float(acc[g][0]), __int_as_float(acc[g][1])), nm);
    const float2 a23 = __fadd2_rn(make_float2(__int_as_float(acc[g][2]), __int_as_float(acc[g][3])), nm);
    p01 = __ffma2_rn(a01, make_float2(s0[g], s0[g]), p01);
    p23 = __ffma2_rn(a23, make_float2(s1[g], s1[g]), p23);
  }
  p[0] = p01.x; p[1] = p01.y; p[2] = p23.x; p[3] = p23.y;
}

// Recombine the digit pair of a thread: after this, lane t = 0 holds vector 0 of row0, t = 1 vector 0 of row1,
// t = 2 vector 1 of row0, t = 3 vector 1 of row1 (still in fixed-point units).
__device__ __forceinline__ float join_digits(const float (&p)[4], int t) {
  const float wa = (t & 1) ? 256.0f : 16777216.0f, wb = (t & 1) ? 1.0f : 65536.0f;
  const float x0 = fmaf(p[0], wa, p[1] * wb), x1 = fmaf(p[2], wa, p[3] * wb);
  const float recv = __shfl_xor_sync(0xffffffffu, (t & 1) ? x0 : x1, 1);
  return ((t & 1) ? x1 : x0) + recv;
}

// The pass of one tile (32 rows = blocks 2w and 2w + 1 of a stage of 8 pieces): on return lane (i, t) holds the sums
// of stage row i * R + 4 w + t against vector 0 (tq) and vector 1 (tk), in fixed-point units.
// codes: shared address of the stage's first piece; pitch: bytes between pieces; scs: the stage's scales [row][NG].
template <int BITS, int UPG, int R>
__device__ __forceinline__ void tile_pass(uint32_t codes, const unsigned short* scs, const uint32_t (&bf)[8],
                                          const int (&ci)[4 / UPG][2], int w, int lane, float& tq, float& tk) {
  constexpr int NG = 4 / UPG;
  constexpr int ROWB = 128 * BITS / 8;
  constexpr int PITCH = R * ROWB + 16;
  const int i = lane >> 2, t = lane & 3;
  // ldmatrix: lane l gives the row address of matrix l / 8, row l % 8: piece l % 8, row 2b + (matrix & 1), byte half
  const uint32_t lrow = codes + (lane & 7) * PITCH + ((lane >> 3) & 1) * ROWB + (lane >> 4) * 16;
  float T[2];
#pragma unroll
  for (int bb = 0; bb < 2; bb++) {
    const int b = 2 * w + bb;
    float p[4] = {0.f, 0.f, 0.f, 0.f};
    block_pass<BITS, UPG>(lrow + 2 * b * ROWB, scs + (i * R + 2 * b) * NG, bf, ci, p);
    T[bb] = join_digits(p, t);
  }
  const float recv = __shfl_xor_sync(0xffffffffu, t < 2 ? T[1] : T[0], 2);
  tq = t < 2 ? T[0] : recv;
  tk = t < 2 ? recv : T[1];
}

// ---- states scaled along v (one scale per column for every group of 32 rows) ------------------------------------------
// The scale varies along the contraction, so it goes into the read-out vectors: group G of a head is read against
// q * scale_G and k * scale_G, in fixed point as above, and the integer sums need no scale afterwards.  A warp takes
// exactly one group: rows 32 w .. 32 w + 31 of the stage = pieces 2w and 2w + 1, and builds its own B fragments for it.
// Block bb (16 rows): fragment row f = row (f >> 1) + 8 bb of piece 2w + (f & 1).  With 64-byte rows (4-bit codes) the
// eight row addresses of an ldmatrix tile then fall on four distinct 16-byte bank groups (a two-way conflict); with
// 128-byte rows they would all collide, so 8-bit codes scaled along v are staged in smaller pieces (below).
// On return lane (i, t) holds the sums of stage row 32 w + 16 (i & 1) + (i >> 1) + 4 (t & 1) + 8 (t >> 1).

// 8-bit codes (128-byte rows) scaled along v come in 32 pieces of FOUR rows instead (pitch 4 * 128 + 16): a group is
// then eight pieces, fragment row i < 8 is row 2 bb of piece 8 w + i and fragment row 8 + i its row 2 bb + 1, and the
// eight row addresses of an ldmatrix tile fall on distinct banks again.  On return lane (i, t) holds stage row
// 32 w + 4 i + t.
constexpr int V8_PIECE_ROWS = 4, V8_PITCH = V8_PIECE_ROWS * 128 + 16;

// This lane's stage row in the layouts above.
template <int BITS>
__device__ __forceinline__ int tile_row_v(int w, int lane) {
  const int i = lane >> 2, t = lane & 3;
  if (BITS == 8) return 32 * w + 4 * i + t;
  return 32 * w + 16 * (i & 1) + (i >> 1) + 4 * (t & 1) + 8 * (t >> 1);
}
// shared address of the ldmatrix row this lane supplies for block bb of warp w's group (first 32 bytes of the rows)
template <int BITS>
__device__ __forceinline__ uint32_t tile_lrow_v(uint32_t codes, int w, int lane, int bb) {
  if (BITS == 8) return codes + (8 * w + (lane & 7)) * V8_PITCH + (2 * bb + ((lane >> 3) & 1)) * 128 + (lane >> 4) * 16;
  constexpr int ROWB = 64, PITCH = 16 * ROWB + 16;
  return codes + (2 * w + (lane & 1)) * PITCH + (((lane & 7) >> 1) + 4 * ((lane >> 3) & 1) + 8 * bb) * ROWB + (lane >> 4) * 16;
}

// The warp's B fragments for its group: sg = the group's 128 column scales (fp16), vq / vk = the read-out vectors
// (fp32, 128 each; vk unused if !TWO).  Bf: the warp's own 1 KB of shared memory.  Returns the fixed-point scales.
template <int BITS, bool TWO>
__device__ __forceinline__ void build_b_v(uint32_t* Bf, const unsigned short* sg, const float* vq, const float* vk, int lane,
                                          uint32_t (&bf)[8], FxScale& fq, FxScale& fk) {
  const uint2 sw = *reinterpret_cast<const uint2*>(sg + 4 * lane);
  const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sw.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&sw.y));
  const float4 q4 = *reinterpret_cast<const float4*>(vq + 4 * lane);
  float eq[4] = {q4.x * s01.x, q4.y * s01.y, q4.z * s23.x, q4.w * s23.y};
  float ek[4] = {0.f, 0.f, 0.f, 0.f};
  if constexpr (TWO) {
    const float4 k4 = *reinterpret_cast<const float4*>(vk + 4 * lane);
    ek[0] = k4.x * s01.x; ek[1] = k4.y * s01.y; ek[2] = k4.z * s23.x; ek[3] = k4.w * s23.y;
  }
  float mq = fmaxf(fmaxf(fabsf(eq[0]), fabsf(eq[1])), fmaxf(fabsf(eq[2]), fabsf(eq[3])));
  float mk = fmaxf(fmaxf(fabsf(ek[0]), fabsf(ek[1])), fmaxf(fabsf(ek[2]), fabsf(ek[3])));
  mq = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(mq)));
  if constexpr (TWO) mk = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(mk)));
  fq = fx30_scale(mq);
  fk = fx30_scale(mk);
  uint32_t yq[4], yk[4];
#pragma unroll
  for (int j = 0; j < 4; j++) { yq[j] = fx30_digits(eq[j], fq); yk[j] = TWO ? fx30_digits(ek[j], fk) : 0u; }
  __syncwarp();                                        // the fragments of the previous stage have been read
  put_b_words<BITS>(Bf, lane, 0, yq[0], yq[1], yq[2], yq[3]);
  put_b_words<BITS>(Bf, lane, 1, yk[0], yk[1], yk[2], yk[3]);
  __syncwarp();
#pragma unroll
  for (int r = 0; r < 8; r++) bf[r] = Bf[r * 32 + lane];
}

// one: shared address of a word holding the fp16 pair (1, 1) (the blocks carry no scale of their own)
template <int BITS>
__device__ __forceinline__ void tile_pass_v(uint32_t codes, const unsigned short* one, const uint32_t (&bf)[8], int w,
                                            int lane, float& tq, float& tk) {
  const int t = lane & 3;
  int ci[1][2];
  acc_start<BITS, 4>(bf, ci);
  float T[2];
#pragma unroll
  for (int bb = 0; bb < 2; bb++) {
    float p[4] = {0.f, 0.f, 0.f, 0.f};
    block_pass<BITS, 4>(tile_lrow_v<BITS>(codes, w, lane, bb), one, bf, ci, p);
    T[bb] = join_digits(p, t);
  }
  const float recv = __shfl_xor_sync(0xffffffffu, t < 2 ? T[1] : T[0], 2);
  tq = t < 2 ? T[0] : recv;
  tk = t < 2 ? recv : T[1];
}

}  // namespace sqb
