// The short causal convolution in front of the decode step, one token per sequence: window of the slot's conv state
// plus the new token, taps, bias, SiLU, and the state shifted by one (see sqb_conv1d_update in the header for the
// arithmetic).  HBM-bound: per row and channel (width - 1) state elements are read and written, one x read, one out
// written; the taps and the bias stay in L2.
//
// conv_update_vec: a thread owns the 16 bytes of x (8 channels of a 16-bit type, 4 of fp32) and moves everything in
// 16-byte pieces; two state layouts, channel-contiguous [line, token, dim] and token-contiguous [line, dim, token].
// conv_update_any: one channel per thread, any strides, any state_len >= width - 1.
#pragma once
#include "common.cuh"

namespace sqb {

struct ConvArgs {
  const uint8_t* x; long long sx;
  uint8_t* out; long long so;
  uint8_t* state; long long s_line, s_dim, s_tok;
  const uint8_t* w; long long sw_dim, sw_tap;
  const uint8_t* bias;
  const int32_t* idx;
  int rows, dim, width, state_len;
  int dt_x, dt_w;
  int silu, null_line;
  int pmode;            // 0: product fused into the fp32 sum; 1: product rounded to bf16 first; 2: to fp16
};

__device__ __forceinline__ float conv_tap(float acc, float x, float w, int pmode) {
  if (pmode == 0) return fmaf(x, w, acc);
  float p = __fmul_rn(x, w);                       // exact in fp32: two significands of at most 11 bits
  p = pmode == 1 ? bf2f(f2bf(p)) : h2f(f2h(p));
  return __fadd_rn(acc, p);
}
__device__ __forceinline__ int conv_line(const ConvArgs& A, int row) {
  const int line = A.idx ? A.idx[row] : row;
  return (line < 0 || line == A.null_line) ? -1 : line;
}

// element e of a register array that holds consecutive elements of ESZ bytes, as fp32 / as raw bits
template <int ESZ>
__device__ __forceinline__ uint32_t el_raw(const uint32_t* r, int e) {
  if (ESZ == 4) return r[e];
  return (r[e >> 1] >> ((e & 1) * 16)) & 0xFFFFu;
}
template <int ESZ>
__device__ __forceinline__ void el_put(uint32_t* r, int e, uint32_t bits) {
  if (ESZ == 4) r[e] = bits;
  else if (e & 1) r[e >> 1] |= bits << 16;
  else r[e >> 1] = bits;
}
__device__ __forceinline__ uint32_t f2raw(float v, int dt) {
  if (dt == DT_F32) return __float_as_uint(v);
  return dt == DT_BF16 ? f2bf(v) : f2h(v);
}
// NB bytes (a multiple of 8) from p, which is aligned to 16 bytes when NB is a multiple of 16 and to 8 otherwise
template <int NB>
__device__ __forceinline__ void ld_bytes(const uint8_t* p, uint32_t* r) {
  if constexpr (NB % 16 == 0) {
#pragma unroll
    for (int i = 0; i < NB / 16; i++) {
      const uint4 t = __ldg(reinterpret_cast<const uint4*>(p) + i);
      r[4 * i] = t.x; r[4 * i + 1] = t.y; r[4 * i + 2] = t.z; r[4 * i + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < NB / 8; i++) {
      const uint2 t = __ldg(reinterpret_cast<const uint2*>(p) + i);
      r[2 * i] = t.x; r[2 * i + 1] = t.y;
    }
  }
}

// the 32-bit word (element e0 | element e1 << 16) of a register array of 16-bit elements
__device__ __forceinline__ uint32_t pair16(const uint32_t* r, int e0, int e1) {
  if ((e0 & 1) == 0 && e1 == e0 + 1) return r[e0 >> 1];
  const uint32_t sel = ((e0 & 1) ? 0x0032u : 0x0010u) | ((e1 & 1) ? 0x7600u : 0x5400u);
  return __byte_perm(r[e0 >> 1], r[e1 >> 1], sel);
}
// SiLU in fp32: acc / (1 + exp(-acc)), the quotient by a reciprocal and one correction step (within an ulp of the
// IEEE quotient; the result is then rounded to the storage type)
__device__ __forceinline__ float conv_silu(float acc) {
  const float d = __fadd_rn(1.0f, expf(-acc));
  if (!(d < 1.0e37f)) return __fdiv_rn(acc, d);               // exp overflowed or nearly: the plain division
  const float r = rcp_approx(d);
  const float q = __fmul_rn(acc, r);
  return fmaf(fmaf(-d, q, acc), r, q);
}

__device__ __forceinline__ float conv_act(float acc, int silu) {
  return silu ? conv_silu(acc) : acc;
}

// LAY 0: state [line, token, dim] (s_dim == ESZ); LAY 1: state [line, dim, token] (s_tok == ESZ, s_dim == (W-1) ESZ).
// state_len == W - 1.  grid: x = row, y = chunk of NT * VEC channels.  x and w of the same 16-bit type: the products
// of two channels at a time by the packed multiply of that type, the sums in packed fp32.
template <int DTX, int DTW, int W, int LAY>
#ifndef SQB_CONV_MINB
#define SQB_CONV_MINB 1
#endif
__global__ void __launch_bounds__(NT, SQB_CONV_MINB) conv_update_vec(const __grid_constant__ ConvArgs A) {
  constexpr int ESZ = DTX == DT_F32 ? 4 : 2, WSZ = DTW == DT_F32 ? 4 : 2;
  constexpr int VEC = 16 / ESZ, T = W - 1, XW = 4;           // XW: 32-bit words of a 16-byte piece
  constexpr bool TYPED = ESZ == 2 && WSZ == 2;
  static_assert(!TYPED || DTX == DTW, "two 16-bit types: one and the same");
  const int row = blockIdx.x;
  const int c0 = (blockIdx.y * NT + threadIdx.x) * VEC;
  if (c0 >= A.dim) return;
  const int line = conv_line(A, row);
  if (line < 0) return;

  // every load of the thread first
  uint32_t xr[XW], sr[T][XW], wr[VEC * W * WSZ / 4], br[VEC * WSZ / 4];
  {
    const uint4 t = *reinterpret_cast<const uint4*>(A.x + (long long)row * A.sx + (long long)c0 * ESZ);
    xr[0] = t.x; xr[1] = t.y; xr[2] = t.z; xr[3] = t.w;
  }
  uint8_t* sb = A.state + (long long)line * A.s_line;
#pragma unroll
  for (int t = 0; t < T; t++) {
    const uint8_t* p = LAY == 0 ? sb + t * A.s_tok + (long long)c0 * ESZ : sb + (long long)c0 * (T * ESZ) + t * 16;
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    sr[t][0] = v.x; sr[t][1] = v.y; sr[t][2] = v.z; sr[t][3] = v.w;
  }
  ld_bytes<VEC * W * WSZ>(A.w + (long long)c0 * (W * WSZ), wr);
  const bool has_bias = A.bias != nullptr;
  if (has_bias) ld_bytes<VEC * WSZ>(A.bias + (long long)c0 * WSZ, br);
  const uint32_t* sflat = &sr[0][0];

  uint32_t orow[XW] = {0u, 0u, 0u, 0u};
  if constexpr (TYPED) {
#pragma unroll
    for (int i = 0; i < VEC; i += 2) {
      float2 acc = make_float2(0.f, 0.f);
      if (has_bias) acc = make_float2(cvt_raw(el_raw<2>(br, i), DTW), cvt_raw(el_raw<2>(br, i + 1), DTW));
#pragma unroll
      for (int j = 0; j < W; j++) {
        uint32_t xp;
        if (j == T) xp = xr[i >> 1];
        else if (LAY == 0) xp = sr[j][i >> 1];
        else xp = pair16(sflat, i * T + j, (i + 1) * T + j);
        const uint32_t wp = pair16(wr, i * W + j, (i + 1) * W + j);
        float2 p;
        uint32_t mb;
        if (DTX == DT_BF16) {
          asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(mb) : "r"(xp), "r"(wp));
          p = make_float2(__uint_as_float(mb << 16), __uint_as_float(mb & 0xFFFF0000u));
        } else {
          asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(mb) : "r"(xp), "r"(wp));
          asm("{\n\t.reg .f16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.f32.f16 %0, lo;\n\tcvt.f32.f16 %1, hi;\n\t}"
              : "=f"(p.x), "=f"(p.y) : "r"(mb));
        }
        acc = __fadd2_rn(acc, p);
      }
      if (A.silu) { acc.x = conv_silu(acc.x); acc.y = conv_silu(acc.y); }
      orow[i >> 1] = f2raw(acc.x, DTX) | (f2raw(acc.y, DTX) << 16);
    }
  } else {
#pragma unroll
    for (int i = 0; i < VEC; i++) {
      float acc = has_bias ? cvt_raw(el_raw<WSZ>(br, i), DTW) : 0.0f;
#pragma unroll
      for (int j = 0; j < W; j++) {
        uint32_t xb;
        if (j == T) xb = el_raw<ESZ>(xr, i);
        else if (LAY == 0) xb = el_raw<ESZ>(sr[j], i);
        else xb = el_raw<ESZ>(sflat, i * T + j);
        acc = fmaf(cvt_raw(xb, DTX), cvt_raw(el_raw<WSZ>(wr, i * W + j), DTW), acc);
      }
      el_put<ESZ>(orow, i, f2raw(A.silu ? conv_silu(acc) : acc, DTX));
    }
  }
  // the state moves up by one token
  if (LAY == 0) {
#pragma unroll
    for (int t = 0; t < T; t++) {
      const uint32_t* s = t + 1 < T ? sr[t + 1] : xr;
      *reinterpret_cast<uint4*>(sb + t * A.s_tok + (long long)c0 * ESZ) = make_uint4(s[0], s[1], s[2], s[3]);
    }
  } else {
    uint32_t nr[T][XW];
#pragma unroll
    for (int e = 0; e < VEC * T; e++) {
      const int i = e / T, t = e % T;
      el_put<ESZ>(&nr[0][0], e, t + 1 < T ? el_raw<ESZ>(sflat, i * T + t + 1) : el_raw<ESZ>(xr, i));
    }
#pragma unroll
    for (int t = 0; t < T; t++)
      *reinterpret_cast<uint4*>(sb + (long long)c0 * (T * ESZ) + t * 16) = make_uint4(nr[t][0], nr[t][1], nr[t][2], nr[t][3]);
  }
  *reinterpret_cast<uint4*>(A.out + (long long)row * A.so + (long long)c0 * ESZ) = make_uint4(orow[0], orow[1], orow[2], orow[3]);
}

// any strides, any state_len >= width - 1; one channel per thread.  grid: x = row, y = chunk of NT channels.
__global__ void __launch_bounds__(NT) conv_update_any(const __grid_constant__ ConvArgs A) {
  const int row = blockIdx.x, c = blockIdx.y * NT + threadIdx.x;
  if (c >= A.dim) return;
  const int line = conv_line(A, row);
  if (line < 0) return;
  const int esz = dt_size(A.dt_x);
  uint8_t* sc = A.state + (long long)line * A.s_line + (long long)c * A.s_dim;
  const uint8_t* wc = A.w + (long long)c * A.sw_dim;
  const uint32_t xb = ld1_raw(A.x + (long long)row * A.sx, A.dt_x, c);
  float acc = A.bias ? ldf(A.bias, A.dt_w, c) : 0.0f;
  for (int j = 0; j < A.width; j++) {
    const uint32_t vb = j == A.width - 1 ? xb : ld1_raw(sc + j * A.s_tok, A.dt_x, 0);
    acc = conv_tap(acc, cvt_raw(vb, A.dt_x), cvt_raw(ld1_raw(wc + j * A.sw_tap, A.dt_w, 0), A.dt_w), A.pmode);
  }
  for (int t = 0; t < A.state_len; t++) {
    const uint32_t vb = t + 1 < A.state_len ? ld1_raw(sc + (t + 1) * A.s_tok, A.dt_x, 0) : xb;
    if (esz == 4) *reinterpret_cast<uint32_t*>(sc + t * A.s_tok) = vb;
    else *reinterpret_cast<unsigned short*>(sc + t * A.s_tok) = static_cast<unsigned short>(vb);
  }
  stf(A.out + (long long)row * A.so, A.dt_x, c, conv_act(acc, A.silu));
}

// 0: launched; < 0: -(1000 + cudaError_t)
inline int launch_conv_update(const ConvArgs& a, cudaStream_t stream) {
  const int esz = dt_size(a.dt_x), wsz = dt_size(a.dt_w), W = a.width, vec = 16 / esz;
  auto al = [](const void* p, int n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; };
  const int wbytes = vec * W * wsz, bbytes = vec * wsz;
  int lay = -1;
  if (a.state_len == W - 1 && a.s_dim == esz && a.s_tok % 16 == 0) lay = 0;
  else if (a.state_len == W - 1 && a.s_tok == esz && a.s_dim == (long long)(W - 1) * esz) lay = 1;
  const bool vecok = lay >= 0 && a.dim % vec == 0 && al(a.x, 16) && a.sx % 16 == 0 && al(a.out, 16) && a.so % 16 == 0 &&
                     al(a.state, 16) && a.s_line % 16 == 0 && a.sw_tap == wsz && a.sw_dim == (long long)W * wsz &&
                     wbytes % 8 == 0 && al(a.w, wbytes % 16 == 0 ? 16 : 8) &&
                     (!a.bias || al(a.bias, bbytes % 16 == 0 ? 16 : 8));
  cudaError_t e = cudaSuccess;
  if (vecok) {
    const dim3 grid(a.rows, (a.dim / vec + NT - 1) / NT);
#define SQB_CONV_CASE(X, S, WW, L) \
    if (a.dt_x == X && a.dt_w == S && W == WW && lay == L) conv_update_vec<X, S, WW, L><<<grid, NT, 0, stream>>>(a);
#define SQB_CONV_W(X, S) SQB_CONV_CASE(X, S, 2, 0) SQB_CONV_CASE(X, S, 2, 1) SQB_CONV_CASE(X, S, 3, 0) \
    SQB_CONV_CASE(X, S, 3, 1) SQB_CONV_CASE(X, S, 4, 0) SQB_CONV_CASE(X, S, 4, 1)
    SQB_CONV_W(DT_BF16, DT_BF16) SQB_CONV_W(DT_F16, DT_F16) SQB_CONV_W(DT_BF16, DT_F32) SQB_CONV_W(DT_F16, DT_F32)
    SQB_CONV_W(DT_F32, DT_F32) SQB_CONV_W(DT_F32, DT_BF16) SQB_CONV_W(DT_F32, DT_F16)
#undef SQB_CONV_W
#undef SQB_CONV_CASE
    e = cudaGetLastError();
  } else {
    conv_update_any<<<dim3(a.rows, (a.dim + NT - 1) / NT), NT, 0, stream>>>(a);
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? 0 : -(1000 + static_cast<int>(e));
}

}  // namespace sqb
