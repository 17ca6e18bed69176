/*
 * CPU oracle of the short causal convolution that feeds the decode step.  TEST INFRASTRUCTURE ONLY (see
 * sq_oracle.c): nothing in the product path may call into this file.
 *
 * The reference (HallerPatrick/StateQuant) does not implement this op; its vLLM forward calls vLLM's
 * `causal_conv1d_update` right before the packed step (src/statequant/integrations/vllm_plugin.py:379-381).  The
 * arithmetic therefore lives in a third-party dependency, vLLM (0.22.x in this image; the reference's pyproject asks
 * for >= 0.32 with the same op), file vllm/model_executor/layers/mamba/ops/causal_conv1d.py, kernel
 * `_causal_conv1d_update_kernel`.  This file restates that kernel's one-token decode case:
 *   - a row whose cache line is the null block returns at once;
 *   - the window is the first width-1 tokens of the line plus the new token;
 *   - the accumulator starts at the bias as fp32 and takes the taps in order j = 0 .. width-1; the product of two
 *     values of one 16-bit type is a value of that type (Triton's typed multiply), otherwise it is an fp32 product
 *     that the compiler contracts with the sum;
 *   - SiLU is acc / (1 + exp(-acc)) in fp32; the result is stored in x's type;
 *   - the line's tokens move up by one and the new token goes last.
 * exp and the division are the C library's / IEEE here; Triton's are approximate instructions, so outputs agree
 * with the Triton kernel to the last bit of a 16-bit type almost always, not always.  The conv state is moved, not
 * computed, and must agree byte for byte.
 *
 * Parity pinned on the GPU against vLLM's own kernel (tests/test_conv_gpu.py), not by golden vectors: the op is a
 * Triton kernel and cannot run without a GPU.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "../include/statequant_b200.h"

static inline float c_f16(uint16_t h) {
  _Float16 x;
  memcpy(&x, &h, 2);
  return (float)x;
}
static inline uint16_t c_to_f16(float f) {
  _Float16 x = (_Float16)f;
  uint16_t h;
  memcpy(&h, &x, 2);
  return h;
}
static inline float c_bf16(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t c_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static inline float c_ld(const uint8_t *p, int dt) {
  if (dt == SQB_F32) {
    float f;
    memcpy(&f, p, 4);
    return f;
  }
  uint16_t h;
  memcpy(&h, p, 2);
  return dt == SQB_BF16 ? c_bf16(h) : c_f16(h);
}
static inline void c_st(uint8_t *p, int dt, float v) {
  if (dt == SQB_F32) {
    memcpy(p, &v, 4);
    return;
  }
  const uint16_t h = dt == SQB_BF16 ? c_to_bf16(v) : c_to_f16(v);
  memcpy(p, &h, 2);
}

int sqo_conv1d_update(const sqb_conv_update_t *a) {
  if (!a || a->width < 2 || a->width > 4 || a->state_len < a->width - 1) return SQB_EINVAL;
  const int es = a->x_dtype == SQB_F32 ? 4 : 2, ws = a->w_dtype == SQB_F32 ? 4 : 2;
  const int typed = es == 2 && ws == 2;                    /* both 16-bit (the same type): typed product */
  if (typed && a->x_dtype != a->w_dtype) return SQB_EINVAL;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < a->rows; r++) {
    const int64_t line = a->idx ? a->idx[r] : r;
    if (line < 0 || line == a->null_line) continue;
    const uint8_t *xr = (const uint8_t *)a->x + r * a->sx;
    uint8_t *orow = (uint8_t *)a->out + r * a->so;
    uint8_t *sl = (uint8_t *)a->state + line * a->s_line;
    for (int64_t c = 0; c < a->dim; c++) {
      uint8_t *sc = sl + c * a->s_dim;
      const uint8_t *wc = (const uint8_t *)a->w + c * a->sw_dim;
      uint8_t xnew[4];
      memcpy(xnew, xr + c * es, (size_t)es);               /* out may be x itself: keep the token's bits */
      float acc = a->bias ? c_ld((const uint8_t *)a->bias + c * ws, a->w_dtype) : 0.0f;
      for (int j = 0; j < a->width; j++) {
        const float xv = j == a->width - 1 ? c_ld(xnew, a->x_dtype) : c_ld(sc + j * a->s_tok, a->x_dtype);
        const float wv = c_ld(wc + j * a->sw_tap, a->w_dtype);
        if (typed) {
          float p = xv * wv;                                 /* exact in fp32 */
          p = a->x_dtype == SQB_BF16 ? c_bf16(c_to_bf16(p)) : c_f16(c_to_f16(p));
          acc = acc + p;
        } else {
          acc = fmaf(xv, wv, acc);
        }
      }
      for (int t = 0; t + 1 < a->state_len; t++) memcpy(sc + t * a->s_tok, sc + (t + 1) * a->s_tok, (size_t)es);
      memcpy(sc + (int64_t)(a->state_len - 1) * a->s_tok, xnew, (size_t)es);
      if (a->silu) acc = acc / (1.0f + expf(-acc));
      c_st(orow + c * es, a->x_dtype, acc);
    }
  }
  return 0;
}
