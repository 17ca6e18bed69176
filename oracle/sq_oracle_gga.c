/*
 * CPU oracle of the GGA / STEP mixed-bit state with the pure-write window.  TEST INFRASTRUCTURE ONLY (see
 * sq_oracle.c).  Restates, on host memory:
 *   STEP's dual-axis fit          src/statequant/step_quant.py:62-96   (torch `fit`; the device statement is
 *                                 src/statequant/kernels/_stepquant_triton.py:37-60)
 *   R_FP8 vectors                 src/statequant/methods_ext/gga.py:225-233   (`fp8_vec`)
 *   the decode step (Algorithm 1) src/statequant/integrations/vllm_gga.py:80-139 (`GGALayout.step`, the fp32
 *                                 emulation) == src/statequant/kernels/_gga_triton.py:207-308
 *   the packed byte layout        src/statequant/kernels/_gga_triton.py:3-13,47-96,105-142 and
 *                                 src/statequant/integrations/vllm_gga.py:169-205
 * The reference has no CPU packer for this layout (its packer is the Triton kernel): the byte order of the codes is
 * restated from the kernel source; values are pinned through fit() and the reference's torch window decoder.
 *
 * Head states are KEY-major here, [d_k, d_v], as in the reference's GGA code.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/statequant_b200.h"

static inline float g_f16_to_f32(uint16_t h) { _Float16 x; memcpy(&x, &h, 2); return (float)x; }
static inline uint16_t g_f32_to_f16(float f) { _Float16 x = (_Float16)f; uint16_t h; memcpy(&h, &x, 2); return h; }
static inline float g_bf16_to_f32(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
static inline uint16_t g_f32_to_bf16(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static inline float g_ld(const void *p, int dt, int64_t i) {
  if (dt == SQB_F32) return ((const float *)p)[i];
  if (dt == SQB_BF16) return g_bf16_to_f32(((const uint16_t *)p)[i]);
  return g_f16_to_f32(((const uint16_t *)p)[i]);
}
static inline void g_st(void *p, int dt, int64_t i, float v) {
  if (dt == SQB_F32) ((float *)p)[i] = v;
  else if (dt == SQB_BF16) ((uint16_t *)p)[i] = g_f32_to_bf16(v);
  else ((uint16_t *)p)[i] = g_f32_to_f16(v);
}
static inline int g_esz(int dt) { return dt == SQB_F32 ? 4 : 2; }

/* step_quant._half: clamp to [2^-24, 65504], round to fp16 */
static inline float halfc(float x) { return g_f16_to_f32(g_f32_to_f16(fminf(fmaxf(x, 5.960464477539063e-08f), 65504.f))); }

/* ---- E4M3 (fn) ------------------------------------------------------------------------------------------ */
/* value of |y| <= 448 rounded to the E4M3 grid, nearest even (spacing 2^(e-3), e >= -6) */
static inline float e4m3_round(float y) {
  if (y == 0.f) return y;
  int e;
  frexpf(fabsf(y), &e);          /* |y| = m 2^e, m in [0.5, 1) -> exponent e - 1 */
  e -= 1;
  if (e < -6) e = -6;
  const float ulp = ldexpf(1.f, e - 3);
  return rintf(y / ulp) * ulp;
}
static inline uint8_t e4m3_byte(float y) {      /* y on the grid, |y| <= 448 */
  uint8_t s = signbit(y) ? 0x80 : 0;
  float a = fabsf(y);
  if (a == 0.f) return s;
  int e;
  float m = frexpf(a, &e);       /* a = m 2^e, m in [0.5, 1) */
  e -= 1;                        /* a = (2m) 2^e */
  if (e < -6) {                  /* subnormal: a = k 2^-9 */
    return (uint8_t)(s | (uint8_t)lrintf(a * 512.f));
  }
  int mant = (int)lrintf((2.f * m - 1.f) * 8.f);
  return (uint8_t)(s | ((e + 7) << 3) | mant);
}
static inline float e4m3_val(uint8_t b) {
  int e = (b >> 3) & 15, m = b & 7;
  float v = e == 0 ? ldexpf((float)m, -9) : ldexpf(1.f + m / 8.f, e - 7);
  return (b & 0x80) ? -v : v;
}
/* fp8_vec of x[n]: codes, scale s = amax / 448 and the reconstruction */
static void fp8_vec(const float *x, int n, uint8_t *code, float *scale, float *rec) {
  float amax = 0.f;
  for (int i = 0; i < n; i++) amax = fmaxf(amax, fabsf(x[i]));
  const float s = amax / 448.f;
  const float safe = s > 0.f ? s : 1.f;
  for (int i = 0; i < n; i++) {
    float y = e4m3_round(fminf(fmaxf(x[i] / safe, -448.f), 448.f));
    if (code) code[i] = e4m3_byte(y);
    if (rec) rec[i] = s > 0.f ? y * safe : 0.f;
  }
  if (scale) *scale = s;
}

/* ---- STEP dual-axis fit of one head x[dk][dv] at width b with impact factors w[dk] ---------------------- */
/* out: r (dk, or dk * dv/group for 2 bits), c[dv], z[dk*dv] (signed levels); returns nothing for b == 16 */
static void fit_parts(const float *x, const float *w, int b, int dk, int dv, int group, float *r, float *c, float *z) {
  const int two = b == 2;
  const float qmax = two ? 3.f : (float)((1 << (b - 1)) - 1);
  const int ng = dv / group;
  float *y0 = (float *)malloc(sizeof(float) * (size_t)dk * dv);
  for (int k = 0; k < dk; k++) {
    if (two) {
      for (int g = 0; g < ng; g++) {
        double s = 0.;
        for (int j = 0; j < group; j++) s += fabsf(x[k * dv + g * group + j]);
        const float mg = (float)s * (1.f / group);
        r[k * ng + g] = halfc(sqrtf(fmaxf(mg, 1e-20f) / w[k]));
      }
    } else {
      double s = 0.;
      for (int v = 0; v < dv; v++) s += fabsf(x[k * dv + v]);
      const float mr = (float)s * (1.f / dv);
      r[k] = halfc(sqrtf(fmaxf(mr, 1e-20f) / w[k]));
    }
    for (int v = 0; v < dv; v++) y0[k * dv + v] = x[k * dv + v] / (two ? r[k * ng + v / group] : r[k]);
  }
#define ENC(y) (two ? ((y) >= 0.f ? 1.f : -1.f) * (fabsf(y) >= 2.f ? 3.f : 1.f) : fminf(fmaxf(rintf(y), -qmax), qmax))
  for (int v = 0; v < dv; v++) {
    float m = 0.f;
    for (int k = 0; k < dk; k++) m = fmaxf(m, fabsf(y0[k * dv + v]) / qmax);
    float cv = halfc(m);
    double num = 0., den = 0.;
    for (int k = 0; k < dk; k++) {
      const float zz = ENC(y0[k * dv + v] / cv);
      const float rf = two ? r[k * ng + v / group] : r[k];
      const float vv = rf * zz, ww = w[k] * w[k];
      num += (double)((ww * vv) * x[k * dv + v]);
      den += (double)(ww * (vv * vv));
    }
    const float nf = (float)num, df = (float)den;
    cv = halfc(df > 0.f ? nf / fmaxf(df, 1e-30f) : cv);
    c[v] = cv;
    for (int k = 0; k < dk; k++) z[k * dv + v] = ENC(y0[k * dv + v] / cv);
  }
#undef ENC
  free(y0);
}

/* fake-quant output of the fit: y = r c z (pivots: fp16 cast) */
static void fit_head(const float *x, const float *w, int b, int dk, int dv, int group, float *y) {
  if (b == 16) {
    for (int i = 0; i < dk * dv; i++) y[i] = g_f16_to_f32(g_f32_to_f16(x[i]));
    return;
  }
  const int ng = dv / group;
  float *r = (float *)malloc(sizeof(float) * ((size_t)dk * (b == 2 ? ng : 1) + dv + (size_t)dk * dv));
  float *c = r + (size_t)dk * (b == 2 ? ng : 1), *z = c + dv;
  fit_parts(x, w, b, dk, dv, group, r, c, z);
  for (int k = 0; k < dk; k++)
    for (int v = 0; v < dv; v++) y[k * dv + v] = ((b == 2 ? r[k * ng + v / group] : r[k]) * c[v]) * z[k * dv + v];
  free(r);
}

/* x, y fp32 [B, H, dk, dv]; bits int32 [H]; w fp32 [H, dk]   == step_quant.fit */
void sqo_stepquant_fit(const float *x, float *y, const int32_t *bits, const float *w, int64_t B, int H, int dk, int dv, int group) {
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t bh = 0; bh < B * H; bh++) {
    const int h = (int)(bh % H);
    fit_head(x + bh * (int64_t)dk * dv, w + (size_t)h * dk, bits[h], dk, dv, group, y + bh * (int64_t)dk * dv);
  }
}

/* ---- packed head: codes + factors (layout of _gga_triton.py:3-13) ---------------------------------------- */
static size_t gga_code_bytes(int b, int dk, int dv) { return (size_t)dk * dv * b / 8; }

static void pack_head_gga(uint8_t *S, const float *x, const float *w, int b, int dk, int dv, int group) {
  if (b == 16) {
    uint16_t *p = (uint16_t *)S;
    for (int i = 0; i < dk * dv; i++) p[i] = g_f32_to_f16(x[i]);
    return;
  }
  const int ng = dv / group, nr = b == 2 ? dk * ng : dk;
  float *r = (float *)malloc(sizeof(float) * ((size_t)nr + dv + (size_t)dk * dv));
  float *c = r + nr, *z = c + dv;
  fit_parts(x, w, b, dk, dv, group, r, c, z);
  const int qmax = (1 << (b - 1)) - 1;
  for (int k = 0; k < dk; k++) {
    uint8_t *row = S + (size_t)k * (dv * b / 8);
    if (b == 8) {
      for (int v = 0; v < dv; v++) row[v] = (uint8_t)((int)z[k * dv + v] + qmax);
    } else if (b == 4) {
      for (int j = 0; j < dv / 2; j++)
        row[j] = (uint8_t)(((int)z[k * dv + 2 * j] + qmax) | (((int)z[k * dv + 2 * j + 1] + qmax) << 4));
    } else if (b == 2) {
      for (int j = 0; j < dv / 4; j++) {
        int e[4];
        for (int t = 0; t < 4; t++) e[t] = (int)((z[k * dv + 4 * j + t] + 3.f) * 0.5f);
        row[j] = (uint8_t)(e[0] | (e[1] << 2) | (e[2] << 4) | (e[3] << 6));
      }
    } else { /* 6 bits: four codes per three bytes, little-endian */
      for (int j = 0; j < dv / 4; j++) {
        uint32_t wd = 0;
        for (int t = 0; t < 4; t++) wd |= (uint32_t)((int)z[k * dv + 4 * j + t] + qmax) << (6 * t);
        row[3 * j] = (uint8_t)(wd & 255); row[3 * j + 1] = (uint8_t)((wd >> 8) & 255); row[3 * j + 2] = (uint8_t)(wd >> 16);
      }
    }
  }
  uint16_t *R = (uint16_t *)(S + gga_code_bytes(b, dk, dv));
  for (int i = 0; i < nr; i++) R[i] = g_f32_to_f16(r[i]);
  uint16_t *C = R + nr;
  for (int v = 0; v < dv; v++) C[v] = g_f32_to_f16(c[v]);
  free(r);
}

static void unpack_head_gga(const uint8_t *S, int b, int dk, int dv, int group, float *x) {
  if (b == 16) {
    const uint16_t *p = (const uint16_t *)S;
    for (int i = 0; i < dk * dv; i++) x[i] = g_f16_to_f32(p[i]);
    return;
  }
  const int ng = dv / group, nr = b == 2 ? dk * ng : dk, qmax = (1 << (b - 1)) - 1;
  const uint16_t *R = (const uint16_t *)(S + gga_code_bytes(b, dk, dv));
  const uint16_t *C = R + nr;
  for (int k = 0; k < dk; k++) {
    const uint8_t *row = S + (size_t)k * (dv * b / 8);
    for (int v = 0; v < dv; v++) {
      float z;
      if (b == 8) z = (float)((int)row[v] - qmax);
      else if (b == 4) z = (float)((int)((row[v / 2] >> (4 * (v & 1))) & 15) - qmax);
      else if (b == 2) z = (float)((row[v / 4] >> (2 * (v & 3))) & 3) * 2.f - 3.f;
      else {
        const uint8_t *t = row + 3 * (v / 4);
        const uint32_t wd = t[0] | (t[1] << 8) | (t[2] << 16);
        z = (float)((int)((wd >> (6 * (v & 3))) & 63) - qmax);
      }
      const float rf = g_f16_to_f32(b == 2 ? R[k * ng + v / group] : R[k]);
      x[k * dv + v] = (rf * g_f16_to_f32(C[v])) * z;
    }
  }
}

/*
 * The GGA slot table of one layer (mirrors sqb_gga_layout_t of the C ABI; host pointers here).
 */
int sqo_gga_store(const sqb_gga_layout_t *L, const int32_t *idx, int64_t P, const float *X) {
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t ph = 0; ph < P * L->hv; ph++) {
    const int64_t seq = idx[ph / L->hv];
    const int h = (int)(ph % L->hv);
    uint8_t *base = (uint8_t *)L->blob + seq * L->stride;
    pack_head_gga(base + L->offs[h], X + ph * (int64_t)L->dk * L->dv, L->w + (size_t)h * L->dk, L->bits[h], L->dk, L->dv, L->group);
    if (h == 0) { ((int32_t *)base)[0] = 0; ((int32_t *)base)[1] = 0; }
  }
  return 0;
}

int sqo_gga_load(const sqb_gga_layout_t *L, const int32_t *idx, int64_t P, float *Y) {
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t ph = 0; ph < P * L->hv; ph++) {
    const int64_t seq = idx[ph / L->hv];
    const int h = (int)(ph % L->hv);
    const uint8_t *base = (const uint8_t *)L->blob + seq * L->stride;
    unpack_head_gga(base + L->offs[h], L->bits[h], L->dk, L->dv, L->group, Y + ph * (int64_t)L->dk * L->dv);
  }
  return 0;
}

/* one decode token on the packed slots (step + counter advance) */
int sqo_gga_step(const sqb_gga_layout_t *L, const sqb_gdn_inputs_t *in) {
  const int hv = L->hv, hk = L->hk, dk = L->dk, dv = L->dv, M = L->m, gqa = hv / hk;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t bh = 0; bh < (int64_t)in->rows * hv; bh++) {
    const int64_t b = bh / hv;
    const int h = (int)(bh % hv), hkk = h / gqa;
    void *orow = (uint8_t *)in->out + b * in->so + (size_t)h * dv * g_esz(in->out_dtype);
    const int64_t seq = in->idx[b];
    if (seq <= 0) { memset(orow, 0, (size_t)dv * g_esz(in->out_dtype)); continue; }
    uint8_t *base = (uint8_t *)L->blob + seq * L->stride;
    float *buf = (float *)malloc(sizeof(float) * (4 * (size_t)dk + 3 * (size_t)dv + 2 * (size_t)dk * dv + (size_t)M * (dk + dv)));
    float *q = buf, *k = q + dk, *bk = k + dk, *tmpk = bk + dk, *v = tmpk + dk, *o = v + dv, *kO = o + dv;
    float *St = kO + dv, *Om = St + (size_t)dk * dv, *Pw = Om + (size_t)dk * dv, *Vw = Pw + (size_t)M * dk;
    /* q, k: l2-normalised (rsqrt form of the emulation is the same value up to rounding; the kernel divides) */
    double sq = 0., sk = 0.;
    for (int i = 0; i < dk; i++) {
      q[i] = g_ld((const uint8_t *)in->q + b * in->sq, in->qk_dtype, (int64_t)hkk * dk + i);
      k[i] = g_ld((const uint8_t *)in->k + b * in->sk, in->qk_dtype, (int64_t)hkk * dk + i);
      sq += (double)q[i] * q[i];
      sk += (double)k[i] * k[i];
    }
    const float nq = sqrtf((float)sq + 1e-6f), nk = sqrtf((float)sk + 1e-6f);
    for (int i = 0; i < dk; i++) { q[i] = q[i] / nq * in->scale; k[i] = k[i] / nk; }
    const float x = g_ld((const uint8_t *)in->a + b * in->sa, in->ab_dtype, h) + g_ld(in->dt_bias, in->dtb_dtype, h);
    const float sp = x <= 20.f ? logf(1.f + expf(x)) : x;
    const float a = expf(-expf(g_ld(in->A_log, in->alog_dtype, h)) * sp);
    const float beta = 1.f / (1.f + expf(-g_ld((const uint8_t *)in->b + b * in->sb, in->ab_dtype, h)));
    for (int i = 0; i < dv; i++) v[i] = g_ld((const uint8_t *)in->v + b * in->sv, in->v_dtype, (int64_t)h * dv + i);
    const int bits = L->bits[h];
    uint8_t *S = base + L->offs[h];
    unpack_head_gga(S, bits, dk, dv, L->group, St);
    for (int j = 0; j < dv; j++) {
      double s = 0.;
      for (int i = 0; i < dk; i++) s += (double)(k[i] * St[i * dv + j]);
      kO[j] = (float)s;
    }
    double bq = 0.;
    for (int i = 0; i < dk; i++) { bk[i] = beta * k[i]; bq += (double)(bk[i] * q[i]); }
    for (int i = 0; i < dk; i++)
      for (int j = 0; j < dv; j++) St[i * dv + j] = a * (St[i * dv + j] - bk[i] * kO[j]);       /* AO */
    for (int j = 0; j < dv; j++) {
      double s = 0.;
      for (int i = 0; i < dk; i++) s += (double)(St[i * dv + j] * q[i]);
      o[j] = (float)s + (float)bq * v[j];
    }
    if (L->pw && bits != 16) {
      const int32_t *ct = (const int32_t *)base;
      const int n = ct[0], hd = ct[1];
      uint8_t *qb = base + L->qoff + (size_t)h * L->qsz;
      uint8_t *PP = qb, *VP = qb + (size_t)M * dk;
      float *PS = (float *)(qb + (size_t)M * (dk + dv)), *VS = PS + M;
      float r0s = 0.f;
      (void)r0s;
      memcpy(Om, St, sizeof(float) * (size_t)dk * dv);
      for (int i = 0; i < M && i < n; i++) {
        const int jj = (hd + i) % M;
        double kp = 0.;
        for (int t = 0; t < dk; t++) { Pw[t] = e4m3_val(PP[jj * dk + t]) * PS[jj]; kp += (double)(k[t] * Pw[t]); }
        for (int t = 0; t < dv; t++) Vw[t] = e4m3_val(VP[jj * dv + t]) * VS[jj];
        for (int t = 0; t < dk; t++) tmpk[t] = a * (Pw[t] - bk[t] * (float)kp);                    /* A p */
        float sc;
        fp8_vec(tmpk, dk, PP + jj * dk, &sc, Pw);                                                /* R(A p), stored */
        PS[jj] = sc;
        double cf = 0.;
        for (int t = 0; t < dk; t++) cf += (double)(Pw[t] * q[t]);
        for (int t = 0; t < dv; t++) o[t] += (float)cf * Vw[t];
        if (i == 0 && n == M)                                                                     /* evicted pair */
          for (int t = 0; t < dk; t++)
            for (int j = 0; j < dv; j++) Om[t * dv + j] = St[t * dv + j] + Pw[t] * Vw[j];
      }
      const int jn = n < M ? (hd + n) % M : hd;
      float sc;
      fp8_vec(bk, dk, PP + jn * dk, &sc, NULL);
      PS[jn] = sc;
      fp8_vec(v, dv, VP + jn * dv, &sc, NULL);
      VS[jn] = sc;
    } else {
      for (int i = 0; i < dk; i++)
        for (int j = 0; j < dv; j++) Om[i * dv + j] = St[i * dv + j] + bk[i] * v[j];
    }
    for (int j = 0; j < dv; j++) g_st(orow, in->out_dtype, j, o[j]);
    pack_head_gga(S, Om, L->w + (size_t)h * dk, bits, dk, dv, L->group);
    free(buf);
  }
  if (L->pw) {
    for (int64_t b = 0; b < in->rows; b++) {       /* counters move after every head has read them */
      const int64_t seq = in->idx[b];
      if (seq <= 0) continue;
      int done = 0;
      for (int64_t b2 = 0; b2 < b; b2++) done |= in->idx[b2] == seq;
      if (done) continue;
      int32_t *ct = (int32_t *)((uint8_t *)L->blob + seq * L->stride);
      const int n = ct[0], hd = ct[1];
      ct[0] = n + 1 < M ? n + 1 : M;
      ct[1] = n == M ? (hd + 1) % M : hd;
    }
  }
  return 0;
}
