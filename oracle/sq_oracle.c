/*
 * CPU oracle of the packed-state decode step.  TEST INFRASTRUCTURE ONLY: nothing in the product path may call
 * into this file; it exists so that tests/, the smoke check and the benchmark's CPU-baseline leg have an
 * independent statement of the arithmetic to compare the CUDA kernels with.
 *
 * It restates, in plain C on host memory, the reference's torch implementation of the path
 * (HallerPatrick/StateQuant, paths inside that project):
 *   pack / unpack            src/statequant/kernels/fold.py:123-173   (Quantizer.fake with fp16 scales,
 *                            src/statequant/quantizer.py:159-193)
 *   buffer rounding          src/statequant/kernels/fold.py:181-191
 *   Gated DeltaNet step/fold src/statequant/kernels/fold.py:233-274   (ReferenceGDNState)
 *   Mamba2 step/fold         src/statequant/kernels/mamba2.py:45-54,176-217 (ReferenceMamba2State)
 *   KDA step/fold            src/statequant/kernels/kda.py:152-186    (ReferenceKDAState)
 *   slot read / write        src/statequant/kernels/slots.py:210-252, kda.py:351-386
 * on the byte layout of src/statequant/kernels/slots.py:76-95.  The reference keeps a dequantised fp32 shadow
 * of the stored state and float copies of the buffered vectors; here the same values are re-derived from the
 * stored codes each time (code * fp16 scale is exact in fp32, so the two are the same numbers).
 *
 * Arithmetic conventions: fp32 everywhere the reference is fp32, separate multiply and add (compile with
 * -ffp-contract=off), round-half-even (rintf), IEEE division and square root.  Sums over d_k, d_v or the
 * buffer slots are accumulated in double and rounded once: the reference leaves their order to torch's
 * vectorised kernels, so no fp32 summation order is canonical.  The fold accumulates slot by slot in fp32 in
 * the reference's order (fold.py:268-269).
 *
 * Parity is pinned against golden vectors produced by the reference itself (tests/golden/).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/statequant_b200.h"

#define FP16_TINY 5.960464477539063e-08f

/* ------------------------------------------------------------------------------------------------------ */
/* scalar conversions                                                                                     */
/* ------------------------------------------------------------------------------------------------------ */
static inline float f16_to_f32(uint16_t h) {
  _Float16 x;
  memcpy(&x, &h, 2);
  return (float)x;
}
static inline uint16_t f32_to_f16(float f) {
  _Float16 x = (_Float16)f; /* round to nearest even, overflow -> inf */
  uint16_t h;
  memcpy(&h, &x, 2);
  return h;
}
static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);                                          /* nearest even */
  return (uint16_t)(u >> 16);
}
static inline float ld(const void *p, int dt, int64_t i) {
  if (dt == SQB_F32) return ((const float *)p)[i];
  if (dt == SQB_BF16) return bf16_to_f32(((const uint16_t *)p)[i]);
  return f16_to_f32(((const uint16_t *)p)[i]);
}
static inline void st_out(void *p, int dt, int64_t i, float v) {
  if (dt == SQB_F32) ((float *)p)[i] = v;
  else if (dt == SQB_BF16) ((uint16_t *)p)[i] = f32_to_bf16(v);
  else ((uint16_t *)p)[i] = f32_to_f16(v);
}
static inline int esz(int dt) { return dt == SQB_F32 ? 4 : 2; }

/* Quantizer._cast_scale with scale_dtype='fp16' (quantizer.py:159-164) after amax.clamp_min(1e-8) / qmax */
static inline float fp16_scale(float amax, float qmax) {
  float s = fmaxf(amax, 1e-8f) / qmax;
  s = f16_to_f32(f32_to_f16(s));
  return fmaxf(s, FP16_TINY);
}
static inline float rclamp(float x, float s, float qmax) {
  float c = rintf(x / s);
  return fminf(fmaxf(c, -qmax), qmax);
}

/* ------------------------------------------------------------------------------------------------------ */
/* pack / unpack of one head, value-major [DV, DK]  (fold.py:123-173)                                     */
/* ------------------------------------------------------------------------------------------------------ */
static int n_groups_k(int dk, int g) { return (dk + g - 1) / g; }

static void pack_head(const float *x, int dv, int dk, int bits, int axis_k, int group, uint8_t *codes,
                      uint16_t *scales) {
  if (bits == 16) {
    uint16_t *c = (uint16_t *)codes;
    for (int i = 0; i < dv * dk; i++) c[i] = f32_to_bf16(x[i]);
    return;
  }
  if (bits == 32) {
    memcpy(codes, x, (size_t)dv * dk * 4);
    return;
  }
  const float qmax = (float)((1 << (bits - 1)) - 1);
  int8_t *tmp = (int8_t *)malloc((size_t)dv * dk);
  if (axis_k) {
    int ng = n_groups_k(dk, group);
    for (int v = 0; v < dv; v++)
      for (int gi = 0; gi < ng; gi++) {
        int k0 = gi * group, k1 = k0 + group < dk ? k0 + group : dk;
        float amax = 0.f;
        for (int k = k0; k < k1; k++) amax = fmaxf(amax, fabsf(x[v * dk + k]));
        float s = fp16_scale(amax, qmax);
        scales[v * ng + gi] = f32_to_f16(s);
        for (int k = k0; k < k1; k++) tmp[v * dk + k] = (int8_t)rclamp(x[v * dk + k], s, qmax);
      }
  } else {
    for (int gv = 0; gv < dv / group; gv++)
      for (int k = 0; k < dk; k++) {
        float amax = 0.f;
        for (int r = 0; r < group; r++) amax = fmaxf(amax, fabsf(x[(gv * group + r) * dk + k]));
        float s = fp16_scale(amax, qmax);
        scales[gv * dk + k] = f32_to_f16(s);
        for (int r = 0; r < group; r++) {
          int v = gv * group + r;
          tmp[v * dk + k] = (int8_t)rclamp(x[v * dk + k], s, qmax);
        }
      }
  }
  if (bits == 4) {
    for (int v = 0; v < dv; v++)
      for (int j = 0; j < dk / 2; j++)
        codes[v * (dk / 2) + j] =
            (uint8_t)((tmp[v * dk + 2 * j] + 8) | ((tmp[v * dk + 2 * j + 1] + 8) << 4));
  } else {
    memcpy(codes, tmp, (size_t)dv * dk);
  }
  free(tmp);
}

static void unpack_head(const uint8_t *codes, const uint16_t *scales, int dv, int dk, int bits, int axis_k,
                        int group, float *x) {
  if (bits == 16) {
    const uint16_t *c = (const uint16_t *)codes;
    for (int i = 0; i < dv * dk; i++) x[i] = bf16_to_f32(c[i]);
    return;
  }
  if (bits == 32) {
    memcpy(x, codes, (size_t)dv * dk * 4);
    return;
  }
  int ng = n_groups_k(dk, group);
  for (int v = 0; v < dv; v++)
    for (int k = 0; k < dk; k++) {
      float c;
      if (bits == 4) {
        uint8_t by = codes[v * (dk / 2) + k / 2];
        c = (float)((k & 1) ? (by >> 4) : (by & 15)) - 8.f;
      } else {
        c = (float)((const int8_t *)codes)[v * dk + k];
      }
      float s = axis_k ? f16_to_f32(scales[v * ng + k / group]) : f16_to_f32(scales[(v / group) * dk + k]);
      x[v * dk + k] = s * c;
    }
}

/* [BH, DV, DK] fp32 -> codes, scales (contiguous per head)  == pack_vk */
void sqo_pack_vk(const float *x, int64_t bh, int dv, int dk, int bits, int axis_k, int group, void *codes,
                 void *scales) {
  size_t cb = bits == 4 ? (size_t)dv * dk / 2 : (size_t)dv * dk * (bits / 8);
  size_t sn = (bits == 4 || bits == 8) ? (axis_k ? (size_t)dv * n_groups_k(dk, group) : (size_t)(dv / group) * dk) : 0;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < bh; i++)
    pack_head(x + i * (int64_t)dv * dk, dv, dk, bits, axis_k, group, (uint8_t *)codes + i * cb,
              (uint16_t *)scales + i * sn);
}

/* inverse == unpack_vk */
void sqo_unpack_vk(const void *codes, const void *scales, int64_t bh, int dv, int dk, int bits, int axis_k,
                   int group, float *x) {
  size_t cb = bits == 4 ? (size_t)dv * dk / 2 : (size_t)dv * dk * (bits / 8);
  size_t sn = (bits == 4 || bits == 8) ? (axis_k ? (size_t)dv * n_groups_k(dk, group) : (size_t)(dv / group) * dk) : 0;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < bh; i++)
    unpack_head((const uint8_t *)codes + i * cb, (const uint16_t *)scales + i * sn, dv, dk, bits, axis_k,
                group, x + i * (int64_t)dv * dk);
}

/* ------------------------------------------------------------------------------------------------------ */
/* the step                                                                                               */
/* ------------------------------------------------------------------------------------------------------ */
enum { KIND_GDN = 0, KIND_M2 = 1, KIND_KDA = 2 };

typedef struct {
  int kind;
  const float *xq;   /* [DK] read-out vector: normalised scaled q (GDN, KDA) or C (Mamba2)             */
  const float *xk;   /* [DK] normalised k (GDN, KDA); NULL for Mamba2                                   */
  const float *kx;   /* [DK] the key that goes into the buffer (GDN: the key head's k; Mamba2: B)       */
  const float *vin;  /* [DV] v (GDN, KDA) or x (Mamba2)                                                 */
  const float *gv;   /* KDA: [DK] log decay of this token                                               */
  float g;           /* GDN, Mamba2: log decay                                                          */
  float beta, dt, D; /* beta (GDN, KDA); dt and D (Mamba2)                                              */
  int has_D;
  float kq;          /* k . q  (Mamba2: B . C)                                                          */
  int write_key;     /* this head stores the buffered key (first value head of its key head)            */
} head_in_t;

static inline size_t code_bytes(const sqb_state_t *st) {
  return st->bits == 4 ? (size_t)st->dv * st->dk / 2 : (size_t)st->dv * st->dk * (st->bits / 8);
}
static inline size_t scale_count(const sqb_state_t *st) {
  if (st->bits > 8) return 0;
  return st->axis_k ? (size_t)st->dv * n_groups_k(st->dk, st->group) : (size_t)(st->dv / st->group) * st->dk;
}

/* buffered vector i of a table: dequantised into out[len] */
static void load_buf(const void *base, const void *sbase, int qbuf, int i, int len, float *out) {
  if (qbuf) {
    const int8_t *p = (const int8_t *)base + (size_t)i * len;
    float s = f16_to_f32(((const uint16_t *)sbase)[i]);
    for (int j = 0; j < len; j++) out[j] = (float)p[j] * s;
  } else {
    const uint16_t *p = (const uint16_t *)base + (size_t)i * len;
    for (int j = 0; j < len; j++) out[j] = bf16_to_f32(p[j]);
  }
}

/* _round_buf (fold.py:186-191) of x[len] into slot i of a table; deq[len] receives the rounded values */
static void store_buf(void *base, void *sbase, int qbuf, int i, int len, const float *x, float *deq, int do_store) {
  if (qbuf) {
    float amax = 0.f;
    for (int j = 0; j < len; j++) amax = fmaxf(amax, fabsf(x[j]));
    float s = fp16_scale(amax, 127.f);
    int8_t *p = (int8_t *)base + (size_t)i * len;
    for (int j = 0; j < len; j++) {
      float c = rclamp(x[j], s, 127.f);
      if (do_store) p[j] = (int8_t)c;
      deq[j] = c * s;
    }
    if (do_store) ((uint16_t *)sbase)[i] = f32_to_f16(s);
  } else {
    uint16_t *p = (uint16_t *)base + (size_t)i * len;
    for (int j = 0; j < len; j++) {
      uint16_t b = f32_to_bf16(x[j]);
      if (do_store) p[j] = b;
      deq[j] = bf16_to_f32(b);
    }
  }
}

static void step_head(const sqb_state_t *st, int64_t seq, int h, const head_in_t *in, void *out, int out_dt) {
  const int dk = st->dk, dv = st->dv, M = st->m, kind = in->kind;
  const int gqa = st->hv / st->hk, hk = h / gqa, qbuf = st->buffer_bits == 8;
  const int bsz = qbuf ? 1 : 2;
  uint8_t *S = (uint8_t *)st->S + seq * st->sS + (size_t)h * code_bytes(st);
  uint16_t *SC = st->bits <= 8 ? (uint16_t *)((uint8_t *)st->SC + seq * st->sSC) + (size_t)h * scale_count(st) : NULL;
  uint8_t *KB = (uint8_t *)st->KB + seq * st->sKB + (size_t)hk * M * dk * bsz;
  uint8_t *UB = (uint8_t *)st->UB + seq * st->sUB + (size_t)h * M * dv * bsz;
  uint16_t *KBS = qbuf ? (uint16_t *)((uint8_t *)st->KBS + seq * st->sKBS) + (size_t)hk * M : NULL;
  uint16_t *UBS = qbuf ? (uint16_t *)((uint8_t *)st->UBS + seq * st->sUBS) + (size_t)h * M : NULL;
  const int gw = kind == KIND_KDA ? dk : 1;              /* width of one decay entry */
  float *GB = (float *)((uint8_t *)st->GB + seq * st->sGB) + (size_t)h * M * gw;
  float *GCUR = (float *)((uint8_t *)st->GCUR + seq * st->sGC) + (size_t)h * gw;
  int32_t *NP = (int32_t *)((uint8_t *)st->NPTR + seq * st->sN) + h;
  const int n = *NP & (M - 1);

  float *S0 = (float *)malloc(sizeof(float) * ((size_t)dv * dk + (size_t)M * dk + (size_t)M * dv + 6 * (size_t)dk + 3 * (size_t)dv + 4 * (size_t)M));
  float *Kb = S0 + (size_t)dv * dk;      /* [M, DK] buffered keys (KDA: times their decay ratio) */
  float *Ub = Kb + (size_t)M * dk;       /* [M, DV] */
  float *gnew = Ub + (size_t)M * dv;     /* [DK] (KDA) */
  float *Aexp = gnew + dk;               /* [DK] (KDA) */
  float *aq = Aexp + dk, *ak = aq + dk;  /* [DK] A*q, A*k (KDA) */
  float *knew = ak + dk;                 /* [DK] rounded new key */
  float *tmpk = knew + dk;
  float *u = tmpk + dk, *unew = u + dv, *sqv = unew + dv; /* [DV] */
  float *cq = sqv + dv, *ck = cq + M, *dec = ck + M;

  unpack_head(S, SC, dv, dk, st->bits, st->axis_k, st->group, S0);
  for (int i = 0; i < n; i++) {
    load_buf(KB, KBS, qbuf, i, dk, Kb + (size_t)i * dk);
    load_buf(UB, UBS, qbuf, i, dv, Ub + (size_t)i * dv);
  }

  float alpha = 1.f, a = 1.f, gcur_s = 0.f, gnew_s = 0.f;
  const float *rq = in->xq, *rk = in->xk;
  if (kind == KIND_KDA) {
    for (int k = 0; k < dk; k++) {
      gnew[k] = GCUR[k] + in->gv[k];
      Aexp[k] = expf(gnew[k]);
      aq[k] = Aexp[k] * in->xq[k];
      ak[k] = Aexp[k] * in->xk[k];
    }
    rq = aq;
    rk = ak;
    for (int i = 0; i < n; i++)         /* Kd_i = K_i * exp(gnew - G_i)   (kda.py:163) */
      for (int k = 0; k < dk; k++) Kb[(size_t)i * dk + k] = Kb[(size_t)i * dk + k] * expf(gnew[k] - GB[(size_t)i * dk + k]);
  } else {
    gcur_s = GCUR[0];
    alpha = expf(gcur_s);
    a = expf(in->g);
    gnew_s = gcur_s + in->g;
  }
  /* buffer coefficients */
  for (int i = 0; i < n; i++) {
    double dq = 0., dkk = 0.;
    for (int k = 0; k < dk; k++) {
      dq += (double)Kb[(size_t)i * dk + k] * (double)in->xq[k];
      if (in->xk) dkk += (double)Kb[(size_t)i * dk + k] * (double)in->xk[k];
    }
    if (kind == KIND_KDA) {
      cq[i] = (float)dq;
      ck[i] = (float)dkk;
    } else {
      float d = expf(gcur_s - GB[i]);
      cq[i] = d * (float)dq;
      ck[i] = d * (float)dkk;
    }
  }
  /* rows */
  for (int v = 0; v < dv; v++) {
    double dq = 0., dkk = 0.;
    const float *row = S0 + (size_t)v * dk;
    for (int k = 0; k < dk; k++) {
      dq += (double)row[k] * (double)rq[k];
      if (rk) dkk += (double)row[k] * (double)rk[k];
    }
    float sq = (float)dq, sk = (float)dkk;
    if (kind != KIND_KDA) {
      sq = alpha * sq;
      sk = alpha * sk;
    }
    if (n) {
      double bq = 0., bk = 0.;
      for (int i = 0; i < n; i++) {
        bq += (double)cq[i] * (double)Ub[(size_t)i * dv + v];
        bk += (double)ck[i] * (double)Ub[(size_t)i * dv + v];
      }
      sq = sq + (float)bq;
      sk = sk + (float)bk;
    }
    float o;
    if (kind == KIND_GDN) {
      u[v] = in->beta * (in->vin[v] - a * sk);
      o = a * sq + in->kq * u[v];
    } else if (kind == KIND_KDA) {
      u[v] = in->beta * (in->vin[v] - sk);
      o = sq + in->kq * u[v];
    } else {
      u[v] = in->dt * in->vin[v];
      o = a * sq + in->kq * u[v];
      if (in->has_D) o = o + in->D * in->vin[v];
    }
    st_out(out, out_dt, v, o);
  }
  /* append at slot n */
  store_buf(UB, UBS, qbuf, n, dv, u, unew, 1);
  store_buf(KB, KBS, qbuf, n, dk, in->kx, knew, in->write_key);
  if (kind == KIND_KDA) {
    for (int k = 0; k < dk; k++) GB[(size_t)n * dk + k] = gnew[k];
  } else {
    GB[n] = gnew_s;
  }
  const int full = n == M - 1;
  if (full) {
    /* fold: S = decay * S0 + sum_i (decayed k_i) u_i^T in slot order, then re-round (fold.py:263-274) */
    memcpy(Kb + (size_t)n * dk, knew, sizeof(float) * dk);
    memcpy(Ub + (size_t)n * dv, unew, sizeof(float) * dv);
    if (kind == KIND_KDA) {
      /* the new key's ratio is exp(0) = 1; S = diag(A) S0 */
      for (int v = 0; v < dv; v++)
        for (int k = 0; k < dk; k++) S0[(size_t)v * dk + k] = Aexp[k] * S0[(size_t)v * dk + k];
      for (int i = 0; i < M; i++)
        for (int v = 0; v < dv; v++) {
          float uu = Ub[(size_t)i * dv + v];
          for (int k = 0; k < dk; k++) S0[(size_t)v * dk + k] = S0[(size_t)v * dk + k] + uu * Kb[(size_t)i * dk + k];
        }
    } else {
      float an = expf(gnew_s);
      for (int i = 0; i < M; i++) dec[i] = expf(gnew_s - (i == n ? gnew_s : GB[i]));
      for (size_t e = 0; e < (size_t)dv * dk; e++) S0[e] = an * S0[e];
      for (int i = 0; i < M; i++)
        for (int v = 0; v < dv; v++) {
          float du = dec[i] * Ub[(size_t)i * dv + v];
          for (int k = 0; k < dk; k++) S0[(size_t)v * dk + k] = S0[(size_t)v * dk + k] + Kb[(size_t)i * dk + k] * du;
        }
    }
    pack_head(S0, dv, dk, st->bits, st->axis_k, st->group, S, SC);
  }
  if (kind == KIND_KDA) {
    for (int k = 0; k < dk; k++) GCUR[k] = full ? 0.f : gnew[k];
  } else {
    GCUR[0] = full ? 0.f : gnew_s;
  }
  *NP = full ? 0 : n + 1;
  free(S0);
}

static void zero_row(void *out, int dt, int n) { memset(out, 0, (size_t)n * esz(dt)); }

static void l2norm(const void *p, int dt, int64_t off, int dk, float mul, float *dst) {
  double ss = 0.;
  for (int k = 0; k < dk; k++) {
    float x = ld(p, dt, off + k);
    ss += (double)x * (double)x;
  }
  float nrm = sqrtf((float)ss + 1e-6f);
  for (int k = 0; k < dk; k++) dst[k] = ld(p, dt, off + k) / nrm * mul;
}


int sqo_gdn_step(const sqb_state_t *st, const sqb_gdn_inputs_t *in) {
  const int hv = st->hv, hk = st->hk, dk = st->dk, dv = st->dv, gqa = hv / hk;
  const int64_t total = (int64_t)in->rows * hv;
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t bh = 0; bh < total; bh++) {
    const int64_t b = bh / hv;
    const int h = (int)(bh % hv), hkk = h / gqa;
    void *orow = (uint8_t *)in->out + b * in->so + (size_t)h * dv * esz(in->out_dtype);
    const int64_t seq = in->idx ? in->idx[b] : b;
    if (in->idx && seq <= 0) {
      zero_row(orow, in->out_dtype, dv);
      continue;
    }
    float *buf = (float *)malloc(sizeof(float) * (3 * (size_t)dk + dv));
    float *qn = buf, *kn = qn + dk, *kx = kn + dk, *vv = kx + dk;
    const int hq = in->qk_per_key_head ? hkk : h;
    const uint8_t *qrow = (const uint8_t *)in->q + b * in->sq, *krow = (const uint8_t *)in->k + b * in->sk;
    l2norm(qrow, in->qk_dtype, (int64_t)hq * dk, dk, in->scale, qn);
    l2norm(krow, in->qk_dtype, (int64_t)hq * dk, dk, 1.f, kn);
    if (in->qk_per_key_head || gqa == 1) memcpy(kx, kn, sizeof(float) * dk);
    else l2norm(krow, in->qk_dtype, (int64_t)(hkk * gqa) * dk, dk, 1.f, kx);
    for (int v = 0; v < dv; v++) vv[v] = ld((const uint8_t *)in->v + b * in->sv, in->v_dtype, (int64_t)h * dv + v);
    head_in_t hi;
    memset(&hi, 0, sizeof hi);
    hi.kind = KIND_GDN;
    hi.xq = qn; hi.xk = kn; hi.kx = kx; hi.vin = vv;
    if (in->gate) {
      /* g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b): the packed step's in-kernel gating
         (src/statequant/kernels/_fused_triton.py:96-100) */
      float x = ld((const uint8_t *)in->a + b * in->sa, in->ab_dtype, h) + ld(in->dt_bias, in->dtb_dtype, h);
      float sp = x <= 20.f ? logf(1.f + expf(x)) : x;
      hi.g = -expf(ld(in->A_log, in->alog_dtype, h)) * sp;
      float bb = ld((const uint8_t *)in->b + b * in->sb, in->ab_dtype, h);
      hi.beta = 1.f / (1.f + expf(-bb));
    } else {
      hi.g = ld((const uint8_t *)in->g + b * in->sg, in->gb_dtype, h);
      hi.beta = ld((const uint8_t *)in->beta + b * in->sbeta, in->gb_dtype, h);
    }
    /* (kn * qn).sum(-1): products in fp32, summed */
    double kq = 0.;
    for (int k = 0; k < dk; k++) kq += (double)(kn[k] * qn[k]);
    hi.kq = (float)kq;
    hi.write_key = (h % gqa) == 0;
    step_head(st, seq, h, &hi, orow, in->out_dtype);
    free(buf);
  }
  return 0;
}

int sqo_mamba2_step(const sqb_state_t *st, const sqb_mamba2_inputs_t *in) {
  const int hv = st->hv, hk = st->hk, dk = st->dk, dv = st->dv, gqa = hv / hk;
  const int64_t total = (int64_t)in->rows * hv;
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t bh = 0; bh < total; bh++) {
    const int64_t b = bh / hv;
    const int h = (int)(bh % hv), hkk = h / gqa;
    void *orow = (uint8_t *)in->out + b * in->so + (size_t)h * dv * esz(in->out_dtype);
    const int64_t seq = in->idx ? in->idx[b] : b;
    if (in->idx && seq <= 0) {
      zero_row(orow, in->out_dtype, dv);
      continue;
    }
    float *buf = (float *)malloc(sizeof(float) * (2 * (size_t)dk + dv));
    float *c = buf, *bx = c + dk, *xv = bx + dk;
    for (int k = 0; k < dk; k++) {
      c[k] = ld((const uint8_t *)in->C + b * in->sC, in->bc_dtype, (int64_t)hkk * dk + k);
      bx[k] = ld((const uint8_t *)in->B + b * in->sB, in->bc_dtype, (int64_t)hkk * dk + k);
    }
    for (int v = 0; v < dv; v++) xv[v] = ld((const uint8_t *)in->x + b * in->sx, in->x_dtype, (int64_t)h * dv + v);
    /* _gate (mamba2.py:45-54) */
    float dt = ld((const uint8_t *)in->dt + b * in->sdt, in->dt_dtype, h);
    if (in->dt_bias) dt = dt + ld(in->dt_bias, in->dtb_dtype, h);
    if (in->dt_softplus) dt = dt <= 20.f ? logf(1.f + expf(dt)) : dt;
    if (in->dt_clamp) dt = fminf(fmaxf(dt, in->dt_min), in->dt_max);
    head_in_t hi;
    memset(&hi, 0, sizeof hi);
    hi.kind = KIND_M2;
    hi.xq = c; hi.xk = NULL; hi.kx = bx; hi.vin = xv;
    hi.dt = dt;
    hi.g = ld(in->A, in->a_dtype, h) * dt;
    hi.has_D = in->D != NULL;
    hi.D = in->D ? ld(in->D, in->d_dtype, h) : 0.f;
    double bc = 0.;
    for (int k = 0; k < dk; k++) bc += (double)(bx[k] * c[k]);
    hi.kq = (float)bc;
    hi.write_key = (h % gqa) == 0;
    step_head(st, seq, h, &hi, orow, in->out_dtype);
    free(buf);
  }
  return 0;
}

int sqo_kda_step(const sqb_state_t *st, const sqb_kda_inputs_t *in) {
  const int hv = st->hv, dk = st->dk, dv = st->dv;
  const int64_t total = (int64_t)in->rows * hv;
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t bh = 0; bh < total; bh++) {
    const int64_t b = bh / hv;
    const int h = (int)(bh % hv);
    void *orow = (uint8_t *)in->out + b * in->so + (size_t)h * dv * esz(in->out_dtype);
    const int64_t seq = in->idx ? in->idx[b] : b;
    if (in->idx && seq <= 0) {
      zero_row(orow, in->out_dtype, dv);
      continue;
    }
    float *buf = (float *)malloc(sizeof(float) * (3 * (size_t)dk + dv));
    float *qn = buf, *kn = qn + dk, *gv = kn + dk, *vv = gv + dk;
    l2norm((const uint8_t *)in->q + b * in->sq, in->qk_dtype, (int64_t)h * dk, dk, in->scale, qn);
    l2norm((const uint8_t *)in->k + b * in->sk, in->qk_dtype, (int64_t)h * dk, dk, 1.f, kn);
    for (int k = 0; k < dk; k++) gv[k] = ld((const uint8_t *)in->g + b * in->sg, in->g_dtype, (int64_t)h * dk + k);
    for (int v = 0; v < dv; v++) vv[v] = ld((const uint8_t *)in->v + b * in->sv, in->v_dtype, (int64_t)h * dv + v);
    head_in_t hi;
    memset(&hi, 0, sizeof hi);
    hi.kind = KIND_KDA;
    hi.xq = qn; hi.xk = kn; hi.kx = kn; hi.vin = vv; hi.gv = gv;
    hi.beta = ld((const uint8_t *)in->beta + b * in->sbeta, in->beta_dtype, h);
    double kq = 0.;
    for (int k = 0; k < dk; k++) kq += (double)(kn[k] * qn[k]);
    hi.kq = (float)kq;
    hi.write_key = 1;
    step_head(st, seq, h, &hi, orow, in->out_dtype);
    free(buf);
  }
  return 0;
}

/* ------------------------------------------------------------------------------------------------------ */
/* prefill side: read (stored state advanced over its pending buffer) and write (slots.py:210-252)        */
/* ------------------------------------------------------------------------------------------------------ */
/* kind: 0 GDN / Mamba2 (scalar decay), 2 KDA (per-channel decay).  out fp32 [P, HV, DV, DK]. */
int sqo_slot_read(const sqb_state_t *st, int kind, const int64_t *slots, int64_t P, float *out) {
  const int hv = st->hv, hk = st->hk, dk = st->dk, dv = st->dv, M = st->m, gqa = hv / hk;
  const int qbuf = st->buffer_bits == 8, bsz = qbuf ? 1 : 2;
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t ph = 0; ph < P * hv; ph++) {
    const int64_t seq = slots[ph / hv];
    const int h = (int)(ph % hv), hkk = h / gqa;
    float *So = out + ph * (int64_t)dv * dk;
    const uint8_t *S = (const uint8_t *)st->S + seq * st->sS + (size_t)h * code_bytes(st);
    const uint16_t *SC = st->bits <= 8 ? (const uint16_t *)((const uint8_t *)st->SC + seq * st->sSC) + (size_t)h * scale_count(st) : NULL;
    const uint8_t *KB = (const uint8_t *)st->KB + seq * st->sKB + (size_t)hkk * M * dk * bsz;
    const uint8_t *UB = (const uint8_t *)st->UB + seq * st->sUB + (size_t)h * M * dv * bsz;
    const uint16_t *KBS = qbuf ? (const uint16_t *)((const uint8_t *)st->KBS + seq * st->sKBS) + (size_t)hkk * M : NULL;
    const uint16_t *UBS = qbuf ? (const uint16_t *)((const uint8_t *)st->UBS + seq * st->sUBS) + (size_t)h * M : NULL;
    const int gw = kind == KIND_KDA ? dk : 1;
    const float *GB = (const float *)((const uint8_t *)st->GB + seq * st->sGB) + (size_t)h * M * gw;
    const float *GCUR = (const float *)((const uint8_t *)st->GCUR + seq * st->sGC) + (size_t)h * gw;
    const int n = *((const int32_t *)((const uint8_t *)st->NPTR + seq * st->sN)) & (M - 1); /* element 0 */
    unpack_head(S, SC, dv, dk, st->bits, st->axis_k, st->group, So);
    float *kb = (float *)malloc(sizeof(float) * ((size_t)dk + dv));
    float *ub = kb + dk;
    for (int v = 0; v < dv; v++)
      for (int k = 0; k < dk; k++) So[(size_t)v * dk + k] = expf(GCUR[kind == KIND_KDA ? k : 0]) * So[(size_t)v * dk + k];
    /* einsum over the live slots, accumulated in double per entry */
    double *acc = (double *)calloc((size_t)dv * dk, sizeof(double));
    for (int i = 0; i < n; i++) {
      load_buf(KB, KBS, qbuf, i, dk, kb);
      load_buf(UB, UBS, qbuf, i, dv, ub);
      if (kind == KIND_KDA) {
        for (int k = 0; k < dk; k++) kb[k] = kb[k] * expf(GCUR[k] - GB[(size_t)i * dk + k]);
      } else {
        float d = expf(GCUR[0] - GB[i]);
        for (int v = 0; v < dv; v++) ub[v] = ub[v] * d;
      }
      for (int v = 0; v < dv; v++)
        for (int k = 0; k < dk; k++) acc[(size_t)v * dk + k] += (double)ub[v] * (double)kb[k];
    }
    if (n)
      for (size_t e = 0; e < (size_t)dv * dk; e++) So[e] = So[e] + (float)acc[e];
    free(acc);
    free(kb);
  }
  return 0;
}

/* S fp32 [P, HV, DV, DK] -> slots: codes + scales, counters and running decay zeroed */
int sqo_slot_write(const sqb_state_t *st, int kind, const int64_t *slots, int64_t P, const float *Sin) {
  const int hv = st->hv, dk = st->dk, dv = st->dv;
  const int nptr_len = hv > 4 ? hv : 4;
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t ph = 0; ph < P * hv; ph++) {
    const int64_t seq = slots[ph / hv];
    const int h = (int)(ph % hv);
    uint8_t *S = (uint8_t *)st->S + seq * st->sS + (size_t)h * code_bytes(st);
    uint16_t *SC = st->bits <= 8 ? (uint16_t *)((uint8_t *)st->SC + seq * st->sSC) + (size_t)h * scale_count(st) : NULL;
    pack_head(Sin + ph * (int64_t)dv * dk, dv, dk, st->bits, st->axis_k, st->group, S, SC);
    const int gw = kind == KIND_KDA ? dk : 1;
    float *GCUR = (float *)((uint8_t *)st->GCUR + seq * st->sGC) + (size_t)h * gw;
    for (int k = 0; k < gw; k++) GCUR[k] = 0.f;
    if (h == 0) {
      int32_t *NP = (int32_t *)((uint8_t *)st->NPTR + seq * st->sN);
      for (int i = 0; i < nptr_len; i++) NP[i] = 0;
    }
  }
  return 0;
}

/* threads the oracle's parallel loops use from now on (the benchmark's CPU legs set this to the host's core count
 * themselves: launchers such as torchrun export OMP_NUM_THREADS=1) */
void sqo_set_num_threads(int n) {
#ifdef _OPENMP
  extern void omp_set_num_threads(int);
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int sqo_num_threads(void) {
#ifdef _OPENMP
  extern int omp_get_max_threads(void);
  return omp_get_max_threads();
#else
  return 1;
#endif
}
