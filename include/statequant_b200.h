/*
 * statequant_b200 - C ABI of the fused packed-state decode step (Gated DeltaNet, Mamba2/SSD, KDA).
 *
 * Every entry point launches hand-written sm_100a CUDA kernels on the given stream and returns at once:
 * no allocation, no host synchronisation, so a call can be captured in a CUDA graph and replayed with
 * different slot tables.  All pointers in the argument structs are DEVICE pointers (the CPU oracle under
 * oracle/ takes the same structs with HOST pointers and is test infrastructure only).  Strides are in BYTES.
 *
 * What each entry point replaces in the reference (HallerPatrick/StateQuant, paths inside that project):
 *   sqb_gdn_step     the Triton launch `_fused_step[(BH,)](...)`   src/statequant/kernels/fold.py:401-407,
 *                                                                   src/statequant/kernels/slots.py:180-186
 *   sqb_mamba2_step  `_m2_step[(rows * HV,)](...)`                  src/statequant/kernels/mamba2.py:232-240
 *   sqb_kda_step     `_kda_step[(rows * HV,)](...)`                 src/statequant/kernels/kda.py:199-204
 *
 * Return value: 0 on success, a negative SQB_E* code otherwise; sqb_last_error() gives the message of the
 * last failure on the calling thread.  Nothing is launched when an error is returned.
 */
#ifndef STATEQUANT_B200_H
#define STATEQUANT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of activation tensors */
enum { SQB_F32 = 0, SQB_BF16 = 1, SQB_F16 = 2 };

/* error codes */
enum {
  SQB_OK = 0,
  SQB_EINVAL = -1,      /* a shape, stride, alignment or format the kernels do not support */
  SQB_ECUDA = -2,       /* the CUDA runtime refused the launch */
  SQB_ENOTBUILT = -3    /* this build has no kernel for the requested (kind, bits, axis) */
};

/*
 * The packed state of one layer, as per-sequence tables.  Sequence (slot) s of table X lives at
 * X + s * sX (bytes).  Field meaning and element layout are the reference's
 * (src/statequant/kernels/slots.py:9-28, kda.py:291-295):
 *
 *   S     codes  bits 4: uint8 [HV, DV, DK/2], byte j = (c[2j]+8) | (c[2j+1]+8) << 4
 *                bits 8: int8 [HV, DV, DK];  bits 16: bf16 [HV, DV, DK];  bits 32: fp32 [HV, DV, DK]
 *   SC    fp16 scales  axis k: [HV, DV, DK/group];  axis v: [HV, DV/group, DK]   (unused for bits 16 / 32)
 *   KB    buffered keys  int8 or bf16 [HK, m, DK]       KBS fp16 [HK, m]  (int8 buffer only)
 *   UB    buffered values int8 or bf16 [HV, m, DV]      UBS fp16 [HV, m]  (int8 buffer only)
 *   GB    fp32 [HV, m]  cumulative log decay of each buffered token   (KDA: [HV, m, DK])
 *   GCUR  fp32 [HV]     running log decay since the last fold          (KDA: [HV, DK])
 *   NPTR  int32 [>= HV] buffer fill counter, one copy per value head
 */
typedef struct sqb_state {
  void *S;      int64_t sS;
  void *SC;     int64_t sSC;
  void *KB;     int64_t sKB;
  void *KBS;    int64_t sKBS;
  void *UB;     int64_t sUB;
  void *UBS;    int64_t sUBS;
  void *GB;     int64_t sGB;
  void *GCUR;   int64_t sGC;
  void *NPTR;   int64_t sN;
  int32_t bits;          /* 4, 8, 16 (bf16 state) or 32 (fp32 state) */
  int32_t axis_k;        /* 1: scale groups run along d_k; 0: along d_v */
  int32_t group;         /* scale group length */
  int32_t buffer_bits;   /* 8: int8 + fp16 absmax scale per vector; 16: bf16 */
  int32_t m;             /* buffer length, a power of two <= 32 */
  int32_t hv, hk;        /* value heads, key heads (Mamba2: heads, groups); hv % hk == 0 */
  int32_t dk, dv;        /* head dims: dk * bits a multiple of 128 (whole 16-byte chunks per row, at most 32: 64, 96,
                            128, 192 ...), dv a multiple of 4; scale groups: a power of two (key-axis: a multiple of
                            128 / bits, the last one may be short; value-axis: dividing dv) */
  int32_t reserved;
} sqb_state_t;

/*
 * Inputs of one Gated DeltaNet decode token for `rows` batch rows.
 *   idx       int32 [rows] slot of each row, or NULL: row b is sequence b (lockstep).  idx <= 0 marks a padding
 *             row: its output row is zeroed and nothing else is touched.
 *   q, k      [rows, hk, dk] (qk_per_key_head = 1) or [rows, hv, dk] (0); raw, l2-normalised in the kernel,
 *             q scaled by `scale`; unit inner stride, row strides sq / sk
 *   v         [rows, hv, dv]
 *   g, beta   [rows, hv] log decay and beta (after the sigmoid)               when gate == 0
 *   a, b      [rows, hv]; A_log fp32 [hv]; dt_bias [hv]                         when gate == 1:
 *             g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b)
 *   out       [rows, hv, dv], row stride so
 */
typedef struct sqb_gdn_inputs {
  const int32_t *idx;
  const void *q;      int64_t sq;
  const void *k;      int64_t sk;
  const void *v;      int64_t sv;
  const void *g;      int64_t sg;
  const void *beta;   int64_t sbeta;
  const void *a;      int64_t sa;
  const void *b;      int64_t sb;
  const void *A_log;
  const void *dt_bias;
  void *out;          int64_t so;
  float scale;
  int32_t rows;
  int32_t qk_per_key_head;
  int32_t gate;
  int32_t qk_dtype, v_dtype, gb_dtype, ab_dtype, alog_dtype, dtb_dtype, out_dtype;
  int32_t reserved;
} sqb_gdn_inputs_t;

/*
 * Inputs of one Mamba2 / SSD decode token.
 *   x [rows, hv, dv], dt [rows, hv] raw, B / C [rows, hk, dk], A / D / dt_bias [hv] (D, dt_bias may be NULL);
 *   dt = softplus(dt + dt_bias) if dt_softplus, clamped to [dt_min, dt_max] if dt_clamp; out [rows, hv, dv].
 */
typedef struct sqb_mamba2_inputs {
  const int32_t *idx;
  const void *x;      int64_t sx;
  const void *dt;     int64_t sdt;
  const void *B;      int64_t sB;
  const void *C;      int64_t sC;
  const void *A;
  const void *D;
  const void *dt_bias;
  void *out;          int64_t so;
  float dt_min, dt_max;
  int32_t rows;
  int32_t dt_softplus, dt_clamp;
  int32_t x_dtype, dt_dtype, bc_dtype, a_dtype, d_dtype, dtb_dtype, out_dtype;
} sqb_mamba2_inputs_t;

/*
 * Inputs of one KDA decode token.
 *   q, k, g [rows, hv, dk] (g: log decay per key channel), v [rows, hv, dv], beta [rows, hv], out [rows, hv, dv].
 */
typedef struct sqb_kda_inputs {
  const int32_t *idx;
  const void *q;      int64_t sq;
  const void *k;      int64_t sk;
  const void *v;      int64_t sv;
  const void *g;      int64_t sg;
  const void *beta;   int64_t sbeta;
  void *out;          int64_t so;
  float scale;
  int32_t rows;
  int32_t qk_dtype, v_dtype, g_dtype, beta_dtype, out_dtype;
  int32_t reserved;
} sqb_kda_inputs_t;

/*
 * The packed GGA / STEP slot table of one layer (mixed per-head widths, optional pure-write window).
 * Slot s lives at blob + s * stride.  Inside a slot (reference: src/statequant/kernels/_gga_triton.py:3-13,
 * src/statequant/integrations/vllm_gga.py:182-205):
 *   0            int32 [4]: n (queued pairs), head (ring index of the oldest pair)
 *   offs[h]      head h at its width bits[h]: 16 -> fp16 [dk, dv]; 4 / 6 / 8 -> codes [dk, dv * b / 8] (u = z + qmax,
 *                little-endian along dv; 6 bit: four codes per three bytes), r fp16 [dk], c fp16 [dv];
 *                2 -> codes [dk, dv / 4] (u = (z + 3) / 2), r fp16 [dk, dv / group], c fp16 [dv].  State = r c z.
 *   qoff + h qsz the window of head h (pw only): P e4m3 [m, dk], V e4m3 [m, dv], PS fp32 [m], VS fp32 [m]
 * offs, bits (int32 [hv]) and w (fp32 [hv, dk], STEP's impact factors) are device arrays of the layer's plan.
 */
typedef struct sqb_gga_layout {
  void *blob;          int64_t stride;
  const int32_t *offs; const int32_t *bits; const float *w;
  int64_t qoff;
  int32_t qsz;
  int32_t hv, hk, dk, dv;
  int32_t m;           /* window length */
  int32_t pw;          /* 1: pure-write window on */
  int32_t group;       /* column group of 2-bit row factors (32) */
  int32_t flags;       /* bit 0 (SQB_GGA_ALL_PACKED, a hint that may be left 0): every head of this layer is 4, 6 or 8
                          bits wide, so the step needs no launch for 2-bit heads and fp16 pivots */
} sqb_gga_layout_t;
#define SQB_GGA_ALL_PACKED 1

/* replaces `_fused_step[(BH,)]`, src/statequant/kernels/fold.py:401-407 and slots.py:180-186 */
int sqb_gdn_step(const sqb_state_t *st, const sqb_gdn_inputs_t *in, void *cuda_stream);
/* replaces `_m2_step[(rows * HV,)]`, src/statequant/kernels/mamba2.py:232-240 */
int sqb_mamba2_step(const sqb_state_t *st, const sqb_mamba2_inputs_t *in, void *cuda_stream);
/* replaces `_kda_step[(rows * HV,)]`, src/statequant/kernels/kda.py:199-204 */
int sqb_kda_step(const sqb_state_t *st, const sqb_kda_inputs_t *in, void *cuda_stream);

/* One GGA decode token: replaces `_gga_step[(B * HV,)]` + `_gga_advance[(B,)]`,
   src/statequant/integrations/vllm_gga.py:252-257.  Takes the gate form of the GDN inputs (gate must be 1). */
int sqb_gga_step(const sqb_gga_layout_t *lay, const sqb_gdn_inputs_t *in, void *cuda_stream);
/* Fit + pack canonical states X fp32 [P, hv, dk, dv] into slots idx [P] and zero their counters: replaces
   `_gga_store[(P * HV,)]`, src/statequant/integrations/vllm_gga.py:317-318 */
int sqb_gga_store(const sqb_gga_layout_t *lay, const int32_t *idx, int64_t P, const float *X, void *cuda_stream);
/* Unpack slots idx [P] into Y fp32 [P, hv, dk, dv] (stored state without the window): replaces
   `_gga_load[(P * HV,)]`, src/statequant/integrations/vllm_gga.py:270-271 */
int sqb_gga_load(const sqb_gga_layout_t *lay, const int32_t *idx, int64_t P, float *Y, void *cuda_stream);
/* STEP's dual-axis fit as a fake-quant pass, x -> y fp32 [B, H, dk, dv], bits int32 [H], w fp32 [H, dk]: replaces
   `_stepquant_fit[(B * H,)]`, src/statequant/kernels/_stepquant_triton.py:86-99 */
int sqb_stepquant_fit(const float *x, float *y, const int32_t *bits, const float *w, int64_t B, int32_t H,
                      int32_t dk, int32_t dv, int32_t group, void *cuda_stream);

/* message of the last error returned on this thread ("" if none) */
/*
 * The prefill boundary of a slot table, on the device (4 / 8-bit states, d_k 64 or 128; SQB_EINVAL otherwise, and the
 * caller keeps its own path).  kind: 0 GDN, 1 Mamba2, 2 KDA.  idx int32 [rows] (NULL: row r is sequence r).
 *   sqb_slot_read   out fp32 [rows, hv, dv, dk] = the state of each slot advanced across its pending buffer,
 *                   S_n = a_n S_0 + sum_{i<n} (a_n / a_i) u_i k_i^T (KDA: decays per key channel); slots are not
 *                   modified.  Replaces the torch gather + einsum of src/statequant/kernels/slots.py:210-233 and
 *                   kernels/kda.py:351-372.
 *   sqb_slot_write  S fp32 [rows, hv, dv, dk] packed into the slots (scales and codes byte for byte those of
 *                   pack_vk, src/statequant/kernels/fold.py:111-147) and their buffers emptied.  Replaces
 *                   kernels/slots.py:236-252, kernels/kda.py:375-386.
 */
int sqb_slot_read(const sqb_state_t *st, int kind, const int32_t *idx, int32_t rows, float *out, void *stream);
int sqb_slot_write(const sqb_state_t *st, int kind, const int32_t *idx, int32_t rows, const float *S, void *stream);

/*
 * The short causal convolution that feeds the decode step (one token per sequence): the op the reference's vLLM
 * forward calls right before `lay.step` (src/statequant/integrations/vllm_plugin.py:379-381,
 * `causal_conv1d_update(mixed_qkv, conv_state, w, bias, activation, conv_state_indices=...)`, vLLM's
 * model_executor/layers/mamba/ops/causal_conv1d.py), whose output rows are the q | k | v the step reads as column
 * slices.  Per row r with line = idx[r] (idx NULL: line = r; line == null_line or line < 0: the row is left alone)
 * and per channel c:
 *     window = state[line, c, 0 .. width-2], x[r, c]
 *     acc    = bias[c] (fp32; 0 without bias);  acc += x_j * w[c, j] for j = 0 .. width-1, in this order
 *              (x and w of the same 16-bit type: the product is rounded to that type first, as the Triton kernel's
 *              typed multiply does; otherwise the product is fused into the fp32 sum)
 *     out[r, c] = silu ? acc / (1 + exp(-acc)) : acc      rounded to x's type
 *     state[line, c, t] = state[line, c, t+1] for t < state_len-1;  state[line, c, state_len-1] = x[r, c]
 * x, out and the state share one element type; out may be x itself (vLLM's kernel works in place).
 */
typedef struct sqb_conv_update {
  void *x;          int64_t sx;            /* [rows, dim], row stride in bytes, unit inner stride */
  void *out;        int64_t so;            /* [rows, dim]; may alias x */
  void *state;      int64_t s_line, s_dim, s_tok;   /* conv state [lines, dim, state_len], strides in bytes */
  const void *w;    int64_t sw_dim, sw_tap;         /* weights [dim, width], strides in bytes */
  const void *bias;                        /* [dim], type of w; may be NULL */
  const int32_t *idx;                      /* [rows] cache lines; may be NULL */
  int32_t rows, dim, width, state_len;     /* width 2 .. 4; state_len >= width - 1 */
  int32_t x_dtype, w_dtype;                /* SQB_F32 / SQB_BF16 / SQB_F16 */
  int32_t silu;
  int32_t null_line;                       /* rows with this line are skipped (vLLM's null block, 0); -1: none */
} sqb_conv_update_t;
int sqb_conv1d_update(const sqb_conv_update_t *a, void *cuda_stream);

const char *sqb_last_error(void);
/* ABI version of this header; bumped whenever a struct changes */
int sqb_abi_version(void);
/* number of kernel launches issued by this library in this process (all threads) */
int64_t sqb_launch_count(void);
/* tuning / test switches.
   "kernel_path" selects the kernel of the decode steps: 0 the best one for the shape (default); 1 the generic kernel
   (direct loads, folds inside its own launch; any supported shape); 2 the staged SIMT kernel (one CTA per batch row
   and key head, the state staged through shared memory by bulk async copies) followed by the fold launch; 3 the
   tensor-core kernel (the state pass as integer mma.sync products) followed by the fold launch; 4 the tensor-core
   kernel with the fold of a slot's m-th token inside its launch (what 0 picks wherever the shape allows).  A path
   that does not take a shape falls through to the next lower one.  "force_generic_kernel" = 1 is the same as
   kernel_path 1 (and sends every GGA head to the tile kernel).  The paths agree up to the order of fp32 sums.
   "wait_limit_us": how long a device-side wait for a bulk copy may last before the CTA gives up (default 1 s).
   "mma_heads_per_cta": value heads a CTA of the tensor-core kernels takes (0: the default, two stages of 128 rows).
   "test_extra_tx": test hook; bytes a stage barrier is told to expect beyond what is copied, so that its wait runs
   out (a multiple of 16; 0 in any real run). */
int sqb_set_option(const char *name, int value);
/* Device-side health word of the current device (synchronises): the number of CTAs whose wait for a bulk copy ran
   out of its time limit since the library was loaded (such a CTA zeroes its output rows and touches no slot).  0 in a healthy run. */
int sqb_device_status(int *wait_timeouts);

#ifdef __cplusplus
}
#endif
#endif
