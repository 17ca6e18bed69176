// C ABI of statequant_b200 (see include/statequant_b200.h): argument checks, kernel selection, launch.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/statequant_b200.h"
#include "delta_step.cuh"
#include "launchers.h"
#include "fold_kernel.cuh"
#include "launch_mma.cuh"
#include "gga.cuh"
#include "conv_update.cuh"

namespace sqb {
__device__ int g_step_status[4];   // [0]: number of CTAs whose bounded wait ran out (0 in a healthy run)
}

namespace {

thread_local char g_err[512] = "";
std::atomic<long long> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
  return code;
}

bool pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }
int ilog2(int x) { int l = 0; while ((1 << l) < x) l++; return l; }
bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// What the kernels support; everything else is refused before any launch.
int check_state(const sqb_state_t* st, int kind, int* lpr_log2) {
  if (!st) return fail(SQB_EINVAL, "state is NULL");
  const int bits = st->bits, dk = st->dk, dv = st->dv, m = st->m, g = st->group;
  if (bits != 4 && bits != 8 && bits != 16 && bits != 32) return fail(SQB_EINVAL, "bits %d: expected 4, 8, 16 or 32", bits);
  if (st->buffer_bits != 8 && st->buffer_bits != 16) return fail(SQB_EINVAL, "buffer_bits %d: expected 8 or 16", st->buffer_bits);
  if (!pow2(m) || m > 32) return fail(SQB_EINVAL, "m %d: expected a power of two <= 32", m);
  if (st->hv <= 0 || st->hk <= 0 || st->hv % st->hk) return fail(SQB_EINVAL, "heads hv %d, hk %d: hv must be a multiple of hk", st->hv, st->hk);
  if (kind == sqb::K_KDA && st->hv != st->hk) return fail(SQB_EINVAL, "KDA: key heads must equal value heads");
  const int cpl = 128 / bits;
  if (dk <= 0 || dk % cpl || dk / cpl > 32)
    return fail(SQB_EINVAL, "d_k %d with %d-bit codes: a row must be 1 to 32 whole 16-byte chunks", dk, bits);
  int lpr = 1;                                // lanes per row, rounded up to a power of two (d_k 96, 192: the last lanes idle)
  while (lpr < dk / cpl) lpr <<= 1;
  const int rpp = 32 / lpr;
  if (dv % 4 || dv <= 0) return fail(SQB_EINVAL, "d_v %d: expected a positive multiple of 4", dv);
  if (bits <= 8) {
    if (!pow2(g)) return fail(SQB_EINVAL, "group %d: expected a power of two", g);
    if (st->axis_k) {
      if (g % cpl) return fail(SQB_EINVAL, "key-axis group %d with %d-bit codes: the group must be a multiple of %d", g, bits, cpl);
    } else {
      if (dv % g) return fail(SQB_EINVAL, "value-axis group %d must divide d_v %d", g, dv);
      if (g % rpp || dv % (sqb::NW * rpp)) return fail(SQB_EINVAL, "value-axis group %d, d_v %d: both must be multiples of %d rows", g, dv, rpp);
      const int wpg = g / rpp < sqb::NW ? g / rpp : sqb::NW;
      if (g / (rpp * wpg) > 64 / cpl) return fail(SQB_EINVAL, "value-axis group %d on d_k %d: at most %d rows per group", g, dk, (64 / cpl) * rpp * sqb::NW);
    }
    if (!st->SC) return fail(SQB_EINVAL, "SC is NULL for an integer state");
  }
  if (!st->S || !st->KB || !st->UB || !st->GB || !st->GCUR || !st->NPTR) return fail(SQB_EINVAL, "a state table pointer is NULL");
  if (st->buffer_bits == 8 && (!st->KBS || !st->UBS)) return fail(SQB_EINVAL, "KBS / UBS are NULL for an int8 buffer");
  if (!al16(st->S) || st->sS % 16) return fail(SQB_EINVAL, "codes table: base and per-sequence stride must be multiples of 16 bytes");
  if ((reinterpret_cast<uintptr_t>(st->KB) & 7) || st->sKB % 8 || (reinterpret_cast<uintptr_t>(st->UB) & 7) || st->sUB % 8)
    return fail(SQB_EINVAL, "buffer tables: base and stride must be multiples of 8 bytes");
  if ((static_cast<long long>(m) * dk) % 8 || (static_cast<long long>(m) * dv) % 8 || (static_cast<long long>(dv) * dk * bits / 8) % 16)
    return fail(SQB_EINVAL, "per-head sizes are not 16-byte multiples (m %d, d_k %d, d_v %d)", m, dk, dv);
  *lpr_log2 = ilog2(lpr);
  return 0;
}

int* status_ptr() {
  static thread_local int* ptr[64];
  int dev = 0;
  cudaGetDevice(&dev);
  int*& p = ptr[dev & 63];
  if (!p) {
    void* q = nullptr;
    if (cudaGetSymbolAddress(&q, sqb::g_step_status) == cudaSuccess) p = static_cast<int*>(q);
  }
  return p;
}

std::atomic<int> g_force_generic{0};     // set through sqb_set_option (tests time and check every kernel)
std::atomic<int> g_kernel_path{0};       // see sqb_set_option in the header
std::atomic<long long> g_wait_ns{1000000000ll};   // bound of a device-side wait for a bulk copy
std::atomic<int> g_test_extra_tx{0};     // test hook: makes the stage barriers of the tensor-core kernels wait in vain
std::atomic<int> g_mma_hpc{0};           // tensor-core kernels: value heads per CTA (0: all of a key head)

int fill_state(sqb::StepArgs& a, const sqb_state_t* st, int lpr_log2) {
  a.status = status_ptr();
  if (!a.status) return fail(SQB_ECUDA, "the device status word is not reachable (cudaGetSymbolAddress failed)");
  a.wait_ns = static_cast<unsigned long long>(g_wait_ns.load(std::memory_order_relaxed));
  a.test_extra_tx = g_test_extra_tx.load(std::memory_order_relaxed);
  a.hpc = g_mma_hpc.load(std::memory_order_relaxed);
  a.S = static_cast<uint8_t*>(st->S); a.SC = static_cast<uint8_t*>(st->SC);
  a.KB = static_cast<uint8_t*>(st->KB); a.KBS = static_cast<uint8_t*>(st->KBS);
  a.UB = static_cast<uint8_t*>(st->UB); a.UBS = static_cast<uint8_t*>(st->UBS);
  a.GB = static_cast<uint8_t*>(st->GB); a.GCUR = static_cast<uint8_t*>(st->GCUR);
  a.NPTR = static_cast<uint8_t*>(st->NPTR);
  a.sS = st->sS; a.sSC = st->sSC; a.sKB = st->sKB; a.sKBS = st->sKBS; a.sUB = st->sUB; a.sUBS = st->sUBS;
  a.sGB = st->sGB; a.sGC = st->sGC; a.sN = st->sN;
  a.group = st->group; a.qbuf = st->buffer_bits == 8; a.M = st->m; a.HV = st->hv; a.HK = st->hk;
  a.DK = st->dk; a.DV = st->dv; a.lpr_log2 = lpr_log2; a.state_f32 = 0;
  return 0;
}

template <int KIND, int BITS, bool AXK>
int launch_one(const sqb::StepArgs& a, cudaStream_t stream) {
  auto kern = sqb::delta_step_kernel<KIND, BITS, AXK>;
  const sqb::Smem plan = sqb::smem_plan(KIND, a.DK, a.DV, a.M, 128 / BITS, 1 << a.lpr_log2);
  const size_t smem = static_cast<size_t>(plan.total) * sizeof(float);
  static sqb::SmemLimit limit;                    // per instantiation
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) return fail(SQB_EINVAL, "shape needs %zu bytes of shared memory per CTA", smem);
    cudaError_t e = limit.ensure(kern, static_cast<int>(smem));
    if (e != cudaSuccess) return fail(SQB_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  const long long ctas = static_cast<long long>(a.rows) * a.HV;
  if (ctas > 2147483647LL) return fail(SQB_EINVAL, "rows * hv = %lld exceeds the grid limit", ctas);
  kern<<<static_cast<unsigned>(ctas), sqb::NT, smem, stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(SQB_ECUDA, "kernel launch: %s", cudaGetErrorString(e));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

// ---- the staged kernel (integer states, d_k 64 or 128, everything 16-byte aligned) -----------------------------------
bool tma_ok(const sqb::StepArgs& a, int bits, bool axk, bool kda) {
  if (bits != 4 && bits != 8) return false;
  if (a.DK != 64 && a.DK != 128) return false;
  if (!a.per_key_head && a.HV != a.HK) return false;      // q, k per value head: generic kernel
  const int lpr = a.DK / 16, rpp = 32 / lpr, bsz = a.qbuf ? 1 : 2, g = a.group;
  if (a.DV % (sqb::NW * rpp)) return false;
  if (axk) {
    if (g % 16 || a.DK % g) return false;
  } else {
    if (g % rpp || a.DV % g) return false;
    const int wpg = g / rpp < sqb::NW ? g / rpp : sqb::NW;
    if (g / (rpp * wpg) > 2) return false;
  }
  const long long codes_b = static_cast<long long>(a.DV) * a.DK * bits / 8;
  const long long scales_b = (axk ? static_cast<long long>(a.DV) * (a.DK / g) : static_cast<long long>(a.DV / g) * a.DK) * 2;
  const long long ub_b = static_cast<long long>(a.M) * a.DV * bsz, kb_b = static_cast<long long>(a.M) * a.DK * bsz;
  if (codes_b % 16 || scales_b % 16 || ub_b % 16 || kb_b % 16) return false;
  auto a16 = [](const void* p, long long s) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && s % 16 == 0; };
  if (!a16(a.S, a.sS) || !a16(a.SC, a.sSC) || !a16(a.UB, a.sUB) || !a16(a.KB, a.sKB)) return false;
  if (kda && (!a16(a.GB, a.sGB) || !a16(a.GCUR, a.sGC))) return false;
  return true;
}

// launchers of the staged kernels and of the fold kernel live in their own translation units (launchers.h)
int sub_rc(int rc) {
  if (rc >= 0) {
    if (rc == 0) g_launches.fetch_add(1, std::memory_order_relaxed);
    return rc;
  }
  return fail(SQB_ECUDA, "kernel launch: %s", cudaGetErrorString(static_cast<cudaError_t>(-rc - 1000)));
}
template <int KIND>
int launch_tma(const sqb::StepArgs& a, int bits, bool axk, cudaStream_t stream) {
  if (KIND == sqb::K_GDN) return sub_rc(sqb::launch_staged_gdn(a, bits, axk, stream));
  if (KIND == sqb::K_M2) return sub_rc(sqb::launch_staged_m2(a, bits, axk, stream));
  return sub_rc(sqb::launch_staged_kda(a, bits, axk, stream));
}

template <int KIND>
int launch_mma_kind(const sqb::StepArgs& a, int bits, int mode, cudaStream_t stream) {
  if (KIND == sqb::K_GDN) return sub_rc(sqb::launch_mma_gdn(a, bits, mode, stream));
  if (KIND == sqb::K_M2) return sub_rc(sqb::launch_mma_m2(a, bits, mode, stream));
  return sub_rc(sqb::launch_mma_kda(a, bits, mode, stream));
}

// the fold launch of this shape fits an SM's shared memory (checked before the step kernel that relies on it starts)
bool fold_fits(const sqb::StepArgs& a, int bits, bool axk, bool kda) {
  return sqb::smemf_plan(kda, bits, axk, a.group, a.DK, a.DV, a.M, a.qbuf).total <= 220 * 1024;
}

template <int KIND>
int launch(const sqb::StepArgs& a0, int bits, bool axk, cudaStream_t stream) {
  const sqb::StepArgs& a = a0;
  const int path = g_force_generic.load(std::memory_order_relaxed) ? 1 : g_kernel_path.load(std::memory_order_relaxed);
  constexpr bool kda = KIND == sqb::K_KDA;
  // Every check that could refuse a launch is made before the first one: a positive "shape not taken" code after a
  // step kernel has appended would leave the slot between two states.
  if ((path == 0 || path >= 3) && sqb::mma_shape_ok(a0, bits, axk, kda, KIND)) {
    sqb::StepArgs a = a0;
    a.axv = axk ? 0 : 1;
    sqb::SmemM plan;
    int nst;
    if ((path == 4 || path == 0) && sqb::mma_fold_inside(a, bits, KIND)) {
      // tensor-core kernel with the fold inside: one launch, the stored state read once per token
      if (sqb::mma_plan<KIND>(a, bits, 3, plan, nst)) {
        const int rc = launch_mma_kind<KIND>(a, bits, 3, stream);
        return rc <= 0 ? rc : fail(SQB_ECUDA, "tensor-core step kernel refused a checked shape");
      }
    } else if (sqb::mma_plan<KIND>(a, bits, 0, plan, nst) && fold_fits(a, bits, axk, kda)) {
      const int rc = launch_mma_kind<KIND>(a, bits, 0, stream);
      if (rc != 0) return rc < 0 ? rc : fail(SQB_ECUDA, "tensor-core step kernel refused a checked shape");
      const int rf = sub_rc(sqb::launch_fold(KIND, a, bits, axk, stream));
      return rf <= 0 ? rf : fail(SQB_ECUDA, "fold kernel refused a checked shape");
    }
  }
  if (path != 1 && tma_ok(a, bits, axk, kda) && fold_fits(a, bits, axk, kda)) {
    // the staged kernel only appends on a slot's m-th token; the fold launch that follows it rewrites the state of
    // the heads whose buffer is full (the generic kernel folds inside its own launch)
    const int rc = launch_tma<KIND>(a, bits, axk, stream);
    if (rc < 0) return rc;
    if (rc == 0) {
      const int rf = sub_rc(sqb::launch_fold(KIND, a, bits, axk, stream));
      return rf <= 0 ? rf : fail(SQB_ECUDA, "fold kernel refused a checked shape");
    }
  }
  switch (bits) {
    case 4: return axk ? launch_one<KIND, 4, true>(a, stream) : launch_one<KIND, 4, false>(a, stream);
    case 8: return axk ? launch_one<KIND, 8, true>(a, stream) : launch_one<KIND, 8, false>(a, stream);
    case 16: return launch_one<KIND, 16, true>(a, stream);
    case 32: return launch_one<KIND, 32, true>(a, stream);
  }
  return fail(SQB_ENOTBUILT, "no kernel for %d-bit states", bits);
}

int check_dtype(int dt, const char* what) {
  if (dt < 0 || dt > 2) return fail(SQB_EINVAL, "%s: element type %d is not fp32 / bf16 / fp16", what, dt);
  return 0;
}

}  // namespace

extern "C" {

const char* sqb_last_error(void) { return g_err; }
int sqb_abi_version(void) { return 1; }
int64_t sqb_launch_count(void) { return g_launches.load(); }

int sqb_set_option(const char* name, int value) {
  if (name && !strcmp(name, "force_generic_kernel")) { g_force_generic = value; return 0; }
  if (name && !strcmp(name, "kernel_path") && value >= 0 && value <= 4) { g_kernel_path = value; return 0; }
  if (name && !strcmp(name, "mma_heads_per_cta") && value >= 0) { g_mma_hpc = value; return 0; }
  if (name && !strcmp(name, "wait_limit_us") && value > 0) { g_wait_ns = 1000ll * value; return 0; }
  if (name && !strcmp(name, "test_extra_tx") && value >= 0 && value % 16 == 0) { g_test_extra_tx = value; return 0; }
  return fail(SQB_EINVAL, "unknown option");
}

int sqb_device_status(int* wait_timeouts) {
  int st[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbol(st, sqb::g_step_status, sizeof st);
  if (e != cudaSuccess) return fail(SQB_ECUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
  if (wait_timeouts) *wait_timeouts = st[0];
  return 0;
}

namespace {
int slot_io_args(const sqb_state_t* st, int kind, const int32_t* idx, int32_t rows, sqb::StepArgs& a) {
  int lpr_log2 = 0;
  if (kind < 0 || kind > 2) return fail(SQB_EINVAL, "kind %d is not 0 (GDN), 1 (Mamba2) or 2 (KDA)", kind);
  if (int rc = check_state(st, kind, &lpr_log2)) return rc;
  if (rows < 0) return fail(SQB_EINVAL, "rows %d < 0", rows);
  memset(&a, 0, sizeof a);
  if (int rc = fill_state(a, st, lpr_log2)) return rc;
  a.rows = rows; a.idx = idx; a.per_key_head = 1;
  if (!tma_ok(a, st->bits, st->bits > 8 || st->axis_k, kind == sqb::K_KDA))
    return fail(SQB_EINVAL, "the device read / write kernels take 4 / 8-bit states with d_k 64 or 128 and 16-byte aligned fields");
  return 0;
}
}  // namespace

int sqb_slot_read(const sqb_state_t* st, int kind, const int32_t* idx, int32_t rows, float* out, void* stream) {
  sqb::StepArgs a;
  if (int rc = slot_io_args(st, kind, idx, rows, a)) return rc;
  if (!out) return fail(SQB_EINVAL, "out is NULL");
  if (reinterpret_cast<uintptr_t>(out) & 15) return fail(SQB_EINVAL, "out must be 16-byte aligned (it is written in 16-byte pieces)");
  if (rows == 0) return 0;
  return sub_rc(sqb::launch_read(kind, a, st->bits, st->axis_k, out, static_cast<cudaStream_t>(stream)));
}

int sqb_slot_write(const sqb_state_t* st, int kind, const int32_t* idx, int32_t rows, const float* S, void* stream) {
  sqb::StepArgs a;
  if (int rc = slot_io_args(st, kind, idx, rows, a)) return rc;
  if (!S) return fail(SQB_EINVAL, "S is NULL");
  if (reinterpret_cast<uintptr_t>(S) & 15) return fail(SQB_EINVAL, "S must be 16-byte aligned (it is read in 16-byte pieces)");
  if (rows == 0) return 0;
  return sub_rc(sqb::launch_write(kind, a, st->bits, st->axis_k, S, static_cast<cudaStream_t>(stream)));
}

int sqb_conv1d_update(const sqb_conv_update_t* c, void* stream) {
  if (!c) return fail(SQB_EINVAL, "arguments are NULL");
  if (c->rows <= 0) return c->rows == 0 ? 0 : fail(SQB_EINVAL, "rows %d < 0", c->rows);
  if (!c->x || !c->out || !c->state || !c->w) return fail(SQB_EINVAL, "x, out, state or w is NULL");
  if (check_dtype(c->x_dtype, "x") || check_dtype(c->w_dtype, "w")) return SQB_EINVAL;
  if (c->width < 2 || c->width > 4) return fail(SQB_EINVAL, "width %d: expected 2, 3 or 4", c->width);
  if (c->state_len < c->width - 1) return fail(SQB_EINVAL, "state_len %d is shorter than width - 1 = %d", c->state_len, c->width - 1);
  if (c->dim <= 0) return fail(SQB_EINVAL, "dim %d <= 0", c->dim);
  const int esz = c->x_dtype == SQB_F32 ? 4 : 2, wsz = c->w_dtype == SQB_F32 ? 4 : 2;
  if (esz == 2 && wsz == 2 && c->x_dtype != c->w_dtype) return fail(SQB_EINVAL, "x and w are different 16-bit types");
  if (c->sx % esz || c->so % esz || c->s_line % esz || c->s_dim % esz || c->s_tok % esz || c->sw_dim % wsz || c->sw_tap % wsz)
    return fail(SQB_EINVAL, "a stride is not a multiple of its element size");
  if ((reinterpret_cast<uintptr_t>(c->x) | reinterpret_cast<uintptr_t>(c->out) | reinterpret_cast<uintptr_t>(c->state)) % esz ||
      (reinterpret_cast<uintptr_t>(c->w) | reinterpret_cast<uintptr_t>(c->bias)) % wsz)
    return fail(SQB_EINVAL, "a pointer is not aligned to its element size");
  sqb::ConvArgs a;
  a.x = static_cast<const uint8_t*>(c->x); a.sx = c->sx;
  a.out = static_cast<uint8_t*>(c->out); a.so = c->so;
  a.state = static_cast<uint8_t*>(c->state); a.s_line = c->s_line; a.s_dim = c->s_dim; a.s_tok = c->s_tok;
  a.w = static_cast<const uint8_t*>(c->w); a.sw_dim = c->sw_dim; a.sw_tap = c->sw_tap;
  a.bias = static_cast<const uint8_t*>(c->bias); a.idx = c->idx;
  a.rows = c->rows; a.dim = c->dim; a.width = c->width; a.state_len = c->state_len;
  a.dt_x = c->x_dtype; a.dt_w = c->w_dtype; a.silu = c->silu != 0; a.null_line = c->null_line;
  a.pmode = (esz == 2 && wsz == 2) ? (c->x_dtype == SQB_BF16 ? 1 : 2) : 0;
  return sub_rc(sqb::launch_conv_update(a, static_cast<cudaStream_t>(stream)));
}

int sqb_gdn_step(const sqb_state_t* st, const sqb_gdn_inputs_t* in, void* stream) {
  int lpr_log2 = 0;
  if (int rc = check_state(st, sqb::K_GDN, &lpr_log2)) return rc;
  if (!in) return fail(SQB_EINVAL, "inputs are NULL");
  if (in->rows <= 0) return in->rows == 0 ? 0 : fail(SQB_EINVAL, "rows %d < 0", in->rows);
  if (!in->q || !in->k || !in->v || !in->out) return fail(SQB_EINVAL, "q, k, v or out is NULL");
  if (in->gate ? (!in->a || !in->b || !in->A_log || !in->dt_bias) : (!in->g || !in->beta))
    return fail(SQB_EINVAL, in->gate ? "gate inputs (a, b, A_log, dt_bias) missing" : "g / beta missing");
  if (check_dtype(in->qk_dtype, "q/k") || check_dtype(in->v_dtype, "v") || check_dtype(in->out_dtype, "out")) return SQB_EINVAL;
  sqb::StepArgs a;
  memset(&a, 0, sizeof a);
  if (int rc = fill_state(a, st, lpr_log2)) return rc;
  a.rows = in->rows; a.idx = in->idx;
  a.q = static_cast<const uint8_t*>(in->q); a.sq = in->sq;
  a.k = static_cast<const uint8_t*>(in->k); a.sk = in->sk;
  a.v = static_cast<const uint8_t*>(in->v); a.sv = in->sv;
  a.g = static_cast<const uint8_t*>(in->g); a.sg = in->sg;
  a.beta = static_cast<const uint8_t*>(in->beta); a.sbeta = in->sbeta;
  a.a = static_cast<const uint8_t*>(in->a); a.sa = in->sa;
  a.b = static_cast<const uint8_t*>(in->b); a.sb = in->sb;
  a.A_log = static_cast<const uint8_t*>(in->A_log); a.dt_bias = static_cast<const uint8_t*>(in->dt_bias);
  a.out = static_cast<uint8_t*>(in->out); a.so = in->so;
  a.dt_qk = in->qk_dtype; a.dt_v = in->v_dtype; a.dt_g = in->gb_dtype; a.dt_beta = in->gb_dtype;
  a.dt_ab = in->ab_dtype; a.dt_alog = in->alog_dtype; a.dt_dtb = in->dtb_dtype; a.dt_out = in->out_dtype;
  a.per_key_head = in->qk_per_key_head; a.gate = in->gate; a.scale = in->scale;
  return launch<sqb::K_GDN>(a, st->bits, st->bits > 8 || st->axis_k, static_cast<cudaStream_t>(stream));
}

int sqb_mamba2_step(const sqb_state_t* st, const sqb_mamba2_inputs_t* in, void* stream) {
  int lpr_log2 = 0;
  if (int rc = check_state(st, sqb::K_M2, &lpr_log2)) return rc;
  if (!in) return fail(SQB_EINVAL, "inputs are NULL");
  if (in->rows <= 0) return in->rows == 0 ? 0 : fail(SQB_EINVAL, "rows %d < 0", in->rows);
  if (!in->x || !in->dt || !in->B || !in->C || !in->A || !in->out) return fail(SQB_EINVAL, "x, dt, B, C, A or out is NULL");
  if (check_dtype(in->x_dtype, "x") || check_dtype(in->bc_dtype, "B/C") || check_dtype(in->out_dtype, "out")) return SQB_EINVAL;
  sqb::StepArgs a;
  memset(&a, 0, sizeof a);
  if (int rc = fill_state(a, st, lpr_log2)) return rc;
  a.rows = in->rows; a.idx = in->idx;
  a.q = static_cast<const uint8_t*>(in->C); a.sq = in->sC;
  a.k = static_cast<const uint8_t*>(in->B); a.sk = in->sB;
  a.v = static_cast<const uint8_t*>(in->x); a.sv = in->sx;
  a.g = static_cast<const uint8_t*>(in->dt); a.sg = in->sdt;
  a.A_log = static_cast<const uint8_t*>(in->A);
  a.beta = static_cast<const uint8_t*>(in->D);
  a.dt_bias = static_cast<const uint8_t*>(in->dt_bias);
  a.out = static_cast<uint8_t*>(in->out); a.so = in->so;
  a.dt_qk = in->bc_dtype; a.dt_v = in->x_dtype; a.dt_g = in->dt_dtype; a.dt_beta = in->d_dtype;
  a.dt_alog = in->a_dtype; a.dt_dtb = in->dtb_dtype; a.dt_out = in->out_dtype;
  a.per_key_head = 1; a.dt_softplus = in->dt_softplus; a.dt_clamp = in->dt_clamp;
  a.dt_min = in->dt_min; a.dt_max = in->dt_max; a.scale = 1.0f;
  return launch<sqb::K_M2>(a, st->bits, st->bits > 8 || st->axis_k, static_cast<cudaStream_t>(stream));
}

int sqb_kda_step(const sqb_state_t* st, const sqb_kda_inputs_t* in, void* stream) {
  int lpr_log2 = 0;
  if (int rc = check_state(st, sqb::K_KDA, &lpr_log2)) return rc;
  if (!in) return fail(SQB_EINVAL, "inputs are NULL");
  if (in->rows <= 0) return in->rows == 0 ? 0 : fail(SQB_EINVAL, "rows %d < 0", in->rows);
  if (!in->q || !in->k || !in->v || !in->g || !in->beta || !in->out) return fail(SQB_EINVAL, "q, k, v, g, beta or out is NULL");
  if (check_dtype(in->qk_dtype, "q/k") || check_dtype(in->v_dtype, "v") || check_dtype(in->g_dtype, "g") ||
      check_dtype(in->out_dtype, "out")) return SQB_EINVAL;
  sqb::StepArgs a;
  memset(&a, 0, sizeof a);
  if (int rc = fill_state(a, st, lpr_log2)) return rc;
  a.rows = in->rows; a.idx = in->idx;
  a.q = static_cast<const uint8_t*>(in->q); a.sq = in->sq;
  a.k = static_cast<const uint8_t*>(in->k); a.sk = in->sk;
  a.v = static_cast<const uint8_t*>(in->v); a.sv = in->sv;
  a.g = static_cast<const uint8_t*>(in->g); a.sg = in->sg;
  a.beta = static_cast<const uint8_t*>(in->beta); a.sbeta = in->sbeta;
  a.out = static_cast<uint8_t*>(in->out); a.so = in->so;
  a.dt_qk = in->qk_dtype; a.dt_v = in->v_dtype; a.dt_g = in->g_dtype; a.dt_beta = in->beta_dtype;
  a.dt_out = in->out_dtype; a.per_key_head = 1; a.scale = in->scale;
  return launch<sqb::K_KDA>(a, st->bits, st->bits > 8 || st->axis_k, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

// ---- GGA / STEP -----------------------------------------------------------------------------------------------------
namespace {

int check_gga(const sqb_gga_layout_t* L, bool need_plan) {
  if (!L || !L->blob) return fail(SQB_EINVAL, "GGA layout or blob is NULL");
  if (need_plan && (!L->offs || !L->bits || !L->w)) return fail(SQB_EINVAL, "GGA plan arrays (offs, bits, w) are NULL");
  if (L->dk <= 0 || L->dv <= 0 || L->dk % 2 || L->dv % 32 || L->dv > 128 || L->dk > 256)
    return fail(SQB_EINVAL, "GGA head dims d_k %d, d_v %d: d_k even <= 256, d_v a multiple of 32 <= 128", L->dk, L->dv);
  if (L->hv <= 0 || L->hk <= 0 || L->hv % L->hk) return fail(SQB_EINVAL, "heads hv %d, hk %d", L->hv, L->hk);
  if (L->group != 32) return fail(SQB_EINVAL, "GGA column group %d: expected 32", L->group);
  if (L->pw && (L->m < 1 || L->m > 64)) return fail(SQB_EINVAL, "window length %d", L->m);
  if (L->stride % 16 || (reinterpret_cast<uintptr_t>(L->blob) & 15)) return fail(SQB_EINVAL, "GGA blob: base and slot stride must be multiples of 16 bytes");
  return 0;
}

void fill_gga(sqb::GgaArgs& a, const sqb_gga_layout_t* L) {
  memset(&a, 0, sizeof a);
  a.blob = static_cast<uint8_t*>(L->blob); a.stride = L->stride;
  a.offs = L->offs; a.bits = L->bits; a.w = L->w; a.qoff = L->qoff; a.qsz = L->qsz;
  a.HV = L->hv; a.HK = L->hk; a.DK = L->dk; a.DV = L->dv; a.M = L->pw ? L->m : 1; a.pw = L->pw; a.group = L->group;
}

// TAG: one instantiation (and so one cached shared-memory limit per device) per kernel
template <int TAG, typename K>
int launch_gga(K kern, const sqb::GgaArgs& a, long long ctas, cudaStream_t stream) {
  const sqb::GgaSmem plan = sqb::gga_smem(a.DK, a.DV, a.M, a.group);
  const int smem = plan.total * static_cast<int>(sizeof(float));
  if (smem > 200 * 1024) return fail(SQB_EINVAL, "GGA tile needs %d bytes of shared memory", smem);
  static sqb::SmemLimit limit;
  cudaError_t e = limit.ensure(kern, smem);
  if (e != cudaSuccess) return fail(SQB_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  if (ctas <= 0) return 0;
  kern<<<static_cast<unsigned>(ctas), sqb::GNT, smem, stream>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(SQB_ECUDA, "kernel launch: %s", cudaGetErrorString(e));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

}  // namespace

extern "C" {

int sqb_gga_step(const sqb_gga_layout_t* L, const sqb_gdn_inputs_t* in, void* stream) {
  if (int rc = check_gga(L, true)) return rc;
  if (!in) return fail(SQB_EINVAL, "inputs are NULL");
  if (in->rows <= 0) return in->rows == 0 ? 0 : fail(SQB_EINVAL, "rows %d < 0", in->rows);
  if (!in->gate || !in->a || !in->b || !in->A_log || !in->dt_bias) return fail(SQB_EINVAL, "the GGA step takes the gate inputs (a, b, A_log, dt_bias)");
  if (!in->idx || !in->q || !in->k || !in->v || !in->out) return fail(SQB_EINVAL, "idx, q, k, v or out is NULL");
  sqb::GgaArgs a;
  fill_gga(a, L);
  a.rows = in->rows; a.idx = in->idx;
  a.q = static_cast<const uint8_t*>(in->q); a.sq = in->sq; a.k = static_cast<const uint8_t*>(in->k); a.sk = in->sk;
  a.v = static_cast<const uint8_t*>(in->v); a.sv = in->sv;
  a.a = static_cast<const uint8_t*>(in->a); a.sa = in->sa; a.b = static_cast<const uint8_t*>(in->b); a.sb = in->sb;
  a.A_log = static_cast<const uint8_t*>(in->A_log); a.dt_bias = static_cast<const uint8_t*>(in->dt_bias);
  a.out = static_cast<uint8_t*>(in->out); a.so = in->so;
  a.dt_qk = in->qk_dtype; a.dt_v = in->v_dtype; a.dt_ab = in->ab_dtype; a.dt_alog = in->alog_dtype;
  a.dt_dtb = in->dtb_dtype; a.dt_out = in->out_dtype; a.scale = in->scale;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long ctas = static_cast<long long>(in->rows) * L->hv;
  a.status = status_ptr();
  if (!a.status) return fail(SQB_ECUDA, "the device status word is not reachable (cudaGetSymbolAddress failed)");
  a.wait_ns = static_cast<unsigned long long>(g_wait_ns.load(std::memory_order_relaxed));
  a.test_extra_tx = g_test_extra_tx.load(std::memory_order_relaxed);
  // heads of width 4 / 6 / 8 (128 x 128): the register-tile kernel; 2-bit heads, pivots and other shapes: the tile kernel
  bool reg = L->dk == 128 && L->dv == 128 && g_kernel_path.load(std::memory_order_relaxed) != 1 &&
             !g_force_generic.load(std::memory_order_relaxed);
  if (reg) {
    const int rc = sqb::launch_gga_reg(a, ctas, st);
    if (rc < 0) return fail(SQB_ECUDA, "kernel launch: %s", cudaGetErrorString(static_cast<cudaError_t>(-rc - 1000)));
    if (rc == 0) g_launches.fetch_add(1, std::memory_order_relaxed);
    else reg = false;
  }
  a.skip_packed = reg ? 1 : 0;
  if (!(reg && (L->flags & SQB_GGA_ALL_PACKED))) {
    if (L->dk == 128 && L->dv == 128) {
      if (int rc = launch_gga<0>(sqb::gga_step_kernel<128, 128>, a, ctas, st)) return rc;
    } else {
      if (int rc = launch_gga<1>(sqb::gga_step_kernel<0, 0>, a, ctas, st)) return rc;
    }
  }
  if (L->pw) {
    sqb::gga_advance_kernel<<<(in->rows + 127) / 128, 128, 0, st>>>(a.blob, a.stride, a.idx, in->rows, L->m);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(SQB_ECUDA, "kernel launch: %s", cudaGetErrorString(e));
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  return 0;
}

int sqb_gga_store(const sqb_gga_layout_t* L, const int32_t* idx, int64_t P, const float* X, void* stream) {
  if (int rc = check_gga(L, true)) return rc;
  if (P <= 0) return P == 0 ? 0 : fail(SQB_EINVAL, "P < 0");
  if (!idx || !X) return fail(SQB_EINVAL, "idx or X is NULL");
  sqb::GgaArgs a;
  fill_gga(a, L);
  a.idx = idx; a.X = X; a.P = P;
  return launch_gga<2>(sqb::gga_store_kernel, a, P * L->hv, static_cast<cudaStream_t>(stream));
}

int sqb_gga_load(const sqb_gga_layout_t* L, const int32_t* idx, int64_t P, float* Y, void* stream) {
  if (int rc = check_gga(L, true)) return rc;
  if (P <= 0) return P == 0 ? 0 : fail(SQB_EINVAL, "P < 0");
  if (!idx || !Y) return fail(SQB_EINVAL, "idx or Y is NULL");
  sqb::GgaArgs a;
  fill_gga(a, L);
  a.idx = idx; a.Y = Y; a.P = P;
  return launch_gga<3>(sqb::gga_load_kernel, a, P * L->hv, static_cast<cudaStream_t>(stream));
}

int sqb_stepquant_fit(const float* x, float* y, const int32_t* bits, const float* w, int64_t B, int32_t H, int32_t dk,
                      int32_t dv, int32_t group, void* stream) {
  if (!x || !y || !bits || !w) return fail(SQB_EINVAL, "x, y, bits or w is NULL");
  if (dk <= 0 || dv <= 0 || dk % 2 || dv % 32 || dv > 128 || dk > 256 || group != 32)
    return fail(SQB_EINVAL, "fit: d_k %d even <= 256, d_v %d a multiple of 32 <= 128, group %d = 32", dk, dv, group);
  if (B <= 0) return B == 0 ? 0 : fail(SQB_EINVAL, "B < 0");
  sqb::GgaArgs a;
  memset(&a, 0, sizeof a);
  a.bits = bits; a.w = w; a.HV = H; a.HK = H; a.DK = dk; a.DV = dv; a.M = 1; a.group = group; a.X = x; a.Y = y;
  return launch_gga<4>(sqb::stepquant_fit_kernel, a, B * H, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
