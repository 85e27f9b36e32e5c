// C-ABI entry points (include/sepflow_b200.h): argument validation, workspace carving, TMA tensor
// map encoding and the launch sequence of each op.  No torch types, no allocation.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>
#include <vector>

#include "../../include/sepflow_b200.h"
#include "kernels.h"

namespace {

using namespace sfb;

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// cuTensorMapEncodeTiled is looked up at run time so the library loads (and its symbols can be
// inspected) on machines without a CUDA driver.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// cuTensorMapEncodeTiled is a driver call and needs a context that is current to the calling thread.  A thread that
// has made no runtime call yet (an autograd worker whose first node is one of these ops) has none.  Whether one is
// current is asked of the driver (cuCtxGetCurrent, which allocates nothing and is legal at any time); only when
// there is none does the thread bind the device's primary context with cudaFree(0), once.
typedef CUresult (*CtxGetCurrentFn)(CUcontext*);
int bind_context() {
  static thread_local bool bound = false;
  if (bound) return SFB_OK;
  static CtxGetCurrentFn get_current = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return reinterpret_cast<CtxGetCurrentFn>(p);
    return static_cast<CtxGetCurrentFn>(nullptr);
  }();
  CUcontext ctx = nullptr;
  if (get_current == nullptr || get_current(&ctx) != CUDA_SUCCESS || ctx == nullptr) {
    cudaError_t e = cudaFree(nullptr);
    if (e != cudaSuccess) return fail(SFB_ERR_CUDA, "cudaFree(0): %s", cudaGetErrorString(e));
  }
  bound = true;
  return SFB_OK;
}
#define SFB_TRY_BIND_CONTEXT()                 \
  do {                                         \
    int rc_ = bind_context();                  \
    if (rc_ != SFB_OK) return rc_;             \
  } while (0)

// Tiled fp32 tensor map, 128-byte swizzle, innermost box = 32 channels (128 bytes), zero fill out of bounds.
// dims/box are innermost-first; strides are implied by a contiguous tensor.
// `pitch0` (elements, optional): distance between consecutive indices of dimension 1 when the rows are padded.
int make_map(CUtensorMap* tm, const void* base, int rank, const uint64_t* dims, const uint32_t* box,
             CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B, bool bf16 = false, uint64_t pitch0 = 0) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(SFB_ERR_CUDA, "cuTensorMapEncodeTiled is not available (no CUDA driver?)");
  if (base == nullptr) return fail(SFB_ERR_INVALID_ARGUMENT, "internal: tensor map over an array this workspace does not hold");
  SFB_TRY_BIND_CONTEXT();
  cuuint64_t gdim[5], gstride[5];
  cuuint32_t bdim[5], estride[5];
  uint64_t stride = bf16 ? 2 : sizeof(float);
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estride[i] = 1;
    stride *= (i == 0 && pitch0 != 0) ? pitch0 : dims[i];
    if (i < rank - 1) gstride[i] = stride;  // byte stride of dimension i+1
  }
  CUresult r = fn(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank,
                  const_cast<void*>(base), gdim, gstride,
                  bdim, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SFB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return SFB_OK;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

namespace sfb {
cudaError_t encode_plain_map(CUtensorMap* tm, const void* base, int rank, const uint64_t* dims,
                             const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr || bind_context() != SFB_OK) return cudaErrorNotSupported;
  cuuint64_t gdim[5], gstride[5];
  cuuint32_t bdim[5], estride[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estride[i] = 1;
    if (i < rank - 1) gstride[i] = strides_bytes[i];
  }
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride, bdim,
                        estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}
}  // namespace sfb

namespace {

// ---- optional per-kernel timing (off by default): CUDA events around each launch on its own stream ----
enum KernelId : int {
  KID_PREPARE = 0, KID_PACK, KID_SWEEP_MAXAVG, KID_SWEEP_COMPRESS, KID_SWEEP_DUMP, KID_GRAD_MAXAVG_IMG1, KID_GRAD_MAXAVG_IMG2,
  KID_GRAD_COMPRESS_IMG1, KID_GRAD_COMPRESS_IMG2, KID_GRAD_FUSED_IMG1, KID_GRAD_FUSED_IMG2, KID_ATTENTION_FWD,
  KID_ATTENTION_BWD, KID_LOOKUP, KID_RESAMPLE, KID_LOOKUP4D, KID_COUNT
};
const char* const kKernelNames[KID_COUNT] = {
    "prepare(round_copy+f2_means)", "pack_kernel/unpack_kernel", "sweep_kernel<maxavg>", "sweep_kernel<compress>", "sweep_kernel<dump>",
    "grad_gemm_kernel<maxavg,image1-major>", "grad_gemm_kernel<maxavg,image2-major>",
    "grad_gemm_kernel<compress,image1-major>", "grad_gemm_kernel<compress,image2-major>",
    "grad_gemm_kernel<fused,image1-major>", "grad_gemm_kernel<fused,image2-major>",
    "attention_forward_kernel", "attention backward (logit, input, weight grads)",
    "lookup kernels (pyramid, forward, backward)", "upsample_displacement kernels",
    "lookup4d kernels (forward, backward)"};
struct TimingRec { cudaEvent_t e0, e1; int id; int launches; };
std::mutex g_timing_mu;
bool g_timing_on = false;
std::vector<TimingRec> g_timing_pending;
std::vector<cudaEvent_t> g_event_pool;
double g_timing_ms[KID_COUNT] = {0};
long long g_timing_launches[KID_COUNT] = {0};

cudaEvent_t take_event() {
  if (!g_event_pool.empty()) { cudaEvent_t e = g_event_pool.back(); g_event_pool.pop_back(); return e; }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}

template <class Launch>
cudaError_t timed(int id, int launches, cudaStream_t st, Launch&& launch) {
  bool on;
  TimingRec rec{nullptr, nullptr, id, launches};
  {
    std::lock_guard<std::mutex> lk(g_timing_mu);
    on = g_timing_on;
    if (on) { rec.e0 = take_event(); rec.e1 = take_event(); }
  }
  if (on) cudaEventRecord(rec.e0, st);
  cudaError_t err = launch();
  if (on) {
    cudaEventRecord(rec.e1, st);
    std::lock_guard<std::mutex> lk(g_timing_mu);
    g_timing_pending.push_back(rec);
  }
  return err;
}

void drain_timing_locked() {
  for (TimingRec& r : g_timing_pending) {
    float ms = 0.f;
    if (cudaEventSynchronize(r.e1) == cudaSuccess && cudaEventElapsedTime(&ms, r.e0, r.e1) == cudaSuccess) {
      g_timing_ms[r.id] += ms;
      g_timing_launches[r.id] += r.launches;
    }
    g_event_pool.push_back(r.e0);
    g_event_pool.push_back(r.e1);
  }
  g_timing_pending.clear();
}

// Operand type of the contractions (sfb_set_sweep_operands): FP16 (default), TF32 or BF16.  Process-wide, because
// a backward runs on an autograd worker thread, not on the thread that chose the precision.
int initial_operands() {  // SFB_OPERANDS=tf32|bf16|fp16 in the environment chooses the initial setting
  const char* e = getenv("SFB_OPERANDS");
  if (e != nullptr) {
    if (strcmp(e, "tf32") == 0) return SFB_OPERANDS_TF32;
    if (strcmp(e, "bf16") == 0) return SFB_OPERANDS_BF16;
  }
  return SFB_OPERANDS_FP16;
}
std::atomic<int> g_sweep_operands{initial_operands()};

// Test hook (sfb_debug_wait_timeout): time limit handed to the kernels' bounded waits and whether the next sweeps
// leave out their last load.  Process-wide; 0 / 0 = normal operation.
std::atomic<unsigned long long> g_wait_limit_ns{0};
std::atomic<int> g_drop_last_load{0};
SweepArgs with_wait_settings(SweepArgs a) {
  a.wait_limit_ns = g_wait_limit_ns.load();
  a.drop_last_load = g_drop_last_load.load();
  return a;
}
GradArgs with_wait_settings(GradArgs a) {
  a.wait_limit_ns = g_wait_limit_ns.load();
  return a;
}

struct Workspace {
  int* status;
  float* scales;  // scale slots of the FP16 operand kind (kernels.h, SCALE_*), in the header after the status word
  float* F1r;
  float* F2r;
  float* aux;
  uint16_t* F1h;  // 16-bit copies (FP16 or BF16) of the three arrays above: operands of the kind::f16 sweeps
  uint16_t* F2h;
  uint16_t* auxh;
  float* xu;   // packed inputs indexed by (u, slot, pixel): (B, H2, Rx, n1p)
  float* xv;   // packed inputs indexed by (v, slot, pixel): (B, W2, Rx, n1p)
  float* ou;   // packed outputs, (B, H2, Ro, n1p)
  float* ov;   // packed outputs, (B, W2, Ro, n1p)
  float* gxu;  // interleaved gradient-GEMM operands, (B, H2, n1p, Rg)
  float* gxv;  // interleaved gradient-GEMM operands, (B, W2, n1p, Rg)
  float* F1t;  // channel-major copies of F1r / F2r for K-major B operands: (B, C, n1p) and, in column blocks of 16
  float* F2t;  // with an even number of rows, (B, C, ceil(W2/16), h2p, 16)
  int h2p;     // H2 rounded up to a multiple of GG_UT
  float* ga_u;  // level backward: attention gradients (B, Kc, W2, N1) / (B, Kc, H2, N1) ...
  float* ga_v;
  float* gm_u;  // ... total gradients of the max/avg channels (B, 2, W2, N1) / (B, 2, H2, N1) ...
  float* gm_v;
  float* at_partial;  // ... and the attention backward's per-block partial sums
  int n1p;
  size_t bytes;
};

int padded_pixels(const Dims& d) { return (d.N1() + TILE_M - 1) / TILE_M * TILE_M; }

// (B, D, slots, n1p) workspace array, optionally starting at slot `slot0`
PixView packed_view(float* base, int D, int slots, int n1p, int slot0 = 0) {
  return PixView{base + (size_t)slot0 * n1p, (long long)D * slots * n1p, (uint32_t)(slots * n1p), (uint32_t)n1p};
}
// (B, slots, D, N1) user tensor
PixView cf_view(const void* base, int slots, int D, int N1) {
  return PixView{static_cast<float*>(const_cast<void*>(base)), (long long)slots * D * N1, (uint32_t)N1, (uint32_t)(D * N1)};
}

// What an op keeps in the workspace: the mean rows of F2, Rx packed input slots, Ro packed output slots.
struct WsPlan { bool aux; int Rx; int Ro; int Rg; bool level_bwd; bool bf16; };
constexpr int MAXAVG_SLOTS = 3;  // max, mean, argmax bits
int chunk_channels(int Kc) { return Kc < KC_MAX_PER_SWEEP ? Kc : KC_MAX_PER_SWEEP; }
int grad_slots(int kc) { return 2 * kc <= 4 ? 4 : 8; }  // two slots per channel, rounded up to a multiple of 4

WsPlan plan_for(int op, const Dims& d) {
  switch (op) {
    case SFB_OP_MAX_AVG_FORWARD: return {true, 0, MAXAVG_SLOTS, 0, false, true};
    case SFB_OP_COMPRESSION_FORWARD: return {false, d.Kc, d.Kc, 0, false, true};
    case SFB_OP_MAX_ARGMAX_AVG_BACKWARD: return {false, 0, 0, 4, false, false};
    case SFB_OP_COMPRESSION_BACKWARD: return {false, d.Kc, d.Kc, grad_slots(chunk_channels(d.Kc)), false, true};
    case SFB_OP_SEPARATION_BACKWARD: return {false, d.Kc, d.Kc, 4 + grad_slots(chunk_channels(d.Kc)), false, true};
    case SFB_OP_MAX_AVG_FORWARD_CF: return {true, 0, 0, 0, false, true};
    case SFB_OP_COMPRESSION_CF: return {false, 0, 0, 0, false, true};
    case SFB_OP_SEPARATION_FEATURE_BACKWARD_CF: return {false, 0, 0, 4 + grad_slots(chunk_channels(d.Kc)), false, false};
    case SFB_OP_SEPARATION_LEVEL_FORWARD: return {true, 0, 0, 0, false, true};
    case SFB_OP_SEPARATION_LEVEL_BACKWARD: return {false, 0, 0, 4 + grad_slots(chunk_channels(d.Kc)), true, true};
    default: return {false, 0, 0, 0, false, false};
  }
}

Workspace carve(const Dims& d, void* base, const WsPlan& plan) {
  Workspace w;
  size_t off = 0;
  char* p = static_cast<char*>(base);
  auto take = [&](size_t floats) {
    float* r = reinterpret_cast<float*>(p + off);
    off += align_up(floats * sizeof(float), 256);
    return r;
  };
  w.status = reinterpret_cast<int*>(p + off);
  w.scales = reinterpret_cast<float*>(p + off + WS_SCALES_OFFSET);
  off += WS_HEADER_BYTES;
  w.n1p = padded_pixels(d);
  w.F1r = take((size_t)d.B * d.N1() * d.C);
  w.F2r = take((size_t)d.B * d.N2() * d.C);
  w.aux = plan.aux ? take((size_t)d.B * d.aux_rows() * d.C) : nullptr;
  w.F1h = w.F2h = w.auxh = nullptr;
  if (plan.bf16) {   // half the floats of the fp32 copies
    w.F1h = reinterpret_cast<uint16_t*>(take(((size_t)d.B * d.N1() * d.C + 1) / 2));
    w.F2h = reinterpret_cast<uint16_t*>(take(((size_t)d.B * d.N2() * d.C + 1) / 2));
    w.auxh = reinterpret_cast<uint16_t*>(take(((size_t)d.B * d.aux_rows() * d.C + 1) / 2));
  }
  w.xu = plan.Rx ? take((size_t)d.B * d.H2 * plan.Rx * w.n1p) : nullptr;
  w.xv = plan.Rx ? take((size_t)d.B * d.W2 * plan.Rx * w.n1p) : nullptr;
  w.ou = plan.Ro ? take((size_t)d.B * d.H2 * plan.Ro * w.n1p) : nullptr;
  w.ov = plan.Ro ? take((size_t)d.B * d.W2 * plan.Ro * w.n1p) : nullptr;
  w.gxu = plan.Rg ? take((size_t)d.B * d.H2 * plan.Rg * w.n1p) : nullptr;
  w.gxv = plan.Rg ? take((size_t)d.B * d.W2 * plan.Rg * w.n1p) : nullptr;
  w.h2p = (d.H2 + GG_UT - 1) / GG_UT * GG_UT;
  w.F1t = w.F2t = nullptr;
  if (plan.Rg) {
    w.F1t = take((size_t)d.B * d.C * w.n1p);
    w.F2t = take((size_t)d.B * d.C * ((d.W2 + GG_VT - 1) / GG_VT) * w.h2p * GG_VT);
  }
  w.ga_u = w.ga_v = w.gm_u = w.gm_v = w.at_partial = nullptr;
  if (plan.level_bwd) {
    const size_t n1 = (size_t)d.N1();
    w.ga_u = take((size_t)d.B * d.Kc * d.W2 * n1);
    w.ga_v = take((size_t)d.B * d.Kc * d.H2 * n1);
    w.gm_u = take((size_t)d.B * 2 * d.W2 * n1);
    w.gm_v = take((size_t)d.B * 2 * d.H2 * n1);
    w.at_partial = take(attention_partial_floats(AttentionDims{d.B, d.Kc, d.H2 > d.W2 ? d.H2 : d.W2, d.H1, d.W1}));
  }
  w.bytes = off;
  return w;
}

int check_shape(const sfb_shape* s, bool need_kc, Dims* d) {
  if (s == nullptr) return fail(SFB_ERR_INVALID_ARGUMENT, "shape is NULL");
  if (s->B < 1 || s->H1 < 1 || s->W1 < 1 || s->H2 < 1 || s->W2 < 1)
    return fail(SFB_ERR_INVALID_ARGUMENT, "B, H1, W1, H2, W2 must be >= 1 (got %d %d %d %d %d)", s->B, s->H1, s->W1,
                s->H2, s->W2);
  if (s->C < 4 || s->C > MAX_C || (s->C % 4) != 0)
    return fail(SFB_ERR_UNSUPPORTED_SHAPE, "feature dimension C=%d unsupported: need a multiple of 4 in [4, %d]", s->C,
                MAX_C);
  if (need_kc && s->Kc < 1) return fail(SFB_ERR_INVALID_ARGUMENT, "Kc must be >= 1 (got %d)", s->Kc);
  if ((long long)s->H1 * s->W1 > (1ll << 21) || (long long)s->H2 * s->W2 > (1ll << 30))
    return fail(SFB_ERR_UNSUPPORTED_SHAPE, "image 1 has more than 2^21 pixels or image 2 more than 2^30");
  {  // element offsets inside one sample's packed array are 32-bit in the kernels
    const long long n1p = ((long long)s->H1 * s->W1 + TILE_M - 1) / TILE_M * TILE_M;
    const long long kc = need_kc ? s->Kc : 0;  // ops without attention channels ignore (and may not initialise) Kc
    const long long slots = kc + 2 > 8 ? kc + 2 : 8;
    if (n1p * slots * (s->H2 > s->W2 ? s->H2 : s->W2) >= (1ll << 32))
      return fail(SFB_ERR_UNSUPPORTED_SHAPE, "H1*W1*max(H2,W2)*slots exceeds 2^32 elements per sample");
  }
  d->B = s->B; d->H1 = s->H1; d->W1 = s->W1; d->H2 = s->H2; d->W2 = s->W2; d->C = s->C;
  d->Kc = need_kc ? s->Kc : 0;
  return SFB_OK;
}

int check_ptr(const void* p, const char* name) {
  if (p == nullptr) return fail(SFB_ERR_INVALID_ARGUMENT, "%s is NULL", name);
  if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return fail(SFB_ERR_INVALID_ARGUMENT, "%s is not 16-byte aligned", name);
  return SFB_OK;
}
#define SFB_CHECK_PTR(p)                       \
  do {                                         \
    int rc_ = check_ptr((p), #p);              \
    if (rc_ != SFB_OK) return rc_;             \
  } while (0)
#define SFB_TRY(expr)                          \
  do {                                         \
    int rc_ = (expr);                          \
    if (rc_ != SFB_OK) return rc_;             \
  } while (0)
#define SFB_CUDA(expr)                                                                           \
  do {                                                                                           \
    cudaError_t e_ = (expr);                                                                     \
    if (e_ != cudaSuccess) return fail(SFB_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_));  \
  } while (0)

int check_workspace(const Dims& d, void* ws, size_t ws_bytes, int op, Workspace* out) {
  if (ws == nullptr) return fail(SFB_ERR_INVALID_ARGUMENT, "workspace is NULL");
  if ((reinterpret_cast<uintptr_t>(ws) & 255u) != 0)
    return fail(SFB_ERR_INVALID_ARGUMENT, "workspace is not 256-byte aligned");
  *out = carve(d, ws, plan_for(op, d));
  if (ws_bytes < out->bytes)
    return fail(SFB_ERR_WORKSPACE_TOO_SMALL, "workspace has %zu bytes, %zu needed", ws_bytes, out->bytes);
  return SFB_OK;
}

// Tensor maps over the rounded copies.
// `swizzle` is the 16-byte-atom 128B swizzle for K-major operands (rows = pixels of the tile) and the
// 32-byte-atom variant for MN-major TF32 operands (the only layout tcgen05.mma accepts for those).
int map_f1_rows(CUtensorMap* tm, const Dims& d, const void* F1r, uint32_t rows,
                CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B, bool bf16 = false) {  // (C, N1, B)
  const uint64_t dims[3] = {(uint64_t)d.C, (uint64_t)d.N1(), (uint64_t)d.B};
  const uint32_t box[3] = {bf16 ? 2u * KBLK : (uint32_t)KBLK, rows, 1};   // one 128-byte row of channels
  return make_map(tm, F1r, 3, dims, box, swizzle, bf16);
}
int map_f2_tile(CUtensorMap* tm, const Dims& d, const void* F2r, uint32_t ut, uint32_t vt,
                CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B, bool bf16 = false) {  // (C, W2, H2, B)
  const uint64_t dims[4] = {(uint64_t)d.C, (uint64_t)d.W2, (uint64_t)d.H2, (uint64_t)d.B};
  const uint32_t box[4] = {bf16 ? 2u * KBLK : (uint32_t)KBLK, vt, ut, 1};
  return make_map(tm, F2r, 4, dims, box, swizzle, bf16);
}
// Interleaved gradient operands (B, D, Q, n1p, 4), seen by TMA as (4*n1p, Q, D, B) so that the innermost box
// dimension is a long contiguous run (`pixels` * 16 bytes): box = (4*pixels, Q groups, `disps` displacements, 1).
int map_operands(CUtensorMap* tm, const float* x, int B, int D, int Q, int n1p, uint32_t pixels, uint32_t disps) {
  const uint64_t dims[4] = {4ull * (uint64_t)n1p, (uint64_t)Q, (uint64_t)D, (uint64_t)B};
  const uint32_t box[4] = {4 * pixels, (uint32_t)Q, disps, 1};
  return make_map(tm, x, 4, dims, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}
int map_aux(CUtensorMap* tm, const Dims& d, const void* aux, bool bf16 = false) {  // (C, H2+W2, B)
  const uint64_t dims[3] = {(uint64_t)d.C, (uint64_t)d.aux_rows(), (uint64_t)d.B};
  const uint32_t box[3] = {bf16 ? 2u * KBLK : (uint32_t)KBLK, (uint32_t)(SWEEP_UT * SWEEP_VT), 1};
  return make_map(tm, aux, 3, dims, box, CU_TENSOR_MAP_SWIZZLE_128B, bf16);
}

// Operand type of this call's contractions: the process-wide switch (sfb_set_sweep_operands), as OP16_NONE (TF32),
// OP16_BF16 or OP16_FP16.
int operand_mode(const Dims& d, int* op16) {
  const int m = g_sweep_operands.load();
  *op16 = m == SFB_OPERANDS_BF16 ? OP16_BF16 : (m == SFB_OPERANDS_FP16 ? OP16_FP16 : OP16_NONE);
  if (d.C % 8 != 0) {  // 16-bit rows must be multiples of 16 bytes for TMA
    if (*op16 == OP16_BF16)
      return fail(SFB_ERR_UNSUPPORTED_SHAPE, "BF16 operands need a feature dimension that is a multiple of 8 (C=%d)", d.C);
    *op16 = OP16_NONE;  // FP16 and TF32 operands have the same precision: such shapes run with TF32
  }
  return SFB_OK;
}
// What the sweeps multiply their outputs by: the inverse of the feature scales of FP16 operands, else nothing.
const float* sweep_out_scale(const Workspace& w, int op16) {
  return op16 == OP16_FP16 ? w.scales + SCALE_INV_F1F2 : nullptr;
}

// Tensor maps of the sweeps' operands in a workspace: the rounded FP32 copies or the 16-bit copies (aux may be null).
int map_sweep_operands(const Dims& d, const Workspace& w, int op16, CUtensorMap* f1, CUtensorMap* f2, CUtensorMap* aux) {
  if (op16) {
    SFB_TRY(map_f1_rows(f1, d, w.F1h, TILE_M, CU_TENSOR_MAP_SWIZZLE_128B, true));
    SFB_TRY(map_f2_tile(f2, d, w.F2h, SWEEP_UT, SWEEP_VT, CU_TENSOR_MAP_SWIZZLE_128B, true));
    if (aux != nullptr) SFB_TRY(map_aux(aux, d, w.auxh, true));
  } else {
    SFB_TRY(map_f1_rows(f1, d, w.F1r, TILE_M));
    SFB_TRY(map_f2_tile(f2, d, w.F2r, SWEEP_UT, SWEEP_VT));
    if (aux != nullptr) SFB_TRY(map_aux(aux, d, w.aux));
  }
  return SFB_OK;
}

// Rounded copies of a call's features (and of the mean rows of image 2 when with_aux), plus 16-bit copies of kind op16.
cudaError_t prepare_operands(const Dims& d, const Workspace& w, const float* F1, const float* F2, bool with_aux,
                             int op16, cudaStream_t st) {
  // (an op without sweeps has no 16-bit copies in its workspace, but its gradient GEMMs still need the feature scales)
  return launch_prepare(d, F1, F2, w.F1r, w.F2r, with_aux ? w.aux : nullptr, w.status, st, op16 ? w.F1h : nullptr,
                        op16 ? w.F2h : nullptr, op16 && with_aux ? w.auxh : nullptr, op16, w.scales);
}

int run_maxavg_forward(const float* F1, const float* F2, float* MA_u, float* MA_v, int32_t* AM_u, int32_t* AM_v,
                       bool with_argmax, const sfb_shape* shape, void* ws, size_t ws_bytes, void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, false, &d));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(MA_u); SFB_CHECK_PTR(MA_v);
  if (with_argmax) { SFB_CHECK_PTR(AM_u); SFB_CHECK_PTR(AM_v); }
  Workspace w;
  SFB_TRY(check_workspace(d, ws, ws_bytes, SFB_OP_MAX_AVG_FORWARD, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  CUtensorMap tm_f1, tm_f2, tm_aux;
  SFB_TRY(map_sweep_operands(d, w, op16, &tm_f1, &tm_f2, &tm_aux));
  SFB_CUDA(timed(KID_PREPARE, 3 + (op16 == OP16_FP16 ? 3 : 0), st, [&] { return prepare_operands(d, w, F1, F2, true, op16, st); }));
  SweepArgs a;
  memset(&a, 0, sizeof(a));
  a.d = d;
  a.op16 = op16;
  a.out_scale = sweep_out_scale(w, op16);
  a.mode = with_argmax ? SWEEP_MAXARGAVG : SWEEP_MAXAVG;
  a.n_valid = w.n1p;
  a.pu = packed_view(w.ou, d.H2, MAXAVG_SLOTS, w.n1p);
  a.pv = packed_view(w.ov, d.W2, MAXAVG_SLOTS, w.n1p);
  a.pu_arg = packed_view(w.ou, d.H2, MAXAVG_SLOTS, w.n1p, 2);
  a.pv_arg = packed_view(w.ov, d.W2, MAXAVG_SLOTS, w.n1p, 2);
  a.status = w.status;
  SFB_CUDA(timed(KID_SWEEP_MAXAVG, 1, st, [&] { return launch_sweep(with_wait_settings(a), tm_f1, tm_f2, tm_aux, st); }));
  // packed (displacement, slot, pixel) -> the reference's (pixel, channel, displacement) tensors
  const int N1 = d.N1(), R = MAXAVG_SLOTS;
  SFB_CUDA(timed(KID_PACK, with_argmax ? 4 : 2, st, [&] {
    launch_unpack(w.ou, MA_u, d.B, N1, w.n1p, 2, d.H2, R, 0, 1, 2, 0, st);
    cudaError_t e = launch_unpack(w.ov, MA_v, d.B, N1, w.n1p, 2, d.W2, R, 0, 1, 2, 0, st);
    if (with_argmax) {
      launch_unpack(w.ou, AM_u, d.B, N1, w.n1p, 1, d.H2, R, 2, 1, 1, 0, st);
      e = launch_unpack(w.ov, AM_v, d.B, N1, w.n1p, 1, d.W2, R, 2, 1, 1, 0, st);
    }
    return e;
  }));
  return SFB_OK;
}

// ou(b,u,k,p) = sum_v S * w_u[k], ov(b,v,k,p) = sum_u S * w_v[k] for all Kc channels, at most KC_MAX_PER_SWEEP
// channels per sweep.  Weight k is slot (slot0 + k*stride) of the views xu (per u: w_v) / xv (per v: w_u).
int run_compress_sweeps(const Dims& d, int* status, const CUtensorMap& tm_f1, const CUtensorMap& tm_f2, PixView xu,
                        PixView xv, int wu_slot0, int wv_slot0, int w_stride, PixView ou, PixView ov, int n_valid,
                        cudaStream_t st, int op16 = 0, const float* out_scale = nullptr) {
  for (int k0 = 0; k0 < d.Kc; k0 += KC_MAX_PER_SWEEP) {
    SweepArgs a;
    memset(&a, 0, sizeof(a));
    a.d = d;
    a.mode = SWEEP_COMPRESS;
    a.n_valid = n_valid;
    a.k0 = k0;
    a.kc = chunk_channels(d.Kc - k0);
    a.xu = xu; a.xv = xv;
    a.wu_slot0 = wu_slot0; a.wv_slot0 = wv_slot0; a.w_stride = w_stride;
    a.ou = ou; a.ov = ov;
    a.op16 = op16;
    a.out_scale = out_scale;
    a.status = status;
    SFB_CUDA(timed(KID_SWEEP_COMPRESS, 1, st, [&] { return launch_sweep(with_wait_settings(a), tm_f1, tm_f2, tm_f2 /* unused */, st); }));
  }
  return SFB_OK;
}

// out_cf: the gradients are written channel-major, (B, C, pixels), gF1 multiplied by scale1.
int run_grad_pair(const Dims& d, const Workspace& w, int mode, int R4, int accumulate, float* gF1, float* gF2,
                  cudaStream_t st, int out_cf = 0, float scale1 = 1.f) {
  // 16-bit form when the operand switch says so (callers have refused feature dimensions that do not allow it); with
  // FP16 the callers have run grad_operand_scales and packed the operands with those scales
  int op16 = OP16_NONE;
  SFB_TRY(operand_mode(d, &op16));
  const float* const s1 = op16 == OP16_FP16 ? w.scales + SCALE_F1 : nullptr;
  const float* const s2 = op16 == OP16_FP16 ? w.scales + SCALE_F2 : nullptr;
  CUtensorMap tm_y, tm_xu, tm_xv;
  GradArgs a;
  memset(&a, 0, sizeof(a));
  a.d = d;
  a.mode = mode;
  a.R4 = R4;
  a.n1p = w.n1p;
  a.accumulate = accumulate;
  a.xu = w.gxu;
  a.xv = w.gxv;
  a.status = w.status;
  a.op16 = op16;
  const int Q = R4 / 4;
  const int kid = mode == GRAD_MAXAVG ? KID_GRAD_MAXAVG_IMG1 : (mode == GRAD_COMPRESS ? KID_GRAD_COMPRESS_IMG1 : KID_GRAD_FUSED_IMG1);
  // K-major B operands: channel-major copies of the rounded features (image 2 in column blocks of 16 with an even
  // number of rows, so that a 2 x 16 block of the image is 32 consecutive values).  Rows and columns of padding must
  // read as zero: they meet the G values of cells outside the image.
  const uint32_t crows = (uint32_t)((d.C + KBLK - 1) / KBLK * KBLK);  // channel rows of one feature block
  // a row of 32 K-values is 128 bytes of FP32 or 64 bytes of a 16-bit type: the swizzle span follows
  const CUtensorMapSwizzle fswz = op16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  const size_t f2t_per_sample = (size_t)d.C * ((d.W2 + GG_VT - 1) / GG_VT) * w.h2p * GG_VT;
  if (!accumulate) {  // later passes over further channel chunks reuse the copies of the first
    SFB_CUDA(timed(KID_PREPARE, 2, st, [&] {
      cudaMemsetAsync(w.F2t, 0, (size_t)d.B * f2t_per_sample * (op16 ? 2 : sizeof(float)), st);
      launch_channel_major(w.F1r, w.F1t, d.B, 1, d.N1(), w.n1p, d.C, 0, op16, s1, st);
      return launch_channel_major(w.F2r, w.F2t, d.B, d.H2, d.W2, w.h2p, d.C, 1, op16, s2, st);
    }));
  }
  // gF1 = G * F2 : rows are image-1 pixels, the K sweep streams 2 x 16 blocks of F2 and 2-row blocks of XU.
  {  // (blocked pixels, C, B); box = 32 consecutive values (2 rows x 16 columns) x all channels
    const uint64_t dims[3] = {(uint64_t)(f2t_per_sample / d.C), (uint64_t)d.C, (uint64_t)d.B};
    const uint32_t box[3] = {GG_KJ, crows, 1};
    SFB_TRY(make_map(&tm_y, w.F2t, 3, dims, box, fswz, op16 != 0));
  }
  SFB_TRY(map_operands(&tm_xu, w.gxu, d.B, d.H2, Q, w.n1p, TILE_M / 2, GG_UT));  // two 64-pixel boxes per block
  a.out_cf = out_cf;
  a.image2_major = 0;
  a.out = gF1;
  a.out_scale = scale1;
  a.dev_scale = op16 == OP16_FP16 ? w.scales + SCALE_INV_GF1 : nullptr;
  SFB_CUDA(timed(kid, 1, st, [&] { return launch_grad_gemm(with_wait_settings(a), tm_y, tm_xu, tm_xu /* unused */, st); }));
  // gF2 = G^T * F1 : rows are an 8 x 16 block of image-2 pixels, the K sweep streams 32 pixels of F1, XU and XV.
  {  // (N1, C, B) with rows padded to n1p; box = 32 pixels x all channels
    const uint64_t dims[3] = {(uint64_t)d.N1(), (uint64_t)d.C, (uint64_t)d.B};
    const uint32_t box[3] = {GG_KJ, crows, 1};
    SFB_TRY(make_map(&tm_y, w.F1t, 3, dims, box, fswz, op16 != 0, (uint64_t)w.n1p));
  }
  SFB_TRY(map_operands(&tm_xu, w.gxu, d.B, d.H2, Q, w.n1p, GG_KJ, GG_ROW_UT));
  SFB_TRY(map_operands(&tm_xv, w.gxv, d.B, d.W2, Q, w.n1p, GG_KJ, GG_ROW_VT));
  a.image2_major = 1;
  a.out = gF2;
  a.out_scale = 1.f;
  a.dev_scale = op16 == OP16_FP16 ? w.scales + SCALE_INV_GF2 : nullptr;
  SFB_CUDA(timed(kid + 1, 1, st, [&] { return launch_grad_gemm(with_wait_settings(a), tm_y, tm_xu, tm_xv, st); }));
  return SFB_OK;
}

// Interleaved slots of the max/avg backward (kernels.h): XU = (mean-gradient / W2, 1, max-gradient, argmax bits),
// XV = (1, mean-gradient / H2, max-gradient, argmax bits); slots 0 and 1 of the two sides multiply to the mean terms.
// `scales` (FP16 operands, else null): the call's scale slots; the gradient values are then multiplied by sg * sa.
void maxavg_slot_sources(const Dims& d, const int32_t* AM_u, const int32_t* AM_v, const float* gMA_u,
                         const float* gMA_v, SlotSources* su, SlotSources* sv, const float* scales) {
  memset(su, 0, sizeof(*su));
  memset(sv, 0, sizeof(*sv));
  su->s[0] = {gMA_u, 2, 1, 1.f / (float)d.W2};
  su->s[1] = {nullptr, 0, 0, 1.f};
  su->s[2] = {gMA_u, 2, 0, 0.f};
  su->s[3] = {AM_u, 1, 0, 0.f};
  sv->s[0] = {nullptr, 0, 0, 1.f};
  sv->s[1] = {gMA_v, 2, 1, 1.f / (float)d.H2};
  sv->s[2] = {gMA_v, 2, 0, 0.f};
  sv->s[3] = {AM_v, 1, 0, 0.f};
  if (scales != nullptr) {
    su->dev_scales = sv->dev_scales = scales;
    su->s[0].dev = su->s[2].dev = sv->s[1].dev = sv->s[2].dev = SCALE_GA + 1;
  }
}
// Interleaved slots of the compression backward for channels k0 .. k0+kc-1, local channel j:
// XU 2j = gC_u, 2j+1 = A_v;  XV 2j = A_u, 2j+1 = gC_v, so that G[p,u,v] = sum_slots XU[u,p,slot] * XV[v,p,slot].
// The gradients may be channels g0.. of a tensor with gK channels (the concatenated tensors of the call site).
// `scales` (FP16 operands, else null): gradients are multiplied by sg, weights by sa.
void compress_slot_sources(int K, int k0, int kc, const float* A_u, const float* A_v, const float* gC_u,
                           const float* gC_v, SlotSources* su, SlotSources* sv, const float* scales, int gK = 0,
                           int g0 = 0) {
  if (gK == 0) gK = K;
  memset(su, 0, sizeof(*su));
  memset(sv, 0, sizeof(*sv));
  for (int j = 0; j < kc; ++j) {
    su->s[2 * j] = {gC_u, gK, g0 + k0 + j, 0.f};
    su->s[2 * j + 1] = {A_v, K, k0 + j, 0.f};
    sv->s[2 * j] = {A_u, K, k0 + j, 0.f};
    sv->s[2 * j + 1] = {gC_v, gK, g0 + k0 + j, 0.f};
    if (scales != nullptr) {
      su->s[2 * j].dev = sv->s[2 * j + 1].dev = SCALE_G + 1;
      su->s[2 * j + 1].dev = sv->s[2 * j].dev = SCALE_A + 1;
    }
  }
  if (scales != nullptr) su->dev_scales = sv->dev_scales = scales;
}

// FP16 operands: the gradient-operand scales of this call (kernels.h, SCALE_*) from the largest magnitudes of the
// gradient tensors and of the weight tensors that multiply them.  No weight tensors: the weights are softmax outputs,
// known to lie in [0, 1], and their scale stays 1.  Runs after the call's launch_prepare, which cleared the slots and
// found the feature scales.
struct AbsmaxSrc { const float* p; size_t n; };
int grad_operand_scales(const Workspace& w, int op16, std::initializer_list<AbsmaxSrc> grads,
                        std::initializer_list<AbsmaxSrc> weights, cudaStream_t st) {
  if (op16 != OP16_FP16) return SFB_OK;
  SFB_CUDA(timed(KID_PREPARE, (int)(grads.size() + weights.size()) + 1, st, [&] {
    for (const AbsmaxSrc& g : grads) launch_absmax(g.p, g.n, 1.f, w.scales + SCALE_AMAX_G, st);
    for (const AbsmaxSrc& a : weights) launch_absmax(a.p, a.n, 1.f, w.scales + SCALE_AMAX_A, st);
    return launch_grad_scales(w.scales, st);
  }));
  return SFB_OK;
}
const float* grad_slot_scales(const Workspace& w, int op16) { return op16 == OP16_FP16 ? w.scales : nullptr; }

// Attention gradients of the compression backward: gA_v[p,k,u] = sum_v S * gC_v[p,k,v] and
// gA_u[p,k,v] = sum_u S * gC_u[p,k,u] -- the forward compression sweep with the upstream gradients in the
// role of the weights (w_u = gC_v, w_v = gC_u).
int run_attention_grads(const Dims& d, const Workspace& w, const float* gC_u, const float* gC_v, float* gA_u,
                        float* gA_v, cudaStream_t st, int op16) {
  CUtensorMap tm_f1, tm_f2;
  SFB_TRY(map_sweep_operands(d, w, op16, &tm_f1, &tm_f2, nullptr));
  const int N1 = d.N1(), K = d.Kc;
  SFB_CUDA(timed(KID_PACK, 2, st, [&] {
    launch_pack(gC_v, w.xv, d.B, N1, w.n1p, K, 0, K, d.W2, K, 0, 1, 0.f, st);
    return launch_pack(gC_u, w.xu, d.B, N1, w.n1p, K, 0, K, d.H2, K, 0, 1, 0.f, st);
  }));
  SFB_TRY(run_compress_sweeps(d, w.status, tm_f1, tm_f2, packed_view(w.xu, d.H2, K, w.n1p), packed_view(w.xv, d.W2, K, w.n1p),
                              0, 0, 1, packed_view(w.ou, d.H2, K, w.n1p), packed_view(w.ov, d.W2, K, w.n1p), w.n1p, st, op16, sweep_out_scale(w, op16)));
  SFB_CUDA(timed(KID_PACK, 2, st, [&] {
    launch_unpack(w.ou, gA_v, d.B, N1, w.n1p, K, d.H2, K, 0, 1, K, 0, st);
    return launch_unpack(w.ov, gA_u, d.B, N1, w.n1p, K, d.W2, K, 0, 1, K, 0, st);
  }));
  return SFB_OK;
}

// ---- scratch that lives in the library image, for callers that must not allocate ----
constexpr size_t STATIC_SCRATCH_BYTES = 32u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_static_mu;
void* g_static_scratch_ptr[MAX_DEVICES] = {nullptr};

// Device address of g_static_scratch on the current device.  In host code the symbol's name is only a
// handle, not an address a kernel could use, so the address is looked up once per device (with that
// device current) and cached.
int static_scratch(void** out) {
  int dev = -1;
  SFB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return fail(SFB_ERR_CUDA, "device ordinal %d outside [0, %d)", dev, MAX_DEVICES);
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    SFB_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    g_static_scratch_ptr[dev] = p;
  }
  *out = g_static_scratch_ptr[dev];
  return SFB_OK;
}

}  // namespace

extern "C" {

size_t sfb_workspace_bytes(int op, const sfb_shape* shape) {
  Dims d;
  if (op < SFB_OP_MAX_AVG_FORWARD || op > SFB_OP_SEPARATION_LEVEL_BACKWARD) return 0;
  const bool need_kc = op == SFB_OP_COMPRESSION_FORWARD || op == SFB_OP_COMPRESSION_BACKWARD ||
                       op == SFB_OP_SEPARATION_BACKWARD || op == SFB_OP_COMPRESSION_CF ||
                       op == SFB_OP_SEPARATION_FEATURE_BACKWARD_CF || op == SFB_OP_SEPARATION_LEVEL_FORWARD ||
                       op == SFB_OP_SEPARATION_LEVEL_BACKWARD;
  if (check_shape(shape, need_kc, &d) != SFB_OK) return 0;
  return carve(d, nullptr, plan_for(op, d)).bytes;
}

int sfb_max_avg_forward(const float* F1, const float* F2, float* MA_u, float* MA_v, const sfb_shape* shape,
                        void* workspace, size_t workspace_bytes, void* stream) {
  return run_maxavg_forward(F1, F2, MA_u, MA_v, nullptr, nullptr, false, shape, workspace, workspace_bytes, stream);
}

int sfb_max_avg_forward_static(const float* F1, const float* F2, float* MA_u, float* MA_v, const sfb_shape* shape,
                               void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, false, &d));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(MA_u); SFB_CHECK_PTR(MA_v);
  WsPlan plan = plan_for(SFB_OP_MAX_AVG_FORWARD, d);
  plan.bf16 = false;  // this entry point always computes with TF32 operands: no room is set aside for 16-bit copies
  const size_t need = carve(d, nullptr, plan).bytes;
  if (need > STATIC_SCRATCH_BYTES)
    return fail(SFB_ERR_UNSUPPORTED_SHAPE,
                "this shape needs %zu bytes of scratch but the built-in scratch holds %zu; use sfb_max_avg_forward "
                "with a caller-provided workspace", need, (size_t)STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  SFB_TRY(static_scratch(&scratch));
  const Workspace w = carve(d, scratch, plan);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap tm_f1, tm_f2, tm_aux;
  SFB_TRY(map_f1_rows(&tm_f1, d, w.F1r, TILE_M));
  SFB_TRY(map_f2_tile(&tm_f2, d, w.F2r, SWEEP_UT, SWEEP_VT));
  SFB_TRY(map_aux(&tm_aux, d, w.aux));
  // launch_prepare clears the status word; every other byte of the scratch that is read below is
  // written first by these launches, so nothing depends on what an earlier call left behind
  SFB_CUDA(launch_prepare(d, F1, F2, w.F1r, w.F2r, w.aux, w.status, st));
  SweepArgs a;
  memset(&a, 0, sizeof(a));
  a.d = d;
  a.mode = SWEEP_MAXAVG;
  a.n_valid = w.n1p;
  a.pu = packed_view(w.ou, d.H2, MAXAVG_SLOTS, w.n1p);
  a.pv = packed_view(w.ov, d.W2, MAXAVG_SLOTS, w.n1p);
  a.status = w.status;
  SFB_CUDA(launch_sweep(with_wait_settings(a), tm_f1, tm_f2, tm_aux, st));
  SFB_CUDA(launch_unpack(w.ou, MA_u, d.B, d.N1(), w.n1p, 2, d.H2, MAXAVG_SLOTS, 0, 1, 2, 0, st));
  SFB_CUDA(launch_unpack(w.ov, MA_v, d.B, d.N1(), w.n1p, 2, d.W2, MAXAVG_SLOTS, 0, 1, 2, 0, st));
  return SFB_OK;
}

size_t sfb_static_scratch_bytes(void) { return STATIC_SCRATCH_BYTES; }

int sfb_static_device_status(void* stream, int32_t* device_status) {
  void* scratch = nullptr;
  SFB_TRY(static_scratch(&scratch));  // the status word is the first word of the built-in scratch
  return sfb_device_status(scratch, stream, device_status);
}

int sfb_max_argmax_avg_forward(const float* F1, const float* F2, float* MA_u, float* MA_v, int32_t* AM_u,
                               int32_t* AM_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                               void* stream) {
  return run_maxavg_forward(F1, F2, MA_u, MA_v, AM_u, AM_v, true, shape, workspace, workspace_bytes, stream);
}

int sfb_compression_forward(const float* F1, const float* F2, const float* A_u, const float* A_v, float* C_u,
                            float* C_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                            void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, true, &d));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(A_u); SFB_CHECK_PTR(A_v); SFB_CHECK_PTR(C_u); SFB_CHECK_PTR(C_v);
  Workspace w;
  SFB_TRY(check_workspace(d, workspace, workspace_bytes, SFB_OP_COMPRESSION_FORWARD, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  CUtensorMap tm_f1, tm_f2;
  SFB_TRY(map_sweep_operands(d, w, op16, &tm_f1, &tm_f2, nullptr));
  SFB_CUDA(timed(KID_PREPARE, 2 + (op16 == OP16_FP16 ? 3 : 0), st, [&] { return prepare_operands(d, w, F1, F2, false, op16, st); }));
  const int N1 = d.N1(), K = d.Kc;
  SFB_CUDA(timed(KID_PACK, 2, st, [&] {
    launch_pack(A_u, w.xv, d.B, N1, w.n1p, K, 0, K, d.W2, K, 0, 1, 0.f, st);         // w_u[k][v] = XV slot k
    return launch_pack(A_v, w.xu, d.B, N1, w.n1p, K, 0, K, d.H2, K, 0, 1, 0.f, st);  // w_v[k][u] = XU slot k
  }));
  SFB_TRY(run_compress_sweeps(d, w.status, tm_f1, tm_f2, packed_view(w.xu, d.H2, K, w.n1p), packed_view(w.xv, d.W2, K, w.n1p),
                              0, 0, 1, packed_view(w.ou, d.H2, K, w.n1p), packed_view(w.ov, d.W2, K, w.n1p), w.n1p, st, op16, sweep_out_scale(w, op16)));
  SFB_CUDA(timed(KID_PACK, 2, st, [&] {
    launch_unpack(w.ou, C_u, d.B, N1, w.n1p, K, d.H2, K, 0, 1, K, 0, st);
    return launch_unpack(w.ov, C_v, d.B, N1, w.n1p, K, d.W2, K, 0, 1, K, 0, st);
  }));
  return SFB_OK;
}

int sfb_max_argmax_avg_backward(const float* F1, const float* F2, const int32_t* AM_u, const int32_t* AM_v,
                                const float* gMA_u, const float* gMA_v, float* gF1, float* gF2,
                                const sfb_shape* shape, void* workspace, size_t workspace_bytes, void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, false, &d));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(AM_u); SFB_CHECK_PTR(AM_v);
  SFB_CHECK_PTR(gMA_u); SFB_CHECK_PTR(gMA_v); SFB_CHECK_PTR(gF1); SFB_CHECK_PTR(gF2);
  Workspace w;
  SFB_TRY(check_workspace(d, workspace, workspace_bytes, SFB_OP_MAX_ARGMAX_AVG_BACKWARD, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  SFB_CUDA(timed(KID_PREPARE, 2 + (op16 == OP16_FP16 ? 3 : 0), st, [&] { return prepare_operands(d, w, F1, F2, false, op16, st); }));
  const size_t pix = (size_t)d.B * d.N1();
  SFB_TRY(grad_operand_scales(w, op16, {{gMA_u, pix * 2 * d.H2}, {gMA_v, pix * 2 * d.W2}}, {}, st));
  SFB_CUDA(timed(KID_PACK, 2, st, [&] {
    SlotSources su, sv;
    maxavg_slot_sources(d, AM_u, AM_v, gMA_u, gMA_v, &su, &sv, grad_slot_scales(w, op16));
    launch_pack_interleaved(su, w.gxu, d.B, d.N1(), w.n1p, d.H2, 4, 1, 0, st);
    return launch_pack_interleaved(sv, w.gxv, d.B, d.N1(), w.n1p, d.W2, 4, 1, 0, st);
  }));
  return run_grad_pair(d, w, GRAD_MAXAVG, 4, 0, gF1, gF2, st);
}

int sfb_compression_backward(const float* F1, const float* F2, const float* A_u, const float* A_v,
                             const float* gC_u, const float* gC_v, float* gF1, float* gF2, float* gA_u,
                             float* gA_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                             void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, true, &d));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(A_u); SFB_CHECK_PTR(A_v); SFB_CHECK_PTR(gC_u); SFB_CHECK_PTR(gC_v);
  SFB_CHECK_PTR(gF1); SFB_CHECK_PTR(gF2); SFB_CHECK_PTR(gA_u); SFB_CHECK_PTR(gA_v);
  Workspace w;
  SFB_TRY(check_workspace(d, workspace, workspace_bytes, SFB_OP_COMPRESSION_BACKWARD, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  SFB_CUDA(timed(KID_PREPARE, 2 + (op16 == OP16_FP16 ? 3 : 0), st, [&] { return prepare_operands(d, w, F1, F2, false, op16, st); }));
  const int N1 = d.N1(), K = d.Kc;
  SFB_TRY(run_attention_grads(d, w, gC_u, gC_v, gA_u, gA_v, st, op16));
  {
    const size_t pk = (size_t)d.B * N1 * K;
    SFB_TRY(grad_operand_scales(w, op16, {{gC_u, pk * d.H2}, {gC_v, pk * d.W2}}, {{A_u, pk * d.W2}, {A_v, pk * d.H2}}, st));
  }
  // gradient GEMMs, at most KC_MAX_PER_SWEEP channels per pass; later passes add to gF1 / gF2.
  for (int k0 = 0; k0 < K; k0 += KC_MAX_PER_SWEEP) {
    const int kc = chunk_channels(K - k0), R4 = grad_slots(kc);
    SFB_CUDA(timed(KID_PACK, 2, st, [&] {
      SlotSources su, sv;
      compress_slot_sources(K, k0, kc, A_u, A_v, gC_u, gC_v, &su, &sv, grad_slot_scales(w, op16));
      launch_pack_interleaved(su, w.gxu, d.B, N1, w.n1p, d.H2, R4, R4 / 4, 0, st);
      return launch_pack_interleaved(sv, w.gxv, d.B, N1, w.n1p, d.W2, R4, R4 / 4, 0, st);
    }));
    SFB_TRY(run_grad_pair(d, w, GRAD_COMPRESS, R4, k0 > 0 ? 1 : 0, gF1, gF2, st));
  }
  return SFB_OK;
}

int sfb_compression_attention_backward(const float* F1, const float* F2, const float* gC_u, const float* gC_v,
                                       float* gA_u, float* gA_v, const sfb_shape* shape, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, true, &d));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(gC_u); SFB_CHECK_PTR(gC_v); SFB_CHECK_PTR(gA_u); SFB_CHECK_PTR(gA_v);
  Workspace w;
  SFB_TRY(check_workspace(d, workspace, workspace_bytes, SFB_OP_COMPRESSION_FORWARD, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  SFB_CUDA(timed(KID_PREPARE, 2 + (op16 == OP16_FP16 ? 3 : 0), st, [&] { return prepare_operands(d, w, F1, F2, false, op16, st); }));
  return run_attention_grads(d, w, gC_u, gC_v, gA_u, gA_v, st, op16);
}

// Feature gradients of both backward ops from one GEMM pair (plus accumulated passes for channels beyond
// KC_MAX_PER_SWEEP).  F1r / F2r must already hold the rounded features.
static int run_fused_feature_grads(const Dims& d, const Workspace& w, const int32_t* AM_u, const int32_t* AM_v,
                                   const float* gMA_u, const float* gMA_v, const float* A_u, const float* A_v,
                                   const float* gC_u, const float* gC_v, float* gF1, float* gF2, cudaStream_t st) {
  const int N1 = d.N1(), K = d.Kc;
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  {
    const size_t pix = (size_t)d.B * N1;
    SFB_TRY(grad_operand_scales(w, op16,
                                {{gMA_u, pix * 2 * d.H2}, {gMA_v, pix * 2 * d.W2}, {gC_u, pix * K * d.H2}, {gC_v, pix * K * d.W2}},
                                {{A_u, pix * K * d.W2}, {A_v, pix * K * d.H2}}, st));
  }
  const float* const gs = grad_slot_scales(w, op16);
  {  // group 0 = max/avg slots, groups 1.. = the first (up to 4) compression channels; G is their sum
    const int kc = chunk_channels(K), Qc = grad_slots(kc) / 4, Q = 1 + Qc;
    SFB_CUDA(timed(KID_PACK, 4, st, [&] {
      SlotSources su, sv;
      maxavg_slot_sources(d, AM_u, AM_v, gMA_u, gMA_v, &su, &sv, gs);
      launch_pack_interleaved(su, w.gxu, d.B, N1, w.n1p, d.H2, 4, Q, 0, st);
      launch_pack_interleaved(sv, w.gxv, d.B, N1, w.n1p, d.W2, 4, Q, 0, st);
      compress_slot_sources(K, 0, kc, A_u, A_v, gC_u, gC_v, &su, &sv, gs);
      launch_pack_interleaved(su, w.gxu, d.B, N1, w.n1p, d.H2, 4 * Qc, Q, 1, st);
      return launch_pack_interleaved(sv, w.gxv, d.B, N1, w.n1p, d.W2, 4 * Qc, Q, 1, st);
    }));
    SFB_TRY(run_grad_pair(d, w, GRAD_FUSED, 4 * Q, 0, gF1, gF2, st));
  }
  for (int k0 = KC_MAX_PER_SWEEP; k0 < K; k0 += KC_MAX_PER_SWEEP) {  // remaining channels: compression form, accumulated
    const int kc = chunk_channels(K - k0), R4 = grad_slots(kc);
    SFB_CUDA(timed(KID_PACK, 2, st, [&] {
      SlotSources su, sv;
      compress_slot_sources(K, k0, kc, A_u, A_v, gC_u, gC_v, &su, &sv, gs);
      launch_pack_interleaved(su, w.gxu, d.B, N1, w.n1p, d.H2, R4, R4 / 4, 0, st);
      return launch_pack_interleaved(sv, w.gxv, d.B, N1, w.n1p, d.W2, R4, R4 / 4, 0, st);
    }));
    SFB_TRY(run_grad_pair(d, w, GRAD_COMPRESS, R4, 1, gF1, gF2, st));
  }
  return SFB_OK;
}

int sfb_separation_feature_backward(const float* F1, const float* F2, const int32_t* AM_u, const int32_t* AM_v,
                                    const float* gMA_u, const float* gMA_v, const float* A_u, const float* A_v,
                                    const float* gC_u, const float* gC_v, float* gF1, float* gF2,
                                    const sfb_shape* shape, void* workspace, size_t workspace_bytes, void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, true, &d));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(AM_u); SFB_CHECK_PTR(AM_v); SFB_CHECK_PTR(gMA_u); SFB_CHECK_PTR(gMA_v);
  SFB_CHECK_PTR(A_u); SFB_CHECK_PTR(A_v); SFB_CHECK_PTR(gC_u); SFB_CHECK_PTR(gC_v); SFB_CHECK_PTR(gF1); SFB_CHECK_PTR(gF2);
  Workspace w;
  SFB_TRY(check_workspace(d, workspace, workspace_bytes, SFB_OP_SEPARATION_BACKWARD, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  SFB_CUDA(timed(KID_PREPARE, 2 + (op16 == OP16_FP16 ? 3 : 0), st, [&] { return prepare_operands(d, w, F1, F2, false, op16, st); }));
  return run_fused_feature_grads(d, w, AM_u, AM_v, gMA_u, gMA_v, A_u, A_v, gC_u, gC_v, gF1, gF2, st);
}

int sfb_separation_backward(const float* F1, const float* F2, const int32_t* AM_u, const int32_t* AM_v,
                            const float* gMA_u, const float* gMA_v, const float* A_u, const float* A_v,
                            const float* gC_u, const float* gC_v, float* gF1, float* gF2, float* gA_u,
                            float* gA_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                            void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, true, &d));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(AM_u); SFB_CHECK_PTR(AM_v); SFB_CHECK_PTR(gMA_u); SFB_CHECK_PTR(gMA_v);
  SFB_CHECK_PTR(A_u); SFB_CHECK_PTR(A_v); SFB_CHECK_PTR(gC_u); SFB_CHECK_PTR(gC_v);
  SFB_CHECK_PTR(gF1); SFB_CHECK_PTR(gF2); SFB_CHECK_PTR(gA_u); SFB_CHECK_PTR(gA_v);
  Workspace w;
  SFB_TRY(check_workspace(d, workspace, workspace_bytes, SFB_OP_SEPARATION_BACKWARD, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  SFB_CUDA(timed(KID_PREPARE, 2 + (op16 == OP16_FP16 ? 3 : 0), st, [&] { return prepare_operands(d, w, F1, F2, false, op16, st); }));
  SFB_TRY(run_attention_grads(d, w, gC_u, gC_v, gA_u, gA_v, st, op16));
  return run_fused_feature_grads(d, w, AM_u, AM_v, gMA_u, gMA_v, A_u, A_v, gC_u, gC_v, gF1, gF2, st);
}

int sfb_max_argmax_avg_forward_cf(const float* F1, const float* F2, float* SEP_v, float* SEP_u, int32_t* AM_u,
                                  int32_t* AM_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, false, &d));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(SEP_v); SFB_CHECK_PTR(SEP_u);
  const bool with_argmax = AM_u != nullptr || AM_v != nullptr;
  if (with_argmax) { SFB_CHECK_PTR(AM_u); SFB_CHECK_PTR(AM_v); }
  Workspace w;
  SFB_TRY(check_workspace(d, workspace, workspace_bytes, SFB_OP_MAX_AVG_FORWARD_CF, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  CUtensorMap tm_f1, tm_f2, tm_aux;
  SFB_TRY(map_sweep_operands(d, w, op16, &tm_f1, &tm_f2, &tm_aux));
  SFB_CUDA(timed(KID_PREPARE, 3 + (op16 == OP16_FP16 ? 3 : 0), st, [&] { return prepare_operands(d, w, F1, F2, true, op16, st); }));
  const int N1 = d.N1();
  SweepArgs a;
  memset(&a, 0, sizeof(a));
  a.d = d;
  a.op16 = op16;
  a.out_scale = sweep_out_scale(w, op16);
  a.mode = with_argmax ? SWEEP_MAXARGAVG : SWEEP_MAXAVG;
  a.n_valid = N1;
  a.pu = cf_view(SEP_v, 2, d.H2, N1);       // per-u channels live in the tensor the call site calls sep_v
  a.pv = cf_view(SEP_u, 2, d.W2, N1);
  a.pu_arg = cf_view(AM_u, 1, d.H2, N1);
  a.pv_arg = cf_view(AM_v, 1, d.W2, N1);
  a.status = w.status;
  SFB_CUDA(timed(KID_SWEEP_MAXAVG, 1, st, [&] { return launch_sweep(with_wait_settings(a), tm_f1, tm_f2, tm_aux, st); }));
  return SFB_OK;
}

// compression sweep on channels-first weights / outputs (forward, or attention gradients with the upstream
// gradients as weights)
static int run_compress_cf(const float* F1, const float* F2, const float* W_u, const float* W_v, float* O_u, float* O_v,
                           const sfb_shape* shape, void* workspace, size_t workspace_bytes, void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, true, &d));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(W_u); SFB_CHECK_PTR(W_v); SFB_CHECK_PTR(O_u); SFB_CHECK_PTR(O_v);
  Workspace w;
  SFB_TRY(check_workspace(d, workspace, workspace_bytes, SFB_OP_COMPRESSION_CF, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  CUtensorMap tm_f1, tm_f2;
  SFB_TRY(map_sweep_operands(d, w, op16, &tm_f1, &tm_f2, nullptr));
  SFB_CUDA(timed(KID_PREPARE, 2 + (op16 == OP16_FP16 ? 3 : 0), st, [&] { return prepare_operands(d, w, F1, F2, false, op16, st); }));
  const int N1 = d.N1(), K = d.Kc;
  // W_u (B,K,W2,N1) weights per v, W_v (B,K,H2,N1) per u; O_u (B,K,H2,N1), O_v (B,K,W2,N1)
  return run_compress_sweeps(d, w.status, tm_f1, tm_f2, cf_view(W_v, K, d.H2, N1), cf_view(W_u, K, d.W2, N1), 0, 0, 1,
                             cf_view(O_u, K, d.H2, N1), cf_view(O_v, K, d.W2, N1), N1, st, op16, sweep_out_scale(w, op16));
}

int sfb_compression_forward_cf(const float* F1, const float* F2, const float* A_u, const float* A_v, float* C_u,
                               float* C_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                               void* stream) {
  return run_compress_cf(F1, F2, A_u, A_v, C_u, C_v, shape, workspace, workspace_bytes, stream);
}

int sfb_compression_attention_backward_cf(const float* F1, const float* F2, const float* gC_u, const float* gC_v,
                                          float* gA_u, float* gA_v, const sfb_shape* shape, void* workspace,
                                          size_t workspace_bytes, void* stream) {
  // gA_v(b,k,u,p) = sum_v S * gC_v(b,k,v,p), gA_u(b,k,v,p) = sum_u S * gC_u(b,k,u,p)
  return run_compress_cf(F1, F2, gC_v, gC_u, gA_v, gA_u, shape, workspace, workspace_bytes, stream);
}

// Channels-first form of run_fused_feature_grads: gMA sources gM_v (B,2,H2,N1) / gM_u (B,2,W2,N1); the compression
// gradients are channels g0.. of tensors with gK channels.
static int run_fused_feature_grads_cf(const Dims& d, const Workspace& w, const int32_t* AM_u, const int32_t* AM_v,
                                      const float* gM_v, const float* gM_u, const float* A_u, const float* A_v,
                                      const float* gC_u, const float* gC_v, int gK, int g0, float* gF1, float* gF2,
                                      cudaStream_t st, int out_cf = 0, float scale1 = 1.f, bool unit_weights = false) {
  const int N1 = d.N1(), K = d.Kc;
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  {  // FP16 operands: scales from the whole gradient tensors (an upper bound when only some channels are this level's);
     // unit_weights: A_u / A_v are softmax outputs
    const size_t bn = (size_t)d.B * N1;
    if (unit_weights)
      SFB_TRY(grad_operand_scales(w, op16, {{gM_v, bn * 2 * d.H2}, {gM_u, bn * 2 * d.W2}, {gC_u, bn * gK * d.H2}, {gC_v, bn * gK * d.W2}}, {}, st));
    else
      SFB_TRY(grad_operand_scales(w, op16, {{gM_v, bn * 2 * d.H2}, {gM_u, bn * 2 * d.W2}, {gC_u, bn * gK * d.H2}, {gC_v, bn * gK * d.W2}},
                                  {{A_u, bn * K * d.W2}, {A_v, bn * K * d.H2}}, st));
  }
  const float* const gs = grad_slot_scales(w, op16);
  {
    const int kc = chunk_channels(K), Qc = grad_slots(kc) / 4, Q = 1 + Qc;
    SFB_CUDA(timed(KID_PACK, 4, st, [&] {
      SlotSources su, sv;
      // channel 0 = max gradient, channel 1 = mean gradient (same slots as the reference layout)
      maxavg_slot_sources(d, AM_u, AM_v, gM_v, gM_u, &su, &sv, gs);
      launch_pack_interleaved_cf(su, w.gxu, d.B, N1, w.n1p, d.H2, 4, Q, 0, st);
      launch_pack_interleaved_cf(sv, w.gxv, d.B, N1, w.n1p, d.W2, 4, Q, 0, st);
      compress_slot_sources(K, 0, kc, A_u, A_v, gC_u, gC_v, &su, &sv, gs, gK, g0);
      launch_pack_interleaved_cf(su, w.gxu, d.B, N1, w.n1p, d.H2, 4 * Qc, Q, 1, st);
      return launch_pack_interleaved_cf(sv, w.gxv, d.B, N1, w.n1p, d.W2, 4 * Qc, Q, 1, st);
    }));
    SFB_TRY(run_grad_pair(d, w, GRAD_FUSED, 4 * Q, 0, gF1, gF2, st, out_cf, scale1));
  }
  for (int k0 = KC_MAX_PER_SWEEP; k0 < K; k0 += KC_MAX_PER_SWEEP) {
    const int kc = chunk_channels(K - k0), R4 = grad_slots(kc);
    SFB_CUDA(timed(KID_PACK, 2, st, [&] {
      SlotSources su, sv;
      compress_slot_sources(K, k0, kc, A_u, A_v, gC_u, gC_v, &su, &sv, gs, gK, g0);
      launch_pack_interleaved_cf(su, w.gxu, d.B, N1, w.n1p, d.H2, R4, R4 / 4, 0, st);
      return launch_pack_interleaved_cf(sv, w.gxv, d.B, N1, w.n1p, d.W2, R4, R4 / 4, 0, st);
    }));
    SFB_TRY(run_grad_pair(d, w, GRAD_COMPRESS, R4, 1, gF1, gF2, st, out_cf, scale1));
  }
  return SFB_OK;
}

int sfb_separation_feature_backward_cf(const float* F1, const float* F2, const int32_t* AM_u, const int32_t* AM_v,
                                       const float* gSEP_v, const float* gSEP_u, const float* A_u, const float* A_v,
                                       const float* gC_u, const float* gC_v, float* gF1, float* gF2,
                                       const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                                       void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, true, &d));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(AM_u); SFB_CHECK_PTR(AM_v); SFB_CHECK_PTR(gSEP_v); SFB_CHECK_PTR(gSEP_u);
  SFB_CHECK_PTR(A_u); SFB_CHECK_PTR(A_v); SFB_CHECK_PTR(gC_u); SFB_CHECK_PTR(gC_v); SFB_CHECK_PTR(gF1); SFB_CHECK_PTR(gF2);
  Workspace w;
  SFB_TRY(check_workspace(d, workspace, workspace_bytes, SFB_OP_SEPARATION_FEATURE_BACKWARD_CF, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  SFB_CUDA(timed(KID_PREPARE, 2 + (op16 == OP16_FP16 ? 3 : 0), st, [&] { return prepare_operands(d, w, F1, F2, false, op16, st); }));
  return run_fused_feature_grads_cf(d, w, AM_u, AM_v, gSEP_v, gSEP_u, A_u, A_v, gC_u, gC_v, d.Kc, 0, gF1, gF2, st);
}

// ---- attention weights: Conv3d(2 -> Kc, 3, padding 1) + softmax over the displacement axis ----
static int check_attention_dims(int B, int Kc, int D, int H1, int W1, AttentionDims* ad) {
  if (B < 1 || Kc < 1 || D < 1 || H1 < 1 || W1 < 1)
    return fail(SFB_ERR_INVALID_ARGUMENT, "B, Kc, D, H1, W1 must be >= 1 (got %d %d %d %d %d)", B, Kc, D, H1, W1);
  if (Kc > 64) return fail(SFB_ERR_UNSUPPORTED_SHAPE, "Kc=%d unsupported: at most 64 attention channels", Kc);
  if ((long long)H1 * W1 > (1ll << 21)) return fail(SFB_ERR_UNSUPPORTED_SHAPE, "image 1 has more than 2^21 pixels");
  *ad = AttentionDims{B, Kc, D, H1, W1};
  return SFB_OK;
}

int sfb_attention_forward(const float* X, int64_t x_batch_stride, const float* weight, const float* bias, float* A,
                          int32_t B, int32_t Kc, int32_t D, int32_t H1, int32_t W1, void* stream) {
  AttentionDims ad;
  SFB_TRY(check_attention_dims(B, Kc, D, H1, W1, &ad));
  if (X == nullptr || weight == nullptr || bias == nullptr || A == nullptr)
    return fail(SFB_ERR_INVALID_ARGUMENT, "X, weight, bias and A must not be NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SFB_CUDA(timed(KID_ATTENTION_FWD, (Kc + 3) / 4, st,
                 [&] { return launch_attention_forward(ad, X, x_batch_stride, weight, bias, A, st); }));
  return SFB_OK;
}

size_t sfb_attention_backward_workspace_bytes(int32_t B, int32_t Kc, int32_t D, int32_t H1, int32_t W1) {
  AttentionDims ad;
  if (check_attention_dims(B, Kc, D, H1, W1, &ad) != SFB_OK) return 0;
  return align_up(attention_partial_floats(ad) * sizeof(float), 256);
}

static int attention_backward_launches(int Kc) { return (Kc + 3) / 4 + 4; }

int sfb_attention_backward(const float* X, int64_t x_batch_stride, const float* weight, const float* A, float* gA,
                           const float* add, int64_t add_batch_stride, float* gX, float* gweight, float* gbias,
                           int32_t B, int32_t Kc, int32_t D, int32_t H1, int32_t W1, void* workspace,
                           size_t workspace_bytes, void* stream) {
  AttentionDims ad;
  SFB_TRY(check_attention_dims(B, Kc, D, H1, W1, &ad));
  if (X == nullptr || weight == nullptr || A == nullptr || gA == nullptr || gX == nullptr || gweight == nullptr ||
      gbias == nullptr)
    return fail(SFB_ERR_INVALID_ARGUMENT, "X, weight, A, gA, gX, gweight and gbias must not be NULL");
  if (workspace == nullptr) return fail(SFB_ERR_INVALID_ARGUMENT, "workspace is NULL");
  const size_t need = sfb_attention_backward_workspace_bytes(B, Kc, D, H1, W1);
  if (workspace_bytes < need)
    return fail(SFB_ERR_WORKSPACE_TOO_SMALL, "workspace has %zu bytes, %zu needed", workspace_bytes, need);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SFB_CUDA(timed(KID_ATTENTION_BWD, attention_backward_launches(Kc), st, [&] {
    return launch_attention_backward(ad, X, x_batch_stride, weight, A, gA, add, add_batch_stride, gX, gweight, gbias,
                                     static_cast<float*>(workspace), st);
  }));
  return SFB_OK;
}

// ---- one pyramid level of the call site ----
// channels c0.. of a concatenated (B, Ktot, D, N1) tensor as a pixel view
static PixView cf_channels(const void* base, int Ktot, int c0, int D, int N1) {
  return PixView{static_cast<float*>(const_cast<void*>(base)) + (size_t)c0 * D * N1, (long long)Ktot * D * N1,
                 (uint32_t)N1, (uint32_t)(D * N1)};
}

// Where a level's (2+Kc)-channel volumes live: channels c0 .. c0+2+Kc-1 of tensors with Ktot channels (the
// concatenated outputs of all pyramid levels); {0, 0} = tensors of their own.
struct Placement { int Ktot, c0; };
static int check_placement(const Dims& d, Placement* pl) {
  const int Kt = 2 + d.Kc;
  if (pl->Ktot == 0 && pl->c0 == 0) pl->Ktot = Kt;
  if (pl->c0 < 0 || pl->c0 + Kt > pl->Ktot)
    return fail(SFB_ERR_INVALID_ARGUMENT, "channels %d..%d do not fit in %d channels", pl->c0, pl->c0 + Kt, pl->Ktot);
  const long long n1p = ((long long)d.N1() + TILE_M - 1) / TILE_M * TILE_M;
  if (n1p * pl->Ktot * (d.H2 > d.W2 ? d.H2 : d.W2) >= (1ll << 32))
    return fail(SFB_ERR_UNSUPPORTED_SHAPE, "H1*W1*max(H2,W2)*channels exceeds 2^32 elements per sample");
  return SFB_OK;
}

// fmaps != 0: F1 / F2 are the model's feature maps (B, C, H, W); F1 is multiplied by scale1 on the way in.
static int level_forward(Placement pl, const float* F1, const float* F2, int fmaps, float scale1, const float* weight_u,
                         const float* bias_u, const float* weight_v, const float* bias_v, float* SEP_u, float* SEP_v,
                         int32_t* AM_u, int32_t* AM_v, float* A_u, float* A_v, const sfb_shape* shape,
                         void* workspace, size_t workspace_bytes, void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, true, &d));
  AttentionDims ad;
  SFB_TRY(check_attention_dims(d.B, d.Kc, d.H2, d.H1, d.W1, &ad));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(SEP_u); SFB_CHECK_PTR(SEP_v); SFB_CHECK_PTR(A_u); SFB_CHECK_PTR(A_v);
  if (weight_u == nullptr || bias_u == nullptr || weight_v == nullptr || bias_v == nullptr)
    return fail(SFB_ERR_INVALID_ARGUMENT, "attention weights and biases must not be NULL");
  SFB_TRY(check_placement(d, &pl));
  const bool with_argmax = AM_u != nullptr || AM_v != nullptr;
  if (with_argmax) { SFB_CHECK_PTR(AM_u); SFB_CHECK_PTR(AM_v); }
  Workspace w;
  SFB_TRY(check_workspace(d, workspace, workspace_bytes, SFB_OP_SEPARATION_LEVEL_FORWARD, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  CUtensorMap tm_f1, tm_f2, tm_aux;
  SFB_TRY(map_sweep_operands(d, w, op16, &tm_f1, &tm_f2, &tm_aux));
  uint16_t* const F1h = op16 ? w.F1h : nullptr;
  uint16_t* const F2h = op16 ? w.F2h : nullptr;
  uint16_t* const auxh = op16 ? w.auxh : nullptr;
  SFB_CUDA(timed(KID_PREPARE, 3 + (op16 == OP16_FP16 ? 3 : 0), st, [&] {
    return fmaps ? launch_prepare_cf(d, F1, F2, scale1, w.F1r, w.F2r, w.aux, w.status, st, F1h, F2h, auxh, op16, w.scales)
                 : launch_prepare(d, F1, F2, w.F1r, w.F2r, w.aux, w.status, st, F1h, F2h, auxh, op16, w.scales);
  }));
  const int N1 = d.N1(), K = d.Kc, Kt = pl.Ktot, c0 = pl.c0;
  SweepArgs a;
  memset(&a, 0, sizeof(a));
  a.d = d;
  a.mode = with_argmax ? SWEEP_MAXARGAVG : SWEEP_MAXAVG;
  a.n_valid = N1;
  a.pu = cf_channels(SEP_v, Kt, c0, d.H2, N1);  // per-u channels live in the tensor the call site calls sep_v
  a.pv = cf_channels(SEP_u, Kt, c0, d.W2, N1);
  a.pu_arg = cf_view(AM_u, 1, d.H2, N1);
  a.pv_arg = cf_view(AM_v, 1, d.W2, N1);
  a.op16 = op16;
  a.out_scale = sweep_out_scale(w, op16);
  a.status = w.status;
  SFB_CUDA(timed(KID_SWEEP_MAXAVG, 1, st, [&] { return launch_sweep(with_wait_settings(a), tm_f1, tm_f2, tm_aux, st); }));
  const long long sb_u = (long long)Kt * d.W2 * N1, sb_v = (long long)Kt * d.H2 * N1;
  SFB_CUDA(timed(KID_ATTENTION_FWD, 2 * ((K + 3) / 4), st, [&] {
    launch_attention_forward(AttentionDims{d.B, K, d.W2, d.H1, d.W1}, SEP_u + (size_t)c0 * d.W2 * N1, sb_u, weight_u,
                             bias_u, A_u, st, w.status);
    return launch_attention_forward(AttentionDims{d.B, K, d.H2, d.H1, d.W1}, SEP_v + (size_t)c0 * d.H2 * N1, sb_v,
                                    weight_v, bias_v, A_v, st, w.status);
  }));
  // C_u (per u, weights A_u per v) -> SEP_v channels 2.., C_v -> SEP_u channels 2..
  return run_compress_sweeps(d, w.status, tm_f1, tm_f2, cf_view(A_v, K, d.H2, N1), cf_view(A_u, K, d.W2, N1), 0, 0, 1,
                             cf_channels(SEP_v, Kt, c0 + 2, d.H2, N1), cf_channels(SEP_u, Kt, c0 + 2, d.W2, N1), N1, st,
                             op16, sweep_out_scale(w, op16));
}

int sfb_separation_level_forward(const float* F1, const float* F2, const float* weight_u, const float* bias_u,
                                 const float* weight_v, const float* bias_v, float* SEP_u, float* SEP_v,
                                 int32_t* AM_u, int32_t* AM_v, float* A_u, float* A_v, const sfb_shape* shape,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  return level_forward(Placement{0, 0}, F1, F2, 0, 1.f, weight_u, bias_u, weight_v, bias_v, SEP_u, SEP_v, AM_u, AM_v, A_u,
                       A_v, shape, workspace, workspace_bytes, stream);
}

int sfb_separation_level_forward_fmaps(const float* fmap1, const float* fmap2, float scale1, const float* weight_u,
                                       const float* bias_u, const float* weight_v, const float* bias_v, float* SEP_u,
                                       float* SEP_v, int32_t sep_channels, int32_t sep_channel0, int32_t* AM_u,
                                       int32_t* AM_v, float* A_u, float* A_v, const sfb_shape* shape, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  return level_forward(Placement{sep_channels, sep_channel0}, fmap1, fmap2, 1, scale1, weight_u, bias_u, weight_v, bias_v,
                       SEP_u, SEP_v, AM_u, AM_v, A_u, A_v, shape, workspace, workspace_bytes, stream);
}

static int level_backward(Placement pl, const float* F1, const float* F2, int fmaps, float scale1, const float* weight_u,
                          const float* weight_v, const float* SEP_u, const float* SEP_v, const int32_t* AM_u,
                          const int32_t* AM_v, const float* A_u, const float* A_v, const float* gSEP_u,
                          const float* gSEP_v, float* gF1, float* gF2, float* gweight_u, float* gbias_u,
                          float* gweight_v, float* gbias_v, const sfb_shape* shape, void* workspace,
                          size_t workspace_bytes, void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, true, &d));
  AttentionDims ad;
  SFB_TRY(check_attention_dims(d.B, d.Kc, d.H2, d.H1, d.W1, &ad));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(SEP_u); SFB_CHECK_PTR(SEP_v); SFB_CHECK_PTR(AM_u); SFB_CHECK_PTR(AM_v);
  SFB_CHECK_PTR(A_u); SFB_CHECK_PTR(A_v); SFB_CHECK_PTR(gSEP_u); SFB_CHECK_PTR(gSEP_v); SFB_CHECK_PTR(gF1); SFB_CHECK_PTR(gF2);
  if (weight_u == nullptr || weight_v == nullptr || gweight_u == nullptr || gbias_u == nullptr || gweight_v == nullptr ||
      gbias_v == nullptr)
    return fail(SFB_ERR_INVALID_ARGUMENT, "attention weights and their gradient buffers must not be NULL");
  SFB_TRY(check_placement(d, &pl));
  Workspace w;
  SFB_TRY(check_workspace(d, workspace, workspace_bytes, SFB_OP_SEPARATION_LEVEL_BACKWARD, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int op16;
  SFB_TRY(operand_mode(d, &op16));
  CUtensorMap tm_f1, tm_f2;
  SFB_TRY(map_sweep_operands(d, w, op16, &tm_f1, &tm_f2, nullptr));
  uint16_t* const F1h = op16 ? w.F1h : nullptr;
  uint16_t* const F2h = op16 ? w.F2h : nullptr;
  SFB_CUDA(timed(KID_PREPARE, 2 + (op16 == OP16_FP16 ? 3 : 0), st, [&] {
    return fmaps ? launch_prepare_cf(d, F1, F2, scale1, w.F1r, w.F2r, nullptr, w.status, st, F1h, F2h, nullptr, op16, w.scales)
                 : launch_prepare(d, F1, F2, w.F1r, w.F2r, nullptr, w.status, st, F1h, F2h, nullptr, op16, w.scales);
  }));
  const int N1 = d.N1(), K = d.Kc, Kt = pl.Ktot, c0 = pl.c0;
  // attention gradients: gA_v(b,k,u,p) = sum_v S * gC_v(b,k,v,p), gA_u(b,k,v,p) = sum_u S * gC_u(b,k,u,p), with
  // gC_u = gSEP_v[:, 2:] (per u) and gC_v = gSEP_u[:, 2:] (per v) in the role of the weights
  SFB_TRY(run_compress_sweeps(d, w.status, tm_f1, tm_f2, cf_channels(gSEP_v, Kt, c0 + 2, d.H2, N1),
                              cf_channels(gSEP_u, Kt, c0 + 2, d.W2, N1), 0, 0, 1, cf_view(w.ga_v, K, d.H2, N1),
                              cf_view(w.ga_u, K, d.W2, N1), N1, st, op16, sweep_out_scale(w, op16)));
  // through softmax and Conv3d: parameter gradients, and the total gradients of the max/avg channels
  const long long sb_u = (long long)Kt * d.W2 * N1, sb_v = (long long)Kt * d.H2 * N1;
  SFB_CUDA(timed(KID_ATTENTION_BWD, 2 * attention_backward_launches(K), st, [&] {
    const size_t ou = (size_t)c0 * d.W2 * N1, ov = (size_t)c0 * d.H2 * N1;  // first channel of this level
    launch_attention_backward(AttentionDims{d.B, K, d.W2, d.H1, d.W1}, SEP_u + ou, sb_u, weight_u, A_u, w.ga_u,
                              gSEP_u + ou, sb_u, w.gm_u, gweight_u, gbias_u, w.at_partial, st, w.status);
    return launch_attention_backward(AttentionDims{d.B, K, d.H2, d.H1, d.W1}, SEP_v + ov, sb_v, weight_v, A_v, w.ga_v,
                                     gSEP_v + ov, sb_v, w.gm_v, gweight_v, gbias_v, w.at_partial, st, w.status);
  }));
  return run_fused_feature_grads_cf(d, w, AM_u, AM_v, w.gm_v, w.gm_u, A_u, A_v, gSEP_v, gSEP_u, Kt, c0 + 2, gF1, gF2, st,
                                    fmaps, fmaps ? scale1 : 1.f, /*unit_weights=*/true);
}

int sfb_separation_level_backward(const float* F1, const float* F2, const float* weight_u, const float* weight_v,
                                  const float* SEP_u, const float* SEP_v, const int32_t* AM_u, const int32_t* AM_v,
                                  const float* A_u, const float* A_v, const float* gSEP_u, const float* gSEP_v,
                                  float* gF1, float* gF2, float* gweight_u, float* gbias_u, float* gweight_v,
                                  float* gbias_v, const sfb_shape* shape, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  return level_backward(Placement{0, 0}, F1, F2, 0, 1.f, weight_u, weight_v, SEP_u, SEP_v, AM_u, AM_v, A_u, A_v, gSEP_u,
                        gSEP_v, gF1, gF2, gweight_u, gbias_u, gweight_v, gbias_v, shape, workspace, workspace_bytes, stream);
}

int sfb_separation_level_backward_fmaps(const float* fmap1, const float* fmap2, float scale1, const float* weight_u,
                                        const float* weight_v, const float* SEP_u, const float* SEP_v,
                                        int32_t sep_channels, int32_t sep_channel0, const int32_t* AM_u,
                                        const int32_t* AM_v, const float* A_u, const float* A_v, const float* gSEP_u,
                                        const float* gSEP_v, float* gfmap1, float* gfmap2, float* gweight_u,
                                        float* gbias_u, float* gweight_v, float* gbias_v, const sfb_shape* shape,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  return level_backward(Placement{sep_channels, sep_channel0}, fmap1, fmap2, 1, scale1, weight_u, weight_v, SEP_u, SEP_v,
                        AM_u, AM_v, A_u, A_v, gSEP_u, gSEP_v, gfmap1, gfmap2, gweight_u, gbias_u, gweight_v, gbias_v, shape,
                        workspace, workspace_bytes, stream);
}


// ---- placement of a level's volumes into the concatenated level-0-sized outputs ----
static int check_resample(const void* a, const void* b, int B, int K, int Dl, int D0, int H1, int W1) {
  if (a == nullptr || b == nullptr) return fail(SFB_ERR_INVALID_ARGUMENT, "tensor pointers must not be NULL");
  if (B < 1 || K < 1 || Dl < 1 || D0 < 1 || H1 < 1 || W1 < 1)
    return fail(SFB_ERR_INVALID_ARGUMENT, "B, K, Dl, D0, H1, W1 must be >= 1");
  if (Dl > D0) return fail(SFB_ERR_UNSUPPORTED_SHAPE, "Dl=%d > D0=%d: only upsampling is supported", Dl, D0);
  if (B * (long long)K > 65535 || D0 > 65535) return fail(SFB_ERR_UNSUPPORTED_SHAPE, "B*K and D0 must be <= 65535");
  if ((long long)H1 * W1 > (1ll << 24)) return fail(SFB_ERR_UNSUPPORTED_SHAPE, "image 1 has more than 2^24 pixels");
  return SFB_OK;
}

int sfb_upsample_displacement(const float* in, float* out, int64_t out_batch_stride, int32_t B, int32_t K, int32_t Dl,
                              int32_t D0, int32_t H1, int32_t W1, void* stream) {
  SFB_TRY(check_resample(in, out, B, K, Dl, D0, H1, W1));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SFB_CUDA(timed(KID_RESAMPLE, 1, st, [&] {
    return launch_upsample_displacement(in, out, out_batch_stride, B, K, Dl, D0, H1 * W1, st);
  }));
  return SFB_OK;
}

int sfb_upsample_displacement_backward(const float* gout, int64_t gout_batch_stride, float* gin, int32_t B, int32_t K,
                                       int32_t Dl, int32_t D0, int32_t H1, int32_t W1, void* stream) {
  SFB_TRY(check_resample(gout, gin, B, K, Dl, D0, H1, W1));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SFB_CUDA(timed(KID_RESAMPLE, 1, st, [&] {
    return launch_upsample_displacement_adjoint(gout, gout_batch_stride, gin, B, K, Dl, D0, H1 * W1, st);
  }));
  return SFB_OK;
}

// ---- lookup on the aggregated 3D volumes (CorrBlock1D) ----
static int check_lookup_dims(int B, int dim, int D, int H1, int W1, int levels, int radius, LookupDims* ld) {
  if (B < 1 || dim < 1 || D < 2 || H1 < 1 || W1 < 1)
    return fail(SFB_ERR_INVALID_ARGUMENT, "B, dim, H1, W1 must be >= 1 and D >= 2 (got %d %d %d %d %d)", B, dim, D, H1, W1);
  if (levels < 1 || levels > LOOKUP_MAX_LEVELS || radius < 0 || radius > 64)
    return fail(SFB_ERR_UNSUPPORTED_SHAPE, "levels must be in [1, %d] and radius in [0, 64] (got %d, %d)",
                LOOKUP_MAX_LEVELS, levels, radius);
  if ((D >> (levels - 1)) < 2)
    return fail(SFB_ERR_UNSUPPORTED_SHAPE, "the coarsest level would have fewer than 2 displacements (D=%d, levels=%d)",
                D, levels);
  if ((long long)H1 * W1 > (1ll << 24)) return fail(SFB_ERR_UNSUPPORTED_SHAPE, "image 1 has more than 2^24 pixels");
  *ld = LookupDims{B, dim, D, H1, W1, levels, radius};
  return SFB_OK;
}

size_t sfb_lookup_pyramid_bytes(int32_t B, int32_t dim, int32_t D, int32_t H1, int32_t W1, int32_t levels) {
  LookupDims ld;
  if (check_lookup_dims(B, dim, D, H1, W1, levels, 0, &ld) != SFB_OK) return 0;
  return lookup_pyramid_floats(ld) * sizeof(float);
}

int sfb_lookup_build_pyramid(const float* corr, float* pyramid, int32_t B, int32_t dim, int32_t D, int32_t H1,
                             int32_t W1, int32_t levels, void* stream) {
  LookupDims ld;
  SFB_TRY(check_lookup_dims(B, dim, D, H1, W1, levels, 0, &ld));
  if (corr == nullptr || (levels > 1 && pyramid == nullptr))
    return fail(SFB_ERR_INVALID_ARGUMENT, "corr and pyramid must not be NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SFB_CUDA(timed(KID_LOOKUP, levels - 1, st, [&] { return launch_lookup_pyramid(ld, corr, pyramid, st); }));
  return SFB_OK;
}

int sfb_lookup_forward(const float* corr, const float* pyramid, const float* coord, int64_t coord_batch_stride,
                       float* out, int32_t B, int32_t dim, int32_t D, int32_t H1, int32_t W1, int32_t levels,
                       int32_t radius, int32_t clamp_unit, void* stream) {
  LookupDims ld;
  SFB_TRY(check_lookup_dims(B, dim, D, H1, W1, levels, radius, &ld));
  if (corr == nullptr || (levels > 1 && pyramid == nullptr) || coord == nullptr || out == nullptr)
    return fail(SFB_ERR_INVALID_ARGUMENT, "corr, pyramid, coord and out must not be NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SFB_CUDA(timed(KID_LOOKUP, 1, st, [&] {
    return launch_lookup_forward(ld, corr, pyramid, coord, coord_batch_stride, out, clamp_unit, st);
  }));
  return SFB_OK;
}

int sfb_lookup_backward(const float* gout, const float* coord, int64_t coord_batch_stride, float* gcorr,
                        float* gpyramid, int32_t B, int32_t dim, int32_t D, int32_t H1, int32_t W1, int32_t levels,
                        int32_t radius, int32_t clamp_unit, void* stream) {
  LookupDims ld;
  SFB_TRY(check_lookup_dims(B, dim, D, H1, W1, levels, radius, &ld));
  if (gout == nullptr || coord == nullptr || gcorr == nullptr || (levels > 1 && gpyramid == nullptr))
    return fail(SFB_ERR_INVALID_ARGUMENT, "gout, coord, gcorr and gpyramid must not be NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SFB_CUDA(timed(KID_LOOKUP, levels > 1 ? 2 : 1, st, [&] {
    return launch_lookup_backward(ld, gout, coord, coord_batch_stride, gcorr, gpyramid, clamp_unit, st);
  }));
  return SFB_OK;
}

namespace {
int check_lookup4d(const void* F1, const void* const* F2, const int32_t* H2, const int32_t* W2, int32_t levels,
                   const void* coords, int32_t B, int32_t H1, int32_t W1, int32_t C, int32_t radius,
                   Lookup4dDims* out) {
  if (B < 1 || H1 < 1 || W1 < 1 || C < 1) return fail(SFB_ERR_INVALID_ARGUMENT, "B, H1, W1 and C must be positive");
  if (C % 4 != 0 || C > 512)
    return fail(SFB_ERR_INVALID_ARGUMENT, "the 4D lookup needs C % 4 == 0 and C <= 512");
  if (levels < 1 || levels > LOOKUP_MAX_LEVELS) return fail(SFB_ERR_INVALID_ARGUMENT, "levels must be in [1, 8]");
  if (radius < 0 || radius > 4) return fail(SFB_ERR_INVALID_ARGUMENT, "radius must be in [0, 4]");
  if (F1 == nullptr || F2 == nullptr || H2 == nullptr || W2 == nullptr || coords == nullptr)
    return fail(SFB_ERR_INVALID_ARGUMENT, "F1, F2_levels, H2, W2 and coords must not be NULL");
  if ((long long)H1 * W1 > INT32_MAX / 4) return fail(SFB_ERR_INVALID_ARGUMENT, "H1*W1 too large");
  if (reinterpret_cast<uintptr_t>(F1) % 16 != 0)
    return fail(SFB_ERR_INVALID_ARGUMENT, "feature pointers of the 4D lookup must be 16-byte aligned");
  out->B = B; out->H1 = H1; out->W1 = W1; out->C = C; out->levels = levels; out->radius = radius;
  for (int l = 0; l < levels; ++l) {
    // grid_sample's normalisation divides by size - 1 (core/utils/utils.py:114-115)
    if (H2[l] < 2 || W2[l] < 2)
      return fail(SFB_ERR_INVALID_ARGUMENT, "every pyramid level needs H2 >= 2 and W2 >= 2");
    if (F2[l] == nullptr) return fail(SFB_ERR_INVALID_ARGUMENT, "F2_levels holds a NULL pointer");
    if (reinterpret_cast<uintptr_t>(F2[l]) % 16 != 0)
      return fail(SFB_ERR_INVALID_ARGUMENT, "feature pointers of the 4D lookup must be 16-byte aligned");
    if ((long long)H2[l] * W2[l] > INT32_MAX / 4) return fail(SFB_ERR_INVALID_ARGUMENT, "H2*W2 too large");
    out->H2[l] = H2[l]; out->W2[l] = W2[l];
  }
  return SFB_OK;
}
}  // namespace

int sfb_lookup4d_forward(const float* F1, const float* const* F2_levels, const int32_t* H2, const int32_t* W2,
                         int32_t levels, const float* coords, float* out, int32_t B, int32_t H1, int32_t W1, int32_t C,
                         int32_t radius, float scale, void* stream) {
  Lookup4dDims ld;
  SFB_TRY(check_lookup4d(F1, reinterpret_cast<const void* const*>(F2_levels), H2, W2, levels, coords, B, H1, W1, C,
                         radius, &ld));
  if (out == nullptr) return fail(SFB_ERR_INVALID_ARGUMENT, "out must not be NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SFB_CUDA(timed(KID_LOOKUP4D, 1, st, [&] { return launch_lookup4d_forward(ld, F1, F2_levels, coords, out, scale, st); }));
  return SFB_OK;
}

int sfb_lookup4d_backward(const float* F1, const float* const* F2_levels, const int32_t* H2, const int32_t* W2,
                          int32_t levels, const float* coords, const float* gout, float* gF1,
                          float* const* gF2_levels, int32_t B, int32_t H1, int32_t W1, int32_t C, int32_t radius,
                          float scale, void* stream) {
  Lookup4dDims ld;
  SFB_TRY(check_lookup4d(F1, reinterpret_cast<const void* const*>(F2_levels), H2, W2, levels, coords, B, H1, W1, C,
                         radius, &ld));
  if (gout == nullptr || gF1 == nullptr || gF2_levels == nullptr)
    return fail(SFB_ERR_INVALID_ARGUMENT, "gout, gF1 and gF2_levels must not be NULL");
  for (int l = 0; l < levels; ++l)
    if (gF2_levels[l] == nullptr || reinterpret_cast<uintptr_t>(gF2_levels[l]) % 16 != 0)
      return fail(SFB_ERR_INVALID_ARGUMENT, "gF2_levels holds a NULL or not 16-byte aligned pointer");
  if (reinterpret_cast<uintptr_t>(gF1) % 16 != 0)
    return fail(SFB_ERR_INVALID_ARGUMENT, "gF1 must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SFB_CUDA(timed(KID_LOOKUP4D, 1, st, [&] {
    return launch_lookup4d_backward(ld, F1, F2_levels, coords, gout, gF1, gF2_levels, scale, st);
  }));
  return SFB_OK;
}

int sfb_set_sweep_operands(int operands) {
  if (operands != SFB_OPERANDS_TF32 && operands != SFB_OPERANDS_BF16 && operands != SFB_OPERANDS_FP16) return -1;
  return g_sweep_operands.exchange(operands);
}
int sfb_get_sweep_operands(void) { return g_sweep_operands.load(); }

int sfb_corr_volume(const float* F1, const float* F2, float* S, const sfb_shape* shape, void* workspace,
                    size_t workspace_bytes, void* stream) {
  Dims d;
  SFB_TRY(check_shape(shape, false, &d));
  SFB_CHECK_PTR(F1); SFB_CHECK_PTR(F2); SFB_CHECK_PTR(S);
  Workspace w;
  SFB_TRY(check_workspace(d, workspace, workspace_bytes, SFB_OP_CORR_VOLUME, &w));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int op16 = OP16_NONE;  // this test aid always computes with TF32 operands (its workspace has no 16-bit copies)
  CUtensorMap tm_f1, tm_f2;
  SFB_TRY(map_sweep_operands(d, w, op16, &tm_f1, &tm_f2, nullptr));
  SFB_CUDA(timed(KID_PREPARE, 2 + (op16 == OP16_FP16 ? 3 : 0), st, [&] { return prepare_operands(d, w, F1, F2, false, op16, st); }));
  SweepArgs a;
  memset(&a, 0, sizeof(a));
  a.d = d;
  a.mode = SWEEP_DUMP;
  a.n_valid = w.n1p;
  a.dump = S;
  a.status = w.status;
  SFB_CUDA(timed(KID_SWEEP_DUMP, 1, st, [&] { return launch_sweep(with_wait_settings(a), tm_f1, tm_f2, tm_f2 /* unused */, st); }));
  return SFB_OK;
}

int sfb_debug_wait_timeout(uint64_t wait_limit_ns, int drop_last_load) {
  g_wait_limit_ns.store(wait_limit_ns);
  g_drop_last_load.store(drop_last_load != 0 ? 1 : 0);
  return SFB_OK;
}

int sfb_device_status(const void* workspace, void* stream, int32_t* device_status) {
  if (workspace == nullptr || device_status == nullptr)
    return fail(SFB_ERR_INVALID_ARGUMENT, "workspace or device_status is NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t v = 0;
  SFB_CUDA(cudaMemcpyAsync(&v, workspace, sizeof(v), cudaMemcpyDeviceToHost, st));
  SFB_CUDA(cudaStreamSynchronize(st));
  *device_status = v;
  if (v != 0) return fail(SFB_ERR_DEVICE_TIMEOUT, "a bounded device-side wait gave up (device status %d)", (int)v);
  return SFB_OK;
}

const char* sfb_status_string(int code) {
  switch (code) {
    case SFB_OK: return "ok";
    case SFB_ERR_INVALID_ARGUMENT: return "invalid argument";
    case SFB_ERR_UNSUPPORTED_SHAPE: return "unsupported shape";
    case SFB_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case SFB_ERR_CUDA: return "CUDA error";
    case SFB_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}

const char* sfb_last_error(void) { return g_err; }

int sfb_kernel_timing_enable(int on) {
  std::lock_guard<std::mutex> lk(g_timing_mu);
  drain_timing_locked();
  g_timing_on = on != 0;
  for (int i = 0; i < KID_COUNT; ++i) { g_timing_ms[i] = 0; g_timing_launches[i] = 0; }
  return SFB_OK;
}

int sfb_kernel_timing_count(void) { return KID_COUNT; }

int sfb_kernel_timing_read(int kernel, const char** name, double* total_ms, int64_t* launches) {
  if (kernel < 0 || kernel >= KID_COUNT) return fail(SFB_ERR_INVALID_ARGUMENT, "kernel index %d out of range", kernel);
  std::lock_guard<std::mutex> lk(g_timing_mu);
  drain_timing_locked();
  if (name) *name = kKernelNames[kernel];
  if (total_ms) *total_ms = g_timing_ms[kernel];
  if (launches) *launches = g_timing_launches[kernel];
  return SFB_OK;
}

int sfb_version(void) { return 100; }

}  // extern "C"
