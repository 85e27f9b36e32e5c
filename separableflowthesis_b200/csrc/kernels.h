// Internal launcher interface between the C-ABI layer (c_abi.cu) and the kernel files.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace sfb {

// Host side.  Runs a per-device set-up step (cudaFuncSetAttribute and the like) once per device instead of before every launch.
// Racing first calls may both run it, which is harmless for idempotent settings.
struct DeviceOnce {
  std::atomic<bool> done[64];
  DeviceOnce() { for (auto& d : done) d.store(false); }
  template <class F>
  cudaError_t run(F&& f) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64) return f();
    if (done[dev].load(std::memory_order_acquire)) return cudaSuccess;
    err = f();
    if (err == cudaSuccess) done[dev].store(true, std::memory_order_release);
    return err;
  }
};

// Problem size of one op call (one pyramid level).  N1 = H1*W1 image-1 pixels, N2 = H2*W2.
struct Dims {
  int B, H1, W1, H2, W2, C, Kc;
  __host__ __device__ int N1() const { return H1 * W1; }
  __host__ __device__ int N2() const { return H2 * W2; }
  __host__ __device__ int aux_rows() const { return H2 + W2; }
};

// Tile constants shared by host and device code.
constexpr int TILE_M = 128;   // TMEM lanes = rows of one accumulator tile
constexpr int KBLK = 32;      // fp32 elements in one 128-byte swizzled row
#ifndef SFB_MAX_KB
#define SFB_MAX_KB 8
#endif
constexpr int MAX_KB = SFB_MAX_KB;  // feature dimension C <= MAX_KB * KBLK
constexpr int MAX_C = MAX_KB * KBLK;
constexpr int SWEEP_UT = 16;  // image-2 rows per correlation tile (16 x 16 = 256 accumulator columns)
constexpr int SWEEP_VT = 16;  // image-2 columns per correlation tile
constexpr int GG_ROW_UT = 8;  // row tile of the image-2-major gradient GEMM: 8 x 16 image-2 pixels = 128 TMEM lanes
constexpr int GG_ROW_VT = 16;
constexpr int GG_UT = 2;      // image-2 rows per K-block of the gradient GEMM (image-1-major form)
constexpr int GG_VT = 16;
constexpr int GG_KJ = 32;     // K extent (pixels of the other image) of one gradient-GEMM block
constexpr int KC_MAX_PER_SWEEP = 4;  // attention channels handled by one compression sweep

// 16-bit operand kinds of the contractions (0 = none: TF32 operands in FP32 storage).
#ifndef SFB_OP16_KINDS
#define SFB_OP16_KINDS
enum : int { OP16_NONE = 0, OP16_BF16 = 1, OP16_FP16 = 2 };
#endif
enum SweepMode : int { SWEEP_MAXAVG = 0, SWEEP_MAXARGAVG = 1, SWEEP_COMPRESS = 2, SWEEP_DUMP = 3 };
enum GradMode : int { GRAD_MAXAVG = 0, GRAD_COMPRESS = 1, GRAD_FUSED = 2 };

// A tensor indexed by (sample b, displacement d, slot, image-1 pixel p) with the pixel fastest:
// element at base + b*sb + d*sd + slot*ss + p.  Two instances of this are used:
//   "packed"         workspace arrays (B, D, slots, n1p): sb = D*slots*n1p, sd = slots*n1p, ss = n1p
//   "channels-first" user tensors   (B, slots, D, N1)  : sb = slots*D*N1,  sd = N1,        ss = D*N1
// (the layout torch's Conv3d produces and consumes at the call site, core/corr.py:437-446).
struct PixView {
  float* base;
  long long sb;      // elements between samples
  uint32_t sd, ss;   // elements between displacements / slots (one sample spans < 2^32 elements: host-checked)
};

// Correlation sweep.  Everything indexed by an image-1 pixel is read and written through PixViews, so a
// warp's 32 lanes (32 consecutive pixels) touch one or two 128-byte lines per access.
//   max/avg    : outputs pu (per u) / pv (per v): slots 0 = max, 1 = mean; argmax (int32 bits) in pu_arg / pv_arg
//   compression: weights  w_v[k][u] = xu(b, u, wv_slot0 + k*w_stride, p),  w_u[k][v] = xv(b, v, wu_slot0 + k*w_stride, p)
//                outputs  ou(b, u, k, p) = sum_v S*w_u,  ov(b, v, k, p) = sum_u S*w_v
// Lanes with p >= n_valid compute but never touch memory (n_valid = n1p for packed arrays, N1 otherwise).
struct SweepArgs {
  Dims d;
  int mode;
  int n_valid;
  int k0, kc;            // compression: first channel and number of channels (<= KC_MAX_PER_SWEEP) of this launch
  PixView pu, pv, pu_arg, pv_arg;
  PixView xu, xv;
  int wu_slot0, wv_slot0, w_stride;
  PixView ou, ov;
  int op16;              // operands are 16-bit copies (64 channels per 128-byte row, tcgen05.mma kind::f16) instead of
                         // TF32: OP16_BF16 or OP16_FP16
  const float* out_scale;  // device scalar every output value is multiplied by before it is stored (null = 1): undoes
                           // the power-of-two scaling of FP16 operands
  float* dump;           // SWEEP_DUMP: dense S (B,N1,H2,W2), test use only
  int* status;           // device status word
  unsigned long long wait_limit_ns;  // time limit of one device-side wait; 0 = the default (2 s)
  int drop_last_load;    // test hook: the producer leaves out its last F2 block, so that one wait runs out
};

// Gradient GEMM.  G = dLoss/dS is generated from two "interleaved" operand sets: for every displacement
// and image-1 pixel the R4 values (slots) that pixel contributes, in groups of four:
//   XU (B, H2, R4/4, n1p, 4)  values that depend on (pixel, u);  XV (B, W2, R4/4, n1p, 4)  (pixel, v)
// n1p = N1 rounded up to a multiple of 128 (padding is zero), R4 = slots rounded up to a multiple of 4.
// One group of four slots of 32 consecutive pixels is 512 contiguous bytes: a 16-byte load per lane, or one
// TMA box row, and conflict-free 16-byte shared-memory reads after a TMA copy.
//   GRAD_COMPRESS: G[p,u,v] = sum_r XU[u,p,r] * XV[v,p,r]            (2 slots per channel, zero padded)
//   GRAD_MAXAVG  : XU slots (mean-gradient / W2, 1, max-gradient, argmax bits), XV slots (1, mean-gradient / H2,
//                  max-gradient, argmax bits), so that slots 0 and 1 multiply to the two mean terms:
//                  G[p,u,v] = XU[u,p,0]*XV[v,p,0] + XU[u,p,1]*XV[v,p,1]
//                             + (XU[u,p,3]==v ? XU[u,p,2] : 0) + (XV[v,p,3]==u ? XV[v,p,2] : 0)
//   GRAD_FUSED   : group 0 as GRAD_MAXAVG, groups 1.. as GRAD_COMPRESS; G is the sum of both
struct GradArgs {
  Dims d;
  int mode;
  int image2_major;      // 0: rows = image-1 pixels, output gF1; 1: rows = image-2 pixels, output gF2
  int R4;                // slots per pixel in the interleaved operands: 4 or 8
  int n1p;               // padded pixel count of the interleaved operands
  int accumulate;        // 0: out = result, 1: out += result (later channel chunks of the compression op)
  int out_cf;            // 0: out is (B, pixels, C); 1: out is (B, C, pixels), the layout of the model's feature maps
  float out_scale;       // the result is multiplied by this before it is stored / added (out_cf only)
  int op16;              // G and the feature copies are 16-bit (tcgen05.mma kind::f16) instead of TF32: OP16_BF16 / OP16_FP16
  const float* dev_scale;  // device scalar the result is multiplied by as well (null = 1), see SweepArgs::out_scale
  const float* xu;
  const float* xv;
  float* out;            // gF1 (B,N1,C) or gF2 (B,N2,C)
  int* status;
  unsigned long long wait_limit_ns;  // time limit of one device-side wait; 0 = the default (2 s)
};

// One source of an interleaved slot: dst[b][d][slot/4][p][slot%4] = scale * src[b][p][k][d] (raw copy when scale == 0);
// src is (B, N1, Ksrc, D).  A null src makes the slot the constant `scale` (zero by default) for every valid pixel.
struct SlotSource {
  const void* src;
  int Ksrc, k;
  float scale;
  int dev;   // 0: nothing more; i > 0: the value is multiplied by dev_scales[i - 1] as well (FP16 operands: the
             // power-of-two scales of the gradient and weight tensors, known on the device only)
};
constexpr int MAX_SLOTS = 8;
struct SlotSources {
  SlotSource s[MAX_SLOTS];
  const float* dev_scales;  // may be null when no slot has dev != 0
};
// Same, from channels-first sources: dst[b][d][q][p][j] = scale * src[b][k][d][p], src is (B, Ksrc, D, N1).
cudaError_t launch_pack_interleaved_cf(const SlotSources& src, float* dst, int B, int N1, int n1p, int D, int R4,
                                       int Qtot, int q0, cudaStream_t stream);
// Writes R4 (4 or 8) slots = R4/4 groups starting at group q0 of dst (B, D, Qtot, n1p, 4); pixels N1 <= p < n1p
// and slots without a source are zero.
cudaError_t launch_pack_interleaved(const SlotSources& src, float* dst, int B, int N1, int n1p, int D, int R4,
                                    int Qtot, int q0, cudaStream_t stream);

// Workspace header: the status word, then (64 bytes in) the scale slots of the FP16 operand kind, all cleared by
// launch_prepare.  amax slots hold float bits (atomicMax), the others floats; every scale is a power of two.
constexpr size_t WS_HEADER_BYTES = 256, WS_SCALES_OFFSET = 64, WS_HEADER_CLEAR_BYTES = 128;
enum : int {
  SCALE_AMAX_F1 = 0, SCALE_AMAX_F2 = 1, SCALE_AMAX_G = 2, SCALE_AMAX_A = 3,
  SCALE_F1 = 4, SCALE_F2 = 5, SCALE_INV_F1F2 = 6,   // F1h = fp16(s1 F1), F2h = fp16(s2 F2), sweep outputs * 1/(s1 s2)
  SCALE_GA = 7, SCALE_G = 8, SCALE_A = 9,           // gradient slots * sg (* sa when no weight multiplies them), weights * sa
  SCALE_INV_GF1 = 10, SCALE_INV_GF2 = 11            // gF1 * 1/(sg sa s2), gF2 * 1/(sg sa s1)
};
// Rounds F1/F2 to TF32 (round-to-nearest) into the workspace copies, optionally builds the
// row/column mean rows of F2, and clears the workspace header.
// F1h / F2h / auxh (optional): the same three arrays as 16-bit operands of kind `op16` from the unrounded values: BF16,
// or FP16 after scaling by the powers of two this call derives from the arrays' largest magnitudes (scales[]).
cudaError_t launch_prepare(const Dims& d, const float* F1, const float* F2, float* F1r, float* F2r, float* aux,
                           int* status, cudaStream_t stream, uint16_t* F1h = nullptr, uint16_t* F2h = nullptr,
                           uint16_t* auxh = nullptr, int op16 = 0, float* scales = nullptr);
// The same from the model's feature maps fmap1 (B, C, H1, W1), fmap2 (B, C, H2, W2): F1r = round(scale1 * fmap1)
// transposed to (B, H1, W1, C), F2r = round(fmap2) transposed (core/corr.py:419-422 does this with
// permute().contiguous() and a division).
cudaError_t launch_prepare_cf(const Dims& d, const float* fmap1, const float* fmap2, float scale1, float* F1r,
                              float* F2r, float* aux, int* status, cudaStream_t stream, uint16_t* F1h = nullptr,
                              uint16_t* F2h = nullptr, uint16_t* auxh = nullptr, int op16 = 0, float* scales = nullptr);
// Largest |x| * premul of n floats, combined into the amax slot; the gradient-operand scales from the amax slots.
cudaError_t launch_absmax(const float* x, size_t n, float premul, float* slot, cudaStream_t stream);
cudaError_t launch_feature_scales(float* scales, cudaStream_t stream);
cudaError_t launch_grad_scales(float* scales, cudaStream_t stream);
// Channel-major copy of a (rounded) pixel-major feature array (B, rows*width, C), as FP32 or (op16 != 0) as 16-bit
// operands (FP16: times the device scalar *scale16); padding is not written.
//   blocked = 0: dst (B, C, pitch) with pixel index row*width + x (rows = 1)
//   blocked = 1: dst (B, C, ceil(width/16), pitch, 16), element (row, x) at ((x/16)*pitch + row)*16 + x%16
cudaError_t launch_channel_major(const float* src, void* dst, int B, int rows, int width, int pitch, int C,
                                 int blocked, int op16, const float* scale16, cudaStream_t stream);
// Pack: dst[b][d][r0 + k*rstride][p] = scale * src[b][p][ksrc0 + k][d] for k < K (raw 32-bit copy when
// scale == 0), zero for N1 <= p < n1p.  src is (B, N1, Ksrc, D), dst is (B, D, R, n1p).
cudaError_t launch_pack(const void* src, float* dst, int B, int N1, int n1p, int Ksrc, int ksrc0, int K, int D,
                        int R, int r0, int rstride, float scale, cudaStream_t stream);
// Unpack: dst[b][p][kdst0 + k][d] = src[b][d][r0 + k*rstride][p] for k < K; dst is (B, N1, Kdst, D).
cudaError_t launch_unpack(const float* src, void* dst, int B, int N1, int n1p, int K, int D, int R, int r0,
                          int rstride, int Kdst, int kdst0, cudaStream_t stream);
cudaError_t launch_sweep(const SweepArgs& a, const CUtensorMap& tm_f1, const CUtensorMap& tm_f2,
                         const CUtensorMap& tm_aux, cudaStream_t stream);
// tm_y: channel-major features of the other image (K-major B operand); tm_xu / tm_xv: interleaved operands (tm_xv is only read by the
// image-2-major form; the image-1-major form keeps its (pixel, v) slots in registers).
cudaError_t launch_grad_gemm(const GradArgs& a, const CUtensorMap& tm_y, const CUtensorMap& tm_xu,
                             const CUtensorMap& tm_xv, cudaStream_t stream);


// Attention weights A = softmax over d of Conv3d(2 -> Kc, 3x3x3, padding 1)(X) on channels-first tensors
// (core/corr.py:437-442): X (B, 2, D, H1, W1) with `x_sb` elements between samples, weight (Kc, 2, 3, 3, 3),
// bias (Kc), A (B, Kc, D, H1, W1).
struct AttentionDims {
  int B, Kc, D, H1, W1;
};
// `status` (optional): a device status word for bounded waits.  With it, and when W1 is a multiple of 4 and x is
// 16-byte aligned, the kernels fetch their pixel tiles (with the stencil's halo, zero-filled outside the image) by
// TMA; otherwise every thread gathers its own neighbourhood.
cudaError_t launch_attention_forward(const AttentionDims& d, const float* x, long long x_sb, const float* weight,
                                     const float* bias, float* a, cudaStream_t stream, int* status = nullptr);
// Tiled fp32 tensor map without swizzle, zero fill out of bounds; dims / box innermost first, `strides_bytes` for
// dimensions 1 .. rank-1.  Implemented next to the other tensor maps (c_abi.cu).
cudaError_t encode_plain_map(CUtensorMap* tm, const void* base, int rank, const uint64_t* dims,
                             const uint64_t* strides_bytes, const uint32_t* box);
// Floats of scratch the backward needs for its per-block partial sums.
size_t attention_partial_floats(const AttentionDims& d);
// Backward: `g` holds dLoss/dA on entry and the logit gradients on return; gx (B, 2, D, H1, W1) = add + dLoss/dX
// where `add` (same shape, `add_sb` elements between samples) may be null; gweight (Kc, 2, 3, 3, 3), gbias (Kc).
cudaError_t launch_attention_backward(const AttentionDims& d, const float* x, long long x_sb, const float* weight,
                                      const float* a, float* g, const float* add, long long add_sb, float* gx,
                                      float* gweight, float* gbias, float* partial, cudaStream_t stream,
                                      int* status = nullptr);


// Linear resampling along the displacement axis (core/corr.py:459-467: trilinear interpolate with unchanged H1, W1):
// in (B, K, Dl, N1) -> K channels of a larger tensor, out[b] at out + b*out_sb, each (K, D0, N1); Dl <= D0.
cudaError_t launch_upsample_displacement(const float* in, float* out, long long out_sb, int B, int K, int Dl, int D0,
                                         int N1, cudaStream_t stream);
// Its adjoint: gin (B, K, Dl, N1) from the gradient of those K channels.
cudaError_t launch_upsample_displacement_adjoint(const float* gout, long long gout_sb, float* gin, int B, int K, int Dl,
                                                 int D0, int N1, cudaStream_t stream);

// Lookup on an aggregated 3D cost volume (the reference's CorrBlock1D, core/corr.py:513-624).
// corr (B, dim, D, H1, W1); pyramid = levels 1 .. levels-1 back to back, level l being (B, dim, D >> l, H1, W1);
// coord: one displacement component per pixel, (B, H1, W1) with `coord_sb` elements between samples;
// out (B, levels*dim*(2*radius+1), H1, W1).
constexpr int LOOKUP_MAX_LEVELS = 8;
struct LookupDims {
  int B, dim, D, H1, W1, levels, radius;
};
size_t lookup_pyramid_floats(const LookupDims& d);
cudaError_t launch_lookup_pyramid(const LookupDims& d, const float* corr, float* pyramid, cudaStream_t stream);
cudaError_t launch_lookup_forward(const LookupDims& d, const float* corr, const float* pyramid, const float* coord,
                                  long long coord_sb, float* out, int clamp_unit, cudaStream_t stream);
// gcorr and gpyramid (same sizes as corr / pyramid) are overwritten; gpyramid is scratch.
cudaError_t launch_lookup_backward(const LookupDims& d, const float* gout, const float* coord, long long coord_sb,
                                   float* gcorr, float* gpyramid, int clamp_unit, cudaStream_t stream);

// Lookup on the 4D correlation volume without storing it (the call core/corr.py:491-510 leaves unimplemented; its
// result is the dense block's lookup, core/corr.py:192-247).  F1 (B, H1, W1, C) and the image-2 feature pyramid
// F2[l] (B, H2[l], W2[l], C), channels innermost; coords (B, 2, H1, W1) = (x, y) per pixel;
// out (B, levels*(2*radius+1)^2, H1, W1), every product times `scale`.  C % 4 == 0, C <= 512, radius <= 4.
struct Lookup4dDims {
  int B, H1, W1, C, levels, radius;
  int H2[LOOKUP_MAX_LEVELS], W2[LOOKUP_MAX_LEVELS];
};
cudaError_t launch_lookup4d_forward(const Lookup4dDims& d, const float* F1, const float* const* F2,
                                    const float* coords, float* out, float scale, cudaStream_t stream);
// gF1 (shape of F1) is overwritten; gF2[l] (shape of F2[l]) is zeroed and then accumulated with float reductions.
cudaError_t launch_lookup4d_backward(const Lookup4dDims& d, const float* F1, const float* const* F2,
                                     const float* coords, const float* gout, float* gF1, float* const* gF2,
                                     float scale, cudaStream_t stream);

}  // namespace sfb
