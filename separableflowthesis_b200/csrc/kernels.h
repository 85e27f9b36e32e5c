// Internal launcher interface between the C-ABI layer (c_abi.cu) and the kernel files.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sfb {

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
constexpr int MAX_KB = 8;     // feature dimension C <= MAX_KB * KBLK
constexpr int MAX_C = MAX_KB * KBLK;
constexpr int SWEEP_UT = 8;   // image-2 rows per correlation tile
constexpr int SWEEP_VT = 16;  // image-2 columns per correlation tile
constexpr int GG_UT = 2;      // image-2 rows per K-block of the gradient GEMM (image-1-major form)
constexpr int GG_VT = 16;
constexpr int GG_KJ = 32;     // K extent (pixels of the other image) of one gradient-GEMM block
constexpr int KC_MAX_PER_SWEEP = 4;  // attention channels handled by one compression sweep

enum SweepMode : int { SWEEP_MAXAVG = 0, SWEEP_MAXARGAVG = 1, SWEEP_COMPRESS = 2, SWEEP_DUMP = 3 };
enum GradMode : int { GRAD_MAXAVG = 0, GRAD_COMPRESS = 1 };

// Correlation sweep.  Everything indexed by an image-1 pixel is read and written in "packed" layout
// (displacement, slot, pixel) with the pixel fastest and the pixel count padded to n1p (multiple of
// 128), so that the 32 lanes of a warp (32 consecutive pixels) touch one 128-byte line:
//   max/avg    : outputs PU (B, H2, 3, n1p), PV (B, W2, 3, n1p); slots 0 = max, 1 = mean, 2 = argmax bits
//   compression: weights  w_v[k][u] = XU[b][u][wv_slot0 + k*w_stride][p]   (B, H2, Rw, n1p)
//                         w_u[k][v] = XV[b][v][wu_slot0 + k*w_stride][p]   (B, W2, Rw, n1p)
//                outputs  OU (B, H2, Ro, n1p) slot k = sum_v S*w_u,  OV (B, W2, Ro, n1p) slot k = sum_u S*w_v
struct SweepArgs {
  Dims d;
  int mode;
  int n1p;
  int k0, kc;            // compression: first channel and number of channels (<= KC_MAX_PER_SWEEP) of this launch
  float* pu; float* pv;  // max/avg packed outputs
  const float* xu; const float* xv;
  int Rw, wu_slot0, wv_slot0, w_stride;
  float* ou; float* ov;
  int Ro;
  float* dump;           // SWEEP_DUMP: dense S (B,N1,H2,W2), test use only
  int* status;           // device status word
};

// Gradient GEMM.  G = dLoss/dS is generated from two "packed" operand sets laid out with the image-1
// pixel index fastest, so that one warp reads 32 consecutive pixels with one 128-byte request:
//   XU (B, H2, R, N1p)  values that depend on (pixel, u);  XV (B, W2, R, N1p)  values that depend on (pixel, v)
// N1p = N1 rounded up to a multiple of 128, padding is zero.
//   GRAD_COMPRESS: G[p,u,v] = sum_r XU[u,r,p] * XV[v,r,p]            (R = 2 * channels of this launch)
//   GRAD_MAXAVG  : R = 3, slots (mean-gradient already divided by the row length, max-gradient, argmax bits):
//                  G[p,u,v] = XU[u,0,p] + XV[v,0,p] + (XU[u,2,p]==v ? XU[u,1,p] : 0) + (XV[v,2,p]==u ? XV[v,1,p] : 0)
struct GradArgs {
  Dims d;
  int mode;
  int image2_major;      // 0: rows = image-1 pixels, output gF1; 1: rows = image-2 pixels, output gF2
  int R;                 // slots of this launch (compile-time variants 2,4,6,8 / 3)
  int Rtot, r0;          // slots per (u | v) in the packed arrays and first slot of this launch
  int n1p;               // padded pixel count of the packed operands
  int accumulate;        // 0: out = result, 1: out += result (later channel chunks of the compression op)
  const float* xu;
  const float* xv;
  float* out;            // gF1 (B,N1,C) or gF2 (B,N2,C)
  int* status;
};

// Rounds F1/F2 to TF32 (round-to-nearest) into the workspace copies, optionally builds the
// row/column mean rows of F2, and clears the status word.
cudaError_t launch_prepare(const Dims& d, const float* F1, const float* F2, float* F1r, float* F2r, float* aux,
                           int* status, cudaStream_t stream);
// Pack: dst[b][d][r0 + k*rstride][p] = scale * src[b][p][ksrc0 + k][d] for k < K (raw 32-bit copy when
// scale == 0), zero for N1 <= p < n1p.  src is (B, N1, Ksrc, D), dst is (B, D, R, n1p).
cudaError_t launch_pack(const void* src, float* dst, int B, int N1, int n1p, int Ksrc, int ksrc0, int K, int D,
                        int R, int r0, int rstride, float scale, cudaStream_t stream);
// Unpack: dst[b][p][kdst0 + k][d] = src[b][d][r0 + k*rstride][p] for k < K; dst is (B, N1, Kdst, D).
cudaError_t launch_unpack(const float* src, void* dst, int B, int N1, int n1p, int K, int D, int R, int r0,
                          int rstride, int Kdst, int kdst0, cudaStream_t stream);
cudaError_t launch_sweep(const SweepArgs& a, const CUtensorMap& tm_f1, const CUtensorMap& tm_f2,
                         const CUtensorMap& tm_aux, cudaStream_t stream);
cudaError_t launch_grad_gemm(const GradArgs& a, const CUtensorMap& tm_y, cudaStream_t stream);

}  // namespace sfb
