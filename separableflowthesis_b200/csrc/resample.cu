// Placement of one pyramid level's separated volumes into the concatenated, level-0-sized outputs of the call site
// (core/corr.py:459-475): F.interpolate(..., mode='trilinear', align_corners=True) to [D0, H1, W1] followed by
// torch.cat over the levels.  H1 and W1 do not change, so the resampling is linear interpolation along the
// displacement axis only; the arithmetic follows torch's upsample_trilinear3d (source index = d * (Dl-1)/(D0-1) in
// float, lower neighbour by truncation, the upper neighbour clamped to the last row).  HBM-bound streaming kernels;
// every output element is written once, the backward (the adjoint) has one thread per (sample, channel, pixel) walk
// the displacement axis, so it needs no atomics.
#include "kernels.h"

namespace sfb {

constexpr int RS_THREADS = 128;

__device__ __forceinline__ void resample_source(int d, float scale, int Dl, int& i0, int& i1, float& l0, float& l1) {
  const float src = scale * (float)d;
  i0 = (int)src;
  if (i0 > Dl - 1) i0 = Dl - 1;
  i1 = i0 + (i0 < Dl - 1 ? 1 : 0);
  l1 = src - (float)i0;
  l0 = 1.f - l1;
}

// grid (ceil(N1/128), ceil(D0/RS_DB), B*K): a thread produces RS_DB output rows of its pixel, all loads first
constexpr int RS_DB = 8;

__global__ void upsample_displacement_kernel(const float* __restrict__ in, float* __restrict__ out, long long out_sb,
                                             int K, int Dl, int D0, int N1, float scale) {
  const int p = blockIdx.x * RS_THREADS + threadIdx.x, d0 = blockIdx.y * RS_DB;
  if (p >= N1) return;
  const int b = blockIdx.z / K, k = blockIdx.z - b * K;
  const float* src = in + ((size_t)blockIdx.z * Dl) * N1 + p;
  float v0[RS_DB], v1[RS_DB], l0[RS_DB], l1[RS_DB];
#pragma unroll
  for (int j = 0; j < RS_DB; ++j) {
    int i0, i1;
    resample_source(min(d0 + j, D0 - 1), scale, Dl, i0, i1, l0[j], l1[j]);
    v0[j] = __ldg(src + (size_t)i0 * N1);
    v1[j] = __ldg(src + (size_t)i1 * N1);
  }
  float* dst = out + (size_t)b * out_sb + ((size_t)k * D0 + d0) * N1 + p;
#pragma unroll
  for (int j = 0; j < RS_DB; ++j)
    if (d0 + j < D0) dst[(size_t)j * N1] = l0[j] * v0[j] + l1[j] * v1[j];
}

// gin[b][k][i][p] = sum over d of the weights with which output row d read input row i.  grid (ceil(N1/128), B*K)
__global__ void upsample_displacement_adjoint_kernel(const float* __restrict__ gout, long long gout_sb,
                                                     float* __restrict__ gin, int K, int Dl, int D0, int N1,
                                                     float scale) {
  const int p = blockIdx.x * RS_THREADS + threadIdx.x;
  if (p >= N1) return;
  const int b = blockIdx.y / K, k = blockIdx.y - b * K;
  const float* g = gout + (size_t)b * gout_sb + ((size_t)k * D0) * N1 + p;
  float* dst = gin + ((size_t)blockIdx.y * Dl) * N1 + p;
  // the source row grows by at most one per output row (Dl <= D0): two running sums cover rows cur and cur + 1
  int cur = 0;
  float acc0 = 0.f, acc1 = 0.f;
  constexpr int DB = 8;  // output rows loaded per batch
  for (int d0 = 0; d0 < D0; d0 += DB) {
    float gv[DB];
#pragma unroll
    for (int j = 0; j < DB; ++j) gv[j] = d0 + j < D0 ? __ldg(g + (size_t)(d0 + j) * N1) : 0.f;
#pragma unroll
    for (int j = 0; j < DB; ++j) {
      if (d0 + j >= D0) break;
      int i0, i1;
      float l0, l1;
      resample_source(d0 + j, scale, Dl, i0, i1, l0, l1);
      while (cur < i0) {  // at most one step
        dst[(size_t)cur * N1] = acc0;
        acc0 = acc1;
        acc1 = 0.f;
        ++cur;
      }
      acc0 = fmaf(l0, gv[j], acc0);
      if (i1 != i0) acc1 = fmaf(l1, gv[j], acc1);
      else acc0 = fmaf(l1, gv[j], acc0);
    }
  }
  dst[(size_t)cur * N1] = acc0;
  if (cur + 1 < Dl) dst[(size_t)(cur + 1) * N1] = acc1;
  for (int i = cur + 2; i < Dl; ++i) dst[(size_t)i * N1] = 0.f;
}

static float resample_scale(int Dl, int D0) { return D0 > 1 ? (float)(Dl - 1) / (float)(D0 - 1) : 0.f; }

cudaError_t launch_upsample_displacement(const float* in, float* out, long long out_sb, int B, int K, int Dl, int D0,
                                         int N1, cudaStream_t st) {
  const dim3 grid((N1 + RS_THREADS - 1) / RS_THREADS, (D0 + RS_DB - 1) / RS_DB, B * K);
  upsample_displacement_kernel<<<grid, RS_THREADS, 0, st>>>(in, out, out_sb, K, Dl, D0, N1, resample_scale(Dl, D0));
  return cudaGetLastError();
}

cudaError_t launch_upsample_displacement_adjoint(const float* gout, long long gout_sb, float* gin, int B, int K, int Dl,
                                                 int D0, int N1, cudaStream_t st) {
  const dim3 grid((N1 + RS_THREADS - 1) / RS_THREADS, B * K);
  upsample_displacement_adjoint_kernel<<<grid, RS_THREADS, 0, st>>>(gout, gout_sb, gin, K, Dl, D0, N1,
                                                                    resample_scale(Dl, D0));
  return cudaGetLastError();
}

}  // namespace sfb
