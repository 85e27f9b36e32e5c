// Lookup on the two aggregated 3D cost volumes (the reference's CorrBlock1D, core/corr.py:513-624): a pyramid of
// each volume over its displacement axis (average pooling by 2, core/corr.py:543-548) and, per refinement
// iteration, 2r+1 linearly interpolated samples per pyramid level around the current displacement estimate of every
// image-1 pixel (core/corr.py:576-594, F.grid_sample with align_corners=True and zero padding, one row high).
//
// HBM-bound gathers.  The volumes stay in the layout the rest of the path produces, (B, dim, D, H1, W1): the
// displacement axis of one pixel is strided by the plane size, a warp handles 32 neighbouring pixels, and because
// neighbouring pixels have similar displacements their gathers mostly fall into the same 128-byte lines.  (The
// reference first permutes to (B*H1*W1, dim, 1, D), core/corr.py:531-541.)
// Backward: every (b, channel, displacement, pixel) element of a level's gradient is touched by one thread only,
// so the scatter needs no atomics; the levels are then folded into the gradient of the volume in one pass.
#include "kernels.h"

namespace sfb {

constexpr int LK_THREADS = 128;

// out[plane][d][p] = (in[plane][2d][p] + in[plane][2d+1][p]) / 2, d < Dout = Din / 2.  grid (ceil(N1/128), Dout, planes)
__global__ void lookup_pool_kernel(const float* __restrict__ in, float* __restrict__ out, int Din, int Dout, int N1) {
  const int p = blockIdx.x * LK_THREADS + threadIdx.x, d = blockIdx.y;
  if (p >= N1) return;
  const float* src = in + ((size_t)blockIdx.z * Din + 2 * d) * N1 + p;
  out[((size_t)blockIdx.z * Dout + d) * N1 + p] = 0.5f * (__ldg(src) + __ldg(src + N1));
}

// Sampling position of tap t at level l, exactly as the reference computes it: displacement estimate / 2^l + offset
// (core/corr.py:581-582), optionally clamped to [-1, 1] (core/corr.py:586, the first volume only), then through
// grid_sample's normalisation and back (core/corr.py:553, align_corners=True).
__device__ __forceinline__ float lookup_position(float c, int level, int t, int radius, int clamp_unit, int Dl) {
  float x = (float)(t - radius) + c / (float)(1 << level);
  if (clamp_unit) x = fminf(fmaxf(x, -1.f), 1.f);
  const float xn = 2.f * x / (float)(Dl - 1) - 1.f;
  return (xn + 1.f) * 0.5f * (float)(Dl - 1);
}

struct LookupLevels {
  const float* ptr[LOOKUP_MAX_LEVELS];   // level l: (B, dim, D_l, N1)
  int D[LOOKUP_MAX_LEVELS];
};
struct LookupLevelsMut {
  float* ptr[LOOKUP_MAX_LEVELS];
  int D[LOOKUP_MAX_LEVELS];
};

// out (B, levels*dim*(2r+1), N1): channel (l*dim + ch)*(2r+1) + t.  grid (ceil(N1/128), B)
__global__ void lookup_forward_kernel(const LookupLevels lv, const float* __restrict__ coord, long long coord_sb,
                                      float* __restrict__ out, int dim, int N1, int levels, int radius,
                                      int clamp_unit) {
  const int p = blockIdx.x * LK_THREADS + threadIdx.x, b = blockIdx.y;
  if (p >= N1) return;
  const float c = __ldg(coord + (size_t)b * coord_sb + p);
  const int taps = 2 * radius + 1;
  float* o = out + (size_t)b * levels * dim * taps * N1 + p;
  for (int l = 0; l < levels; ++l) {
    const int Dl = lv.D[l];
    for (int t = 0; t < taps; ++t) {
      const float ix = lookup_position(c, l, t, radius, clamp_unit, Dl);
      const float fl = floorf(ix);
      const float w1 = ix - fl, w0 = 1.f - w1;
      // a position far outside the volume (or NaN) samples zeros; clamp before the conversion to int
      const int i0 = (int)fminf(fmaxf(fl, -2.f), (float)Dl), i1 = i0 + 1;
      const bool in0 = i0 >= 0 && i0 < Dl && fl == (float)i0, in1 = i1 >= 0 && i1 < Dl && fl == (float)i0;
      for (int ch = 0; ch < dim; ++ch) {
        const float* v = lv.ptr[l] + ((size_t)(b * dim + ch) * Dl) * N1 + p;
        float r = 0.f;
        if (in0) r = w0 * __ldg(v + (size_t)i0 * N1);
        if (in1) r = fmaf(w1, __ldg(v + (size_t)i1 * N1), r);
        o[(size_t)((l * dim + ch) * taps + t) * N1] = r;
      }
    }
  }
}

// Scatter of the output gradients into the (zero-initialised) gradients of the levels.  Same grid.
__global__ void lookup_backward_kernel(const LookupLevelsMut gl, const float* __restrict__ coord, long long coord_sb,
                                       const float* __restrict__ gout, int dim, int N1, int levels, int radius,
                                       int clamp_unit) {
  const int p = blockIdx.x * LK_THREADS + threadIdx.x, b = blockIdx.y;
  if (p >= N1) return;
  const float c = __ldg(coord + (size_t)b * coord_sb + p);
  const int taps = 2 * radius + 1;
  const float* go = gout + (size_t)b * levels * dim * taps * N1 + p;
  for (int l = 0; l < levels; ++l) {
    const int Dl = gl.D[l];
    for (int t = 0; t < taps; ++t) {
      const float ix = lookup_position(c, l, t, radius, clamp_unit, Dl);
      const float fl = floorf(ix);
      const float w1 = ix - fl, w0 = 1.f - w1;
      const int i0 = (int)fminf(fmaxf(fl, -2.f), (float)Dl), i1 = i0 + 1;
      const bool in0 = i0 >= 0 && i0 < Dl && fl == (float)i0, in1 = i1 >= 0 && i1 < Dl && fl == (float)i0;
      for (int ch = 0; ch < dim; ++ch) {
        const float g = __ldg(go + (size_t)((l * dim + ch) * taps + t) * N1);
        float* v = gl.ptr[l] + ((size_t)(b * dim + ch) * Dl) * N1 + p;
        // this thread is the only writer of its pixel's column, and its taps run in program order
        if (in0) v[(size_t)i0 * N1] += w0 * g;
        if (in1) v[(size_t)i1 * N1] += w1 * g;
      }
    }
  }
}

// gcorr[plane][i][p] += sum_{l >= 1} glevel_l[plane][i >> l][p] / 2^l  (the pooling of level l spreads its gradient
// evenly over the 2^l entries it averaged; entries dropped by the floor of an odd size get none).
// grid (ceil(N1/128), D, planes)
__global__ void lookup_fold_kernel(const LookupLevelsMut gl, int N1, int levels) {
  const int p = blockIdx.x * LK_THREADS + threadIdx.x, i = blockIdx.y;
  if (p >= N1) return;
  float acc = 0.f, scale = 1.f;
  int parent_ok = 1;
  for (int l = 1; l < levels; ++l) {
    scale *= 0.5f;
    const int j = i >> l;
    // entry i is inside level l's pooling window only if it was inside every finer level's
    parent_ok = parent_ok && (i >> (l - 1)) < 2 * gl.D[l] && j < gl.D[l];
    if (!parent_ok) break;
    acc = fmaf(scale, gl.ptr[l][((size_t)blockIdx.z * gl.D[l] + j) * N1 + p], acc);
  }
  float* dst = gl.ptr[0] + ((size_t)blockIdx.z * gl.D[0] + i) * N1 + p;
  *dst += acc;
}

// Backward in one pass for radius <= LK_RMAX: per level, the taps of a pixel touch a window of at most 2r+3
// consecutive rows, which the thread accumulates in shared memory (its own column, no barrier); it then writes its
// whole displacement column of the volume gradient once, folding the levels in as it goes (a level-l entry spreads
// evenly over the 2^l level-0 entries it averaged).  No memset, no read-modify-write, no pyramid scratch.
// grid (ceil(N1/128), B * dim)
constexpr int LK_RMAX = 4;
constexpr int LK_WIN = 2 * LK_RMAX + 4;

__global__ void __launch_bounds__(LK_THREADS)
lookup_backward_window_kernel(const float* __restrict__ coord, long long coord_sb, const float* __restrict__ gout,
                              float* __restrict__ gcorr, int dim, int D, int N1, int levels, int radius,
                              int clamp_unit) {
  __shared__ float win[LOOKUP_MAX_LEVELS][LK_WIN][LK_THREADS];
  const int p = blockIdx.x * LK_THREADS + threadIdx.x, b = blockIdx.y / dim, ch = blockIdx.y - b * dim;
  if (p >= N1) return;
  const int tid = threadIdx.x;
  const float c = __ldg(coord + (size_t)b * coord_sb + p);
  const int taps = 2 * radius + 1;
  const float* go = gout + (size_t)b * levels * dim * taps * N1 + p;
  int wbase[LOOKUP_MAX_LEVELS], Dl[LOOKUP_MAX_LEVELS];
  int Dcur = D;
  for (int l = 0; l < levels; ++l, Dcur /= 2) {
    Dl[l] = Dcur;
    for (int s = 0; s < LK_WIN; ++s) win[l][s][tid] = 0.f;
    for (int t = 0; t < taps; ++t) {
      const float ix = lookup_position(c, l, t, radius, clamp_unit, Dcur);
      const float fl = floorf(ix);
      const float w1 = ix - fl, w0 = 1.f - w1;
      const int i0 = (int)fminf(fmaxf(fl, -2.f), (float)Dcur);
      if (t == 0) wbase[l] = i0;
      const float g = __ldg(go + (size_t)((l * dim + ch) * taps + t) * N1);
      const int s0 = i0 - wbase[l];   // positions grow with t: 0 <= s0 <= 2r+1 (+1 of rounding slack)
      if (s0 >= 0 && s0 + 1 < LK_WIN) {
        win[l][s0][tid] += w0 * g;      // rows outside the volume are dropped when the column is written
        win[l][s0 + 1][tid] += w1 * g;
      }
    }
  }
  float* dst = gcorr + ((size_t)(b * dim + ch) * D) * N1 + p;
  // rows below / above every level's window get no gradient: plain zero stores
  int lo = D, hi = 0;
  for (int l = 0; l < levels; ++l) {
    lo = min(lo, max(wbase[l], 0) << l);
    hi = max(hi, min((wbase[l] + LK_WIN) << l, D));
  }
  lo = min(lo, D);
  for (int i = 0; i < lo; ++i) dst[(size_t)i * N1] = 0.f;
  for (int i = max(hi, lo); i < D; ++i) dst[(size_t)i * N1] = 0.f;
  for (int i = lo; i < max(hi, lo); ++i) {
    float acc = 0.f, scale = 1.f;
    for (int l = 0; l < levels; ++l, scale *= 0.5f) {
      const int j = i >> l;
      if (j >= Dl[l]) break;            // dropped by the floor of an odd size: no coarser level sees it either
      const int s = j - wbase[l];
      if (s >= 0 && s < LK_WIN) acc = fmaf(scale, win[l][s][tid], acc);
    }
    dst[(size_t)i * N1] = acc;
  }
}

// ---- launchers ---------------------------------------------------------------------------------------
size_t lookup_pyramid_floats(const LookupDims& d) {  // levels 1 .. levels-1
  size_t n = 0;
  int Dl = d.D;
  for (int l = 1; l < d.levels; ++l) { Dl /= 2; n += (size_t)d.B * d.dim * Dl * d.H1 * d.W1; }
  return n;
}

template <class L, class P>
static void fill_levels(L& lv, const LookupDims& d, P* level0, P* pyramid) {
  int Dl = d.D;
  P* next = pyramid;
  for (int l = 0; l < LOOKUP_MAX_LEVELS; ++l) { lv.ptr[l] = nullptr; lv.D[l] = 0; }
  for (int l = 0; l < d.levels; ++l) {
    lv.ptr[l] = l == 0 ? level0 : next;
    lv.D[l] = Dl;
    if (l > 0) next += (size_t)d.B * d.dim * Dl * d.H1 * d.W1;
    Dl /= 2;
  }
}

cudaError_t launch_lookup_pyramid(const LookupDims& d, const float* corr, float* pyramid, cudaStream_t st) {
  LookupLevelsMut lv;
  fill_levels(lv, d, const_cast<float*>(corr), pyramid);
  const int N1 = d.H1 * d.W1;
  for (int l = 1; l < d.levels; ++l) {
    if (lv.D[l] == 0) continue;
    const dim3 grid((N1 + LK_THREADS - 1) / LK_THREADS, lv.D[l], d.B * d.dim);
    lookup_pool_kernel<<<grid, LK_THREADS, 0, st>>>(lv.ptr[l - 1], lv.ptr[l], lv.D[l - 1], lv.D[l], N1);
  }
  return cudaGetLastError();
}

cudaError_t launch_lookup_forward(const LookupDims& d, const float* corr, const float* pyramid, const float* coord,
                                  long long coord_sb, float* out, int clamp_unit, cudaStream_t st) {
  LookupLevels lv;
  fill_levels(lv, d, corr, pyramid);
  const int N1 = d.H1 * d.W1;
  const dim3 grid((N1 + LK_THREADS - 1) / LK_THREADS, d.B);
  lookup_forward_kernel<<<grid, LK_THREADS, 0, st>>>(lv, coord, coord_sb, out, d.dim, N1, d.levels, d.radius, clamp_unit);
  return cudaGetLastError();
}

cudaError_t launch_lookup_backward(const LookupDims& d, const float* gout, const float* coord, long long coord_sb,
                                   float* gcorr, float* gpyramid, int clamp_unit, cudaStream_t st) {
  const int N1 = d.H1 * d.W1;
  if (d.radius <= LK_RMAX) {
    const dim3 wgrid((N1 + LK_THREADS - 1) / LK_THREADS, d.B * d.dim);
    lookup_backward_window_kernel<<<wgrid, LK_THREADS, 0, st>>>(coord, coord_sb, gout, gcorr, d.dim, d.D, N1, d.levels,
                                                               d.radius, clamp_unit);
    return cudaGetLastError();
  }
  LookupLevelsMut gl;
  fill_levels(gl, d, gcorr, gpyramid);
  cudaError_t err = cudaMemsetAsync(gcorr, 0, (size_t)d.B * d.dim * d.D * N1 * sizeof(float), st);
  if (err != cudaSuccess) return err;
  const size_t pyr = lookup_pyramid_floats(d);
  if (pyr > 0) {
    err = cudaMemsetAsync(gpyramid, 0, pyr * sizeof(float), st);
    if (err != cudaSuccess) return err;
  }
  const dim3 grid((N1 + LK_THREADS - 1) / LK_THREADS, d.B);
  lookup_backward_kernel<<<grid, LK_THREADS, 0, st>>>(gl, coord, coord_sb, gout, d.dim, N1, d.levels, d.radius,
                                                     clamp_unit);
  if (d.levels > 1) {
    const dim3 fgrid((N1 + LK_THREADS - 1) / LK_THREADS, d.D, d.B * d.dim);
    lookup_fold_kernel<<<fgrid, LK_THREADS, 0, st>>>(gl, N1, d.levels);
  }
  return cudaGetLastError();
}

}  // namespace sfb
