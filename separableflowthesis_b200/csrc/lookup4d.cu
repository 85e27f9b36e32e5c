// Lookup on the 4D correlation volume WITHOUT storing it: the part the reference leaves unimplemented for its
// memory-saving block (core/corr.py:491-510 raises NotImplementedError and then sketches the call it would make,
// alt_cuda_corr.forward(fmap1 (B,H1,W1,C), fmap2_l (B,H2_l,W2_l,C), coords / 2^l, radius) per pyramid level).  The
// result is the dense block's lookup (core/corr.py:192-247): for every image-1 pixel and pyramid level l a
// (2r+1) x (2r+1) window of the level-l volume around coords / 2^l, bilinearly interpolated with zero padding
// (core/utils/utils.py:110-118, F.grid_sample with align_corners=True), divided by sqrt(C) (core/corr.py:286).
// Averaging the volume over 2x2 blocks of image-2 positions (core/corr.py:36-39) equals correlating with the
// average-pooled image-2 features, so level l needs only the pooled features, never the volume.
//
// Work per (pixel, level): the (2r+2)^2 dot products of the pixel's feature row with the image-2 feature rows at
// the integer positions under its window, then (2r+1)^2 bilinear combinations of them.  A gather bound by the
// L1/L2 path of the image-2 rows (1 KB each at C = 256), so the kernel shares them: a warp takes four
// neighbouring pixels, whose windows mostly overlap because neighbouring pixels move alike, walks the bounding box
// of the four windows once, and uses every loaded image-2 row for all four pixels (feature rows of the four pixels
// in registers, lanes split the channels).  Partial sums of 32 (position, pixel) pairs are reduced together with a
// 31-shuffle transpose.  When the four windows lie far apart (a motion boundary, a wrap to the next image row) the
// warp falls back to one pixel at a time.  A CTA covers 32 consecutive pixels and stages its outputs in shared
// memory so that the (B, levels*(2r+1)^2, H1, W1) result is written in full 128-byte lines.
//
// Backward (features only: the model detaches the coordinates, core/sepflow.py:193): the same walk with the roles
// swapped.  The gradient of a pixel's window is spread back onto the integer positions (each takes from at most four
// window entries), gF1 accumulates in registers over all positions and levels and is stored once, and the
// image-2 feature gradient of every position receives one 16-byte vector reduction per lane (red.global.add.v4.f32).
#include <climits>

#include "kernels.h"

namespace sfb {

constexpr int L4_THREADS = 256;
constexpr int L4_WARPS = L4_THREADS / 32;
constexpr int L4_PX = 4;                       // pixels per warp
constexpr int L4_TILE = L4_WARPS * L4_PX;      // pixels per CTA
constexpr int L4_RMAX = 4;
constexpr int L4_WIN = 2 * L4_RMAX + 1;        // window side
constexpr int L4_BW = 16, L4_BH = 12;          // largest bounding box a four-pixel pass accepts
constexpr int L4_BMAX = L4_BW * L4_BH;
#ifndef L4_BWD_STEP
#define L4_BWD_STEP 2
#endif
static_assert(L4_TILE == 32, "the output staging assumes 32 pixels per CTA");
static_assert((2 * L4_RMAX + 2) * (2 * L4_RMAX + 2) <= L4_BMAX, "one pixel's positions must fit the buffer");

struct Lookup4dLevels {
  const float* f2[LOOKUP_MAX_LEVELS];   // level l: (B, H2_l, W2_l, C)
  float* g2[LOOKUP_MAX_LEVELS];         // gradient of the same (backward only)
  int H2[LOOKUP_MAX_LEVELS], W2[LOOKUP_MAX_LEVELS];
};

// A position through grid_sample's normalisation and back (core/utils/utils.py:114-115 and torch's
// grid_sampler_unnormalize for align_corners=True), in the reference's order of float operations.
__device__ __forceinline__ float l4_unnormalise(float x, int size) {
  const float g = 2.f * x / (float)(size - 1) - 1.f;
  return (g + 1.f) * 0.5f * (float)(size - 1);
}

// floor() to an int that later +-radius arithmetic cannot overflow; positions that far out sample only padding.
__device__ __forceinline__ int l4_floor(float x) {
  if (!(x > -1.0e6f)) return -1000000;   // also NaN
  if (x > 1.0e6f) return 1000000;
  return (int)floorf(x);
}

struct L4Pixel {     // geometry of one pixel at one level
  float cx, cy;      // coords / 2^l
  int bx, by;        // integer position under the window centre
};

__device__ __forceinline__ float dot4(const float4& a, const float4& b, float acc) {
  return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, fmaf(a.w, b.w, acc))));
}

// v[i] of all lanes summed; lane i keeps the total of v[i].  31 shuffles for 32 values.
__device__ __forceinline__ float warp_transpose_reduce(float (&v)[32], int lane) {
#pragma unroll
  for (int s = 0; s < 5; ++s) {
    const int off = 16 >> s, n = 32 >> s;
    const bool up = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const float send = up ? v[i] : v[i + n / 2];
      const float keep = up ? v[i + n / 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  return v[0];
}

// Interpolation weight pair of window entry t along one axis: the reference's position of that entry
// (centre / 2^l + t - r, then normalised and back), expressed against the integer position base + t - r.
__device__ __forceinline__ float l4_fraction(float c, int base, int t, int radius, int size) {
  const float pos = l4_unnormalise(c + (float)(t - radius), size);
  return pos - (float)(base + t - radius);
}

__device__ __forceinline__ void l4_pixel_geometry(const float* __restrict__ coords, int b, int p, int N1, int level,
                                                  int H2, int W2, L4Pixel& g) {
  const float inv = 1.f / (float)(1 << level);
  g.cx = __ldg(coords + ((size_t)b * 2 + 0) * N1 + p) * inv;
  g.cy = __ldg(coords + ((size_t)b * 2 + 1) * N1 + p) * inv;
  g.bx = l4_floor(l4_unnormalise(g.cx, W2));
  g.by = l4_floor(l4_unnormalise(g.cy, H2));
}

// Dot products of NPX pixels' feature rows with the image-2 rows of a bounding box (ox, oy, bw x bh), scaled, into
// S[px][row * bw + col]; zero outside the image.
template <int NCH, int NPX>
__device__ __forceinline__ void l4_box_products(const float4 (&f1)[L4_PX][NCH], const float* __restrict__ F2b, int H2,
                                                int W2, int C, int ox, int oy, int bw, int bh, float scale,
                                                float (*S)[L4_BMAX], int px0, int lane) {
  constexpr int QB = 32 / NPX;
  const int nq = bw * bh;
  for (int q0 = 0; q0 < nq; q0 += QB) {
    float v[32];
#pragma unroll
    for (int qi = 0; qi < QB; ++qi) {
      const int q = q0 + qi;
      const int row = q / bw, col = q - row * bw;
      const int x = ox + col, y = oy + row;
      const bool in = q < nq && x >= 0 && x < W2 && y >= 0 && y < H2;
      float4 f2[NCH];
#pragma unroll
      for (int ch = 0; ch < NCH; ++ch) {
        const int c = ch * 128 + lane * 4;
        f2[ch] = (in && c < C) ? __ldg(reinterpret_cast<const float4*>(F2b + ((size_t)y * W2 + x) * C + c))
                               : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int px = 0; px < NPX; ++px) {
        float acc = 0.f;
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) acc = dot4(f1[px][ch], f2[ch], acc);
        v[qi * NPX + px] = acc;
      }
    }
    const float total = warp_transpose_reduce(v, lane);
    const int q = q0 + lane / NPX;
    if (q < nq) S[px0 + lane % NPX][q] = total * scale;
  }
}

// grid (ceil(N1 / 32), levels, B)
template <int NCH>
__global__ void __launch_bounds__(L4_THREADS, 2)
lookup4d_forward_kernel(const float* __restrict__ F1, Lookup4dLevels lv, const float* __restrict__ coords,
                        float* __restrict__ out, int N1, int C, int radius, int levels, float scale) {
  __shared__ float s_S[L4_WARPS][L4_PX][L4_BMAX];
  __shared__ float s_out[L4_WIN * L4_WIN][L4_TILE + 1];
  __shared__ L4Pixel s_geo[L4_WARPS][L4_PX];

  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int level = blockIdx.y, b = blockIdx.z;
  const int H2 = lv.H2[level], W2 = lv.W2[level];
  const float* F2b = lv.f2[level] + (size_t)b * H2 * W2 * C;
  const int p0 = blockIdx.x * L4_TILE + w * L4_PX;
  const int win = 2 * radius + 1;

  // geometry of the warp's pixels and the bounding box of their windows
  int xmin = INT_MAX, xmax = INT_MIN, ymin = INT_MAX, ymax = INT_MIN;
  if (lane < L4_PX && p0 + lane < N1) {
    L4Pixel g;
    l4_pixel_geometry(coords, b, p0 + lane, N1, level, H2, W2, g);
    s_geo[w][lane] = g;
    xmin = xmax = g.bx;
    ymin = ymax = g.by;
  }
#pragma unroll
  for (int off = 1; off < L4_PX; off <<= 1) {
    xmin = min(xmin, __shfl_xor_sync(0xffffffffu, xmin, off));
    xmax = max(xmax, __shfl_xor_sync(0xffffffffu, xmax, off));
    ymin = min(ymin, __shfl_xor_sync(0xffffffffu, ymin, off));
    ymax = max(ymax, __shfl_xor_sync(0xffffffffu, ymax, off));
  }
  xmin = __shfl_sync(0xffffffffu, xmin, 0); xmax = __shfl_sync(0xffffffffu, xmax, 0);
  ymin = __shfl_sync(0xffffffffu, ymin, 0); ymax = __shfl_sync(0xffffffffu, ymax, 0);
  __syncwarp();
  const int npx = min(L4_PX, N1 - p0);   // <= 0: nothing to do for this warp

  if (npx > 0) {
    float4 f1[L4_PX][NCH];
#pragma unroll
    for (int px = 0; px < L4_PX; ++px)
#pragma unroll
      for (int ch = 0; ch < NCH; ++ch) {
        const int c = ch * 128 + lane * 4;
        f1[px][ch] = (px < npx && c < C)
                         ? __ldg(reinterpret_cast<const float4*>(F1 + ((size_t)b * N1 + p0 + px) * C + c))
                         : make_float4(0.f, 0.f, 0.f, 0.f);
      }

    const int bw = xmax - xmin + 2 * radius + 2, bh = ymax - ymin + 2 * radius + 2;
    const bool together = bw <= L4_BW && bh <= L4_BH;
    if (together) {
      l4_box_products<NCH, L4_PX>(f1, F2b, H2, W2, C, xmin - radius, ymin - radius, bw, bh, scale, s_S[w], 0, lane);
    } else {
#pragma unroll
      for (int px = 0; px < L4_PX; ++px) {
        if (px >= npx) break;
        float4 one[L4_PX][NCH];
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) one[0][ch] = f1[px][ch];
        const L4Pixel g = s_geo[w][px];
        l4_box_products<NCH, 1>(one, F2b, H2, W2, C, g.bx - radius, g.by - radius, 2 * radius + 2, 2 * radius + 2,
                                scale, s_S[w], px, lane);
      }
    }
    __syncwarp();

    // bilinear combinations
    for (int idx = lane; idx < npx * win * win; idx += 32) {
      const int px = idx / (win * win), o = idx - px * win * win;
      const int a = o / win, bb = o - a * win;
      const L4Pixel g = s_geo[w][px];
      const int ox = together ? xmin - radius : g.bx - radius;
      const int oy = together ? ymin - radius : g.by - radius;
      const int sbw = together ? bw : 2 * radius + 2;
      const float fx = l4_fraction(g.cx, g.bx, a, radius, W2);
      const float fy = l4_fraction(g.cy, g.by, bb, radius, H2);
      const float* S = s_S[w][px] + (g.by + bb - radius - oy) * sbw + (g.bx + a - radius - ox);
      const float top = S[0] + fx * (S[1] - S[0]);
      const float bot = S[sbw] + fx * (S[sbw + 1] - S[sbw]);
      s_out[o][w * L4_PX + px] = top + fy * (bot - top);
    }
  }
  __syncthreads();
  const int pbase = blockIdx.x * L4_TILE;
  for (int i = threadIdx.x; i < win * win * L4_TILE; i += L4_THREADS) {
    const int o = i / L4_TILE, pp = i % L4_TILE;
    if (pbase + pp < N1)
      out[(((size_t)b * levels + level) * win * win + o) * N1 + pbase + pp] = s_out[o][pp];
  }
}

__device__ __forceinline__ void red_add_v4(float* addr, const float4& v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// One walk of a bounding box in the backward: gS[px][q] (already scaled) is in shared memory.
template <int NCH, int NPX>
__device__ __forceinline__ void l4_box_gradients(const float4 (&f1)[L4_PX][NCH], float4 (&gf1)[L4_PX][NCH],
                                                 const float* __restrict__ F2b, float* __restrict__ G2b, int H2, int W2,
                                                 int C, int ox, int oy, int bw, int bh, float (*gS)[L4_BMAX], int px0,
                                                 int lane) {
  // L4_BWD_STEP positions of a row per step: their image-2 rows are all requested before any is used
  constexpr int J = L4_BWD_STEP;
  for (int row = 0; row < bh; ++row) {
    const int y = oy + row;
    if (y < 0 || y >= H2) continue;
    for (int col = 0; col < bw; col += J) {
      bool in[J];
      float4 f2[J][NCH];
      float g[J][NPX];
      size_t at[J];
#pragma unroll
      for (int j = 0; j < J; ++j) {
        const int x = ox + col + j;
        in[j] = col + j < bw && x >= 0 && x < W2;
        at[j] = ((size_t)y * W2 + (in[j] ? x : 0)) * C;
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          const int c = ch * 128 + lane * 4;
          f2[j][ch] = (in[j] && c < C) ? __ldg(reinterpret_cast<const float4*>(F2b + at[j] + c))
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int j = 0; j < J; ++j) {
        bool any = false;
#pragma unroll
        for (int px = 0; px < NPX; ++px) {
          g[j][px] = in[j] ? gS[px0 + px][row * bw + col + j] : 0.f;
          any |= g[j][px] != 0.f;
        }
        if (!any) continue;   // outside the image, or no pixel of the pass has this position in its window
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          const int c = ch * 128 + lane * 4;
          float4 g2 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int px = 0; px < NPX; ++px) {
            float4& a = gf1[px0 + px][ch];   // a compile-time index once the caller's loop is unrolled
            a.x = fmaf(g[j][px], f2[j][ch].x, a.x); a.y = fmaf(g[j][px], f2[j][ch].y, a.y);
            a.z = fmaf(g[j][px], f2[j][ch].z, a.z); a.w = fmaf(g[j][px], f2[j][ch].w, a.w);
            const float4& s = f1[px0 + px][ch];
            g2.x = fmaf(g[j][px], s.x, g2.x); g2.y = fmaf(g[j][px], s.y, g2.y);
            g2.z = fmaf(g[j][px], s.z, g2.z); g2.w = fmaf(g[j][px], s.w, g2.w);
          }
          if (c < C) red_add_v4(G2b + at[j] + c, g2);
        }
      }
    }
  }
}

// grid (ceil(N1 / 32), 1, B); every CTA walks all levels so that gF1 is stored once.
template <int NCH>
__global__ void __launch_bounds__(L4_THREADS, 2)
lookup4d_backward_kernel(const float* __restrict__ F1, Lookup4dLevels lv, const float* __restrict__ coords,
                         const float* __restrict__ gout, float* __restrict__ gF1, int N1, int C, int radius, int levels,
                         float scale) {
  __shared__ float s_gS[L4_WARPS][L4_PX][L4_BMAX];
  __shared__ float s_g[L4_WIN * L4_WIN][L4_TILE + 1];
  __shared__ L4Pixel s_geo[L4_WARPS][L4_PX];

  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int b = blockIdx.z;
  const int pbase = blockIdx.x * L4_TILE;
  const int p0 = pbase + w * L4_PX;
  const int win = 2 * radius + 1, side = 2 * radius + 2;
  const int npx = min(L4_PX, N1 - p0);

  float4 f1[L4_PX][NCH], gf1[L4_PX][NCH];
#pragma unroll
  for (int px = 0; px < L4_PX; ++px)
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = ch * 128 + lane * 4;
      f1[px][ch] = (px < npx && c < C)
                       ? __ldg(reinterpret_cast<const float4*>(F1 + ((size_t)b * N1 + p0 + px) * C + c))
                       : make_float4(0.f, 0.f, 0.f, 0.f);
      gf1[px][ch] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

  for (int level = 0; level < levels; ++level) {
    const int H2 = lv.H2[level], W2 = lv.W2[level];
    const float* F2b = lv.f2[level] + (size_t)b * H2 * W2 * C;
    float* G2b = lv.g2[level] + (size_t)b * H2 * W2 * C;

    __syncthreads();   // the previous level's s_g is no longer read
    for (int i = threadIdx.x; i < win * win * L4_TILE; i += L4_THREADS) {
      const int o = i / L4_TILE, pp = i % L4_TILE;
      s_g[o][pp] = pbase + pp < N1 ? __ldg(gout + (((size_t)b * levels + level) * win * win + o) * N1 + pbase + pp)
                                   : 0.f;
    }
    int xmin = INT_MAX, xmax = INT_MIN, ymin = INT_MAX, ymax = INT_MIN;
    if (lane < L4_PX && p0 + lane < N1) {
      L4Pixel g;
      l4_pixel_geometry(coords, b, p0 + lane, N1, level, H2, W2, g);
      s_geo[w][lane] = g;
      xmin = xmax = g.bx;
      ymin = ymax = g.by;
    }
#pragma unroll
    for (int off = 1; off < L4_PX; off <<= 1) {
      xmin = min(xmin, __shfl_xor_sync(0xffffffffu, xmin, off));
      xmax = max(xmax, __shfl_xor_sync(0xffffffffu, xmax, off));
      ymin = min(ymin, __shfl_xor_sync(0xffffffffu, ymin, off));
      ymax = max(ymax, __shfl_xor_sync(0xffffffffu, ymax, off));
    }
    xmin = __shfl_sync(0xffffffffu, xmin, 0); xmax = __shfl_sync(0xffffffffu, xmax, 0);
    ymin = __shfl_sync(0xffffffffu, ymin, 0); ymax = __shfl_sync(0xffffffffu, ymax, 0);
    __syncthreads();
    if (npx <= 0) continue;

    const int bw = xmax - xmin + side, bh = ymax - ymin + side;
    const bool together = bw <= L4_BW && bh <= L4_BH;
    const int sbw = together ? bw : side, sbh = together ? bh : side;

    // gradient of the integer positions: position (i, j) of a pixel's (2r+2)^2 grid takes from window entries
    // a in {i-1, i}, b in {j-1, j} with the weight that entry gives it
    for (int idx = lane; idx < npx * sbw * sbh; idx += 32) {
      const int px = idx / (sbw * sbh), q = idx - px * sbw * sbh;
      const int row = q / sbw, col = q - row * sbw;
      const L4Pixel g = s_geo[w][px];
      const int ox = together ? xmin - radius : g.bx - radius;
      const int oy = together ? ymin - radius : g.by - radius;
      const int i = ox + col - (g.bx - radius), j = oy + row - (g.by - radius);
      float acc = 0.f;
      if (i >= 0 && i < side && j >= 0 && j < side) {
#pragma unroll
        for (int da = 0; da < 2; ++da) {
          const int a = i - da;
          if (a < 0 || a >= win) continue;
          const float fx = l4_fraction(g.cx, g.bx, a, radius, W2);
          const float wx = da ? fx : 1.f - fx;
#pragma unroll
          for (int db = 0; db < 2; ++db) {
            const int bb = j - db;
            if (bb < 0 || bb >= win) continue;
            const float fy = l4_fraction(g.cy, g.by, bb, radius, H2);
            const float wy = db ? fy : 1.f - fy;
            acc = fmaf(wx * wy, s_g[a * win + bb][w * L4_PX + px], acc);
          }
        }
      }
      s_gS[w][px][q] = acc * scale;
    }
    __syncwarp();

    if (together) {
      l4_box_gradients<NCH, L4_PX>(f1, gf1, F2b, G2b, H2, W2, C, xmin - radius, ymin - radius, bw, bh, s_gS[w], 0, lane);
    } else {
#pragma unroll
      for (int px = 0; px < L4_PX; ++px) {
        if (px >= npx) break;
        const L4Pixel g = s_geo[w][px];
        l4_box_gradients<NCH, 1>(f1, gf1, F2b, G2b, H2, W2, C, g.bx - radius, g.by - radius, side, side, s_gS[w], px,
                                 lane);
      }
    }
    __syncwarp();
  }

#pragma unroll
  for (int px = 0; px < L4_PX; ++px)
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = ch * 128 + lane * 4;
      if (px < npx && c < C)
        *reinterpret_cast<float4*>(gF1 + ((size_t)b * N1 + p0 + px) * C + c) = gf1[px][ch];
    }
}

static Lookup4dLevels make_levels(const Lookup4dDims& d, const float* const* F2, float* const* gF2) {
  Lookup4dLevels lv{};
  for (int l = 0; l < d.levels; ++l) {
    lv.f2[l] = F2[l];
    lv.g2[l] = gF2 ? gF2[l] : nullptr;
    lv.H2[l] = d.H2[l];
    lv.W2[l] = d.W2[l];
  }
  return lv;
}

cudaError_t launch_lookup4d_forward(const Lookup4dDims& d, const float* F1, const float* const* F2,
                                    const float* coords, float* out, float scale, cudaStream_t stream) {
  const int N1 = d.H1 * d.W1;
  const Lookup4dLevels lv = make_levels(d, F2, nullptr);
  const dim3 grid((N1 + L4_TILE - 1) / L4_TILE, d.levels, d.B);
  switch ((d.C + 127) / 128) {
    case 1: lookup4d_forward_kernel<1><<<grid, L4_THREADS, 0, stream>>>(F1, lv, coords, out, N1, d.C, d.radius, d.levels, scale); break;
    case 2: lookup4d_forward_kernel<2><<<grid, L4_THREADS, 0, stream>>>(F1, lv, coords, out, N1, d.C, d.radius, d.levels, scale); break;
    case 3: lookup4d_forward_kernel<3><<<grid, L4_THREADS, 0, stream>>>(F1, lv, coords, out, N1, d.C, d.radius, d.levels, scale); break;
    case 4: lookup4d_forward_kernel<4><<<grid, L4_THREADS, 0, stream>>>(F1, lv, coords, out, N1, d.C, d.radius, d.levels, scale); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_lookup4d_backward(const Lookup4dDims& d, const float* F1, const float* const* F2,
                                     const float* coords, const float* gout, float* gF1, float* const* gF2,
                                     float scale, cudaStream_t stream) {
  const int N1 = d.H1 * d.W1;
  for (int l = 0; l < d.levels; ++l) {
    const cudaError_t err =
        cudaMemsetAsync(gF2[l], 0, (size_t)d.B * d.H2[l] * d.W2[l] * d.C * sizeof(float), stream);
    if (err != cudaSuccess) return err;
  }
  const Lookup4dLevels lv = make_levels(d, F2, gF2);
  const dim3 grid((N1 + L4_TILE - 1) / L4_TILE, 1, d.B);
  switch ((d.C + 127) / 128) {
    case 1: lookup4d_backward_kernel<1><<<grid, L4_THREADS, 0, stream>>>(F1, lv, coords, gout, gF1, N1, d.C, d.radius, d.levels, scale); break;
    case 2: lookup4d_backward_kernel<2><<<grid, L4_THREADS, 0, stream>>>(F1, lv, coords, gout, gF1, N1, d.C, d.radius, d.levels, scale); break;
    case 3: lookup4d_backward_kernel<3><<<grid, L4_THREADS, 0, stream>>>(F1, lv, coords, gout, gF1, N1, d.C, d.radius, d.levels, scale); break;
    case 4: lookup4d_backward_kernel<4><<<grid, L4_THREADS, 0, stream>>>(F1, lv, coords, gout, gF1, N1, d.C, d.radius, d.levels, scale); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace sfb
