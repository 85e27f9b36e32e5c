// Attention weights of the separation (HBM-bound stencil kernels, no tensor cores):
//   A = softmax_over_d( Conv3d(2 -> Kc, 3x3x3, padding 1)(X) )       core/corr.py:437-442, core/sepflow.py:59-60
// on the channels-first tensors X (B, 2, D, H1, W1) -> A (B, Kc, D, H1, W1), and its backward.
//
// Every kernel gives one thread one image-1 pixel (h, w) and lets it walk the displacement axis d, so that a
// warp reads 32 neighbouring pixels of a (channel, d) plane per load and the softmax over d stays inside the
// thread.  The 3x3x3 stencil is applied in "scatter" form: the 3x3 neighbourhood of the plane that was just
// loaded is added into the three outputs (d-1, d, d+1) it belongs to, which are kept in registers; nothing but
// the current plane's neighbourhood is live, and a plane is read from L1/L2 once per thread.
//   forward     : logits -> A (raw logits are parked in A, then normalised in a second walk by the same thread)
//   logit grads : gL = A * (gA - sum_d gA*A), in place over gA; per-block sums of gL for the bias gradient
//   input grads : gX = transposed stencil of gL (+ an optional addend: the direct gradient of the max/avg channels)
//   weight grads: gW[k,c,tap] = sum X(shifted by tap) * gL, per-block partial sums, reduced in a fixed order by
//                 a second kernel (bit-reproducible; no floating-point atomics)
#include "kernels.h"

namespace sfb {

constexpr int AT_THREADS = 128;
constexpr int AT_TAPS = 27;

// Offsets of the 3x3 neighbourhood of pixel (h, w) inside a plane, and which of them exist.
struct Neighbourhood {
  int off[9];
  unsigned valid;  // bit (3*th + tw)
  __device__ Neighbourhood(int h, int w, int H1, int W1) {
    valid = 0;
#pragma unroll
    for (int th = 0; th < 3; ++th)
#pragma unroll
      for (int tw = 0; tw < 3; ++tw) {
        const int hh = h + th - 1, ww = w + tw - 1;
        off[3 * th + tw] = (th - 1) * W1 + (tw - 1);
        if (hh >= 0 && hh < H1 && ww >= 0 && ww < W1) valid |= 1u << (3 * th + tw);
      }
  }
  __device__ float load(const float* plane_at_pixel, int nb) const {
    return ((valid >> nb) & 1u) ? __ldg(plane_at_pixel + off[nb]) : 0.f;
  }
};

// ---- forward ------------------------------------------------------------------------------------------
// grid (ceil(N1/128), B), block 128.  Channels k0 .. k0+KC-1 of Kc.
template <int KC>
__global__ void __launch_bounds__(AT_THREADS)
attention_forward_kernel(const float* __restrict__ x, long long x_sb, const float* __restrict__ weight,
                         const float* __restrict__ bias, float* __restrict__ a, int Kc, int k0, int D, int H1,
                         int W1) {
  __shared__ float ws[2 * AT_TAPS][4];  // [c*27 + tap][k]
  const int N1 = H1 * W1;
  for (int i = threadIdx.x; i < 2 * AT_TAPS * 4; i += AT_THREADS) {
    const int k = i & 3, ct = i >> 2;
    ws[ct][k] = k < KC ? __ldg(weight + (size_t)(k0 + k) * 2 * AT_TAPS + ct) : 0.f;
  }
  __syncthreads();
  const int p = blockIdx.x * AT_THREADS + threadIdx.x, b = blockIdx.y;
  if (p >= N1) return;
  const int h = p / W1, w = p - h * W1;
  const Neighbourhood nb(h, w, H1, W1);
  const size_t plane = (size_t)N1;
  const float* x0 = x + (size_t)b * x_sb + p;       // channel 0, plane 0
  const float* x1 = x0 + (size_t)D * plane;         // channel 1
  float* out = a + ((size_t)b * Kc + k0) * D * plane + p;

  float bk[KC], acc[3][KC], m[KC], l[KC];
#pragma unroll
  for (int k = 0; k < KC; ++k) {
    bk[k] = __ldg(bias + k0 + k);
    acc[0][k] = acc[1][k] = acc[2][k] = bk[k];
    m[k] = -INFINITY;
    l[k] = 0.f;
  }
  auto emit = [&](int d) {  // logit d is complete in acc[0]
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const float L = acc[0][k];
      out[((size_t)k * D + d) * plane] = L;
      if (L > m[k]) { l[k] = l[k] * __expf(m[k] - L) + 1.f; m[k] = L; }
      else l[k] += __expf(L - m[k]);
    }
  };
  for (int e = 0; e < D; ++e) {  // plane e feeds logits e+1 (tap td=0), e (td=1), e-1 (td=2)
    float xv[2][9];
#pragma unroll
    for (int n = 0; n < 9; ++n) { xv[0][n] = nb.load(x0, n); xv[1][n] = nb.load(x1, n); }
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int n = 0; n < 9; ++n) {
        const float4 w0 = *reinterpret_cast<const float4*>(ws[c * AT_TAPS + n]);
        const float4 w1 = *reinterpret_cast<const float4*>(ws[c * AT_TAPS + 9 + n]);
        const float4 w2 = *reinterpret_cast<const float4*>(ws[c * AT_TAPS + 18 + n]);
        const float wk0[4] = {w0.x, w0.y, w0.z, w0.w}, wk1[4] = {w1.x, w1.y, w1.z, w1.w}, wk2[4] = {w2.x, w2.y, w2.z, w2.w};
#pragma unroll
        for (int k = 0; k < KC; ++k) {
          acc[2][k] = fmaf(xv[c][n], wk0[k], acc[2][k]);
          acc[1][k] = fmaf(xv[c][n], wk1[k], acc[1][k]);
          acc[0][k] = fmaf(xv[c][n], wk2[k], acc[0][k]);
        }
      }
    if (e >= 1) emit(e - 1);
#pragma unroll
    for (int k = 0; k < KC; ++k) { acc[0][k] = acc[1][k]; acc[1][k] = acc[2][k]; acc[2][k] = bk[k]; }
    x0 += plane;
    x1 += plane;
  }
  emit(D - 1);
  float inv[KC];
#pragma unroll
  for (int k = 0; k < KC; ++k) inv[k] = 1.f / l[k];
  for (int d = 0; d < D; ++d) {  // the thread re-reads its own stores
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      float* q = out + ((size_t)k * D + d) * plane;
      *q = __expf(*q - m[k]) * inv[k];
    }
  }
}

// ---- sums over a block, written to partial[row][col0 + i] ---------------------------------------------
template <int N>
__device__ void block_sums_to(float (&v)[N], float* smem /* [AT_THREADS/32][N] */, float* dst) {
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float s = v[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    v[i] = s;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) smem[warp * N + i] = v[i];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < N; i += AT_THREADS) {
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < AT_THREADS / 32; ++wv) s += smem[wv * N + i];
    dst[i] = s;
  }
}

// ---- logit gradients (softmax backward), in place -------------------------------------------------------
// grid (ceil(N1/128), B), block 128.  bias_partial: (B * gridDim.x, Kc).
template <int KC>
__global__ void __launch_bounds__(AT_THREADS)
attention_logit_grad_kernel(const float* __restrict__ a, float* __restrict__ g, float* __restrict__ bias_partial,
                            int Kc, int k0, int D, int N1) {
  __shared__ float red[(AT_THREADS / 32) * KC];
  const int p = blockIdx.x * AT_THREADS + threadIdx.x, b = blockIdx.y;
  const size_t plane = (size_t)N1;
  float bsum[KC];
#pragma unroll
  for (int k = 0; k < KC; ++k) bsum[k] = 0.f;
  if (p < N1) {
    const size_t base = ((size_t)b * Kc + k0) * D * plane + p;
    float s[KC];
#pragma unroll
    for (int k = 0; k < KC; ++k) s[k] = 0.f;
    for (int d = 0; d < D; ++d)
#pragma unroll
      for (int k = 0; k < KC; ++k) {
        const size_t i = base + ((size_t)k * D + d) * plane;
        s[k] = fmaf(g[i], __ldg(a + i), s[k]);
      }
    for (int d = 0; d < D; ++d)
#pragma unroll
      for (int k = 0; k < KC; ++k) {
        const size_t i = base + ((size_t)k * D + d) * plane;
        const float gl = __ldg(a + i) * (g[i] - s[k]);
        g[i] = gl;
        bsum[k] += gl;
      }
  }
  block_sums_to<KC>(bsum, red, bias_partial + ((size_t)b * gridDim.x + blockIdx.x) * Kc + k0);
}

// ---- input gradients -----------------------------------------------------------------------------------
// gX[c, d, h, w] = add[c, d, h, w] + sum_{k, td, th, tw} W[k, c, td, th, tw] * gL[k, d - td + 1, h - th + 1, w - tw + 1]
// grid (ceil(N1/128), B), block 128, dynamic shared memory Kc * 9 * 8 floats.
template <int KC>  // KC > 0: Kc == KC, unrolled; KC == 0: any Kc
__global__ void __launch_bounds__(AT_THREADS)
attention_input_grad_kernel(const float* __restrict__ gl, const float* __restrict__ weight,
                            const float* __restrict__ add, long long add_sb, float* __restrict__ gx, int Kc, int D,
                            int H1, int W1) {
  extern __shared__ float4 wt[];  // [k][neighbour][2] : (c0td0, c0td1, c0td2, c1td0), (c1td1, c1td2, -, -)
  const int N1 = H1 * W1;
  float* wts = reinterpret_cast<float*>(wt);
  for (int i = threadIdx.x; i < Kc * 9 * 8; i += AT_THREADS) {
    const int j = i & 7, n = (i >> 3) % 9, k = i / 72;
    // neighbour n = (nh, nw) holds gL at (h + nh - 1, w + nw - 1), which meets tap th = 2 - nh, tw = 2 - nw
    const int th = 2 - n / 3, tw = 2 - n % 3, c = j / 3, td = j % 3;
    wts[i] = j < 6 ? __ldg(weight + ((size_t)(k * 2 + c) * 3 + td) * 9 + th * 3 + tw) : 0.f;
  }
  __syncthreads();
  const int p = blockIdx.x * AT_THREADS + threadIdx.x, b = blockIdx.y;
  if (p >= N1) return;
  const int h = p / W1, w = p - h * W1;
  const Neighbourhood nb(h, w, H1, W1);
  const size_t plane = (size_t)N1;
  const float* g0 = gl + (size_t)b * Kc * D * plane + p;
  float* o0 = gx + (size_t)b * 2 * D * plane + p;
  const float* ad = add != nullptr ? add + (size_t)b * add_sb + p : nullptr;
  float acc[2][3];  // [c][output d = e-1, e, e+1]
#pragma unroll
  for (int c = 0; c < 2; ++c) acc[c][0] = acc[c][1] = acc[c][2] = 0.f;
  auto emit = [&](int d) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const size_t i = ((size_t)c * D + d) * plane;
      o0[i] = acc[c][0] + (ad != nullptr ? __ldg(ad + i) : 0.f);
    }
  };
  const int kn = KC > 0 ? KC : Kc;
  for (int e = 0; e < D; ++e) {  // plane e of gL feeds gX planes e-1 (td=0), e (td=1), e+1 (td=2)
#pragma unroll
    for (int k = 0; k < kn; ++k) {
      const float* gk = g0 + ((size_t)k * D + e) * plane;
#pragma unroll
      for (int n = 0; n < 9; ++n) {
        const float v = nb.load(gk, n);
        const float4 wa = wt[(k * 9 + n) * 2], wb = wt[(k * 9 + n) * 2 + 1];
        acc[0][0] = fmaf(v, wa.x, acc[0][0]);
        acc[0][1] = fmaf(v, wa.y, acc[0][1]);
        acc[0][2] = fmaf(v, wa.z, acc[0][2]);
        acc[1][0] = fmaf(v, wa.w, acc[1][0]);
        acc[1][1] = fmaf(v, wb.x, acc[1][1]);
        acc[1][2] = fmaf(v, wb.y, acc[1][2]);
      }
    }
    if (e >= 1) emit(e - 1);
#pragma unroll
    for (int c = 0; c < 2; ++c) { acc[c][0] = acc[c][1]; acc[c][1] = acc[c][2]; acc[c][2] = 0.f; }
  }
  emit(D - 1);
}

// ---- weight gradients ----------------------------------------------------------------------------------
// gW[k, c, td, th, tw] = sum_{b, d, h, w} gL[k, d, h, w] * X[c, d + td - 1, h + th - 1, w + tw - 1]
// grid (ceil(N1/128), B, Kc), block 128.  partial: (B * gridDim.x, Kc, 54).
__global__ void __launch_bounds__(AT_THREADS)
attention_weight_grad_kernel(const float* __restrict__ x, long long x_sb, const float* __restrict__ gl,
                             float* __restrict__ partial, int Kc, int D, int H1, int W1) {
  __shared__ float red[(AT_THREADS / 32) * 2 * AT_TAPS];
  const int N1 = H1 * W1;
  const int p = blockIdx.x * AT_THREADS + threadIdx.x, b = blockIdx.y, k = blockIdx.z;
  float acc[2 * AT_TAPS];  // [c][td][neighbour]
#pragma unroll
  for (int i = 0; i < 2 * AT_TAPS; ++i) acc[i] = 0.f;
  if (p < N1) {
    const int h = p / W1, w = p - h * W1;
    const Neighbourhood nb(h, w, H1, W1);
    const size_t plane = (size_t)N1;
    const float* x0 = x + (size_t)b * x_sb + p;
    const float* x1 = x0 + (size_t)D * plane;
    const float* g = gl + ((size_t)b * Kc + k) * D * plane + p;
    float g_prev = 0.f, g_cur = __ldg(g), g_next;
    for (int e = 0; e < D; ++e) {  // plane e of X meets gL at d = e+1 (td=0), e (td=1), e-1 (td=2)
      g_next = e + 1 < D ? __ldg(g + (size_t)(e + 1) * plane) : 0.f;
#pragma unroll
      for (int n = 0; n < 9; ++n) {
        const float v0 = nb.load(x0, n), v1 = nb.load(x1, n);
        acc[n] = fmaf(g_next, v0, acc[n]);
        acc[9 + n] = fmaf(g_cur, v0, acc[9 + n]);
        acc[18 + n] = fmaf(g_prev, v0, acc[18 + n]);
        acc[AT_TAPS + n] = fmaf(g_next, v1, acc[AT_TAPS + n]);
        acc[AT_TAPS + 9 + n] = fmaf(g_cur, v1, acc[AT_TAPS + 9 + n]);
        acc[AT_TAPS + 18 + n] = fmaf(g_prev, v1, acc[AT_TAPS + 18 + n]);
      }
      g_prev = g_cur;
      g_cur = g_next;
      x0 += plane;
      x1 += plane;
    }
  }
  block_sums_to<2 * AT_TAPS>(acc, red, partial + (((size_t)b * gridDim.x + blockIdx.x) * Kc + k) * 2 * AT_TAPS);
}

// out[i] = sum over rows of partial[row][i], rows added in order.  One thread per column.
__global__ void attention_reduce_partials_kernel(const float* __restrict__ partial, int rows, int cols,
                                                 float* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= cols) return;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int r = 0;
  for (; r + 4 <= rows; r += 4) {
    s0 += __ldg(partial + (size_t)r * cols + i);
    s1 += __ldg(partial + (size_t)(r + 1) * cols + i);
    s2 += __ldg(partial + (size_t)(r + 2) * cols + i);
    s3 += __ldg(partial + (size_t)(r + 3) * cols + i);
  }
  for (; r < rows; ++r) s0 += __ldg(partial + (size_t)r * cols + i);
  out[i] = (s0 + s1) + (s2 + s3);
}

// ---- launchers ---------------------------------------------------------------------------------------
static dim3 pixel_grid(const AttentionDims& d) { return dim3((d.H1 * d.W1 + AT_THREADS - 1) / AT_THREADS, d.B); }

size_t attention_partial_floats(const AttentionDims& d) {
  const size_t rows = (size_t)pixel_grid(d).x * d.B;
  return rows * d.Kc * (2 * AT_TAPS + 1);
}

cudaError_t launch_attention_forward(const AttentionDims& d, const float* x, long long x_sb, const float* weight,
                                     const float* bias, float* a, cudaStream_t st) {
  const dim3 grid = pixel_grid(d);
  for (int k0 = 0; k0 < d.Kc; k0 += 4) {
    const int kc = d.Kc - k0 < 4 ? d.Kc - k0 : 4;
#define SFB_AT_FWD(KC) attention_forward_kernel<KC><<<grid, AT_THREADS, 0, st>>>(x, x_sb, weight, bias, a, d.Kc, k0, d.D, d.H1, d.W1)
    if (kc == 1) SFB_AT_FWD(1); else if (kc == 2) SFB_AT_FWD(2); else if (kc == 3) SFB_AT_FWD(3); else SFB_AT_FWD(4);
#undef SFB_AT_FWD
  }
  return cudaGetLastError();
}

cudaError_t launch_attention_backward(const AttentionDims& d, const float* x, long long x_sb, const float* weight,
                                      const float* a, float* g, const float* add, long long add_sb, float* gx,
                                      float* gweight, float* gbias, float* partial, cudaStream_t st) {
  const dim3 grid = pixel_grid(d);
  const int rows = (int)(grid.x * grid.y), N1 = d.H1 * d.W1;
  float* bias_partial = partial;                                   // (rows, Kc)
  float* weight_partial = partial + (size_t)rows * d.Kc;           // (rows, Kc, 54)
  for (int k0 = 0; k0 < d.Kc; k0 += 4) {
    const int kc = d.Kc - k0 < 4 ? d.Kc - k0 : 4;
#define SFB_AT_LG(KC) attention_logit_grad_kernel<KC><<<grid, AT_THREADS, 0, st>>>(a, g, bias_partial, d.Kc, k0, d.D, N1)
    if (kc == 1) SFB_AT_LG(1); else if (kc == 2) SFB_AT_LG(2); else if (kc == 3) SFB_AT_LG(3); else SFB_AT_LG(4);
#undef SFB_AT_LG
  }
  const size_t smem = (size_t)d.Kc * 9 * 8 * sizeof(float);
#define SFB_AT_IG(KC) attention_input_grad_kernel<KC><<<grid, AT_THREADS, smem, st>>>(g, weight, add, add_sb, gx, d.Kc, d.D, d.H1, d.W1)
  if (d.Kc == 1) SFB_AT_IG(1); else if (d.Kc == 2) SFB_AT_IG(2); else if (d.Kc == 3) SFB_AT_IG(3);
  else if (d.Kc == 4) SFB_AT_IG(4); else SFB_AT_IG(0);
#undef SFB_AT_IG
  attention_weight_grad_kernel<<<dim3(grid.x, grid.y, d.Kc), AT_THREADS, 0, st>>>(x, x_sb, g, weight_partial, d.Kc,
                                                                                   d.D, d.H1, d.W1);
  const int wcols = d.Kc * 2 * AT_TAPS;
  attention_reduce_partials_kernel<<<(wcols + 63) / 64, 64, 0, st>>>(weight_partial, rows, wcols, gweight);
  attention_reduce_partials_kernel<<<(d.Kc + 63) / 64, 64, 0, st>>>(bias_partial, rows, d.Kc, gbias);
  return cudaGetLastError();
}

}  // namespace sfb
