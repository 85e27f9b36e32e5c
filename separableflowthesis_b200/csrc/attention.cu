// Attention weights of the separation (stencil kernels on the FP32 pipes, no tensor cores):
//   A = softmax_over_d( Conv3d(2 -> Kc, 3x3x3, padding 1)(X) )       core/corr.py:437-442, core/sepflow.py:59-60
// on the channels-first tensors X (B, 2, D, H1, W1) -> A (B, Kc, D, H1, W1), and its backward.
//
// Every kernel gives one thread one image-1 pixel (h, w) and lets it walk the displacement axis d, so that a
// warp reads 32 neighbouring pixels of a (channel, d) plane per load and the softmax over d stays inside the
// thread.  The 3x3x3 stencil is applied in "scatter" form: the 3x3 neighbourhood of the plane that was just
// loaded is added into the three outputs (d-1, d, d+1) it belongs to, which are kept in registers.
//
// Two things decide the speed of such a walk, and both are handled explicitly:
//  * latency: a thread needs plane e+1 only after it is done with plane e, so on its own it has one plane of
//    loads in flight.  Each thread therefore prefetches its neighbourhoods a few planes ahead with cp.async into
//    a ring of shared-memory slots that only it reads (no block barrier), see PlaneRing.
//  * operand bandwidth: all threads multiply by the same 54*Kc filter weights.  Reading them from shared memory
//    costs a 32-lane register write per weight, more than the FMA they feed; instead the weights of the (up to
//    four) channels being processed are staged in __constant__ memory, where an FMA reads them as an operand.
//
//   forward     : logits -> A (raw logits are parked in A, then normalised in a second walk by the same thread)
//   logit grads : gL = A * (gA - sum_d gA*A), in place over gA; per-block sums of gL for the bias gradient
//   input grads : gX = transposed stencil of gL (+ an optional addend: the direct gradient of the max/avg channels)
//   weight grads: gW[k,c,tap] = sum X(shifted by tap) * gL, per-block partial sums, reduced in a fixed order by
//                 a second kernel (bit-reproducible; no floating-point atomics)
#include <mutex>

#include "kernels.h"
#include "sm100_primitives.cuh"

namespace sfb {

constexpr int AT_THREADS = 128;
constexpr int AT_TAPS = 27;
constexpr int AT_KC = 4;  // channels per launch of the forward / logit-gradient kernels and per constant-memory stage

// Filter weights (k, c, td, th, tw) of the channels the running kernel works on.
__constant__ float c_att_weights[AT_KC * 2 * AT_TAPS];

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
  __device__ bool has(int nb) const { return (valid >> nb) & 1u; }
};

// ---- per-thread prefetch ring -------------------------------------------------------------------------
// ring[stage][value][thread]: a thread copies the NV values it will need for plane e into stage e % STAGES with
// 4-byte cp.async (zero fill for values that do not exist) and reads them back itself STAGES-1 planes later.
__device__ __forceinline__ void cp_async4(float* smem_dst, const float* src, bool valid) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int bytes = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int NV, int STAGES>
struct PlaneRing {
  float* base;  // this thread's column: value v of stage s at base[(s * NV + v) * AT_THREADS]
  __device__ PlaneRing(float* smem) : base(smem + threadIdx.x) {}
  __device__ float* slot(int stage, int v) const { return base + (stage * NV + v) * AT_THREADS; }
  static constexpr size_t bytes() { return (size_t)STAGES * NV * AT_THREADS * sizeof(float); }
};

// ---- forward ------------------------------------------------------------------------------------------
// grid (ceil(N1/128), B), block 128.  Channels k0 .. k0+KC-1 of Kc, whose weights are in c_att_weights.
constexpr int FW_STAGES = 4;

template <int KC>
__global__ void __launch_bounds__(AT_THREADS)
attention_forward_kernel(const float* __restrict__ x, long long x_sb, const float* __restrict__ bias,
                         float* __restrict__ a, int Kc, int k0, int D, int H1, int W1) {
  __shared__ float ring_mem[FW_STAGES * 18 * AT_THREADS];
  const int N1 = H1 * W1;
  const int p = blockIdx.x * AT_THREADS + threadIdx.x, b = blockIdx.y;
  if (p >= N1) return;
  const int h = p / W1, w = p - h * W1;
  const Neighbourhood nb(h, w, H1, W1);
  const PlaneRing<18, FW_STAGES> ring(ring_mem);
  const size_t plane = (size_t)N1;
  const float* x0 = x + (size_t)b * x_sb + p;       // channel 0, plane 0
  const float* x1 = x0 + (size_t)D * plane;         // channel 1
  float* out = a + ((size_t)b * Kc + k0) * D * plane + p;

  auto issue = [&](int e) {  // neighbourhoods of plane e (both channels) -> stage e % FW_STAGES
    if (e < D) {
      const int s = e % FW_STAGES;
      const float* q0 = x0 + (size_t)e * plane;
      const float* q1 = x1 + (size_t)e * plane;
#pragma unroll
      for (int n = 0; n < 9; ++n) {
        cp_async4(ring.slot(s, n), nb.has(n) ? q0 + nb.off[n] : q0, nb.has(n));
        cp_async4(ring.slot(s, 9 + n), nb.has(n) ? q1 + nb.off[n] : q1, nb.has(n));
      }
    }
    cp_async_commit();
  };

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
#pragma unroll
  for (int s = 0; s < FW_STAGES - 1; ++s) issue(s);
  for (int e = 0; e < D; ++e) {  // plane e feeds logits e+1 (tap td=0), e (td=1), e-1 (td=2)
    issue(e + FW_STAGES - 1);
    cp_async_wait<FW_STAGES - 1>();
    const int s = e % FW_STAGES;
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int n = 0; n < 9; ++n) {
        const float xv = *ring.slot(s, c * 9 + n);
#pragma unroll
        for (int k = 0; k < KC; ++k) {
          acc[2][k] = fmaf(xv, c_att_weights[(k * 2 + c) * AT_TAPS + n], acc[2][k]);
          acc[1][k] = fmaf(xv, c_att_weights[(k * 2 + c) * AT_TAPS + 9 + n], acc[1][k]);
          acc[0][k] = fmaf(xv, c_att_weights[(k * 2 + c) * AT_TAPS + 18 + n], acc[0][k]);
        }
      }
    if (e >= 1) emit(e - 1);
#pragma unroll
    for (int k = 0; k < KC; ++k) { acc[0][k] = acc[1][k]; acc[1][k] = acc[2][k]; acc[2][k] = bk[k]; }
  }
  emit(D - 1);
#pragma unroll
  for (int k = 0; k < KC; ++k) l[k] = 1.f / l[k];
  // the thread re-reads its own stores, four displacements at a time so that the loads overlap
  constexpr int DB = 4;
  for (int d0 = 0; d0 < D; d0 += DB) {
    float v[DB][KC];
#pragma unroll
    for (int i = 0; i < DB; ++i)
#pragma unroll
      for (int k = 0; k < KC; ++k) v[i][k] = d0 + i < D ? out[((size_t)k * D + d0 + i) * plane] : 0.f;
#pragma unroll
    for (int i = 0; i < DB; ++i)
#pragma unroll
      for (int k = 0; k < KC; ++k)
        if (d0 + i < D) out[((size_t)k * D + d0 + i) * plane] = __expf(v[i][k] - m[k]) * l[k];
  }
}

// ---- forward, pixel tiles fetched by TMA -----------------------------------------------------------------
// A block owns a tile of AT_TW x AT_TH image-1 pixels.  A producer warp fetches, plane by plane, the tile of both
// input channels with its one-pixel halo as ONE tiled TMA load into a ring of stages (the box starts 4 pixels to the
// left so that its x coordinate is a multiple of 16 bytes; pixels outside the image arrive as zeros, which is the
// convolution's zero padding), and the 128 pixel threads read their 18 neighbours from shared memory at constant
// offsets.  Against the gather above this removes the 18 per-thread copies per plane and their address arithmetic,
// which were a third of the instructions of an issue-bound kernel.  Needs W1 % 4 == 0 (TMA strides are multiples of
// 16 bytes).  grid (ceil(W1/32), ceil(H1/4), B), block 128 + 32.
constexpr int AT_TW = 32, AT_TH = 4;
constexpr int AT_BOX_W = AT_TW + 8, AT_BOX_H = AT_TH + 2;
constexpr int AT_TSTAGES = 6;

// A TMA destination in shared memory must be 128-byte aligned; one channel's tile is 960 bytes, so every stage is
// padded to a multiple of 128.
constexpr uint32_t AT_TILE_BYTES = AT_BOX_H * AT_BOX_W * sizeof(float);
template <int NCH>
struct alignas(128) AttentionTileStage {
  float v[NCH][AT_BOX_H][AT_BOX_W];
};
template <int NCH>
struct AttentionTileSmem {
  AttentionTileStage<NCH> x[AT_TSTAGES];
  uint64_t full[AT_TSTAGES];
  uint64_t empty[AT_TSTAGES];
  WaitCtl ctl;
};

template <int KC>
__global__ void __launch_bounds__(AT_THREADS + 32)
attention_forward_tiled_kernel(const __grid_constant__ CUtensorMap tm_x, const float* __restrict__ bias,
                               float* __restrict__ a, int Kc, int k0, int D, int H1, int W1, int* status) {
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  __shared__ __align__(128) AttentionTileSmem<2> sm;
  const int w0 = blockIdx.x * AT_TW, h0 = blockIdx.y * AT_TH, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < AT_TSTAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], AT_THREADS / 32); }
    wait_ctl_init(&sm.ctl, 0);
    fence_barrier_init();
    prefetch_tensormap(&tm_x);
  }
  __syncthreads();
  if (warp == AT_THREADS / 32) {  // producer
    if (lane == 0) {
      for (int e = 0; e < D; ++e) {
        const uint32_t s = e % AT_TSTAGES, ph = (e / AT_TSTAGES) & 1u;
        if (!mbar_wait(&sm.empty[s], ph ^ 1u, &sm.ctl, status, DEV_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&sm.full[s], 2 * AT_TILE_BYTES);
        tma_load_5d(sm.x[s].v, &tm_x, &sm.full[s], w0 - 4, h0 - 1, e, 0, b);
      }
    }
    return;
  }
  const int tx = lane, ty = warp;
  const int h = h0 + ty, w = w0 + tx;
  const bool valid = h < H1 && w < W1;
  const size_t plane = (size_t)H1 * W1;
  float* out = a + ((size_t)b * Kc + k0) * D * plane + (size_t)(valid ? h * W1 + w : 0);

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
      if (valid) out[((size_t)k * D + d) * plane] = L;
      if (L > m[k]) { l[k] = l[k] * __expf(m[k] - L) + 1.f; m[k] = L; }
      else l[k] += __expf(L - m[k]);
    }
  };
  for (int e = 0; e < D; ++e) {  // plane e feeds logits e+1 (tap td=0), e (td=1), e-1 (td=2)
    const uint32_t s = e % AT_TSTAGES, ph = (e / AT_TSTAGES) & 1u;
    const bool ok = mbar_wait(&sm.full[s], ph, &sm.ctl, status, DEV_TIMEOUT_EPILOGUE);
    if (!__all_sync(0xffffffffu, ok)) return;
    float xv[2][9];
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int n = 0; n < 9; ++n) xv[c][n] = sm.x[s].v[c][ty + n / 3][tx + 3 + n % 3];
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.empty[s]);  // the neighbourhoods are in registers
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int n = 0; n < 9; ++n) {
#pragma unroll
        for (int k = 0; k < KC; ++k) {
          acc[2][k] = fmaf(xv[c][n], c_att_weights[(k * 2 + c) * AT_TAPS + n], acc[2][k]);
          acc[1][k] = fmaf(xv[c][n], c_att_weights[(k * 2 + c) * AT_TAPS + 9 + n], acc[1][k]);
          acc[0][k] = fmaf(xv[c][n], c_att_weights[(k * 2 + c) * AT_TAPS + 18 + n], acc[0][k]);
        }
      }
    if (e >= 1) emit(e - 1);
#pragma unroll
    for (int k = 0; k < KC; ++k) { acc[0][k] = acc[1][k]; acc[1][k] = acc[2][k]; acc[2][k] = bk[k]; }
  }
  emit(D - 1);
  if (!valid) return;
#pragma unroll
  for (int k = 0; k < KC; ++k) l[k] = 1.f / l[k];
  // the thread re-reads its own stores, four displacements at a time so that the loads overlap
  constexpr int DB = 4;
  for (int d0 = 0; d0 < D; d0 += DB) {
    float v[DB][KC];
#pragma unroll
    for (int i = 0; i < DB; ++i)
#pragma unroll
      for (int k = 0; k < KC; ++k) v[i][k] = d0 + i < D ? out[((size_t)k * D + d0 + i) * plane] : 0.f;
#pragma unroll
    for (int i = 0; i < DB; ++i)
#pragma unroll
      for (int k = 0; k < KC; ++k)
        if (d0 + i < D) out[((size_t)k * D + d0 + i) * plane] = __expf(v[i][k] - m[k]) * l[k];
  }
}

// Tensor map over a channels-first tensor (B, nch, D, H1, W1) whose samples are `sb` elements apart; the box is one
// plane's pixel tile of `box_ch` channels, with the stencil's halo or without.
static cudaError_t tile_map(CUtensorMap* tm, const float* x, long long sb, int nch, int box_ch, const AttentionDims& d,
                            bool halo) {
  const uint64_t N1 = (uint64_t)d.H1 * d.W1;
  const uint64_t dims[5] = {(uint64_t)d.W1, (uint64_t)d.H1, (uint64_t)d.D, (uint64_t)nch, (uint64_t)d.B};
  const uint64_t strides[4] = {(uint64_t)d.W1 * 4, N1 * 4, (uint64_t)d.D * N1 * 4, (uint64_t)sb * 4};
  const uint32_t box[5] = {(uint32_t)(halo ? AT_BOX_W : AT_TW), (uint32_t)(halo ? AT_BOX_H : AT_TH), 1, (uint32_t)box_ch, 1};
  return encode_plain_map(tm, x, 5, dims, strides, box);
}
static bool tileable(const AttentionDims& d, const void* x, long long sb) {
  return d.W1 % 4 == 0 && sb % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
}

// ---- sums over a block, written to dst[i] -------------------------------------------------------------
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
    constexpr int DB = 4;  // displacements per batch: all loads of a batch are issued before they are used
    for (int d0 = 0; d0 < D; d0 += DB) {
      float gv[DB][KC], av[DB][KC];
#pragma unroll
      for (int i = 0; i < DB; ++i)
#pragma unroll
        for (int k = 0; k < KC; ++k) {
          const size_t idx = base + ((size_t)k * D + d0 + i) * plane;
          gv[i][k] = d0 + i < D ? g[idx] : 0.f;
          av[i][k] = d0 + i < D ? __ldg(a + idx) : 0.f;
        }
#pragma unroll
      for (int i = 0; i < DB; ++i)
#pragma unroll
        for (int k = 0; k < KC; ++k) s[k] = fmaf(gv[i][k], av[i][k], s[k]);
    }
    for (int d0 = 0; d0 < D; d0 += DB) {
      float gv[DB][KC], av[DB][KC];
#pragma unroll
      for (int i = 0; i < DB; ++i)
#pragma unroll
        for (int k = 0; k < KC; ++k) {
          const size_t idx = base + ((size_t)k * D + d0 + i) * plane;
          gv[i][k] = d0 + i < D ? g[idx] : 0.f;
          av[i][k] = d0 + i < D ? __ldg(a + idx) : 0.f;
        }
#pragma unroll
      for (int i = 0; i < DB; ++i)
#pragma unroll
        for (int k = 0; k < KC; ++k) {
          const float gl = av[i][k] * (gv[i][k] - s[k]);
          if (d0 + i < D) g[base + ((size_t)k * D + d0 + i) * plane] = gl;
          bsum[k] += gl;
        }
    }
  }
  block_sums_to<KC>(bsum, red, bias_partial + ((size_t)b * gridDim.x + blockIdx.x) * Kc + k0);
}

// ---- input gradients -----------------------------------------------------------------------------------
// gX[c, d, h, w] = add[c, d, h, w] + sum_{k, td, th, tw} W[k, c, td, th, tw] * gL[k, d - td + 1, h - th + 1, w - tw + 1]
// Channels k0 .. k0+KC-1 (weights in c_att_weights); a later chunk adds to what the earlier ones stored.
// grid (ceil(N1/128), B), block 128, dynamic shared memory PlaneRing<9*KC, IG_STAGES>::bytes().
constexpr int IG_STAGES = 3;

template <int KC>
__global__ void __launch_bounds__(AT_THREADS)
attention_input_grad_kernel(const float* __restrict__ gl, const float* __restrict__ add, long long add_sb,
                            float* __restrict__ gx, int accumulate, int Kc, int k0, int D, int H1, int W1) {
  extern __shared__ float ring_dyn[];
  const int N1 = H1 * W1;
  const int p = blockIdx.x * AT_THREADS + threadIdx.x, b = blockIdx.y;
  if (p >= N1) return;
  const int h = p / W1, w = p - h * W1;
  const Neighbourhood nb(h, w, H1, W1);
  const PlaneRing<9 * KC, IG_STAGES> ring(ring_dyn);
  const size_t plane = (size_t)N1;
  const float* g0 = gl + ((size_t)b * Kc + k0) * D * plane + p;
  float* o0 = gx + (size_t)b * 2 * D * plane + p;
  const float* ad = add != nullptr ? add + (size_t)b * add_sb + p : nullptr;

  auto issue = [&](int e) {
    if (e < D) {
      const int s = e % IG_STAGES;
#pragma unroll
      for (int k = 0; k < KC; ++k) {
        const float* q = g0 + ((size_t)k * D + e) * plane;
#pragma unroll
        for (int n = 0; n < 9; ++n) cp_async4(ring.slot(s, k * 9 + n), nb.has(n) ? q + nb.off[n] : q, nb.has(n));
      }
    }
    cp_async_commit();
  };
  float acc[2][3];  // [c][output d = e-1, e, e+1]
#pragma unroll
  for (int c = 0; c < 2; ++c) acc[c][0] = acc[c][1] = acc[c][2] = 0.f;
  auto emit = [&](int d) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const size_t i = ((size_t)c * D + d) * plane;
      float v = acc[c][0];
      if (ad != nullptr) v += __ldg(ad + i);
      if (accumulate) v += o0[i];
      o0[i] = v;
    }
  };
#pragma unroll
  for (int s = 0; s < IG_STAGES - 1; ++s) issue(s);
  for (int e = 0; e < D; ++e) {  // plane e of gL feeds gX planes e-1 (td=0), e (td=1), e+1 (td=2)
    issue(e + IG_STAGES - 1);
    cp_async_wait<IG_STAGES - 1>();
    const int s = e % IG_STAGES;
#pragma unroll
    for (int k = 0; k < KC; ++k)
#pragma unroll
      for (int n = 0; n < 9; ++n) {
        // neighbour n = (nh, nw) holds gL at (h + nh - 1, w + nw - 1), which meets tap th = 2 - nh, tw = 2 - nw
        const int t = (2 - n / 3) * 3 + (2 - n % 3);
        const float v = *ring.slot(s, k * 9 + n);
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int td = 0; td < 3; ++td)
            acc[c][td] = fmaf(v, c_att_weights[(k * 2 + c) * AT_TAPS + td * 9 + t], acc[c][td]);
      }
    if (e >= 1) emit(e - 1);
#pragma unroll
    for (int c = 0; c < 2; ++c) { acc[c][0] = acc[c][1]; acc[c][1] = acc[c][2]; acc[c][2] = 0.f; }
  }
  emit(D - 1);
}

// ---- weight gradients ----------------------------------------------------------------------------------
// gW[k, c, td, th, tw] = sum_{b, d, h, w} gL[k, d, h, w] * X[c, d + td - 1, h + th - 1, w + tw - 1]
// grid (ceil(N1/128), B, 2 * ceil(Kc/KW)), block 128: a thread owns input channel c and KW output channels;
// its KW*27 sums live in registers, every X value it reads feeds 3*KW of them.
// partial: (B * gridDim.x, Kc, 2, 27).
constexpr int WG_STAGES = 4;

template <int KW>
__global__ void __launch_bounds__(AT_THREADS)
attention_weight_grad_kernel(const float* __restrict__ x, long long x_sb, const float* __restrict__ gl,
                             float* __restrict__ partial, int Kc, int D, int H1, int W1) {
  constexpr int NV = 9 + KW;
  __shared__ float ring_mem[WG_STAGES * NV * AT_THREADS];
  __shared__ float red[(AT_THREADS / 32) * KW * AT_TAPS];
  const int N1 = H1 * W1;
  const int b = blockIdx.y, c = blockIdx.z & 1, k0 = (blockIdx.z >> 1) * KW;
  const size_t plane = (size_t)N1;
  const int p = blockIdx.x * AT_THREADS + threadIdx.x;
  float acc[KW * AT_TAPS];  // [k][td][neighbour]
#pragma unroll
  for (int i = 0; i < KW * AT_TAPS; ++i) acc[i] = 0.f;
  if (p < N1) {
    const int h = p / W1, w = p - h * W1;
    const Neighbourhood nb(h, w, H1, W1);
    const PlaneRing<NV, WG_STAGES> ring(ring_mem);
    const float* xc = x + (size_t)b * x_sb + (size_t)c * D * plane + p;
    const float* g = gl + ((size_t)b * Kc + k0) * D * plane + p;
    auto issue = [&](int e) {  // X neighbourhood of plane e and gL of plane e+1
      if (e < D) {
        const int s = e % WG_STAGES;
        const float* q = xc + (size_t)e * plane;
#pragma unroll
        for (int n = 0; n < 9; ++n) cp_async4(ring.slot(s, n), nb.has(n) ? q + nb.off[n] : q, nb.has(n));
#pragma unroll
        for (int k = 0; k < KW; ++k) {
          const bool ok = e + 1 < D && k0 + k < Kc;
          cp_async4(ring.slot(s, 9 + k), ok ? g + ((size_t)k * D + e + 1) * plane : g, ok);
        }
      }
      cp_async_commit();
    };
    float g_prev[KW], g_cur[KW], g_next[KW];
#pragma unroll
    for (int k = 0; k < KW; ++k) {
      g_prev[k] = 0.f;
      g_cur[k] = k0 + k < Kc ? __ldg(g + (size_t)k * D * plane) : 0.f;
    }
#pragma unroll
    for (int s = 0; s < WG_STAGES - 1; ++s) issue(s);
    for (int e = 0; e < D; ++e) {  // plane e of X meets gL at d = e+1 (td=0), e (td=1), e-1 (td=2)
      issue(e + WG_STAGES - 1);
      cp_async_wait<WG_STAGES - 1>();
      const int s = e % WG_STAGES;
      float v[9];
#pragma unroll
      for (int n = 0; n < 9; ++n) v[n] = *ring.slot(s, n);
#pragma unroll
      for (int k = 0; k < KW; ++k) g_next[k] = *ring.slot(s, 9 + k);
#pragma unroll
      for (int k = 0; k < KW; ++k)
#pragma unroll
        for (int n = 0; n < 9; ++n) {
          acc[k * AT_TAPS + n] = fmaf(g_next[k], v[n], acc[k * AT_TAPS + n]);
          acc[k * AT_TAPS + 9 + n] = fmaf(g_cur[k], v[n], acc[k * AT_TAPS + 9 + n]);
          acc[k * AT_TAPS + 18 + n] = fmaf(g_prev[k], v[n], acc[k * AT_TAPS + 18 + n]);
        }
#pragma unroll
      for (int k = 0; k < KW; ++k) { g_prev[k] = g_cur[k]; g_cur[k] = g_next[k]; }
    }
  }
  // reduce over the block; thread i < KW*27 then holds column (k, td, n) and stores it at [k0 + k][c][td*9 + n]
#pragma unroll
  for (int i = 0; i < KW * AT_TAPS; ++i) {
    float s = acc[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    acc[i] = s;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < KW * AT_TAPS; ++i) red[warp * KW * AT_TAPS + i] = acc[i];
  }
  __syncthreads();
  float* dst = partial + ((size_t)b * gridDim.x + blockIdx.x) * Kc * 2 * AT_TAPS;
  for (int i = threadIdx.x; i < KW * AT_TAPS; i += AT_THREADS) {
    const int k = i / AT_TAPS, t = i - k * AT_TAPS;
    if (k0 + k >= Kc) continue;
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < AT_THREADS / 32; ++wv) s += red[wv * KW * AT_TAPS + i];
    dst[((size_t)(k0 + k) * 2 + c) * AT_TAPS + t] = s;
  }
}

// out[i] = sum over rows of partial[row][i].  One block per column: thread t adds rows t, t + 256, ... in order, then
// the 256 partial sums are combined in a fixed tree, so the result does not depend on scheduling (bit-reproducible).
constexpr int RP_THREADS = 256;
__global__ void __launch_bounds__(RP_THREADS)
attention_reduce_partials_kernel(const float* __restrict__ partial, int rows, int cols, float* __restrict__ out) {
  __shared__ float red[RP_THREADS];
  const int i = blockIdx.x;
  float s = 0.f;
  for (int r = threadIdx.x; r < rows; r += RP_THREADS) s += __ldg(partial + (size_t)r * cols + i);
  red[threadIdx.x] = s;
  __syncthreads();
#pragma unroll
  for (int o = RP_THREADS / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[i] = red[0];
}

// ---- input and weight gradients, pixel tiles fetched by TMA -------------------------------------------------
// Same arithmetic as the two gather kernels above with the tile scheme of attention_forward_tiled_kernel.
// Input gradients: the stage holds the tile (with halo) of the KC logit-gradient channels of one plane.
template <int KC>
__global__ void __launch_bounds__(AT_THREADS + 32)
attention_input_grad_tiled_kernel(const __grid_constant__ CUtensorMap tm_gl, const float* __restrict__ add,
                                  long long add_sb, float* __restrict__ gx, int accumulate, int k0, int D, int H1,
                                  int W1, int* status) {
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  __shared__ __align__(128) AttentionTileSmem<KC> sm;
  const int w0 = blockIdx.x * AT_TW, h0 = blockIdx.y * AT_TH, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < AT_TSTAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], AT_THREADS / 32); }
    wait_ctl_init(&sm.ctl, 0);
    fence_barrier_init();
    prefetch_tensormap(&tm_gl);
  }
  __syncthreads();
  if (warp == AT_THREADS / 32) {  // producer
    if (lane == 0) {
      for (int e = 0; e < D; ++e) {
        const uint32_t s = e % AT_TSTAGES, ph = (e / AT_TSTAGES) & 1u;
        if (!mbar_wait(&sm.empty[s], ph ^ 1u, &sm.ctl, status, DEV_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&sm.full[s], KC * AT_TILE_BYTES);
        tma_load_5d(sm.x[s].v, &tm_gl, &sm.full[s], w0 - 4, h0 - 1, e, k0, b);
      }
    }
    return;
  }
  const int tx = lane, ty = warp;
  const int h = h0 + ty, w = w0 + tx;
  const bool valid = h < H1 && w < W1;
  const size_t plane = (size_t)H1 * W1, p = valid ? (size_t)h * W1 + w : 0;
  float* o0 = gx + (size_t)b * 2 * D * plane + p;
  const float* ad = add != nullptr ? add + (size_t)b * add_sb + p : nullptr;
  float acc[2][3];  // [c][output d = e-1, e, e+1]
#pragma unroll
  for (int c = 0; c < 2; ++c) acc[c][0] = acc[c][1] = acc[c][2] = 0.f;
  auto emit = [&](int d) {
    if (!valid) return;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const size_t i = ((size_t)c * D + d) * plane;
      float v = acc[c][0];
      if (ad != nullptr) v += __ldg(ad + i);
      if (accumulate) v += o0[i];
      o0[i] = v;
    }
  };
  for (int e = 0; e < D; ++e) {  // plane e of gL feeds gX planes e-1 (td=0), e (td=1), e+1 (td=2)
    const uint32_t s = e % AT_TSTAGES, ph = (e / AT_TSTAGES) & 1u;
    const bool ok = mbar_wait(&sm.full[s], ph, &sm.ctl, status, DEV_TIMEOUT_EPILOGUE);
    if (!__all_sync(0xffffffffu, ok)) return;
    float v[KC][9];
#pragma unroll
    for (int k = 0; k < KC; ++k)
#pragma unroll
      for (int n = 0; n < 9; ++n) v[k][n] = sm.x[s].v[k][ty + n / 3][tx + 3 + n % 3];
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.empty[s]);
#pragma unroll
    for (int k = 0; k < KC; ++k)
#pragma unroll
      for (int n = 0; n < 9; ++n) {
        // neighbour n = (nh, nw) holds gL at (h + nh - 1, w + nw - 1), which meets tap th = 2 - nh, tw = 2 - nw
        const int t = (2 - n / 3) * 3 + (2 - n % 3);
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int td = 0; td < 3; ++td)
            acc[c][td] = fmaf(v[k][n], c_att_weights[(k * 2 + c) * AT_TAPS + td * 9 + t], acc[c][td]);
      }
    if (e >= 1) emit(e - 1);
#pragma unroll
    for (int c = 0; c < 2; ++c) { acc[c][0] = acc[c][1]; acc[c][1] = acc[c][2]; acc[c][2] = 0.f; }
  }
  emit(D - 1);
}

// Weight gradients: a thread owns input channel c and KW output channels; the stage holds the tile (with halo) of
// plane e of X[c] and the tile (without halo) of plane e+1 of the KW logit-gradient channels.
// grid (ceil(W1/32), ceil(H1/4), B * 2 * chunks); partial: (B * tiles, Kc, 2, 27).
template <int KW>
struct WeightGradTileSmem {
  struct alignas(128) Stage {   // both parts are TMA destinations: 128-byte aligned
    alignas(128) float x[AT_BOX_H][AT_BOX_W];
    alignas(128) float g[KW][AT_TH][AT_TW];
  } st[AT_TSTAGES];
  uint64_t full[AT_TSTAGES];
  uint64_t empty[AT_TSTAGES];
  WaitCtl ctl;
  float red[(AT_THREADS / 32) * KW * AT_TAPS];
};

template <int KW>
__global__ void __launch_bounds__(AT_THREADS + 32)
attention_weight_grad_tiled_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gl,
                                   const float* __restrict__ gl, float* __restrict__ partial, int Kc, int B, int D,
                                   int H1, int W1, int* status) {
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  __shared__ __align__(128) WeightGradTileSmem<KW> sm;
  const int w0 = blockIdx.x * AT_TW, h0 = blockIdx.y * AT_TH;
  const int b = blockIdx.z % B, zc = blockIdx.z / B, c = zc & 1, k0 = (zc >> 1) * KW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < AT_TSTAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], AT_THREADS / 32); }
    wait_ctl_init(&sm.ctl, 0);
    fence_barrier_init();
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_gl);
  }
  __syncthreads();
  if (warp == AT_THREADS / 32) {  // producer
    if (lane == 0) {
      for (int e = 0; e < D; ++e) {
        const uint32_t s = e % AT_TSTAGES, ph = (e / AT_TSTAGES) & 1u;
        if (!mbar_wait(&sm.empty[s], ph ^ 1u, &sm.ctl, status, DEV_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&sm.full[s], AT_TILE_BYTES + KW * AT_TH * AT_TW * (uint32_t)sizeof(float));
        tma_load_5d(sm.st[s].x, &tm_x, &sm.full[s], w0 - 4, h0 - 1, e, c, b);
        tma_load_5d(sm.st[s].g, &tm_gl, &sm.full[s], w0, h0, e + 1, k0, b);  // plane D and channels >= Kc read as zero
      }
    }
    return;
  }
  const int tx = lane, ty = warp;
  const int h = h0 + ty, w = w0 + tx;
  const bool valid = h < H1 && w < W1;
  const size_t plane = (size_t)H1 * W1;
  float acc[KW * AT_TAPS];  // [k][td][neighbour]
#pragma unroll
  for (int i = 0; i < KW * AT_TAPS; ++i) acc[i] = 0.f;
  float g_prev[KW], g_cur[KW], g_next[KW];
#pragma unroll
  for (int k = 0; k < KW; ++k) {
    g_prev[k] = 0.f;
    g_cur[k] = (valid && k0 + k < Kc) ? __ldg(gl + (((size_t)b * Kc + k0 + k) * D) * plane + (size_t)h * W1 + w) : 0.f;
  }
  bool alive = true;
  for (int e = 0; e < D; ++e) {  // plane e of X meets gL at d = e+1 (td=0), e (td=1), e-1 (td=2)
    const uint32_t s = e % AT_TSTAGES, ph = (e / AT_TSTAGES) & 1u;
    const bool ok = mbar_wait(&sm.full[s], ph, &sm.ctl, status, DEV_TIMEOUT_EPILOGUE);
    if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
    float v[9];
#pragma unroll
    for (int n = 0; n < 9; ++n) v[n] = sm.st[s].x[ty + n / 3][tx + 3 + n % 3];
#pragma unroll
    for (int k = 0; k < KW; ++k) g_next[k] = sm.st[s].g[k][ty][tx];
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.empty[s]);
#pragma unroll
    for (int k = 0; k < KW; ++k)
#pragma unroll
      for (int n = 0; n < 9; ++n) {
        acc[k * AT_TAPS + n] = fmaf(g_next[k], v[n], acc[k * AT_TAPS + n]);
        acc[k * AT_TAPS + 9 + n] = fmaf(g_cur[k], v[n], acc[k * AT_TAPS + 9 + n]);
        acc[k * AT_TAPS + 18 + n] = fmaf(g_prev[k], v[n], acc[k * AT_TAPS + 18 + n]);
      }
#pragma unroll
    for (int k = 0; k < KW; ++k) { g_prev[k] = g_cur[k]; g_cur[k] = g_next[k]; }
  }
  // reduce over the block's 128 pixel threads (named barrier 1: the producer warp has left);
  // thread i < KW*27 then holds column (k, td, n) and stores it at [k0 + k][c][td*9 + n]
#pragma unroll
  for (int i = 0; i < KW * AT_TAPS; ++i) {
    float sum = alive ? acc[i] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    acc[i] = sum;
  }
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < KW * AT_TAPS; ++i) sm.red[warp * KW * AT_TAPS + i] = acc[i];
  }
  named_bar_sync(1, AT_THREADS);
  const int tiles = gridDim.x * gridDim.y;
  float* dst = partial + ((size_t)b * tiles + blockIdx.y * gridDim.x + blockIdx.x) * Kc * 2 * AT_TAPS;
  for (int i = threadIdx.x; i < KW * AT_TAPS; i += AT_THREADS) {
    const int k = i / AT_TAPS, t = i - k * AT_TAPS;
    if (k0 + k >= Kc) continue;
    float sum = 0.f;
#pragma unroll
    for (int wv = 0; wv < AT_THREADS / 32; ++wv) sum += sm.red[wv * KW * AT_TAPS + i];
    dst[((size_t)(k0 + k) * 2 + c) * AT_TAPS + t] = sum;
  }
}

// ---- staging of the filter weights in constant memory ---------------------------------------------------
// c_att_weights is one array per device.  Work on one stream is ordered anyway; a call on another stream first
// waits for the event the previous user recorded after its last kernel, so the copy below never overtakes a
// kernel that still reads the old weights.  The lock is held from the copy to that record.
namespace {
constexpr int AT_MAX_DEVICES = 64;
struct WeightStage {
  std::mutex mu;
  cudaEvent_t done[AT_MAX_DEVICES] = {nullptr};
  cudaStream_t last[AT_MAX_DEVICES] = {nullptr};
  bool used[AT_MAX_DEVICES] = {false};
} g_stage;

class StagedWeights {
 public:
  explicit StagedWeights(cudaStream_t st) : lock_(g_stage.mu), st_(st) {
    err_ = cudaGetDevice(&dev_);
    if (err_ == cudaSuccess && (dev_ < 0 || dev_ >= AT_MAX_DEVICES)) err_ = cudaErrorInvalidDevice;
    if (err_ != cudaSuccess) return;
    if (g_stage.done[dev_] == nullptr) err_ = cudaEventCreateWithFlags(&g_stage.done[dev_], cudaEventDisableTiming);
    if (err_ == cudaSuccess && g_stage.used[dev_] && g_stage.last[dev_] != st_)
      err_ = cudaStreamWaitEvent(st_, g_stage.done[dev_], 0);
  }
  cudaError_t put(const float* device_weights, int channels) {  // weights of `channels` <= AT_KC channels
    if (err_ != cudaSuccess) return err_;
    err_ = cudaMemcpyToSymbolAsync(c_att_weights, device_weights, (size_t)channels * 2 * AT_TAPS * sizeof(float), 0,
                                   cudaMemcpyDeviceToDevice, st_);
    return err_;
  }
  ~StagedWeights() {
    if (err_ != cudaSuccess) return;
    if (cudaEventRecord(g_stage.done[dev_], st_) == cudaSuccess) {
      g_stage.last[dev_] = st_;
      g_stage.used[dev_] = true;
    }
  }

 private:
  std::lock_guard<std::mutex> lock_;
  cudaStream_t st_;
  int dev_ = 0;
  cudaError_t err_ = cudaSuccess;
};
}  // namespace

// ---- launchers ---------------------------------------------------------------------------------------
static dim3 pixel_grid(const AttentionDims& d) { return dim3((d.H1 * d.W1 + AT_THREADS - 1) / AT_THREADS, d.B); }

static size_t tile_count(const AttentionDims& d) {
  return (size_t)((d.W1 + AT_TW - 1) / AT_TW) * ((d.H1 + AT_TH - 1) / AT_TH);
}
size_t attention_partial_floats(const AttentionDims& d) {  // bias partials per pixel block, weight partials per block / tile
  const size_t blocks = (size_t)pixel_grid(d).x, tiles = tile_count(d);
  return (size_t)d.B * d.Kc * (blocks + 2 * AT_TAPS * (blocks > tiles ? blocks : tiles));
}

cudaError_t launch_attention_forward(const AttentionDims& d, const float* x, long long x_sb, const float* weight,
                                     const float* bias, float* a, cudaStream_t st, int* status) {
  const dim3 grid = pixel_grid(d);
  const bool tiled = status != nullptr && tileable(d, x, x_sb);
  CUtensorMap tm_x;
  if (tiled) {
    cudaError_t err = tile_map(&tm_x, x, x_sb, 2, 2, d, true);
    if (err != cudaSuccess) return err;
  }
  const dim3 tgrid((d.W1 + AT_TW - 1) / AT_TW, (d.H1 + AT_TH - 1) / AT_TH, d.B);
  StagedWeights staged(st);
  for (int k0 = 0; k0 < d.Kc; k0 += AT_KC) {
    const int kc = d.Kc - k0 < AT_KC ? d.Kc - k0 : AT_KC;
    cudaError_t err = staged.put(weight + (size_t)k0 * 2 * AT_TAPS, kc);
    if (err != cudaSuccess) return err;
    if (tiled) {
#define SFB_AT_FWD_T(KC) attention_forward_tiled_kernel<KC><<<tgrid, AT_THREADS + 32, 0, st>>>(tm_x, bias, a, d.Kc, k0, d.D, d.H1, d.W1, status)
      if (kc == 1) SFB_AT_FWD_T(1); else if (kc == 2) SFB_AT_FWD_T(2); else if (kc == 3) SFB_AT_FWD_T(3); else SFB_AT_FWD_T(4);
#undef SFB_AT_FWD_T
      continue;
    }
#define SFB_AT_FWD(KC) attention_forward_kernel<KC><<<grid, AT_THREADS, 0, st>>>(x, x_sb, bias, a, d.Kc, k0, d.D, d.H1, d.W1)
    if (kc == 1) SFB_AT_FWD(1); else if (kc == 2) SFB_AT_FWD(2); else if (kc == 3) SFB_AT_FWD(3); else SFB_AT_FWD(4);
#undef SFB_AT_FWD
  }
  return cudaGetLastError();
}

template <int KC>
static cudaError_t launch_input_grad(const dim3 grid, const float* g, const float* add, long long add_sb, float* gx,
                                     int accumulate, const AttentionDims& d, int k0, cudaStream_t st) {
  constexpr size_t smem = PlaneRing<9 * KC, IG_STAGES>::bytes();
  static bool configured[AT_MAX_DEVICES] = {false};  // benign race: setting the attribute twice is harmless
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (smem > 48 * 1024 && dev >= 0 && dev < AT_MAX_DEVICES && !configured[dev]) {
    err = cudaFuncSetAttribute(attention_input_grad_kernel<KC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    configured[dev] = true;
  }
  attention_input_grad_kernel<KC><<<grid, AT_THREADS, smem, st>>>(g, add, add_sb, gx, accumulate, d.Kc, k0, d.D, d.H1,
                                                                  d.W1);
  return cudaGetLastError();
}

cudaError_t launch_attention_backward(const AttentionDims& d, const float* x, long long x_sb, const float* weight,
                                      const float* a, float* g, const float* add, long long add_sb, float* gx,
                                      float* gweight, float* gbias, float* partial, cudaStream_t st, int* status) {
  const int N1 = d.H1 * d.W1;
  const dim3 grid = pixel_grid(d);
  const int rows = (int)(grid.x * grid.y);
  float* bias_partial = partial;                            // (rows, Kc)
  float* weight_partial = partial + (size_t)rows * d.Kc;    // (rows or tiles, Kc, 54)
  const long long g_sb = (long long)d.Kc * d.D * N1;
  const bool tiled = status != nullptr && tileable(d, x, x_sb) && tileable(d, g, g_sb);
  const dim3 tgrid((d.W1 + AT_TW - 1) / AT_TW, (d.H1 + AT_TH - 1) / AT_TH, d.B);
  for (int k0 = 0; k0 < d.Kc; k0 += AT_KC) {
    const int kc = d.Kc - k0 < AT_KC ? d.Kc - k0 : AT_KC;
#define SFB_AT_LG(KC) attention_logit_grad_kernel<KC><<<grid, AT_THREADS, 0, st>>>(a, g, bias_partial, d.Kc, k0, d.D, N1)
    if (kc == 1) SFB_AT_LG(1); else if (kc == 2) SFB_AT_LG(2); else if (kc == 3) SFB_AT_LG(3); else SFB_AT_LG(4);
#undef SFB_AT_LG
  }
  {
    StagedWeights staged(st);
    for (int k0 = 0; k0 < d.Kc; k0 += AT_KC) {
      const int kc = d.Kc - k0 < AT_KC ? d.Kc - k0 : AT_KC;
      cudaError_t err = staged.put(weight + (size_t)k0 * 2 * AT_TAPS, kc);
      if (err != cudaSuccess) return err;
      const float* ad = k0 == 0 ? add : nullptr;
      const int accumulate = k0 == 0 ? 0 : 1;
      if (tiled) {
        CUtensorMap tm_gl;
        err = tile_map(&tm_gl, g, g_sb, d.Kc, kc, d, true);
        if (err != cudaSuccess) return err;
#define SFB_AT_IG_T(KC) attention_input_grad_tiled_kernel<KC><<<tgrid, AT_THREADS + 32, 0, st>>>(tm_gl, ad, add_sb, gx, accumulate, k0, d.D, d.H1, d.W1, status)
        if (kc == 1) SFB_AT_IG_T(1); else if (kc == 2) SFB_AT_IG_T(2); else if (kc == 3) SFB_AT_IG_T(3); else SFB_AT_IG_T(4);
#undef SFB_AT_IG_T
        continue;
      }
      if (kc == 1) err = launch_input_grad<1>(grid, g, ad, add_sb, gx, accumulate, d, k0, st);
      else if (kc == 2) err = launch_input_grad<2>(grid, g, ad, add_sb, gx, accumulate, d, k0, st);
      else if (kc == 3) err = launch_input_grad<3>(grid, g, ad, add_sb, gx, accumulate, d, k0, st);
      else err = launch_input_grad<4>(grid, g, ad, add_sb, gx, accumulate, d, k0, st);
      if (err != cudaSuccess) return err;
    }
  }
  const int kw = d.Kc >= 4 ? 4 : d.Kc, chunks = (d.Kc + kw - 1) / kw;
  int wrows = rows;
  if (tiled) {
    CUtensorMap tm_x, tm_gl;
    cudaError_t err = tile_map(&tm_x, x, x_sb, 2, 1, d, true);
    if (err == cudaSuccess) err = tile_map(&tm_gl, g, g_sb, d.Kc, kw, d, false);
    if (err != cudaSuccess) return err;
    const dim3 wgrid(tgrid.x, tgrid.y, d.B * 2 * chunks);
    wrows = (int)(tile_count(d) * d.B);
#define SFB_AT_WG_T(KW) attention_weight_grad_tiled_kernel<KW><<<wgrid, AT_THREADS + 32, 0, st>>>(tm_x, tm_gl, g, weight_partial, d.Kc, d.B, d.D, d.H1, d.W1, status)
    if (kw == 1) SFB_AT_WG_T(1); else if (kw == 2) SFB_AT_WG_T(2); else if (kw == 3) SFB_AT_WG_T(3); else SFB_AT_WG_T(4);
#undef SFB_AT_WG_T
  } else {
#define SFB_AT_WG(KW) attention_weight_grad_kernel<KW><<<dim3(grid.x, grid.y, 2 * chunks), AT_THREADS, 0, st>>>(x, x_sb, g, weight_partial, d.Kc, d.D, d.H1, d.W1)
    if (kw == 1) SFB_AT_WG(1); else if (kw == 2) SFB_AT_WG(2); else if (kw == 3) SFB_AT_WG(3); else SFB_AT_WG(4);
#undef SFB_AT_WG
  }
  const int wcols = d.Kc * 2 * AT_TAPS;
  attention_reduce_partials_kernel<<<wcols, RP_THREADS, 0, st>>>(weight_partial, wrows, wcols, gweight);
  attention_reduce_partials_kernel<<<d.Kc, RP_THREADS, 0, st>>>(bias_partial, rows, d.Kc, gbias);
  return cudaGetLastError();
}

}  // namespace sfb
