// Operand preparation (HBM-bound, a few percent of an op's time):
//  * copies of F1 and F2 rounded to TF32 with round-to-nearest.  tcgen05.mma kind::tf32 ignores the
//    low 13 mantissa bits of its fp32 operands, i.e. truncates; truncation shrinks every product by
//    ~2^-10 and would put a bias of that relative size on every S value, rounding does not.
//  * the "aux" rows of F2 used for the mean channels: row u of aux = mean over v of F2[u,v,:],
//    row H2+v = mean over u of F2[u,v,:]  (mean_v S[p,u,v] = F1[p] . mean_v F2[u,v], the same sum the
//    reference accumulates cell by cell, MemorySaver_kernel_forward.cu:286-290).
//  * 16-bit operand copies (BF16, or FP16 for the operand type with TF32's mantissa at twice its tensor-core rate).
//    FP16 has a narrow exponent range, so every tensor that becomes an FP16 operand is first multiplied by a power
//    of two that brings its largest magnitude next to 1 (exact, undone when results are stored): absmax_kernel
//    finds the magnitudes, *_scales_kernel turn them into the multipliers, all on the device.
#include <algorithm>

#include <cuda_bf16.h>

#include "kernels.h"
#include "sm100_primitives.cuh"

namespace sfb {

// Largest |x| * premul of an array, as the bits of a non-negative float, combined into *out with atomicMax (integer
// order = float order for non-negative values; NaNs are ignored).  n4 = number of float4.
__global__ void absmax_kernel(const float4* __restrict__ x, size_t n4, int tail, float premul,
                              unsigned* __restrict__ out) {
  float m = 0.f;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = __ldg(x + i);
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
  if (blockIdx.x == 0 && (int)threadIdx.x < tail) m = fmaxf(m, fabsf(__ldg(reinterpret_cast<const float*>(x + n4) + threadIdx.x)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(out, __float_as_uint(m * fabsf(premul)));
}

cudaError_t launch_absmax(const float* x, size_t n, float premul, float* slot, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  const size_t n4 = n / 4;  // the arrays are 16-byte aligned; up to three trailing values are read one by one
  const int threads = 256;
  const unsigned blocks = (unsigned)std::max<size_t>(1, std::min<size_t>((n4 + threads - 1) / threads, 148 * 8));
  absmax_kernel<<<blocks, threads, 0, stream>>>(reinterpret_cast<const float4*>(x), n4, (int)(n - 4 * n4), premul,
                                                reinterpret_cast<unsigned*>(slot));
  return cudaGetLastError();
}

// The power of two that brings a largest magnitude (float bits in `amax_bits`) into [target, 2*target); 1 when the
// magnitude is zero, not finite or subnormal, and never beyond 2^+-40, so that products of three scales stay finite
// (tensors whose largest magnitude lies outside about 1e-12 .. 1e12 are not brought all the way into FP16's range;
// TF32 operands are the choice for such data).
__device__ __forceinline__ float pow2_scale(unsigned amax_bits, int target_log2) {
  const int e = (int)(amax_bits >> 23) & 0xff;
  if (e == 0 || e == 255) return 1.f;
  int shift = target_log2 - (e - 127);
  shift = max(-40, min(40, shift));
  return __uint_as_float((unsigned)(127 + shift) << 23);
}

// scales[] (SCALE_* in kernels.h): feature scales from the two magnitudes found by absmax_kernel.
__global__ void feature_scales_kernel(float* scales) {
  const float s1 = pow2_scale(__float_as_uint(scales[SCALE_AMAX_F1]), 0);
  const float s2 = pow2_scale(__float_as_uint(scales[SCALE_AMAX_F2]), 0);
  scales[SCALE_F1] = s1;
  scales[SCALE_F2] = s2;
  scales[SCALE_INV_F1F2] = 1.f / (s1 * s2);
}
// Gradient-operand scales (after feature_scales_kernel of the same call): G is generated as (sg * sa) * G.
__global__ void grad_scales_kernel(float* scales) {
  const float sg = pow2_scale(__float_as_uint(scales[SCALE_AMAX_G]), 7);   // largest gradient value -> [128, 256)
  const float sa = pow2_scale(__float_as_uint(scales[SCALE_AMAX_A]), 0);   // largest weight -> [1, 2)
  scales[SCALE_GA] = sg * sa;
  scales[SCALE_G] = sg;
  scales[SCALE_A] = sa;
  scales[SCALE_INV_GF1] = 1.f / (sg * sa * scales[SCALE_F2]);   // gF1 = G * F2
  scales[SCALE_INV_GF2] = 1.f / (sg * sa * scales[SCALE_F1]);   // gF2 = G^T * F1
}
cudaError_t launch_feature_scales(float* scales, cudaStream_t stream) {
  feature_scales_kernel<<<1, 1, 0, stream>>>(scales);
  return cudaGetLastError();
}
cudaError_t launch_grad_scales(float* scales, cudaStream_t stream) {
  grad_scales_kernel<<<1, 1, 0, stream>>>(scales);
  return cudaGetLastError();
}

// `outh` (optional): the same values as 16-bit operands of kind `op16` instead (BF16, or FP16 of the value times the
// device scalar *scale16).
__global__ void round_copy_kernel(const float4* __restrict__ in, float4* __restrict__ out, size_t n4,
                                  uint2* __restrict__ outh, int op16, const float* __restrict__ scale16) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const float sc = (outh != nullptr && scale16 != nullptr) ? __ldg(scale16) : 1.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 v = __ldg(in + i);
    if (outh != nullptr) {
      if (op16 == OP16_FP16) outh[i] = make_uint2(pack_fp16x2(v.x * sc, v.y * sc), pack_fp16x2(v.z * sc, v.w * sc));
      else outh[i] = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
    }
    v.x = round_tf32(v.x); v.y = round_tf32(v.y); v.z = round_tf32(v.z); v.w = round_tf32(v.w);
    out[i] = v;
  }
}

// grid (H2 + W2, B), block = min(C, 256) threads over channels.
__global__ void f2_means_kernel(const float* __restrict__ F2, float* __restrict__ aux, int H2, int W2, int C,
                                uint16_t* __restrict__ auxh, int op16, const float* __restrict__ scale16) {
  const int r = blockIdx.x, b = blockIdx.y;
  const float* base = F2 + (size_t)b * H2 * W2 * C;
  float* dst = aux + ((size_t)b * (H2 + W2) + r) * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    if (r < H2) {
      const float* row = base + (size_t)r * W2 * C + c;
      for (int v = 0; v < W2; ++v) acc += __ldg(row + (size_t)v * C);
      acc /= (float)W2;
    } else {
      const float* col = base + (size_t)(r - H2) * C + c;
      for (int u = 0; u < H2; ++u) acc += __ldg(col + (size_t)u * W2 * C);
      acc /= (float)H2;
    }
    dst[c] = round_tf32(acc);
    if (auxh != nullptr)
      auxh[((size_t)b * (H2 + W2) + r) * C + c] = to_op16(op16 == OP16_FP16 && scale16 != nullptr ? acc * __ldg(scale16) : acc, op16);
  }
}

// Tiled transposes between the reference's per-pixel layout (B, N1, K, D) (displacement d fastest) and the
// packed layout (B, D, R, n1p) (pixel fastest) the kernels use.  A block moves a patch of 128 pixels x 32
// displacements through shared memory so that both sides are coalesced; every thread keeps 16 loads in flight,
// and the displacement tiles are the fastest grid dimension so that blocks running together read neighbouring
// 128-byte pieces of the same rows.  grid (ceil(D/32), n1p/128, B*K), block (32, 8).
constexpr int PACK_PX = 128;

__global__ void pack_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, int N1, int n1p, int Ksrc,
                            int ksrc0, int K, int D, int R, int r0, int rstride, float scale) {
  __shared__ uint32_t tile[PACK_PX][33];
  const int b = blockIdx.z / K, k = blockIdx.z - b * K, d0 = blockIdx.x * 32, p0 = blockIdx.y * PACK_PX;
  const int tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
  for (int j = ty; j < PACK_PX; j += 8) {
    const int p = p0 + j, d = d0 + tx;
    uint32_t v = 0;
    if (p < N1 && d < D) v = __ldg(src + (((size_t)b * N1 + p) * Ksrc + ksrc0 + k) * D + d);
    tile[j][tx] = v;
  }
  __syncthreads();
  const int r = r0 + k * rstride;
#pragma unroll
  for (int i = ty; i < 32 * (PACK_PX / 32); i += 8) {
    const int d = d0 + i / (PACK_PX / 32), p = (i % (PACK_PX / 32)) * 32 + tx;
    if (d < D) {
      uint32_t v = tile[p][i / (PACK_PX / 32)];
      if (scale != 0.f) v = __float_as_uint(__uint_as_float(v) * scale);
      dst[(((size_t)b * D + d) * R + r) * n1p + p0 + p] = v;
    }
  }
}

__global__ void unpack_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, int N1, int n1p, int K,
                              int D, int R, int r0, int rstride, int Kdst, int kdst0) {
  __shared__ uint32_t tile[PACK_PX][33];
  const int b = blockIdx.z / K, k = blockIdx.z - b * K, d0 = blockIdx.x * 32, p0 = blockIdx.y * PACK_PX;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int r = r0 + k * rstride;
#pragma unroll
  for (int i = ty; i < 32 * (PACK_PX / 32); i += 8) {
    const int dl = i / (PACK_PX / 32), p = (i % (PACK_PX / 32)) * 32 + tx;
    tile[p][dl] = (d0 + dl < D) ? __ldg(src + (((size_t)b * D + d0 + dl) * R + r) * n1p + p0 + p) : 0u;
  }
  __syncthreads();
#pragma unroll
  for (int j = ty; j < PACK_PX; j += 8) {
    const int p = p0 + j, d = d0 + tx;
    if (p < N1 && d < D) dst[(((size_t)b * N1 + p) * Kdst + kdst0 + k) * D + d] = tile[j][tx];
  }
}

// Interleaved pack: every block transposes a 32-pixel x 32-displacement patch of each source through
// shared memory, then writes, per displacement, the R4 slots of its 32 pixels as one contiguous run.
template <int R4>
__global__ void pack_interleaved_kernel(const SlotSources src, uint32_t* __restrict__ dst, int N1, int n1p, int D,
                                        int Qtot, int q0) {
  constexpr int RS = 32 * 33 + 32 / R4;  // slot stride chosen so that the interleaved read below is conflict-free
  __shared__ uint32_t tile[R4 * RS];
  const int b = blockIdx.z, d0 = blockIdx.x * 32, p0 = blockIdx.y * 32;  // displacement tiles fastest
  const int tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
  for (int r = 0; r < R4; ++r) {
    const uint32_t* s = static_cast<const uint32_t*>(src.s[r].src);
    for (int j = ty; j < 32; j += 8) {
      const int p = p0 + j, d = d0 + tx;
      uint32_t v = 0;
      if (p < N1 && d < D) {
        if (s == nullptr) {
          v = __float_as_uint(src.s[r].scale);  // constant slot
        } else {
          v = __ldg(s + (((size_t)b * N1 + p) * src.s[r].Ksrc + src.s[r].k) * D + d);
          if (src.s[r].scale != 0.f) v = __float_as_uint(__uint_as_float(v) * src.s[r].scale);
          if (src.s[r].dev != 0) v = __float_as_uint(__uint_as_float(v) * __ldg(src.dev_scales + src.s[r].dev - 1));
        }
      }
      tile[r * RS + j * 33 + tx] = v;
    }
  }
  __syncthreads();
  // per displacement and group of four slots: 32 pixels x 4 slots = 128 consecutive words
  const int t = ty * 32 + tx;
  for (int j = 0; j < 32; ++j) {
    const int d = d0 + j;
    if (d >= D) break;
    for (int i = t; i < 32 * R4; i += 256) {
      const int q = i / 128, w = i % 128;  // group, word inside the group's 32-pixel run
      dst[((((size_t)b * D + d) * Qtot + q0 + q) * n1p + p0) * 4 + w] = tile[(q * 4 + (w & 3)) * RS + (w >> 2) * 33 + j];
    }
  }
}

cudaError_t launch_pack_interleaved(const SlotSources& src, float* dst, int B, int N1, int n1p, int D, int R4,
                                    int Qtot, int q0, cudaStream_t stream) {
  const dim3 grid((D + 31) / 32, n1p / 32, B), block(32, 8);
  uint32_t* out = reinterpret_cast<uint32_t*>(dst);
  if (R4 == 4) pack_interleaved_kernel<4><<<grid, block, 0, stream>>>(src, out, N1, n1p, D, Qtot, q0);
  else if (R4 == 8) pack_interleaved_kernel<8><<<grid, block, 0, stream>>>(src, out, N1, n1p, D, Qtot, q0);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

// Channels-first sources are already pixel-fastest: one thread per pixel gathers the four slots of a group
// and stores them as one 16-byte word, for PI_DB displacements at a time (all loads issued before the stores,
// so that a thread keeps 4*Q*PI_DB loads in flight).  grid (n1p/256, ceil(D/PI_DB), B), block 256.
constexpr int PI_DB = 4;

template <int Q>
__global__ void pack_interleaved_cf_kernel(const SlotSources src, float4* __restrict__ dst, int N1, int n1p, int D,
                                           int Qtot, int q0) {
  const int p = blockIdx.x * 256 + threadIdx.x, d0 = blockIdx.y * PI_DB, b = blockIdx.z;
  if (p >= n1p) return;
  // per slot: the factor its values are multiplied by (0 = raw 32-bit copy): host scale times device scale
  float fac[Q][4];
#pragma unroll
  for (int q = 0; q < Q; ++q)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const SlotSource& ss = src.s[4 * q + j];
      fac[q][j] = ss.scale;
      if (ss.dev != 0 && ss.src != nullptr) fac[q][j] = (ss.scale != 0.f ? ss.scale : 1.f) * __ldg(src.dev_scales + ss.dev - 1);
    }
  uint32_t w[PI_DB][Q][4];
#pragma unroll
  for (int i = 0; i < PI_DB; ++i)
#pragma unroll
    for (int q = 0; q < Q; ++q)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const SlotSource& ss = src.s[4 * q + j];
        w[i][q][j] = 0;
        if (ss.src != nullptr && p < N1 && d0 + i < D)
          w[i][q][j] = __ldg(static_cast<const uint32_t*>(ss.src) + (((size_t)b * ss.Ksrc + ss.k) * D + d0 + i) * N1 + p);
        else if (ss.src == nullptr && p < N1)
          w[i][q][j] = __float_as_uint(ss.scale);  // constant slot
      }
#pragma unroll
  for (int i = 0; i < PI_DB; ++i) {
    if (d0 + i >= D) break;
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const SlotSource& ss = src.s[4 * q + j];
        v[j] = (fac[q][j] != 0.f && ss.src != nullptr) ? __uint_as_float(w[i][q][j]) * fac[q][j] : __uint_as_float(w[i][q][j]);
      }
      dst[(((size_t)b * D + d0 + i) * Qtot + q0 + q) * n1p + p] = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
}

cudaError_t launch_pack_interleaved_cf(const SlotSources& src, float* dst, int B, int N1, int n1p, int D, int R4,
                                       int Qtot, int q0, cudaStream_t stream) {
  const dim3 grid((n1p + 255) / 256, (D + PI_DB - 1) / PI_DB, B);
  float4* out = reinterpret_cast<float4*>(dst);
  if (R4 == 4) pack_interleaved_cf_kernel<1><<<grid, 256, 0, stream>>>(src, out, N1, n1p, D, Qtot, q0);
  else if (R4 == 8) pack_interleaved_cf_kernel<2><<<grid, 256, 0, stream>>>(src, out, N1, n1p, D, Qtot, q0);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t launch_pack(const void* src, float* dst, int B, int N1, int n1p, int Ksrc, int ksrc0, int K, int D,
                        int R, int r0, int rstride, float scale, cudaStream_t stream) {
  const dim3 grid((D + 31) / 32, n1p / PACK_PX, B * K), block(32, 8);
  pack_kernel<<<grid, block, 0, stream>>>(static_cast<const uint32_t*>(src), reinterpret_cast<uint32_t*>(dst), N1,
                                          n1p, Ksrc, ksrc0, K, D, R, r0, rstride, scale);
  return cudaGetLastError();
}

cudaError_t launch_unpack(const float* src, void* dst, int B, int N1, int n1p, int K, int D, int R, int r0,
                          int rstride, int Kdst, int kdst0, cudaStream_t stream) {
  const dim3 grid((D + 31) / 32, n1p / PACK_PX, B * K), block(32, 8);
  unpack_kernel<<<grid, block, 0, stream>>>(reinterpret_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), N1,
                                            n1p, K, D, R, r0, rstride, Kdst, kdst0);
  return cudaGetLastError();
}

// (B, C, N) -> (B, N, C), scaled and rounded to TF32.  32 x 32 tiles through shared memory; grid
// (ceil(N/32), ceil(C/32), B), block (32, 8).
__global__ void transpose_round_kernel(const float* __restrict__ in, float* __restrict__ out, int C, int N,
                                       float scale, uint16_t* __restrict__ outh, int op16,
                                       const float* __restrict__ scale16) {
  __shared__ float tile[32][33];
  const float sc16 = (outh != nullptr && op16 == OP16_FP16 && scale16 != nullptr) ? __ldg(scale16) : 1.f;
  const int b = blockIdx.z, p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
  for (int j = ty; j < 32; j += 8) {
    const int c = c0 + j, p = p0 + tx;
    tile[j][tx] = (c < C && p < N) ? __ldg(in + ((size_t)b * C + c) * N + p) : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int j = ty; j < 32; j += 8) {
    const int p = p0 + j, c = c0 + tx;
    if (p < N && c < C) {
      const float v = tile[tx][j] * scale;
      out[((size_t)b * N + p) * C + c] = round_tf32(v);
      if (outh != nullptr) outh[((size_t)b * N + p) * C + c] = to_op16(v * sc16, op16);
    }
  }
}

// Channel-major copies of a pixel-major feature array (B, rows*width, C), the K-major B operands of the gradient GEMMs.
//   blocked = 0: dst (B, C, pitch), pixel index = row*width + x (image 1: rows = 1, width = N1, pitch = n1p)
//   blocked = 1: dst (B, C, ceil(width/16), pitch, 16): columns in blocks of 16, so that the 2 rows x 16 columns of one
//                K block of the image-1-major GEMM are 32 consecutive values (image 2: pitch = H2 rounded up to even)
// Padding is not written (the caller clears the array).  32 x 32 tiles through shared memory; grid (ceil(width/32),
// ceil(C/32), B*rows), block (32, 8).
template <typename T>
__global__ void channel_major_kernel(const float* __restrict__ in, T* __restrict__ out, int rows, int width,
                                     int pitch, int C, int blocked, int op16, const float* __restrict__ scale16) {
  __shared__ float tile[32][33];
  const float sc16 = (op16 == OP16_FP16 && scale16 != nullptr) ? __ldg(scale16) : 1.f;
  const int b = blockIdx.z / rows, row = blockIdx.z - b * rows, x0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const float* src = in + ((size_t)b * rows + row) * width * C;
#pragma unroll
  for (int j = ty; j < 32; j += 8) {
    const int x = x0 + j, c = c0 + tx;
    tile[j][tx] = (x < width && c < C) ? __ldg(src + (size_t)x * C + c) : 0.f;
  }
  __syncthreads();
  const size_t per_channel = blocked ? (size_t)((width + 15) / 16) * pitch * 16 : (size_t)pitch;
#pragma unroll
  for (int j = ty; j < 32; j += 8) {
    const int c = c0 + j, x = x0 + tx;
    if (c < C && x < width) {
      const size_t off = blocked ? ((size_t)(x >> 4) * pitch + row) * 16 + (x & 15) : (size_t)x;
      if constexpr (sizeof(T) == 2) out[((size_t)b * C + c) * per_channel + off] = to_op16(tile[tx][j] * sc16, op16);
      else out[((size_t)b * C + c) * per_channel + off] = tile[tx][j];
    }
  }
}

cudaError_t launch_channel_major(const float* src, void* dst, int B, int rows, int width, int pitch, int C,
                                 int blocked, int op16, const float* scale16, cudaStream_t stream) {
  const dim3 grid((width + 31) / 32, (C + 31) / 32, B * rows), block(32, 8);
  if (op16)
    channel_major_kernel<<<grid, block, 0, stream>>>(src, static_cast<uint16_t*>(dst), rows, width, pitch, C, blocked,
                                                     op16, scale16);
  else
    channel_major_kernel<<<grid, block, 0, stream>>>(src, static_cast<float*>(dst), rows, width, pitch, C, blocked, 0,
                                                     nullptr);
  return cudaGetLastError();
}

// Clears the workspace header (status word and scale slots) and, for FP16 operands, finds the two feature scales.
static cudaError_t begin_prepare(const Dims& d, const float* F1, const float* F2, float premul1, int* status, int op16,
                                 float* scales, cudaStream_t stream) {
  cudaError_t err = cudaMemsetAsync(status, 0, WS_HEADER_CLEAR_BYTES, stream);
  if (err != cudaSuccess || op16 != OP16_FP16 || scales == nullptr) return err;
  launch_absmax(F1, (size_t)d.B * d.N1() * d.C, premul1, scales + SCALE_AMAX_F1, stream);
  launch_absmax(F2, (size_t)d.B * d.N2() * d.C, 1.f, scales + SCALE_AMAX_F2, stream);
  return launch_feature_scales(scales, stream);
}

cudaError_t launch_prepare_cf(const Dims& d, const float* fmap1, const float* fmap2, float scale1, float* F1r,
                              float* F2r, float* aux, int* status, cudaStream_t stream, uint16_t* F1h, uint16_t* F2h,
                              uint16_t* auxh, int op16, float* scales) {
  cudaError_t err = begin_prepare(d, fmap1, fmap2, scale1, status, op16, scales, stream);
  if (err != cudaSuccess) return err;
  const float* s1 = (op16 == OP16_FP16 && scales != nullptr) ? scales + SCALE_F1 : nullptr;
  const float* s2 = (op16 == OP16_FP16 && scales != nullptr) ? scales + SCALE_F2 : nullptr;
  const dim3 block(32, 8);
  transpose_round_kernel<<<dim3((d.N1() + 31) / 32, (d.C + 31) / 32, d.B), block, 0, stream>>>(
      fmap1, F1r, d.C, d.N1(), scale1, F1h, op16, s1);
  transpose_round_kernel<<<dim3((d.N2() + 31) / 32, (d.C + 31) / 32, d.B), block, 0, stream>>>(
      fmap2, F2r, d.C, d.N2(), 1.f, F2h, op16, s2);
  if (aux != nullptr) {  // mean rows from the transposed copy (already rounded: the means differ by < 2^-12 relative)
    const dim3 grid(d.H2 + d.W2, d.B);
    f2_means_kernel<<<grid, std::min(d.C, 256), 0, stream>>>(F2r, aux, d.H2, d.W2, d.C, auxh, op16, s2);
  }
  return cudaGetLastError();
}

cudaError_t launch_prepare(const Dims& d, const float* F1, const float* F2, float* F1r, float* F2r, float* aux,
                           int* status, cudaStream_t stream, uint16_t* F1h, uint16_t* F2h, uint16_t* auxh, int op16,
                           float* scales) {
  cudaError_t err = begin_prepare(d, F1, F2, 1.f, status, op16, scales, stream);
  if (err != cudaSuccess) return err;
  const float* s1 = (op16 == OP16_FP16 && scales != nullptr) ? scales + SCALE_F1 : nullptr;
  const float* s2 = (op16 == OP16_FP16 && scales != nullptr) ? scales + SCALE_F2 : nullptr;
  const size_t n1 = (size_t)d.B * d.N1() * d.C / 4, n2 = (size_t)d.B * d.N2() * d.C / 4;  // C % 4 == 0
  const int threads = 256;
  auto blocks = [&](size_t n) { return (unsigned)std::min<size_t>((n + threads - 1) / threads, 148 * 16); };
  round_copy_kernel<<<blocks(n1), threads, 0, stream>>>(reinterpret_cast<const float4*>(F1),
                                                        reinterpret_cast<float4*>(F1r), n1,
                                                        reinterpret_cast<uint2*>(F1h), op16, s1);
  round_copy_kernel<<<blocks(n2), threads, 0, stream>>>(reinterpret_cast<const float4*>(F2),
                                                        reinterpret_cast<float4*>(F2r), n2,
                                                        reinterpret_cast<uint2*>(F2h), op16, s2);
  if (aux != nullptr) {
    const dim3 grid(d.H2 + d.W2, d.B);
    f2_means_kernel<<<grid, std::min(d.C, 256), 0, stream>>>(F2, aux, d.H2, d.W2, d.C, auxh, op16, s2);
  }
  return cudaGetLastError();
}

}  // namespace sfb
