// Correlation sweep: S = F1 * F2^T computed tile by tile on the tcgen05 tensor cores with the
// accumulator in TMEM, reduced in the epilogue so that S never reaches HBM.
//
// One CTA owns 128 consecutive image-1 pixels of one sample (the rows / TMEM lanes of every
// accumulator tile) and sweeps all image-2 pixels in tiles of SWEEP_UT x SWEEP_VT (8 rows x 16
// columns = 128 accumulator columns), column-blocks outermost.  Warp roles:
//   warp 0      TMA producer: F1 tile once (stays resident), F2 tiles through a ring of stages
//   warp 1      allocates TMEM, issues tcgen05.mma (TF32 in, FP32 accumulate), 4 accumulators in flight
//   warps 2..5  epilogue: one thread per image-1 pixel reads its accumulator lane with tcgen05.ld
// Epilogues
//   max/avg      : running column-direction max(+argmax) in registers across the inner row-block
//                  loop, row-direction max(+argmax) merged through global memory once per tile;
//                  the two mean channels come from extra tiles whose "image-2 pixels" are the
//                  row-mean and column-mean feature rows of F2 (mean_v S[u,v] = F1 . mean_v F2[u,v]).
//   compression  : C_u[k,u] = sum_v S*W_u[k,v] (reduced per tile, accumulated with red.add),
//                  C_v[k,v] = sum_u S*W_v[k,u] (register accumulators across the inner loop).
// Replaces the reference kernels MemorySaver_kernel_forward.cu:128-313, :328-533, :550-753.
#include <math_constants.h>

#include "kernels.h"
#include "sm100_primitives.cuh"

namespace sfb {

constexpr int SW_NSTAGE = 5;
constexpr int SW_NACC = 4;
constexpr int SW_TILE_N = SWEEP_UT * SWEEP_VT;  // 128 accumulator columns
constexpr int SW_THREADS = 192;
constexpr uint32_t SW_STAGE_BYTES = SW_TILE_N * KBLK * 4;
constexpr uint32_t SW_F1_BLOCK_BYTES = TILE_M * KBLK * 4;
constexpr uint32_t SW_TMEM_COLS = 512;
static_assert(SW_NACC * SW_TILE_N <= 512, "accumulators exceed TMEM");

struct SweepSmem {
  float f1[MAX_KB][TILE_M * KBLK];        // resident image-1 tile, one 128B-swizzled block per 32 channels
  float f2[SW_NSTAGE][SW_TILE_N * KBLK];  // ring of image-2 tile blocks
  uint64_t f1_full;
  uint64_t full[SW_NSTAGE];
  uint64_t empty[SW_NSTAGE];
  uint64_t acc_full[SW_NACC];
  uint64_t acc_empty[SW_NACC];
  uint32_t tmem_base;
  int abort_flag;
};
constexpr size_t SW_SMEM_BYTES = sizeof(SweepSmem) + 1024;  // + slack to align the base to 1024 B

struct SweepSched {
  int b, m0, nkb, n_ub, n_vb, t_main, t_total;
};

// ---------------------------------------------------------------------------------- producer
__device__ void sweep_producer(SweepSmem& sm, const SweepArgs& a, const SweepSched& sc, const CUtensorMap* tm_f1,
                               const CUtensorMap* tm_f2, const CUtensorMap* tm_aux) {
  mbar_expect_tx(&sm.f1_full, sc.nkb * SW_F1_BLOCK_BYTES);
  for (int kb = 0; kb < sc.nkb; ++kb) tma_load_3d(sm.f1[kb], tm_f1, &sm.f1_full, kb * KBLK, sc.m0, sc.b);
  uint32_t it = 0;
  for (int t = 0; t < sc.t_total; ++t) {
    const bool main_tile = t < sc.t_main;
    const int vb = t / sc.n_ub, ub = t - vb * sc.n_ub;
    for (int kb = 0; kb < sc.nkb; ++kb, ++it) {
      const uint32_t s = it % SW_NSTAGE, ph = (it / SW_NSTAGE) & 1u;
      if (!mbar_wait(&sm.empty[s], ph ^ 1u, &sm.abort_flag, a.status, DEV_TIMEOUT_PRODUCER)) return;
      mbar_expect_tx(&sm.full[s], SW_STAGE_BYTES);
      if (main_tile)
        tma_load_4d(sm.f2[s], tm_f2, &sm.full[s], kb * KBLK, vb * SWEEP_VT, ub * SWEEP_UT, sc.b);
      else
        tma_load_3d(sm.f2[s], tm_aux, &sm.full[s], kb * KBLK, (t - sc.t_main) * SW_TILE_N, sc.b);
    }
  }
}

// ---------------------------------------------------------------------------------- MMA issuer
__device__ void sweep_mma(SweepSmem& sm, const SweepArgs& a, const SweepSched& sc) {
  constexpr uint32_t idesc = make_idesc_tf32(TILE_M, SW_TILE_N, false, false);
  if (!mbar_wait(&sm.f1_full, 0, &sm.abort_flag, a.status, DEV_TIMEOUT_MMA)) return;
  tc_fence_after();
  uint32_t it = 0;
  for (int t = 0; t < sc.t_total; ++t) {
    const uint32_t acc = t % SW_NACC, aph = (t / SW_NACC) & 1u;
    if (!mbar_wait(&sm.acc_empty[acc], aph ^ 1u, &sm.abort_flag, a.status, DEV_TIMEOUT_MMA)) return;
    tc_fence_after();
    const uint32_t d_tmem = sm.tmem_base + acc * SW_TILE_N;
    for (int kb = 0; kb < sc.nkb; ++kb, ++it) {
      const uint32_t s = it % SW_NSTAGE, ph = (it / SW_NSTAGE) & 1u;
      if (!mbar_wait(&sm.full[s], ph, &sm.abort_flag, a.status, DEV_TIMEOUT_MMA)) return;
      tc_fence_after();
      const uint64_t adesc = make_smem_desc_sw128(smem_u32(sm.f1[kb]), 16, 1024);
      const uint64_t bdesc = make_smem_desc_sw128(smem_u32(sm.f2[s]), 16, 1024);
#pragma unroll
      for (int k = 0; k < KBLK / 8; ++k)  // one instruction consumes K = 8 TF32 values = 32 bytes of each row
        umma_tf32(d_tmem, desc_advance(adesc, k * 32), desc_advance(bdesc, k * 32), idesc, (kb | k) != 0);
      umma_commit(&sm.empty[s]);  // stage reusable once these MMAs have read it
    }
    umma_commit(&sm.acc_full[acc]);
  }
}

// ---------------------------------------------------------------------------------- epilogues
struct EpiCtx {
  int q, lane, p;
  bool valid;
  size_t row;       // b*N1 + p (0 when the lane is past the image)
  uint32_t tbase;   // TMEM address of this warp's lane quarter, column 0
};

// Waits for accumulator `t`; the result is warp-uniform so that the warp-collective tcgen05.ld that
// follows is executed by all lanes or by none.
__device__ __forceinline__ bool epi_wait(SweepSmem& sm, const SweepArgs& a, int t) {
  const uint32_t acc = t % SW_NACC, aph = (t / SW_NACC) & 1u;
  const bool ok = mbar_wait(&sm.acc_full[acc], aph, &sm.abort_flag, a.status, DEV_TIMEOUT_EPILOGUE);
  const bool all_ok = __all_sync(0xffffffffu, ok);
  if (all_ok) tc_fence_after();
  return all_ok;
}
__device__ __forceinline__ void epi_release(SweepSmem& sm, int t, int lane) {
  tc_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive(&sm.acc_empty[t % SW_NACC]);
}

template <bool ARG>
__device__ void epilogue_maxavg(SweepSmem& sm, const SweepArgs& a, const SweepSched& sc, const EpiCtx& e) {
  const int H2 = a.d.H2, W2 = a.d.W2;
  float* mau = a.ma_u + e.row * 2 * H2;
  float* mav = a.ma_v + e.row * 2 * W2;
  int32_t* amu = ARG ? a.am_u + e.row * H2 : nullptr;
  int32_t* amv = ARG ? a.am_v + e.row * W2 : nullptr;

  float cm[SWEEP_VT];
  int ca[SWEEP_VT];
  for (int t = 0; t < sc.t_main; ++t) {
    const int vb = t / sc.n_ub, ub = t - vb * sc.n_ub;
    const int v0 = vb * SWEEP_VT, u0 = ub * SWEEP_UT;
    const int nu = min(SWEEP_UT, H2 - u0), nv = min(SWEEP_VT, W2 - v0);
    if (ub == 0) {
#pragma unroll
      for (int j = 0; j < SWEEP_VT; ++j) { cm[j] = -CUDART_INF_F; ca[j] = 0; }
    }
    // row-direction state of earlier column blocks (issued before the wait to hide the latency)
    float rold[SWEEP_UT];
#pragma unroll
    for (int ul = 0; ul < SWEEP_UT; ++ul)
      rold[ul] = (e.valid && vb > 0 && ul < nu) ? mau[u0 + ul] : -CUDART_INF_F;

    if (!epi_wait(sm, a, t)) return;
    const uint32_t tacc = e.tbase + (t % SW_NACC) * SW_TILE_N;
    float rm[SWEEP_UT];
    int ra[SWEEP_UT];
#pragma unroll
    for (int ul = 0; ul < SWEEP_UT; ++ul) {
      rm[ul] = -CUDART_INF_F;
      ra[ul] = 0;
      if (ul < nu) {  // warp-uniform
        float s[SWEEP_VT];
        tmem_ld16(tacc + ul * SWEEP_VT, s);
        if (nv < SWEEP_VT) {
#pragma unroll
          for (int j = 0; j < SWEEP_VT; ++j)
            if (j >= nv) s[j] = -CUDART_INF_F;  // padded columns never win a max
        }
        float m = s[0];
        int arg = 0;
#pragma unroll
        for (int j = 1; j < SWEEP_VT; ++j) {
          if (s[j] > m) { m = s[j]; arg = j; }  // strict: lowest v wins ties
        }
        rm[ul] = m;
        ra[ul] = v0 + arg;
#pragma unroll
        for (int j = 0; j < SWEEP_VT; ++j) {
          if (s[j] > cm[j]) { cm[j] = s[j]; ca[j] = u0 + ul; }  // strict: lowest u wins ties
        }
      }
    }
    epi_release(sm, t, e.lane);
    if (e.valid) {
#pragma unroll
      for (int ul = 0; ul < SWEEP_UT; ++ul) {
        if (ul < nu && (vb == 0 || rm[ul] > rold[ul])) {
          mau[u0 + ul] = rm[ul];
          if (ARG) amu[u0 + ul] = ra[ul];
        }
      }
      if (ub == sc.n_ub - 1) {
#pragma unroll
        for (int j = 0; j < SWEEP_VT; ++j) {
          if (j < nv) {
            mav[v0 + j] = cm[j];
            if (ARG) amv[v0 + j] = ca[j];
          }
        }
      }
    }
  }
  // mean channels: accumulator column r of an aux tile is F1[p] . (row-mean u=r | column-mean v=r-H2)
  const int naux = H2 + W2;
  for (int t = sc.t_main; t < sc.t_total; ++t) {
    if (!epi_wait(sm, a, t)) return;
    const uint32_t tacc = e.tbase + (t % SW_NACC) * SW_TILE_N;
    const int rbase = (t - sc.t_main) * SW_TILE_N;
#pragma unroll
    for (int c = 0; c < SW_TILE_N / 16; ++c) {
      const int r0 = rbase + c * 16;
      if (r0 < naux) {  // warp-uniform
        float s[16];
        tmem_ld16(tacc + c * 16, s);
        if (e.valid) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int r = r0 + j;
            if (r < H2) mau[H2 + r] = s[j];
            else if (r < naux) mav[W2 + (r - H2)] = s[j];
          }
        }
      }
    }
    epi_release(sm, t, e.lane);
  }
}

template <int KC>
__device__ void epilogue_compress(SweepSmem& sm, const SweepArgs& a, const SweepSched& sc, const EpiCtx& e) {
  const int H2 = a.d.H2, W2 = a.d.W2, Kc = a.d.Kc;
  const float* wu = a.w_u + (e.row * Kc + a.k0) * W2;
  const float* wv = a.w_v + (e.row * Kc + a.k0) * H2;
  float* cu = a.c_u + (e.row * Kc + a.k0) * H2;
  float* cvo = a.c_v + (e.row * Kc + a.k0) * W2;

  float au[KC][SWEEP_VT], cv[KC][SWEEP_VT];
  for (int t = 0; t < sc.t_main; ++t) {
    const int vb = t / sc.n_ub, ub = t - vb * sc.n_ub;
    const int v0 = vb * SWEEP_VT, u0 = ub * SWEEP_UT;
    const int nu = min(SWEEP_UT, H2 - u0), nv = min(SWEEP_VT, W2 - v0);
    if (ub == 0) {
#pragma unroll
      for (int k = 0; k < KC; ++k)
#pragma unroll
        for (int j = 0; j < SWEEP_VT; ++j) {
          au[k][j] = (e.valid && j < nv) ? __ldg(wu + (size_t)k * W2 + v0 + j) : 0.f;
          cv[k][j] = 0.f;
        }
    }
    float av[KC][SWEEP_UT];
#pragma unroll
    for (int k = 0; k < KC; ++k)
#pragma unroll
      for (int ul = 0; ul < SWEEP_UT; ++ul)
        av[k][ul] = (e.valid && ul < nu) ? __ldg(wv + (size_t)k * H2 + u0 + ul) : 0.f;

    if (!epi_wait(sm, a, t)) return;
    const uint32_t tacc = e.tbase + (t % SW_NACC) * SW_TILE_N;
#pragma unroll
    for (int ul = 0; ul < SWEEP_UT; ++ul) {
      if (ul < nu) {  // warp-uniform; padded cells hold S = 0 (zero-filled F2 rows) and weight 0
        float s[SWEEP_VT];
        tmem_ld16(tacc + ul * SWEEP_VT, s);
#pragma unroll
        for (int k = 0; k < KC; ++k) {
          float r = 0.f;
#pragma unroll
          for (int j = 0; j < SWEEP_VT; ++j) {
            r = fmaf(s[j], au[k][j], r);
            cv[k][j] = fmaf(s[j], av[k][ul], cv[k][j]);
          }
          if (e.valid) {
            float* dst = cu + (size_t)k * H2 + u0 + ul;
            if (vb == 0) *dst = r;          // first column block initialises the output
            else atomicAdd(dst, r);         // later blocks accumulate (same thread, same address: ordered)
          }
        }
      }
    }
    epi_release(sm, t, e.lane);
    if (e.valid && ub == sc.n_ub - 1) {
#pragma unroll
      for (int k = 0; k < KC; ++k)
#pragma unroll
        for (int j = 0; j < SWEEP_VT; ++j)
          if (j < nv) cvo[(size_t)k * W2 + v0 + j] = cv[k][j];
    }
  }
}

// Test aid: writes the dense volume of a (small) problem so the tensor-core plumbing can be checked alone.
__device__ void epilogue_dump(SweepSmem& sm, const SweepArgs& a, const SweepSched& sc, const EpiCtx& e) {
  const int H2 = a.d.H2, W2 = a.d.W2;
  float* out = a.dump + e.row * H2 * W2;
  for (int t = 0; t < sc.t_main; ++t) {
    const int vb = t / sc.n_ub, ub = t - vb * sc.n_ub;
    const int v0 = vb * SWEEP_VT, u0 = ub * SWEEP_UT;
    const int nu = min(SWEEP_UT, H2 - u0), nv = min(SWEEP_VT, W2 - v0);
    if (!epi_wait(sm, a, t)) return;
    const uint32_t tacc = e.tbase + (t % SW_NACC) * SW_TILE_N;
#pragma unroll
    for (int ul = 0; ul < SWEEP_UT; ++ul) {
      if (ul < nu) {
        float s[SWEEP_VT];
        tmem_ld16(tacc + ul * SWEEP_VT, s);
        if (e.valid) {
#pragma unroll
          for (int j = 0; j < SWEEP_VT; ++j)
            if (j < nv) out[(size_t)(u0 + ul) * W2 + v0 + j] = s[j];
        }
      }
    }
    epi_release(sm, t, e.lane);
  }
}

// ---------------------------------------------------------------------------------- kernel
template <int MODE, int KC>
__global__ void __launch_bounds__(SW_THREADS, 1)
sweep_kernel(const __grid_constant__ CUtensorMap tm_f1, const __grid_constant__ CUtensorMap tm_f2,
             const __grid_constant__ CUtensorMap tm_aux, const SweepArgs a) {
  if (*reinterpret_cast<volatile int*>(a.status) != 0) return;  // an earlier CTA gave up: do not pile on

  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  SweepSmem& sm = *reinterpret_cast<SweepSmem*>(smem_raw + pad);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int N1 = a.d.N1();
  const int tiles_per_sample = (N1 + TILE_M - 1) / TILE_M;

  SweepSched sc;
  sc.b = blockIdx.x / tiles_per_sample;
  sc.m0 = (blockIdx.x - sc.b * tiles_per_sample) * TILE_M;
  sc.nkb = (a.d.C + KBLK - 1) / KBLK;
  sc.n_ub = (a.d.H2 + SWEEP_UT - 1) / SWEEP_UT;
  sc.n_vb = (a.d.W2 + SWEEP_VT - 1) / SWEEP_VT;
  sc.t_main = sc.n_ub * sc.n_vb;
  const bool has_aux = (MODE == SWEEP_MAXAVG || MODE == SWEEP_MAXARGAVG);
  sc.t_total = sc.t_main + (has_aux ? (a.d.H2 + a.d.W2 + SW_TILE_N - 1) / SW_TILE_N : 0);

  if (threadIdx.x == 0) {
    mbar_init(&sm.f1_full, 1);
    for (int s = 0; s < SW_NSTAGE; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    for (int i = 0; i < SW_NACC; ++i) { mbar_init(&sm.acc_full[i], 1); mbar_init(&sm.acc_empty[i], 4); }
    sm.abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tm_f1);
    prefetch_tensormap(&tm_f2);
    if (has_aux) prefetch_tensormap(&tm_aux);
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, SW_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (warp == 0) {
    if (lane == 0) sweep_producer(sm, a, sc, &tm_f1, &tm_f2, &tm_aux);
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) sweep_mma(sm, a, sc);
    __syncwarp();
  } else {
    EpiCtx e;
    e.q = warp & 3;  // tcgen05.ld lets a warp read TMEM lanes 32*(warp%4) .. +31 only
    e.lane = lane;
    e.p = sc.m0 + e.q * 32 + lane;
    e.valid = e.p < N1;
    e.row = (size_t)sc.b * N1 + (e.valid ? e.p : 0);
    e.tbase = sm.tmem_base + (static_cast<uint32_t>(e.q * 32) << 16);
    if (MODE == SWEEP_MAXAVG) epilogue_maxavg<false>(sm, a, sc, e);
    else if (MODE == SWEEP_MAXARGAVG) epilogue_maxavg<true>(sm, a, sc, e);
    else if (MODE == SWEEP_COMPRESS) epilogue_compress<KC>(sm, a, sc, e);
    else epilogue_dump(sm, a, sc, e);
  }

  tc_fence_before();
  __syncthreads();
  if (*reinterpret_cast<volatile int*>(&sm.abort_flag)) {
    // A wait ran out.  Give copies that are still in flight time to land before the CTA's shared
    // memory is released (TMA latency is a few microseconds), then free TMEM as usual.
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(sm.tmem_base, SW_TMEM_COLS);
  }
}

template <int MODE, int KC>
static cudaError_t launch_one(const SweepArgs& a, const CUtensorMap& tm_f1, const CUtensorMap& tm_f2,
                              const CUtensorMap& tm_aux, cudaStream_t stream) {
  auto kern = sweep_kernel<MODE, KC>;
  cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SW_SMEM_BYTES);
  if (err != cudaSuccess) return err;
  const int tiles_per_sample = (a.d.N1() + TILE_M - 1) / TILE_M;
  const dim3 grid(a.d.B * tiles_per_sample);
  kern<<<grid, SW_THREADS, SW_SMEM_BYTES, stream>>>(tm_f1, tm_f2, tm_aux, a);
  return cudaGetLastError();
}

cudaError_t launch_sweep(const SweepArgs& a, const CUtensorMap& tm_f1, const CUtensorMap& tm_f2,
                         const CUtensorMap& tm_aux, cudaStream_t stream) {
  switch (a.mode) {
    case SWEEP_MAXAVG: return launch_one<SWEEP_MAXAVG, 1>(a, tm_f1, tm_f2, tm_aux, stream);
    case SWEEP_MAXARGAVG: return launch_one<SWEEP_MAXARGAVG, 1>(a, tm_f1, tm_f2, tm_aux, stream);
    case SWEEP_DUMP: return launch_one<SWEEP_DUMP, 1>(a, tm_f1, tm_f2, tm_aux, stream);
    case SWEEP_COMPRESS:
      switch (a.kc) {
        case 1: return launch_one<SWEEP_COMPRESS, 1>(a, tm_f1, tm_f2, tm_aux, stream);
        case 2: return launch_one<SWEEP_COMPRESS, 2>(a, tm_f1, tm_f2, tm_aux, stream);
        case 3: return launch_one<SWEEP_COMPRESS, 3>(a, tm_f1, tm_f2, tm_aux, stream);
        case 4: return launch_one<SWEEP_COMPRESS, 4>(a, tm_f1, tm_f2, tm_aux, stream);
        default: return cudaErrorInvalidValue;
      }
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace sfb
