// Correlation sweep: S = F1 * F2^T computed tile by tile on the tcgen05 tensor cores with the
// accumulator in TMEM, reduced in the epilogue so that S never reaches HBM.
//
// One CTA owns 128 consecutive image-1 pixels of one sample (the rows / TMEM lanes of every
// accumulator tile) and sweeps all image-2 pixels in tiles of SWEEP_UT x SWEEP_VT (16 rows x 16
// columns = 256 accumulator columns), column-blocks outermost.  Warp roles:
//   warp 0      TMA producer: F1 tile once (stays resident), F2 tiles through a ring of stages
//   warp 1      allocates TMEM, issues tcgen05.mma (TF32 in, FP32 accumulate), 2 accumulators in flight
//   warps 2..   epilogue warpgroups (two, or four for the compression epilogue); in each, one thread per
//               image-1 pixel reads its accumulator lane with tcgen05.ld.  All groups consume every tile and
//               split its work.
// Everything indexed by an image-1 pixel is read and written in the packed, pixel-fastest layout
// (kernels.h), so a warp's 32 lanes touch one 128-byte line per access.
// Epilogues
//   max/avg      : group g takes tile rows 8g..8g+7.  Running column-direction max(+argmax) in
//                  registers across the inner row-block loop (the two groups' partial results are merged
//                  once per column block), row-direction max(+argmax) merged through the packed output
//                  once per tile.  The two mean channels come from extra tiles whose "image-2 pixels"
//                  are the row-mean and column-mean feature rows of F2 (mean_v S[u,v] = F1 . mean_v F2[u,v]).
//   compression  : group g takes channel g.  OU[k,u] = sum_v S*w_u[k,v] (reduced per tile, accumulated
//                  with red.add), OV[k,v] = sum_u S*w_v[k,u] (register accumulators across the inner loop).
// Replaces the reference kernels MemorySaver_kernel_forward.cu:128-313, :328-533, :550-753.
#include <math_constants.h>

#include "kernels.h"
#include "sm100_primitives.cuh"

namespace sfb {

constexpr int SW_NSTAGE = 3;                    // 3 x 32 KB of F2 blocks next to the 128 KB resident F1 tile
constexpr int SW_NACC = 2;                      // 2 x 256 TMEM columns
constexpr int SW_TILE_N = SWEEP_UT * SWEEP_VT;  // 256 accumulator columns: tcgen05.mma issues at a fixed
                                                // rate per instruction, so the widest N does the most work
// Epilogue warps: two warpgroups for the max/avg and dump epilogues (each takes half of a tile's rows), four for
// the compression epilogue (each takes one channel and reads the whole tile): its work per cell is 2 FMAs per
// channel, and with 16 warps the FP32 pipes keep up with the tensor pipe.
__host__ __device__ constexpr int sw_epi_warps(int mode) { return mode == SWEEP_COMPRESS ? 16 : 8; }
__host__ __device__ constexpr int sw_threads(int mode) { return 64 + sw_epi_warps(mode) * 32; }
constexpr int SW_RW = SWEEP_UT / 2;             // tile rows of one epilogue warpgroup
constexpr int SW_NMERGE = 4;                    // ring of column-merge barriers (> SW_NACC tiles of run-ahead)
constexpr uint32_t SW_STAGE_BYTES = SW_TILE_N * KBLK * 4;
constexpr uint32_t SW_F1_BLOCK_BYTES = TILE_M * KBLK * 4;
constexpr uint32_t SW_TMEM_COLS = 512;
static_assert(SW_NACC * SW_TILE_N <= 512, "accumulators exceed TMEM");
static_assert(SW_NMERGE > SW_NACC, "a warpgroup can run SW_NACC tiles ahead of the other");
static_assert(SW_TILE_N == 256 && SW_RW * SWEEP_VT == 128, "epilogues read two 64-column halves per warpgroup");

struct SweepSmem {
  float f1[MAX_KB][TILE_M * KBLK];        // resident image-1 tile, one 128B-swizzled block per 32 channels
  float f2[SW_NSTAGE][SW_TILE_N * KBLK];  // ring of image-2 tile blocks
  uint64_t f1_full;
  uint64_t full[SW_NSTAGE];
  uint64_t empty[SW_NSTAGE];
  uint64_t acc_full[SW_NACC];
  uint64_t acc_empty[SW_NACC];
  uint64_t merge[SW_NMERGE];              // group 1 -> group 0: partial column results are in memory
  uint32_t tmem_base;
  WaitCtl ctl;
};
constexpr size_t SW_SMEM_BYTES = sizeof(SweepSmem) + 1024;  // + slack to align the base to 1024 B

struct SweepSched {
  int b, m0, nkb, n_ub, n_vb, t_main, t_total;
};

// ---------------------------------------------------------------------------------- producer
__device__ void sweep_producer(SweepSmem& sm, const SweepArgs& a, const SweepSched& sc, const CUtensorMap* tm_f1,
                               const CUtensorMap* tm_f2, const CUtensorMap* tm_aux) {
  const int kel = a.op16 ? 2 * KBLK : KBLK;  // channels in one 128-byte row
  mbar_expect_tx(&sm.f1_full, sc.nkb * SW_F1_BLOCK_BYTES);
  for (int kb = 0; kb < sc.nkb; ++kb) tma_load_3d(sm.f1[kb], tm_f1, &sm.f1_full, kb * kel, sc.m0, sc.b);
  uint32_t it = 0;
  int vb = 0, ub = 0;
  for (int t = 0; t < sc.t_total; ++t) {
    const bool main_tile = t < sc.t_main;
    for (int kb = 0; kb < sc.nkb; ++kb, ++it) {
      const uint32_t s = it % SW_NSTAGE, ph = (it / SW_NSTAGE) & 1u;
      if (!mbar_wait(&sm.empty[s], ph ^ 1u, &sm.ctl, a.status, DEV_TIMEOUT_PRODUCER)) return;
      if (a.drop_last_load && t == sc.t_total - 1 && kb == sc.nkb - 1) return;  // test hook: this block never arrives
      mbar_expect_tx(&sm.full[s], SW_STAGE_BYTES);
      if (main_tile)
        tma_load_4d(sm.f2[s], tm_f2, &sm.full[s], kb * kel, vb * SWEEP_VT, ub * SWEEP_UT, sc.b);
      else
        tma_load_3d(sm.f2[s], tm_aux, &sm.full[s], kb * kel, (t - sc.t_main) * SW_TILE_N, sc.b);
    }
    if (++ub == sc.n_ub) { ub = 0; ++vb; }
  }
}

// ---------------------------------------------------------------------------------- MMA issuer
__device__ void sweep_mma(SweepSmem& sm, const SweepArgs& a, const SweepSched& sc) {
  constexpr uint32_t idesc_tf32 = make_idesc_tf32(TILE_M, SW_TILE_N, false, false);
  const uint32_t idesc_16 = make_idesc_op16(a.op16, TILE_M, SW_TILE_N);  // BF16 or FP16 operands
  const bool op16 = a.op16 != 0;
  if (!mbar_wait(&sm.f1_full, 0, &sm.ctl, a.status, DEV_TIMEOUT_MMA)) return;
  tc_fence_after();
  uint32_t it = 0;
  for (int t = 0; t < sc.t_total; ++t) {
    const uint32_t acc = t % SW_NACC, aph = (t / SW_NACC) & 1u;
    if (!mbar_wait(&sm.acc_empty[acc], aph ^ 1u, &sm.ctl, a.status, DEV_TIMEOUT_MMA)) return;
    tc_fence_after();
    const uint32_t d_tmem = sm.tmem_base + acc * SW_TILE_N;
    for (int kb = 0; kb < sc.nkb; ++kb, ++it) {
      const uint32_t s = it % SW_NSTAGE, ph = (it / SW_NSTAGE) & 1u;
      if (!mbar_wait(&sm.full[s], ph, &sm.ctl, a.status, DEV_TIMEOUT_MMA)) return;
      tc_fence_after();
      const uint64_t adesc = make_smem_desc_sw128(smem_u32(sm.f1[kb]), 16, 1024);
      const uint64_t bdesc = make_smem_desc_sw128(smem_u32(sm.f2[s]), 16, 1024);
      if (op16) {
#pragma unroll
        for (int k = 0; k < 4; ++k)  // one instruction consumes K = 16 16-bit values = 32 bytes of each row
          umma_bf16(d_tmem, desc_advance(adesc, k * 32), desc_advance(bdesc, k * 32), idesc_16, (kb | k) != 0);
      } else {
#pragma unroll
        for (int k = 0; k < KBLK / 8; ++k)  // one instruction consumes K = 8 TF32 values = 32 bytes of each row
          umma_tf32(d_tmem, desc_advance(adesc, k * 32), desc_advance(bdesc, k * 32), idesc_tf32, (kb | k) != 0);
      }
      umma_commit(&sm.empty[s]);  // stage reusable once these MMAs have read it
    }
    umma_commit(&sm.acc_full[acc]);
  }
}

// ---------------------------------------------------------------------------------- epilogues
struct EpiCtx {
  int wg;           // epilogue warpgroup 0 / 1
  int lane;
  int p;            // pixel index inside the sample: m0 + 32*quarter + lane
  bool valid;       // p < n_valid: lanes past the end compute but never touch memory
  uint32_t tbase;   // TMEM address of this warp's lane quarter, column 0
  float osc;        // every stored value is multiplied by this (1, or the inverse of the FP16 operands' scaling: a
                    // power of two, so the order of values and exact ties are unchanged)
};

// Waits for accumulator `t`; the result is warp-uniform so that the warp-collective tcgen05.ld that
// follows is executed by all lanes or by none.
__device__ __forceinline__ bool epi_wait(SweepSmem& sm, const SweepArgs& a, int t) {
  const uint32_t acc = t % SW_NACC, aph = (t / SW_NACC) & 1u;
  const bool ok = mbar_wait(&sm.acc_full[acc], aph, &sm.ctl, a.status, DEV_TIMEOUT_EPILOGUE);
  const bool all_ok = __all_sync(0xffffffffu, ok);
  if (all_ok) tc_fence_after();
  return all_ok;
}
__device__ __forceinline__ void epi_release(SweepSmem& sm, int t, int lane) {
  tc_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive(&sm.acc_empty[t % SW_NACC]);
}

// Maximum of 16 values and the LOWEST index holding it: pairwise tournament, the left (lower-index)
// entry survives ties.  Same comparison count as a linear scan but only four dependent steps.
__device__ __forceinline__ void max16_first(const float* r, float& m, int& arg) {
  float v8[8], v4[4], v2[2];
  int i8[8], i4[4], i2[2];
#pragma unroll
  for (int i = 0; i < 8; ++i) { const bool g = r[2 * i + 1] > r[2 * i]; v8[i] = g ? r[2 * i + 1] : r[2 * i]; i8[i] = g ? 2 * i + 1 : 2 * i; }
#pragma unroll
  for (int i = 0; i < 4; ++i) { const bool g = v8[2 * i + 1] > v8[2 * i]; v4[i] = g ? v8[2 * i + 1] : v8[2 * i]; i4[i] = g ? i8[2 * i + 1] : i8[2 * i]; }
#pragma unroll
  for (int i = 0; i < 2; ++i) { const bool g = v4[2 * i + 1] > v4[2 * i]; v2[i] = g ? v4[2 * i + 1] : v4[2 * i]; i2[i] = g ? i4[2 * i + 1] : i4[2 * i]; }
  const bool g = v2[1] > v2[0];
  m = g ? v2[1] : v2[0];
  arg = g ? i2[1] : i2[0];
}

template <bool ARG>
__device__ void epilogue_maxavg(SweepSmem& sm, const SweepArgs& a, const SweepSched& sc, const EpiCtx& e) {
  const int H2 = a.d.H2, W2 = a.d.W2;
  // per-thread views: value of (displacement d, slot) at ptr[d*sd + slot*ss]
  float* pu = a.pu.base + sc.b * a.pu.sb + e.p;
  float* pv = a.pv.base + sc.b * a.pv.sb + e.p;
  float* pua = ARG ? a.pu_arg.base + sc.b * a.pu_arg.sb + e.p : nullptr;
  float* pva = ARG ? a.pv_arg.base + sc.b * a.pv_arg.sb + e.p : nullptr;
  const uint32_t usd = a.pu.sd, uss = a.pu.ss, vsd = a.pv.sd, vss = a.pv.ss, uasd = a.pu_arg.sd, vasd = a.pv_arg.sd;
  const bool valid = e.valid;

  float cm[SWEEP_VT];
  int ca[SWEEP_VT];
  int vb = 0, ub = 0;
  for (int t = 0; t < sc.t_main; ++t) {
    const int v0 = vb * SWEEP_VT, ubase = ub * SWEEP_UT + e.wg * SW_RW;
    const int nu = min(SW_RW, H2 - ubase), nv = min(SWEEP_VT, W2 - v0);  // nu may be <= 0
    if (ub == 0) {
#pragma unroll
      for (int j = 0; j < SWEEP_VT; ++j) { cm[j] = -CUDART_INF_F; ca[j] = 0; }
    }
    // row-direction state of earlier column blocks (issued before the wait to hide the latency)
    float rold[SW_RW];
#pragma unroll
    for (int ul = 0; ul < SW_RW; ++ul)
      rold[ul] = (valid && vb > 0 && ul < nu) ? pu[(ubase + ul) * usd] : -CUDART_INF_F;

    if (!epi_wait(sm, a, t)) return;
    const uint32_t tacc = e.tbase + (t % SW_NACC) * SW_TILE_N + e.wg * (SW_RW * SWEEP_VT);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float s[64];
      tmem_ld64(tacc + half * 64, s);
      if (half == 1) epi_release(sm, t, e.lane);  // all values are in registers: hand the accumulator back
#pragma unroll
      for (int hl = 0; hl < SW_RW / 2; ++hl) {
        const int ul = half * (SW_RW / 2) + hl;
        if (ul < nu) {  // warp-uniform
          float* r = &s[hl * SWEEP_VT];
          if (nv < SWEEP_VT) {
#pragma unroll
            for (int j = 0; j < SWEEP_VT; ++j)
              if (j >= nv) r[j] = -CUDART_INF_F;  // padded columns never win a max
          }
          const int u = ubase + ul;
          float m;
          int arg;
          if (ARG) {
            max16_first(r, m, arg);
#pragma unroll
            for (int j = 0; j < SWEEP_VT; ++j) {
              if (r[j] > cm[j]) { cm[j] = r[j]; ca[j] = u; }  // strict: lowest u of this group wins ties
            }
          } else {
            m = r[0];
            arg = 0;
#pragma unroll
            for (int j = 1; j < SWEEP_VT; ++j) m = fmaxf(m, r[j]);
#pragma unroll
            for (int j = 0; j < SWEEP_VT; ++j) cm[j] = fmaxf(cm[j], r[j]);
          }
          m *= e.osc;  // memory holds scaled-back values; compare and store in that domain
          if (valid && (vb == 0 || m > rold[ul])) {  // strict: the lowest column block wins ties
            pu[u * usd] = m;
            if (ARG) pua[u * uasd] = __int_as_float(v0 + arg);
          }
        }
      }
    }
    if (ub == sc.n_ub - 1) {
      // end of a column block: group 1 publishes its partial column maxima, group 0 merges and stores
      uint64_t* bar = &sm.merge[vb % SW_NMERGE];
      if (e.wg == 1) {
#pragma unroll
        for (int j = 0; j < SWEEP_VT; ++j) {
          if (valid && j < nv) {
            pv[(v0 + j) * vsd] = cm[j] * e.osc;
            if (ARG) pva[(v0 + j) * vasd] = __int_as_float(ca[j]);
          }
        }
        __threadfence_block();
        __syncwarp();
        if (e.lane == 0) mbar_arrive(bar);
      } else {
        const bool ok = mbar_wait(bar, (vb / SW_NMERGE) & 1u, &sm.ctl, a.status, DEV_TIMEOUT_EPILOGUE);
        if (!__all_sync(0xffffffffu, ok)) return;
#pragma unroll
        for (int j = 0; j < SWEEP_VT; ++j) {
          if (valid && j < nv) {
            float* dst = pv + (v0 + j) * vsd;
            const float om = __ldcg(dst);
            float best = cm[j] * e.osc;
            int besta = ca[j];
            if (ARG) {
              float* dsta = pva + (v0 + j) * vasd;
              const int oa = __float_as_int(__ldcg(dsta));
              if (om > best || (om == best && oa < besta)) { best = om; besta = oa; }  // lowest u on ties
              *dsta = __int_as_float(besta);
            } else {
              best = fmaxf(best, om);
            }
            dst[0] = best;
          }
        }
      }
    }
    if (++ub == sc.n_ub) { ub = 0; ++vb; }
  }
  // mean channels: accumulator column r of an aux tile is F1[p] . (row-mean u=r | column-mean v=r-H2)
  const int naux = H2 + W2;
  for (int t = sc.t_main; t < sc.t_total; ++t) {
    if (!epi_wait(sm, a, t)) return;
    const uint32_t tacc = e.tbase + (t % SW_NACC) * SW_TILE_N + e.wg * 128;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r0 = (t - sc.t_main) * SW_TILE_N + e.wg * 128 + half * 64;
      if (r0 < naux) {  // warp-uniform
        float s[64];
        tmem_ld64(tacc + half * 64, s);
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const int r = r0 + j;
          if (!valid) continue;
          if (r < H2) pu[r * usd + uss] = s[j] * e.osc;
          else if (r < naux) pv[(r - H2) * vsd + vss] = s[j] * e.osc;
        }
      }
    }
    epi_release(sm, t, e.lane);
  }
}

__device__ void epilogue_compress(SweepSmem& sm, const SweepArgs& a, const SweepSched& sc, const EpiCtx& e) {
  const int H2 = a.d.H2, W2 = a.d.W2;
  const bool active = e.wg < a.kc;            // this warpgroup's channel exists (warp-uniform)
  const bool valid = e.valid && active;
  const uint32_t xusd = a.xu.sd, xvsd = a.xv.sd, ousd = a.ou.sd, ovsd = a.ov.sd;
  // this thread's pixel and channel in sample b of each view; displacement d at ptr[d*sd], 32-bit offsets
  const int k = a.k0 + e.wg;
  const float* wu = a.xv.base + sc.b * a.xv.sb + e.p + (a.wu_slot0 + k * a.w_stride) * a.xv.ss;  // w_u[k][v]
  const float* wv = a.xu.base + sc.b * a.xu.sb + e.p + (a.wv_slot0 + k * a.w_stride) * a.xu.ss;  // w_v[k][u]
  float* ou = a.ou.base + sc.b * a.ou.sb + e.p + k * a.ou.ss;
  float* ov = a.ov.base + sc.b * a.ov.sb + e.p + k * a.ov.ss;

  // Both sums run on packed FP32 pairs (two neighbouring columns per fma.rn.f32x2), which halves the
  // instructions per cell: the epilogue warps share their schedulers' issue slots, and with scalar FMAs
  // those slots, not the tensor pipe, set the pace of this sweep.
  //   au2[j] = (w_u[v0+2j], w_u[v0+2j+1])         weights of this column block, per column pair
  //   cv2[j] = running (OV[v0+2j], OV[v0+2j+1])   over the rows of the column block
  // Cells outside the image hold S = 0 (TMA zero-fills the missing F2 rows) and get weight 0, so every
  // tile is processed whole and only the loads and stores at the edges are predicated.
  uint64_t au2[SWEEP_VT / 2], cv2[SWEEP_VT / 2];
  int vb = 0, ub = 0;
  for (int t = 0; t < sc.t_main; ++t) {
    const int v0 = vb * SWEEP_VT, u0 = ub * SWEEP_UT;
    const int nu = min(SWEEP_UT, H2 - u0), nv = min(SWEEP_VT, W2 - v0);
    if (ub == 0) {
      const float* wu_t = wu + v0 * xvsd;
#pragma unroll
      for (int j = 0; j < SWEEP_VT / 2; ++j) {
        const float lo = (valid && 2 * j < nv) ? __ldg(wu_t + (2 * j) * xvsd) : 0.f;
        const float hi = (valid && 2 * j + 1 < nv) ? __ldg(wu_t + (2 * j + 1) * xvsd) : 0.f;
        au2[j] = pack2(lo, hi);
        cv2[j] = 0ull;
      }
    }
    float av[SWEEP_UT];
    {
      const float* wv_t = wv + u0 * xusd;
#pragma unroll
      for (int ul = 0; ul < SWEEP_UT; ++ul) av[ul] = (valid && ul < nu) ? __ldg(wv_t + ul * xusd) : 0.f;
    }

    if (!epi_wait(sm, a, t)) return;
    const uint32_t tacc = e.tbase + (t % SW_NACC) * SW_TILE_N;
    if (active) {
      float* ou_t = ou + u0 * ousd;
      const bool first = vb == 0;  // the first column block initialises the output, later ones accumulate
#pragma unroll
      for (int pr = 0; pr < SWEEP_UT / 2; ++pr) {
        float s[2 * SWEEP_VT];
        tmem_ld32(tacc + pr * 2 * SWEEP_VT, s);
        if (pr == SWEEP_UT / 2 - 1) epi_release(sm, t, e.lane);  // last read of this tile
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int ul = 2 * pr + h;
          const uint64_t av2 = pack2(av[ul], av[ul]);
          uint64_t r2 = 0ull;
#pragma unroll
          for (int j = 0; j < SWEEP_VT / 2; ++j) {
            const uint64_t s2 = pack2(s[h * SWEEP_VT + 2 * j], s[h * SWEEP_VT + 2 * j + 1]);
            r2 = j == 0 ? mul2(s2, au2[0]) : fma2(s2, au2[j], r2);
            cv2[j] = fma2(s2, av2, cv2[j]);
          }
          if (valid && ul < nu) {
            float* dst = ou_t + ul * ousd;
            const float r = sum2(r2) * e.osc;
            if (first) *dst = r;
            else atomicAdd(dst, r);  // same thread, same address in every column block: ordered
          }
        }
      }
    } else {
      epi_release(sm, t, e.lane);
    }
    if (ub == sc.n_ub - 1) {
      float* ov_t = ov + v0 * ovsd;
#pragma unroll
      for (int j = 0; j < SWEEP_VT / 2; ++j) {
        float lo, hi;
        unpack2(cv2[j], lo, hi);
        if (valid && 2 * j < nv) ov_t[(2 * j) * ovsd] = lo * e.osc;
        if (valid && 2 * j + 1 < nv) ov_t[(2 * j + 1) * ovsd] = hi * e.osc;
      }
    }
    if (++ub == sc.n_ub) { ub = 0; ++vb; }
  }
}

// Test aid: writes the dense volume of a (small) problem so the tensor-core plumbing can be checked alone.
__device__ void epilogue_dump(SweepSmem& sm, const SweepArgs& a, const SweepSched& sc, const EpiCtx& e) {
  const int H2 = a.d.H2, W2 = a.d.W2, N1 = a.d.N1();
  const bool valid = e.p < N1;
  float* out = a.dump + ((size_t)sc.b * N1 + (valid ? e.p : 0)) * H2 * W2;
  int vb = 0, ub = 0;
  for (int t = 0; t < sc.t_main; ++t) {
    const int v0 = vb * SWEEP_VT, ubase = ub * SWEEP_UT + e.wg * SW_RW;
    const int nu = min(SW_RW, H2 - ubase), nv = min(SWEEP_VT, W2 - v0);
    if (!epi_wait(sm, a, t)) return;
    const uint32_t tacc = e.tbase + (t % SW_NACC) * SW_TILE_N + e.wg * 128;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float s[64];
      tmem_ld64(tacc + half * 64, s);
      if (half == 1) epi_release(sm, t, e.lane);
      if (valid) {
#pragma unroll
        for (int hl = 0; hl < SW_RW / 2; ++hl)
#pragma unroll
          for (int j = 0; j < SWEEP_VT; ++j) {
            const int ul = half * (SW_RW / 2) + hl;
            if (ul < nu && j < nv) out[(size_t)(ubase + ul) * W2 + v0 + j] = s[hl * SWEEP_VT + j] * e.osc;
          }
      }
    }
    if (++ub == sc.n_ub) { ub = 0; ++vb; }
  }
}

// ---------------------------------------------------------------------------------- kernel
template <int MODE>
__global__ void __launch_bounds__(sw_threads(MODE), 1)
sweep_kernel(const __grid_constant__ CUtensorMap tm_f1, const __grid_constant__ CUtensorMap tm_f2,
             const __grid_constant__ CUtensorMap tm_aux, const SweepArgs a) {
  if (*reinterpret_cast<volatile int*>(a.status) != 0) return;  // an earlier CTA gave up: do not pile on

  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (1024u - (smem_u32(smem_raw) & 1023u)) & 1023u;
  SweepSmem& sm = *reinterpret_cast<SweepSmem*>(smem_raw + pad);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_per_sample = (a.d.N1() + TILE_M - 1) / TILE_M;

  SweepSched sc;
  sc.b = blockIdx.x / tiles_per_sample;
  sc.m0 = (blockIdx.x - sc.b * tiles_per_sample) * TILE_M;
  sc.nkb = a.op16 ? (a.d.C + 2 * KBLK - 1) / (2 * KBLK) : (a.d.C + KBLK - 1) / KBLK;
  sc.n_ub = (a.d.H2 + SWEEP_UT - 1) / SWEEP_UT;
  sc.n_vb = (a.d.W2 + SWEEP_VT - 1) / SWEEP_VT;
  sc.t_main = sc.n_ub * sc.n_vb;
  const bool has_aux = (MODE == SWEEP_MAXAVG || MODE == SWEEP_MAXARGAVG);
  sc.t_total = sc.t_main + (has_aux ? (a.d.H2 + a.d.W2 + SW_TILE_N - 1) / SW_TILE_N : 0);

  if (threadIdx.x == 0) {
    mbar_init(&sm.f1_full, 1);
    for (int s = 0; s < SW_NSTAGE; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    for (int i = 0; i < SW_NACC; ++i) { mbar_init(&sm.acc_full[i], 1); mbar_init(&sm.acc_empty[i], sw_epi_warps(MODE)); }
    for (int i = 0; i < SW_NMERGE; ++i) mbar_init(&sm.merge[i], 4);  // the four warps of max/avg group 1
    wait_ctl_init(&sm.ctl, a.wait_limit_ns);
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
    const int q = warp & 3;  // tcgen05.ld lets a warp read TMEM lanes 32*(warp%4) .. +31 only
    e.wg = (warp - 2) >> 2;
    e.lane = lane;
    e.p = sc.m0 + q * 32 + lane;
    e.valid = e.p < a.n_valid;
    e.tbase = sm.tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    e.osc = a.out_scale != nullptr ? __ldg(a.out_scale) : 1.f;
    if (MODE == SWEEP_MAXAVG) epilogue_maxavg<false>(sm, a, sc, e);
    else if (MODE == SWEEP_MAXARGAVG) epilogue_maxavg<true>(sm, a, sc, e);
    else if (MODE == SWEEP_COMPRESS) epilogue_compress(sm, a, sc, e);
    else epilogue_dump(sm, a, sc, e);
  }

  tc_fence_before();
  __syncthreads();
  if (wait_ctl_aborted(&sm.ctl)) {
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

template <int MODE>
static cudaError_t launch_one(const SweepArgs& a, const CUtensorMap& tm_f1, const CUtensorMap& tm_f2,
                              const CUtensorMap& tm_aux, cudaStream_t stream) {
  auto kern = sweep_kernel<MODE>;
  static DeviceOnce configured;  // the attribute is per device and stays set
  cudaError_t err = configured.run([&] {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SW_SMEM_BYTES);
  });
  if (err != cudaSuccess) return err;
  const int tiles_per_sample = (a.d.N1() + TILE_M - 1) / TILE_M;
  const dim3 grid(a.d.B * tiles_per_sample);
  kern<<<grid, sw_threads(MODE), SW_SMEM_BYTES, stream>>>(tm_f1, tm_f2, tm_aux, a);
  return cudaGetLastError();
}

cudaError_t launch_sweep(const SweepArgs& a, const CUtensorMap& tm_f1, const CUtensorMap& tm_f2,
                         const CUtensorMap& tm_aux, cudaStream_t stream) {
  switch (a.mode) {
    case SWEEP_MAXAVG: return launch_one<SWEEP_MAXAVG>(a, tm_f1, tm_f2, tm_aux, stream);
    case SWEEP_MAXARGAVG: return launch_one<SWEEP_MAXARGAVG>(a, tm_f1, tm_f2, tm_aux, stream);
    case SWEEP_DUMP: return launch_one<SWEEP_DUMP>(a, tm_f1, tm_f2, tm_aux, stream);
    case SWEEP_COMPRESS:
      if (a.kc < 1 || a.kc > KC_MAX_PER_SWEEP) return cudaErrorInvalidValue;
      return launch_one<SWEEP_COMPRESS>(a, tm_f1, tm_f2, tm_aux, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace sfb
