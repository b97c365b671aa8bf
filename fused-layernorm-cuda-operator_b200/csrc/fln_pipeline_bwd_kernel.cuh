// Pipelined backward: the kernel, the fused column reduce in its tail and the launch helper.
// See fln_pipeline.cuh for the ring.  The kernel is instantiated in three translation units:
// fln_pipeline_bwd.cu (16-byte vectors, a power-of-two number per thread, and the entry point),
// fln_pipeline_bwd_odd.cu (odd numbers of vectors, short vectors) and fln_pipeline_bwd_pair.cu
// (a row shared by the two CTAs of a cluster; rows whose last vector is ragged).
#pragma once
#include <atomic>

#include "fln_pipeline.cuh"

namespace fln {

// ----------------------------------------------------------------------------------------
// Fused column reduce, the tail of the pipelined backward.  The partial rows were written a
// moment ago and sit in L2; after the grid barrier CTA q sums columns [128 q, 128 q + 128)
// over all partial rows: a warp per 512-byte row segment, the rows split over the 16 warps,
// every thread's (up to ten) 16-byte loads issued before its first add, then the 16 warps
// combined through the now idle stage memory `sb` (16 x 128 floats).  The order of the adds
// is fixed, so the sums are reproducible.  Kept out of line so that the register allocation
// of the streaming loop does not depend on it.  A CTA that gave up in the streaming loop
// (`aborted`) only counts itself in and out, so that the others do not wait for it.
// ----------------------------------------------------------------------------------------
struct ReduceArgs {
  const float* partials;
  unsigned long long* sync;
  unsigned long long token;
  float* dgb_f32;
  void* dgamma;
  void* dbeta;
  int cols;
  int P;  // partial rows
  unsigned long long wait_ns;
  int* status;
  const int* fault;
};
template <typename T, int NR>
__device__ __noinline__ void fused_column_reduce(const ReduceArgs p, float* sb, bool aborted) {
  const int tid = threadIdx.x;
  __syncthreads();
  bool met = !aborted;
  if (tid == 0) {
    grid_arrive(p.sync);
    if (!aborted) {
      const unsigned int expect = gridDim.x + ((*p.fault & 2) != 0 ? 1u : 0u);  // test hook
      met = grid_wait(p.sync, p.token, expect, p.wait_ns);
      if (!met) atomicOr(p.status, 2);
    }
  }
  if (!__syncthreads_and(met ? 1 : 0)) {
    if (tid == 0) grid_depart(p.sync, gridDim.x);
    return;
  }
  const int ncols = NR * p.cols;
  const int n4 = ncols >> 2;
  const int P = p.P;
  const int cl = tid & 31, rg = tid >> 5;
  for (int q = blockIdx.x; q * 32 < n4; q += gridDim.x) {
    const int c4 = q * 32 + cl;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c4 < n4 && rg < 16) {
      const float4* __restrict__ src = reinterpret_cast<const float4*>(p.partials) + c4;
      for (int base = rg; base < P; base += 160) {
        float4 v[10];
#pragma unroll
        for (int j = 0; j < 10; ++j) {
          const int idx = base + j * 16;
          v[j] = idx < P ? __ldcg(src + (int64_t)idx * n4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 10; ++j) {
          acc.x += v[j].x;
          acc.y += v[j].y;
          acc.z += v[j].z;
          acc.w += v[j].w;
        }
      }
    }
    if (rg < 16) *reinterpret_cast<float4*>(sb + rg * 128 + cl * 4) = acc;
    __syncthreads();
    const int c = q * 128 + tid;
    if (tid < 128 && c < ncols) {
      float t = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) t += sb[i * 128 + tid];
      if (p.dgb_f32 != nullptr) p.dgb_f32[c] = t;
      if (c < p.cols) {
        if (p.dgamma != nullptr) reinterpret_cast<T*>(p.dgamma)[c] = Cvt<T>::from_f(t);
      } else {
        if (p.dbeta != nullptr) reinterpret_cast<T*>(p.dbeta)[c - p.cols] = Cvt<T>::from_f(t);
      }
    }
    __syncthreads();
  }
  if (tid == 0) grid_depart(p.sync, gridDim.x);
}

// ----------------------------------------------------------------------------------------
// backward (stage 1: dx and per-CTA partial sums of dgamma / dbeta)
//
// Per pair of elements, on register pairs: two widening shifts and two masks, xhat as one fma,
// g = dy * gamma, two running sums, then dx = rstd * ((g - c2) - xhat * c1) and the two column
// accumulators.
//
// Each staged tensor has its own producer thread, in a warp of its own (thread 0: dy, thread
// 32: x, thread 64: the residual-stream gradient): issuing a bulk copy holds the issuing warp
// for some 160 cycles and all warps of the CTA move in step, so two copies issued by one
// thread put twice that in front of every row (128.1 vs 131.9 us at 16384 x 8192 bf16).
// ----------------------------------------------------------------------------------------
// DRES: an incoming gradient of the residual stream (same shape as dx) is staged as a third
// tensor and added into dx; each thread parks its (still packed) part in registers before the
// barrier that releases the stage.
// LT >= 0: geometry known at compile time (a CTA of 512 threads, 2^LT threads per row, rows of
// exactly K * VEC * 2^LT elements), as in the forward: 15.1 instead of 19.9 instructions per
// element for bf16 at 16384 x 8192.
// PAIR: launched as clusters of two CTAs that share every row: CTA `rank` of the cluster stages
// and differentiates columns [rank * cols, rank * cols + cols) of a row of 2 * cols (cols = the
// half row, K * VEC * 512: one row per tile, 512 threads per half row).  The two partial row
// sums of each CTA's 16 warps go into the partner's shared memory as well, by st.async counted
// on an mbarrier of the partner (two of them, rows alternate): a CTA waits -- bounded like every
// wait here -- for the partner's 16 x NR values of the row, then meets its own threads at the
// CTA barrier as every other instantiation does, and both CTAs add the 32 values of a sum in
// the same order.  Nothing in the row loop fences: the cluster barrier (arrive.release) that
// an earlier form used per row also waited for the dx stores of the row before, 0.5 us a row.
// A CTA that gives up stops sending; its partner's wait then runs out as well.
// TAIL: rows whole, every vector whole except the last of a thread's K (rows that fit no exact
// plan, 1600 columns); the row length comes from the launch parameters, the split from LT.
// BSM: the per-thread column sums of dy (dbeta) live in shared memory behind the stages, one
// float2 per thread and column pair (consecutive threads consecutive 8-byte words: conflict
// free), instead of in registers.  For the 24-column plans of 16-bit LayerNorm (12288 columns):
// with 48 accumulator registers besides gamma and the row itself the kernel ran at 5000 GB/s,
// RMSNorm (24 accumulators) at 6400 on the same plan.
template <typename T, int K, int KIND, bool FULL, bool FUSE, bool DRES, int VB = 16, int LT = -1, bool PAIR = false,
          bool TAIL = false, bool BSM = false>
__global__ void __launch_bounds__(512) norm_bwd_pipe_kernel(const BwdParams p, const PipeGeom g) {
  constexpr int VEC = VB / sizeof(T);  // even
  constexpr int V2 = VEC / 2;
  constexpr int NR = KIND == FLN_LAYERNORM ? 2 : 1;
  constexpr int NPROD = DRES ? 3 : 2;
  constexpr bool CT = LT >= 0;
  constexpr int LTC = CT ? LT : 0;
  static_assert(!CT || FULL, "compile-time geometry is for the FULL kernel");
  static_assert(!TAIL || CT, "the ragged-last-vector kernel: split at compile time");
// vector k of this thread lies in the row: known at compile time except for the last of a TAIL plan
#define FLN_WHOLE(k) (FULL && !(TAIL && (k) == K - 1))
  static_assert(!PAIR || (LT == 9 && !FUSE && !DRES), "a shared row: 512 threads per half row, plain stage 1");
  static_assert(!BSM || (KIND == FLN_LAYERNORM && CT && !PAIR), "dbeta sums in shared memory: LayerNorm, 512 threads");
  const int tpr = CT ? (1 << LTC) : g.tpr;
  const int log2_tpr = CT ? LTC : g.log2_tpr;
  const int R = CT ? (512 >> LTC) : g.R;
  // (a shared ragged row: this CTA's half of it)
  const int cols = (CT && !TAIL) ? ((K * VEC) << LTC) : (PAIR ? p.cols >> 1 : p.cols);
  const uint32_t row_bytes = (CT && !TAIL) ? (uint32_t)((K * VB) << LTC) : g.row_bytes;
  const uint32_t second_off = CT ? row_bytes * (uint32_t)R : g.second_off;
  const uint32_t stage_stride = CT ? second_off * (uint32_t)NPROD : g.stage_stride;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* xbar = reinterpret_cast<uint64_t*>(smem + 192);  // PAIR: the partner's sums of even / odd rows land here
  float* s_red = reinterpret_cast<float*>(smem + 256);  // 2 x 64 floats (PAIR: 2 x [2 ranks][64])
  unsigned char* stages = smem + kSmemHeader;

  const int tid = threadIdx.x;
  const int lane_r = tid & (tpr - 1);
  const int r_in = tid >> log2_tpr;
  const int S = g.S;
  // row slots of the static split: CTAs, or clusters when two CTAs share a row
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  // Measured, not derived: the 16-bit kernels are a third slower (16384 x 8192 bf16: 177 against
  // 133 us) when the slot and the slot count live in registers across the row loop instead of
  // being read from the special registers at each use, and the fp32 kernels are a tenth faster
  // (16384 x 8192: 239 against 266 us).  Register counts are the same within three either way.
  constexpr bool HOLD = sizeof(T) == 4;
  const int slot_r = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int nslot_r = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
#define FLN_SLOT (HOLD ? (int64_t)slot_r : (int64_t)(PAIR ? (blockIdx.x >> 1) : blockIdx.x))
#define FLN_NSLOT (HOLD ? (int64_t)nslot_r : (int64_t)(PAIR ? (gridDim.x >> 1) : gridDim.x))
  const int ld = PAIR ? 2 * cols : cols;            // elements from one row to the next
  const int coff = PAIR ? (int)rank * cols : 0;     // first column of this CTA
  const int64_t n_tiles = (p.rows + R - 1) / R;
  const int my_tiles = (int64_t)FLN_SLOT < n_tiles ? (int)((n_tiles - FLN_SLOT + FLN_NSLOT - 1) / FLN_NSLOT) : 0;
  const float inv_n = 1.0f / (float)ld;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&full[s], NPROD);
    if (PAIR) {
      mbar_init(&xbar[0], 1);
      mbar_init(&xbar[1], 1);
    }
    mbar_init_fence();
    if (PAIR) {
      mbar_expect_tx(&xbar[0], 16u * NR * 4u);
      mbar_expect_tx(&xbar[1], 16u * NR * 4u);
    }
  }
  if (FUSE && tid == 96) grid_barrier_init(p.sync, p.token);
  if (PAIR) cluster_sync_all();  // the partner's barriers exist before anything remote happens
  else __syncthreads();

  // producer `which` (0: dy, 1: x, 2: dres_in) arms stage s with its share of tile i
  const int which = tid >> 5;
  const bool is_producer = (tid & 31) == 0 && which < NPROD;
  auto issue = [&](int i, int s, bool skip_copy) {
    const int64_t row0 = ((int64_t)FLN_SLOT + (int64_t)i * FLN_NSLOT) * R;
    const int64_t left = p.rows - row0;
    const uint32_t bytes = (uint32_t)(left < R ? left : R) * row_bytes;
    unsigned char* dst = stages + (size_t)s * stage_stride + (size_t)which * second_off;
    const T* src = reinterpret_cast<const T*>(which == 0 ? p.dy : (which == 1 ? p.x : p.dres_in));
    mbar_expect_tx(&full[s], bytes);
    if (!skip_copy) bulk_g2s(dst, src + row0 * ld + coff, bytes, &full[s]);
  };
  if (is_producer) {
    // test hook (fln_set_test_fault bit 0): CTA 0 arms its first stage without the dy copy
    const bool fault = tid == 0 && blockIdx.x == 0 && (*p.fault & 1) != 0;
    const int pre = my_tiles < S ? my_tiles : S;
    for (int i = 0; i < pre; ++i) issue(i, i, fault && i == 0);
  }

  float2 acc_g[K][V2], acc_b[BSM ? 1 : K][BSM ? 1 : V2], gam[K][V2];
  float2* s_accb = reinterpret_cast<float2*>(stages + (size_t)g.S * stage_stride) + tid;  // BSM: [K * V2][512]
  bool vok[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int iv = lane_r + k * tpr;
    vok[k] = FLN_WHOLE(k) ? true : iv < (PAIR ? p.nv >> 1 : p.nv);
#pragma unroll
    for (int e = 0; e < V2; ++e) {
      acc_g[k][e] = f2(0.f);
      if constexpr (BSM) s_accb[(k * V2 + e) * 512] = f2(0.f);
      else acc_b[k][e] = f2(0.f);
      gam[k][e] = f2(1.f);
    }
    if (p.gamma != nullptr && vok[k])
      unpack2<T, VEC>(ld_param<T, VEC>(reinterpret_cast<const T*>(p.gamma) + coff + (int64_t)iv * VEC), gam[k]);
  }

  // per-row statistics of the next tile are fetched one iteration ahead
  int64_t row = (int64_t)FLN_SLOT * R + r_in;
  const int64_t row_step = (int64_t)FLN_NSLOT * R;
  float mean_n = 0.f, rstd_n = 0.f;
  if (my_tiles > 0 && row < p.rows) {
    if (KIND == FLN_LAYERNORM) mean_n = __ldg(p.mean + row);
    rstd_n = __ldg(p.rstd + row);
  }

  int s = 0;
  uint32_t phase = 0;
  bool aborted = false;
  const uint32_t my_off = (uint32_t)r_in * row_bytes + (uint32_t)lane_r * (uint32_t)VB;
  const uint32_t k_off = (uint32_t)tpr * (uint32_t)VB;
  int i = 0;
  for (; i < my_tiles; ++i, row += row_step) {
    const bool row_ok = FULL ? true : row < p.rows;
    const float mean = mean_n, rstd = rstd_n;
    if (i + 1 < my_tiles) {
      const int64_t rown = row + row_step;
      mean_n = 0.f;
      rstd_n = 0.f;
      if (rown < p.rows) {
        if (KIND == FLN_LAYERNORM) mean_n = __ldg(p.mean + rown);
        rstd_n = __ldg(p.rstd + rown);
      }
    }
    const bool landed = mbar_wait_bounded(&full[s], phase, p.wait_ns);
    const unsigned char* st = stages + (size_t)s * stage_stride + my_off;
    // 16-bit inputs: xhat as ONE fma, x * rstd - mean * rstd.  The rounding of mean * rstd
    // costs 2^-24 |mean| / std in xhat, and 16-bit data cannot hold |mean| / std beyond 2^11,
    // so this stays three orders below the output's own rounding.  fp32 keeps (x - mean) * rstd.
    const float2 r2 = f2(rstd);
    const float2 nmr = f2(-mean * rstd), nm = f2(-mean);

    float2 xh[K][V2], dyf[K][V2];
    Pack<T, VEC> dres[DRES ? K : 1];
    float2 r0 = f2(0.f), r1 = f2(0.f);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (FLN_WHOLE(k) || (row_ok && vok[k])) {
        unpack2<T, VEC>(stage_vec<T, VEC>(st + k * k_off), dyf[k]);
        unpack2<T, VEC>(stage_vec<T, VEC>(st + second_off + k * k_off), xh[k]);
        if (DRES) dres[k] = stage_vec<T, VEC>(st + 2 * second_off + k * k_off);
#pragma unroll
        for (int e = 0; e < V2; ++e)
          xh[k][e] = sizeof(T) == 2 ? f2fma(xh[k][e], r2, nmr) : f2mul(f2add(xh[k][e], nm), r2);
      } else {
#pragma unroll
        for (int e = 0; e < V2; ++e) {
          dyf[k][e] = f2(0.f);
          xh[k][e] = f2(0.f);
        }
      }
#pragma unroll
      for (int e = 0; e < V2; ++e) {
        const float2 gg = f2mul(dyf[k][e], gam[k][e]);
        r0 = f2fma(gg, xh[k][e], r0);
        if (KIND == FLN_LAYERNORM) r1 = f2add(r1, gg);
      }
    }
    float red[NR];
    red[0] = r0.x + r0.y;
    if (KIND == FLN_LAYERNORM) red[NR - 1] = r1.x + r1.y;
    float* sr = s_red + (i & 1) * (PAIR ? 128 : 64);
    if constexpr (PAIR) {
      // the warp's sums into this CTA's half of the table and into the partner's copy of it
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int n = 0; n < NR; ++n) red[n] += __shfl_xor_sync(0xffffffffu, red[n], off);
      }
      if ((tid & 31) == 0) {
        float* mine = sr + rank * 64 + (tid >> 5);
        const uint32_t theirs = map_to_cta(mine, rank ^ 1u);
        const uint32_t their_bar = map_to_cta(&xbar[i & 1], rank ^ 1u);
#pragma unroll
        for (int n = 0; n < NR; ++n) {
          mine[n * 32] = red[n];
          st_async_f32(theirs + n * 32 * 4, red[n], their_bar);
        }
      }
      // the column sums do not need the row sums: they go here, under the exchange's latency
#pragma unroll
      for (int k = 0; k < K; ++k) {
#pragma unroll
        for (int e = 0; e < V2; ++e) {
          acc_g[k][e] = f2fma(dyf[k][e], xh[k][e], acc_g[k][e]);
          if constexpr (BSM) s_accb[(k * V2 + e) * 512] = f2add(s_accb[(k * V2 + e) * 512], dyf[k][e]);
          else if (KIND == FLN_LAYERNORM) acc_b[k][e] = f2add(acc_b[k][e], dyf[k][e]);
        }
      }
      const bool theirs_landed = mbar_wait_bounded(&xbar[i & 1], (uint32_t)(i >> 1) & 1u, p.wait_ns);
      if (!__syncthreads_and(landed && theirs_landed ? 1 : 0)) {
        aborted = true;
        break;
      }
      // the partner sends row i + 2 only after it has this CTA's row i + 1, which every warp
      // here sends after reading the sums of row i: the table and the barrier are free again
      if (tid == 0 && i + 2 < my_tiles) mbar_expect_tx(&xbar[i & 1], 16u * NR * 4u);
      if (is_producer && i + S < my_tiles) issue(i + S, s, false);
#pragma unroll
      for (int n = 0; n < NR; ++n) red[n] = sum_w<16>(sr + n * 32) + sum_w<16>(sr + 64 + n * 32);
    } else {
      rowsum_warp<NR>(red, tpr, sr);
      if (!__syncthreads_and(landed ? 1 : 0)) {
        aborted = true;
        break;
      }
      if (is_producer && i + S < my_tiles) issue(i + S, s, false);
      rowsum_cta<NR>(red, tpr, sr);
    }
    // dx = rstd * ((g - c2) - xhat * c1): the subtraction comes first so that rows whose g
    // is (nearly) constant cancel exactly instead of leaving a rounding residue times rstd
    const float2 nc1 = f2(-(red[0] * inv_n));
    const float c2s = KIND == FLN_LAYERNORM ? red[NR - 1] * inv_n : 0.f;
    const float2 nc2 = f2(-c2s);

    if (p.dx != nullptr) {
      T* __restrict__ dxr = reinterpret_cast<T*>(p.dx) + row * (int64_t)ld + coff + (int64_t)lane_r * VEC;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        if (FLN_WHOLE(k) || (row_ok && vok[k])) {
          float2 o[V2];
#pragma unroll
          for (int e = 0; e < V2; ++e) {
            // the product of two 16-bit values is exact in fp32, so the fma equals
            // (dy * gamma) - c2 bit for bit there and saves the multiply
            const float2 gc =
                sizeof(T) == 2 ? f2fma(dyf[k][e], gam[k][e], nc2) : f2add(f2mul(dyf[k][e], gam[k][e]), nc2);
            o[e] = f2mul(r2, f2fma(xh[k][e], nc1, gc));
          }
          if (DRES) {
            float2 dr[V2];
            unpack2<T, VEC>(dres[k], dr);
#pragma unroll
            for (int e = 0; e < V2; ++e) o[e] = f2add(o[e], dr[e]);
          }
          Pack<T, VEC> out;
          pack2<T, VEC>(o, out);
          st_stream<T, VEC>(dxr + (int64_t)k * tpr * VEC, out);
        }
      }
    }
    if constexpr (!PAIR) {
#pragma unroll
      for (int k = 0; k < K; ++k) {
#pragma unroll
        for (int e = 0; e < V2; ++e) {
          acc_g[k][e] = f2fma(dyf[k][e], xh[k][e], acc_g[k][e]);
          if constexpr (BSM) s_accb[(k * V2 + e) * 512] = f2add(s_accb[(k * V2 + e) * 512], dyf[k][e]);
          else if (KIND == FLN_LAYERNORM) acc_b[k][e] = f2add(acc_b[k][e], dyf[k][e]);
        }
      }
    }
    if (++s == S) {
      s = 0;
      phase ^= 1u;
    }
  }
  if (aborted && tid == 0) pipeline_abort(p.status, full, S, s, phase, my_tiles - i < S ? my_tiles - i : S, p.wait_ns);

  if (p.partials != nullptr && !aborted) {
    const int64_t prow = (int64_t)FLN_SLOT * R + r_in;
    float* __restrict__ pg = p.partials + prow * (int64_t)(NR * ld) + coff;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int iv = lane_r + k * tpr;
      if (vok[k]) {
        if constexpr (VEC % 4 == 0) {
#pragma unroll
          for (int e = 0; e < V2; e += 2) {
            *reinterpret_cast<float4*>(pg + (int64_t)iv * VEC + 2 * e) =
                make_float4(acc_g[k][e].x, acc_g[k][e].y, acc_g[k][e + 1].x, acc_g[k][e + 1].y);
            if (KIND == FLN_LAYERNORM)
              *reinterpret_cast<float4*>(pg + ld + (int64_t)iv * VEC + 2 * e) =
                  BSM ? make_float4(s_accb[(k * V2 + e) * 512].x, s_accb[(k * V2 + e) * 512].y,
                                    s_accb[(k * V2 + e + 1) * 512].x, s_accb[(k * V2 + e + 1) * 512].y)
                      : make_float4(acc_b[BSM ? 0 : k][BSM ? 0 : e].x, acc_b[BSM ? 0 : k][BSM ? 0 : e].y,
                                    acc_b[BSM ? 0 : k][BSM ? 0 : e + 1].x, acc_b[BSM ? 0 : k][BSM ? 0 : e + 1].y);
          }
        } else {
#pragma unroll
          for (int e = 0; e < V2; ++e) {
            *reinterpret_cast<float2*>(pg + (int64_t)iv * VEC + 2 * e) = acc_g[k][e];
            if (KIND == FLN_LAYERNORM)
              *reinterpret_cast<float2*>(pg + ld + (int64_t)iv * VEC + 2 * e) =
                  BSM ? s_accb[(k * V2 + e) * 512] : acc_b[BSM ? 0 : k][BSM ? 0 : e];
          }
        }
      }
    }
  }

  // neither CTA of a cluster leaves while the other might still write into its shared memory
  if (PAIR) cluster_sync_all();

  if (FUSE) {
    ReduceArgs a;
    a.partials = p.partials;
    a.sync = p.sync;
    a.token = p.token;
    a.dgb_f32 = p.dgb_f32;
    a.dgamma = p.dgamma;
    a.dbeta = p.dbeta;
    a.cols = cols;
    a.P = (int)gridDim.x * R;
    a.wait_ns = p.wait_ns;
    a.status = p.status;
    a.fault = p.fault;
    fused_column_reduce<T, NR>(a, reinterpret_cast<float*>(stages), aborted);
  }
}

#undef FLN_SLOT
#undef FLN_NSLOT
#undef FLN_WHOLE

template <typename KernelT>
static int launch_bwd_kernel(KernelT kern, const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;
  if (P.pair) {
    // clusters of two CTAs; the grid never exceeds what is resident at once
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)P.grid);
    cfg.blockDim = dim3((unsigned)P.threads);
    cfg.dynamicSmemBytes = P.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    static std::atomic<int> asked[64];
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && asked[dev].load(std::memory_order_relaxed) == 0) {
      int n = 0;
      cudaLaunchConfig_t probe = cfg;
      probe.gridDim = dim3(2u * (unsigned)(usable_sms() / 2 > 0 ? usable_sms() / 2 : 1));
      if (cudaOccupancyMaxActiveClusters(&n, kern, &probe) == cudaSuccess && n > 0) set_pair_slots(n);
      else cudaGetLastError();
      asked[dev].store(1, std::memory_order_relaxed);
      if (n > 0 && 2 * n < P.grid) return FLN_PIPE_NOT_APPLICABLE;  // planned for more clusters than fit: plan again
    }
    if (cudaLaunchKernelEx(&cfg, kern, p, P.g) != cudaSuccess) {
      cudaGetLastError();
      return FLN_ERR_LAUNCH;
    }
    FLN_CHECK_LAUNCH();
    return FLN_OK;
  }
  if (p.sync != nullptr) {
    // the grid barrier needs every CTA resident: cooperative launch
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)P.grid);
    cfg.blockDim = dim3((unsigned)P.threads);
    cfg.dynamicSmemBytes = P.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeCooperative;
    attr.val.cooperative = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, p, P.g) != cudaSuccess) {
      cudaGetLastError();
      return FLN_ERR_LAUNCH;
    }
  } else {
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);
  }
  FLN_CHECK_LAUNCH();
  return FLN_OK;
}

// dispatch of the plans that fln_pipeline_bwd.cu does not instantiate itself; FLN_PIPE_NOT_APPLICABLE
// if no instantiation serves the plan
int bwd_pipe_odd_any(int kind, int dtype, const BwdParams& p, const PipePlan& P, cudaStream_t st);
int bwd_pipe_pair_any(int kind, int dtype, const BwdParams& p, const PipePlan& P, cudaStream_t st);
int bwd_pipe_wide_any(int kind, int dtype, const BwdParams& p, const PipePlan& P, cudaStream_t st);
int bwd_pipe_tail_any(int kind, int dtype, const BwdParams& p, const PipePlan& P, cudaStream_t st);

}  // namespace fln
