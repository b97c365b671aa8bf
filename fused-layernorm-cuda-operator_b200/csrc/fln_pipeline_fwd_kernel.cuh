// Pipelined forward: the kernel.  See fln_pipeline.cuh for the ring and the scheduling of tiles.
// Instantiated in fln_pipeline_fwd.cu (the forward entry point) and fln_pipeline_fwd_fp8.cu (the
// fp8 outputs).
#pragma once
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "fln_philox.cuh"
#include "fln_pipeline.cuh"

namespace fln {

// ----------------------------------------------------------------------------------------
// forward
//
// Per pair of elements: one shift and one mask (widen), then on the register pair: shift by c
// and add (row sum), centre, one fma (sum of squares), one multiply and one fma (normalize +
// affine), one paired convert.  Statistics are the two-pass form on the row shifted by its
// first element, each pass reduced by a warp butterfly plus one shared-memory hop.
//
// Tiles: every CTA starts with tiles b, b + grid, ..., b + (S - 1) grid (no round trip before
// its first copies leave), then claims further tiles from the launch's counter, one claim
// ahead of need so that the atomic's latency never sits in front of a refill.  The thread
// that refills a stage notes the stage's tile in shared memory in front of arming the
// barrier; a stage whose claim came back beyond the last tile is armed without a copy and
// marked empty, and a CTA that meets an empty stage is done (claims only grow).
// ----------------------------------------------------------------------------------------
// MODE 0: general (bounds-checked); 1: FULL (no predication in the loop).
// MODE 4: FULL with gamma / beta parked in shared memory (in the I/O type) instead of in
// registers as floats, for plans that give a thread more than 32 elements (row lengths
// 5 * 2^a in 16-bit types: 40 elements per thread keep the 16-byte vectors and move more
// bytes per barrier than 20 elements in 8-byte vectors)
// MODE 5: rows whole, every vector whole except the last of a thread's K (rows that fit no
// exact plan, 1600 columns: K = 7, lanes beyond the row idle in the seventh vector only); the
// row length comes from the launch parameters, the split from LT.
// LT >= 0: the geometry is known at compile time -- a CTA of 256 threads (512 for LT = 9), 2^LT threads per row,
// rows of exactly K * VEC * 2^LT elements (FULL).  Row length, byte offsets of a thread's
// vectors and the shape of the reductions then fold into immediates: the bf16 forward at
// 16384 x 8192 executes 8.4 instead of 11.3 instructions per element and takes 83 instead of
// 101 us.  LT < 0 takes all of it from the launch parameters.
// QM > 0: the quantized outputs.  y is not stored in TO; max |y| of the launch goes to *p.amax
// (if set) and
//   QM 1: if p.q is set, y * *p.scale_in goes out as saturating e4m3 codes, two per conversion;
//   QM 2: e4m3 codes with one scale per row, 448 / max |y| of the row (written to p.row_scale);
//   QM 3: MXFP8 -- e4m3 codes with one power-of-two scale (an E8M0 byte in p.block_scale) per 32
//         consecutive elements, 2^(floor(log2(block max)) - 8); the 32 elements sit in four
//         neighbouring lanes;
//   QM 4: NVFP4-style -- e2m1 codes, two per byte, one e4m3 scale per 16 elements (two
//         neighbouring lanes), b = e4m3(block max * S / 6), q = e2m1(y * S / float(b)), S =
//         *p.scale_in.
// DROP: dropout in front of the residual add -- x is replaced by round(x * scale) where the
// Philox mask keeps it and by 0 elsewhere (one 128-bit Philox output per 16-byte vector; group,
// counter and key as in fln_dropout.cu), the mask byte goes to p.keep_bits if that is set, and
// the sum (or, without a residual, the dropped x) goes to p.sum_out if that is set.
template <typename TI, typename TO, int K, int KIND, int ACT, int MODE, int VB = 16, int LT = -1, int QM = 0,
          bool DROP = false>
// MODE 6: FULL with gamma / beta fetched from global memory (L1 / L2) for every row instead of
// living in registers, and the kernel held to 64 registers: two 512-thread CTAs per SM for rows
// that need 512 threads (one CTA of 512 threads per SM walks its rows in lockstep at a quarter
// of the warp slots).
__global__ void __launch_bounds__(512, (MODE == 6 || MODE == 8) ? 2 : 1) norm_fwd_pipe_kernel(const FwdParams p, const PipeGeom g) {
  constexpr int VEC = VB / sizeof(TI);  // a multiple of 4 (the statistics run four chains)
  constexpr int V2 = VEC / 2;
  constexpr bool FULL = MODE >= 1;
  constexpr bool PSM = MODE == 4 || MODE == 7;  // MODE 7: the ragged last vector and the parameters in shared memory
  constexpr bool PGL = MODE == 6 || MODE == 8;  // MODE 8: the same with a ragged last vector
  constexpr bool TAIL = MODE == 5 || MODE == 7 || MODE == 8;
  constexpr bool Q8 = QM > 0;
  static_assert(QM == 0 || (VEC == 8 && MODE == 1), "quantized outputs: 16-bit input, 16-byte vectors, exact rows");
  static_assert(!DROP || (VEC == 8 && MODE == 1), "dropout: 16-bit input, 16-byte vectors, exact rows");
  constexpr bool CT = LT >= 0;
  constexpr int LTC = CT ? LT : 0;
  constexpr int NT = LTC > 8 ? (1 << LTC) : 256;  // threads per CTA of the compile-time geometry
  static_assert(!CT || MODE == 1 || (MODE >= 4 && MODE <= 8), "compile-time geometry is for the FULL kernels");
  static_assert(!TAIL || CT, "the ragged-last-vector kernel has its split at compile time");
// vector k of this thread lies in the row: known at compile time except for the last of a TAIL plan
#define FLN_WHOLE(k) (FULL && !(TAIL && (k) == K - 1))
  const int tpr = CT ? (1 << LTC) : g.tpr;
  const int log2_tpr = CT ? LTC : g.log2_tpr;
  const int R = CT ? (NT >> LTC) : g.R;
  const int cols = (CT && !TAIL) ? ((K * VEC) << LTC) : p.cols;
  const uint32_t row_bytes = (CT && !TAIL) ? (uint32_t)((K * VB) << LTC) : g.row_bytes;
  const uint32_t second_off = CT ? row_bytes * (uint32_t)R : g.second_off;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  unsigned int* tile_of = reinterpret_cast<unsigned int*>(smem + 128);
  float* s_red = reinterpret_cast<float*>(smem + 256);  // 2 x 64 + 2 x 32 floats
  unsigned char* stages = smem + kSmemHeader;

  const int tid = threadIdx.x;
  const int lane_r = tid & (tpr - 1);
  const int r_in = tid >> log2_tpr;
  const int S = g.S;
  const unsigned int n_tiles = (unsigned int)((p.rows + R - 1) / R);
  const bool has_res = p.res != nullptr;
  const float inv_n = 1.0f / (float)cols;
  const float eps = p.eps;
  unsigned int* sched = p.sched;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  __syncthreads();

  // ---- producer (thread 0)
  const unsigned int dyn_base = gridDim.x * (unsigned int)S;
  unsigned int next_t = kNoTile;  // the tile claimed ahead
  auto fill = [&](unsigned int t, int s, bool skip_copy) {
    if (t < n_tiles) {
      const int64_t row0 = (int64_t)t * R;
      const int64_t left = p.rows - row0;
      const uint32_t bytes = (uint32_t)(left < R ? left : R) * row_bytes;
      unsigned char* dst = stages + (size_t)s * g.stage_stride;
      tile_of[s] = t;
      mbar_expect_tx(&full[s], has_res ? 2 * bytes : bytes);
      if (!skip_copy) {
        bulk_g2s(dst, reinterpret_cast<const TI*>(p.x) + row0 * cols, bytes, &full[s]);
        if (has_res)
          bulk_g2s(dst + second_off, reinterpret_cast<const TI*>(p.res) + row0 * cols, bytes, &full[s]);
      }
    } else {
      tile_of[s] = kNoTile;
      mbar_arrive(&full[s]);
    }
  };
  if (tid == 0) {
    // test hook (fln_set_test_fault bit 0): CTA 0 arms its first stage without the copy
    const bool fault = blockIdx.x == 0 && (*p.fault & 1) != 0;
    for (int s = 0; s < S; ++s) fill(blockIdx.x + (unsigned int)s * gridDim.x, s, fault && s == 0);
    next_t = dyn_base + atomicAdd(sched, 1u);
  }

  float2 gam[(PSM || PGL) ? 1 : K][V2], bet[(PSM || PGL) ? 1 : K][V2];
  bool vok[K];  // does vector k of this thread exist in the row
  unsigned char* s_gamma = stages + (size_t)S * g.stage_stride;  // PSM: [cols] gamma, then [cols] beta
  unsigned char* s_beta = s_gamma + row_bytes;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int iv = lane_r + k * tpr;
    vok[k] = FLN_WHOLE(k) ? true : iv < p.nv;
    if constexpr (PSM) {
      if (r_in == 0 && vok[k]) {
        Pack<TI, VEC> one, zero;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          one.e[e] = Cvt<TI>::from_f(1.f);
          zero.e[e] = Cvt<TI>::from_f(0.f);
        }
        *reinterpret_cast<Pack<TI, VEC>*>(s_gamma + (size_t)iv * VB) =
            p.gamma != nullptr ? ld_param<TI, VEC>(reinterpret_cast<const TI*>(p.gamma) + (int64_t)iv * VEC) : one;
        *reinterpret_cast<Pack<TI, VEC>*>(s_beta + (size_t)iv * VB) =
            p.beta != nullptr ? ld_param<TI, VEC>(reinterpret_cast<const TI*>(p.beta) + (int64_t)iv * VEC) : zero;
      }
    } else if constexpr (!PGL) {
#pragma unroll
      for (int e = 0; e < V2; ++e) {
        gam[k][e] = f2(1.f);
        bet[k][e] = f2(0.f);
      }
      if (vok[k]) {
        if (p.gamma != nullptr)
          unpack2<TI, VEC>(ld_param<TI, VEC>(reinterpret_cast<const TI*>(p.gamma) + (int64_t)iv * VEC), gam[k]);
        if (p.beta != nullptr)
          unpack2<TI, VEC>(ld_param<TI, VEC>(reinterpret_cast<const TI*>(p.beta) + (int64_t)iv * VEC), bet[k]);
      }
    }
  }
  if constexpr (PSM) __syncthreads();

  float amax = 0.f;
  float2 qs2 = f2(1.f);
  if constexpr (QM == 1) {
    if (p.q != nullptr) qs2 = f2(__ldg(p.scale_in));
  }
  if constexpr (QM == 4) qs2 = f2(__ldg(p.scale_in));
  int s = 0;
  uint32_t phase = 0;
  bool aborted = false;
  const uint32_t my_off = (uint32_t)r_in * row_bytes + (uint32_t)lane_r * (uint32_t)VB;
  const uint32_t k_off = (uint32_t)tpr * (uint32_t)VB;
  for (int i = 0;; ++i) {
    const bool landed = mbar_wait_bounded(&full[s], phase, p.wait_ns);
    // written by the producer before the last CTA barrier at the latest, so every thread reads
    // the same value here whether or not its wait succeeded
    const unsigned int tile = tile_of[s];
    if (tile == kNoTile) break;
    const int64_t row = (int64_t)tile * R + r_in;
    const bool row_ok = FULL ? true : row < p.rows;
    const unsigned char* st = stages + (size_t)s * g.stage_stride + my_off;
    float* redA = s_red + (i & 1) * 64;
    float* redB = s_red + 128 + (i & 1) * 32;

    float2 f[K][V2];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (FLN_WHOLE(k) || (row_ok && vok[k])) {
        unpack2<TI, VEC>(stage_vec<TI, VEC>(st + k * k_off), f[k]);
      } else {
#pragma unroll
        for (int e = 0; e < V2; ++e) f[k][e] = f2(0.f);
      }
    }
    if constexpr (DROP) {
      const float2 sc2 = f2(p.drop_scale);
      const unsigned long long g0 = (unsigned long long)row * (unsigned long long)(cols >> 3) + (unsigned int)lane_r;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const unsigned long long grp = g0 + (unsigned long long)(k * tpr);
        unsigned int lanes[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
        unsigned int m = 0xffu;
        if (p.drop_threshold != 0) m = keep_lanes8(grp, p.drop_seed, p.drop_offset, p.drop_threshold, lanes);
        if (p.keep_bits != nullptr) p.keep_bits[grp] = (unsigned char)m;
#pragma unroll
        for (int e = 0; e < V2; ++e) f[k][e] = f2mul(f[k][e], sc2);
        Pack<TI, VEC> q;
        pack2<TI, VEC>(f[k], q);  // rounds to the I/O type
        unsigned int* w = reinterpret_cast<unsigned int*>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) w[e] &= lanes[e];
        if (!has_res && p.sum_out != nullptr)
          st_stream<TI, VEC>(reinterpret_cast<TI*>(p.sum_out) + row * (int64_t)cols + (int64_t)(lane_r + k * tpr) * VEC, q);
        unpack2<TI, VEC>(q, f[k]);
      }
    }
    if (has_res) {
      TI* __restrict__ sr = reinterpret_cast<TI*>(p.sum_out) + row * (int64_t)cols + (int64_t)lane_r * VEC;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        if (FLN_WHOLE(k) || (row_ok && vok[k])) {
          float2 r[V2];
          unpack2<TI, VEC>(stage_vec<TI, VEC>(st + second_off + k * k_off), r);
#pragma unroll
          for (int e = 0; e < V2; ++e) f[k][e] = f2add(f[k][e], r[e]);
          // the sum is rounded to the I/O type first: that value is normalized and stored
          Pack<TI, VEC> q;
          pack2<TI, VEC>(f[k], q);
          st_stream<TI, VEC>(sr + (int64_t)k * tpr * VEC, q);
          unpack2<TI, VEC>(q, f[k]);
        }
      }
    }

    float mean = 0.f;
    if (KIND == FLN_LAYERNORM) {
      // shift by element 0 of the row (a broadcast read of the stage): a constant row then
      // sums to exactly zero whatever its magnitude, and |mean| >> std costs no accuracy
      const unsigned char* st0 = st - (size_t)lane_r * VB;
      float c = Cvt<TI>::to_f(*reinterpret_cast<const TI*>(st0));
      if (has_res)
        c = Cvt<TI>::to_f(Cvt<TI>::from_f(c + Cvt<TI>::to_f(*reinterpret_cast<const TI*>(st0 + second_off))));
      const float2 nc = f2(-c);
      float2 a01 = f2(0.f), a23 = f2(0.f);  // four chains: the adds are latency-bound
#pragma unroll
      for (int k = 0; k < K; ++k) {
        if (FLN_WHOLE(k) || vok[k]) {  // padding vectors stay zero
#pragma unroll
          for (int e = 0; e < V2; e += 2) {
            f[k][e] = f2add(f[k][e], nc);
            f[k][e + 1] = f2add(f[k][e + 1], nc);
            a01 = f2add(a01, f[k][e]);
            a23 = f2add(a23, f[k][e + 1]);
          }
        }
      }
      float ar[1] = {(a01.x + a01.y) + (a23.x + a23.y)};
      rowsum_warp<1>(ar, tpr, redA);
      // The first barrier of a tile also proves that every thread has pulled its part of
      // stage s into registers, so the producer may refill the stage right after it.
      if (!__syncthreads_and(landed ? 1 : 0)) {
        aborted = true;
        break;
      }
      if (tid == 0) {
        fill(next_t, s, false);
        if (next_t < n_tiles) next_t = dyn_base + atomicAdd(sched, 1u);
      }
      rowsum_cta<1>(ar, tpr, redA);
      const float ms = ar[0] * inv_n;  // mean of the shifted row
      mean = c + ms;
      const float2 nms = f2(-ms);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        if (FLN_WHOLE(k) || vok[k]) {
#pragma unroll
          for (int e = 0; e < V2; ++e) f[k][e] = f2add(f[k][e], nms);
        }
      }
    }
    float2 q01 = f2(0.f), q23 = f2(0.f);
#pragma unroll
    for (int k = 0; k < K; ++k) {
#pragma unroll
      for (int e = 0; e < V2; e += 2) {
        q01 = f2fma(f[k][e], f[k][e], q01);
        q23 = f2fma(f[k][e + 1], f[k][e + 1], q23);
      }
    }
    float q[1] = {(q01.x + q01.y) + (q23.x + q23.y)};
    rowsum_warp<1>(q, tpr, redB);
    if (KIND == FLN_LAYERNORM) {
      __syncthreads();
    } else {
      if (!__syncthreads_and(landed ? 1 : 0)) {
        aborted = true;
        break;
      }
      if (tid == 0) {
        fill(next_t, s, false);
        if (next_t < n_tiles) next_t = dyn_base + atomicAdd(sched, 1u);
      }
    }
    rowsum_cta<1>(q, tpr, redB);
    const float rstd = rsqrtf(fmaf(q[0], inv_n, eps));

    if (row_ok && lane_r == 0) {
      if (KIND == FLN_LAYERNORM && p.mean != nullptr) p.mean[row] = mean;
      if (p.rstd != nullptr) p.rstd[row] = rstd;
    }
    TO* __restrict__ yr = reinterpret_cast<TO*>(p.y) + row * (int64_t)cols + (int64_t)lane_r * VEC;
    const float2 r2 = f2(rstd);
    if constexpr (QM == 2) {
      // the row's maximum first (y is cheap to form twice: two operations per pair), then its scale
      float rm = 0.f;
#pragma unroll
      for (int k = 0; k < K; ++k) {
#pragma unroll
        for (int e = 0; e < V2; ++e) {
          const float2 o = f2fma(f2mul(f[k][e], r2), gam[k][e], bet[k][e]);
          rm = fmaxf(rm, fmaxf(fabsf(o.x), fabsf(o.y)));
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) rm = fmaxf(rm, __shfl_xor_sync(0xffffffffu, rm, off));
      if (tpr > 32) {
        float* s_rmax = reinterpret_cast<float*>(smem + 1024) + (i & 1) * 32;
        const int warp = tid >> 5, wpr = tpr >> 5;
        if ((tid & 31) == 0) s_rmax[warp] = rm;
        __syncthreads();
        const int gbase = warp & ~(wpr - 1);
        rm = s_rmax[gbase];
        for (int j = 1; j < wpr; ++j) rm = fmaxf(rm, s_rmax[gbase + j]);
      }
      amax = fmaxf(amax, rm);
      const float rs = rm > 0.f ? 448.0f / rm : 1.0f;
      qs2 = f2(rs);
      if (lane_r == 0) p.row_scale[row] = rs;
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (FLN_WHOLE(k) || (row_ok && vok[k])) {
        float2 o[V2];
        if constexpr (PSM) {
          float2 gw[V2], bw[V2];
          const size_t po = (size_t)(lane_r + k * tpr) * VB;
          unpack2<TI, VEC>(stage_vec<TI, VEC>(s_gamma + po), gw);
          unpack2<TI, VEC>(stage_vec<TI, VEC>(s_beta + po), bw);
#pragma unroll
          for (int e = 0; e < V2; ++e) o[e] = f2fma(f2mul(f[k][e], r2), gw[e], bw[e]);
        } else if constexpr (PGL) {
          float2 gw[V2], bw[V2];
#pragma unroll
          for (int e = 0; e < V2; ++e) {
            gw[e] = f2(1.f);
            bw[e] = f2(0.f);
          }
          const int64_t po = (int64_t)(lane_r + k * tpr) * VEC;
          if (p.gamma != nullptr) unpack2<TI, VEC>(ld_param<TI, VEC>(reinterpret_cast<const TI*>(p.gamma) + po), gw);
          if (p.beta != nullptr) unpack2<TI, VEC>(ld_param<TI, VEC>(reinterpret_cast<const TI*>(p.beta) + po), bw);
#pragma unroll
          for (int e = 0; e < V2; ++e) o[e] = f2fma(f2mul(f[k][e], r2), gw[e], bw[e]);
        } else {
#pragma unroll
          for (int e = 0; e < V2; ++e) o[e] = f2fma(f2mul(f[k][e], r2), gam[k][e], bet[k][e]);
        }
        if (ACT != FLN_ACT_NONE) {
#pragma unroll
          for (int e = 0; e < V2; ++e) o[e] = apply_act2<ACT>(o[e]);
        }
        if constexpr (Q8) {
#pragma unroll
          for (int e = 0; e < V2; ++e) amax = fmaxf(amax, fmaxf(fabsf(o[e].x), fabsf(o[e].y)));  // fmaxf drops NaN
          if constexpr (QM == 1 || QM == 2) {
            if (QM == 2 || p.q != nullptr) {
              Pack<unsigned char, VEC> out;
              unsigned short* w = reinterpret_cast<unsigned short*>(&out);
#pragma unroll
              for (int e = 0; e < V2; ++e)
                w[e] = __nv_cvt_float2_to_fp8x2(f2mul(o[e], qs2), __NV_SATFINITE, __NV_E4M3);
              st_stream<unsigned char, VEC>(reinterpret_cast<unsigned char*>(p.q) + row * (int64_t)cols +
                                                (int64_t)(lane_r + k * tpr) * VEC,
                                            out);
            }
          } else {
            // block-scaled: the maximum of this thread's vector, then of the block's lanes
            const int iv = lane_r + k * tpr;
            float bm = 0.f;
#pragma unroll
            for (int e = 0; e < V2; ++e) bm = fmaxf(bm, fmaxf(fabsf(o[e].x), fabsf(o[e].y)));
            constexpr int G = (QM == 3 ? 32 : 16) / VEC;
#pragma unroll
            for (int off = 1; off < G; off <<= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, off));
            if constexpr (QM == 3) {
              const unsigned int ef = (__float_as_uint(bm) >> 23) & 0xffu;  // biased exponent of the block maximum
              const unsigned int e8 = ef > 8u ? ef - 8u : 0u;               // the scale is 2^(e8 - 127)
              const float2 inv = f2(__uint_as_float((254u - e8) << 23));    // 2^(127 - e8), exact
              Pack<unsigned char, VEC> out;
              unsigned short* w = reinterpret_cast<unsigned short*>(&out);
#pragma unroll
              for (int e = 0; e < V2; ++e)
                w[e] = __nv_cvt_float2_to_fp8x2(f2mul(o[e], inv), __NV_SATFINITE, __NV_E4M3);
              st_stream<unsigned char, VEC>(reinterpret_cast<unsigned char*>(p.q) + row * (int64_t)cols +
                                                (int64_t)iv * VEC,
                                            out);
              if ((lane_r & (G - 1)) == 0) p.block_scale[row * (int64_t)(cols / 32) + iv / G] = (unsigned char)e8;
            } else {
              const float S = qs2.x;
              const unsigned char sb = (unsigned char)__nv_cvt_float_to_fp8(__fmul_rn(__fmul_rn(bm, S), 1.0f / 6.0f),
                                                                            __NV_SATFINITE, __NV_E4M3);
              const float fb = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb, __NV_E4M3)));
              const float invs = fb > 0.f ? __fdiv_rn(S, fb) : 0.f;
              Pack<unsigned char, VEC / 2> out;
#pragma unroll
              for (int e = 0; e < V2; ++e)
                out.e[e] = (unsigned char)__nv_cvt_float2_to_fp4x2(
                    make_float2(__fmul_rn(o[e].x, invs), __fmul_rn(o[e].y, invs)), __NV_E2M1, cudaRoundNearest);
              st_stream<unsigned char, VEC / 2>(
                  reinterpret_cast<unsigned char*>(p.q) + ((row * (int64_t)cols) >> 1) + (int64_t)iv * (VEC / 2), out);
              if ((lane_r & (G - 1)) == 0) p.block_scale[row * (int64_t)(cols / 16) + iv / G] = sb;
            }
          }
        } else {
          Pack<TO, VEC> out;
          pack2<TO, VEC>(o, out);
          st_stream<TO, VEC>(yr + (int64_t)k * tpr * VEC, out);
        }
      }
    }
    if (++s == S) {
      s = 0;
      phase ^= 1u;
    }
  }

  if constexpr (Q8) {
    // max |y| of this CTA's rows, one atomic per CTA (non-negative floats order like their bit
    // patterns).  Every thread arrives here: the loop is left by all threads of a CTA together.
    if (p.amax != nullptr) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
      __syncthreads();  // the reductions of the last tile are done with s_red
      if ((tid & 31) == 0) s_red[tid >> 5] = amax;
      __syncthreads();
      if (tid < 32) {
        float t = tid < (int)(blockDim.x >> 5) ? s_red[tid] : 0.f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, off));
        if (tid == 0 && t > 0.f) atomicMax(reinterpret_cast<unsigned int*>(p.amax), __float_as_uint(t));
      }
    }
  }

  // ---- exit: every CTA counts itself out; the last one puts the launch's counter pair back
  // to zero and checks that the claims add up (every tile beyond the static ones claimed once,
  // and one claim beyond the end per CTA)
  if (tid == 0) {
    if (aborted) pipeline_abort(p.status, full, S, s, phase, S, p.wait_ns);  // every stage of this ring is always armed
    __threadfence();
    const unsigned int done = atomicAdd(sched + 1, 1u);
    if (done == gridDim.x - 1) {
      const unsigned int claims = atomicExch(sched, 0u);
      const unsigned int dyn_tiles = n_tiles > dyn_base ? n_tiles - dyn_base : 0u;
      if (claims != dyn_tiles + gridDim.x && (*p.status & 1) == 0) atomicOr(p.status, 4);
      atomicExch(sched + 1, 0u);
    }
  }
}
#undef FLN_WHOLE

// what every launch of the kernel needs besides the caller's pointers: the tile counters, the
// wait limit, the status and test-hook words.  false if the device words cannot be had.
bool fwd_pipe_prepare(FwdParams* p);
// the ragged-last-vector instantiations (fln_pipeline_fwd_tail.cu)
int fwd_pipe_tail_any(int kind, int dtype, const FwdParams& p, const PipePlan& P, cudaStream_t st);

}  // namespace fln
