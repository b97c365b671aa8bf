// (residual +) LayerNorm / RMSNorm forward with fp8-e4m3 output and a per-tensor scale
// computed on the device, for sm_100a.
//
// The scale depends on amax over the whole tensor, so the work is two launches:
//   phase 1  norm_amax_kernel: read x (+ residual) once, write the bf16/f16/f32 sum s and
//            the per-row statistics, reduce max|y| per CTA and fold it into *amax with
//            one atomicMax per CTA (non-negative floats order like their bit patterns);
//   phase 2  norm_quant_kernel: re-read s, recompute y, store sat_e4m3(y * 448/amax).
//            Rows are walked from the last to the first so the rows phase 1 wrote most
//            recently are still in L2.
// There is no grid-wide wait anywhere.  The reference has no counterpart.
//
// Two one-pass forms avoid the second read of s (7 instead of 9 bytes per element):
//   delayed scaling  the caller supplies the scale (typically 448 / amax of the previous
//                    step); the kernel quantizes with it and reports this call's amax;
//   per-row scaling  every row gets its own scale 448 / max|y_row|, known once the row is
//                    in registers, and the scales are returned as an fp32 vector.
// Both are norm_amax_kernel with QMODE 1 / 2: same loads, same statistics, then the codes.
//   block scaling    (QMODE 3) the OCP microscaling form MXFP8 that Blackwell's block-scaled
//                    tensor-core instructions consume: every 32 consecutive elements of a row
//                    share one power-of-two scale, stored as an E8M0 byte, chosen as
//                    2^(floor(log2(block max)) - 8); the elements are e4m3.  The 32 elements
//                    sit in 4 (16-bit input) or 8 (fp32) neighbouring lanes, so the block
//                    maximum is two or three shuffles; one pass, 7 + 1/32 bytes per element.
//
// Both kernels follow the register-resident forward (fln_forward.cu): the row lives in
// registers as floats, statistics are the shifted two-pass form with sum reductions, 16-bit
// values are widened / narrowed in pairs, fp8 codes are produced two at a time, and the FULL
// instantiation carries no bounds checks.
#include <cuda_fp4.h>

#include "fln_common.cuh"

namespace fln {

struct Fp8Params {
  const void* x;
  const void* res;
  const void* gamma;
  const void* beta;
  void* q;
  void* sum_out;
  float* mean;
  float* rstd;
  float* amax;
  float* scale;
  const float* scale_in;  // QMODE 1: one fp32, read by every CTA
  float* row_scale;       // QMODE 2: [rows] fp32, written
  unsigned char* block_scale;  // QMODE 3: [rows, cols / 32] E8M0 bytes; QMODE 4: [rows, cols / 16] e4m3 bytes; written
  int64_t rows;
  int cols;
  int nv;
  int tpr;
  int log2_tpr;
  float eps;
};

// Up to four vectors per thread the kernels fit 64 registers, i.e. 1024 threads per SM (one CTA
// of 1024 or two of 512).  The four-vector form says so to the compiler (two CTAs per SM):
// left alone, its MXFP8 instantiation took 66 registers and with that half the resident CTAs,
// 428 instead of 372 us at 32768 x 8192.  Eight vectors per thread need more than 64.
template <int K>
struct Fp8MaxThreads {
  static constexpr int value = K <= 2 ? 1024 : 512;
};

// y (before quantization) of this thread's vectors, from the centred row and the statistics
template <typename TI, int VEC>
__device__ __forceinline__ void affine(float (&o)[VEC], const float (&f)[VEC], float rstd, const TI* gp,
                                       const TI* bp, int64_t off) {
#pragma unroll
  for (int i = 0; i < VEC; ++i) o[i] = f[i] * rstd;
  if (gp != nullptr) {
    float g[VEC];
    unpack<TI, VEC>(ld_param<TI, VEC>(gp + off), g);
    if (bp != nullptr) {
      float b[VEC];
      unpack<TI, VEC>(ld_param<TI, VEC>(bp + off), b);
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = fmaf(o[i], g[i], b[i]);
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] *= g[i];
    }
  } else if (bp != nullptr) {
    float b[VEC];
    unpack<TI, VEC>(ld_param<TI, VEC>(bp + off), b);
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] += b[i];
  }
}

// VEC saturating e4m3 codes from VEC floats, two per conversion instruction
template <int VEC>
__device__ __forceinline__ void pack_fp8(const float (&v)[VEC], Pack<unsigned char, VEC>& o) {
  if constexpr (VEC >= 2) {
    unsigned short* w = reinterpret_cast<unsigned short*>(&o);
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j)
      w[j] = __nv_cvt_float2_to_fp8x2(make_float2(v[2 * j], v[2 * j + 1]), __NV_SATFINITE, __NV_E4M3);
  } else {
    o.e[0] = (unsigned char)__nv_cvt_float_to_fp8(v[0], __NV_SATFINITE, __NV_E4M3);
  }
}

// CTA-wide max of a non-negative value, folded into *dst with one atomic per CTA
// (non-negative floats order like their bit patterns).  Contains a CTA barrier.
__device__ __forceinline__ void cta_max_to_global(float m, float* s_max, float* dst) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) s_max[warp] = m;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    float t = lane < nw ? s_max[lane] : 0.f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, off));
    if (lane == 0 && t > 0.f) atomicMax(reinterpret_cast<unsigned int*>(dst), __float_as_uint(t));
  }
}
// max over the tpr threads that own a row; every one of them gets the result
__device__ __forceinline__ float row_max(float m, int tpr, float* smem) {
  if (tpr >= 32) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  } else {
    for (int off = tpr >> 1; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  }
  if (tpr > 32) {
    const int warp = threadIdx.x >> 5, wpr = tpr >> 5;
    if ((threadIdx.x & 31) == 0) smem[warp] = m;
    __syncthreads();
    const int gbase = warp & ~(wpr - 1);
    m = smem[gbase];
    for (int j = 1; j < wpr; ++j) m = fmaxf(m, smem[gbase + j]);
  }
  return m;
}

// QMODE 0: phase 1 of the two-launch form (amax only); 1: quantize with *scale_in; 2: per-row
// scale; 3: one E8M0 scale per block of 32 elements (MXFP8)
template <typename TI, int VEC, int K, int KIND, bool FULL, int QMODE>
__global__ void __launch_bounds__(Fp8MaxThreads<K>::value, K == 4 ? 2 : 1) norm_amax_kernel(const Fp8Params p) {
  __shared__ __align__(16) float s_red[2][32];
  __shared__ float s_max[32];
  __shared__ float s_rmax[32];

  const int tid = threadIdx.x;
  const int tpr = p.tpr;
  const int lane_r = tid & (tpr - 1);
  const int row_in_cta = tid >> p.log2_tpr;
  const int rows_per_cta = blockDim.x >> p.log2_tpr;
  const int64_t row = (int64_t)blockIdx.x * rows_per_cta + row_in_cta;
  const bool row_ok = FULL ? true : row < p.rows;
  const int64_t base = row_ok ? row * (int64_t)p.cols : 0;
  const float inv_n = 1.0f / (float)p.cols;
  const TI* __restrict__ xr = reinterpret_cast<const TI*>(p.x) + base;

  float c = 0.f;  // shift for the LayerNorm statistics: element 0 of the (summed) row
  if (KIND == FLN_LAYERNORM) {
    c = Cvt<TI>::to_f(ld_param<TI, 1>(xr).e[0]);
    if (p.res != nullptr)
      c = Cvt<TI>::to_f(Cvt<TI>::from_f(c + Cvt<TI>::to_f(ld_param<TI, 1>(reinterpret_cast<const TI*>(p.res) + base).e[0])));
  }
  float f[K][VEC];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int iv = lane_r + k * tpr;
    if (FULL || (row_ok && iv < p.nv)) {
      unpack<TI, VEC>(ld_stream<TI, VEC>(xr + (int64_t)iv * VEC), f[k]);
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) f[k][i] = 0.f;
    }
  }
  if (p.res != nullptr) {
    const TI* __restrict__ rr = reinterpret_cast<const TI*>(p.res) + base;
    TI* __restrict__ sr = reinterpret_cast<TI*>(p.sum_out) + base;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int iv = lane_r + k * tpr;
      if (FULL || (row_ok && iv < p.nv)) {
        float r[VEC];
        unpack<TI, VEC>(ld_stream<TI, VEC>(rr + (int64_t)iv * VEC), r);
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[k][i] += r[i];
        Pack<TI, VEC> q;
        pack<TI, VEC>(f[k], q);
        // two-launch form: plain store, phase 2 wants to find these lines in L2
        if (QMODE == 0) {
          st_plain<TI, VEC>(sr + (int64_t)iv * VEC, q);
        } else {
          st_stream<TI, VEC>(sr + (int64_t)iv * VEC, q);
        }
        unpack<TI, VEC>(q, f[k]);
      }
    }
  }

  float mean = 0.f;
  if (KIND == FLN_LAYERNORM) {
    float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (FULL || lane_r + k * tpr < p.nv) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          f[k][i] -= c;
          a4[(k * VEC + i) & 3] += f[k][i];
        }
      }
    }
    float a[1] = {(a4[0] + a4[1]) + (a4[2] + a4[3])};
    rowsum_warp<1>(a, tpr, s_red[0]);
    if (tpr > 32) __syncthreads();
    rowsum_cta<1>(a, tpr, s_red[0]);
    const float ms = a[0] * inv_n;
    mean = c + ms;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (FULL || lane_r + k * tpr < p.nv) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[k][i] -= ms;
      }
    }
  }
  float q4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int k = 0; k < K; ++k) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) q4[(k * VEC + i) & 3] = fmaf(f[k][i], f[k][i], q4[(k * VEC + i) & 3]);
  }
  float qs[1] = {(q4[0] + q4[1]) + (q4[2] + q4[3])};
  rowsum_warp<1>(qs, tpr, s_red[1]);
  if (tpr > 32) __syncthreads();
  rowsum_cta<1>(qs, tpr, s_red[1]);
  const float rstd = rsqrtf(qs[0] * inv_n + p.eps);
  if (row_ok && lane_r == 0) {
    if (KIND == FLN_LAYERNORM && p.mean != nullptr) p.mean[row] = mean;
    if (p.rstd != nullptr) p.rstd[row] = rstd;
  }

  const TI* __restrict__ gp = reinterpret_cast<const TI*>(p.gamma);
  const TI* __restrict__ bp = reinterpret_cast<const TI*>(p.beta);
  unsigned char* __restrict__ qr = reinterpret_cast<unsigned char*>(p.q) + base;
  float amax = 0.f;
  float qscale = 1.f;
  if (QMODE == 1) qscale = __ldg(p.scale_in);
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int iv = lane_r + k * tpr;
    if (QMODE != 3 && QMODE != 4 && (FULL || (row_ok && iv < p.nv))) {
      float o[VEC];
      affine<TI, VEC>(o, f[k], rstd, gp, bp, (int64_t)iv * VEC);
#pragma unroll
      for (int i = 0; i < VEC; ++i) amax = fmaxf(amax, fabsf(o[i]));  // fmaxf drops NaN
      if (QMODE == 1) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] *= qscale;
        Pack<unsigned char, VEC> out;
        pack_fp8<VEC>(o, out);
        st_stream<unsigned char, VEC>(qr + (int64_t)iv * VEC, out);
      }
    }
  }
  if (QMODE == 3) {
    constexpr int G = 32 / VEC;  // neighbouring lanes that hold one block of 32 elements
    unsigned char* __restrict__ bs = p.block_scale + (row_ok ? row : 0) * (int64_t)(p.cols / 32);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int iv = lane_r + k * tpr;
      const bool act = FULL || (row_ok && iv < p.nv);
      float o[VEC];
      float bm = 0.f;
      if (act) {
        affine<TI, VEC>(o, f[k], rstd, gp, bp, (int64_t)iv * VEC);
#pragma unroll
        for (int i = 0; i < VEC; ++i) bm = fmaxf(bm, fabsf(o[i]));
      }
      amax = fmaxf(amax, bm);
      // cols % 32 == 0, so the G lanes of a block are all active or all idle; every lane
      // takes part in the shuffles
#pragma unroll
      for (int off = 1; off < G; off <<= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, off));
      const unsigned int ef = (__float_as_uint(bm) >> 23) & 0xffu;  // biased exponent of the block maximum
      const unsigned int e8 = ef > 8u ? ef - 8u : 0u;               // the scale is 2^(e8 - 127)
      const float inv = __uint_as_float((254u - e8) << 23);         // 2^(127 - e8), exact
      if (act) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] *= inv;
        Pack<unsigned char, VEC> out;
        pack_fp8<VEC>(o, out);
        st_stream<unsigned char, VEC>(qr + (int64_t)iv * VEC, out);
        if ((lane_r & (G - 1)) == 0) bs[iv / G] = (unsigned char)e8;
      }
    }
  }
  if (QMODE == 4) {
    // NVFP4-style: e2m1 elements (two per byte, the even element in the low nibble), one e4m3
    // scale per 16 consecutive elements of a row, one fp32 scale S for the tensor, supplied by
    // the caller (typically 448 * 6 / amax of the previous step):
    //   block scale  b = e4m3(block max * S / 6)     (round to nearest even, saturating)
    //   element      q = e2m1(y * S / float(b))      (round to nearest even, saturating at 6)
    // and y ~ e2m1(q) * float(b) / S.  The 16 elements of a block sit in G neighbouring lanes.
    constexpr int G = 16 / VEC;
    const float S = __ldg(p.scale_in);
    unsigned char* __restrict__ bs = p.block_scale + (row_ok ? row : 0) * (int64_t)(p.cols / 16);
    unsigned char* __restrict__ q4 = reinterpret_cast<unsigned char*>(p.q) + (base >> 1);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int iv = lane_r + k * tpr;
      const bool act = FULL || (row_ok && iv < p.nv);
      float o[VEC];
      float bm = 0.f;
      if (act) {
        affine<TI, VEC>(o, f[k], rstd, gp, bp, (int64_t)iv * VEC);
#pragma unroll
        for (int i = 0; i < VEC; ++i) bm = fmaxf(bm, fabsf(o[i]));
      }
      amax = fmaxf(amax, bm);
      // cols % 16 == 0, so the G lanes of a block are all active or all idle
#pragma unroll
      for (int off = 1; off < G; off <<= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, off));
      const unsigned char sb = (unsigned char)__nv_cvt_float_to_fp8(__fmul_rn(__fmul_rn(bm, S), 1.0f / 6.0f), __NV_SATFINITE, __NV_E4M3);
      const float fb = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb, __NV_E4M3)));
      const float inv = fb > 0.f ? __fdiv_rn(S, fb) : 0.f;
      if (act) {
        Pack<unsigned char, VEC / 2> out;
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i)
          out.e[i] = (unsigned char)__nv_cvt_float2_to_fp4x2(make_float2(__fmul_rn(o[2 * i], inv), __fmul_rn(o[2 * i + 1], inv)),
                                                            __NV_E2M1, cudaRoundNearest);
        st_stream<unsigned char, VEC / 2>(q4 + (int64_t)iv * (VEC / 2), out);
        if ((lane_r & (G - 1)) == 0) bs[iv / G] = sb;
      }
    }
  }
  if (QMODE == 2) {
    const float rmax = row_max(amax, tpr, s_rmax);
    qscale = rmax > 0.f ? 448.0f / rmax : 1.0f;
    if (row_ok && lane_r == 0) p.row_scale[row] = qscale;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int iv = lane_r + k * tpr;
      if (FULL || (row_ok && iv < p.nv)) {
        float o[VEC];
        affine<TI, VEC>(o, f[k], rstd, gp, bp, (int64_t)iv * VEC);
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] *= qscale;
        Pack<unsigned char, VEC> out;
        pack_fp8<VEC>(o, out);
        st_stream<unsigned char, VEC>(qr + (int64_t)iv * VEC, out);
      }
    }
  }
  // tensor-wide amax: always in the two-launch form, on request otherwise
  if (QMODE == 0 || p.amax != nullptr) cta_max_to_global(amax, s_max, p.amax);
}

template <typename TI, int VEC, int K, int KIND, bool FULL>
__global__ void __launch_bounds__(Fp8MaxThreads<K>::value) norm_quant_kernel(const Fp8Params p) {
  const int tid = threadIdx.x;
  const int tpr = p.tpr;
  const int lane_r = tid & (tpr - 1);
  const int row_in_cta = tid >> p.log2_tpr;
  const int rows_per_cta = blockDim.x >> p.log2_tpr;
  // last rows first
  const int64_t row = p.rows - 1 - ((int64_t)blockIdx.x * rows_per_cta + row_in_cta);
  if (!FULL && row < 0) return;
  const int64_t base = row * (int64_t)p.cols;
  const TI* __restrict__ sr = reinterpret_cast<const TI*>(p.res != nullptr ? p.sum_out : p.x) + base;

  float f[K][VEC];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int iv = lane_r + k * tpr;
    if (FULL || iv < p.nv) unpack<TI, VEC>(ld_stream<TI, VEC>(sr + (int64_t)iv * VEC), f[k]);
  }
  const float am = *p.amax;
  const float scale = am > 0.f ? 448.0f / am : 1.0f;
  if (blockIdx.x == 0 && tid == 0) *p.scale = scale;
  const float mean = KIND == FLN_LAYERNORM ? __ldg(p.mean + row) : 0.f;
  const float rstd = __ldg(p.rstd + row);

  const TI* __restrict__ gp = reinterpret_cast<const TI*>(p.gamma);
  const TI* __restrict__ bp = reinterpret_cast<const TI*>(p.beta);
  unsigned char* __restrict__ qr = reinterpret_cast<unsigned char*>(p.q) + base;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int iv = lane_r + k * tpr;
    if (FULL || iv < p.nv) {
      float o[VEC];
      if (KIND == FLN_LAYERNORM) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[k][i] -= mean;
      }
      affine<TI, VEC>(o, f[k], rstd, gp, bp, (int64_t)iv * VEC);
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] *= scale;
      Pack<unsigned char, VEC> out;
      pack_fp8<VEC>(o, out);
      st_stream<unsigned char, VEC>(qr + (int64_t)iv * VEC, out);
    }
  }
}

// phase1_done: the pipelined forward has already written the sum, the statistics and amax of
// the two-launch form; only the quantizing launch is left
template <typename TI, int KIND>
static int run_fp8(Fp8Params p, int qmode, cudaStream_t st, bool phase1_done) {
  constexpr int VFULL = 16 / sizeof(TI);
  Plan pl = make_plan(false, p.rows, p.cols, (int)sizeof(TI), true);
  if (pl.generic || pl.vec != VFULL) return FLN_ERR_UNSUPPORTED;
  // block-scaled outputs: the vectors of one block must sit in neighbouring lanes, so a row needs
  // at least as many threads as a block has vectors (very short rows: spread them out)
  const int block_lanes = qmode == 3 ? 32 / VFULL : (qmode == 4 ? 16 / VFULL : 1);
  if (pl.tpr < block_lanes && (qmode != 3 || p.cols % 32 == 0)) {
    const int nvv = p.cols / VFULL;
    int k = 1;
    while (k * block_lanes < nvv) k <<= 1;
    if (k <= 8) {
      pl.tpr = block_lanes;
      pl.log2_tpr = block_lanes == 1 ? 0 : (block_lanes == 2 ? 1 : (block_lanes == 4 ? 2 : 3));
      pl.K = k;
      pl.rows_per_cta = pl.threads / pl.tpr;
    }
  }
  p.tpr = pl.tpr;
  p.log2_tpr = pl.log2_tpr;
  p.nv = p.cols / VFULL;
  const unsigned grid = (unsigned)((p.rows + pl.rows_per_cta - 1) / pl.rows_per_cta);
  const bool full = pl.tpr >= 32 && (int64_t)pl.K * pl.tpr == p.nv && p.rows % pl.rows_per_cta == 0;
  if (qmode == 3 && (p.cols % 32 != 0 || pl.tpr < 32 / VFULL)) return FLN_ERR_UNSUPPORTED;
  if (qmode == 4 && (p.cols % 16 != 0 || pl.tpr < 16 / VFULL)) return FLN_ERR_UNSUPPORTED;
  if (!phase1_done && p.amax != nullptr && cudaMemsetAsync(p.amax, 0, sizeof(float), st) != cudaSuccess)
    return FLN_ERR_LAUNCH;
#define FLN_FP8_LAUNCH(KK, FF)                                                                  \
  if (qmode == 0) {                                                                             \
    if (!phase1_done) norm_amax_kernel<TI, VFULL, KK, KIND, FF, 0><<<grid, pl.threads, 0, st>>>(p); \
    norm_quant_kernel<TI, VFULL, KK, KIND, FF><<<grid, pl.threads, 0, st>>>(p);                 \
  } else if (qmode == 1) {                                                                      \
    norm_amax_kernel<TI, VFULL, KK, KIND, FF, 1><<<grid, pl.threads, 0, st>>>(p);               \
  } else if (qmode == 3) {                                                                      \
    norm_amax_kernel<TI, VFULL, KK, KIND, FF, 3><<<grid, pl.threads, 0, st>>>(p);               \
  } else if (qmode == 4) {                                                                      \
    norm_amax_kernel<TI, VFULL, KK, KIND, FF, 4><<<grid, pl.threads, 0, st>>>(p);               \
  } else {                                                                                      \
    norm_amax_kernel<TI, VFULL, KK, KIND, FF, 2><<<grid, pl.threads, 0, st>>>(p);               \
  }
#define FLN_FP8_CASE(KK)          \
  case KK:                        \
    if (full) {                   \
      FLN_FP8_LAUNCH(KK, true)    \
    } else {                      \
      FLN_FP8_LAUNCH(KK, false)   \
    }                             \
    break;
  switch (pl.K) {
    FLN_FP8_CASE(1)
    FLN_FP8_CASE(2)
    FLN_FP8_CASE(4)
    FLN_FP8_CASE(8)
    default:
      return FLN_ERR_ARG;
  }
#undef FLN_FP8_CASE
#undef FLN_FP8_LAUNCH
  FLN_CHECK_LAUNCH();
  return FLN_OK;
}

}  // namespace fln

using namespace fln;

static int fp8_entry(int qmode, int kind, const void* x, const void* residual, const void* gamma,
                     const void* beta, void* q, void* sum_out, float* mean, float* rstd, float* amax,
                     float* scale, const float* scale_in, float* row_scale, int64_t rows, int64_t cols,
                     int io_dtype, float eps, void* stream, unsigned char* block_scale = nullptr,
                     bool part = false) {
  // part: a slice of the rows of a larger call (below) -- no further split, amax not reset
  if (kind != FLN_LAYERNORM && kind != FLN_RMSNORM) return FLN_ERR_ARG;
  if (rows < 0 || cols <= 0 || cols > 0x7fffffff || rows > 0x7fffffff) return FLN_ERR_SHAPE;
  if (io_dtype != FLN_F32 && io_dtype != FLN_BF16 && io_dtype != FLN_F16) return FLN_ERR_DTYPE;
  if (qmode == 0 && (amax == nullptr || scale == nullptr)) return FLN_ERR_NULL;
  if ((qmode == 1 || qmode == 4) && scale_in == nullptr) return FLN_ERR_NULL;
  if (qmode == 2 && row_scale == nullptr) return FLN_ERR_NULL;
  if ((qmode == 3 || qmode == 4) && block_scale == nullptr) return FLN_ERR_NULL;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (rows == 0) {
    // empty tensor: amax = 0, scale = 1
    const float one = 1.0f;
    if (amax != nullptr && cudaMemsetAsync(amax, 0, sizeof(float), st) != cudaSuccess) return FLN_ERR_LAUNCH;
    if (scale != nullptr &&
        cudaMemcpyAsync(scale, &one, sizeof(float), cudaMemcpyHostToDevice, st) != cudaSuccess)
      return FLN_ERR_LAUNCH;
    return FLN_OK;
  }
  if (x == nullptr || q == nullptr) return FLN_ERR_NULL;
  if (qmode == 0 && rstd == nullptr) return FLN_ERR_NULL;  // phase 2 reads it
  if (residual != nullptr && sum_out == nullptr) return FLN_ERR_NULL;
  if (kind == FLN_LAYERNORM && qmode == 0 && mean == nullptr) return FLN_ERR_NULL;
  if (kind == FLN_RMSNORM && (beta != nullptr || mean != nullptr)) return FLN_ERR_ARG;
  const int es = io_dtype == FLN_F32 ? 4 : 2;
  if (cols % (16 / es) != 0) return FLN_ERR_UNSUPPORTED;
  if (!(is_aligned16(x) && is_aligned16(residual) && is_aligned16(sum_out) && is_aligned16(q) &&
        is_aligned16(gamma) && is_aligned16(beta)))
    return FLN_ERR_UNSUPPORTED;

  // A row count that does not fill the row slots of the pipelined plan (16-bit input, scale
  // known before the launch): all but the last few rows through that plan, those through the
  // register kernels; both fold their max |y| into the same word.
  if (qmode != 0 && io_dtype != FLN_F32 && !part) {
    const int64_t odd = fwd_fp8_pipeline_odd_rows(rows, (int)cols, residual != nullptr ? 2 : 1);
    const int64_t m = rows - odd;
    const size_t q_row = qmode == 4 ? (size_t)cols / 2 : (size_t)cols;
    const size_t bs_row = qmode == 3 ? (size_t)cols / 32 : (qmode == 4 ? (size_t)cols / 16 : 0);
    if (odd > 0 && ((size_t)m * q_row) % 16 == 0) {
      if (amax != nullptr && cudaMemsetAsync(amax, 0, sizeof(float), st) != cudaSuccess) return FLN_ERR_LAUNCH;
      int rc = fp8_entry(qmode, kind, x, residual, gamma, beta, q, sum_out, mean, rstd, amax, scale, scale_in,
                         row_scale, m, cols, io_dtype, eps, stream, block_scale, true);
      if (rc != FLN_OK) return rc;
      const size_t off = (size_t)m * (size_t)cols * (size_t)es;
      return fp8_entry(qmode, kind, static_cast<const unsigned char*>(x) + off,
                       residual != nullptr ? static_cast<const unsigned char*>(residual) + off : nullptr, gamma, beta,
                       static_cast<unsigned char*>(q) + (size_t)m * q_row,
                       sum_out != nullptr ? static_cast<unsigned char*>(sum_out) + off : nullptr,
                       mean != nullptr ? mean + m : nullptr, rstd != nullptr ? rstd + m : nullptr, amax, scale, scale_in,
                       row_scale != nullptr ? row_scale + m : nullptr, odd, cols, io_dtype, eps, stream,
                       block_scale != nullptr ? block_scale + (size_t)m * bs_row : nullptr, true);
    }
  }

  Fp8Params p;
  p.x = x;
  p.res = residual;
  p.gamma = gamma;
  p.beta = beta;
  p.q = q;
  p.sum_out = sum_out;
  p.mean = mean;
  p.rstd = rstd;
  p.amax = amax;
  p.scale = scale;
  p.scale_in = scale_in;
  p.row_scale = row_scale;
  p.block_scale = block_scale;
  p.rows = rows;
  p.cols = (int)cols;
  p.nv = 0;
  p.tpr = 0;
  p.log2_tpr = 0;
  p.eps = eps;
  // Large 16-bit problems: the normalization itself runs in the persistent pipelined forward --
  // all of the delayed-scale, per-row, MXFP8 and NVFP4 forms, phase 1 (sum, statistics, amax) of
  // the two-launch form.
  bool phase1_done = false;
  if (io_dtype != FLN_F32) {
    FwdParams f;
    f.x = x;
    f.res = residual;
    f.gamma = gamma;
    f.beta = beta;
    f.y = nullptr;
    f.sum_out = sum_out;
    f.mean = mean;
    f.rstd = rstd;
    f.rows = rows;
    f.cols = (int)cols;
    f.nv = 0;
    f.tpr = 0;
    f.log2_tpr = 0;
    f.eps = eps;
    f.sched = nullptr;
    f.wait_ns = 0;
    f.status = nullptr;
    f.fault = nullptr;
    f.q = qmode == 0 ? nullptr : q;
    f.scale_in = scale_in;
    f.amax = amax;
    f.block_scale = block_scale;
    f.row_scale = row_scale;
    f.keep_bits = nullptr;
    f.drop_seed = 0;
    f.drop_offset = 0;
    f.drop_threshold = 0;
    f.drop_scale = 1.f;
    if (amax != nullptr && !part && cudaMemsetAsync(amax, 0, sizeof(float), st) != cudaSuccess) return FLN_ERR_LAUNCH;
    const int rc = launch_fwd_pipeline_fp8(kind, io_dtype, qmode == 0 ? 1 : qmode, f, st);
    if (rc == FLN_OK) {
      if (qmode != 0) return FLN_OK;
      phase1_done = true;
    } else if (rc != FLN_PIPE_NOT_APPLICABLE) {
      return rc;
    }
  }
  // (a slice: the register kernels must not reset amax either; for these forms the flag means
  // nothing else)
  if (part && qmode != 0) phase1_done = true;
#define FLN_RUN(T)                                                                  \
  (kind == FLN_LAYERNORM ? run_fp8<T, FLN_LAYERNORM>(p, qmode, st, phase1_done)     \
                         : run_fp8<T, FLN_RMSNORM>(p, qmode, st, phase1_done))
  if (io_dtype == FLN_F32) return FLN_RUN(float);
  if (io_dtype == FLN_BF16) return FLN_RUN(__nv_bfloat16);
  return FLN_RUN(__half);
#undef FLN_RUN
}

extern "C" int fln_norm_forward_fp8(int kind, const void* x, const void* residual,
                                    const void* gamma, const void* beta, void* q, void* sum_out,
                                    float* mean, float* rstd, float* amax, float* scale,
                                    int64_t rows, int64_t cols, int io_dtype, float eps,
                                    void* stream) {
  return fp8_entry(0, kind, x, residual, gamma, beta, q, sum_out, mean, rstd, amax, scale, nullptr, nullptr,
                   rows, cols, io_dtype, eps, stream);
}

extern "C" int fln_norm_forward_fp8_delayed(int kind, const void* x, const void* residual,
                                            const void* gamma, const void* beta, void* q, void* sum_out,
                                            float* mean, float* rstd, const float* scale_in,
                                            float* amax_out, int64_t rows, int64_t cols, int io_dtype,
                                            float eps, void* stream) {
  return fp8_entry(1, kind, x, residual, gamma, beta, q, sum_out, mean, rstd, amax_out, nullptr, scale_in,
                   nullptr, rows, cols, io_dtype, eps, stream);
}

extern "C" int fln_norm_forward_fp8_rowwise(int kind, const void* x, const void* residual,
                                            const void* gamma, const void* beta, void* q, void* sum_out,
                                            float* mean, float* rstd, float* row_scale, float* amax_out,
                                            int64_t rows, int64_t cols, int io_dtype, float eps,
                                            void* stream) {
  return fp8_entry(2, kind, x, residual, gamma, beta, q, sum_out, mean, rstd, amax_out, nullptr, nullptr,
                   row_scale, rows, cols, io_dtype, eps, stream);
}

extern "C" int fln_norm_forward_mxfp8(int kind, const void* x, const void* residual, const void* gamma,
                                      const void* beta, void* q, unsigned char* block_scale, void* sum_out,
                                      float* mean, float* rstd, float* amax_out, int64_t rows, int64_t cols,
                                      int io_dtype, float eps, void* stream) {
  return fp8_entry(3, kind, x, residual, gamma, beta, q, sum_out, mean, rstd, amax_out, nullptr, nullptr, nullptr,
                   rows, cols, io_dtype, eps, stream, block_scale);
}

extern "C" int fln_norm_forward_nvfp4(int kind, const void* x, const void* residual, const void* gamma,
                                      const void* beta, void* q, unsigned char* block_scale, void* sum_out,
                                      float* mean, float* rstd, const float* tensor_scale_in, float* amax_out,
                                      int64_t rows, int64_t cols, int io_dtype, float eps, void* stream) {
  if (cols > 0 && cols % 16 != 0) return FLN_ERR_UNSUPPORTED;
  return fp8_entry(4, kind, x, residual, gamma, beta, q, sum_out, mean, rstd, amax_out, nullptr, tensor_scale_in,
                   nullptr, rows, cols, io_dtype, eps, stream, block_scale);
}
