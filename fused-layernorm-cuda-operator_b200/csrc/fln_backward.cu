// LayerNorm / RMSNorm backward for sm_100a.
//
// Stage 1 (norm_bwd_kernel): persistent CTAs walk row groups.  A row is owned by `tpr`
// threads, each holding K vectors of dy and x in registers (HBM read once), gamma packed
// in registers for the whole kernel.  Per row: one fused two-value reduction
// (sum g*xhat, sum g), then dx.  Every thread also accumulates dy*xhat and dy for its own
// columns in fp32 registers across all rows it visits and finally writes one partial row
// to the workspace.
// Stage 2 (colreduce_kernel): sums the partial rows column-wise in a fixed order, so
// dgamma/dbeta are deterministic (no float atomics).
//
// The reference declares this operation (layernorm_backward_cuda, csrc/layernorm.h:24-32)
// and calls it (csrc/layernorm_cuda.cpp:135-138) but ships no kernel; its intended
// semantics are those of torch autograd through nn.LayerNorm (tests/test_layernorm.py:128-178).
#include <type_traits>

#include "fln_common.cuh"

namespace fln {


template <int C>  // columns per thread
struct BwdMaxThreads {
  static constexpr int value = C <= 4 ? 1024 : (C <= 16 ? 512 : 256);
};

template <typename T, int VEC, int K, int KIND>
__global__ void __launch_bounds__(BwdMaxThreads<VEC * K>::value) norm_bwd_kernel(const BwdParams p) {
  constexpr int NR = KIND == FLN_LAYERNORM ? 2 : 1;
  __shared__ __align__(16) float s_red[2][NR * 32];

  const int tid = threadIdx.x;
  const int tpr = p.tpr;
  const int lane_r = tid & (tpr - 1);
  const int row_in_cta = tid >> p.log2_tpr;
  const int rows_per_cta = blockDim.x >> p.log2_tpr;
  const float inv_n = 1.0f / (float)p.cols;

  float acc_g[K][VEC], acc_b[K][VEC];
  float gam[K][VEC];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int iv = lane_r + k * tpr;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      acc_g[k][i] = 0.f;
      acc_b[k][i] = 0.f;
      gam[k][i] = 1.f;
    }
    if (p.gamma != nullptr && iv < p.nv) {
      Pack<T, VEC> g = ld_param<T, VEC>(reinterpret_cast<const T*>(p.gamma) + (int64_t)iv * VEC);
#pragma unroll
      for (int i = 0; i < VEC; ++i) gam[k][i] = Cvt<T>::to_f(g.e[i]);
    }
  }

  int parity = 0;
  for (int64_t rg = blockIdx.x; rg < p.row_groups; rg += gridDim.x, parity ^= 1) {
    const int64_t row = rg * rows_per_cta + row_in_cta;
    const bool row_ok = row < p.rows;
    const int64_t base = row * (int64_t)p.cols;
    const T* __restrict__ dyr = reinterpret_cast<const T*>(p.dy) + base;
    const T* __restrict__ xr = reinterpret_cast<const T*>(p.x) + base;

    Pack<T, VEC> rdy[K], rx[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int iv = lane_r + k * tpr;
      if (row_ok && iv < p.nv) {
        rdy[k] = ld_stream<T, VEC>(dyr + (int64_t)iv * VEC);
        rx[k] = ld_stream<T, VEC>(xr + (int64_t)iv * VEC);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          rdy[k].e[i] = Cvt<T>::from_f(0.f);
          rx[k].e[i] = Cvt<T>::from_f(0.f);
        }
      }
    }
    float mean = 0.f, rstd = 0.f;
    if (row_ok) {
      if (KIND == FLN_LAYERNORM) mean = __ldg(p.mean + row);
      rstd = __ldg(p.rstd + row);
    }

    // xhat and dy as floats; padding lanes carry dy == 0 so they add nothing anywhere
    float xh[K][VEC], dyf[K][VEC];
    float ra[2] = {0.f, 0.f}, rb[2] = {0.f, 0.f};  // two chains per sum
#pragma unroll
    for (int k = 0; k < K; ++k) {
      unpack<T, VEC>(rdy[k], dyf[k]);
      unpack<T, VEC>(rx[k], xh[k]);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        xh[k][i] = (xh[k][i] - mean) * rstd;
        const float g = dyf[k][i] * gam[k][i];
        ra[i & 1] = fmaf(g, xh[k][i], ra[i & 1]);
        if (KIND == FLN_LAYERNORM) rb[i & 1] += g;
      }
    }
    float red[NR];
    red[0] = ra[0] + ra[1];
    if (KIND == FLN_LAYERNORM) red[NR - 1] = rb[0] + rb[1];
    rowsum_warp<NR>(red, tpr, s_red[parity]);
    if (tpr > 32) __syncthreads();
    rowsum_cta<NR>(red, tpr, s_red[parity]);
    // dx = rstd * ((g - c2) - xhat * c1): the subtraction comes first so that rows whose g
    // is (nearly) constant cancel exactly instead of leaving a rounding residue times rstd
    const float nc1 = -(red[0] * inv_n);
    const float c2 = KIND == FLN_LAYERNORM ? red[NR - 1] * inv_n : 0.f;

    if (p.dx != nullptr) {
      T* __restrict__ dxr = reinterpret_cast<T*>(p.dx) + base;
      const T* __restrict__ drr =
          p.dres_in ? reinterpret_cast<const T*>(p.dres_in) + base : nullptr;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int iv = lane_r + k * tpr;
        if (row_ok && iv < p.nv) {
          float o[VEC];
#pragma unroll
          for (int i = 0; i < VEC; ++i)
            o[i] = rstd * fmaf(xh[k][i], nc1, dyf[k][i] * gam[k][i] - c2);
          if (drr != nullptr) {
            float d[VEC];
            unpack<T, VEC>(ld_stream<T, VEC>(drr + (int64_t)iv * VEC), d);
#pragma unroll
            for (int i = 0; i < VEC; ++i) o[i] += d[i];
          }
          Pack<T, VEC> out;
          pack<T, VEC>(o, out);
          st_stream<T, VEC>(dxr + (int64_t)iv * VEC, out);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        acc_g[k][i] = fmaf(dyf[k][i], xh[k][i], acc_g[k][i]);
        if (KIND == FLN_LAYERNORM) acc_b[k][i] += dyf[k][i];
      }
    }
  }

  if (p.partials != nullptr) {
    const int64_t prow = (int64_t)blockIdx.x * rows_per_cta + row_in_cta;
    float* __restrict__ pg = p.partials + prow * (int64_t)(NR * p.cols);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int iv = lane_r + k * tpr;
      if (iv < p.nv) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          pg[(int64_t)iv * VEC + i] = acc_g[k][i];
          if (KIND == FLN_LAYERNORM) pg[p.cols + (int64_t)iv * VEC + i] = acc_b[k][i];
        }
      }
    }
  }
}

// ----------------------------------------------------------------------------------------
// Fallback for long or ragged rows: dx with one CTA per row (row re-read from L1/L2), and
// a column-walking kernel that builds the same partial-row layout for stage 2.
// ----------------------------------------------------------------------------------------
template <typename T, int KIND>
__global__ void __launch_bounds__(512) norm_bwd_dx_generic_kernel(const BwdParams p) {
  constexpr int NR = KIND == FLN_LAYERNORM ? 2 : 1;
  __shared__ float s_red[NR * 32];
  const int64_t row = blockIdx.x;
  const int64_t base = row * (int64_t)p.cols;
  const T* __restrict__ dyr = reinterpret_cast<const T*>(p.dy) + base;
  const T* __restrict__ xr = reinterpret_cast<const T*>(p.x) + base;
  const T* __restrict__ gp = reinterpret_cast<const T*>(p.gamma);
  const float mean = KIND == FLN_LAYERNORM ? p.mean[row] : 0.f;
  const float rstd = p.rstd[row];
  float red[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) red[r] = 0.f;
  for (int j = threadIdx.x; j < p.cols; j += blockDim.x) {
    float g = Cvt<T>::to_f(dyr[j]) * (gp ? Cvt<T>::to_f(gp[j]) : 1.f);
    float xh = (Cvt<T>::to_f(xr[j]) - mean) * rstd;
    red[0] += g * xh;
    if (KIND == FLN_LAYERNORM) red[NR - 1] += g;
  }
  group_reduce_sum<NR>(red, blockDim.x, s_red);
  const float inv_n = 1.0f / (float)p.cols;
  const float c1 = red[0] * inv_n;
  const float c2 = KIND == FLN_LAYERNORM ? red[NR - 1] * inv_n : 0.f;
  T* __restrict__ dxr = reinterpret_cast<T*>(p.dx) + base;
  const T* __restrict__ drr = p.dres_in ? reinterpret_cast<const T*>(p.dres_in) + base : nullptr;
  for (int j = threadIdx.x; j < p.cols; j += blockDim.x) {
    float g = Cvt<T>::to_f(dyr[j]) * (gp ? Cvt<T>::to_f(gp[j]) : 1.f);
    float xh = (Cvt<T>::to_f(xr[j]) - mean) * rstd;
    float o = rstd * (g - c2 - xh * c1);
    if (drr != nullptr) o += Cvt<T>::to_f(drr[j]);
    dxr[j] = Cvt<T>::from_f(o);
  }
}

// grid = (ceil(cols/256), P): CTA (bx, by) sums rows by, by+P, ... for its 256 columns.
template <typename T, int KIND>
__global__ void __launch_bounds__(256) norm_bwd_cols_generic_kernel(const BwdParams p) {
  constexpr int NR = KIND == FLN_LAYERNORM ? 2 : 1;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= p.cols) return;
  float ag = 0.f, ab = 0.f;
  for (int64_t row = blockIdx.y; row < p.rows; row += gridDim.y) {
    const int64_t idx = row * (int64_t)p.cols + j;
    float dy = Cvt<T>::to_f(reinterpret_cast<const T*>(p.dy)[idx]);
    float mean = KIND == FLN_LAYERNORM ? p.mean[row] : 0.f;
    float xh = (Cvt<T>::to_f(reinterpret_cast<const T*>(p.x)[idx]) - mean) * p.rstd[row];
    ag += dy * xh;
    ab += dy;
  }
  float* pg = p.partials + (int64_t)blockIdx.y * (NR * p.cols);
  pg[j] = ag;
  if (KIND == FLN_LAYERNORM) pg[p.cols + j] = ab;
}

// ----------------------------------------------------------------------------------------
// Rows too long for the register-resident and pipelined kernels (more than 16 columns per
// thread of a 512-thread CTA), but aligned and a whole number of 16-byte vectors: the same
// two kernels with 128-bit accesses.
//   dx:   one CTA per row; pass 1 streams the row for the two row sums, pass 2 re-reads it
//         (L1 / L2 hits: a row is at most a few hundred KB) and writes dx.
//   cols: thread = one vector of columns, CTA row blockIdx.y walks rows y, y + P, ... with
//         four rows in flight and writes one partial row.
// dy and x are read from HBM twice (10 instead of 6 bytes per element).  Running the pair
// over L2-sized chunks of rows so that the second read hits the 126 MB L2 was measured
// slower (744 vs 480 us at 21824 x 12288 bf16): every chunk has to add into the partial rows,
// and that traffic outweighs the saved reads.
// ----------------------------------------------------------------------------------------
template <typename T, int KIND>
__global__ void __launch_bounds__(512) norm_bwd_dx_wide_kernel(const BwdParams p) {
  constexpr int VEC = 16 / sizeof(T);
  constexpr int NR = KIND == FLN_LAYERNORM ? 2 : 1;
  __shared__ float s_red[NR * 32];
  const int64_t row = blockIdx.x;
  const int64_t base = row * (int64_t)p.cols;
  const T* __restrict__ dyr = reinterpret_cast<const T*>(p.dy) + base;
  const T* __restrict__ xr = reinterpret_cast<const T*>(p.x) + base;
  const T* __restrict__ gp = reinterpret_cast<const T*>(p.gamma);
  const float mean = KIND == FLN_LAYERNORM ? __ldg(p.mean + row) : 0.f;
  const float rstd = __ldg(p.rstd + row);
  const int nv = p.cols / VEC;
  float r0[2] = {0.f, 0.f}, r1[2] = {0.f, 0.f};
  for (int v = threadIdx.x; v < nv; v += blockDim.x) {
    float dy[VEC], xx[VEC], gg[VEC];
    unpack<T, VEC>(ld_plain<T, VEC>(dyr + (int64_t)v * VEC), dy);
    unpack<T, VEC>(ld_plain<T, VEC>(xr + (int64_t)v * VEC), xx);
    if (gp != nullptr) {
      unpack<T, VEC>(ld_param<T, VEC>(gp + (int64_t)v * VEC), gg);
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) gg[e] = 1.f;
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const float g = dy[e] * gg[e];
      r0[e & 1] = fmaf(g, (xx[e] - mean) * rstd, r0[e & 1]);
      if (KIND == FLN_LAYERNORM) r1[e & 1] += g;
    }
  }
  float red[NR];
  red[0] = r0[0] + r0[1];
  if (KIND == FLN_LAYERNORM) red[NR - 1] = r1[0] + r1[1];
  group_reduce_sum<NR>(red, blockDim.x, s_red);
  const float inv_n = 1.0f / (float)p.cols;
  const float nc1 = -(red[0] * inv_n);
  const float c2 = KIND == FLN_LAYERNORM ? red[NR - 1] * inv_n : 0.f;
  T* __restrict__ dxr = reinterpret_cast<T*>(p.dx) + base;
  const T* __restrict__ drr = p.dres_in ? reinterpret_cast<const T*>(p.dres_in) + base : nullptr;
  for (int v = threadIdx.x; v < nv; v += blockDim.x) {
    float dy[VEC], xx[VEC], gg[VEC], o[VEC];
    unpack<T, VEC>(ld_plain<T, VEC>(dyr + (int64_t)v * VEC), dy);
    unpack<T, VEC>(ld_plain<T, VEC>(xr + (int64_t)v * VEC), xx);
    if (gp != nullptr) {
      unpack<T, VEC>(ld_param<T, VEC>(gp + (int64_t)v * VEC), gg);
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) gg[e] = 1.f;
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) o[e] = rstd * fmaf((xx[e] - mean) * rstd, nc1, dy[e] * gg[e] - c2);
    if (drr != nullptr) {
      float dr[VEC];
      unpack<T, VEC>(ld_stream<T, VEC>(drr + (int64_t)v * VEC), dr);
#pragma unroll
      for (int e = 0; e < VEC; ++e) o[e] += dr[e];
    }
    Pack<T, VEC> out;
    pack<T, VEC>(o, out);
    st_stream<T, VEC>(dxr + (int64_t)v * VEC, out);
  }
}

template <typename T, int KIND>
__global__ void __launch_bounds__(128) norm_bwd_cols_wide_kernel(const BwdParams p) {
  constexpr int VEC = 16 / sizeof(T);
  constexpr int NR = KIND == FLN_LAYERNORM ? 2 : 1;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= p.cols / VEC) return;
  const T* __restrict__ dyp = reinterpret_cast<const T*>(p.dy) + (int64_t)v * VEC;
  const T* __restrict__ xp = reinterpret_cast<const T*>(p.x) + (int64_t)v * VEC;
  float ag[VEC], ab[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    ag[e] = 0.f;
    ab[e] = 0.f;
  }
  const int64_t end = p.rows;
  const int64_t step = gridDim.y;
  int64_t r = blockIdx.y;
  for (; r + 3 * step < end; r += 4 * step) {
    Pack<T, VEC> qd[4], qx[4];
    float mu[4], rs[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t rr = r + j * step;
      qd[j] = ld_stream<T, VEC>(dyp + rr * (int64_t)p.cols);
      qx[j] = ld_stream<T, VEC>(xp + rr * (int64_t)p.cols);
      mu[j] = KIND == FLN_LAYERNORM ? __ldg(p.mean + rr) : 0.f;
      rs[j] = __ldg(p.rstd + rr);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float dy[VEC], xx[VEC];
      unpack<T, VEC>(qd[j], dy);
      unpack<T, VEC>(qx[j], xx);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        ag[e] = fmaf(dy[e], (xx[e] - mu[j]) * rs[j], ag[e]);
        if (KIND == FLN_LAYERNORM) ab[e] += dy[e];
      }
    }
  }
  for (; r < end; r += step) {
    float dy[VEC], xx[VEC];
    unpack<T, VEC>(ld_stream<T, VEC>(dyp + r * (int64_t)p.cols), dy);
    unpack<T, VEC>(ld_stream<T, VEC>(xp + r * (int64_t)p.cols), xx);
    const float mu = KIND == FLN_LAYERNORM ? __ldg(p.mean + r) : 0.f;
    const float rs = __ldg(p.rstd + r);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      ag[e] = fmaf(dy[e], (xx[e] - mu) * rs, ag[e]);
      if (KIND == FLN_LAYERNORM) ab[e] += dy[e];
    }
  }
  float* __restrict__ pg = p.partials + (int64_t)blockIdx.y * (NR * p.cols) + (int64_t)v * VEC;
#pragma unroll
  for (int e = 0; e < VEC; e += 4) {
    *reinterpret_cast<float4*>(pg + e) = make_float4(ag[e], ag[e + 1], ag[e + 2], ag[e + 3]);
    if (KIND == FLN_LAYERNORM)
      *reinterpret_cast<float4*>(pg + p.cols + e) = make_float4(ab[e], ab[e + 1], ab[e + 2], ab[e + 3]);
  }
}

// ----------------------------------------------------------------------------------------
// Stage 2: out[c] = sum_p partials[p][c], c in [0, ncols).  A warp reads 32 consecutive
// columns of one partial row; the 8 warps of a CTA take rows p = w, w+8, ... and their
// sums are combined in warp order.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) colreduce_kernel(const float* __restrict__ partials, int P,
                                                        int ncols, int cols, float* dgb_f32,
                                                        T* dgamma, T* dbeta) {
  __shared__ float s[8][33];
  const int lane = threadIdx.x & 31;
  const int w = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  if (c < ncols) {
    int pidx = w;
    for (; pidx + 24 < P; pidx += 32) {
      a0 += partials[(int64_t)pidx * ncols + c];
      a1 += partials[(int64_t)(pidx + 8) * ncols + c];
      a2 += partials[(int64_t)(pidx + 16) * ncols + c];
      a3 += partials[(int64_t)(pidx + 24) * ncols + c];
    }
    for (; pidx < P; pidx += 8) a0 += partials[(int64_t)pidx * ncols + c];
  }
  s[w][lane] = (a0 + a1) + (a2 + a3);
  __syncthreads();
  if (w == 0 && c < ncols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += s[i][lane];
    if (dgb_f32 != nullptr) dgb_f32[c] = t;
    if (c < cols) {
      if (dgamma != nullptr) dgamma[c] = Cvt<T>::from_f(t);
    } else {
      if (dbeta != nullptr) dbeta[c - cols] = Cvt<T>::from_f(t);
    }
  }
}

// The same sum for 16-byte aligned partial rows with ncols % 4 == 0: a CTA owns 64 columns
// (16 float4 lanes) and splits the partial rows over 16 groups, so a thread issues all of
// its (up to 10 per pass) independent 16-byte loads before the first add.  With 148 partial
// rows the whole workspace is requested in one round trip instead of five.  The order of the
// adds is fixed: rows rg, rg + 16, ... inside a thread, then the 16 groups in order.
template <typename T>
__global__ void __launch_bounds__(256) colreduce4_kernel(const float* __restrict__ partials, int P,
                                                         int ncols, int cols, float* dgb_f32,
                                                         T* dgamma, T* dbeta) {
  __shared__ __align__(16) float s[16][64];
  const int cl = threadIdx.x & 15;
  const int rg = threadIdx.x >> 4;
  const int c4 = blockIdx.x * 16 + cl;  // float4 column
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c4 * 4 < ncols) {
    const float4* __restrict__ src = reinterpret_cast<const float4*>(partials) + c4;
    const int64_t stride4 = ncols >> 2;
    for (int base = rg; base < P; base += 160) {
      float4 v[10];
#pragma unroll
      for (int j = 0; j < 10; ++j) {
        const int idx = base + j * 16;
        v[j] = idx < P ? __ldcg(src + (int64_t)idx * stride4) : make_float4(0.f, 0.f, 0.f, 0.f);
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
  *reinterpret_cast<float4*>(&s[rg][cl * 4]) = acc;
  __syncthreads();
  const int c = blockIdx.x * 64 + threadIdx.x;
  if (threadIdx.x < 64 && c < ncols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) t += s[i][threadIdx.x];
    if (dgb_f32 != nullptr) dgb_f32[c] = t;
    if (c < cols) {
      if (dgamma != nullptr) dgamma[c] = Cvt<T>::from_f(t);
    } else {
      if (dbeta != nullptr) dbeta[c - cols] = Cvt<T>::from_f(t);
    }
  }
}

template <typename T>
static void launch_colreduce(const float* partials, int P, int ncols, int cols, float* dgb_f32, T* dgamma,
                             T* dbeta, cudaStream_t st) {
  if ((ncols & 3) == 0 && is_aligned16(partials) && P >= 16) {
    colreduce4_kernel<T><<<(ncols / 4 + 15) / 16, 256, 0, st>>>(partials, P, ncols, cols, dgb_f32, dgamma, dbeta);
  } else {
    colreduce_kernel<T><<<(ncols + 31) / 32, 256, 0, st>>>(partials, P, ncols, cols, dgb_f32, dgamma, dbeta);
  }
}

template <typename T>
__global__ void cast_from_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = Cvt<T>::from_f(src[i]);
}

// ----------------------------------------------------------------------------------------
// host
// ----------------------------------------------------------------------------------------
struct BwdLaunch {
  Plan pl;
  int64_t row_groups;
  int64_t grid;  // stage-1 CTAs (register path) or partial rows (generic path)
  int64_t P;     // partial rows in the workspace
  bool wide;     // long aligned rows: the vectorised, L2-chunked pair of kernels
};

template <typename T, int VEC, int K, int KIND>
static int occupancy_of(int threads) {
  // cached per (device, log2 threads); the query is too slow for the latency-bound shapes
  static int cache[16][12];
  int dev = 0;
  cudaGetDevice(&dev);
  int l2 = 0;
  while ((1 << l2) < threads) ++l2;
  if (dev < 0 || dev >= 16 || l2 >= 12) return 1;
  int v = cache[dev][l2];
  if (v == 0) {
    int nb = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, norm_bwd_kernel<T, VEC, K, KIND>,
                                                      threads, 0) != cudaSuccess ||
        nb < 1)
      nb = 1;
    cache[dev][l2] = v = nb;
  }
  return v;
}

template <typename T, int KIND>
static int occupancy_dispatch(const Plan& pl) {
  constexpr int FULL = 16 / sizeof(T);
#define FLN_OCC(V, KK)  \
  if (pl.vec == V && pl.K == KK) return occupancy_of<T, V, KK, KIND>(pl.threads);
  FLN_OCC(FULL, 1) FLN_OCC(FULL, 2) FLN_OCC(FULL, 4) FLN_OCC(1, 1) FLN_OCC(1, 2) FLN_OCC(1, 4)
  FLN_OCC(1, 8)
  if (FULL * 8 <= 32) {
    if (pl.vec == FULL && pl.K == 8) return occupancy_of<T, (FULL * 8 <= 32 ? FULL : 1), 8, KIND>(pl.threads);
  }
#undef FLN_OCC
  return 1;
}

template <typename T, int KIND>
static BwdLaunch plan_bwd(int64_t rows, int cols, bool aligned) {
  BwdLaunch L;
  L.pl = make_plan(true, rows, cols, (int)sizeof(T), aligned);
  L.wide = false;
  if (L.pl.generic && aligned && cols % (16 / (int)sizeof(T)) == 0 && (cols * (int64_t)sizeof(T)) % 16 == 0) {
    // vectorised long-row kernels: enough partial rows for about 8 CTAs of 128 threads per SM
    L.wide = true;
    L.row_groups = rows;
    const int nv = cols / (16 / (int)sizeof(T));
    int64_t Pw = 8LL * sm_count() / ((nv + 127) / 128);
    if (Pw < 1) Pw = 1;
    if (Pw > 256) Pw = 256;
    L.P = rows < Pw ? rows : Pw;
    L.grid = rows;
    return L;
  }
  if (L.pl.generic) {
    L.row_groups = rows;
    int64_t Pmax = 4LL * sm_count() / ((cols + 255) / 256);
    if (Pmax < 1) Pmax = 1;
    if (Pmax > 1024) Pmax = 1024;
    L.P = rows < Pmax ? rows : Pmax;
    L.grid = rows;
    return L;
  }
  L.row_groups = (rows + L.pl.rows_per_cta - 1) / L.pl.rows_per_cta;
  int64_t cap = (int64_t)usable_sms() * occupancy_dispatch<T, KIND>(L.pl);
  L.grid = L.row_groups < cap ? L.row_groups : cap;
  L.P = L.grid * L.pl.rows_per_cta;
  return L;
}

template <typename T, int VEC, int KIND>
static int launch_bwd_k(const BwdParams& p, const BwdLaunch& L, cudaStream_t st) {
  const unsigned g = (unsigned)L.grid;
  const int t = L.pl.threads;
  switch (L.pl.K) {
    case 1:
      norm_bwd_kernel<T, VEC, 1, KIND><<<g, t, 0, st>>>(p);
      break;
    case 2:
      norm_bwd_kernel<T, VEC, 2, KIND><<<g, t, 0, st>>>(p);
      break;
    case 4:
      norm_bwd_kernel<T, VEC, 4, KIND><<<g, t, 0, st>>>(p);
      break;
    case 8:
      if (VEC * 8 <= 32) {
        norm_bwd_kernel<T, (VEC * 8 <= 32 ? VEC : 1), 8, KIND><<<g, t, 0, st>>>(p);
        break;
      }
      return FLN_ERR_ARG;
    default:
      return FLN_ERR_ARG;
  }
  FLN_CHECK_LAUNCH();
  return FLN_OK;
}

// partial_rows_out != nullptr: stage 1 only -- the partial rows stay in the workspace, their
// number is reported, and nothing is reduced (fln_norm_backward_partial)
template <typename T, int KIND>
static int run_bwd(BwdParams p, void* dgamma, void* dbeta, float* dgb_f32, void* workspace,
                   size_t workspace_bytes, bool aligned, cudaStream_t st, int64_t* partial_rows_out = nullptr) {
  constexpr int NR = KIND == FLN_LAYERNORM ? 2 : 1;
  constexpr int FULL = 16 / sizeof(T);
  const bool defer = partial_rows_out != nullptr;
  const bool want_params = defer || dgamma != nullptr || dbeta != nullptr || dgb_f32 != nullptr;
  // large aligned problems: persistent bulk-async pipeline for stage 1
  const int dt = sizeof(T) == 4 ? FLN_F32 : (std::is_same<T, __half>::value ? FLN_F16 : FLN_BF16);
  // A row count that does not fill the fast plan's row slots: all but the last few rows through
  // that plan (its column sums left as partial rows), those few through the register kernels
  // (stage 1 only, their partial rows behind the pipeline's), then one column reduce over both.
  const int64_t odd = aligned ? bwd_pipeline_odd_rows(dt, p.rows, p.cols, p.dres_in != nullptr) : 0;
  if (odd > 0) {
    const int64_t main_rows = p.rows - odd;
    const int64_t mainP = bwd_pipeline_partial_rows(KIND, dt, main_rows, p.cols, p.dres_in != nullptr);
    const size_t head = (size_t)mainP * NR * p.cols * sizeof(float);
    if (mainP > 0 && (!want_params || (workspace != nullptr && is_aligned16(workspace) && workspace_bytes >= head))) {
      BwdParams pm = p;
      pm.rows = main_rows;
      pm.partials = want_params ? reinterpret_cast<float*>(workspace) : nullptr;
      pm.sync = nullptr;  // no column reduce in the kernel's tail
      bool reduced = false;
      int rc = launch_bwd_pipeline(KIND, dt, pm, st, &reduced);
      if (rc != FLN_PIPE_NOT_APPLICABLE) {
        if (rc != FLN_OK) return rc;
        BwdParams pr = p;
        const size_t off = (size_t)main_rows * (size_t)p.cols * sizeof(T);
        pr.dy = static_cast<const unsigned char*>(p.dy) + off;
        pr.x = static_cast<const unsigned char*>(p.x) + off;
        if (p.dres_in != nullptr) pr.dres_in = static_cast<const unsigned char*>(p.dres_in) + off;
        if (p.dx != nullptr) pr.dx = static_cast<unsigned char*>(p.dx) + off;
        if (p.mean != nullptr) pr.mean = p.mean + main_rows;
        pr.rstd = p.rstd + main_rows;
        pr.rows = odd;
        int64_t extra = 0;
        rc = want_params ? run_bwd<T, KIND>(pr, nullptr, nullptr, nullptr, static_cast<unsigned char*>(workspace) + head,
                                            workspace_bytes - head, aligned, st, &extra)
                         : run_bwd<T, KIND>(pr, nullptr, nullptr, nullptr, nullptr, 0, aligned, st, nullptr);
        if (rc != FLN_OK) return rc;
        if (defer) {
          *partial_rows_out = mainP + extra;
          return FLN_OK;
        }
        if (want_params) {
          launch_colreduce<T>(pm.partials, (int)(mainP + extra), NR * p.cols, p.cols, dgb_f32,
                              reinterpret_cast<T*>(dgamma), reinterpret_cast<T*>(dbeta), st);
          FLN_CHECK_LAUNCH();
        }
        return FLN_OK;
      }
    }
  }
  const int64_t pipeP =
      aligned ? bwd_pipeline_partial_rows(KIND, dt, p.rows, p.cols, p.dres_in != nullptr) : 0;
  if (pipeP > 0) {
    if (want_params) {
      const size_t need = (size_t)pipeP * NR * p.cols * sizeof(float);
      if (workspace == nullptr || workspace_bytes < need || !is_aligned16(workspace))
        return FLN_ERR_WORKSPACE;
      p.partials = reinterpret_cast<float*>(workspace);
      // a workspace of the full advertised size has one more 16-byte slot behind the
      // partial rows: the word the fused column reduce synchronises on
      const size_t sync_off = (need + 15) & ~(size_t)15;
      if (!defer && workspace_bytes >= sync_off + 16) {
        p.sync = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(workspace) + sync_off);
        p.dgb_f32 = dgb_f32;
        p.dgamma = dgamma;
        p.dbeta = dbeta;
      }
    } else {
      p.partials = nullptr;
    }
    bool reduced = false;
    const int rc = launch_bwd_pipeline(KIND, dt, p, st, &reduced);
    if (rc != FLN_PIPE_NOT_APPLICABLE) {
      if (rc != FLN_OK) return rc;
      if (defer) {
        *partial_rows_out = pipeP;
        return FLN_OK;
      }
      if (want_params && !reduced) {
        const int ncols = NR * p.cols;
        launch_colreduce<T>(p.partials, (int)pipeP, ncols, p.cols, dgb_f32, reinterpret_cast<T*>(dgamma),
                            reinterpret_cast<T*>(dbeta), st);
        FLN_CHECK_LAUNCH();
      }
      return FLN_OK;
    }
  }
  BwdLaunch L = plan_bwd<T, KIND>(p.rows, p.cols, aligned);
  if (want_params) {
    const size_t need = (size_t)L.P * NR * p.cols * sizeof(float);
    if (workspace == nullptr || workspace_bytes < need) return FLN_ERR_WORKSPACE;
    if (!is_aligned16(workspace)) return FLN_ERR_WORKSPACE;
    p.partials = reinterpret_cast<float*>(workspace);
  } else {
    p.partials = nullptr;
  }
  p.tpr = L.pl.tpr;
  p.log2_tpr = L.pl.log2_tpr;
  p.row_groups = L.row_groups;
  if (L.wide) {
    constexpr int VEC = 16 / (int)sizeof(T);
    const unsigned gx = (unsigned)((p.cols / VEC + 127) / 128);
    if (p.dx != nullptr) {
      norm_bwd_dx_wide_kernel<T, KIND><<<(unsigned)p.rows, 512, 0, st>>>(p);
      FLN_CHECK_LAUNCH();
    }
    if (want_params) {
      norm_bwd_cols_wide_kernel<T, KIND><<<dim3(gx, (unsigned)L.P), 128, 0, st>>>(p);
      FLN_CHECK_LAUNCH();
    }
  } else if (L.pl.generic) {
    if (p.dx != nullptr) {
      norm_bwd_dx_generic_kernel<T, KIND><<<(unsigned)p.rows, 512, 0, st>>>(p);
      FLN_CHECK_LAUNCH();
    }
    if (want_params) {
      dim3 grid((p.cols + 255) / 256, (unsigned)L.P);
      norm_bwd_cols_generic_kernel<T, KIND><<<grid, 256, 0, st>>>(p);
      FLN_CHECK_LAUNCH();
    }
  } else {
    p.nv = p.cols / L.pl.vec;
    int rc = L.pl.vec == FULL ? launch_bwd_k<T, FULL, KIND>(p, L, st)
                              : launch_bwd_k<T, 1, KIND>(p, L, st);
    if (rc != FLN_OK) return rc;
  }
  if (defer) {
    *partial_rows_out = L.P;
    return FLN_OK;
  }
  if (want_params) {
    const int ncols = NR * p.cols;
    launch_colreduce<T>(p.partials, (int)L.P, ncols, p.cols, dgb_f32, reinterpret_cast<T*>(dgamma),
                        reinterpret_cast<T*>(dbeta), st);
    FLN_CHECK_LAUNCH();
  }
  return FLN_OK;
}

template <typename T>
static size_t ws_bytes_typed(int64_t rows, int cols) {
  // LayerNorm needs the larger layout; RMSNorm callers may pass the same size
  BwdLaunch L = plan_bwd<T, FLN_LAYERNORM>(rows, cols, true);
  BwdLaunch L1 = plan_bwd<T, FLN_LAYERNORM>(rows, cols, false);
  BwdLaunch R = plan_bwd<T, FLN_RMSNORM>(rows, cols, true);
  BwdLaunch R1 = plan_bwd<T, FLN_RMSNORM>(rows, cols, false);
  int64_t P = L.P;
  if (L1.P > P) P = L1.P;
  if (R.P > P) P = R.P;
  if (R1.P > P) P = R1.P;
  const int dt = sizeof(T) == 4 ? FLN_F32 : (std::is_same<T, __half>::value ? FLN_F16 : FLN_BF16);
  const int64_t pipeP = bwd_pipeline_partial_rows(FLN_LAYERNORM, dt, rows, cols, false);
  if (pipeP > P) P = pipeP;
  const int64_t pipeP3 = bwd_pipeline_partial_rows(FLN_LAYERNORM, dt, rows, cols, true);
  if (pipeP3 > P) P = pipeP3;
  // a row count split between the pipeline and the register kernels (run_bwd): both sets of
  // partial rows
  for (int with_dres = 0; with_dres <= 1; ++with_dres) {
    const int64_t odd = bwd_pipeline_odd_rows(dt, rows, cols, with_dres != 0);
    if (odd > 0) {
      const int64_t mainP = bwd_pipeline_partial_rows(FLN_LAYERNORM, dt, rows - odd, cols, with_dres != 0);
      const BwdLaunch O = plan_bwd<T, FLN_LAYERNORM>(odd, cols, true);
      const BwdLaunch O1 = plan_bwd<T, FLN_RMSNORM>(odd, cols, true);
      int64_t oddP = O.P > O1.P ? O.P : O1.P;
      // (the forced-pipeline test hook sends even these few rows through the pipeline)
      const int64_t oddPipe = bwd_pipeline_partial_rows(FLN_LAYERNORM, dt, odd, cols, with_dres != 0);
      if (oddPipe > oddP) oddP = oddPipe;
      const int64_t both = mainP + oddP;
      if (both > P) P = both;
    }
  }
  // + one 16-byte slot for the grid barrier of the fused column reduce
  return (((size_t)P * 2 * cols * sizeof(float) + 15) & ~(size_t)15) + 16;
}

}  // namespace fln

using namespace fln;

extern "C" size_t fln_backward_workspace_bytes(int64_t rows, int64_t cols, int dtype) {
  if (rows <= 0 || cols <= 0 || cols > 0x7fffffff) return 0;
  switch (dtype) {
    case FLN_F32:
      return ws_bytes_typed<float>(rows, (int)cols);
    case FLN_BF16:
      return ws_bytes_typed<__nv_bfloat16>(rows, (int)cols);
    case FLN_F16:
      return ws_bytes_typed<__half>(rows, (int)cols);
  }
  return 0;
}

static int norm_backward_impl(int kind, const void* dy, const void* x, const float* mean,
                              const float* rstd, const void* gamma, const void* dres_in,
                              void* dx, void* dgamma, void* dbeta, float* dgb_f32,
                              void* workspace, size_t workspace_bytes, int64_t rows,
                              int64_t cols, int dtype, void* stream, int64_t* partial_rows_out) {
  if (kind != FLN_LAYERNORM && kind != FLN_RMSNORM) return FLN_ERR_ARG;
  if (rows < 0 || cols <= 0 || cols > 0x7fffffff || rows > 0x7fffffff) return FLN_ERR_SHAPE;
  if (dtype != FLN_F32 && dtype != FLN_BF16 && dtype != FLN_F16) return FLN_ERR_DTYPE;
  if (kind == FLN_RMSNORM && dbeta != nullptr) return FLN_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (rows == 0) {
    if (partial_rows_out != nullptr) {
      *partial_rows_out = 0;  // nothing to sum
      return FLN_OK;
    }
    // an empty shard contributes zeros
    const size_t es = dtype == FLN_F32 ? 4 : 2;
    if (dgamma) cudaMemsetAsync(dgamma, 0, (size_t)cols * es, st);
    if (dbeta) cudaMemsetAsync(dbeta, 0, (size_t)cols * es, st);
    if (dgb_f32) cudaMemsetAsync(dgb_f32, 0, (size_t)cols * 4 * (kind == FLN_LAYERNORM ? 2 : 1), st);
    FLN_CHECK_LAUNCH();
    return FLN_OK;
  }
  if (dy == nullptr || x == nullptr || rstd == nullptr) return FLN_ERR_NULL;
  if (kind == FLN_LAYERNORM && mean == nullptr) return FLN_ERR_NULL;
  if (dres_in != nullptr && dx == nullptr) return FLN_ERR_NULL;
  if (partial_rows_out == nullptr && dx == nullptr && dgamma == nullptr && dbeta == nullptr && dgb_f32 == nullptr)
    return FLN_OK;

  BwdParams p;
  p.dy = dy;
  p.x = x;
  p.mean = mean;
  p.rstd = rstd;
  p.gamma = gamma;
  p.dres_in = dres_in;
  p.dx = dx;
  p.partials = nullptr;
  p.rows = rows;
  p.row_groups = 0;
  p.cols = (int)cols;
  p.nv = 0;
  p.tpr = 0;
  p.log2_tpr = 0;
  p.sync = nullptr;
  p.token = 0;
  p.dgb_f32 = nullptr;
  p.dgamma = nullptr;
  p.dbeta = nullptr;
  p.wait_ns = 0;
  p.status = nullptr;
  p.fault = nullptr;
  const bool aligned = is_aligned16(dy) && is_aligned16(x) && is_aligned16(gamma) &&
                       is_aligned16(dres_in) && is_aligned16(dx);
#define FLN_RUN(T)                                                                         \
  (kind == FLN_LAYERNORM                                                                   \
       ? run_bwd<T, FLN_LAYERNORM>(p, dgamma, dbeta, dgb_f32, workspace, workspace_bytes,  \
                                   aligned, st, partial_rows_out)                          \
       : run_bwd<T, FLN_RMSNORM>(p, dgamma, dbeta, dgb_f32, workspace, workspace_bytes,    \
                                 aligned, st, partial_rows_out))
  if (dtype == FLN_F32) return FLN_RUN(float);
  if (dtype == FLN_BF16) return FLN_RUN(__nv_bfloat16);
  return FLN_RUN(__half);
#undef FLN_RUN
}

extern "C" int fln_norm_backward(int kind, const void* dy, const void* x, const float* mean,
                                 const float* rstd, const void* gamma, const void* dres_in,
                                 void* dx, void* dgamma, void* dbeta, float* dgb_f32,
                                 void* workspace, size_t workspace_bytes, int64_t rows,
                                 int64_t cols, int dtype, void* stream) {
  return norm_backward_impl(kind, dy, x, mean, rstd, gamma, dres_in, dx, dgamma, dbeta, dgb_f32, workspace,
                            workspace_bytes, rows, cols, dtype, stream, nullptr);
}

extern "C" int fln_norm_backward_partial(int kind, const void* dy, const void* x, const float* mean,
                                         const float* rstd, const void* gamma, const void* dres_in,
                                         void* dx, void* workspace, size_t workspace_bytes,
                                         int64_t rows, int64_t cols, int dtype, void* stream,
                                         int64_t* partial_rows) {
  if (partial_rows == nullptr || workspace == nullptr) return FLN_ERR_NULL;
  *partial_rows = 0;
  return norm_backward_impl(kind, dy, x, mean, rstd, gamma, dres_in, dx, nullptr, nullptr, nullptr, workspace,
                            workspace_bytes, rows, cols, dtype, stream, partial_rows);
}

extern "C" int fln_layernorm_backward(const void* dy, const void* x, const float* mean,
                                      const float* rstd, const void* gamma, void* dx,
                                      void* dgamma, void* dbeta, void* workspace,
                                      size_t workspace_bytes, int64_t rows, int64_t cols,
                                      int dtype, void* stream) {
  return fln_norm_backward(FLN_LAYERNORM, dy, x, mean, rstd, gamma, nullptr, dx, dgamma, dbeta,
                           nullptr, workspace, workspace_bytes, rows, cols, dtype, stream);
}

extern "C" int fln_cast_from_f32(const float* src, void* dst, int64_t n, int dtype, void* stream) {
  if (n < 0) return FLN_ERR_SHAPE;
  if (n == 0) return FLN_OK;
  if (src == nullptr || dst == nullptr) return FLN_ERR_NULL;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((n + 255) / 256);
  switch (dtype) {
    case FLN_F32:
      cast_from_f32_kernel<float><<<grid, 256, 0, st>>>(src, reinterpret_cast<float*>(dst), n);
      break;
    case FLN_BF16:
      cast_from_f32_kernel<__nv_bfloat16>
          <<<grid, 256, 0, st>>>(src, reinterpret_cast<__nv_bfloat16*>(dst), n);
      break;
    case FLN_F16:
      cast_from_f32_kernel<__half><<<grid, 256, 0, st>>>(src, reinterpret_cast<__half*>(dst), n);
      break;
    default:
      return FLN_ERR_DTYPE;
  }
  FLN_CHECK_LAUNCH();
  return FLN_OK;
}

extern "C" int fln_sum_rows_f32(const float* rows_in, int64_t n_rows, int64_t ncols, float* out_f32,
                                void* out_cast, int dtype, void* stream) {
  if (n_rows <= 0 || ncols <= 0 || ncols > INT32_MAX || n_rows > INT32_MAX) return FLN_ERR_SHAPE;
  if (rows_in == nullptr || (out_f32 == nullptr && out_cast == nullptr)) return FLN_ERR_NULL;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int nc = (int)ncols, P = (int)n_rows;
  // the column-reduce kernels with every column on the "dgamma" side of the split
  switch (dtype) {
    case FLN_F32:
      launch_colreduce<float>(rows_in, P, nc, nc, out_f32, reinterpret_cast<float*>(out_cast), nullptr, st);
      break;
    case FLN_BF16:
      launch_colreduce<__nv_bfloat16>(rows_in, P, nc, nc, out_f32, reinterpret_cast<__nv_bfloat16*>(out_cast),
                                      nullptr, st);
      break;
    case FLN_F16:
      launch_colreduce<__half>(rows_in, P, nc, nc, out_f32, reinterpret_cast<__half*>(out_cast), nullptr, st);
      break;
    default:
      return FLN_ERR_DTYPE;
  }
  FLN_CHECK_LAUNCH();
  return FLN_OK;
}
