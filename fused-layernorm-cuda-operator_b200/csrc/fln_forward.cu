// Row-wise LayerNorm / RMSNorm forward for sm_100a.
//
// One row is owned by `tpr` consecutive threads; each thread keeps K vectors of the row in
// registers (as floats), so the row is read from HBM exactly once.  Statistics are fp32 and
// two-pass over the registers: the row is shifted by its first element, summed (warp
// butterfly + one hop through shared memory) to get the mean, centred, and the squared
// deviations are summed the same way.  At bf16 this kernel is bound by instruction issue,
// not by HBM, so the element loop is kept to a handful of instructions: paired widen /
// narrow conversions, fused multiply-adds, rsqrt.  The epilogue (affine, GELU, down-cast) is
// applied on the registers and stored with 16-byte vector stores.
//
// Stands in for layernorm_kernel / layernorm_gelu_kernel of the reference
// (csrc/layernorm_cuda_kernel.cu:39-92, 95-148), which read every row three times with
// scalar loads, and for layernorm_forward_kernel_optimized
// (csrc/layernorm_cuda_kernel_optimized.cu:54-168), whose mean/rstd outputs it keeps.
#include "fln_common.cuh"

namespace fln {


template <int K>
struct MaxThreads {
  static constexpr int value = K <= 2 ? 1024 : 512;
};

// FULL: the row is exactly K * tpr vectors long, every CTA holds only valid rows and a row
// spans at least a warp, so the body carries no bounds checks at all.
// MODE 0: general; 1: FULL; 2: FULL and the CTA owns exactly one row (one-barrier LayerNorm
// statistics, see below; the launcher selects it for fp32 rows only: in 16-bit types the extra
// registers make it slower).
template <typename TI, typename TO, int VEC, int K, int KIND, int ACT, int MODE>
__global__ void __launch_bounds__(MaxThreads<K>::value) norm_fwd_kernel(const FwdParams p) {
  constexpr bool FULL = MODE >= 1;
  constexpr bool ONE = MODE == 2 && KIND == FLN_LAYERNORM;
  __shared__ __align__(16) float s_red[3][32];

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

  // Launched with programmatic stream serialization (small grids, see launch_k), this CTA may
  // have started while the kernel in front of it in the stream was still draining: wait for
  // that kernel's memory before the first access, then let the kernel behind this one start
  // its CTAs.  Both are no-ops in an ordinary launch.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");

  float c = 0.f;  // shift: element 0 of the row (one extra broadcast load, in flight with the rest)
  if (KIND == FLN_LAYERNORM) {
    c = Cvt<TI>::to_f(ld_param<TI, 1>(xr).e[0]);
    if (p.res != nullptr)
      c = Cvt<TI>::to_f(Cvt<TI>::from_f(c + Cvt<TI>::to_f(ld_param<TI, 1>(reinterpret_cast<const TI*>(p.res) + base).e[0])));
  }
  // The whole row goes into registers as floats: HBM is read once.
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
    // s = x + residual, rounded to the I/O type first: that rounded value is what gets
    // normalized and what the residual stream carries on.
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
        st_stream<TI, VEC>(sr + (int64_t)iv * VEC, q);
        unpack<TI, VEC>(q, f[k]);
      }
    }
  }

  // ---- statistics: fp32, on the row shifted by its first element c ----------------------
  // The shift makes a constant row sum to exactly zero whatever its magnitude, and keeps
  // |mean| >> std from costing accuracy.  General form: two passes (sum, then centred sum of
  // squares), one reduction each.  ONE (the CTA owns exactly one row): both sums in one
  // reduction, variance = E[d^2] - E[d]^2; its relative error grows like eps (1 + 2 ms^2 /
  // var), so it is trusted only when the shift element lay within two standard deviations
  // of the mean, else the exact centred pass runs.  ms and var1 are bit-identical in every
  // thread of the CTA, so that branch and its barrier are uniform.
  float mean = 0.f, rstd = 0.f;
  bool need_second = true;
  if (KIND == FLN_LAYERNORM) {
    float a4[4] = {0.f, 0.f, 0.f, 0.f};  // independent chains: the adds are latency-bound
    float b4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (FULL || lane_r + k * tpr < p.nv) {  // padding vectors stay zero
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          f[k][i] -= c;
          a4[(k * VEC + i) & 3] += f[k][i];
          if (ONE) b4[(k * VEC + i) & 3] = fmaf(f[k][i], f[k][i], b4[(k * VEC + i) & 3]);
        }
      }
    }
    constexpr int NA = ONE ? 2 : 1;
    float a[NA];
    a[0] = (a4[0] + a4[1]) + (a4[2] + a4[3]);
    if (ONE) a[NA - 1] = (b4[0] + b4[1]) + (b4[2] + b4[3]);
    rowsum_warp<NA>(a, tpr, s_red[0]);
    if (tpr > 32) __syncthreads();
    rowsum_cta<NA>(a, tpr, s_red[0]);
    const float ms = a[0] * inv_n;  // mean of the shifted row
    mean = c + ms;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (FULL || lane_r + k * tpr < p.nv) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[k][i] -= ms;
      }
    }
    if (ONE) {
      const float var1 = fmaf(a[NA - 1], inv_n, -ms * ms);
      if (ms * ms <= 4.f * var1) {
        need_second = false;
        rstd = rsqrtf(var1 + p.eps);
      }
    }
  }
  if (need_second) {
    float q4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < K; ++k) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) q4[(k * VEC + i) & 3] = fmaf(f[k][i], f[k][i], q4[(k * VEC + i) & 3]);
    }
    float q[1] = {(q4[0] + q4[1]) + (q4[2] + q4[3])};
    rowsum_warp<1>(q, tpr, s_red[2]);
    if (tpr > 32) __syncthreads();
    rowsum_cta<1>(q, tpr, s_red[2]);
    rstd = rsqrtf(q[0] * inv_n + p.eps);
  }

  if (row_ok && lane_r == 0) {
    if (KIND == FLN_LAYERNORM && p.mean != nullptr) p.mean[row] = mean;
    if (p.rstd != nullptr) p.rstd[row] = rstd;
  }

  // ---- normalize + epilogue ---------------------------------------------------------
  const TI* __restrict__ gp = reinterpret_cast<const TI*>(p.gamma);
  const TI* __restrict__ bp = reinterpret_cast<const TI*>(p.beta);
  TO* __restrict__ yr = reinterpret_cast<TO*>(p.y) + base;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int iv = lane_r + k * tpr;
    if (FULL || (row_ok && iv < p.nv)) {
      float o[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = f[k][i] * rstd;
      if (gp != nullptr && bp != nullptr) {  // the usual case: one fma per element
        float g[VEC], b[VEC];
        unpack<TI, VEC>(ld_param<TI, VEC>(gp + (int64_t)iv * VEC), g);
        unpack<TI, VEC>(ld_param<TI, VEC>(bp + (int64_t)iv * VEC), b);
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] = fmaf(o[i], g[i], b[i]);
      } else if (gp != nullptr) {
        float g[VEC];
        unpack<TI, VEC>(ld_param<TI, VEC>(gp + (int64_t)iv * VEC), g);
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] *= g[i];
      } else if (bp != nullptr) {
        float b[VEC];
        unpack<TI, VEC>(ld_param<TI, VEC>(bp + (int64_t)iv * VEC), b);
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] += b[i];
      }
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = apply_act<ACT>(o[i]);
      Pack<TO, VEC> out;
      pack<TO, VEC>(o, out);
      st_stream<TO, VEC>(yr + (int64_t)iv * VEC, out);
    }
  }
}

// ----------------------------------------------------------------------------------------
// Fallback for rows that do not fit the register budget or are too ragged for it:
// one CTA per row, the row is re-read (it sits in L1/L2 after the first pass).
// ----------------------------------------------------------------------------------------
template <typename TI, typename TO, int KIND, int ACT>
__global__ void __launch_bounds__(512) norm_fwd_generic_kernel(const FwdParams p) {
  __shared__ float s_red[2][96];
  const int64_t row = blockIdx.x;
  const int64_t base = row * (int64_t)p.cols;
  const TI* __restrict__ xr = reinterpret_cast<const TI*>(p.x) + base;
  const TI* __restrict__ rr = p.res ? reinterpret_cast<const TI*>(p.res) + base : nullptr;
  TI* __restrict__ sr = p.res ? reinterpret_cast<TI*>(p.sum_out) + base : nullptr;
  const int tpr = blockDim.x;

  auto load_s = [&](int j) -> float {
    float v = Cvt<TI>::to_f(xr[j]);
    if (rr != nullptr) v = Cvt<TI>::to_f(Cvt<TI>::from_f(v + Cvt<TI>::to_f(rr[j])));
    return v;
  };

  float mean = 0.f, rstd;
  if (KIND == FLN_LAYERNORM) {
    float s1[1] = {0.f};
    for (int j = threadIdx.x; j < p.cols; j += blockDim.x) s1[0] += load_s(j);
    group_reduce_sum<1>(s1, tpr, s_red[0]);
    mean = s1[0] / (float)p.cols;
    float s2[1] = {0.f};
    for (int j = threadIdx.x; j < p.cols; j += blockDim.x) {
      float d = load_s(j) - mean;
      s2[0] += d * d;
    }
    group_reduce_sum<1>(s2, tpr, s_red[1]);
    rstd = 1.0f / sqrtf(s2[0] / (float)p.cols + p.eps);
  } else {
    float s2[1] = {0.f};
    for (int j = threadIdx.x; j < p.cols; j += blockDim.x) {
      float v = load_s(j);
      s2[0] += v * v;
    }
    group_reduce_sum<1>(s2, tpr, s_red[0]);
    rstd = 1.0f / sqrtf(s2[0] / (float)p.cols + p.eps);
  }
  if (threadIdx.x == 0) {
    if (KIND == FLN_LAYERNORM && p.mean != nullptr) p.mean[row] = mean;
    if (p.rstd != nullptr) p.rstd[row] = rstd;
  }
  const TI* __restrict__ gp = reinterpret_cast<const TI*>(p.gamma);
  const TI* __restrict__ bp = reinterpret_cast<const TI*>(p.beta);
  TO* __restrict__ yr = reinterpret_cast<TO*>(p.y) + base;
  for (int j = threadIdx.x; j < p.cols; j += blockDim.x) {
    float s = load_s(j);
    if (sr != nullptr) sr[j] = Cvt<TI>::from_f(s);
    float v = (s - mean) * rstd;
    if (gp != nullptr) v *= Cvt<TI>::to_f(gp[j]);
    if (bp != nullptr) v += Cvt<TI>::to_f(bp[j]);
    yr[j] = Cvt<TO>::from_f(apply_act<ACT>(v));
  }
}

// ----------------------------------------------------------------------------------------
// dispatch
// ----------------------------------------------------------------------------------------
// Grids of less than a wave are latency-bound: back to back in a stream, most of a call is the
// gap between one kernel's last CTA and the next kernel's first.  Such launches allow
// programmatic stream serialization: the next kernel's CTAs are placed while this one runs and
// wait at their griddepcontrol.wait (32 x 768 fp32 in a loop: 4.1 us per launch without).
template <typename KernelT>
static int launch_reg(KernelT kern, const FwdParams& p, int64_t grid, int threads, cudaStream_t st) {
  if (grid <= sm_count()) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) {
      cudaGetLastError();
      return FLN_ERR_LAUNCH;
    }
    return FLN_OK;
  }
  kern<<<(unsigned)grid, threads, 0, st>>>(p);
  FLN_CHECK_LAUNCH();
  return FLN_OK;
}

template <typename TI, typename TO, int VEC, int KIND, int ACT, int FULL>
static int launch_k(const FwdParams& p, const Plan& pl, int64_t grid, cudaStream_t st) {
  switch (pl.K) {
    case 1:
      return launch_reg(norm_fwd_kernel<TI, TO, VEC, 1, KIND, ACT, FULL>, p, grid, pl.threads, st);
    case 2:
      return launch_reg(norm_fwd_kernel<TI, TO, VEC, 2, KIND, ACT, FULL>, p, grid, pl.threads, st);
    case 4:
      return launch_reg(norm_fwd_kernel<TI, TO, VEC, 4, KIND, ACT, FULL>, p, grid, pl.threads, st);
    case 8:
      return launch_reg(norm_fwd_kernel<TI, TO, VEC, 8, KIND, ACT, FULL>, p, grid, pl.threads, st);
    default:
      return FLN_ERR_ARG;
  }
}

template <typename TI, typename TO, int KIND, int ACT>
static int launch_typed(FwdParams p, bool aligned, cudaStream_t st) {
  constexpr int FULL = 16 / (sizeof(TI) > sizeof(TO) ? sizeof(TI) : sizeof(TO));
  // a vector of the wider type must still be <= 16 bytes; alignment of the narrower
  // type's rows follows from cols % FULL == 0 only when its pointer is aligned as well,
  // which `aligned` asserts for every matrix pointer at 16 bytes.
  Plan pl = make_plan(false, p.rows, p.cols, (int)(16 / FULL), aligned);
  p.tpr = pl.tpr;
  p.log2_tpr = pl.log2_tpr;
  if (pl.generic) {
    norm_fwd_generic_kernel<TI, TO, KIND, ACT><<<(unsigned)p.rows, 512, 0, st>>>(p);
    FLN_CHECK_LAUNCH();
    return FLN_OK;
  }
  p.nv = p.cols / pl.vec;
  const int64_t grid = (p.rows + pl.rows_per_cta - 1) / pl.rows_per_cta;
  if (pl.vec == FULL) {
    const bool full = pl.tpr >= 32 && (int64_t)pl.K * pl.tpr == p.nv && p.rows % pl.rows_per_cta == 0;
    // fp32 LayerNorm, one row per CTA: both sums in one reduction (one barrier per row instead
    // of two; the exact centred pass still runs for rows whose first element lies far from
    // the mean).  Measured 161.8 vs 172.1 us at 32768 x 4096; in 16-bit types it is slower
    // (117.6 vs 108 us at 16384 x 8192 bf16: more registers per element), so it is fp32 only.
    if (full && pl.rows_per_cta == 1 && KIND == FLN_LAYERNORM && sizeof(TI) == 4)
      return launch_k<TI, TO, FULL, KIND, ACT, 2>(p, pl, grid, st);
    return full ? launch_k<TI, TO, FULL, KIND, ACT, 1>(p, pl, grid, st)
                : launch_k<TI, TO, FULL, KIND, ACT, 0>(p, pl, grid, st);
  }
  return launch_k<TI, TO, 1, KIND, ACT, 0>(p, pl, grid, st);
}

template <typename TI, typename TO>
static int launch_kind_act(int kind, int act, const FwdParams& p, bool aligned, cudaStream_t st) {
  if (kind == FLN_RMSNORM) {
    if (act != FLN_ACT_NONE) return FLN_ERR_UNSUPPORTED;
    return launch_typed<TI, TO, FLN_RMSNORM, FLN_ACT_NONE>(p, aligned, st);
  }
  switch (act) {
    case FLN_ACT_NONE:
      return launch_typed<TI, TO, FLN_LAYERNORM, FLN_ACT_NONE>(p, aligned, st);
    case FLN_ACT_GELU_TANH:
      return launch_typed<TI, TO, FLN_LAYERNORM, FLN_ACT_GELU_TANH>(p, aligned, st);
    case FLN_ACT_GELU_ERF:
      return launch_typed<TI, TO, FLN_LAYERNORM, FLN_ACT_GELU_ERF>(p, aligned, st);
  }
  return FLN_ERR_ARG;
}

}  // namespace fln

using namespace fln;

extern "C" int fln_norm_forward(int kind, const void* x, const void* residual, const void* gamma,
                                const void* beta, void* y, void* sum_out, float* mean,
                                float* rstd, int64_t rows, int64_t cols, int io_dtype,
                                int out_dtype, float eps, int act, void* stream) {
  if (kind != FLN_LAYERNORM && kind != FLN_RMSNORM) return FLN_ERR_ARG;
  if (act < FLN_ACT_NONE || act > FLN_ACT_GELU_ERF) return FLN_ERR_ARG;
  if (rows < 0 || cols <= 0 || cols > 0x7fffffff || rows > 0x7fffffff) return FLN_ERR_SHAPE;
  if (io_dtype != FLN_F32 && io_dtype != FLN_BF16 && io_dtype != FLN_F16) return FLN_ERR_DTYPE;
  if (out_dtype != io_dtype && !(io_dtype == FLN_F32 && out_dtype == FLN_BF16)) return FLN_ERR_DTYPE;
  if (rows == 0) return FLN_OK;
  if (x == nullptr || y == nullptr) return FLN_ERR_NULL;
  if (residual != nullptr && sum_out == nullptr) return FLN_ERR_NULL;
  if (kind == FLN_RMSNORM && (beta != nullptr || mean != nullptr)) return FLN_ERR_ARG;

  FwdParams p;
  p.x = x;
  p.res = residual;
  p.gamma = gamma;
  p.beta = beta;
  p.y = y;
  p.sum_out = sum_out;
  p.mean = mean;
  p.rstd = rstd;
  p.rows = rows;
  p.cols = (int)cols;
  p.nv = 0;
  p.tpr = 0;
  p.log2_tpr = 0;
  p.eps = eps;
  p.sched = nullptr;
  p.wait_ns = 0;
  p.status = nullptr;
  p.fault = nullptr;
  p.q = nullptr;
  p.scale_in = nullptr;
  p.amax = nullptr;
  p.block_scale = nullptr;
  p.row_scale = nullptr;
  p.keep_bits = nullptr;
  p.drop_seed = 0;
  p.drop_offset = 0;
  p.drop_threshold = 0;
  p.drop_scale = 1.f;
  const bool aligned = is_aligned16(x) && is_aligned16(y) && is_aligned16(residual) &&
                       is_aligned16(sum_out) && is_aligned16(gamma) && is_aligned16(beta);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (kind == FLN_RMSNORM && act != FLN_ACT_NONE) return FLN_ERR_UNSUPPORTED;
  if (aligned) {
    // large aligned problems: persistent bulk-async pipeline
    // (a row count that does not fill the fast plan's row slots: all but the last few rows
    // through that plan, those through the register kernels below)
    const int64_t odd = fwd_pipeline_odd_rows(act, io_dtype, out_dtype, p);
    if (odd > 0) {
      FwdParams pm = p;
      pm.rows = p.rows - odd;
      const int rc = launch_fwd_pipeline(kind, act, io_dtype, out_dtype, pm, st);
      if (rc != FLN_PIPE_NOT_APPLICABLE) {
        if (rc != FLN_OK) return rc;
        const size_t es_in = io_dtype == FLN_F32 ? 4 : 2, es_out = out_dtype == FLN_F32 ? 4 : 2;
        const size_t off = (size_t)pm.rows * (size_t)p.cols;
        p.x = static_cast<const unsigned char*>(p.x) + off * es_in;
        if (p.res != nullptr) p.res = static_cast<const unsigned char*>(p.res) + off * es_in;
        if (p.sum_out != nullptr) p.sum_out = static_cast<unsigned char*>(p.sum_out) + off * es_in;
        p.y = static_cast<unsigned char*>(p.y) + off * es_out;
        if (p.mean != nullptr) p.mean += pm.rows;
        if (p.rstd != nullptr) p.rstd += pm.rows;
        p.rows = odd;
      }
    }
    if (odd == 0 || p.rows != odd) {
      const int rc = launch_fwd_pipeline(kind, act, io_dtype, out_dtype, p, st);
      if (rc != FLN_PIPE_NOT_APPLICABLE) return rc;
    }
  }
  if (io_dtype == FLN_F32 && out_dtype == FLN_F32)
    return launch_kind_act<float, float>(kind, act, p, aligned, st);
  if (io_dtype == FLN_F32 && out_dtype == FLN_BF16)
    return launch_kind_act<float, __nv_bfloat16>(kind, act, p, aligned, st);
  if (io_dtype == FLN_BF16)
    return launch_kind_act<__nv_bfloat16, __nv_bfloat16>(kind, act, p, aligned, st);
  return launch_kind_act<__half, __half>(kind, act, p, aligned, st);
}

extern "C" int fln_layernorm_forward(const void* x, const void* gamma, const void* beta, void* y,
                                     float* mean, float* rstd, int64_t rows, int64_t cols,
                                     int dtype, float eps, void* stream) {
  return fln_norm_forward(FLN_LAYERNORM, x, nullptr, gamma, beta, y, nullptr, mean, rstd, rows,
                          cols, dtype, dtype, eps, FLN_ACT_NONE, stream);
}

extern "C" int fln_layernorm_gelu_forward(const void* x, const void* gamma, const void* beta,
                                          void* y, int64_t rows, int64_t cols, int dtype,
                                          float eps, int approximate, void* stream) {
  if (approximate != FLN_ACT_GELU_TANH && approximate != FLN_ACT_GELU_ERF) return FLN_ERR_ARG;
  return fln_norm_forward(FLN_LAYERNORM, x, nullptr, gamma, beta, y, nullptr, nullptr, nullptr,
                          rows, cols, dtype, dtype, eps, approximate, stream);
}
