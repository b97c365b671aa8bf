// Fused dropout -> residual add -> LayerNorm / RMSNorm forward, and the dropout backward.
//
// The step in front of the normalization in a pre-norm transformer block:
//     d = dropout(x, p)           kept elements scaled by 1 / (1 - p), rounded to the I/O type
//     s = d + residual            rounded to the I/O type, written out (the residual stream)
//     y = norm(s) * gamma + beta
// in one pass over x and residual (8 bytes per element in 16-bit types plus one mask bit,
// instead of the 18 of the three unfused kernels).  The reference has no counterpart; the
// semantics are those of the unfused torch composition, with the mask taken from this
// generator.
//
// Random numbers: Philox4x32-10 (Salmon, Moraes, Dror, Shaw, SC'11), counter-based, so the
// mask is a pure function of (seed, offset, element index) and the backward can either read
// the stored keep bits or regenerate them.  One 128-bit output serves 8 consecutive elements,
// 16 bits each:
//     group g = (row * cols + col) / 8        counter = {g lo, g hi, offset lo, offset hi}
//     key = {seed lo, seed hi}                element j of the group: bits 16 (j & 1) .. of word j >> 1
//     keep iff that 16-bit value >= threshold,  threshold = round(p * 65536) in [0, 65535]
// so the drop probability is threshold / 65536 and the scale 65536 / (65536 - threshold).
// keep_bits holds one byte per group (bit j = element j kept).
//
// Kernel: one CTA per row, the row in registers (K groups of 8 elements per thread), two-pass
// statistics.  Non-persistent, so the hardware scheduler balances the rows.
#include "fln_philox.cuh"

namespace fln {

struct DropParams {
  const void* x;
  const void* res;    // may be NULL
  const void* gamma;  // may be NULL
  const void* beta;   // may be NULL
  void* y;
  void* sum_out;
  float* mean;  // may be NULL
  float* rstd;  // may be NULL
  unsigned char* keep_bits;  // may be NULL
  int64_t rows;
  int cols;
  int groups;  // cols / 8
  float eps;
  float scale;
  unsigned int threshold;
  unsigned long long seed, offset;
  int64_t row0;  // first row this launch takes (the rows before it went through the pipelined forward)
};

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    unpack<T, 8>(ld_stream<T, 8>(p), f);
  } else {
    float a[4], b[4];
    unpack<T, 4>(ld_stream<T, 4>(p), a);
    unpack<T, 4>(ld_stream<T, 4>(p + 4), b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[i] = a[i];
      f[4 + i] = b[i];
    }
  }
}
template <typename T>
__device__ __forceinline__ void load8_param(const T* p, float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    unpack<T, 8>(ld_param<T, 8>(p), f);
  } else {
    float a[4], b[4];
    unpack<T, 4>(ld_param<T, 4>(p), a);
    unpack<T, 4>(ld_param<T, 4>(p + 4), b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[i] = a[i];
      f[4 + i] = b[i];
    }
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    Pack<T, 8> q;
    pack<T, 8>(f, q);
    st_stream<T, 8>(p, q);
  } else {
    float a[4] = {f[0], f[1], f[2], f[3]}, b[4] = {f[4], f[5], f[6], f[7]};
    Pack<T, 4> qa, qb;
    pack<T, 4>(a, qa);
    pack<T, 4>(b, qb);
    st_stream<T, 4>(p, qa);
    st_stream<T, 4>(p + 4, qb);
  }
}
// the value a round trip through T leaves
template <typename T>
__device__ __forceinline__ float round_io(float v) {
  return Cvt<T>::to_f(Cvt<T>::from_f(v));
}

// sum over the CTA, result in every thread (same order everywhere)
__device__ __forceinline__ float cta_sum(float v, float* smem) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  const int nw = blockDim.x >> 5;
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += smem[i];
  __syncthreads();
  return t;
}

template <typename T, int K, int KIND>
__global__ void __launch_bounds__(K == 4 ? 512 : 1024) dropout_add_norm_fwd_kernel(const DropParams p) {
  __shared__ float s_red[32];
  const int64_t row = p.row0 + blockIdx.x;
  const int64_t base = row * (int64_t)p.cols;
  const T* __restrict__ x = reinterpret_cast<const T*>(p.x) + base;
  const T* __restrict__ res = p.res != nullptr ? reinterpret_cast<const T*>(p.res) + base : nullptr;
  float f[K][8];
  bool ok[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int gi = threadIdx.x + k * blockDim.x;  // group inside the row
    ok[k] = gi < p.groups;
    if (ok[k]) {
      load8<T>(x + (int64_t)gi * 8, f[k]);
      const unsigned long long g = (unsigned long long)(base / 8) + (unsigned long long)gi;
      const unsigned int m = p.threshold == 0 ? 0xffu : keep_mask8(g, p.seed, p.offset, p.threshold);
      if (p.keep_bits != nullptr) p.keep_bits[g] = (unsigned char)m;
#pragma unroll
      for (int j = 0; j < 8; ++j) f[k][j] = ((m >> j) & 1u) ? round_io<T>(f[k][j] * p.scale) : 0.f;
      if (res != nullptr) {
        float r[8];
        load8<T>(res + (int64_t)gi * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[k][j] = round_io<T>(f[k][j] + r[j]);
      }
      if (p.sum_out != nullptr) store8<T>(reinterpret_cast<T*>(p.sum_out) + base + (int64_t)gi * 8, f[k]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[k][j] = 0.f;
    }
  }
  const float inv_n = 1.0f / (float)p.cols;
  float mean = 0.f;
  if (KIND == FLN_LAYERNORM) {
    float a = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) a += f[k][j];
    mean = cta_sum(a, s_red) * inv_n;
  }
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    if (ok[k]) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[k][j] -= mean;
        q = fmaf(f[k][j], f[k][j], q);
      }
    }
  }
  const float rstd = rsqrtf(fmaf(cta_sum(q, s_red), inv_n, p.eps));
  if (threadIdx.x == 0) {
    if (KIND == FLN_LAYERNORM && p.mean != nullptr) p.mean[row] = mean;
    if (p.rstd != nullptr) p.rstd[row] = rstd;
  }
#pragma unroll
  for (int k = 0; k < K; ++k) {
    if (ok[k]) {
      const int gi = threadIdx.x + k * blockDim.x;
      float g8[8], b8[8], o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        g8[j] = 1.f;
        b8[j] = 0.f;
      }
      if (p.gamma != nullptr) load8_param<T>(reinterpret_cast<const T*>(p.gamma) + (int64_t)gi * 8, g8);
      if (p.beta != nullptr) load8_param<T>(reinterpret_cast<const T*>(p.beta) + (int64_t)gi * 8, b8);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = fmaf(f[k][j] * rstd, g8[j], b8[j]);
      store8<T>(reinterpret_cast<T*>(p.y) + base + (int64_t)gi * 8, o);
    }
  }
}

// d_x = d_sum * scale where kept, 0 where dropped; the mask is read (keep_bits) or regenerated
template <typename T>
__global__ void __launch_bounds__(256) dropout_bwd_kernel(const T* __restrict__ d_sum, const unsigned char* __restrict__ keep_bits,
                                                          T* __restrict__ d_x, int64_t groups, float scale,
                                                          unsigned int threshold, unsigned long long seed,
                                                          unsigned long long offset) {
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += (int64_t)gridDim.x * blockDim.x) {
    float f[8];
    load8<T>(d_sum + g * 8, f);
    const unsigned int m = keep_bits != nullptr
                               ? keep_bits[g]
                               : (threshold == 0 ? 0xffu : keep_mask8((unsigned long long)g, seed, offset, threshold));
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = ((m >> j) & 1u) ? f[j] * scale : 0.f;
    store8<T>(d_x + g * 8, f);
  }
}

static bool drop_prob(float p, unsigned int* threshold, float* scale) {
  if (!(p >= 0.f) || !(p < 1.f)) return false;
  double t = (double)p * 65536.0 + 0.5;
  unsigned int thr = (unsigned int)t;
  if (thr > 65535u) thr = 65535u;
  *threshold = thr;
  *scale = (float)(65536.0 / (65536.0 - (double)thr));
  return true;
}

template <typename T, int KIND>
static int launch_drop_fwd(const DropParams& p, cudaStream_t st) {
  // K groups of 8 elements per thread: enough threads for about 256 per row, at most 1024.
  // (The kernel is bound by instruction issue: 52 thread instructions per element, three
  // quarters of the issue slots taken at 16384 x 4096 bf16, 122 us.  Tried and slower: one group
  // per thread on 512 threads, full occupancy at 31 registers, 142.5 us; a second table in
  // place of the second barrier of cta_sum, 128 us.)
  int K = 1;
  while (K < 4 && (p.groups + K - 1) / K > 256) K <<= 1;
  int threads = (p.groups + K - 1) / K;
  threads = (threads + 31) & ~31;
  if (threads > (K == 4 ? 512 : 1024)) return FLN_ERR_UNSUPPORTED;
  const unsigned grid = (unsigned)(p.rows - p.row0);
  switch (K) {
    case 1:
      dropout_add_norm_fwd_kernel<T, 1, KIND><<<grid, threads, 0, st>>>(p);
      break;
    case 2:
      dropout_add_norm_fwd_kernel<T, 2, KIND><<<grid, threads, 0, st>>>(p);
      break;
    default:
      dropout_add_norm_fwd_kernel<T, 4, KIND><<<grid, threads, 0, st>>>(p);
      break;
  }
  FLN_CHECK_LAUNCH();
  return FLN_OK;
}

}  // namespace fln

using namespace fln;

extern "C" int fln_dropout_add_norm_forward(int kind, const void* x, const void* residual, const void* gamma,
                                            const void* beta, void* y, void* sum_out, float* mean, float* rstd,
                                            unsigned char* keep_bits, int64_t rows, int64_t cols, int dtype,
                                            float eps, float p, unsigned long long seed, unsigned long long offset,
                                            void* stream) {
  if (kind != FLN_LAYERNORM && kind != FLN_RMSNORM) return FLN_ERR_ARG;
  if (rows < 0 || cols <= 0 || cols > 0x7fffffff || rows > 0x7fffffff) return FLN_ERR_SHAPE;
  if (dtype != FLN_F32 && dtype != FLN_BF16 && dtype != FLN_F16) return FLN_ERR_DTYPE;
  DropParams q;
  if (!drop_prob(p, &q.threshold, &q.scale)) return FLN_ERR_ARG;
  if (kind == FLN_RMSNORM && (beta != nullptr || mean != nullptr)) return FLN_ERR_ARG;
  if (rows == 0) return FLN_OK;
  if (x == nullptr || y == nullptr) return FLN_ERR_NULL;
  if (residual != nullptr && sum_out == nullptr) return FLN_ERR_NULL;
  // groups of 8 elements, 16-byte vectors; rows of up to 4 x 512 groups
  if (cols % 8 != 0 || cols > 16384) return FLN_ERR_UNSUPPORTED;
  if (!(is_aligned16(x) && is_aligned16(residual) && is_aligned16(y) && is_aligned16(sum_out) && is_aligned16(gamma) &&
        is_aligned16(beta)))
    return FLN_ERR_UNSUPPORTED;
  q.x = x;
  q.res = residual;
  q.gamma = gamma;
  q.beta = beta;
  q.y = y;
  q.sum_out = sum_out;
  q.mean = mean;
  q.rstd = rstd;
  q.keep_bits = keep_bits;
  q.rows = rows;
  q.cols = (int)cols;
  q.groups = (int)(cols / 8);
  q.eps = eps;
  q.seed = seed;
  q.offset = offset;
  q.row0 = 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype != FLN_F32) {
    // large 16-bit problems: the persistent pipelined forward with the dropout folded in
    FwdParams f;
    f.x = x;
    f.res = residual;
    f.gamma = gamma;
    f.beta = beta;
    f.y = y;
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
    f.q = nullptr;
    f.scale_in = nullptr;
    f.amax = nullptr;
    f.block_scale = nullptr;
    f.row_scale = nullptr;
    f.keep_bits = keep_bits;
    f.drop_seed = seed;
    f.drop_offset = offset;
    f.drop_threshold = q.threshold;
    f.drop_scale = q.scale;
    // a row count that does not fill the pipelined plan's row slots: all but the last few rows
    // through that plan, those through the kernel below (the mask depends on the element's
    // position in the whole tensor, so both parts draw the bits an unsplit call would)
    const int64_t odd = fwd_fp8_pipeline_odd_rows(rows, (int)cols, residual != nullptr ? 2 : 1);
    if (odd > 0) {
      f.rows = rows - odd;
      const int rc = launch_fwd_pipeline_dropout(kind, dtype, f, st);
      if (rc == FLN_OK) q.row0 = rows - odd;
      else if (rc != FLN_PIPE_NOT_APPLICABLE) return rc;
      f.rows = rows;
    }
    if (q.row0 == 0) {
      const int rc = launch_fwd_pipeline_dropout(kind, dtype, f, st);
      if (rc != FLN_PIPE_NOT_APPLICABLE) return rc;
    }
  }
#define FLN_RUN(T) \
  (kind == FLN_LAYERNORM ? launch_drop_fwd<T, FLN_LAYERNORM>(q, st) : launch_drop_fwd<T, FLN_RMSNORM>(q, st))
  if (dtype == FLN_F32) return FLN_RUN(float);
  if (dtype == FLN_BF16) return FLN_RUN(__nv_bfloat16);
  return FLN_RUN(__half);
#undef FLN_RUN
}

extern "C" int fln_dropout_backward(const void* d_sum, const unsigned char* keep_bits, void* d_x, int64_t rows,
                                    int64_t cols, int dtype, float p, unsigned long long seed,
                                    unsigned long long offset, void* stream) {
  if (rows < 0 || cols <= 0 || cols > 0x7fffffff || rows > 0x7fffffff) return FLN_ERR_SHAPE;
  if (dtype != FLN_F32 && dtype != FLN_BF16 && dtype != FLN_F16) return FLN_ERR_DTYPE;
  unsigned int threshold;
  float scale;
  if (!drop_prob(p, &threshold, &scale)) return FLN_ERR_ARG;
  if (rows == 0) return FLN_OK;
  if (d_sum == nullptr || d_x == nullptr) return FLN_ERR_NULL;
  if (cols % 8 != 0 || !is_aligned16(d_sum) || !is_aligned16(d_x)) return FLN_ERR_UNSUPPORTED;
  const int64_t groups = rows * (cols / 8);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int64_t blocks = (groups + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  switch (dtype) {
    case FLN_F32:
      dropout_bwd_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(reinterpret_cast<const float*>(d_sum), keep_bits,
                                                                  reinterpret_cast<float*>(d_x), groups, scale, threshold,
                                                                  seed, offset);
      break;
    case FLN_BF16:
      dropout_bwd_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
          reinterpret_cast<const __nv_bfloat16*>(d_sum), keep_bits, reinterpret_cast<__nv_bfloat16*>(d_x), groups, scale,
          threshold, seed, offset);
      break;
    default:
      dropout_bwd_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(reinterpret_cast<const __half*>(d_sum), keep_bits,
                                                                   reinterpret_cast<__half*>(d_x), groups, scale,
                                                                   threshold, seed, offset);
      break;
  }
  FLN_CHECK_LAUNCH();
  return FLN_OK;
}
