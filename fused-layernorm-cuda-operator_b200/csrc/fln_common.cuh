// Shared device/host helpers for the sm_100a row-normalization kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "fln_b200.h"

namespace fln {

// ------------------------------------------------------------------------------------
// element conversion
// ------------------------------------------------------------------------------------
template <typename T>
struct Cvt;
template <>
struct Cvt<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <>
struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct Cvt<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};

// ------------------------------------------------------------------------------------
// VEC elements moved by one load/store instruction (2, 4, 8 or 16 bytes)
// ------------------------------------------------------------------------------------
template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) Pack {
  T e[VEC];
};

template <int BYTES>
struct Raw;
template <>
struct Raw<16> {
  using type = uint4;
};
template <>
struct Raw<8> {
  using type = uint2;
};
template <>
struct Raw<4> {
  using type = unsigned int;
};
template <>
struct Raw<2> {
  using type = unsigned short;
};
template <>
struct Raw<1> {
  using type = unsigned char;
};

// streaming load: the matrices are touched once per kernel, keep them out of the way of
// gamma/beta in L1/L2
template <typename T, int VEC>
__device__ __forceinline__ Pack<T, VEC> ld_stream(const T* p) {
  using R = typename Raw<sizeof(T) * VEC>::type;
  Pack<T, VEC> out;
  *reinterpret_cast<R*>(&out) = __ldcs(reinterpret_cast<const R*>(p));
  return out;
}
// cached read-only load (parameters, re-read by every CTA)
template <typename T, int VEC>
__device__ __forceinline__ Pack<T, VEC> ld_param(const T* p) {
  using R = typename Raw<sizeof(T) * VEC>::type;
  Pack<T, VEC> out;
  *reinterpret_cast<R*>(&out) = __ldg(reinterpret_cast<const R*>(p));
  return out;
}
// plain load (data that a later kernel of ours wants to find in L2)
template <typename T, int VEC>
__device__ __forceinline__ Pack<T, VEC> ld_plain(const T* p) {
  using R = typename Raw<sizeof(T) * VEC>::type;
  Pack<T, VEC> out;
  *reinterpret_cast<R*>(&out) = *reinterpret_cast<const R*>(p);
  return out;
}
template <typename T, int VEC>
__device__ __forceinline__ void st_stream(T* p, const Pack<T, VEC>& v) {
  using R = typename Raw<sizeof(T) * VEC>::type;
  __stcs(reinterpret_cast<R*>(p), *reinterpret_cast<const R*>(&v));
}
template <typename T, int VEC>
__device__ __forceinline__ void st_plain(T* p, const Pack<T, VEC>& v) {
  using R = typename Raw<sizeof(T) * VEC>::type;
  *reinterpret_cast<R*>(p) = *reinterpret_cast<const R*>(&v);
}

// ------------------------------------------------------------------------------------
// whole-vector conversions.  The hot loops are issue-bound at bf16, so a 16-bit pair is
// widened with one shift / one mask and narrowed with one paired round-to-nearest-even
// convert, instead of element-by-element conversions.
// ------------------------------------------------------------------------------------
template <typename T, int VEC>
__device__ __forceinline__ void unpack(const Pack<T, VEC>& p, float (&f)[VEC]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = Cvt<T>::to_f(p.e[i]);
  } else if constexpr (VEC >= 2) {
    const unsigned int* w = reinterpret_cast<const unsigned int*>(&p);
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        f[2 * j] = __uint_as_float(w[j] << 16);
        f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      } else {
        float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        f[2 * j] = t.x;
        f[2 * j + 1] = t.y;
      }
    }
  } else {
    f[0] = Cvt<T>::to_f(p.e[0]);
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void pack(const float (&f)[VEC], Pack<T, VEC>& p) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) p.e[i] = Cvt<T>::from_f(f[i]);
  } else if constexpr (VEC >= 2) {
    unsigned int* w = reinterpret_cast<unsigned int*>(&p);
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
        w[j] = *reinterpret_cast<unsigned int*>(&t);
      } else {
        __half2 t = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
        w[j] = *reinterpret_cast<unsigned int*>(&t);
      }
    }
  } else {
    p.e[0] = Cvt<T>::from_f(f[0]);
  }
}

// ------------------------------------------------------------------------------------
// Packed fp32 arithmetic (sm_100: add / mul / fma on a register pair in one instruction).
// Each half is the ordinary IEEE round-to-nearest operation, so results equal the scalar
// form bit for bit; what changes is the number of issue slots, which is what bounds the
// 16-bit kernels.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ float2 f2(float v) { return make_float2(v, v); }
__device__ __forceinline__ float2 f2add(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 f2mul(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 f2fma(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

// a vector of VEC elements (VEC even) widened into VEC / 2 register pairs, and back
template <typename T, int VEC>
__device__ __forceinline__ void unpack2(const Pack<T, VEC>& p, float2 (&f)[VEC / 2]) {
  static_assert(VEC % 2 == 0, "pairs");
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) f[j] = make_float2(Cvt<T>::to_f(p.e[2 * j]), Cvt<T>::to_f(p.e[2 * j + 1]));
  } else {
    const unsigned int* w = reinterpret_cast<const unsigned int*>(&p);
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        f[j] = make_float2(__uint_as_float(w[j] << 16), __uint_as_float(w[j] & 0xffff0000u));
      } else {
        f[j] = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
      }
    }
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void pack2(const float2 (&f)[VEC / 2], Pack<T, VEC>& p) {
  static_assert(VEC % 2 == 0, "pairs");
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) {
      p.e[2 * j] = Cvt<T>::from_f(f[j].x);
      p.e[2 * j + 1] = Cvt<T>::from_f(f[j].y);
    }
  } else {
    unsigned int* w = reinterpret_cast<unsigned int*>(&p);
#pragma unroll
    for (int j = 0; j < VEC / 2; ++j) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        __nv_bfloat162 t = __floats2bfloat162_rn(f[j].x, f[j].y);
        w[j] = *reinterpret_cast<unsigned int*>(&t);
      } else {
        __half2 t = __floats2half2_rn(f[j].x, f[j].y);
        w[j] = *reinterpret_cast<unsigned int*>(&t);
      }
    }
  }
}

// Sum over the `tpr` threads that own a row, in two halves around the caller's CTA
// barrier.  *_warp: butterfly inside the warp and, for groups of several warps, the warp's
// value is parked in shared memory.  *_cta: every thread of the group combines the per-warp
// values in the same fixed order, so all of them hold bit-identical totals.
//
// A pair of sums (NV == 2) is reduced "transposed": after one exchange across the half-warps
// the lower 16 lanes carry sum 0 and the upper 16 lanes sum 1, so the remaining four butterfly
// steps move one register instead of two (12 instead of 20 shuffle + add slots per row, and
// these kernels are bound by instruction issue).  x + y == y + x bit for bit, so every lane
// still ends with the same value as the plain butterfly would give.
__device__ __forceinline__ void unzip_pair(float keep, bool hi, float (&v)[2]) {
  const float other = __shfl_xor_sync(0xffffffffu, keep, 16);
  v[0] = hi ? other : keep;
  v[1] = hi ? keep : other;
}
template <int NV>
__device__ __forceinline__ void rowsum_warp(float (&v)[NV], int tpr, float* smem) {
  if (tpr >= 32) {  // the usual case, fully unrolled
    if constexpr (NV == 2) {
      const int lane = threadIdx.x & 31;
      const bool hi = (lane & 16) != 0;
      float keep = hi ? v[1] : v[0];
      keep += __shfl_xor_sync(0xffffffffu, hi ? v[0] : v[1], 16);
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, off);
      if (tpr > 32) {
        if ((lane & 15) == 0) smem[(lane >> 4) * 32 + (threadIdx.x >> 5)] = keep;
      } else {
        unzip_pair(keep, hi, v);
      }
      return;
    } else {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int i = 0; i < NV; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], off);
      }
    }
  } else {
    for (int off = tpr >> 1; off > 0; off >>= 1) {
#pragma unroll
      for (int i = 0; i < NV; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], off);
    }
  }
  if (tpr > 32 && (threadIdx.x & 31) == 0) {
    const int warp = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < NV; ++i) smem[i * 32 + warp] = v[i];
  }
}
template <int W>
__device__ __forceinline__ float sum_w(const float* s) {  // s is 16-byte aligned when W >= 4
  if constexpr (W == 2) {
    return s[0] + s[1];
  } else {
    // all loads first (broadcast reads, one round trip), then a tree of adds
    float t[W / 4];
#pragma unroll
    for (int j = 0; j < W / 4; ++j) {
      const float4 q = *reinterpret_cast<const float4*>(s + 4 * j);
      t[j] = (q.x + q.y) + (q.z + q.w);
    }
#pragma unroll
    for (int n = W / 4; n > 1; n >>= 1) {
#pragma unroll
      for (int j = 0; j < n / 2; ++j) t[j] = t[2 * j] + t[2 * j + 1];
    }
    return t[0];
  }
}
// Every thread of the row group reads all per-warp values with broadcast 128-bit loads and
// adds them in the same fixed tree, so all threads hold bit-identical totals.  (A second
// butterfly over one word per lane needs fewer instructions but four dependent shuffles; with
// every warp of the CTA in the same phase the latency counted for more: 126.7 vs 129.0 us in
// the bf16 backward at 16384 x 8192.)
template <int NV>
__device__ __forceinline__ void rowsum_cta(float (&v)[NV], int tpr, const float* smem) {
  if (tpr > 32) {
    const int wpr = tpr >> 5;
    const int gbase = (threadIdx.x >> 5) & ~(wpr - 1);  // wpr is a power of two
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const float* s = smem + i * 32 + gbase;
      switch (wpr) {
        case 2:
          v[i] = sum_w<2>(s);
          break;
        case 4:
          v[i] = sum_w<4>(s);
          break;
        case 8:
          v[i] = sum_w<8>(s);
          break;
        case 16:
          v[i] = sum_w<16>(s);
          break;
        default:
          v[i] = sum_w<32>(s);
          break;
      }
    }
  }
}

// ------------------------------------------------------------------------------------
// activations
// ------------------------------------------------------------------------------------
// GELU without tanhf / erff (25 - 30 instructions each, which made LayerNorm + GELU at 16384 x
// 8192 bf16 twice as slow as LayerNorm alone: 173 / 191 against 87 us).
//   tanh form: 0.5 v (1 + tanh(u)) = v / (1 + exp(-2u)), u = sqrt(2/pi) (v + 0.044715 v^3): one
//   ex2.approx and one rcp.approx, relative error about 1e-6, and no cancellation for negative v
//   (1 + tanh(u) loses every digit there).
//   exact form: v Phi(v) with Phi from erfc(z) = (a1 t + ... + a5 t^5) exp(-z^2), t = 1 / (1 + p z),
//   z = |v| / sqrt(2) (Abramowitz & Stegun 7.1.26, absolute error 1.5e-7): Phi = erfc / 2 for
//   negative v, 1 - erfc / 2 otherwise.
// Both stay within the parity bounds (1e-5 absolute / relative in fp32, one unit in the last
// place of a 16-bit output).
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
constexpr float kGeluK = -2.0f * 0.7978845608028654f * 1.4426950408889634f;  // -2 sqrt(2/pi) log2(e)
constexpr float kGeluKA = kGeluK * 0.044715f;
constexpr float kErfP = 0.3275911f * 0.7071067811865476f;  // p / sqrt(2): t = 1 / (1 + kErfP |v|)
constexpr float kErfE = -0.5f * 1.4426950408889634f;       // exp(-z^2) = 2^(kErfE v^2)
// a1 .. a5 of 7.1.26, halved (Phi = erfc / 2)
constexpr float kErfA1 = 0.5f * 0.254829592f, kErfA2 = 0.5f * -0.284496736f, kErfA3 = 0.5f * 1.421413741f,
                kErfA4 = 0.5f * -1.453152027f, kErfA5 = 0.5f * 1.061405429f;

template <int ACT>
__device__ __forceinline__ float apply_act(float v) {
  if (ACT == FLN_ACT_GELU_TANH) {
    const float w = v * v;
    const float e = ex2_approx(v * fmaf(w, kGeluKA, kGeluK));  // exp(-2u)
    return v * rcp_approx(1.0f + e);
  } else if (ACT == FLN_ACT_GELU_ERF) {
    const float t = rcp_approx(fmaf(fabsf(v), kErfP, 1.0f));
    const float e = ex2_approx(v * v * kErfE);
    const float poly = t * fmaf(t, fmaf(t, fmaf(t, fmaf(t, kErfA5, kErfA4), kErfA3), kErfA2), kErfA1);
    const float h = poly * e;  // erfc(|v| / sqrt 2) / 2
    return v * (v < 0.f ? h : 1.0f - h);
  }
  return v;
}
// the same on a register pair (packed fp32 arithmetic where the operation exists)
template <int ACT>
__device__ __forceinline__ float2 apply_act2(float2 v) {
  if (ACT == FLN_ACT_GELU_TANH) {
    const float2 w = f2mul(v, v);
    const float2 a = f2mul(v, f2fma(w, f2(kGeluKA), f2(kGeluK)));
    const float2 d = f2add(make_float2(ex2_approx(a.x), ex2_approx(a.y)), f2(1.0f));
    return f2mul(v, make_float2(rcp_approx(d.x), rcp_approx(d.y)));
  } else if (ACT == FLN_ACT_GELU_ERF) {
    const float2 az = make_float2(fabsf(v.x), fabsf(v.y));
    const float2 den = f2fma(az, f2(kErfP), f2(1.0f));
    const float2 t = make_float2(rcp_approx(den.x), rcp_approx(den.y));
    const float2 ea = f2mul(f2mul(v, v), f2(kErfE));
    const float2 e = make_float2(ex2_approx(ea.x), ex2_approx(ea.y));
    float2 poly = f2fma(t, f2(kErfA5), f2(kErfA4));
    poly = f2fma(t, poly, f2(kErfA3));
    poly = f2fma(t, poly, f2(kErfA2));
    poly = f2fma(t, poly, f2(kErfA1));
    const float2 h = f2mul(f2mul(poly, t), e);
    const float2 up = f2add(f2(1.0f), make_float2(-h.x, -h.y));
    return f2mul(v, make_float2(v.x < 0.f ? h.x : up.x, v.y < 0.f ? h.y : up.y));
  }
  return v;
}

// ------------------------------------------------------------------------------------
// row-group reductions.  A row is owned by `tpr` consecutive threads (power of two).
// tpr <= 32: the group is a slice of one warp.  tpr > 32: the group is tpr/32 whole warps
// and partial results take one hop through shared memory.
// ------------------------------------------------------------------------------------
// sum of NV values per thread over the row group; all threads get bit-identical results.
// smem: NV * 32 floats per buffer.
template <int NV>
__device__ __forceinline__ void group_reduce_sum(float (&v)[NV], int tpr, float* smem) {
  const int lane = threadIdx.x & 31;
  const int lim = tpr < 32 ? tpr : 32;
  for (int off = lim >> 1; off > 0; off >>= 1) {
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], off);
  }
  if (tpr > 32) {
    const int warp = threadIdx.x >> 5;
    const int wpr = tpr >> 5;
    const int gbase = (warp / wpr) * wpr;
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < NV; ++i) smem[i * 32 + warp] = v[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = lane < wpr ? smem[i * 32 + gbase + lane] : 0.f;
    // lanes >= wpr hold zeros: a full-warp butterfly leaves the total in every lane
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
      for (int i = 0; i < NV; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], off);
    }
  }
}

// ------------------------------------------------------------------------------------
// kernel parameter blocks (shared by the register-resident and the pipelined kernels)
// ------------------------------------------------------------------------------------
struct FwdParams {
  const void* x;
  const void* res;
  const void* gamma;
  const void* beta;
  void* y;
  void* sum_out;
  float* mean;
  float* rstd;
  int64_t rows;
  int cols;
  int nv;  // vectors per row
  int tpr;
  int log2_tpr;
  float eps;
  // pipelined forward only (set by its launcher): the pair of words {next tile, CTAs finished}
  // this launch claims its tiles from, how long a wait may last (ns), and the device's status
  // word and test-hook word
  unsigned int* sched;
  unsigned long long wait_ns;
  int* status;
  const int* fault;
  // fp8 forms of the pipelined forward only: e4m3 codes out (NULL: none), the scale they are
  // made with, where max |y| of the call goes (NULL: nowhere)
  void* q;
  const float* scale_in;
  float* amax;
  unsigned char* block_scale;  // MXFP8: [rows, cols / 32] E8M0 bytes; NVFP4: [rows, cols / 16] e4m3 bytes
  float* row_scale;            // per-row scales: [rows]
  // dropout form of the pipelined forward only
  unsigned char* keep_bits;  // one byte per 8 elements, or NULL
  unsigned long long drop_seed, drop_offset;
  unsigned int drop_threshold;  // 0: keep everything
  float drop_scale;
};

struct BwdParams {
  const void* dy;
  const void* x;
  const float* mean;
  const float* rstd;
  const void* gamma;
  const void* dres_in;
  void* dx;
  float* partials;  // [P][2][cols] (LayerNorm) or [P][1][cols] (RMSNorm); may be NULL
  int64_t rows;
  int64_t row_groups;
  int cols;
  int nv;
  int tpr;
  int log2_tpr;
  // Pipelined backward only: when `sync` is set the launch is cooperative, the grid meets at
  // a barrier once the partial rows are written, and every CTA sums a slab of columns, so
  // no second kernel is needed.  `sync` is one 8-byte word of the caller's workspace whose
  // contents may be anything; `token` (never 0, different for every launch that is not a
  // replay) lets the first arrival recognise and overwrite stale contents.
  unsigned long long* sync;
  unsigned long long token;
  float* dgb_f32;
  void* dgamma;
  void* dbeta;
  // pipelined backward only (set by its launcher): how long a wait may last (ns), the device's
  // status word and test-hook word
  unsigned long long wait_ns;
  int* status;
  const int* fault;
};

// Pipelined (bulk-async staged, persistent) variants, fln_pipeline.cu.  They return
// FLN_PIPE_NOT_APPLICABLE when the shape is better served by the register kernels.
constexpr int FLN_PIPE_NOT_APPLICABLE = -1;
int launch_fwd_pipeline(int kind, int act, int io_dtype, int out_dtype, const FwdParams& p,
                        cudaStream_t st);
// fp8 forms: e4m3 codes made with *p.scale_in into p.q when p.q is set, max |y| into *p.amax when
// that is set (p.y is not written)
// qm 1: per-tensor scale as above; 2: one scale per row (p.row_scale); 3: MXFP8; 4: NVFP4-style
// (both with p.block_scale)
int launch_fwd_pipeline_fp8(int kind, int io_dtype, int qm, const FwdParams& p, cudaStream_t st);
// dropout -> residual add -> norm (p.keep_bits, p.drop_*); p.sum_out may be NULL
int launch_fwd_pipeline_dropout(int kind, int io_dtype, const FwdParams& p, cudaStream_t st);
// *reduced tells whether dgamma / dbeta / dgb_f32 were produced by the launch itself (fused
// column reduce); otherwise the caller reduces p.partials.
int launch_bwd_pipeline(int kind, int dtype, const BwdParams& p, cudaStream_t st, bool* reduced);
// the pipelined plan of a shape, for fln_describe_launch (returns false when the register or
// generic kernels serve it)
struct PipeDescription {
  int vector_bytes, K, tpr, threads, rows_per_cta, stages;
  int64_t grid;
};
bool describe_pipeline(bool backward, int64_t rows, int cols, int elem_bytes, PipeDescription* out);
// partial rows the pipelined backward writes for this shape (0 = not applicable)
int64_t bwd_pipeline_partial_rows(int kind, int dtype, int64_t rows, int cols, bool with_dres);
// Row counts that do not fill the row slots of the fast plan of their row length (2, 4, 8 or 16
// rows per CTA) would run a bounds-checked or padded plan, 10 - 35 % slower.  These return how
// many trailing rows to hand to the register kernels so that the rest runs the fast plan (0:
// nothing to gain).
int64_t fwd_pipeline_odd_rows(int act, int io_dtype, int out_dtype, const FwdParams& p);
int64_t bwd_pipeline_odd_rows(int dtype, int64_t rows, int cols, bool with_dres);
// (the quantizing and dropout forms of the pipelined forward: 16-bit input, `tensors` = 2 with a
// residual)
int64_t fwd_fp8_pipeline_odd_rows(int64_t rows, int cols, int tensors);

// ------------------------------------------------------------------------------------
// host side: launch plan
// ------------------------------------------------------------------------------------
struct Plan {
  int generic;  // 1: use the looping fallback kernel
  int vec;      // elements per vector access
  int K;        // vectors per thread (1, 2, 4, 8)
  int tpr;      // threads per row (power of two)
  int log2_tpr;
  int threads;  // per CTA
  int rows_per_cta;
};

int sm_count();    // of the current device, cached
int usable_sms();  // sm_count() minus the SMs persistent grids are asked to leave free
Plan make_plan(bool backward, int64_t rows, int cols, int elem_bytes, bool aligned16);
void plan_override(int* K, int* tpr);

inline bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define FLN_CHECK_LAUNCH()                                   \
  do {                                                       \
    cudaError_t e__ = cudaGetLastError();                    \
    if (e__ != cudaSuccess) return FLN_ERR_LAUNCH;           \
  } while (0)

}  // namespace fln
