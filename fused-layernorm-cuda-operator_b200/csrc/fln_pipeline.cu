// Persistent, bulk-async staged LayerNorm / RMSNorm forward and backward for sm_100a.
//
// Every CTA is persistent and owns a ring of S shared-memory stages; one elected thread
// keeps the ring full with 1-D bulk copies (cp.async.bulk global -> shared, completion
// signalled on an mbarrier with complete_tx::bytes), so up to S tiles per CTA are in flight
// regardless of register use.  A tile is R consecutive rows, which are contiguous in
// memory, so one tile is ONE bulk copy per input tensor.  Consumers wait on the stage's
// mbarrier, pull their vectors from shared memory into registers, and the first CTA barrier
// of the row reduction doubles as the "stage is free again" signal after which the producer
// refills it.  gamma / beta live in registers as floats for the life of the CTA, so the only
// L2 traffic per row is the row itself.
//
// At bf16 these kernels are bound by instruction issue before they are bound by HBM, so the
// per-element instruction count is what matters.  The FULL instantiation (row length equal
// to K * threads-per-row, no ragged last tile, at least a warp per row) has no predication
// at all in the loop; the general instantiation keeps the bounds checks.
//
// No cluster multicast is used anywhere; every copy is CTA-local.
//
// Every mbarrier wait is bounded: on a time-out the CTA votes, raises the device status word
// (fln_device_status), lets its producer wait -- again bounded -- for copies still in flight,
// and returns.
#include <string.h>

#include <atomic>

#include "fln_common.cuh"

namespace fln {

__device__ int g_device_status = 0;

struct PipeGeom {
  int R;         // rows per tile
  int tpr;       // threads per row
  int log2_tpr;
  int S;         // stages
  uint32_t row_bytes;
  uint32_t second_off;    // byte offset of the second tensor inside a stage
  uint32_t stage_stride;  // bytes per stage
};

constexpr int kSmemHeader = 2048;  // mbarriers + reduction scratch in front of the stages
constexpr uint32_t kWaitLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// global -> this CTA's shared memory, 16-byte aligned on both sides, bytes % 16 == 0
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < kWaitLimit; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// One 16-byte vector of a stage as ONE 128-bit shared-memory load.  (Handing the stage to the
// conversion helper by reference lets the compiler read it word by word: four times the load
// instructions and the shared-memory pipe becomes the stall.)
template <typename T>
__device__ __forceinline__ Pack<T, 16 / sizeof(T)> ld_smem16(const unsigned char* p) {
  Pack<T, 16 / sizeof(T)> out;
  *reinterpret_cast<uint4*>(&out) = *reinterpret_cast<const uint4*>(p);
  return out;
}

// How a kernel takes one vector out of a stage.  16-bit types: by value through the 128-bit
// load above (measured 246.8 vs 285.7 us for the bf16 forward + backward).  fp32: by reference,
// which lets the compiler schedule four 32-bit loads; that form measured faster for fp32
// (backward 245 vs 277 us at 16384 x 8192), where the kernel is HBM-bound anyway.
// Vectors shorter than 16 bytes (row lengths 3, 5 or 7 times a power of two are split into 8- or
// 4-byte vectors so that they divide evenly over the threads) are read with one load of that
// width.
template <typename T, int VEC = 16 / sizeof(T)>
__device__ __forceinline__ decltype(auto) stage_vec(const unsigned char* p) {
  if constexpr (VEC * sizeof(T) == 16 && sizeof(T) == 4) {
    return (*reinterpret_cast<const Pack<T, 4>*>(p));
  } else if constexpr (VEC * sizeof(T) == 16) {
    return ld_smem16<T>(p);
  } else {
    using R = typename Raw<sizeof(T) * VEC>::type;
    Pack<T, VEC> out;
    *reinterpret_cast<R*>(&out) = *reinterpret_cast<const R*>(p);
    return out;
  }
}

// tiles of CTA b: t = b + i * gridDim.x  (evaluated once per CTA)
__device__ __forceinline__ int my_tile_count(int64_t n_tiles) {
  return (int64_t)blockIdx.x < n_tiles ? (int)((n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
}

// After a failed vote: thread 0 raises the status word and gives copies already issued a
// bounded chance to land before the CTA's shared memory is released.
__device__ __forceinline__ void pipeline_abort(uint64_t* full, int S, int s, uint32_t phase, int outstanding) {
  if (threadIdx.x == 0) {
    atomicExch(&g_device_status, 1);
    for (int j = 0; j < outstanding; ++j) {
      mbar_wait_bounded(&full[s], phase);
      if (++s == S) {
        s = 0;
        phase ^= 1u;
      }
    }
  }
}

// ----------------------------------------------------------------------------------------
// Grid barrier of a cooperative launch on one 64-bit word of caller memory with undefined
// initial contents:  [63:24] token of the launch | [23:12] CTAs departed | [11:0] CTAs arrived.
// The first CTA to look finds a foreign token and starts the count afresh; the last CTA to
// depart writes 0 (no token is 0), so a graph replay with the same token starts clean as well.
// Called by ONE thread per CTA, after a CTA barrier that follows the CTA's global writes.
// The wait is bounded like every other wait here.
// ----------------------------------------------------------------------------------------
constexpr uint32_t kGridWaitLimit = 1u << 21;  // polls, >= 64 ns apart

// At kernel start, one thread per CTA: make sure the word carries this launch's token.  One
// compare-and-swap at most and no retry: if it fails, another CTA has initialised the word
// (or has already counted itself in), which is all that is needed.  (Counting arrivals with a
// compare-and-swap loop instead costs a round trip to L2 per CTA *in sequence*: 53 us for 148.)
__device__ __forceinline__ void grid_barrier_init(unsigned long long* w, unsigned long long token) {
  const unsigned long long old = *reinterpret_cast<volatile unsigned long long*>(w);
  if ((old >> 24) != token) atomicCAS(w, old, token << 24);
}
__device__ __forceinline__ bool grid_arrive_and_wait(unsigned long long* w, unsigned long long token,
                                                     unsigned int grid) {
  __threadfence();
  atomicAdd(w, 1ull);
  for (uint32_t it = 0; it < kGridWaitLimit; ++it) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(w) : "memory");
    if ((v >> 24) == token && (unsigned int)(v & 0xfffull) == grid) return true;
    __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ void grid_depart(unsigned long long* w, unsigned int grid) {
  const unsigned long long old = atomicAdd(w, 1ull << 12);
  if ((unsigned int)((old >> 12) & 0xfffull) == grid - 1) atomicExch(w, 0ull);
}

// ----------------------------------------------------------------------------------------
// forward
//
// Per element: one shift or mask (widen), shift by c and add (row sum), centre, one fma
// (sum of squares), one multiply and one fma (normalize + affine), half a paired convert.
// Statistics are the two-pass form on the row shifted by its first element, each pass
// reduced by a warp butterfly plus one shared-memory hop.
// ----------------------------------------------------------------------------------------
// MODE 0: general (bounds-checked); 1: FULL (no predication in the loop); 2: FULL and the
// CTA owns exactly one row, which allows the one-barrier LayerNorm statistics below (no launch
// path of this file instantiates it: it measured no faster than MODE 1 in the ring).
template <typename TI, typename TO, int K, int KIND, int ACT, int MODE, int VB = 16>
__global__ void __launch_bounds__(512) norm_fwd_pipe_kernel(const FwdParams p, const PipeGeom g) {
  constexpr int VEC = VB / sizeof(TI);  // a multiple of 4 (the statistics run four chains)
  constexpr bool FULL = MODE >= 1;
  constexpr bool ONE = MODE == 2 && KIND == FLN_LAYERNORM;
  // MODE 4: FULL with gamma / beta parked in shared memory (in the I/O type) instead of in
  // registers as floats, for plans that give a thread more than 32 elements (row lengths
  // 5 * 2^a in 16-bit types: 40 elements per thread keep the 16-byte vectors and move more
  // bytes per barrier than 20 elements in 8-byte vectors)
  constexpr bool PSM = MODE == 4;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  float* s_red = reinterpret_cast<float*>(smem + 256);  // 2 x 64 + 2 x 32 floats
  unsigned char* stages = smem + kSmemHeader;

  const int tid = threadIdx.x;
  const int tpr = g.tpr;
  const int lane_r = tid & (tpr - 1);
  const int r_in = tid >> g.log2_tpr;
  const int S = g.S;
  const int my_tiles = my_tile_count((p.rows + g.R - 1) / g.R);
  const bool has_res = p.res != nullptr;
  const float inv_n = 1.0f / (float)p.cols;
  const float eps = p.eps;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  __syncthreads();

  // tile i of this CTA into stage s (the caller tracks s; no division in the loop)
  auto issue = [&](int i, int s) {
    const int64_t row0 = ((int64_t)blockIdx.x + (int64_t)i * gridDim.x) * g.R;
    const int64_t left = p.rows - row0;
    const uint32_t bytes = (uint32_t)(left < g.R ? left : g.R) * g.row_bytes;
    unsigned char* dst = stages + (size_t)s * g.stage_stride;
    mbar_expect_tx(&full[s], has_res ? 2 * bytes : bytes);
    bulk_g2s(dst, reinterpret_cast<const TI*>(p.x) + row0 * p.cols, bytes, &full[s]);
    if (has_res) bulk_g2s(dst + g.second_off, reinterpret_cast<const TI*>(p.res) + row0 * p.cols, bytes, &full[s]);
  };
  if (tid == 0) {
    const int pre = my_tiles < S ? my_tiles : S;
    for (int i = 0; i < pre; ++i) issue(i, i);
  }

  float gam[PSM ? 1 : K][VEC], bet[PSM ? 1 : K][VEC];
  bool vok[K];  // does vector k of this thread exist in the row
  unsigned char* s_gamma = stages + (size_t)S * g.stage_stride;  // PSM: [cols] gamma, then [cols] beta
  unsigned char* s_beta = s_gamma + g.row_bytes;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int iv = lane_r + k * tpr;
    vok[k] = FULL ? true : iv < p.nv;
    if constexpr (PSM) {
      if (r_in == 0) {
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
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        gam[k][e] = 1.f;
        bet[k][e] = 0.f;
      }
      if (vok[k]) {
        if (p.gamma != nullptr)
          unpack<TI, VEC>(ld_param<TI, VEC>(reinterpret_cast<const TI*>(p.gamma) + (int64_t)iv * VEC), gam[k]);
        if (p.beta != nullptr)
          unpack<TI, VEC>(ld_param<TI, VEC>(reinterpret_cast<const TI*>(p.beta) + (int64_t)iv * VEC), bet[k]);
      }
    }
  }
  if constexpr (PSM) __syncthreads();

  int s = 0;
  uint32_t phase = 0;
  int64_t row = (int64_t)blockIdx.x * g.R + r_in;
  const int64_t row_step = (int64_t)gridDim.x * g.R;
  const uint32_t my_off = (uint32_t)r_in * g.row_bytes + (uint32_t)lane_r * (uint32_t)VB;
  const uint32_t k_off = (uint32_t)tpr * (uint32_t)VB;
  for (int i = 0; i < my_tiles; ++i, row += row_step) {
    const bool landed = mbar_wait_bounded(&full[s], phase);
    const bool row_ok = FULL ? true : row < p.rows;
    const unsigned char* st = stages + (size_t)s * g.stage_stride + my_off;
    float* redA = s_red + (i & 1) * 64;
    float* redB = s_red + 128 + (i & 1) * 32;

    float f[K][VEC];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (FULL || (row_ok && vok[k])) {
        unpack<TI, VEC>(stage_vec<TI, VEC>(st + k * k_off), f[k]);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) f[k][e] = 0.f;
      }
    }
    if (has_res) {
      TI* __restrict__ sr = reinterpret_cast<TI*>(p.sum_out) + row * (int64_t)p.cols + (int64_t)lane_r * VEC;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        if (FULL || (row_ok && vok[k])) {
          float r[VEC];
          unpack<TI, VEC>(stage_vec<TI, VEC>(st + g.second_off + k * k_off), r);
#pragma unroll
          for (int e = 0; e < VEC; ++e) f[k][e] += r[e];
          // the sum is rounded to the I/O type first: that value is normalized and stored
          Pack<TI, VEC> q;
          pack<TI, VEC>(f[k], q);
          st_stream<TI, VEC>(sr + (int64_t)k * tpr * VEC, q);
          unpack<TI, VEC>(q, f[k]);
        }
      }
    }

    float mean = 0.f, rstd = 0.f;
    bool need_second = true;  // is the exact centred pass needed
    if (KIND == FLN_LAYERNORM) {
      // shift by element 0 of the row (a broadcast read of the stage): a constant row then
      // sums to exactly zero whatever its magnitude, and |mean| >> std costs no accuracy
      const unsigned char* st0 = st - (size_t)lane_r * VB;
      float c = Cvt<TI>::to_f(*reinterpret_cast<const TI*>(st0));
      if (has_res)
        c = Cvt<TI>::to_f(Cvt<TI>::from_f(c + Cvt<TI>::to_f(*reinterpret_cast<const TI*>(st0 + g.second_off))));
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;  // four chains: the adds are latency-bound
      float b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        if (FULL || vok[k]) {  // padding vectors stay zero
#pragma unroll
          for (int e = 0; e < VEC; e += 4) {
            f[k][e] -= c;
            f[k][e + 1] -= c;
            f[k][e + 2] -= c;
            f[k][e + 3] -= c;
            a0 += f[k][e];
            a1 += f[k][e + 1];
            a2 += f[k][e + 2];
            a3 += f[k][e + 3];
            if (ONE) {
              b0 = fmaf(f[k][e], f[k][e], b0);
              b1 = fmaf(f[k][e + 1], f[k][e + 1], b1);
              b2 = fmaf(f[k][e + 2], f[k][e + 2], b2);
              b3 = fmaf(f[k][e + 3], f[k][e + 3], b3);
            }
          }
        }
      }
      constexpr int NA = ONE ? 2 : 1;
      float ar[NA];
      ar[0] = (a0 + a1) + (a2 + a3);
      if (ONE) ar[NA - 1] = (b0 + b1) + (b2 + b3);
      rowsum_warp<NA>(ar, tpr, redA);
      // The first barrier of a tile also proves that every thread has pulled its part of
      // stage s into registers, so the producer may refill the stage right after it.
      if (!__syncthreads_and(landed ? 1 : 0)) {
        pipeline_abort(full, S, s, phase, my_tiles - i < S ? my_tiles - i : S);
        return;
      }
      if (tid == 0 && i + S < my_tiles) issue(i + S, s);
      rowsum_cta<NA>(ar, tpr, redA);
      const float ms = ar[0] * inv_n;  // mean of the shifted row
      mean = c + ms;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        if (FULL || vok[k]) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) f[k][e] -= ms;
        }
      }
      if (ONE) {
        // One-pass variance of the shifted row, E[d^2] - E[d]^2.  Its relative error grows
        // like eps * (1 + 2 ms^2 / var), so it is trusted only when the shift element lay
        // within two standard deviations of the mean; otherwise the exact centred pass
        // below runs.  The CTA owns one row here and ms, var1 are bit-identical in all its
        // threads, so the branch (and the barrier inside it) is uniform.
        const float var1 = fmaf(ar[NA - 1], inv_n, -ms * ms);
        if (ms * ms <= 4.f * var1) {
          need_second = false;
          rstd = rsqrtf(var1 + eps);
        }
      }
    }
    if (need_second) {
      float q0 = 0.f, q1 = 0.f, q2 = 0.f, q3 = 0.f;
#pragma unroll
      for (int k = 0; k < K; ++k) {
#pragma unroll
        for (int e = 0; e < VEC; e += 4) {
          q0 = fmaf(f[k][e], f[k][e], q0);
          q1 = fmaf(f[k][e + 1], f[k][e + 1], q1);
          q2 = fmaf(f[k][e + 2], f[k][e + 2], q2);
          q3 = fmaf(f[k][e + 3], f[k][e + 3], q3);
        }
      }
      float q[1] = {(q0 + q1) + (q2 + q3)};
      rowsum_warp<1>(q, tpr, redB);
      if (KIND == FLN_LAYERNORM) {
        __syncthreads();
      } else {
        if (!__syncthreads_and(landed ? 1 : 0)) {
          pipeline_abort(full, S, s, phase, my_tiles - i < S ? my_tiles - i : S);
          return;
        }
        if (tid == 0 && i + S < my_tiles) issue(i + S, s);
      }
      rowsum_cta<1>(q, tpr, redB);
      rstd = rsqrtf(fmaf(q[0], inv_n, eps));
    }

    if (row_ok && lane_r == 0) {
      if (KIND == FLN_LAYERNORM && p.mean != nullptr) p.mean[row] = mean;
      if (p.rstd != nullptr) p.rstd[row] = rstd;
    }
    TO* __restrict__ yr = reinterpret_cast<TO*>(p.y) + row * (int64_t)p.cols + (int64_t)lane_r * VEC;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (FULL || (row_ok && vok[k])) {
        float o[VEC];
        if constexpr (PSM) {
          float gw[VEC], bw[VEC];
          const size_t po = (size_t)(lane_r + k * tpr) * VB;
          unpack<TI, VEC>(stage_vec<TI, VEC>(s_gamma + po), gw);
          unpack<TI, VEC>(stage_vec<TI, VEC>(s_beta + po), bw);
#pragma unroll
          for (int e = 0; e < VEC; ++e) o[e] = apply_act<ACT>(fmaf(f[k][e] * rstd, gw[e], bw[e]));
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) o[e] = apply_act<ACT>(fmaf(f[k][e] * rstd, gam[k][e], bet[k][e]));
        }
        Pack<TO, VEC> out;
        pack<TO, VEC>(o, out);
        st_stream<TO, VEC>(yr + (int64_t)k * tpr * VEC, out);
      }
    }
    if (++s == S) {
      s = 0;
      phase ^= 1u;
    }
  }
}

// ----------------------------------------------------------------------------------------
// Fused column reduce, the tail of the pipelined backward.  The partial rows were written a
// moment ago and sit in L2; after the grid barrier CTA q sums columns [128 q, 128 q + 128)
// over all partial rows: a warp per 512-byte row segment, the rows split over the 16 warps,
// every thread's (up to ten) 16-byte loads issued before its first add, then the 16 warps
// combined through the now idle stage memory `sb` (16 x 128 floats).  The order of the adds
// is fixed, so the sums are reproducible.  Kept out of line so that the register allocation
// of the streaming loop does not depend on it.
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
};
template <typename T, int NR>
__device__ __noinline__ void fused_column_reduce(const ReduceArgs p, float* sb) {
  const int tid = threadIdx.x;
  __syncthreads();
  bool met = true;
  if (tid == 0) met = grid_arrive_and_wait(p.sync, p.token, gridDim.x);
  if (!__syncthreads_and(met ? 1 : 0)) {
    if (tid == 0) atomicExch(&g_device_status, 2);
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
// Per element: two widening shifts, (x - mean) * rstd, g = dy * gamma, two running sums,
// then dx = rstd * ((g - c2) - xhat * c1) and the two column accumulators.
// ----------------------------------------------------------------------------------------
// DRES: an incoming gradient of the residual stream (same shape as dx) is staged as a third
// tensor and added into dx; each thread parks its (still packed) part in registers before the
// barrier that releases the stage.
template <typename T, int K, int KIND, bool FULL, bool FUSE, bool DRES, int VB = 16>
__global__ void __launch_bounds__(512) norm_bwd_pipe_kernel(const BwdParams p, const PipeGeom g) {
  constexpr int VEC = VB / sizeof(T);  // even
  constexpr int NR = KIND == FLN_LAYERNORM ? 2 : 1;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  float* s_red = reinterpret_cast<float*>(smem + 256);  // 2 x 64 floats
  unsigned char* stages = smem + kSmemHeader;

  const int tid = threadIdx.x;
  const int tpr = g.tpr;
  const int lane_r = tid & (tpr - 1);
  const int r_in = tid >> g.log2_tpr;
  const int S = g.S;
  const int my_tiles = my_tile_count((p.rows + g.R - 1) / g.R);
  const float inv_n = 1.0f / (float)p.cols;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  if (FUSE && tid == 32) grid_barrier_init(p.sync, p.token);
  __syncthreads();

  auto issue = [&](int i, int s) {
    const int64_t row0 = ((int64_t)blockIdx.x + (int64_t)i * gridDim.x) * g.R;
    const int64_t left = p.rows - row0;
    const uint32_t bytes = (uint32_t)(left < g.R ? left : g.R) * g.row_bytes;
    unsigned char* dst = stages + (size_t)s * g.stage_stride;
    mbar_expect_tx(&full[s], (DRES ? 3 : 2) * bytes);
    bulk_g2s(dst, reinterpret_cast<const T*>(p.dy) + row0 * p.cols, bytes, &full[s]);
    bulk_g2s(dst + g.second_off, reinterpret_cast<const T*>(p.x) + row0 * p.cols, bytes, &full[s]);
    if (DRES)
      bulk_g2s(dst + 2 * g.second_off, reinterpret_cast<const T*>(p.dres_in) + row0 * p.cols, bytes, &full[s]);
  };
  if (tid == 0) {
    const int pre = my_tiles < S ? my_tiles : S;
    for (int i = 0; i < pre; ++i) issue(i, i);
  }

  float acc_g[K][VEC], acc_b[K][VEC], gam[K][VEC];
  bool vok[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int iv = lane_r + k * tpr;
    vok[k] = FULL ? true : iv < p.nv;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      acc_g[k][e] = 0.f;
      acc_b[k][e] = 0.f;
      gam[k][e] = 1.f;
    }
    if (p.gamma != nullptr && vok[k])
      unpack<T, VEC>(ld_param<T, VEC>(reinterpret_cast<const T*>(p.gamma) + (int64_t)iv * VEC), gam[k]);
  }

  // per-row statistics of the next tile are fetched one iteration ahead
  int64_t row = (int64_t)blockIdx.x * g.R + r_in;
  const int64_t row_step = (int64_t)gridDim.x * g.R;
  float mean_n = 0.f, rstd_n = 0.f;
  if (my_tiles > 0 && row < p.rows) {
    if (KIND == FLN_LAYERNORM) mean_n = __ldg(p.mean + row);
    rstd_n = __ldg(p.rstd + row);
  }

  int s = 0;
  uint32_t phase = 0;
  const uint32_t my_off = (uint32_t)r_in * g.row_bytes + (uint32_t)lane_r * (uint32_t)VB;
  const uint32_t k_off = (uint32_t)tpr * (uint32_t)VB;
  for (int i = 0; i < my_tiles; ++i, row += row_step) {
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
    const bool landed = mbar_wait_bounded(&full[s], phase);
    const unsigned char* st = stages + (size_t)s * g.stage_stride + my_off;
    // 16-bit inputs: xhat as ONE fma, x * rstd - mean * rstd.  The rounding of mean * rstd
    // costs 2^-24 |mean| / std in xhat, and 16-bit data cannot hold |mean| / std beyond 2^11,
    // so this stays three orders below the output's own rounding.  fp32 keeps (x - mean) * rstd.
    const float nmr = -mean * rstd;

    float xh[K][VEC], dyf[K][VEC];
    Pack<T, VEC> dres[DRES ? K : 1];
    float r0a = 0.f, r0b = 0.f, r1a = 0.f, r1b = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (FULL || (row_ok && vok[k])) {
        unpack<T, VEC>(stage_vec<T, VEC>(st + k * k_off), dyf[k]);
        unpack<T, VEC>(stage_vec<T, VEC>(st + g.second_off + k * k_off), xh[k]);
        if (DRES) dres[k] = stage_vec<T, VEC>(st + 2 * g.second_off + k * k_off);
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          xh[k][e] = sizeof(T) == 2 ? fmaf(xh[k][e], rstd, nmr) : (xh[k][e] - mean) * rstd;
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          dyf[k][e] = 0.f;
          xh[k][e] = 0.f;
        }
      }
#pragma unroll
      for (int e = 0; e < VEC; e += 2) {
        const float g0 = dyf[k][e] * gam[k][e], g1 = dyf[k][e + 1] * gam[k][e + 1];
        r0a = fmaf(g0, xh[k][e], r0a);
        r0b = fmaf(g1, xh[k][e + 1], r0b);
        if (KIND == FLN_LAYERNORM) {
          r1a += g0;
          r1b += g1;
        }
      }
    }
    float red[NR];
    red[0] = r0a + r0b;
    if (KIND == FLN_LAYERNORM) red[NR - 1] = r1a + r1b;
    float* sr = s_red + (i & 1) * 64;
    rowsum_warp<NR>(red, tpr, sr);
    if (!__syncthreads_and(landed ? 1 : 0)) {
      pipeline_abort(full, S, s, phase, my_tiles - i < S ? my_tiles - i : S);
      return;
    }
    if (tid == 0 && i + S < my_tiles) issue(i + S, s);
    rowsum_cta<NR>(red, tpr, sr);
    // dx = rstd * ((g - c2) - xhat * c1): the subtraction comes first so that rows whose g
    // is (nearly) constant cancel exactly instead of leaving a rounding residue times rstd
    const float nc1 = -(red[0] * inv_n);
    const float c2 = KIND == FLN_LAYERNORM ? red[NR - 1] * inv_n : 0.f;

    if (p.dx != nullptr) {
      T* __restrict__ dxr = reinterpret_cast<T*>(p.dx) + row * (int64_t)p.cols + (int64_t)lane_r * VEC;
#pragma unroll
      for (int k = 0; k < K; ++k) {
        if (FULL || (row_ok && vok[k])) {
          float o[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            // the product of two 16-bit values is exact in fp32, so the fma equals
            // (dy * gamma) - c2 bit for bit there and saves the multiply
            const float gc = sizeof(T) == 2 ? fmaf(dyf[k][e], gam[k][e], -c2) : dyf[k][e] * gam[k][e] - c2;
            o[e] = rstd * fmaf(xh[k][e], nc1, gc);
          }
          if (DRES) {
            float dr[VEC];
            unpack<T, VEC>(dres[k], dr);
#pragma unroll
            for (int e = 0; e < VEC; ++e) o[e] += dr[e];
          }
          Pack<T, VEC> out;
          pack<T, VEC>(o, out);
          st_stream<T, VEC>(dxr + (int64_t)k * tpr * VEC, out);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        acc_g[k][e] = fmaf(dyf[k][e], xh[k][e], acc_g[k][e]);
        if (KIND == FLN_LAYERNORM) acc_b[k][e] += dyf[k][e];
      }
    }
    if (++s == S) {
      s = 0;
      phase ^= 1u;
    }
  }

  if (p.partials != nullptr) {
    const int64_t prow = (int64_t)blockIdx.x * g.R + r_in;
    float* __restrict__ pg = p.partials + prow * (int64_t)(NR * p.cols);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int iv = lane_r + k * tpr;
      if (vok[k]) {
        if constexpr (VEC % 4 == 0) {
#pragma unroll
          for (int e = 0; e < VEC; e += 4) {
            *reinterpret_cast<float4*>(pg + (int64_t)iv * VEC + e) =
                make_float4(acc_g[k][e], acc_g[k][e + 1], acc_g[k][e + 2], acc_g[k][e + 3]);
            if (KIND == FLN_LAYERNORM)
              *reinterpret_cast<float4*>(pg + p.cols + (int64_t)iv * VEC + e) =
                  make_float4(acc_b[k][e], acc_b[k][e + 1], acc_b[k][e + 2], acc_b[k][e + 3]);
          }
        } else {
#pragma unroll
          for (int e = 0; e < VEC; e += 2) {
            *reinterpret_cast<float2*>(pg + (int64_t)iv * VEC + e) = make_float2(acc_g[k][e], acc_g[k][e + 1]);
            if (KIND == FLN_LAYERNORM)
              *reinterpret_cast<float2*>(pg + p.cols + (int64_t)iv * VEC + e) = make_float2(acc_b[k][e], acc_b[k][e + 1]);
          }
        }
      }
    }
  }

  if (FUSE) {
    ReduceArgs a;
    a.partials = p.partials;
    a.sync = p.sync;
    a.token = p.token;
    a.dgb_f32 = p.dgb_f32;
    a.dgamma = p.dgamma;
    a.dbeta = p.dbeta;
    a.cols = p.cols;
    a.P = (int)gridDim.x * g.R;
    fused_column_reduce<T, NR>(a, reinterpret_cast<float*>(stages));
  }
}

// ----------------------------------------------------------------------------------------
// host: geometry and dispatch
// ----------------------------------------------------------------------------------------
// 0 auto, 1 register kernels only, 2 pipeline whenever it fits, 3 as 2 with the column reduce
// as a second kernel
static std::atomic<int> g_path_override{0};

struct PipePlan {
  bool ok;
  bool full;  // branch-free instantiation applies
  int vb;     // bytes per vector: 16, or 8 / 4 where that makes the row divide evenly
  int K;
  int threads;
  int grid;
  size_t smem;
  PipeGeom g;
};

static int ilog2i(int v) {
  int l = 0;
  while ((1 << l) < v) ++l;
  return l;
}
static int next_pow2i(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

// tensors: how many input tensors are staged per tile (1 or 2)
static PipePlan plan_pipeline(bool backward, int64_t rows, int cols, int elem_bytes, int tensors,
                              bool allow_params_in_smem = true) {
  PipePlan P;
  memset(&P, 0, sizeof(P));
  const int vec = 16 / elem_bytes;
  if (cols % vec != 0 || rows <= 0) return P;
  const int nv = cols / vec;
  const int cta_threads = backward ? 512 : 256;
  // vectors per thread: forward 64 B per thread, backward about 16 columns per thread
  const int pref = backward ? (16 / vec) : 4;
  // register budget at 512 threads (128 registers): backward at most 16 columns per
  // thread, forward at most 32 elements per thread
  const int maxK = backward ? 16 / vec : 32 / vec;
  int K = 0, tpr = 0;
  int fK = 0, ftpr = 0;
  plan_override(&fK, &ftpr);
  if (fK > 0 && ftpr >= 8 && ftpr <= 512 && (ftpr & (ftpr - 1)) == 0 && fK <= maxK &&
      (fK & (fK - 1)) == 0 && (int64_t)fK * ftpr >= nv) {
    K = fK;
    tpr = ftpr;
  }
  for (int k = pref; k <= maxK && K == 0; k <<= 1) {
    int t = next_pow2i((nv + k - 1) / k);
    if (t > 512) continue;
    if (t < 8) t = 8;
    int kk = next_pow2i((nv + t - 1) / t);
    K = kk;
    tpr = t;
  }
  // Row lengths 3, 5 or 7 times a power of two (768, 1280, 2560, 5120, 6144, 12288 ...) do not
  // divide over a power-of-two number of threads with a power-of-two number of 16-byte vectors
  // each; the padded plan above would run them through the bounds-checked kernel with a
  // quarter or more of the lanes idle.  Look for an exact fit with K in {3, 5, 7} and, if
  // need be, 8- or 4-byte vectors; the branch-free instantiation then applies.
  int vb = 16;
  // Elements per thread the odd plans may use.  Backward, 16-bit types: 20 columns per thread
  // (K = 5 vectors of 4) still compile without spills at 128 registers and run faster than
  // the 16-column plans; 24 columns spill a little and are slower than 12 (6144 columns: 3986
  // vs 5237 GB/s), but faster than the two-kernel long-row path (12288 columns: 4018 vs 3365
  // GB/s), so they serve only rows that fit no other plan.  fp32 backward stays at 16.
  // Forward, 16-bit types: 40 elements per thread (K = 5 vectors of 8) with gamma / beta parked
  // in shared memory instead of registers.
  const int caps[2] = {backward ? (elem_bytes == 2 ? 20 : 16) : (elem_bytes == 2 && allow_params_in_smem ? 40 : 32),
                       backward && elem_bytes == 2 ? 24 : 0};
  for (int pass = 0; pass < 2; ++pass) {
    const int cap_elems = caps[pass];
    if (cap_elems == 0 || fK != 0) break;
    if (pass == 0 ? !(K == 0 || (int64_t)K * tpr != nv) : K != 0) break;
    const int min_vb = backward ? (elem_bytes == 4 ? 8 : 4) : (elem_bytes == 4 ? 16 : 8);
    int best_elems = 0;
    for (int cvb = 16; cvb >= min_vb; cvb >>= 1) {
      const int cvec = cvb / elem_bytes;
      if (cols % cvec != 0) continue;
      const int cnv = cols / cvec;
      for (int ck = 3; ck <= 7; ck += 2) {
        if (ck * cvec > cap_elems || cnv % ck != 0) continue;
        const int t = cnv / ck;
        if (t < 32 || t > 512 || (t & (t - 1)) != 0) continue;
        const int thr = t > cta_threads ? t : cta_threads;
        if (rows % (thr / t) != 0) continue;  // only the branch-free kernel exists for these
        if (ck * cvec > best_elems) {
          best_elems = ck * cvec;
          K = ck;
          tpr = t;
          vb = cvb;
        }
      }
    }
  }
  if (K == 0) return P;
  const int threads = tpr > cta_threads ? tpr : cta_threads;
  const int R = threads / tpr;
  const uint32_t row_bytes = (uint32_t)cols * elem_bytes;
  const uint32_t tile_bytes = row_bytes * R;
  const uint32_t stage = tile_bytes * tensors;
  // forward: two CTAs per SM with ~100 KB each; backward: one 512-thread CTA with ~200 KB
  const size_t budget = backward ? 200 * 1024 : 100 * 1024;
  int S = (int)((budget - kSmemHeader) / stage);
  if (S > 16) S = 16;
  if (S < 2) {
    // try the whole SM for one CTA
    S = (int)((220 * 1024 - kSmemHeader) / stage);
    if (S > 16) S = 16;
    if (S < 2) return P;
  }
  P.ok = true;
  P.full = tpr >= 32 && (int64_t)K * tpr == cols / (vb / elem_bytes) && rows % R == 0;
  P.vb = vb;
  P.K = K;
  P.threads = threads;
  // forward plans beyond 32 elements per thread keep gamma and beta behind the stages
  const bool params_in_smem = !backward && K * (vb / elem_bytes) > 32;
  if (params_in_smem) {
    S = (int)((budget - kSmemHeader - 2 * (size_t)row_bytes) / stage);
    if (S > 16) S = 16;
    // no room for two stages beside the parameters (two staged tensors of a long row): plan
    // again with at most 32 elements per thread
    if (S < 2) return plan_pipeline(backward, rows, cols, elem_bytes, tensors, false);
  }
  P.smem = kSmemHeader + (size_t)S * stage + (params_in_smem ? 2 * (size_t)row_bytes : 0);
  P.g.R = R;
  P.g.tpr = tpr;
  P.g.log2_tpr = ilog2i(tpr);
  P.g.S = S;
  P.g.row_bytes = row_bytes;
  P.g.second_off = tile_bytes;
  P.g.stage_stride = stage;
  const int64_t n_tiles = (rows + R - 1) / R;
  const int by_smem = (int)((227 * 1024) / P.smem), by_threads = 2048 / threads;
  const int per_sm = by_smem < by_threads ? by_smem : by_threads;
  const int64_t cap = (int64_t)usable_sms() * (per_sm < 1 ? 1 : per_sm);
  P.grid = (int)(n_tiles < cap ? n_tiles : cap);
  return P;
}

static bool pipeline_wanted(const PipePlan& P, int64_t rows) {
  const int ov = g_path_override.load(std::memory_order_relaxed);
  if (!P.ok || P.g.R <= 0 || P.grid <= 0 || ov == 1) return false;
  if (ov == 2 || ov == 3) return true;
  // worth it once every CTA streams several tiles
  const int64_t n_tiles = (rows + P.g.R - 1) / P.g.R;
  return n_tiles >= 4LL * P.grid || n_tiles >= 8LL * sm_count();
}

template <typename F>
static int set_smem(F kernel, size_t smem) {
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      cudaGetLastError();
      return FLN_ERR_LAUNCH;
    }
  }
  return FLN_OK;
}

// one branch-free instantiation with an odd K and / or short vectors; combinations that make no
// sense for the type (too many elements per thread, vectors shorter than four elements) are
// not instantiated
template <typename TI, typename TO, int KIND, int ACT, int KK, int VB>
static int fwd_pipe_odd(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  constexpr int VEC = VB / (int)sizeof(TI);
  if constexpr (VEC >= 4 && KK * VEC == 40 && sizeof(TI) == 2) {
    auto kern = norm_fwd_pipe_kernel<TI, TO, KK, KIND, ACT, 4, VB>;
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);
    FLN_CHECK_LAUNCH();
    return FLN_OK;
  } else if constexpr (VEC >= 4 && KK * VEC <= 32) {
    auto kern = norm_fwd_pipe_kernel<TI, TO, KK, KIND, ACT, 1, VB>;
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);
    FLN_CHECK_LAUNCH();
    return FLN_OK;
  } else {
    return FLN_PIPE_NOT_APPLICABLE;
  }
}

template <typename TI, typename TO, int KIND, int ACT>
static int fwd_pipe_k(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (P.vb != 16 || P.K == 3 || P.K == 5 || P.K == 7) {
    if (!P.full) return FLN_PIPE_NOT_APPLICABLE;
#define FLN_ODD(KK, VBB) \
  if (P.K == KK && P.vb == VBB) return fwd_pipe_odd<TI, TO, KIND, ACT, KK, VBB>(p, P, st);
    FLN_ODD(3, 16) FLN_ODD(5, 16) FLN_ODD(7, 16) FLN_ODD(3, 8) FLN_ODD(5, 8) FLN_ODD(7, 8)
#undef FLN_ODD
    return FLN_PIPE_NOT_APPLICABLE;
  }
#define FLN_LAUNCH(KK, FF)                                                                   \
  {                                                                                          \
    auto kern = norm_fwd_pipe_kernel<TI, TO, KK, KIND, ACT, FF>;                             \
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                             \
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                                         \
  }
#define FLN_CASE(KK)                                                \
  case KK:                                                          \
    if (P.full) FLN_LAUNCH(KK, 1)                                   \
    else FLN_LAUNCH(KK, 0)                                          \
    break;
  switch (P.K) {
    FLN_CASE(1) FLN_CASE(2) FLN_CASE(4) FLN_CASE(8)
    default:
      return FLN_PIPE_NOT_APPLICABLE;
  }
#undef FLN_CASE
#undef FLN_LAUNCH
  FLN_CHECK_LAUNCH();
  return FLN_OK;
}

template <typename TI, typename TO>
static int fwd_pipe_typed(int kind, int act, const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (kind == FLN_RMSNORM) return fwd_pipe_k<TI, TO, FLN_RMSNORM, FLN_ACT_NONE>(p, P, st);
  switch (act) {
    case FLN_ACT_NONE:
      return fwd_pipe_k<TI, TO, FLN_LAYERNORM, FLN_ACT_NONE>(p, P, st);
    case FLN_ACT_GELU_TANH:
      return fwd_pipe_k<TI, TO, FLN_LAYERNORM, FLN_ACT_GELU_TANH>(p, P, st);
    case FLN_ACT_GELU_ERF:
      return fwd_pipe_k<TI, TO, FLN_LAYERNORM, FLN_ACT_GELU_ERF>(p, P, st);
  }
  return FLN_PIPE_NOT_APPLICABLE;
}

int launch_fwd_pipeline(int kind, int act, int io_dtype, int out_dtype, const FwdParams& p0,
                        cudaStream_t st) {
  const int es = io_dtype == FLN_F32 ? 4 : 2;
  PipePlan P = plan_pipeline(false, p0.rows, p0.cols, es, p0.res != nullptr ? 2 : 1);
  if (!pipeline_wanted(P, p0.rows)) return FLN_PIPE_NOT_APPLICABLE;
  // Measured exceptions (automatic selection only).  A plain RMSNorm forward has one barrier per
  // row and little arithmetic; the non-persistent register-resident kernel then streams faster
  // than the ring (16384 x 8192 bf16: 88 vs 100 us; fp32 at every row length tried) unless its
  // power-of-two plan has to pad the row (1280, 5120, 12288 columns in 16-bit types).  The same
  // holds for the fp32 LayerNorm forward up to 4096 columns.
  if (g_path_override.load(std::memory_order_relaxed) == 0 && p0.res == nullptr && act == FLN_ACT_NONE &&
      io_dtype == out_dtype) {
    const Plan rp = make_plan(false, p0.rows, p0.cols, es, true);
    const bool exact = !rp.generic && rp.vec == 16 / es && (int64_t)rp.K * rp.tpr * rp.vec == p0.cols;
    if (kind == FLN_RMSNORM && !rp.generic && rp.vec == 16 / es && (exact || es == 4)) return FLN_PIPE_NOT_APPLICABLE;
    if (kind == FLN_LAYERNORM && es == 4 && exact && p0.cols <= 4096) return FLN_PIPE_NOT_APPLICABLE;
  }
  FwdParams p = p0;
  p.nv = p.cols / (P.vb / es);
  if (io_dtype == FLN_F32 && out_dtype == FLN_F32) return fwd_pipe_typed<float, float>(kind, act, p, P, st);
  if (io_dtype == FLN_F32 && out_dtype == FLN_BF16) return fwd_pipe_typed<float, __nv_bfloat16>(kind, act, p, P, st);
  if (io_dtype == FLN_BF16) return fwd_pipe_typed<__nv_bfloat16, __nv_bfloat16>(kind, act, p, P, st);
  return fwd_pipe_typed<__half, __half>(kind, act, p, P, st);
}

template <typename KernelT>
static int launch_bwd_kernel(KernelT kern, const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;
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

// branch-free instantiations with an odd K and short vectors (see plan_pipeline)
template <typename T, int KIND, int KK, int VB>
static int bwd_pipe_odd(const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  constexpr int VEC = VB / (int)sizeof(T);
  if constexpr (VEC >= 2 && KK * VEC <= (sizeof(T) == 2 ? 24 : 16)) {
    const bool fuse = p.sync != nullptr, dr = p.dres_in != nullptr;
    if (fuse && dr) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, true, true, VB>, p, P, st);
    if (fuse) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, true, false, VB>, p, P, st);
    if (dr) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, false, true, VB>, p, P, st);
    return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, false, false, VB>, p, P, st);
  } else {
    return FLN_PIPE_NOT_APPLICABLE;
  }
}

template <typename T, int KIND>
static int bwd_pipe_k(const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(T);
  if (P.vb != 16 || P.K == 3 || P.K == 5 || P.K == 7) {
    if (!P.full) return FLN_PIPE_NOT_APPLICABLE;
#define FLN_ODD(KK, VBB) \
  if (P.K == KK && P.vb == VBB) return bwd_pipe_odd<T, KIND, KK, VBB>(p, P, st);
    FLN_ODD(3, 16) FLN_ODD(3, 8) FLN_ODD(5, 8) FLN_ODD(7, 8) FLN_ODD(3, 4) FLN_ODD(5, 4) FLN_ODD(7, 4)
#undef FLN_ODD
    return FLN_PIPE_NOT_APPLICABLE;
  }
#define FLN_LAUNCH(KK, FF, DR)                                                               \
  {                                                                                          \
    if (p.sync != nullptr) {                                                                 \
      /* the grid barrier needs every CTA resident: cooperative launch */                   \
      auto kern = norm_bwd_pipe_kernel<T, (VEC * KK <= 16 ? KK : 1), KIND, FF, true, DR>;    \
      if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                           \
      cudaLaunchConfig_t cfg;                                                                \
      memset(&cfg, 0, sizeof(cfg));                                                          \
      cfg.gridDim = dim3((unsigned)P.grid);                                                  \
      cfg.blockDim = dim3((unsigned)P.threads);                                              \
      cfg.dynamicSmemBytes = P.smem;                                                         \
      cfg.stream = st;                                                                       \
      cudaLaunchAttribute attr;                                                              \
      attr.id = cudaLaunchAttributeCooperative;                                              \
      attr.val.cooperative = 1;                                                              \
      cfg.attrs = &attr;                                                                     \
      cfg.numAttrs = 1;                                                                      \
      if (cudaLaunchKernelEx(&cfg, kern, p, P.g) != cudaSuccess) {                           \
        cudaGetLastError();                                                                  \
        return FLN_ERR_LAUNCH;                                                               \
      }                                                                                      \
    } else {                                                                                 \
      auto kern = norm_bwd_pipe_kernel<T, (VEC * KK <= 16 ? KK : 1), KIND, FF, false, DR>;   \
      if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                           \
      kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                                       \
    }                                                                                        \
  }
#define FLN_CASE(KK)                                       \
  case KK:                                                 \
    if (VEC * KK > 16) return FLN_PIPE_NOT_APPLICABLE;     \
    if (p.dres_in != nullptr) {                            \
      if (P.full) FLN_LAUNCH(KK, true, true)               \
      else FLN_LAUNCH(KK, false, true)                     \
    } else if (P.full) FLN_LAUNCH(KK, true, false)         \
    else FLN_LAUNCH(KK, false, false)                      \
    break;
  switch (P.K) {
    FLN_CASE(1) FLN_CASE(2) FLN_CASE(4)
    default:
      return FLN_PIPE_NOT_APPLICABLE;
  }
#undef FLN_CASE
#undef FLN_LAUNCH
  FLN_CHECK_LAUNCH();
  return FLN_OK;
}

static PipePlan plan_bwd_pipeline(int64_t rows, int cols, int es, bool with_dres) {
  return plan_pipeline(true, rows, cols, es, with_dres ? 3 : 2);
}

bool describe_pipeline(bool backward, int64_t rows, int cols, int elem_bytes, PipeDescription* out) {
  PipePlan P = backward ? plan_bwd_pipeline(rows, cols, elem_bytes, false) : plan_pipeline(false, rows, cols, elem_bytes, 1);
  if (!pipeline_wanted(P, rows)) return false;
  if (!backward && elem_bytes == 4 && cols <= 4096 && g_path_override.load(std::memory_order_relaxed) == 0) {
    // the fp32 LayerNorm forward of short exact rows goes to the register kernel (launch_fwd_pipeline)
    const Plan rp = make_plan(false, rows, cols, elem_bytes, true);
    if (!rp.generic && rp.vec == 4 && (int64_t)rp.K * rp.tpr * rp.vec == cols) return false;
  }
  // the odd plans exist only as branch-free instantiations; K = 8 only for fp32 forward
  if ((P.vb != 16 || P.K == 3 || P.K == 5 || P.K == 7) && !P.full) return false;
  out->vector_bytes = P.vb;
  out->K = P.K;
  out->tpr = P.g.tpr;
  out->threads = P.threads;
  out->rows_per_cta = P.g.R;
  out->stages = P.g.S;
  out->grid = P.grid;
  return true;
}

int64_t bwd_pipeline_partial_rows(int kind, int dtype, int64_t rows, int cols, bool with_dres) {
  (void)kind;
  const int es = dtype == FLN_F32 ? 4 : 2;
  PipePlan P = plan_bwd_pipeline(rows, cols, es, with_dres);
  if (!pipeline_wanted(P, rows)) return 0;
  return (int64_t)P.grid * P.g.R;
}

static bool cooperative_launch_supported() {
  static int cache[64];  // 0 unknown, 1 no, 2 yes
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  if (cache[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess) {
      cudaGetLastError();
      v = 0;
    }
    cache[dev] = v ? 2 : 1;
  }
  return cache[dev] == 2;
}

static unsigned long long next_launch_token() {
  static std::atomic<unsigned long long> ctr{0x5bd1e995ull};
  unsigned long long t;
  do {
    t = ctr.fetch_add(1, std::memory_order_relaxed) & ((1ull << 40) - 1);
  } while (t == 0);
  return t;
}

int launch_bwd_pipeline(int kind, int dtype, const BwdParams& p0, cudaStream_t st, bool* reduced) {
  const int es = dtype == FLN_F32 ? 4 : 2;
  *reduced = false;
  PipePlan P = plan_bwd_pipeline(p0.rows, p0.cols, es, p0.dres_in != nullptr);
  if (!pipeline_wanted(P, p0.rows)) return FLN_PIPE_NOT_APPLICABLE;
  BwdParams p = p0;
  p.nv = p.cols / (P.vb / es);
  // Fused column reduce: one CTA per SM (so the whole grid is resident at once), the
  // one-row kernel, stage memory large enough for the 16 x 128 floats of the combine step.
  const bool fuse = p.sync != nullptr && p.partials != nullptr && P.grid <= usable_sms() &&
                    P.grid < 4096 && P.smem >= (size_t)kSmemHeader + 16 * 128 * sizeof(float) &&
                    g_path_override.load(std::memory_order_relaxed) != 3 && cooperative_launch_supported();
  if (fuse) {
    p.token = next_launch_token();
    *reduced = true;
  } else {
    p.sync = nullptr;
  }
#define FLN_RUN(T) \
  (kind == FLN_LAYERNORM ? bwd_pipe_k<T, FLN_LAYERNORM>(p, P, st) : bwd_pipe_k<T, FLN_RMSNORM>(p, P, st))
  int rc = dtype == FLN_F32 ? FLN_RUN(float) : (dtype == FLN_BF16 ? FLN_RUN(__nv_bfloat16) : FLN_RUN(__half));
  if (rc == FLN_ERR_LAUNCH && fuse) {
    // the cooperative launch was refused (the device is shared in a way that rules out a
    // resident grid): run the plain launch and let the caller reduce the partial rows
    p.sync = nullptr;
    *reduced = false;
    rc = dtype == FLN_F32 ? FLN_RUN(float) : (dtype == FLN_BF16 ? FLN_RUN(__nv_bfloat16) : FLN_RUN(__half));
  }
  return rc;
#undef FLN_RUN
}

}  // namespace fln

using namespace fln;

extern "C" void fln_set_path_override(int mode) { g_path_override.store(mode, std::memory_order_relaxed); }

// Host-only consistency check of the pipeline planner over a grid of shapes: every plan it
// accepts must describe a launch that exists (at least two stages, shared memory within the
// opt-in limit, a row that divides exactly where the branch-free kernel is claimed, a grid).
// Returns the number of violations.  Needs no GPU.
extern "C" int fln_planner_selftest(void) {
  static const int kCols[] = {8,    16,   64,   96,   256,  512,  768,  1000, 1024, 1280, 1536,  1600,  2048, 2560,
                              3072, 4096, 5120, 6144, 7168, 8192, 9216, 10240, 12288, 14336, 16384, 20480, 32768};
  static const int64_t kRows[] = {1, 7, 64, 600, 2049, 4096, 16384, 131072};
  int bad = 0;
  for (int cols : kCols)
    for (int64_t rows : kRows)
      for (int es = 2; es <= 4; es += 2)
        for (int backward = 0; backward <= 1; ++backward)
          for (int tensors = backward ? 2 : 1; tensors <= (backward ? 3 : 2); ++tensors) {
            const PipePlan P = plan_pipeline(backward != 0, rows, cols, es, tensors);
            if (!P.ok) continue;
            const int vec = P.vb / es;
            bool ok = P.g.S >= 2 && P.g.R >= 1 && P.grid >= 1 && P.smem <= 227u * 1024u && P.threads >= 32 &&
                      P.threads <= 512 && P.K >= 1 && vec >= 1 && cols % vec == 0 &&
                      (int64_t)P.K * P.g.tpr >= cols / vec && P.g.tpr * P.g.R == P.threads &&
                      P.smem >= (size_t)kSmemHeader + (size_t)P.g.S * P.g.stage_stride;
            if (P.full) ok = ok && (int64_t)P.K * P.g.tpr * vec == cols && rows % P.g.R == 0;
            // odd K or short vectors exist only as branch-free instantiations
            if ((P.vb != 16 || P.K == 3 || P.K == 5 || P.K == 7) && !P.full) ok = false;
            if (!ok) ++bad;
          }
  return bad;
}

extern "C" int fln_device_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  }
  return v;
}
