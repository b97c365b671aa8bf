// Pipelined forward: the kernel and its dispatch.  See fln_pipeline.cuh for the ring and the
// scheduling of tiles.
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
template <typename TI, typename TO, int K, int KIND, int ACT, int MODE, int VB = 16, int LT = -1>
__global__ void __launch_bounds__(512) norm_fwd_pipe_kernel(const FwdParams p, const PipeGeom g) {
  constexpr int VEC = VB / sizeof(TI);  // a multiple of 4 (the statistics run four chains)
  constexpr int V2 = VEC / 2;
  constexpr bool FULL = MODE >= 1;
  constexpr bool PSM = MODE == 4;
  constexpr bool TAIL = MODE == 5;
  constexpr bool CT = LT >= 0;
  constexpr int LTC = CT ? LT : 0;
  constexpr int NT = LTC > 8 ? (1 << LTC) : 256;  // threads per CTA of the compile-time geometry
  static_assert(!CT || MODE == 1 || MODE == 4 || MODE == 5, "compile-time geometry is for the FULL kernels");
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

  float2 gam[PSM ? 1 : K][V2], bet[PSM ? 1 : K][V2];
  bool vok[K];  // does vector k of this thread exist in the row
  unsigned char* s_gamma = stages + (size_t)S * g.stage_stride;  // PSM: [cols] gamma, then [cols] beta
  unsigned char* s_beta = s_gamma + row_bytes;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int iv = lane_r + k * tpr;
    vok[k] = FLN_WHOLE(k) ? true : iv < p.nv;
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
        } else {
#pragma unroll
          for (int e = 0; e < V2; ++e) o[e] = f2fma(f2mul(f[k][e], r2), gam[k][e], bet[k][e]);
        }
        if (ACT != FLN_ACT_NONE) {
#pragma unroll
          for (int e = 0; e < V2; ++e) o[e] = make_float2(apply_act<ACT>(o[e].x), apply_act<ACT>(o[e].y));
        }
        Pack<TO, VEC> out;
        pack2<TO, VEC>(o, out);
        st_stream<TO, VEC>(yr + (int64_t)k * tpr * VEC, out);
      }
    }
    if (++s == S) {
      s = 0;
      phase ^= 1u;
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

// one branch-free instantiation with an odd K and / or short vectors; combinations that make no
// sense for the type (too many elements per thread, vectors shorter than four elements) are
// not instantiated
template <typename TI, typename TO, int KIND, int ACT, int KK, int VB>
static int fwd_pipe_odd(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  constexpr int VEC = VB / (int)sizeof(TI);
  constexpr int MODE =
      (VEC >= 4 && KK * VEC > 32 && KK * VEC <= 48 && sizeof(TI) == 2) ? 4 : ((VEC >= 4 && KK * VEC <= 32) ? 1 : -1);
  if constexpr (MODE > 0) {
#define FLN_GO(LTT)                                                             \
  {                                                                             \
    auto kern = norm_fwd_pipe_kernel<TI, TO, KK, KIND, ACT, MODE, VB, LTT>;     \
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                \
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                            \
    FLN_CHECK_LAUNCH();                                                         \
    return FLN_OK;                                                              \
  }
    // geometry as template arguments for the plain forward (no GELU, same type out as in)
    if constexpr (ACT == FLN_ACT_NONE && std::is_same<TI, TO>::value) {
      const int nt = P.g.tpr > 256 ? P.g.tpr : 256;
      if (P.threads == nt) {
        if (P.g.tpr == 32) FLN_GO(5)
        if (P.g.tpr == 64) FLN_GO(6)
        if (P.g.tpr == 128) FLN_GO(7)
        if (P.g.tpr == 256) FLN_GO(8)
        if (P.g.tpr == 512) FLN_GO(9)
      }
    }
    FLN_GO(-1)
#undef FLN_GO
  } else {
    return FLN_PIPE_NOT_APPLICABLE;
  }
}

// rows whose last vector is ragged (plan_pipeline's `tail` plans): K = 7 vectors of 8 bytes
// (16-bit types) or 16 bytes (fp32); plain forward only
template <typename TI, typename TO, int KIND, int ACT>
static int fwd_pipe_tail(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  if constexpr (ACT == FLN_ACT_NONE && std::is_same<TI, TO>::value) {
    constexpr int VB = sizeof(TI) == 2 ? 8 : 16;
    const int nt = P.g.tpr > 256 ? P.g.tpr : 256;
    if (P.K != 7 || P.vb != VB || P.threads != nt) return FLN_PIPE_NOT_APPLICABLE;
#define FLN_GO(LTT)                                                          \
  if (P.g.tpr == (1 << LTT)) {                                               \
    auto kern = norm_fwd_pipe_kernel<TI, TO, 7, KIND, ACT, 5, VB, LTT>;      \
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;             \
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                         \
    FLN_CHECK_LAUNCH();                                                      \
    return FLN_OK;                                                           \
  }
    FLN_GO(5) FLN_GO(6) FLN_GO(7) FLN_GO(8) FLN_GO(9)
#undef FLN_GO
  }
  return FLN_PIPE_NOT_APPLICABLE;
}

template <typename TI, typename TO, int KIND, int ACT>
static int fwd_pipe_k(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (P.tail) return fwd_pipe_tail<TI, TO, KIND, ACT>(p, P, st);
  if (P.vb != 16 || P.K == 3 || P.K == 5 || P.K == 6 || P.K == 7) {
    if (!P.full) return FLN_PIPE_NOT_APPLICABLE;
#define FLN_ODD(KK, VBB) \
  if (P.K == KK && P.vb == VBB) return fwd_pipe_odd<TI, TO, KIND, ACT, KK, VBB>(p, P, st);
    FLN_ODD(3, 16) FLN_ODD(5, 16) FLN_ODD(6, 16) FLN_ODD(7, 16) FLN_ODD(3, 8) FLN_ODD(5, 8) FLN_ODD(7, 8)
#undef FLN_ODD
    return FLN_PIPE_NOT_APPLICABLE;
  }
#define FLN_LAUNCH(KK, FF)                                                                   \
  {                                                                                          \
    auto kern = norm_fwd_pipe_kernel<TI, TO, KK, KIND, ACT, FF>;                             \
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                             \
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                                         \
  }
#define FLN_LAUNCH_CT(KK, LTT)                                                               \
  {                                                                                          \
    auto kern = norm_fwd_pipe_kernel<TI, TO, KK, KIND, ACT, 1, 16, LTT>;                     \
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                             \
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                                         \
  }
  // the planner's preferred split (64 bytes per thread) with whole rows in a 256-thread CTA:
  // geometry as template arguments
#define FLN_CASE(KK)                                                \
  case KK:                                                          \
    if constexpr (KK == 4) {                                        \
      if (P.full && P.threads == 256 && P.g.tpr == 256) FLN_LAUNCH_CT(KK, 8)      \
      else if (P.full && P.threads == 256 && P.g.tpr == 128) FLN_LAUNCH_CT(KK, 7) \
      else if (P.full && P.threads == 256 && P.g.tpr == 64) FLN_LAUNCH_CT(KK, 6)  \
      else if (P.full && P.threads == 256 && P.g.tpr == 32) FLN_LAUNCH_CT(KK, 5)  \
      else if (P.full && P.threads == 512 && P.g.tpr == 512) FLN_LAUNCH_CT(KK, 9) \
      else if (P.full) FLN_LAUNCH(KK, 1)                            \
      else FLN_LAUNCH(KK, 0)                                        \
    } else if constexpr (KK * 16 / sizeof(TI) <= 32) {              \
      if (P.full) FLN_LAUNCH(KK, 1)                                 \
      else FLN_LAUNCH(KK, 0)                                        \
    } else {                                                        \
      return FLN_PIPE_NOT_APPLICABLE;                               \
    }                                                               \
    break;
  switch (P.K) {
    FLN_CASE(1) FLN_CASE(2) FLN_CASE(4) FLN_CASE(8)
    default:
      return FLN_PIPE_NOT_APPLICABLE;
  }
#undef FLN_CASE
#undef FLN_LAUNCH
#undef FLN_LAUNCH_CT
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
  // the ragged-last-vector plans exist for the plain forward only
  const bool allow_tail = act == FLN_ACT_NONE && io_dtype == out_dtype;
  PipePlan P = plan_pipeline(false, p0.rows, p0.cols, es, p0.res != nullptr ? 2 : 1, true, allow_tail);
  if (!pipeline_wanted(P, p0.rows)) return FLN_PIPE_NOT_APPLICABLE;
  // Measured exceptions (automatic selection only): fp32 rows that the non-persistent
  // register-resident kernel holds exactly stream faster there than through the ring -- a plain
  // RMSNorm forward at every row length tried, the LayerNorm forward up to 4096 columns, where
  // the ring runs 16 elements per thread (1024 / 2048 / 4096: 6743 / 6753 / 6658 vs 5651 / 5797 /
  // 5504 GB/s; from 24 elements per thread the ring wins, 8192: 6651 vs 5497).  In 16-bit types
  // the ring with its tiles handed out on demand is the faster one (RMSNorm 16384 x 8192 bf16:
  // 84.1 vs 86.4 us).
  if (path_override() == 0 && p0.res == nullptr && act == FLN_ACT_NONE &&
      io_dtype == out_dtype) {
    const Plan rp = make_plan(false, p0.rows, p0.cols, es, true);
    const bool exact = !rp.generic && rp.vec == 16 / es && (int64_t)rp.K * rp.tpr * rp.vec == p0.cols;
    // (padded register plans of long rows excepted -- 6144 columns: 6188 vs 6707 GB/s)
    if (kind == FLN_RMSNORM && !rp.generic && rp.vec == 16 / es && es == 4 && (exact || p0.cols <= 4096))
      return FLN_PIPE_NOT_APPLICABLE;
    if (kind == FLN_LAYERNORM && es == 4 && exact && p0.cols <= 4096) return FLN_PIPE_NOT_APPLICABLE;
  }
  FwdParams p = p0;
  p.nv = p.cols / (P.vb / es);
  DeviceWords w;
  if (!device_words(&w)) return FLN_ERR_LAUNCH;
  p.sched = w.sched + 2 * next_sched_slot();
  p.wait_ns = wait_limit_ns();
  p.status = w.status;
  p.fault = w.fault;
  if (io_dtype == FLN_F32 && out_dtype == FLN_F32) return fwd_pipe_typed<float, float>(kind, act, p, P, st);
  if (io_dtype == FLN_F32 && out_dtype == FLN_BF16) return fwd_pipe_typed<float, __nv_bfloat16>(kind, act, p, P, st);
  if (io_dtype == FLN_BF16) return fwd_pipe_typed<__nv_bfloat16, __nv_bfloat16>(kind, act, p, P, st);
  return fwd_pipe_typed<__half, __half>(kind, act, p, P, st);
}

}  // namespace fln
