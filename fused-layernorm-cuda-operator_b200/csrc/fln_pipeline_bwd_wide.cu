// Pipelined backward for 16-bit rows of 10248 .. 16384 columns: one 512-thread CTA per row, up to
// 32 columns per thread, in two passes over the staged row.
//
// 32 columns per thread do not fit the registers of the one-pass kernel (the row as floats, gamma
// and two accumulators per column), and a row shared by a cluster pair pays half a microsecond
// per row for the exchange of the row sums, as much as half the row's bytes take in 16-bit
// types.  Here pass 1 reads dy and x from the stage and forms the two row sums without keeping
// anything; after the reduction pass 2 reads the stage again and produces dx and the column
// sums.  What stays in registers across rows: gamma in the I/O type (16 registers) and the
// dgamma accumulators (32); the dbeta accumulators sit in shared memory behind the stages
// (conflict-free float2 per thread and column pair).  Two CTA barriers per row: the reduction,
// and the release of the stage after pass 2.
//
// Rows of 16384 and 14336 columns divide exactly (4 vectors of 16 bytes, 7 of 8 bytes per
// thread).  Any other row length that is a multiple of 8 runs the TAIL form: 3 or 4 vectors of 16
// bytes per thread of which only the last is tested against the end of the row (11008 = 43 *
// 256, 12800, 13824 = 27 * 512 columns ...).
#include "fln_pipeline_bwd_kernel.cuh"

namespace fln {

// rows of K * (VB / 2) * 512 columns: (K, VB) = (4, 16) -> 16384, (7, 8) -> 14336; TAIL: rows of
// more than (K - 1) * (VB / 2) * 512 and fewer than K * (VB / 2) * 512 columns
template <typename T, int KIND, int K, int VB, bool TAIL = false>
__global__ void __launch_bounds__(512) norm_bwd_twopass_kernel(const BwdParams p, const PipeGeom g) {
  constexpr int VEC = VB / 2, V2 = VEC / 2, NR = KIND == FLN_LAYERNORM ? 2 : 1;
  const int cols = TAIL ? p.cols : K * VEC * 512;
  const uint32_t row_bytes = (uint32_t)cols * 2u, stage_stride = 2u * row_bytes;
  constexpr uint32_t k_off = 512 * VB;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  float* s_red = reinterpret_cast<float*>(smem + 256);
  unsigned char* stages = smem + kSmemHeader;
  const int tid = threadIdx.x;
  const int S = g.S;
  // this thread's last vector lies in the row (the others do for every thread)
  const bool last_ok = !TAIL || tid + (K - 1) * 512 < p.nv;
#define FLN_IN_ROW(k) (!TAIL || (k) < K - 1 || last_ok)
  float2* s_accb = reinterpret_cast<float2*>(stages + (size_t)S * stage_stride) + tid;  // [K * V2][512]

  const int my_tiles = my_tile_count(p.rows);
  if (tid == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&full[s], 2);
    mbar_init_fence();
  }
  __syncthreads();

  const int which = tid >> 5;
  const bool is_producer = (tid & 31) == 0 && which < 2;
  auto issue = [&](int i, int s, bool skip_copy) {
    const int64_t row0 = (int64_t)blockIdx.x + (int64_t)i * gridDim.x;
    unsigned char* dst = stages + (size_t)s * stage_stride + (size_t)which * row_bytes;
    const T* src = reinterpret_cast<const T*>(which == 0 ? p.dy : p.x);
    mbar_expect_tx(&full[s], row_bytes);
    if (!skip_copy) bulk_g2s(dst, src + row0 * cols, row_bytes, &full[s]);
  };
  if (is_producer) {
    const bool fault = tid == 0 && blockIdx.x == 0 && (*p.fault & 1) != 0;
    const int pre = my_tiles < S ? my_tiles : S;
    for (int i = 0; i < pre; ++i) issue(i, i, fault && i == 0);
  }

  Pack<T, VEC> gp[K];
  float2 acc_g[K][V2];
#pragma unroll
  for (int k = 0; k < K; ++k) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) gp[k].e[e] = Cvt<T>::from_f(1.f);
    if (p.gamma != nullptr && FLN_IN_ROW(k)) gp[k] = ld_param<T, VEC>(reinterpret_cast<const T*>(p.gamma) + (int64_t)(tid + k * 512) * VEC);
#pragma unroll
    for (int e = 0; e < V2; ++e) {
      acc_g[k][e] = f2(0.f);
      if (KIND == FLN_LAYERNORM) s_accb[(k * V2 + e) * 512] = f2(0.f);
    }
  }

  int64_t row = blockIdx.x;
  float mean_n = 0.f, rstd_n = 0.f;
  if (my_tiles > 0) {
    if (KIND == FLN_LAYERNORM) mean_n = __ldg(p.mean + row);
    rstd_n = __ldg(p.rstd + row);
  }
  const float inv_n = 1.0f / (float)cols;
  int s = 0;
  uint32_t phase = 0;
  bool aborted = false;
  int i = 0;
  for (; i < my_tiles; ++i, row += gridDim.x) {
    const float mean = mean_n, rstd = rstd_n;
    if (i + 1 < my_tiles) {
      if (KIND == FLN_LAYERNORM) mean_n = __ldg(p.mean + row + gridDim.x);
      rstd_n = __ldg(p.rstd + row + gridDim.x);
    }
    const bool landed = mbar_wait_bounded(&full[s], phase, p.wait_ns);
    const unsigned char* st = stages + (size_t)s * stage_stride + (uint32_t)tid * (uint32_t)VB;
    const float2 r2 = f2(rstd), nmr = f2(-mean * rstd);

    // ---- pass 1: the row sums
    float2 r0 = f2(0.f), r1 = f2(0.f);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (!FLN_IN_ROW(k)) continue;
      float2 dyf[V2], xh[V2], gm[V2];
      unpack2<T, VEC>(stage_vec<T, VEC>(st + k * k_off), dyf);
      unpack2<T, VEC>(stage_vec<T, VEC>(st + row_bytes + k * k_off), xh);
      unpack2<T, VEC>(gp[k], gm);
#pragma unroll
      for (int e = 0; e < V2; ++e) {
        const float2 xhat = f2fma(xh[e], r2, nmr);
        const float2 gg = f2mul(dyf[e], gm[e]);
        r0 = f2fma(gg, xhat, r0);
        if (KIND == FLN_LAYERNORM) r1 = f2add(r1, gg);
      }
    }
    float red[NR];
    red[0] = r0.x + r0.y;
    if (KIND == FLN_LAYERNORM) red[NR - 1] = r1.x + r1.y;
    float* sr = s_red + (i & 1) * 64;
    rowsum_warp<NR>(red, 512, sr);
    if (!__syncthreads_and(landed ? 1 : 0)) {
      aborted = true;
      break;
    }
    rowsum_cta<NR>(red, 512, sr);
    const float2 nc1 = f2(-(red[0] * inv_n));
    const float2 nc2 = f2(KIND == FLN_LAYERNORM ? -(red[NR - 1] * inv_n) : 0.f);

    // ---- pass 2: dx and the column sums, from a second read of the stage
    T* __restrict__ dxr = reinterpret_cast<T*>(p.dx) + row * (int64_t)cols + (int64_t)tid * VEC;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (!FLN_IN_ROW(k)) continue;
      float2 dyf[V2], xh[V2], gm[V2];
      unpack2<T, VEC>(stage_vec<T, VEC>(st + k * k_off), dyf);
      unpack2<T, VEC>(stage_vec<T, VEC>(st + row_bytes + k * k_off), xh);
      unpack2<T, VEC>(gp[k], gm);
      float2 o[V2];
#pragma unroll
      for (int e = 0; e < V2; ++e) {
        const float2 xhat = f2fma(xh[e], r2, nmr);
        // the product of two 16-bit values is exact in fp32: the fma equals (dy * gamma) - c2
        const float2 gc = f2fma(dyf[e], gm[e], nc2);
        o[e] = f2mul(r2, f2fma(xhat, nc1, gc));
        acc_g[k][e] = f2fma(dyf[e], xhat, acc_g[k][e]);
        if (KIND == FLN_LAYERNORM) s_accb[(k * V2 + e) * 512] = f2add(s_accb[(k * V2 + e) * 512], dyf[e]);
      }
      if (p.dx != nullptr) {
        Pack<T, VEC> out;
        pack2<T, VEC>(o, out);
        st_stream<T, VEC>(dxr + (int64_t)k * 512 * VEC, out);
      }
    }
    __syncthreads();  // every thread is done with stage s
    if (is_producer && i + S < my_tiles) issue(i + S, s, false);
    if (++s == S) {
      s = 0;
      phase ^= 1u;
    }
  }
  if (aborted && tid == 0) pipeline_abort(p.status, full, S, s, phase, my_tiles - i < S ? my_tiles - i : S, p.wait_ns);

  if (p.partials != nullptr && !aborted) {
    float* __restrict__ pg = p.partials + (int64_t)blockIdx.x * (int64_t)(NR * cols);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      if (!FLN_IN_ROW(k)) continue;
      const int64_t c0 = (int64_t)(tid + k * 512) * VEC;
#pragma unroll
      for (int e = 0; e < V2; e += 2) {  // V2 is 4 or 2
        *reinterpret_cast<float4*>(pg + c0 + 2 * e) =
            make_float4(acc_g[k][e].x, acc_g[k][e].y, acc_g[k][e + 1].x, acc_g[k][e + 1].y);
        if (KIND == FLN_LAYERNORM) {
          const float2 b0 = s_accb[(k * V2 + e) * 512], b1 = s_accb[(k * V2 + e + 1) * 512];
          *reinterpret_cast<float4*>(pg + cols + c0 + 2 * e) = make_float4(b0.x, b0.y, b1.x, b1.y);
        }
      }
    }
  }
#undef FLN_IN_ROW
}

template <typename T, int KIND, int K, int VB, bool TAIL = false>
static int launch_twopass(const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  auto kern = norm_bwd_twopass_kernel<T, KIND, K, VB, TAIL>;
  if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;
  kern<<<P.grid, 512, P.smem, st>>>(p, P.g);
  FLN_CHECK_LAUNCH();
  return FLN_OK;
}

template <typename T>
static int twopass_typed(int kind, const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (P.tail) {
    if (P.vb != 16 || p.cols % 8 != 0 || p.cols <= (P.K - 1) * 4096 || p.cols >= P.K * 4096) return FLN_PIPE_NOT_APPLICABLE;
    if (P.K == 3)
      return kind == FLN_LAYERNORM ? launch_twopass<T, FLN_LAYERNORM, 3, 16, true>(p, P, st)
                                   : launch_twopass<T, FLN_RMSNORM, 3, 16, true>(p, P, st);
    if (P.K == 4)
      return kind == FLN_LAYERNORM ? launch_twopass<T, FLN_LAYERNORM, 4, 16, true>(p, P, st)
                                   : launch_twopass<T, FLN_RMSNORM, 4, 16, true>(p, P, st);
    return FLN_PIPE_NOT_APPLICABLE;
  }
  if (P.K == 4 && P.vb == 16 && p.cols == 16384)
    return kind == FLN_LAYERNORM ? launch_twopass<T, FLN_LAYERNORM, 4, 16>(p, P, st)
                                 : launch_twopass<T, FLN_RMSNORM, 4, 16>(p, P, st);
  if (P.K == 7 && P.vb == 8 && p.cols == 14336)
    return kind == FLN_LAYERNORM ? launch_twopass<T, FLN_LAYERNORM, 7, 8>(p, P, st)
                                 : launch_twopass<T, FLN_RMSNORM, 7, 8>(p, P, st);
  return FLN_PIPE_NOT_APPLICABLE;
}

int bwd_pipe_wide_any(int kind, int dtype, const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (!P.wide || p.dres_in != nullptr || p.sync != nullptr) return FLN_PIPE_NOT_APPLICABLE;
  if (dtype == FLN_BF16) return twopass_typed<__nv_bfloat16>(kind, p, P, st);
  if (dtype == FLN_F16) return twopass_typed<__half>(kind, p, P, st);
  return FLN_PIPE_NOT_APPLICABLE;
}

}  // namespace fln
