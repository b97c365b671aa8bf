// Pipelined backward: instantiations with an odd number of vectors per thread and / or vectors
// shorter than 16 bytes (row lengths 3, 5, 7 times a power of two; see plan_pipeline).
#include "fln_pipeline_bwd_kernel.cuh"

namespace fln {

// branch-free instantiations with an odd K and short vectors (see plan_pipeline)
template <typename T, int KIND, int KK, int VB>
static int bwd_pipe_odd(const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  constexpr int VEC = VB / (int)sizeof(T);
  // fp32 with 20 columns per thread: LayerNorm only with its dbeta accumulators in shared memory
  // (below), RMSNorm has none
  constexpr int kMaxCols = sizeof(T) == 2 ? 24 : ((KK == 5 && VB == 16) ? 20 : 16);
  if constexpr (VEC >= 2 && KK * VEC <= kMaxCols) {
    const bool fuse = p.sync != nullptr, dr = p.dres_in != nullptr;
    // 24 columns per thread, LayerNorm: the dbeta accumulators in shared memory
    if constexpr (KIND == FLN_LAYERNORM && VB == 16 && ((sizeof(T) == 2 && KK == 3) || (sizeof(T) == 4 && KK == 5))) {
      if (!dr && P.bsm && P.threads == 512) {
#define FLN_BSM_LT(L)                                                                                                       \
  if (P.g.tpr == (1 << L)) {                                                                                                \
    if (fuse)                                                                                                               \
      return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, true, false, VB, L, false, false, true>, p, P, st); \
    return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, false, false, VB, L, false, false, true>, p, P, st);  \
  }
        FLN_BSM_LT(9) FLN_BSM_LT(8) FLN_BSM_LT(7) FLN_BSM_LT(6) FLN_BSM_LT(5)
#undef FLN_BSM_LT
      }
    }
    if constexpr (KIND == FLN_LAYERNORM && sizeof(T) == 4 && KK * VEC > 16) return FLN_PIPE_NOT_APPLICABLE;
    // geometry as template arguments for rows of 32 to 512 threads (no residual-stream gradient)
    if (!dr && P.threads == 512) {
#define FLN_ODD_LT(L)                                                                                              \
  if (P.g.tpr == (1 << L)) {                                                                                       \
    if (fuse) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, true, false, VB, L>, p, P, st);     \
    return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, false, false, VB, L>, p, P, st);              \
  }
      FLN_ODD_LT(9) FLN_ODD_LT(8) FLN_ODD_LT(7) FLN_ODD_LT(6) FLN_ODD_LT(5)
#undef FLN_ODD_LT
    }
    if (fuse && dr) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, true, true, VB>, p, P, st);
    if (fuse) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, true, false, VB>, p, P, st);
    if (dr) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, false, true, VB>, p, P, st);
    return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, false, false, VB>, p, P, st);
  } else {
    return FLN_PIPE_NOT_APPLICABLE;
  }
}

template <typename T, int KIND>
static int bwd_pipe_odd_k(const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (!P.full) return FLN_PIPE_NOT_APPLICABLE;
#define FLN_ODD(KK, VBB) \
  if (P.K == KK && P.vb == VBB) return bwd_pipe_odd<T, KIND, KK, VBB>(p, P, st);
  FLN_ODD(3, 16) FLN_ODD(5, 16) FLN_ODD(3, 8) FLN_ODD(5, 8) FLN_ODD(7, 8) FLN_ODD(3, 4) FLN_ODD(5, 4) FLN_ODD(7, 4)
#undef FLN_ODD
  return FLN_PIPE_NOT_APPLICABLE;
}

#define FLN_BY_TYPE(FN)                                                                               \
  if (kind == FLN_LAYERNORM) {                                                                        \
    if (dtype == FLN_F32) return FN<float, FLN_LAYERNORM>(p, P, st);                                  \
    if (dtype == FLN_BF16) return FN<__nv_bfloat16, FLN_LAYERNORM>(p, P, st);                         \
    return FN<__half, FLN_LAYERNORM>(p, P, st);                                                       \
  }                                                                                                   \
  if (dtype == FLN_F32) return FN<float, FLN_RMSNORM>(p, P, st);                                      \
  if (dtype == FLN_BF16) return FN<__nv_bfloat16, FLN_RMSNORM>(p, P, st);                             \
  return FN<__half, FLN_RMSNORM>(p, P, st);

int bwd_pipe_odd_any(int kind, int dtype, const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  FLN_BY_TYPE(bwd_pipe_odd_k)
}
#undef FLN_BY_TYPE

}  // namespace fln
