// Pipelined backward: rows shared by the two CTAs of a thread-block cluster.
#include "fln_pipeline_bwd_kernel.cuh"

namespace fln {

// a row shared by the two CTAs of a cluster: the half row's plan decides the instantiation
template <typename T, int KIND>
static int bwd_pipe_pair(const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  constexpr int VEC = 16 / (int)sizeof(T);
#define FLN_PAIR(KK, VBB)                                                                                       \
  if (P.K == KK && P.vb == VBB) {                                                                               \
    if constexpr ((VBB / (int)sizeof(T)) >= 2 && KK * (VBB / (int)sizeof(T)) <= 20)                             \
      return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, false, false, VBB, 9, true>, p, P, st);  \
  }
  FLN_PAIR(16 / VEC, 16) FLN_PAIR(3, 8) FLN_PAIR(5, 8) FLN_PAIR(7, 8) FLN_PAIR(3, 16) FLN_PAIR(5, 4)
  FLN_PAIR(7, 4) FLN_PAIR(3, 4)
#undef FLN_PAIR
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

int bwd_pipe_pair_any(int kind, int dtype, const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (P.pair) {
    FLN_BY_TYPE(bwd_pipe_pair)
  }
  return FLN_PIPE_NOT_APPLICABLE;
}
#undef FLN_BY_TYPE

}  // namespace fln
