// Pipelined forward with dropout in front of the residual add: instantiations and dispatch.
// Serves 16-bit inputs whose rows divide exactly into 16-byte vectors, a power-of-two number of
// threads and 3 or 4 vectors per thread, once the problem is large enough for the persistent
// kernel; everything else stays with the one-CTA-per-row kernel of fln_dropout.cu.
#include "fln_pipeline_fwd_kernel.cuh"

namespace fln {

template <typename TI, int KIND, int KK>
static int fwd_pipe_drop_k(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
#define FLN_GO(LTT)                                                                                \
  if (P.g.tpr == (1 << LTT)) {                                                                     \
    auto kern = norm_fwd_pipe_kernel<TI, TI, KK, KIND, FLN_ACT_NONE, 1, 16, LTT, 0, true>;         \
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                                   \
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                                               \
    FLN_CHECK_LAUNCH();                                                                            \
    return FLN_OK;                                                                                 \
  }
  FLN_GO(5) FLN_GO(6) FLN_GO(7) FLN_GO(8) FLN_GO(9)
#undef FLN_GO
  return FLN_PIPE_NOT_APPLICABLE;
}

template <typename TI>
static int fwd_pipe_drop_typed(int kind, const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (kind == FLN_LAYERNORM) {
    if (P.K == 4) return fwd_pipe_drop_k<TI, FLN_LAYERNORM, 4>(p, P, st);
    if (P.K == 3) return fwd_pipe_drop_k<TI, FLN_LAYERNORM, 3>(p, P, st);
  } else {
    if (P.K == 4) return fwd_pipe_drop_k<TI, FLN_RMSNORM, 4>(p, P, st);
    if (P.K == 3) return fwd_pipe_drop_k<TI, FLN_RMSNORM, 3>(p, P, st);
  }
  return FLN_PIPE_NOT_APPLICABLE;
}

int launch_fwd_pipeline_dropout(int kind, int io_dtype, const FwdParams& p0, cudaStream_t st) {
  if (io_dtype != FLN_BF16 && io_dtype != FLN_F16) return FLN_PIPE_NOT_APPLICABLE;
  // at most 32 elements per thread (gamma / beta in registers), no ragged last vector
  PipePlan P = plan_pipeline(false, p0.rows, p0.cols, 2, p0.res != nullptr ? 2 : 1, false, false);
  if (!pipeline_wanted(P, p0.rows) || !P.full || P.vb != 16 || (P.K != 3 && P.K != 4)) return FLN_PIPE_NOT_APPLICABLE;
  if (P.threads != (P.g.tpr > 256 ? P.g.tpr : 256)) return FLN_PIPE_NOT_APPLICABLE;
  FwdParams p = p0;
  p.nv = p.cols / 8;
  if (!fwd_pipe_prepare(&p)) return FLN_ERR_LAUNCH;
  if (io_dtype == FLN_BF16) return fwd_pipe_drop_typed<__nv_bfloat16>(kind, p, P, st);
  return fwd_pipe_drop_typed<__half>(kind, p, P, st);
}

}  // namespace fln
