// Pipelined forward with fp8-e4m3 output: instantiations and dispatch.  Serves 16-bit inputs
// whose rows divide exactly into 16-byte vectors, a power-of-two number of threads and 3 or 4
// vectors per thread, once the problem is large enough for the persistent kernel; everything
// else stays with the register-resident kernels of fln_fp8.cu.
#include "fln_pipeline_fwd_kernel.cuh"

namespace fln {

template <typename TI, int KIND, int KK, int QM>
static int fwd_pipe_fp8_k(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
#define FLN_GO(LTT)                                                                                \
  if (P.g.tpr == (1 << LTT)) {                                                                     \
    auto kern = norm_fwd_pipe_kernel<TI, TI, KK, KIND, FLN_ACT_NONE, 1, 16, LTT, QM>;              \
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                                   \
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                                               \
    FLN_CHECK_LAUNCH();                                                                            \
    return FLN_OK;                                                                                 \
  }
  FLN_GO(5) FLN_GO(6) FLN_GO(7) FLN_GO(8) FLN_GO(9)
#undef FLN_GO
  return FLN_PIPE_NOT_APPLICABLE;
}

template <typename TI, int QM>
static int fwd_pipe_fp8_typed(int kind, const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (kind == FLN_LAYERNORM) {
    if (P.K == 4) return fwd_pipe_fp8_k<TI, FLN_LAYERNORM, 4, QM>(p, P, st);
    if (P.K == 3) return fwd_pipe_fp8_k<TI, FLN_LAYERNORM, 3, QM>(p, P, st);
  } else {
    if (P.K == 4) return fwd_pipe_fp8_k<TI, FLN_RMSNORM, 4, QM>(p, P, st);
    if (P.K == 3) return fwd_pipe_fp8_k<TI, FLN_RMSNORM, 3, QM>(p, P, st);
  }
  return FLN_PIPE_NOT_APPLICABLE;
}

// the plans this file has instantiations for
static bool fp8_plan_ok(const PipePlan& P, int64_t rows) {
  return pipeline_wanted(P, rows) && P.full && P.vb == 16 && (P.K == 3 || P.K == 4) &&
         P.threads == (P.g.tpr > 256 ? P.g.tpr : 256);
}

int64_t fwd_fp8_pipeline_odd_rows(int64_t rows, int cols, int tensors) {
  if (rows < 32 || rows % 16 == 0) return 0;
  const int64_t main16 = rows - rows % 16;  // every plan's rows per CTA divide 16
  const PipePlan M = plan_pipeline(false, main16, cols, 2, tensors, false, false);
  if (!fp8_plan_ok(M, main16) || M.g.R <= 1) return 0;
  const PipePlan P = plan_pipeline(false, rows, cols, 2, tensors, false, false);
  if (fp8_plan_ok(P, rows)) return 0;
  return rows % M.g.R;
}

int launch_fwd_pipeline_fp8(int kind, int io_dtype, int qm, const FwdParams& p0, cudaStream_t st) {
  if (io_dtype != FLN_BF16 && io_dtype != FLN_F16) return FLN_PIPE_NOT_APPLICABLE;
  if (qm < 1 || qm > 4) return FLN_PIPE_NOT_APPLICABLE;
  // at most 32 elements per thread (gamma / beta in registers), no ragged last vector
  PipePlan P = plan_pipeline(false, p0.rows, p0.cols, 2, p0.res != nullptr ? 2 : 1, false, false);
  if (!fp8_plan_ok(P, p0.rows)) return FLN_PIPE_NOT_APPLICABLE;
  if ((qm == 3 && p0.cols % 32 != 0) || (qm == 4 && p0.cols % 16 != 0)) return FLN_PIPE_NOT_APPLICABLE;
  FwdParams p = p0;
  p.nv = p.cols / 8;
  if (!fwd_pipe_prepare(&p)) return FLN_ERR_LAUNCH;
#define FLN_Q(QMM)                                                                             \
  if (qm == QMM) {                                                                             \
    if (io_dtype == FLN_BF16) return fwd_pipe_fp8_typed<__nv_bfloat16, QMM>(kind, p, P, st);   \
    return fwd_pipe_fp8_typed<__half, QMM>(kind, p, P, st);                                    \
  }
  FLN_Q(1) FLN_Q(2) FLN_Q(3) FLN_Q(4)
#undef FLN_Q
  return FLN_PIPE_NOT_APPLICABLE;
}

}  // namespace fln
