// Ragged-last-vector backward, fp32 rows, and the dispatch by type.
#include "fln_pipeline_bwd_tail.cuh"

namespace fln {

int bwd_pipe_tail_f32(int kind, const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  return bwd_tail_typed<float>(kind, p, P, st);
}

int bwd_pipe_tail_any(int kind, int dtype, const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (dtype == FLN_F32) return bwd_pipe_tail_f32(kind, p, P, st);
  if (dtype == FLN_BF16) return bwd_pipe_tail_bf16(kind, p, P, st);
  if (dtype == FLN_F16) return bwd_pipe_tail_f16(kind, p, P, st);
  return FLN_PIPE_NOT_APPLICABLE;
}

}  // namespace fln
