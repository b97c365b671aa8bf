// Ragged-last-vector forward, bf16 rows.
#include "fln_pipeline_fwd_tail.cuh"

namespace fln {

int fwd_pipe_tail_bf16(int kind, const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  return fwd_tail_typed<__nv_bfloat16>(kind, p, P, st);
}

}  // namespace fln
