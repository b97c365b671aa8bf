// Ragged-last-vector backward, fp16 rows.
#include "fln_pipeline_bwd_tail.cuh"

namespace fln {

int bwd_pipe_tail_f16(int kind, const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  return bwd_tail_typed<__half>(kind, p, P, st);
}

}  // namespace fln
