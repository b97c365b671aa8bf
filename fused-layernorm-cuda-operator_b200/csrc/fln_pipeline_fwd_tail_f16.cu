// Ragged-last-vector forward, fp16 rows.
#include "fln_pipeline_fwd_tail.cuh"

namespace fln {

int fwd_pipe_tail_f16(int kind, const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  return fwd_tail_typed<__half>(kind, p, P, st);
}

}  // namespace fln
