// Pipelined backward for rows whose last vector is ragged (plan_pipeline's `tail` plans): the
// instantiations of one element type.  Included by one translation unit per type so that they
// compile side by side.
//
// Every thread of a row owns K vectors of which the first K - 1 are whole and only the last is
// tested; rows fill the 512-thread CTA.  Columns per thread stay within what the one-pass
// kernel holds in registers (the row as floats, gamma and two accumulators per column):
//   fp32    16-byte vectors x 3, 4 and 8-byte vectors x 5, 7   (10 .. 16 columns)
//   16-bit  8-byte vectors x 3, 4, 5 and 4-byte vectors x 7    (12 .. 20 columns),
//           16-byte vectors x 3 with the dbeta accumulators in shared memory (24 columns)
// With the column sums reduced by the kernel's own tail (cooperative launch) or left to a
// second launch.  Longer ragged rows are shared by the two CTAs of a cluster, each half row
// planned the same way (fp32 9216, 11008, 13824 columns; 16-bit 18432).
#pragma once
#include "fln_pipeline_bwd_kernel.cuh"

namespace fln {

template <typename T, int KIND, int KK, int VB>
static int bwd_tail_go(const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  const bool fuse = p.sync != nullptr;
  // with an incoming gradient of the residual stream: the form with the column sums in the
  // kernel's tail only (a caller that sums the partial rows itself runs the register kernels)
  if (p.dres_in != nullptr) {
    if (!fuse) return FLN_PIPE_NOT_APPLICABLE;
#define FLN_TAIL_LT(L) \
  if (P.g.tpr == (1 << L)) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, true, true, VB, L, false, true>, p, P, st);
    FLN_TAIL_LT(6) FLN_TAIL_LT(7) FLN_TAIL_LT(8) FLN_TAIL_LT(9)
#undef FLN_TAIL_LT
    return FLN_PIPE_NOT_APPLICABLE;
  }
#define FLN_TAIL_LT(L)                                                                                                      \
  if (P.g.tpr == (1 << L)) {                                                                                                \
    if (fuse) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, true, false, VB, L, false, true>, p, P, st); \
    return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, false, false, VB, L, false, true>, p, P, st);          \
  }
  FLN_TAIL_LT(6) FLN_TAIL_LT(7) FLN_TAIL_LT(8) FLN_TAIL_LT(9)
#undef FLN_TAIL_LT
  return FLN_PIPE_NOT_APPLICABLE;
}

// 16-bit rows with three 16-byte vectors per thread (24 columns, up to 256 threads per row):
// LayerNorm keeps its dbeta accumulators in shared memory (`bsm` plans), RMSNorm has none
template <typename T, int KIND>
static int bwd_tail_24_go(const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  if constexpr (sizeof(T) == 2) {
    const bool fuse = p.sync != nullptr;
    if (KIND == FLN_LAYERNORM && !P.bsm) return FLN_PIPE_NOT_APPLICABLE;
    constexpr bool BSM = KIND == FLN_LAYERNORM;
#define FLN_TAIL_LT(L)                                                                                                        \
  if (P.g.tpr == (1 << L)) {                                                                                                  \
    if (fuse) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, 3, KIND, true, true, false, 16, L, false, true, BSM>, p, P, st); \
    return launch_bwd_kernel(norm_bwd_pipe_kernel<T, 3, KIND, true, false, false, 16, L, false, true, BSM>, p, P, st);        \
  }
    FLN_TAIL_LT(6) FLN_TAIL_LT(7) FLN_TAIL_LT(8)
#undef FLN_TAIL_LT
  }
  return FLN_PIPE_NOT_APPLICABLE;
}

// a ragged row shared by the two CTAs of a cluster: each half row on 512 threads
template <typename T, int KIND, int KK, int VB>
static int bwd_tail_pair_go(const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (P.g.tpr != 512 || p.sync != nullptr) return FLN_PIPE_NOT_APPLICABLE;
  return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, true, false, false, VB, 9, true, true>, p, P, st);
}

template <typename T, int KIND>
static int bwd_tail_kind(const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (!P.tail || P.threads != 512 || (p.dres_in != nullptr && (P.pair || P.bsm))) return FLN_PIPE_NOT_APPLICABLE;
#define FLN_TAIL(KK, VBB)         \
  if (P.K == KK && P.vb == VBB) { \
    if (P.pair) return bwd_tail_pair_go<T, KIND, KK, VBB>(p, P, st); \
    return bwd_tail_go<T, KIND, KK, VBB>(p, P, st);                  \
  }
  if constexpr (sizeof(T) == 4) {
    FLN_TAIL(4, 16) FLN_TAIL(3, 16) FLN_TAIL(7, 8) FLN_TAIL(5, 8)
  } else {
    if (P.K == 3 && P.vb == 16 && !P.pair) return p.dres_in != nullptr ? FLN_PIPE_NOT_APPLICABLE : bwd_tail_24_go<T, KIND>(p, P, st);
    FLN_TAIL(5, 8) FLN_TAIL(4, 8) FLN_TAIL(3, 8) FLN_TAIL(7, 4)
  }
#undef FLN_TAIL
  return FLN_PIPE_NOT_APPLICABLE;
}

template <typename T>
static int bwd_tail_typed(int kind, const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  return kind == FLN_LAYERNORM ? bwd_tail_kind<T, FLN_LAYERNORM>(p, P, st) : bwd_tail_kind<T, FLN_RMSNORM>(p, P, st);
}

int bwd_pipe_tail_f32(int kind, const BwdParams& p, const PipePlan& P, cudaStream_t st);
int bwd_pipe_tail_bf16(int kind, const BwdParams& p, const PipePlan& P, cudaStream_t st);
int bwd_pipe_tail_f16(int kind, const BwdParams& p, const PipePlan& P, cudaStream_t st);

}  // namespace fln
