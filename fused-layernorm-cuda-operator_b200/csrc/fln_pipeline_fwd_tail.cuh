// Pipelined forward for rows whose last vector is ragged (plan_pipeline's `tail` plans): the
// instantiations of one element type, one per (vectors per thread, bytes per vector, threads
// per row).  Included by one translation unit per type so that they compile side by side.
//
// A row of 4608 = 9 * 512 or 1600 = 25 * 64 columns divides into no power-of-two number of
// threads times a vector count the exact kernels have.  These plans give every thread K vectors
// of which the first K - 1 are whole for every thread of the row and only the last one is
// tested, so the kernel is branch-free up to that vector and at most 1 / K of the lanes idle in
// it.  Plain forward only (no activation, output in the input's type).
//   fp32    16-byte vectors x 3 .. 8 (12 .. 32 elements per thread)
//   16-bit  16-byte vectors x 5 .. 7 with gamma / beta in shared memory (40 .. 56 elements),
//           16-byte vectors x 3, 4 and 8-byte vectors x 7 with them in registers; rows of 512
//           threads x 4 vectors with them fetched per row, two CTAs per SM
#pragma once
#include "fln_pipeline_fwd_kernel.cuh"

namespace fln {

template <typename T, int KIND, int KK, int MODE, int VB>
static int fwd_tail_go(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
#define FLN_GO(LTT)                                                                \
  if (P.g.tpr == (1 << LTT)) {                                                     \
    auto kern = norm_fwd_pipe_kernel<T, T, KK, KIND, FLN_ACT_NONE, MODE, VB, LTT>; \
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                   \
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                               \
    FLN_CHECK_LAUNCH();                                                            \
    return FLN_OK;                                                                 \
  }
  FLN_GO(5) FLN_GO(6) FLN_GO(7) FLN_GO(8) FLN_GO(9)
#undef FLN_GO
  return FLN_PIPE_NOT_APPLICABLE;
}

template <typename T, int KIND>
static int fwd_tail_kind(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  const int nt = P.g.tpr > 256 ? P.g.tpr : 256;
  if (!P.tail || P.threads != nt) return FLN_PIPE_NOT_APPLICABLE;
  // 16-bit rows of 512 threads, two CTAs per SM, gamma / beta fetched per row (`pgl` plans)
  if (P.pgl) {
    if constexpr (sizeof(T) == 2) {
      if (P.K == 4 && P.vb == 16 && P.g.tpr == 512) {
        auto kern = norm_fwd_pipe_kernel<T, T, 4, KIND, FLN_ACT_NONE, 8, 16, 9>;
        if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;
        kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);
        FLN_CHECK_LAUNCH();
        return FLN_OK;
      }
    }
    return FLN_PIPE_NOT_APPLICABLE;
  }
#define FLN_TAIL(KK, VBB, MODE) \
  if (P.K == KK && P.vb == VBB) return fwd_tail_go<T, KIND, KK, MODE, VBB>(p, P, st);
  if constexpr (sizeof(T) == 4) {
    FLN_TAIL(3, 16, 5) FLN_TAIL(4, 16, 5) FLN_TAIL(5, 16, 5) FLN_TAIL(6, 16, 5) FLN_TAIL(7, 16, 5) FLN_TAIL(8, 16, 5)
  } else {
    FLN_TAIL(5, 16, 7) FLN_TAIL(6, 16, 7) FLN_TAIL(7, 16, 7)
    FLN_TAIL(3, 16, 5) FLN_TAIL(4, 16, 5) FLN_TAIL(7, 8, 5)
  }
#undef FLN_TAIL
  return FLN_PIPE_NOT_APPLICABLE;
}

template <typename T>
static int fwd_tail_typed(int kind, const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  return kind == FLN_LAYERNORM ? fwd_tail_kind<T, FLN_LAYERNORM>(p, P, st) : fwd_tail_kind<T, FLN_RMSNORM>(p, P, st);
}

int fwd_pipe_tail_f32(int kind, const FwdParams& p, const PipePlan& P, cudaStream_t st);
int fwd_pipe_tail_bf16(int kind, const FwdParams& p, const PipePlan& P, cudaStream_t st);
int fwd_pipe_tail_f16(int kind, const FwdParams& p, const PipePlan& P, cudaStream_t st);

}  // namespace fln
