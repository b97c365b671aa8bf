// Pipelined forward: dispatch and entry point.  The kernel is in fln_pipeline_fwd_kernel.cuh.
#include "fln_pipeline_fwd_kernel.cuh"

namespace fln {

// one branch-free instantiation with an odd K and / or short vectors; combinations that make no
// sense for the type (too many elements per thread, vectors shorter than four elements) are
// not instantiated
template <typename TI, typename TO, int KIND, int ACT, int KK, int VB>
static int fwd_pipe_odd(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  constexpr int VEC = VB / (int)sizeof(TI);
  constexpr int MODE =
      (VEC >= 4 && KK * VEC > 32 && KK * VEC <= 48 && sizeof(TI) == 2) ? 4 : ((VEC >= 4 && KK * VEC <= 32) ? 1 : -1);
  if constexpr (MODE > 0) {
#define FLN_GO(LTT)                                                             \
  {                                                                             \
    auto kern = norm_fwd_pipe_kernel<TI, TO, KK, KIND, ACT, MODE, VB, LTT>;     \
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                \
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                            \
    FLN_CHECK_LAUNCH();                                                         \
    return FLN_OK;                                                              \
  }
    // geometry as template arguments for the plain forward (no GELU, same type out as in)
    if constexpr (ACT == FLN_ACT_NONE && std::is_same<TI, TO>::value) {
      const int nt = P.g.tpr > 256 ? P.g.tpr : 256;
      if (P.threads == nt) {
        if (P.g.tpr == 16) FLN_GO(4)
        if (P.g.tpr == 32) FLN_GO(5)
        if (P.g.tpr == 64) FLN_GO(6)
        if (P.g.tpr == 128) FLN_GO(7)
        if (P.g.tpr == 256) FLN_GO(8)
        if (P.g.tpr == 512) FLN_GO(9)
      }
    }
    FLN_GO(-1)
#undef FLN_GO
  } else {
    return FLN_PIPE_NOT_APPLICABLE;
  }
}

// rows whose last vector is ragged (plan_pipeline's `tail` plans): instantiated in
// fln_pipeline_fwd_tail.cu; plain forward only
template <typename TI, typename TO, int KIND, int ACT>
static int fwd_pipe_tail(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  if constexpr (ACT == FLN_ACT_NONE && std::is_same<TI, TO>::value) {
    constexpr int dtype = std::is_same<TI, float>::value ? FLN_F32 : (std::is_same<TI, __half>::value ? FLN_F16 : FLN_BF16);
    return fwd_pipe_tail_any(KIND, dtype, p, P, st);
  }
  return FLN_PIPE_NOT_APPLICABLE;
}

// rows of 512 threads with two CTAs per SM (plan_pipeline's `pgl` plans): 4 vectors of 16 bytes
// per thread in 16-bit types, gamma / beta fetched per row; plain forward only
template <typename TI, typename TO, int KIND, int ACT>
static int fwd_pipe_pgl(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  if constexpr (ACT == FLN_ACT_NONE && std::is_same<TI, TO>::value) {
    if (P.vb != 16 || P.threads != 512 || P.g.tpr != 512) return FLN_PIPE_NOT_APPLICABLE;
#define FLN_GO(KK)                                                                                  \
  if (P.K == KK) {                                                                                  \
    if constexpr (sizeof(TI) == 2) {                                                                \
      auto kern = norm_fwd_pipe_kernel<TI, TO, KK, KIND, ACT, 6, 16, 9>;                            \
      if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                                  \
      kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                                              \
      FLN_CHECK_LAUNCH();                                                                           \
      return FLN_OK;                                                                                \
    }                                                                                               \
  }
    FLN_GO(4)
#undef FLN_GO
  }
  return FLN_PIPE_NOT_APPLICABLE;
}

template <typename TI, typename TO, int KIND, int ACT>
static int fwd_pipe_k(const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (P.tail) return fwd_pipe_tail<TI, TO, KIND, ACT>(p, P, st);
  if (P.pgl) return fwd_pipe_pgl<TI, TO, KIND, ACT>(p, P, st);
  if (P.vb != 16 || P.K == 3 || P.K == 5 || P.K == 6 || P.K == 7) {
    if (!P.full) return FLN_PIPE_NOT_APPLICABLE;
#define FLN_ODD(KK, VBB) \
  if (P.K == KK && P.vb == VBB) return fwd_pipe_odd<TI, TO, KIND, ACT, KK, VBB>(p, P, st);
    FLN_ODD(3, 16) FLN_ODD(5, 16) FLN_ODD(6, 16) FLN_ODD(7, 16) FLN_ODD(3, 8) FLN_ODD(5, 8) FLN_ODD(7, 8)
#undef FLN_ODD
    return FLN_PIPE_NOT_APPLICABLE;
  }
#define FLN_LAUNCH(KK, FF)                                                                   \
  {                                                                                          \
    auto kern = norm_fwd_pipe_kernel<TI, TO, KK, KIND, ACT, FF>;                             \
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                             \
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                                         \
  }
#define FLN_LAUNCH_CT(KK, LTT)                                                               \
  {                                                                                          \
    auto kern = norm_fwd_pipe_kernel<TI, TO, KK, KIND, ACT, 1, 16, LTT>;                     \
    if (set_smem(kern, P.smem) != FLN_OK) return FLN_ERR_LAUNCH;                             \
    kern<<<P.grid, P.threads, P.smem, st>>>(p, P.g);                                         \
  }
  // the planner's preferred split (64 bytes per thread) with whole rows in a 256-thread CTA:
  // geometry as template arguments
#define FLN_CASE(KK)                                                \
  case KK:                                                          \
    if constexpr (KK == 4) {                                        \
      if (P.full && P.threads == 256 && P.g.tpr == 256) FLN_LAUNCH_CT(KK, 8)      \
      else if (P.full && P.threads == 256 && P.g.tpr == 128) FLN_LAUNCH_CT(KK, 7) \
      else if (P.full && P.threads == 256 && P.g.tpr == 64) FLN_LAUNCH_CT(KK, 6)  \
      else if (P.full && P.threads == 256 && P.g.tpr == 32) FLN_LAUNCH_CT(KK, 5)  \
      else if (P.full && P.threads == 512 && P.g.tpr == 512) FLN_LAUNCH_CT(KK, 9) \
      else if (P.full) FLN_LAUNCH(KK, 1)                            \
      else FLN_LAUNCH(KK, 0)                                        \
    } else if constexpr (KK * 16 / sizeof(TI) <= 32) {              \
      if (P.full) FLN_LAUNCH(KK, 1)                                 \
      else FLN_LAUNCH(KK, 0)                                        \
    } else {                                                        \
      return FLN_PIPE_NOT_APPLICABLE;                               \
    }                                                               \
    break;
  switch (P.K) {
    FLN_CASE(1) FLN_CASE(2) FLN_CASE(4) FLN_CASE(8)
    default:
      return FLN_PIPE_NOT_APPLICABLE;
  }
#undef FLN_CASE
#undef FLN_LAUNCH
#undef FLN_LAUNCH_CT
  FLN_CHECK_LAUNCH();
  return FLN_OK;
}

template <typename TI, typename TO>
static int fwd_pipe_typed(int kind, int act, const FwdParams& p, const PipePlan& P, cudaStream_t st) {
  if (kind == FLN_RMSNORM) return fwd_pipe_k<TI, TO, FLN_RMSNORM, FLN_ACT_NONE>(p, P, st);
  switch (act) {
    case FLN_ACT_NONE:
      return fwd_pipe_k<TI, TO, FLN_LAYERNORM, FLN_ACT_NONE>(p, P, st);
    case FLN_ACT_GELU_TANH:
      return fwd_pipe_k<TI, TO, FLN_LAYERNORM, FLN_ACT_GELU_TANH>(p, P, st);
    case FLN_ACT_GELU_ERF:
      return fwd_pipe_k<TI, TO, FLN_LAYERNORM, FLN_ACT_GELU_ERF>(p, P, st);
  }
  return FLN_PIPE_NOT_APPLICABLE;
}

bool fwd_pipe_prepare(FwdParams* p) {
  DeviceWords w;
  if (!device_words(&w)) return false;
  p->sched = w.sched + 2 * next_sched_slot();
  p->wait_ns = wait_limit_ns();
  p->status = w.status;
  p->fault = w.fault;
  return true;
}

int64_t fwd_pipeline_odd_rows(int act, int io_dtype, int out_dtype, const FwdParams& p0) {
  const bool allow_tail = act == FLN_ACT_NONE && io_dtype == out_dtype;
  return fwd_plan_odd_rows(p0.rows, p0.cols, io_dtype == FLN_F32 ? 4 : 2, p0.res != nullptr ? 2 : 1, allow_tail);
}

int launch_fwd_pipeline(int kind, int act, int io_dtype, int out_dtype, const FwdParams& p0,
                        cudaStream_t st) {
  const int es = io_dtype == FLN_F32 ? 4 : 2;
  // the ragged-last-vector plans exist for the plain forward only
  const bool allow_tail = act == FLN_ACT_NONE && io_dtype == out_dtype;
  PipePlan P = plan_pipeline(false, p0.rows, p0.cols, es, p0.res != nullptr ? 2 : 1, true, allow_tail);
  if (!pipeline_wanted(P, p0.rows)) return FLN_PIPE_NOT_APPLICABLE;
  // Measured exceptions (automatic selection only): fp32 rows that the non-persistent
  // register-resident kernel holds exactly stream faster there than through the ring -- a plain
  // RMSNorm forward at every row length tried, the LayerNorm forward up to 4096 columns, where
  // the ring runs 16 elements per thread (1024 / 2048 / 4096: 6743 / 6753 / 6658 vs 5651 / 5797 /
  // 5504 GB/s; from 24 elements per thread the ring wins, 8192: 6651 vs 5497).  In 16-bit types
  // the ring with its tiles handed out on demand is the faster one (RMSNorm 16384 x 8192 bf16:
  // 84.1 vs 86.4 us).
  if (path_override() == 0 && p0.res == nullptr && act == FLN_ACT_NONE &&
      io_dtype == out_dtype) {
    const Plan rp = make_plan(false, p0.rows, p0.cols, es, true);
    const bool exact = !rp.generic && rp.vec == 16 / es && (int64_t)rp.K * rp.tpr * rp.vec == p0.cols;
    // (padded register plans of long rows excepted -- 6144 columns: 6188 vs 6707 GB/s)
    if (kind == FLN_RMSNORM && !rp.generic && rp.vec == 16 / es && es == 4 && (exact || p0.cols <= 4096))
      return FLN_PIPE_NOT_APPLICABLE;
    if (kind == FLN_LAYERNORM && es == 4 && exact && p0.cols <= 4096) return FLN_PIPE_NOT_APPLICABLE;
  }
  FwdParams p = p0;
  p.nv = p.cols / (P.vb / es);
  if (!fwd_pipe_prepare(&p)) return FLN_ERR_LAUNCH;
  if (io_dtype == FLN_F32 && out_dtype == FLN_F32) return fwd_pipe_typed<float, float>(kind, act, p, P, st);
  if (io_dtype == FLN_F32 && out_dtype == FLN_BF16) return fwd_pipe_typed<float, __nv_bfloat16>(kind, act, p, P, st);
  if (io_dtype == FLN_BF16) return fwd_pipe_typed<__nv_bfloat16, __nv_bfloat16>(kind, act, p, P, st);
  return fwd_pipe_typed<__half, __half>(kind, act, p, P, st);
}

}  // namespace fln
