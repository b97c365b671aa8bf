// Pipelined backward: entry point, and the instantiations with 16-byte vectors, a power-of-two
// number per thread.  The kernel itself is in fln_pipeline_bwd_kernel.cuh.
#include "fln_pipeline_bwd_kernel.cuh"

namespace fln {

// 16-byte vectors, K a power of two; LT >= 0 selects the compile-time geometry
template <typename T, int KIND, int KK, bool FF, int LT>
static int bwd_pipe_pow2(const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  const bool fuse = p.sync != nullptr, dr = p.dres_in != nullptr;
  if (fuse && dr) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, FF, true, true, 16, LT>, p, P, st);
  if (fuse) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, FF, true, false, 16, LT>, p, P, st);
  if (dr) return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, FF, false, true, 16, LT>, p, P, st);
  return launch_bwd_kernel(norm_bwd_pipe_kernel<T, KK, KIND, FF, false, false, 16, LT>, p, P, st);
}

template <typename T, int KIND>
static int bwd_pipe_k(const BwdParams& p, const PipePlan& P, cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(T);
#define FLN_CASE(KK)                                                                                   \
  case KK:                                                                                             \
    if constexpr (VEC * KK <= 16) {                                                                    \
      /* the planner's preferred split (16 columns per thread) with whole rows in the 512-thread CTA: */ \
      /* geometry as template arguments */                                                             \
      if constexpr (VEC * KK == 16) {                                                                  \
        if (P.full && P.threads == 512 && P.g.tpr == 512) return bwd_pipe_pow2<T, KIND, KK, true, 9>(p, P, st); \
        if (P.full && P.threads == 512 && P.g.tpr == 256) return bwd_pipe_pow2<T, KIND, KK, true, 8>(p, P, st); \
        if (P.full && P.threads == 512 && P.g.tpr == 128) return bwd_pipe_pow2<T, KIND, KK, true, 7>(p, P, st); \
        if (P.full && P.threads == 512 && P.g.tpr == 64) return bwd_pipe_pow2<T, KIND, KK, true, 6>(p, P, st);  \
      }                                                                                                \
      if (P.full) return bwd_pipe_pow2<T, KIND, KK, true, -1>(p, P, st);                               \
      return bwd_pipe_pow2<T, KIND, KK, false, -1>(p, P, st);                                          \
    }                                                                                                  \
    return FLN_PIPE_NOT_APPLICABLE;
  switch (P.K) {
    FLN_CASE(1) FLN_CASE(2) FLN_CASE(4)
    default:
      return FLN_PIPE_NOT_APPLICABLE;
  }
#undef FLN_CASE
}

static bool cooperative_launch_supported() {
  static int cache[64];  // 0 unknown, 1 no, 2 yes
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  if (cache[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess) {
      cudaGetLastError();
      v = 0;
    }
    cache[dev] = v ? 2 : 1;
  }
  return cache[dev] == 2;
}

static unsigned long long next_launch_token() {
  static std::atomic<unsigned long long> ctr{0x5bd1e995ull};
  unsigned long long t;
  do {
    t = ctr.fetch_add(1, std::memory_order_relaxed) & ((1ull << 40) - 1);
  } while (t == 0);
  return t;
}

int launch_bwd_pipeline(int kind, int dtype, const BwdParams& p0, cudaStream_t st, bool* reduced) {
  const int es = dtype == FLN_F32 ? 4 : 2;
  *reduced = false;
  PipePlan P = plan_bwd_pipeline(p0.rows, p0.cols, es, p0.dres_in != nullptr);
  if (!pipeline_wanted(P, p0.rows)) return FLN_PIPE_NOT_APPLICABLE;
  BwdParams p = p0;
  p.nv = p.cols / (P.vb / es);
  DeviceWords w;
  if (!device_words(&w)) return FLN_ERR_LAUNCH;
  p.wait_ns = wait_limit_ns();
  p.status = w.status;
  p.fault = w.fault;
  // Fused column reduce: one CTA per SM (so the whole grid is resident at once), the
  // one-row kernel, stage memory large enough for the 16 x 128 floats of the combine step.
  const bool fuse = !P.pair && !P.wide && p.sync != nullptr && p.partials != nullptr && P.grid <= usable_sms() &&
                    P.grid < 4096 && P.smem >= (size_t)kSmemHeader + 16 * 128 * sizeof(float) &&
                    path_override() != 3 && cooperative_launch_supported();
  if (fuse) {
    p.token = next_launch_token();
    *reduced = true;
  } else {
    p.sync = nullptr;
  }
  // plans served by the other translation units
  const bool shared_row = P.pair;
  const bool odd = P.vb != 16 || P.K == 3 || P.K == 5 || P.K == 7;
#define FLN_RUN(T)                                                                          \
  (P.wide ? bwd_pipe_wide_any(kind, dtype, p, P, st) :                                      \
   P.tail ? bwd_pipe_tail_any(kind, dtype, p, P, st) :                                      \
   shared_row ? bwd_pipe_pair_any(kind, dtype, p, P, st)                                    \
              : (odd ? bwd_pipe_odd_any(kind, dtype, p, P, st)                              \
                     : (kind == FLN_LAYERNORM ? bwd_pipe_k<T, FLN_LAYERNORM>(p, P, st)      \
                                              : bwd_pipe_k<T, FLN_RMSNORM>(p, P, st))))
  int rc = dtype == FLN_F32 ? FLN_RUN(float) : (dtype == FLN_BF16 ? FLN_RUN(__nv_bfloat16) : FLN_RUN(__half));
  if (rc == FLN_ERR_LAUNCH && fuse) {
    // the cooperative launch was refused (the device is shared in a way that rules out a
    // resident grid): run the plain launch and let the caller reduce the partial rows
    p.sync = nullptr;
    *reduced = false;
    rc = dtype == FLN_F32 ? FLN_RUN(float) : (dtype == FLN_BF16 ? FLN_RUN(__nv_bfloat16) : FLN_RUN(__half));
  }
  return rc;
#undef FLN_RUN
}

}  // namespace fln
