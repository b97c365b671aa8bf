// Host-side parts of libfln_b200: launch planning, CUDA-graph record/replay, and the
// advisory helpers that mirror the reference's host utilities
// (csrc/layernorm_cuda.cpp:144-195, 230-237).
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <new>
#include <string>

#include "fln_common.cuh"

namespace fln {

static std::atomic<int> g_force_k{0};
static std::atomic<int> g_force_tpr{0};

int sm_count() {
  static std::atomic<int> cache[16];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 0 || dev >= 16) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 148;
  }
  int v = cache[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 148;  // B200; also what a planning query without a device reports
    }
    cache[dev].store(n, std::memory_order_relaxed);
    v = n;
  }
  return v;
}

static std::atomic<int> g_sm_reserve{0};

int usable_sms() {
  const int n = sm_count() - g_sm_reserve.load(std::memory_order_relaxed);
  return n > 1 ? n : 1;
}

void plan_override(int* K, int* tpr) {
  *K = g_force_k.load(std::memory_order_relaxed);
  *tpr = g_force_tpr.load(std::memory_order_relaxed);
}

static int next_pow2(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}
static int ilog2(int v) {
  int l = 0;
  while ((1 << l) < v) ++l;
  return l;
}

// Threads a kernel instantiation with K vectors of `vec` elements per thread may be
// launched with (mirrors the __launch_bounds__ of the kernels).
static int max_threads(bool backward, int vec, int K) {
  if (backward) return vec * K <= 4 ? 1024 : (vec * K <= 16 ? 512 : 256);
  return K <= 2 ? 1024 : 512;
}
static bool k_allowed(bool backward, int vec, int K) {
  if (K != 1 && K != 2 && K != 4 && K != 8) return false;
  if (backward && vec * K > 32) return false;
  return true;
}

Plan make_plan(bool backward, int64_t rows, int cols, int elem_bytes, bool aligned16) {
  Plan pl;
  memset(&pl, 0, sizeof(pl));
  const int full = 16 / elem_bytes;
  pl.vec = (aligned16 && cols % full == 0) ? full : 1;
  const int nv = cols / pl.vec;

  // Preferred vectors per thread.  Forward: 64 B of the row per thread.  Backward: about
  // 16 columns per thread, because each column also costs two fp32 accumulators.
  int pref = backward ? (16 / pl.vec > 0 ? 16 / pl.vec : 1) : 4;
  if (pref > 8) pref = 8;
  // Latency-bound problems (less than one wave of work): spread the row over more
  // threads so each one has a short dependent chain.
  const int sms = sm_count();
  if ((int64_t)rows * nv <= (int64_t)sms * 1024) pref = pref > 2 ? 2 : pref;

  int fK = 0, ftpr = 0;
  plan_override(&fK, &ftpr);
  int K = 0, tpr = 0;
  if (fK > 0 && ftpr > 0 && k_allowed(backward, pl.vec, fK) && (ftpr & (ftpr - 1)) == 0 &&
      ftpr <= max_threads(backward, pl.vec, fK) && (int64_t)fK * ftpr >= nv) {
    K = fK;
    tpr = ftpr;
  } else {
    // candidates in order of preference: pref, then larger K, then smaller K
    int order[8], n = 0;
    for (int k = pref; k <= 8; k <<= 1) order[n++] = k;
    for (int k = pref >> 1; k >= 1; k >>= 1) order[n++] = k;
    for (int i = 0; i < n && K == 0; ++i) {
      const int k = order[i];
      if (!k_allowed(backward, pl.vec, k)) continue;
      const int t = next_pow2((nv + k - 1) / k);
      if (t > max_threads(backward, pl.vec, k)) continue;
      // do not keep a K whose last vectors would be entirely padding
      int kk = (nv + t - 1) / t;
      kk = next_pow2(kk);
      if (!k_allowed(backward, pl.vec, kk)) continue;
      K = kk;
      tpr = t;
    }
  }
  if (K == 0) {
    pl.generic = 1;
    pl.vec = 1;
    pl.K = 0;
    pl.tpr = 512;
    pl.log2_tpr = 9;
    pl.threads = 512;
    pl.rows_per_cta = 1;
    return pl;
  }
  pl.K = K;
  pl.tpr = tpr;
  pl.log2_tpr = ilog2(tpr);
  // CTA of ~256 threads holding several rows when rows are short; fewer rows per CTA
  // when that would leave SMs idle.
  int threads = tpr > 256 ? tpr : 256;
  int rpc = threads / tpr;
  const int min_threads = tpr > 32 ? tpr : 32;
  while (rpc > 1 && threads / 2 >= min_threads && (rows + rpc - 1) / rpc < 2LL * sms) {
    rpc >>= 1;
    threads >>= 1;
  }
  pl.threads = threads;
  pl.rows_per_cta = threads / tpr;
  return pl;
}

}  // namespace fln

using namespace fln;

extern "C" void fln_set_plan_override(int vecs_per_thread, int threads_per_row) {
  g_force_k.store(vecs_per_thread, std::memory_order_relaxed);
  g_force_tpr.store(threads_per_row, std::memory_order_relaxed);
}

extern "C" void fln_set_sm_reserve(int sms) { g_sm_reserve.store(sms < 0 ? 0 : sms, std::memory_order_relaxed); }

extern "C" const char* fln_status_string(int status) {
  switch (status) {
    case FLN_OK:
      return "ok";
    case FLN_ERR_DTYPE:
      return "unsupported dtype";
    case FLN_ERR_SHAPE:
      return "invalid shape";
    case FLN_ERR_NULL:
      return "required pointer is NULL";
    case FLN_ERR_WORKSPACE:
      return "workspace missing, misaligned or too small";
    case FLN_ERR_LAUNCH:
      return "CUDA launch failed";
    case FLN_ERR_UNSUPPORTED:
      return "unsupported combination of arguments";
    case FLN_ERR_GRAPH:
      return "CUDA graph operation failed";
    case FLN_ERR_ARG:
      return "invalid argument";
    case FLN_ERR_STATIC_SCRATCH:
      return "problem needs more scratch than the built-in static array holds (FLN_STATIC_SCRATCH_BYTES); "
             "use fln_layernorm_backward with a caller-provided workspace";
  }
  return "unknown status";
}

extern "C" const char* fln_version(void) { return "1.0.0"; }
extern "C" int fln_cuda_runtime_version(void) { return CUDART_VERSION; }

extern "C" int64_t fln_get_memory_usage(int batch_size, int hidden_size, int use_mixed_precision) {
  const int64_t b = batch_size, h = hidden_size;
  const int64_t e = use_mixed_precision ? 2 : 4;
  const int64_t fwd = 2 * b * h * e + 2 * b * (int64_t)sizeof(float);  // in/out + mean/rstd
  const int64_t bwd = b * h * e + 2 * h * e;                            // dx + dgamma/dbeta
  const int64_t scratch = b * 32 * (int64_t)sizeof(float);
  return fwd + bwd + scratch;
}

extern "C" int fln_get_performance_hints(int batch_size, int hidden_size, char* buf, size_t buf_len) {
  std::string s;
  if (hidden_size % 32 != 0)
    s += "Warning: hidden_size is not divisible by 32, may impact performance.\n";
  if (hidden_size > 8192)
    s += "Info: Large hidden dimension detected. Consider using mixed precision.\n";
  if (batch_size < 8) s += "Info: Small batch size may not fully utilize GPU.\n";
  if (batch_size < sm_count()) s += "Info: Not enough blocks to saturate GPU. Consider batching.\n";
  if (buf != nullptr && buf_len > 0) {
    size_t n = s.size() < buf_len - 1 ? s.size() : buf_len - 1;
    memcpy(buf, s.data(), n);
    buf[n] = '\0';
  }
  return (int)s.size();
}

extern "C" int fln_describe_launch(int backward, int64_t rows, int64_t cols, int dtype,
                                   int aligned16, fln_launch_info* out) {
  if (out == nullptr) return FLN_ERR_NULL;
  if (rows < 0 || cols <= 0 || cols > 0x7fffffff) return FLN_ERR_SHAPE;
  if (dtype != FLN_F32 && dtype != FLN_BF16 && dtype != FLN_F16) return FLN_ERR_DTYPE;
  const int es = dtype == FLN_F32 ? 4 : 2;
  Plan pl = make_plan(backward != 0, rows, (int)cols, es, aligned16 != 0);
  out->generic = pl.generic;
  out->vec_elems = pl.vec;
  out->vecs_per_thread = pl.K;
  out->threads_per_row = pl.tpr;
  out->threads_per_cta = pl.threads;
  out->rows_per_cta = pl.rows_per_cta;
  out->sm_count = sm_count();
  int64_t groups = (rows + pl.rows_per_cta - 1) / pl.rows_per_cta;
  if (backward && !pl.generic) {
    // the persistent grid is capped by residency; report the workspace-derived figure
    size_t ws = fln_backward_workspace_bytes(rows, cols, dtype);
    int64_t P = (int64_t)(ws / (2 * (size_t)cols * sizeof(float)));
    int64_t g = P / pl.rows_per_cta;
    out->grid = g < groups && g > 0 ? g : groups;
  } else {
    out->grid = groups;
  }
  out->pipelined = 0;
  out->stages = 0;
  out->vector_bytes = pl.vec * es;
  PipeDescription pd;
  if (aligned16 != 0 && rows > 0 && describe_pipeline(backward != 0, rows, (int)cols, es, &pd)) {
    out->generic = 0;
    out->pipelined = 1;
    out->vec_elems = pd.vector_bytes / es;
    out->vecs_per_thread = pd.K;
    out->threads_per_row = pd.tpr;
    out->threads_per_cta = pd.threads;
    out->rows_per_cta = pd.rows_per_cta;
    out->grid = pd.grid;
    out->stages = pd.stages;
    out->vector_bytes = pd.vector_bytes;
  }
  return FLN_OK;
}

// ----------------------------------------------------------------------------------------
// CUDA-graph record / replay
// ----------------------------------------------------------------------------------------
struct fln_graph {
  cudaStream_t cap_stream;
  cudaGraph_t graph;
  cudaGraphExec_t exec;
  int capturing;
};

extern "C" int fln_graph_begin(fln_graph** out) {
  if (out == nullptr) return FLN_ERR_NULL;
  *out = nullptr;
  fln_graph* g = new (std::nothrow) fln_graph;
  if (g == nullptr) return FLN_ERR_GRAPH;
  g->cap_stream = nullptr;
  g->graph = nullptr;
  g->exec = nullptr;
  g->capturing = 0;
  if (cudaStreamCreateWithFlags(&g->cap_stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete g;
    return FLN_ERR_GRAPH;
  }
  if (cudaStreamBeginCapture(g->cap_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
    cudaStreamDestroy(g->cap_stream);
    delete g;
    return FLN_ERR_GRAPH;
  }
  g->capturing = 1;
  *out = g;
  return FLN_OK;
}

extern "C" void* fln_graph_stream(fln_graph* g) { return g ? (void*)g->cap_stream : nullptr; }

extern "C" int fln_graph_end(fln_graph* g) {
  if (g == nullptr) return FLN_ERR_NULL;
  if (!g->capturing) return FLN_ERR_GRAPH;
  g->capturing = 0;
  if (cudaStreamEndCapture(g->cap_stream, &g->graph) != cudaSuccess || g->graph == nullptr) {
    cudaGetLastError();
    return FLN_ERR_GRAPH;
  }
  if (cudaGraphInstantiate(&g->exec, g->graph, 0) != cudaSuccess) {
    cudaGetLastError();
    return FLN_ERR_GRAPH;
  }
  return FLN_OK;
}

extern "C" int fln_graph_launch(fln_graph* g, void* stream) {
  if (g == nullptr || g->exec == nullptr) return FLN_ERR_GRAPH;
  if (cudaGraphLaunch(g->exec, reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess) {
    cudaGetLastError();
    return FLN_ERR_GRAPH;
  }
  return FLN_OK;
}

extern "C" int fln_graph_destroy(fln_graph* g) {
  if (g == nullptr) return FLN_OK;
  if (g->capturing) {
    cudaGraph_t tmp = nullptr;
    cudaStreamEndCapture(g->cap_stream, &tmp);
    if (tmp) cudaGraphDestroy(tmp);
  }
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  if (g->cap_stream) cudaStreamDestroy(g->cap_stream);
  cudaGetLastError();
  delete g;
  return FLN_OK;
}
