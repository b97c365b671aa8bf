// Host side of the pipelined kernels: the launch plan (rows per tile, threads per row, stages,
// grid), the tuning hooks, the device words the kernels share (status, test hook, tile counters)
// and the C entry points around them.  The kernels are in fln_pipeline_fwd.cu / _bwd.cu.
#include <atomic>
#include <mutex>

#include "fln_pipeline.cuh"

namespace fln {

__device__ int g_device_status = 0;
__device__ int g_test_fault = 0;
__device__ unsigned int g_tile_sched[kSchedSlots][2];

bool device_words(DeviceWords* out) {
  static std::mutex mu;
  static DeviceWords cache[64];
  static bool have[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return false;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev]) {
    DeviceWords w;
    void *a = nullptr, *b = nullptr, *c = nullptr;
    if (cudaGetSymbolAddress(&a, g_device_status) != cudaSuccess || cudaGetSymbolAddress(&b, g_test_fault) != cudaSuccess ||
        cudaGetSymbolAddress(&c, g_tile_sched) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    w.status = static_cast<int*>(a);
    w.fault = static_cast<int*>(b);
    w.sched = static_cast<unsigned int*>(c);
    cache[dev] = w;
    have[dev] = true;
  }
  *out = cache[dev];
  return true;
}

// ----------------------------------------------------------------------------------------
// host: geometry
// ----------------------------------------------------------------------------------------
// 0 auto, 1 register kernels only, 2 pipeline whenever it fits, 3 as 2 with the column reduce
// as a second kernel
static std::atomic<int> g_path_override{0};
// stages per ring: 0 automatic, >= 2 forced (clamped to what fits)
static std::atomic<int> g_stage_override{0};
// every pipelined forward launch takes the next pair of g_tile_sched
static std::atomic<unsigned int> g_sched_seq{0};
// How long a wait inside a kernel may last, in nanoseconds.  It travels in the kernel parameters
// (constant bank): a wait that reads it from global memory pays a trip to L2 whenever its first
// probe fails, which in a memory-bound kernel is most of the time (the backward at 16384 x 8192
// bf16 took 205 instead of 145 us that way).
static std::atomic<unsigned long long> g_wait_limit_ns{1000ull * 1000ull * 1000ull};


static int ilog2i(int v) {
  int l = 0;
  while ((1 << l) < v) ++l;
  return l;
}
static int next_pow2i(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

// tensors: how many input tensors are staged per tile (1 or 2)
PipePlan plan_pipeline(bool backward, int64_t rows, int cols, int elem_bytes, int tensors,
                       bool allow_params_in_smem, bool allow_tail) {
  PipePlan P;
  memset(&P, 0, sizeof(P));
  const int vec = 16 / elem_bytes;
  if (cols % vec != 0 || rows <= 0) return P;
  const int nv = cols / vec;
  const int cta_threads = backward ? 512 : 256;
  // vectors per thread: forward 64 B per thread, backward about 16 columns per thread
  const int pref = backward ? (16 / vec) : 4;
  // register budget at 512 threads (128 registers): backward at most 16 columns per
  // thread, forward at most 32 elements per thread
  const int maxK = backward ? 16 / vec : 32 / vec;
  int K = 0, tpr = 0;
  int fK = 0, ftpr = 0;
  plan_override(&fK, &ftpr);
  if (fK > 0 && ftpr >= 8 && ftpr <= 512 && (ftpr & (ftpr - 1)) == 0 && fK <= maxK &&
      (fK & (fK - 1)) == 0 && (int64_t)fK * ftpr >= nv) {
    K = fK;
    tpr = ftpr;
  }
  for (int k = pref; k <= maxK && K == 0; k <<= 1) {
    int t = next_pow2i((nv + k - 1) / k);
    if (t > 512) continue;
    // forward: two CTAs of 256 threads per SM rather than one of 512 while the register budget
    // allows more vectors per thread (fp32 8192 columns: 8 vectors for each of 256 threads)
    if (!backward && t > cta_threads && (k << 1) <= maxK) continue;
    if (t < 8) t = 8;
    int kk = next_pow2i((nv + t - 1) / t);
    K = kk;
    tpr = t;
  }
  // Row lengths 3, 5 or 7 times a power of two (768, 1280, 2560, 5120, 6144, 12288 ...) do not
  // divide over a power-of-two number of threads with a power-of-two number of 16-byte vectors
  // each; the padded plan above would run them through the bounds-checked kernel with a
  // quarter or more of the lanes idle.  Look for an exact fit with K in {3, 5, 7} and, if
  // need be, 8- or 4-byte vectors; the branch-free instantiation then applies.
  int vb = 16;
  // Elements per thread the odd plans may use.  Backward, 16-bit types: 20 columns per thread
  // (K = 5 vectors of 4) still compile without spills at 128 registers and run faster than
  // the 16-column plans; 24 columns spill a little and are slower than 12 (6144 columns: 3986
  // vs 5237 GB/s), but faster than the two-kernel long-row path (12288 columns: 4018 vs 3365
  // GB/s), so they serve only rows that fit no other plan.  fp32 backward stays at 16.
  // Forward, 16-bit types: 40 or 48 elements per thread (K = 5 or 6 vectors of 8) with gamma /
  // beta parked in shared memory instead of registers.
  const bool wide_fwd = !backward && elem_bytes == 2 && allow_params_in_smem;
  // (24 columns at once for the plain 16-bit backward: its LayerNorm form parks the dbeta
  // accumulators in shared memory, see `bsm` below, and then beats the 12-column plans)
  const int caps[2] = {backward ? (elem_bytes == 2 ? (tensors == 2 ? 24 : 20) : (tensors == 2 ? 20 : 16))
                                : (wide_fwd ? 48 : 32),
                       backward && elem_bytes == 2 ? 24 : 0};
  for (int pass = 0; pass < 2; ++pass) {
    const int cap_elems = caps[pass];
    if (cap_elems == 0 || fK != 0) break;
    if (pass == 0 ? !(K == 0 || (int64_t)K * tpr != nv) : K != 0) break;
    const int min_vb = backward ? (elem_bytes == 4 ? 8 : 4) : (elem_bytes == 4 ? 16 : 8);
    int best_elems = 0;
    for (int cvb = 16; cvb >= min_vb; cvb >>= 1) {
      const int cvec = cvb / elem_bytes;
      if (cols % cvec != 0) continue;
      const int cnv = cols / cvec;
      for (int ck = 3; ck <= 7; ++ck) {
        if (ck == 4 || (ck == 6 && (backward || cvb != 16))) continue;
        if (ck * cvec > cap_elems || cnv % ck != 0) continue;
        const int t = cnv / ck;
        // (half-warp rows only for the 48-element forward plan: 768 columns in 16-bit types)
        if (t < ((wide_fwd && ck == 6) ? 16 : 32) || t > 512 || (t & (t - 1)) != 0) continue;
        if (backward && elem_bytes == 4 && ck * cvec == 20 && t != 512) continue;  // fp32, 20 columns: 10240 only
        const int thr = t > cta_threads ? t : cta_threads;
        if (rows % (thr / t) != 0) continue;  // only the branch-free kernel exists for these
        // half-warp rows make tiles of 16 rows: only where every CTA still streams four of them
        if (t == 16 && rows / (thr / t) < 8LL * usable_sms()) continue;
        if (ck * cvec > best_elems) {
          best_elems = ck * cvec;
          K = ck;
          tpr = t;
          vb = cvb;
        }
      }
    }
  }
  // Rows that fit none of the exact plans (1600 = 25 * 64, 4608 = 9 * 512, 5376 = 21 * 256
  // columns ...): K vectors on the power-of-two number of threads for which only the last
  // vector is ragged, (K - 1) t < vectors per row <= K t -- at most 1 / K of the lanes idle in
  // that one vector, against up to half of all lanes in the padded power-of-two plan.  The
  // first candidate that fits is taken: most elements per thread first, except that the
  // backward prefers seven short vectors to four of twice the length where both fit (fewer idle
  // lanes in the last vector; bf16 1600 / 3200 / 6400 / 3456 columns: 5701 / 5684 / 5450 / 5952
  // against 5505 / 5550 / 5373 / 5822 GB/s; fp32 within 3 % either way except 3200 columns,
  // 6385 against 5903).  The kernels know at compile time that vectors 0 .. K - 2 are whole
  // (the `tail` instantiations); rows must fill the CTA's row slots.  The (K, bytes per vector)
  // pairs are the ones instantiated:
  //   forward   fp32    16 B x 8 .. 3                          (32 .. 12 elements)
  //             16-bit  16 B x 7 .. 5, gamma / beta in shared memory (56 .. 40), 16 B x 4, 8 B x 7, 16 B x 3
  //   backward  fp32    8 B x 7, 16 B x 4, 3, 8 B x 5          (10 .. 16 columns)
  //             16-bit  4 B x 7, 8 B x 5, 4, 16 B x 3, 8 B x 3     (12 .. 24 columns)
  // 16-bit forward rows of 14336 columns divide into 7 x 8 bytes x 512 threads, one CTA per SM;
  // four 16-byte vectors with the last one ragged run two CTAs per SM (5829 against 5200 GB/s)
  // and rows of 7 x 8 bytes on fewer threads are served better by the ragged kernel's seven 16-byte
  // vectors on half the threads with gamma / beta in shared memory, although no vector is
  // ragged (7168 columns: 6237 -> 6492 GB/s as measured on 7160)
  const bool prefer_ragged = !backward && elem_bytes == 2 && K == 7 && vb == 8 &&
                             ((tensors == 1 && tpr == 512) || (wide_fwd && tpr >= 64));
  bool tail = false;
  if (allow_tail && fK == 0 && tensors <= (backward ? 3 : 2) &&
      (K == 0 || (int64_t)K * tpr != cols / (vb / elem_bytes) || prefer_ragged)) {
    struct Cand {
      int k, vb;
    };
    static const Cand kFwd32[] = {{8, 16}, {7, 16}, {6, 16}, {5, 16}, {4, 16}, {3, 16}};
    static const Cand kFwd16Wide[] = {{7, 16}, {6, 16}, {5, 16}, {4, 16}, {7, 8}, {3, 16}};
    static const Cand kFwd16[] = {{4, 16}, {7, 8}, {3, 16}};
    static const Cand kBwd32[] = {{7, 8}, {4, 16}, {3, 16}, {5, 8}};
    static const Cand kBwd16[] = {{7, 4}, {5, 8}, {4, 8}, {3, 16}, {3, 8}};
    const Cand* cand = backward ? (elem_bytes == 4 ? kBwd32 : kBwd16) : (elem_bytes == 4 ? kFwd32 : (wide_fwd ? kFwd16Wide : kFwd16));
    const int ncand = backward ? (elem_bytes == 4 ? 4 : 5) : (elem_bytes == 4 ? 6 : (wide_fwd ? 6 : 3));
    for (int c = 0; c < ncand && !tail; ++c) {
      const int ck = cand[c].k, cvb = cand[c].vb, cvec = cvb / elem_bytes;
      if (cols % cvec != 0) continue;
      const int cnv = cols / cvec;
      const int t = next_pow2i((cnv + ck - 1) / ck);
      if (t < (backward ? 64 : 32) || t > 512 || (int64_t)(ck - 1) * t >= cnv) continue;
      // 24 columns per thread in the 16-bit backward: dbeta accumulators in shared memory, rows
      // of up to 256 threads (longer rows run the two-pass kernel)
      if (backward && elem_bytes == 2 && ck == 3 && cvb == 16 && (t > 256 || tensors != 2)) continue;
      const int thr = t > cta_threads ? t : cta_threads;
      if (rows % (thr / t) != 0) continue;
      K = ck;
      tpr = t;
      vb = cvb;
      tail = true;
    }
  }
  if (K == 0) return P;
  const int threads = tpr > cta_threads ? tpr : cta_threads;
  const int R = threads / tpr;
  const uint32_t row_bytes = (uint32_t)cols * elem_bytes;
  const uint32_t tile_bytes = row_bytes * R;
  const uint32_t stage = tile_bytes * tensors;
  // Shared memory a CTA may use -- forward: two CTAs per SM with ~100 KB each; backward: one
  // 512-thread CTA with ~200 KB -- and the bytes it wants in flight.  More stages than the
  // memory latency needs do harm: with the SMs oversubscribing the memory system its
  // arbitration gets unfair and the slowest SMs set the time of a launch whose split is static
  // (ring copy, 16 KB tiles, one CTA per SM: 3 stages 6383 GB/s, 6 stages 5943).  About 96 KB
  // in flight per SM measured best for both directions at 16384 x 8192 bf16 (backward with 6 /
  // 5 / 4 / 3 / 2 stages of 32 KB: 126.7 / 126.1 / 125.5 / 124.6 / 127.8 us; forward, dynamic
  // tiles, 2 CTAs with 6 / 4 / 3 / 2 stages of 16 KB: 85.9 / 84.1 / 83.5 / 84.1 us).
  // CTAs per SM by design: the 512-thread kernels are capped at 128 registers per thread by
  // their launch bounds and use most of them, so one such CTA fills an SM's register file and
  // two 256-thread CTAs do
  // 16-bit forward rows of 16384 columns (512 threads, 4 vectors each): two CTAs per SM (64
  // registers each) with gamma / beta fetched per row (plain forward only): 5420 -> 5884 GB/s.
  // With 5 or 6 vectors per thread the same form was slower than one CTA per SM (bf16 20480:
  // 5072 against 5831 GB/s, fp32 12288: 5108 against 5727; fp32 10240 unchanged).
  // The same with a ragged last vector (12296 .. 16376 columns).
  const bool pgl = !backward && allow_tail && threads == 512 && tpr == 512 && tensors == 1 && vb == 16 &&
                   elem_bytes == 2 && K == 4 && (tail || (int64_t)K * tpr == cols / (vb / elem_bytes)) &&
                   (size_t)kSmemHeader + 2 * (size_t)stage <= 100 * 1024;
  const int ctas_per_sm = (threads >= 512 && !pgl) ? 1 : 2;
  const size_t budget = (size_t)(200 * 1024) / ctas_per_sm;
  const size_t in_flight = (size_t)(96 * 1024) / ctas_per_sm;
  int S_fit = (int)((budget - kSmemHeader) / stage);
  if (S_fit < 2) S_fit = (int)((220 * 1024 - kSmemHeader) / stage);  // try the whole SM for one CTA
  if (S_fit > kMaxStages) S_fit = kMaxStages;
  if (S_fit < 2) return P;
  int S = (int)((in_flight + stage - 1) / stage);
  if (S < 2) S = 2;
  const int fS = g_stage_override.load(std::memory_order_relaxed);
  if (fS >= 2) S = fS;
  if (S > S_fit) S = S_fit;
  P.ok = true;
  P.full = !tail && (tpr >= 32 || (!backward && K == 6 && tpr == 16)) && (int64_t)K * tpr == cols / (vb / elem_bytes) &&
           rows % R == 0;  // a `tail` plan runs its own instantiations even where its last vector happens to be whole
  P.tail = tail;
  P.pgl = pgl;
  P.vb = vb;
  P.K = K;
  P.threads = threads;
  // forward plans beyond 32 elements per thread keep gamma and beta behind the stages
  const bool params_in_smem = !backward && !pgl && K * (vb / elem_bytes) > 32;
  if (params_in_smem) {
    const int room = (int)((budget - kSmemHeader - 2 * (size_t)row_bytes) / stage);
    if (S > room) S = room;
    // no room for two stages beside the parameters (two staged tensors of a long row): plan
    // again with at most 32 elements per thread
    if (S < 2) return plan_pipeline(backward, rows, cols, elem_bytes, tensors, false, allow_tail);
  }
  // 16-bit backward with 24 columns per thread: the dbeta accumulators (12 float2 per thread)
  // go behind the stages; the LayerNorm instantiation uses them, RMSNorm has none
  // (and the fp32 backward with 20 columns per thread, 10240 columns)
  bool bsm = backward && vb == 16 && threads == 512 && tensors == 2 && (P.full || (tail && elem_bytes == 2)) &&
             ((elem_bytes == 2 && K == 3) || (elem_bytes == 4 && K == 5));
  size_t bsm_bytes = bsm ? (size_t)(K * (16 / elem_bytes) / 2) * 512 * sizeof(float2) : 0;
  if ((size_t)kSmemHeader + (size_t)S * stage + bsm_bytes > 220 * 1024) {
    bsm = false;
    bsm_bytes = 0;
  }
  P.bsm = bsm;
  P.smem = kSmemHeader + (size_t)S * stage + (params_in_smem ? 2 * (size_t)row_bytes : 0) + bsm_bytes;
  P.g.R = R;
  P.g.tpr = tpr;
  P.g.log2_tpr = ilog2i(tpr);
  P.g.S = S;
  P.g.row_bytes = row_bytes;
  P.g.second_off = tile_bytes;
  P.g.stage_stride = stage;
  const int64_t n_tiles = (rows + R - 1) / R;
  // the grid must not exceed what is resident at once: a CTA of a second wave would start its
  // share of the rows when the first wave is done
  const int by_smem = (int)((227 * 1024) / P.smem);
  const int per_sm = by_smem < ctas_per_sm ? by_smem : ctas_per_sm;
  // The SMs a caller asked to be left free (fln_set_sm_reserve) matter to the backward's static
  // split only: a forward CTA that starts late behind somebody else's kernel just claims fewer
  // tiles, so the forward fills every SM.
  const int64_t cap = (int64_t)(backward ? usable_sms() : sm_count()) * (per_sm < 1 ? 1 : per_sm);
  P.grid = (int)(n_tiles < cap ? n_tiles : cap);
  return P;
}

bool pipeline_wanted(const PipePlan& P, int64_t rows) {
  const int ov = g_path_override.load(std::memory_order_relaxed);
  if (!P.ok || P.g.R <= 0 || P.grid <= 0 || ov == 1) return false;
  if (ov == 2 || ov == 3) return true;
  // worth it once every CTA streams several tiles
  const int64_t n_tiles = (rows + P.g.R - 1) / P.g.R;
  return n_tiles >= 4LL * P.grid || n_tiles >= 8LL * sm_count();
}

// clusters of two backward CTAs that are resident at once on the current device: half the SMs
// until the backward's launcher has asked the runtime (cudaOccupancyMaxActiveClusters)
static std::atomic<int> g_pair_slots[64];
int pair_slots() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    dev = 0;
  }
  const int v = g_pair_slots[dev].load(std::memory_order_relaxed);
  const int half = usable_sms() / 2;
  return v > 0 && v < half ? v : (half > 0 ? half : 1);
}
void set_pair_slots(int n) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return;
  }
  g_pair_slots[dev].store(n, std::memory_order_relaxed);
}

// Rows beyond the register budget of one CTA (16-bit rows above 12288 columns, fp32 rows above
// 8192) are shared by the two CTAs of a
// thread-block cluster: each CTA stages and differentiates half of every row, the two row sums
// cross through distributed shared memory.  The plan is the half row's plan (512 threads per
// half row, one row per tile) with `pair` set and the grid counted in CTAs (two per row slot).
PipePlan plan_bwd_pipeline(int64_t rows, int cols, int es, bool with_dres) {
  PipePlan P = plan_pipeline(true, rows, cols, es, with_dres ? 3 : 2);
  // 16-bit rows beyond the one-pass kernel's columns per thread, up to 16384 columns: one CTA
  // per row, two passes over the staged row (fln_pipeline_bwd_wide.cu); stages of dy + x and
  // the dbeta accumulators behind them.  16384 and 14336 columns divide exactly (4 vectors of
  // 16 bytes, 7 of 8 bytes per thread); other multiples of 8 columns get 3 or 4 vectors of 16
  // bytes of which the last is ragged.
  if (!P.ok && !with_dres && es == 2 && cols > 8192 && cols <= 16384 && cols % 8 == 0 && cols != 12288 && rows > 0 &&
      g_path_override.load(std::memory_order_relaxed) != 3) {
    PipePlan W;
    memset(&W, 0, sizeof(W));
    W.ok = true;
    W.wide = true;
    W.vb = cols == 14336 ? 8 : 16;
    W.K = cols == 14336 ? 7 : (cols > 12288 ? 4 : 3);
    W.tail = cols != 14336 && cols != W.K * 4096;
    W.threads = 512;
    W.g.R = 1;
    W.g.tpr = 512;
    W.g.log2_tpr = 9;
    W.g.row_bytes = (uint32_t)cols * 2;
    W.g.second_off = W.g.row_bytes;
    W.g.stage_stride = 2 * W.g.row_bytes;
    // dbeta accumulators: one float2 per thread and column pair
    const size_t accb = (size_t)W.K * (W.vb / 4) * 512 * sizeof(float2);
    W.g.S = W.K == 3 ? 3 : 2;
    W.smem = (size_t)kSmemHeader + (size_t)W.g.S * W.g.stage_stride + accb;
    const int64_t cap = usable_sms();
    W.grid = (int)(rows < cap ? rows : cap);
    return W;
  }
  if (!P.ok && !with_dres && cols % 2 == 0 && g_path_override.load(std::memory_order_relaxed) != 3) {
    PipePlan H = plan_pipeline(true, rows, cols / 2, es, 2);
    // (a ragged half row: its first column must sit on a 16-byte boundary for the bulk copies)
    if (H.ok && (H.full || (H.tail && cols % (32 / es) == 0)) && !H.bsm && H.threads == 512 && H.g.tpr == 512 &&
        H.g.R == 1 && H.K * (H.vb / es) <= 20) {
      H.pair = true;
      const int64_t slots = pair_slots();
      H.grid = (int)(2 * (rows < slots ? rows : slots));
      return H;
    }
  }
  return P;
}

bool describe_pipeline(bool backward, int64_t rows, int cols, int elem_bytes, PipeDescription* out) {
  // (a row count that does not fill the fast plan's row slots runs that plan on all but its last
  // few rows)
  rows -= backward ? bwd_pipeline_odd_rows(elem_bytes == 4 ? FLN_F32 : FLN_BF16, rows, cols, false)
                   : fwd_plan_odd_rows(rows, cols, elem_bytes, 1, true);
  PipePlan P = backward ? plan_bwd_pipeline(rows, cols, elem_bytes, false) : plan_pipeline(false, rows, cols, elem_bytes, 1);
  if (!pipeline_wanted(P, rows)) return false;
  if (!backward && elem_bytes == 4 && cols <= 4096 && g_path_override.load(std::memory_order_relaxed) == 0) {
    // the fp32 LayerNorm forward of short exact rows goes to the register kernel (launch_fwd_pipeline)
    const Plan rp = make_plan(false, rows, cols, elem_bytes, true);
    if (!rp.generic && rp.vec == 4 && (int64_t)rp.K * rp.tpr * rp.vec == cols) return false;
  }
  // the odd plans exist only as branch-free instantiations; K = 8 only for fp32 forward
  if ((P.vb != 16 || P.K == 3 || P.K == 5 || P.K == 6 || P.K == 7) && !P.full && !P.tail && !P.wide) return false;
  out->vector_bytes = P.vb;
  out->K = P.K;
  out->tpr = P.g.tpr;
  out->threads = P.threads;
  out->rows_per_cta = P.g.R;
  out->stages = P.g.S;
  out->grid = P.grid;
  return true;
}

int64_t bwd_pipeline_partial_rows(int kind, int dtype, int64_t rows, int cols, bool with_dres) {
  (void)kind;
  const int es = dtype == FLN_F32 ? 4 : 2;
  PipePlan P = plan_bwd_pipeline(rows, cols, es, with_dres);
  if (!pipeline_wanted(P, rows)) return 0;
  return P.pair ? (int64_t)(P.grid / 2) : (int64_t)P.grid * P.g.R;
}


int64_t fwd_plan_odd_rows(int64_t rows, int cols, int es, int tensors, bool allow_tail) {
  if (rows < 32 || rows % 16 == 0) return 0;
  // the plan a row count that fills every row slot would get: if this row count gets another
  // one (a bounds-checked instantiation, or a later candidate with fewer rows per CTA), split
  const int64_t main16 = rows - rows % 16;  // every plan's rows per CTA divide 16
  const PipePlan M = plan_pipeline(false, main16, cols, es, tensors, true, allow_tail);
  if (!M.ok || !(M.full || M.tail) || M.g.R <= 1 || !pipeline_wanted(M, main16)) return 0;
  const PipePlan P = plan_pipeline(false, rows, cols, es, tensors, true, allow_tail);
  if (P.ok && (P.full || P.tail) && P.K == M.K && P.vb == M.vb && P.g.tpr == M.g.tpr) return 0;
  return rows % M.g.R;
}

int64_t bwd_pipeline_odd_rows(int dtype, int64_t rows, int cols, bool with_dres) {
  const int es = dtype == FLN_F32 ? 4 : 2;
  if (rows < 32 || rows % 16 == 0) return 0;
  // the plan a row count that fills every row slot would get: if this row count gets another
  // one (a bounds-checked instantiation, or a later candidate with fewer rows per CTA), split
  const int64_t main16 = rows - rows % 16;  // every plan's rows per CTA divide 16
  const PipePlan M = plan_bwd_pipeline(main16, cols, es, with_dres);
  if (!M.ok || !(M.full || M.tail) || M.wide || M.pair || M.g.R <= 1 || !pipeline_wanted(M, main16)) return 0;
  const PipePlan P = plan_bwd_pipeline(rows, cols, es, with_dres);
  if (P.ok && (P.full || P.tail) && P.K == M.K && P.vb == M.vb && P.g.tpr == M.g.tpr) return 0;
  return rows % M.g.R;
}

int path_override() { return g_path_override.load(std::memory_order_relaxed); }
unsigned long long wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }
unsigned int next_sched_slot() {
  return g_sched_seq.fetch_add(1, std::memory_order_relaxed) % (unsigned int)kSchedSlots;
}

}  // namespace fln

using namespace fln;

extern "C" void fln_set_path_override(int mode) { g_path_override.store(mode, std::memory_order_relaxed); }
extern "C" void fln_set_stage_override(int stages) { g_stage_override.store(stages, std::memory_order_relaxed); }

extern "C" int fln_set_wait_limit_ns(unsigned long long ns) {
  g_wait_limit_ns.store(ns == 0 ? 1000ull * 1000ull * 1000ull : ns, std::memory_order_relaxed);
  return FLN_OK;
}

extern "C" int fln_set_test_fault(int bits) {
  if (cudaMemcpyToSymbol(g_test_fault, &bits, sizeof(bits)) != cudaSuccess) {
    cudaGetLastError();
    return FLN_ERR_LAUNCH;
  }
  return FLN_OK;
}

// Host-only consistency check of the pipeline planner over a grid of shapes: every plan it
// accepts must describe a launch that exists (at least two stages, shared memory within the
// opt-in limit, a row that divides exactly where the branch-free kernel is claimed, a grid).
// Returns the number of violations.  Needs no GPU.
extern "C" int fln_planner_selftest(void) {
  static const int kCols[] = {8,    16,   64,   96,   256,  512,  768,  1000, 1024, 1280, 1536,  1600,  2048, 2560,
                              3072, 4096, 5120, 6144, 7168, 8192, 9216, 10240, 12288, 14336, 16384, 20480, 32768};
  static const int64_t kRows[] = {1, 7, 64, 600, 2049, 4096, 16384, 131072};
  int bad = 0;
  for (int cols : kCols)
    for (int64_t rows : kRows)
      for (int es = 2; es <= 4; es += 2)
        for (int backward = 0; backward <= 1; ++backward)
          for (int tensors = backward ? 2 : 1; tensors <= (backward ? 3 : 2); ++tensors) {
            const PipePlan P = plan_pipeline(backward != 0, rows, cols, es, tensors);
            if (!P.ok) continue;
            const int vec = P.vb / es;
            bool ok = P.g.S >= 2 && P.g.R >= 1 && P.grid >= 1 && P.smem <= 227u * 1024u && P.threads >= 32 &&
                      P.threads <= 512 && P.K >= 1 && vec >= 1 && cols % vec == 0 &&
                      (int64_t)P.K * P.g.tpr >= cols / vec && P.g.tpr * P.g.R == P.threads &&
                      P.smem >= (size_t)kSmemHeader + (size_t)P.g.S * P.g.stage_stride;
            if (P.full) ok = ok && (int64_t)P.K * P.g.tpr * vec == cols && rows % P.g.R == 0;
            // odd K or short vectors exist only as branch-free instantiations
            if ((P.vb != 16 || P.K == 3 || P.K == 5 || P.K == 6 || P.K == 7) && !P.full && !P.tail) ok = false;
            // a ragged last vector: vectors 0 .. K - 2 whole, rows fill the CTA
            if (P.tail)
              ok = ok && P.K >= 3 && P.K <= 8 && !P.full && (int64_t)(P.K - 1) * P.g.tpr < cols / vec && rows % P.g.R == 0;
            if (!ok) ++bad;
          }
  return bad;
}

extern "C" int fln_device_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  }
  return v;
}

