// Shared parts of the persistent, bulk-async staged LayerNorm / RMSNorm forward and backward for sm_100a.
//
// Every CTA is persistent and owns a ring of S shared-memory stages; elected threads keep the
// ring full with 1-D bulk copies (cp.async.bulk global -> shared, completion signalled on an
// mbarrier with complete_tx::bytes), so up to S tiles per CTA are in flight regardless of
// register use.  A tile is R consecutive rows, which are contiguous in memory, so one tile is
// ONE bulk copy per input tensor.  Consumers wait on the stage's mbarrier, pull their vectors
// from shared memory into registers, and the first CTA barrier of the row reduction doubles as
// the "stage is free again" signal after which the stage is refilled.  gamma / beta live in
// registers as floats for the life of the CTA, so the only L2 traffic per row is the row itself.
//
// Which CTA works on which tile.  A B200's SMs do not all see the same memory bandwidth once
// the memory system is saturated, so a static split (CTA b takes tiles b, b + grid, ...) ends
// with the slowest SMs still working while the others idle: a ring copy of 16384 rows of 16 KB
// measured 5800 - 5900 GB/s with the static split and 6420 GB/s with tiles handed out on
// demand, as much as one-CTA-per-row launches reach.  The forward therefore claims its tiles
// from a global counter (results do not depend on which CTA normalizes a row).  The backward
// keeps the static split, because its per-CTA partial sums of dgamma / dbeta must add up in
// the same order on every run; it limits the bytes in flight instead, which narrows the gap.
//
// At bf16 these kernels are bound by instruction issue before they are bound by HBM, so the
// per-element instruction count is what matters: the arithmetic runs on register pairs with
// the packed fp32 instructions of sm_100 (same results bit for bit, half the issue slots), and
// the FULL instantiation (row length equal to K * threads-per-row, no ragged last tile, at
// least a warp per row) has no predication at all in the loop.
//
// No cluster multicast is used anywhere; every copy is CTA-local.
//
// Every wait is bounded by elapsed time (fln_set_wait_limit_ns): on a time-out the CTA votes,
// raises the device status word (fln_device_status), gives copies still in flight a bounded
// chance to land, and leaves through the same exit path as a CTA that finished.
//
// This header holds what the forward (fln_pipeline_fwd.cu) and the backward (fln_pipeline_bwd.cu)
// share: the ring's geometry, the mbarrier / bulk-copy / bounded-wait helpers, the grid barrier,
// and the host-side launch plan (fln_pipeline.cu).
#pragma once

#include <string.h>

#include "fln_common.cuh"

namespace fln {

struct PipeGeom {
  int R;         // rows per tile
  int tpr;       // threads per row
  int log2_tpr;
  int S;         // stages
  uint32_t row_bytes;
  uint32_t second_off;    // byte offset of the second tensor inside a stage
  uint32_t stage_stride;  // bytes per stage
};

// shared-memory header in front of the stages: mbarriers (16 x 8 bytes), the tile held by each
// stage (16 x 4 bytes, at byte 128), reduction scratch (from byte 256)
constexpr int kSmemHeader = 2048;
constexpr int kMaxStages = 16;
constexpr unsigned int kNoTile = 0xffffffffu;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// global -> this CTA's shared memory, 16-byte aligned on both sides, bytes % 16 == 0
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits until the barrier's phase `parity` has completed, for at most about limit_ns.  The
// common case -- the copy has landed or lands within a few probes -- reads no clock at all.
// After 64 failed probes the wait is timed with the SM's cycle counter, read once per 32
// probes, against limit_ns * 2 cycles (the SM clock never exceeds 2 GHz, so the wait lasts at
// least limit_ns and at most about 1.5 times that at the lowest clocks seen under load); the
// outer loop also has an iteration cap.  The limit arrives as a kernel parameter: fetching it
// from global memory whenever a first probe failed put a trip to L2 in front of most rows.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, unsigned long long limit_ns) {
#pragma unroll 1
  for (int it = 0; it < 64; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  const long long limit_cycles = (long long)(limit_ns << 1);
  for (uint32_t outer = 0; outer < (1u << 26); ++outer) {
#pragma unroll 1
    for (int it = 0; it < 32; ++it)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > limit_cycles) return false;
  }
  return false;
}

// ----------------------------------------------------------------------------------------
// Thread-block cluster helpers (a row shared by the two CTAs of a cluster, backward only):
// distributed shared memory by plain st.shared::cluster -- no multicast of any kind -- and the
// hardware cluster barrier.
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  cluster_arrive();
  cluster_wait();
}
// address of `p` (a shared-memory address of this CTA) in the shared memory of CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
// one float into another CTA's shared memory, counted as four bytes of transaction on an
// mbarrier of that CTA: the receiver's wait on that barrier makes the value visible, and the
// sender needs no fence (a release fence here would also wait for the sender's global stores)
__device__ __forceinline__ void st_async_f32(uint32_t addr, float v, uint32_t mbar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(addr),
               "r"(__float_as_uint(v)), "r"(mbar)
               : "memory");
}
// One 16-byte vector of a stage as ONE 128-bit shared-memory load.  (Handing the stage to the
// conversion helper by reference lets the compiler read it word by word: four times the load
// instructions and the shared-memory pipe becomes the stall.)
template <typename T>
__device__ __forceinline__ Pack<T, 16 / sizeof(T)> ld_smem16(const unsigned char* p) {
  Pack<T, 16 / sizeof(T)> out;
  *reinterpret_cast<uint4*>(&out) = *reinterpret_cast<const uint4*>(p);
  return out;
}

// How a kernel takes one vector out of a stage.  16-bit types: by value through the 128-bit
// load above (measured 246.8 vs 285.7 us for the bf16 forward + backward).  fp32: by reference,
// which lets the compiler schedule four 32-bit loads; that form measured faster for fp32
// (backward 245 vs 277 us at 16384 x 8192), where the kernel is HBM-bound anyway.
// Vectors shorter than 16 bytes (row lengths 3, 5 or 7 times a power of two are split into 8- or
// 4-byte vectors so that they divide evenly over the threads) are read with one load of that
// width.
template <typename T, int VEC = 16 / sizeof(T)>
__device__ __forceinline__ decltype(auto) stage_vec(const unsigned char* p) {
  if constexpr (VEC * sizeof(T) == 16 && sizeof(T) == 4) {
    return (*reinterpret_cast<const Pack<T, 4>*>(p));
  } else if constexpr (VEC * sizeof(T) == 16) {
    return ld_smem16<T>(p);
  } else {
    using R = typename Raw<sizeof(T) * VEC>::type;
    Pack<T, VEC> out;
    *reinterpret_cast<R*>(&out) = *reinterpret_cast<const R*>(p);
    return out;
  }
}

// tiles of CTA b under the static split: t = b + i * gridDim.x  (evaluated once per CTA)
__device__ __forceinline__ int my_tile_count(int64_t n_tiles) {
  return (int64_t)blockIdx.x < n_tiles ? (int)((n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
}

// After a failed vote, one thread: raise the status word and give the copies that were issued
// a bounded chance to land before the CTA's shared memory is released.  `armed` stages,
// starting with stage s in the phase in progress, have been armed and not consumed yet.
__device__ __forceinline__ void pipeline_abort(int* status, uint64_t* full, int S, int s, uint32_t phase,
                                               int armed, unsigned long long limit_ns) {
  atomicOr(status, 1);
  for (int j = 0; j < armed; ++j) {
    mbar_wait_bounded(&full[s], phase, limit_ns);
    if (++s == S) {
      s = 0;
      phase ^= 1u;
    }
  }
}

// ----------------------------------------------------------------------------------------
// Grid barrier of a cooperative launch on one 64-bit word of caller memory with undefined
// initial contents:  [63:24] token of the launch | [23:12] CTAs departed | [11:0] CTAs arrived.
// The first CTA to look finds a foreign token and starts the count afresh; the last CTA to
// depart writes 0 (no token is 0), so a graph replay with the same token starts clean as well.
// Every CTA of the grid arrives and departs exactly once on every path, including the ones on
// which it gave up waiting, so the word is back at 0 after any launch whose CTAs all ran.
// Called by ONE thread per CTA, after a CTA barrier that follows the CTA's global writes.
// ----------------------------------------------------------------------------------------
// At kernel start, one thread per CTA: make sure the word carries this launch's token.  One
// compare-and-swap at most and no retry: if it fails, another CTA has initialised the word
// (or has already counted itself in), which is all that is needed.  (Counting arrivals with a
// compare-and-swap loop instead costs a round trip to L2 per CTA *in sequence*: 53 us for 148.)
__device__ __forceinline__ void grid_barrier_init(unsigned long long* w, unsigned long long token) {
  const unsigned long long old = *reinterpret_cast<volatile unsigned long long*>(w);
  if ((old >> 24) != token) atomicCAS(w, old, token << 24);
}
__device__ __forceinline__ void grid_arrive(unsigned long long* w) {
  __threadfence();
  atomicAdd(w, 1ull);
}
// Polls the word until `expect` CTAs of this launch have arrived, for at most about limit_ns
// (timed like mbar_wait_bounded: SM cycle counter against limit_ns * 2 cycles, read once per 16
// polls).
__device__ __forceinline__ bool grid_wait(unsigned long long* w, unsigned long long token, unsigned int expect,
                                          unsigned long long limit_ns) {
  const long long t0 = clock64();
  const long long limit_cycles = (long long)(limit_ns << 1);
  for (uint32_t it = 0; it < (1u << 30); ++it) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(w) : "memory");
    if ((v >> 24) == token && (unsigned int)(v & 0xfffull) == expect) return true;
    if ((it & 15u) == 15u && clock64() - t0 > limit_cycles) return false;
    __nanosleep(32);
  }
  return false;
}
__device__ __forceinline__ void grid_depart(unsigned long long* w, unsigned int grid) {
  const unsigned long long old = atomicAdd(w, 1ull << 12);
  if ((unsigned int)((old >> 12) & 0xfffull) == grid - 1) atomicExch(w, 0ull);
}

// ----------------------------------------------------------------------------------------
// host side (fln_pipeline.cu)
// ----------------------------------------------------------------------------------------
struct PipePlan {
  bool ok;
  bool full;  // branch-free instantiation applies
  bool pair;  // backward only: a row is shared by the two CTAs of a cluster (each half a row)
  bool tail;  // rows are whole but the last of a thread's K vectors is ragged (lanes beyond the row idle)
  bool bsm;   // backward only: the dbeta accumulators live in shared memory behind the stages (24-column plans)
  bool wide;  // backward only: 16-bit rows of 16384 columns, one CTA per row in two passes over the stage
  bool pgl;   // forward only: 512 threads per row, gamma / beta fetched per row, two CTAs per SM
  int vb;     // bytes per vector: 16, or 8 / 4 where that makes the row divide evenly
  int K;
  int threads;
  int grid;
  size_t smem;
  PipeGeom g;
};

// tensors: how many input tensors are staged per tile (forward 1 or 2, backward 2 or 3)
PipePlan plan_pipeline(bool backward, int64_t rows, int cols, int elem_bytes, int tensors,
                       bool allow_params_in_smem = true, bool allow_tail = true);
// trailing rows to split off a forward so that the rest fills the row slots of the fast plan (0: none)
int64_t fwd_plan_odd_rows(int64_t rows, int cols, int elem_bytes, int tensors, bool allow_tail);
PipePlan plan_bwd_pipeline(int64_t rows, int cols, int es, bool with_dres);
bool pipeline_wanted(const PipePlan& P, int64_t rows);
int path_override();                  // fln_set_path_override
unsigned long long wait_limit_ns();   // fln_set_wait_limit_ns

// Words in device memory that the kernels of both files share, looked up once per device
// (cudaGetSymbolAddress) and handed to the kernels as parameters:
//   status  bits: 1 a wait for a bulk copy ran out, 2 the grid barrier's wait ran out, 4 the
//           forward's tile counter was found inconsistent at the end of a launch
//   fault   test hook (fln_set_test_fault)
//   sched   kSchedSlots pairs {next tile, CTAs finished} of the dynamically scheduled forward,
//           all zero between launches (the last CTA of a launch puts its pair back to zero)
struct DeviceWords {
  int* status;
  int* fault;
  unsigned int* sched;
};
constexpr int kSchedSlots = 1024;
bool device_words(DeviceWords* out);  // of the current device; false if they cannot be had
unsigned int next_sched_slot();       // every pipelined forward launch takes the next pair
int pair_slots();                     // clusters of two 512-thread CTAs resident at once (set by the backward)
void set_pair_slots(int n);

template <typename F>
static int set_smem(F kernel, size_t smem) {
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      cudaGetLastError();
      return FLN_ERR_LAUNCH;
    }
  }
  return FLN_OK;
}

}  // namespace fln
