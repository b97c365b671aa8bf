/*
 * fln_b200.h -- C ABI of the B200 (sm_100a) row-normalization library, libfln_b200.so.
 *
 * Every entry point takes plain device pointers, sizes and enums; nothing here depends
 * on PyTorch.  Unless stated otherwise an entry point
 *   - launches asynchronously on `stream` (a cudaStream_t passed as void*; NULL = the
 *     legacy default stream) of the CUDA device that is current on the calling thread,
 *   - allocates nothing: the caller owns inputs, outputs and scratch,
 *   - returns FLN_OK (0) or one of the fln_status codes below and never aborts.
 * Matrices are row-major and contiguous: `rows` x `cols`, row pitch == cols.
 *
 * Each declaration names the interface of the reference project
 * (JonSnow1807/Fused-LayerNorm-CUDA-Operator, paths relative to its root) it stands in for.
 */
#ifndef FLN_B200_H
#define FLN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of matrices and parameters */
typedef enum {
  FLN_F32 = 0,
  FLN_BF16 = 1,
  FLN_F16 = 2,
  FLN_FP8_E4M3 = 3 /* output only */
} fln_dtype;

typedef enum { FLN_LAYERNORM = 0, FLN_RMSNORM = 1 } fln_kind;

/* epilogue applied to the normalized value before it is stored.
 * FLN_ACT_GELU_TANH is the reference's formula (csrc/layernorm_cuda_kernel.cu:31-36). */
typedef enum { FLN_ACT_NONE = 0, FLN_ACT_GELU_TANH = 1, FLN_ACT_GELU_ERF = 2 } fln_act;

typedef enum {
  FLN_OK = 0,
  FLN_ERR_DTYPE = 1,       /* dtype not supported by this entry point            */
  FLN_ERR_SHAPE = 2,       /* rows < 0 or > INT32_MAX, cols <= 0 or > INT32_MAX  */
  FLN_ERR_NULL = 3,        /* a required pointer is NULL                         */
  FLN_ERR_WORKSPACE = 4,   /* scratch buffer missing or too small                */
  FLN_ERR_LAUNCH = 5,      /* the CUDA runtime reported an error at launch       */
  FLN_ERR_UNSUPPORTED = 6, /* combination not implemented (e.g. fp8 with odd cols) */
  FLN_ERR_GRAPH = 7,       /* CUDA-graph capture / instantiate / launch failed   */
  FLN_ERR_ARG = 8,         /* bad enum value or inconsistent arguments           */
  FLN_ERR_STATIC_SCRATCH = 9 /* problem too large for the built-in scratch array  */
} fln_status;

/* Human-readable text for a status code (static storage). */
const char* fln_status_string(int status);
/* Library version "major.minor.patch" and the CUDA runtime it was built against.
 * Stand in for the module attributes __version__ / __cuda_version__
 * (csrc/layernorm_cuda.cpp:230-237). */
const char* fln_version(void);
int fln_cuda_runtime_version(void);

/* ----------------------------------------------------------------------------------
 * Forward
 * -------------------------------------------------------------------------------- */

/* y = (x - mean) * rstd * gamma + beta, per row; statistics in fp32.
 * gamma and beta may each be NULL (treated as 1 and 0; the reference applies the affine
 * only when both are present, csrc/layernorm_cuda_kernel.cu:87).  mean / rstd ([rows],
 * fp32) may be NULL when the caller does not need them.
 * Replaces layernorm_cuda (csrc/layernorm_cuda_kernel.cu:152-178, called from
 * csrc/bindings.cpp:19-28) and layernorm_forward_cuda / layernorm_forward_cuda_optimized
 * (declared csrc/layernorm_cuda.cpp:14-31, csrc/layernorm.h:15-22; defined
 * csrc/layernorm_cuda_kernel_optimized.cu:171-212). */
int fln_layernorm_forward(const void* x, const void* gamma, const void* beta, void* y,
                          float* mean, float* rstd, int64_t rows, int64_t cols, int dtype,
                          float eps, void* stream);

/* y = gelu(layernorm(x)); `approximate` is FLN_ACT_GELU_TANH (the reference's formula)
 * or FLN_ACT_GELU_ERF.  Replaces layernorm_gelu_cuda
 * (csrc/layernorm_cuda_kernel.cu:180-206, called from csrc/bindings.cpp:30-39). */
int fln_layernorm_gelu_forward(const void* x, const void* gamma, const void* beta, void* y,
                               int64_t rows, int64_t cols, int dtype, float eps,
                               int approximate, void* stream);

/* General forward.  s = x (+ residual, rounded to io_dtype and written to sum_out when
 * residual != NULL); y = act(norm(s)) stored as out_dtype.
 *   kind      FLN_LAYERNORM (writes mean and rstd) or FLN_RMSNORM (writes rstd only;
 *             beta and mean must be NULL)
 *   io_dtype  type of x, residual, sum_out, gamma, beta: F32 / BF16 / F16
 *   out_dtype type of y: io_dtype, or FLN_BF16 when io_dtype is FLN_F32
 * No counterpart in the reference beyond the two entry points above; this is the fused
 * residual-add / RMSNorm / down-cast variant of the same row kernel. */
int fln_norm_forward(int kind, const void* x, const void* residual, const void* gamma,
                     const void* beta, void* y, void* sum_out, float* mean, float* rstd,
                     int64_t rows, int64_t cols, int io_dtype, int out_dtype, float eps,
                     int act, void* stream);

/* Forward with fp8-e4m3 output and a per-tensor scale computed on the device.
 * Phase 1 reads x (+ residual), writes sum_out, mean/rstd, and reduces amax = max|y|
 * over the whole tensor; phase 2 re-reads s and writes q = sat_e4m3(y * scale) with
 * scale = 448 / amax (1 when amax == 0).  Two launches and one 4-byte memset, all on
 * `stream`; there is no grid-wide wait.
 *   q        [rows, cols] bytes (e4m3 codes)
 *   sum_out  [rows, cols] io_dtype; required when residual != NULL, else may be NULL
 *   mean     [rows] fp32, required for FLN_LAYERNORM, must be NULL for FLN_RMSNORM
 *   rstd     [rows] fp32, required (phase 2 reads it)
 *   amax, scale  one fp32 each, required
 * cols must be a multiple of 16 / sizeof(io element) and every matrix pointer 16-byte
 * aligned, otherwise FLN_ERR_UNSUPPORTED.  No counterpart in the reference. */
int fln_norm_forward_fp8(int kind, const void* x, const void* residual, const void* gamma,
                         const void* beta, void* q, void* sum_out, float* mean, float* rstd,
                         float* amax, float* scale, int64_t rows, int64_t cols, int io_dtype,
                         float eps, void* stream);

/* One-pass fp8-e4m3 forward with a scale the caller supplies ("delayed scaling": typically
 * 448 / amax of the previous step).  One launch: reads x (+ residual) once, writes sum_out and
 * q = sat_e4m3(y * *scale_in); 7 bytes per element with a residual instead of the 9 of the
 * two-launch form above.
 *   scale_in  one fp32 on the device, required
 *   amax_out  one fp32 on the device or NULL: max|y| of THIS call (for the next step's scale)
 *   mean, rstd  optional here (nothing re-reads them)
 * Values beyond +-448 after scaling saturate.  Same shape / alignment rules as
 * fln_norm_forward_fp8.  No counterpart in the reference. */
int fln_norm_forward_fp8_delayed(int kind, const void* x, const void* residual, const void* gamma,
                                 const void* beta, void* q, void* sum_out, float* mean, float* rstd,
                                 const float* scale_in, float* amax_out, int64_t rows, int64_t cols,
                                 int io_dtype, float eps, void* stream);

/* One-pass fp8-e4m3 forward with one scale per row: row_scale[r] = 448 / max|y[r, :]| (1 for an
 * all-zero row), q[r, :] = sat_e4m3(y[r, :] * row_scale[r]).  The row is in registers when its
 * maximum is known, so this is also one launch and 7 bytes per element.
 *   row_scale [rows] fp32 on the device, required (dequantize with q / row_scale[r])
 *   amax_out  one fp32 or NULL: max|y| over the whole tensor
 * No counterpart in the reference. */
int fln_norm_forward_fp8_rowwise(int kind, const void* x, const void* residual, const void* gamma,
                                 const void* beta, void* q, void* sum_out, float* mean, float* rstd,
                                 float* row_scale, float* amax_out, int64_t rows, int64_t cols,
                                 int io_dtype, float eps, void* stream);

/* One-pass MXFP8 output (OCP microscaling, the block-scaled form Blackwell's tensor cores
 * consume): every 32 consecutive elements of a row share a power-of-two scale
 * 2^(floor(log2(max|y| over the block)) - 8), stored as an E8M0 byte (value 2^(byte - 127); an
 * all-zero block stores 0); q = sat_e4m3(y / scale).
 *   q            [rows, cols] bytes (e4m3 codes)
 *   block_scale  [rows, cols / 32] bytes (E8M0), required; cols must be a multiple of 32
 *   amax_out     one fp32 or NULL: max|y| over the whole tensor
 * Otherwise as fln_norm_forward_fp8_rowwise.  No counterpart in the reference. */
int fln_norm_forward_mxfp8(int kind, const void* x, const void* residual, const void* gamma,
                           const void* beta, void* q, unsigned char* block_scale, void* sum_out,
                           float* mean, float* rstd, float* amax_out, int64_t rows, int64_t cols,
                           int io_dtype, float eps, void* stream);

/* ----------------------------------------------------------------------------------
 * Backward
 * -------------------------------------------------------------------------------- */

/* Bytes of scratch fln_*_backward needs for this problem on the current device
 * (per-CTA fp32 partial sums of dgamma/dbeta).  0 when rows == 0. */
size_t fln_backward_workspace_bytes(int64_t rows, int64_t cols, int dtype);

/* dx, dgamma, dbeta of LayerNorm from the saved per-row mean / rstd.
 *   xhat = (x - mean) * rstd, g = dy * gamma
 *   dx = rstd * (g - mean_j(g) - xhat * mean_j(g * xhat))
 *   dgamma = sum_i dy * xhat,  dbeta = sum_i dy      (fp32 accumulation, fixed order)
 * dx, dgamma, dbeta may each be NULL (that gradient is skipped); gamma may be NULL (== 1).
 * `workspace` must hold fln_backward_workspace_bytes() bytes whenever dgamma or dbeta is
 * requested.  Replaces layernorm_backward_cuda, which the reference declares
 * (csrc/layernorm.h:24-32, csrc/layernorm_cuda.cpp:33-41) and calls
 * (csrc/layernorm_cuda.cpp:135-138) but never defines. */
int fln_layernorm_backward(const void* dy, const void* x, const float* mean,
                           const float* rstd, const void* gamma, void* dx, void* dgamma,
                           void* dbeta, void* workspace, size_t workspace_bytes,
                           int64_t rows, int64_t cols, int dtype, void* stream);

/* General backward.
 *   kind      FLN_LAYERNORM or FLN_RMSNORM (mean, dbeta ignored / must be NULL)
 *   x         the tensor that was normalized (s = x + residual for the fused-add forward)
 *   dres_in   optional [rows, cols] gradient arriving on the residual stream; added to dx
 *   dgb_f32   optional fp32 [2*cols] buffer receiving [dgamma | dbeta] unrounded (the
 *             buffer a row-sharded job all-reduces); [cols] for FLN_RMSNORM
 * No counterpart in the reference. */
int fln_norm_backward(int kind, const void* dy, const void* x, const float* mean,
                      const float* rstd, const void* gamma, const void* dres_in, void* dx,
                      void* dgamma, void* dbeta, float* dgb_f32, void* workspace,
                      size_t workspace_bytes, int64_t rows, int64_t cols, int dtype,
                      void* stream);

/* Stage 1 of fln_norm_backward on its own: dx, and the per-CTA partial sums of dgamma / dbeta
 * left unreduced in `workspace` as an fp32 matrix [*partial_rows, NR * cols] (NR = 2 for
 * LayerNorm: dgamma sums then dbeta sums; 1 for RMSNorm), row pitch NR * cols.  The caller adds
 * the rows with fln_sum_rows_f32 when and where it likes -- typically on another stream, so
 * that the kernel after the backward does not wait for the column sums (they are needed at the
 * optimizer step, not before).  The kernel of this entry point ends without a grid-wide barrier,
 * so the next kernel's CTAs start while its last CTAs finish: 123 instead of 133 us per call at
 * 16384 x 8192 bf16, back to back.  The sums are added in a fixed order either way.
 * *partial_rows is 0 for rows == 0.  No counterpart in the reference (its backward is declared
 * in csrc/layernorm.h:24-32 and defined nowhere). */
int fln_norm_backward_partial(int kind, const void* dy, const void* x, const float* mean,
                              const float* rstd, const void* gamma, const void* dres_in, void* dx,
                              void* workspace, size_t workspace_bytes, int64_t rows, int64_t cols,
                              int dtype, void* stream, int64_t* partial_rows);

/* LayerNorm backward that allocates nothing and asks the caller for no scratch either.
 * It has no counterpart in the reference.  It exists for hosts that must not allocate device
 * memory once they are running: runtimes with a fixed memory plan (all device memory is
 * handed out at start-up), loops that cannot tolerate the device-wide synchronization of
 * cudaMalloc / cudaFree, plain C callers without a caching allocator.  Same arguments and
 * results as fln_layernorm_backward minus the workspace pair; the partial sums go to a
 * built-in __device__ array of FLN_STATIC_SCRATCH_BYTES that every GPU which loads the library
 * holds until the process exits.
 *   - Problems whose fln_backward_workspace_bytes() exceeds FLN_STATIC_SCRATCH_BYTES are
 *     refused with FLN_ERR_STATIC_SCRATCH and nothing is launched.
 *   - The first call made on a device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call outside any stream capture.
 *   - All calls share the one array and it keeps the last call's contents.  Nothing in it has
 *     to be zero beforehand (every partial row that is read is written first), but two calls
 *     that overlap on the GPU -- different streams, or graphs replayed concurrently -- race on
 *     it; serialize them.
 *   - It calls no cudaMalloc, cudaFree or allocating library routine. */
#define FLN_STATIC_SCRATCH_BYTES (24u << 20)
int fln_layernorm_backward_static(const void* dy, const void* x, const float* mean,
                                  const float* rstd, const void* gamma, void* dx, void* dgamma,
                                  void* dbeta, int64_t rows, int64_t cols, int dtype, void* stream);
/* Lowers the size beyond which fln_layernorm_backward_static refuses a problem (never above
 * FLN_STATIC_SCRATCH_BYTES; 0 restores that).  On a B200 no plan of the present launcher needs
 * more than 19.4 MB (148 SMs x 512 threads x 32 columns x 8 bytes), so the refusal can only be
 * seen by lowering the limit; tests do.  No counterpart in the reference. */
void fln_set_static_scratch_limit(size_t bytes);

/* dst[i] = (dtype) src[i] for n fp32 values: turns an all-reduced dgb_f32 buffer into
 * parameter-typed gradients.  No counterpart in the reference. */
int fln_cast_from_f32(const float* src, void* dst, int64_t n, int dtype, void* stream);

/* out[c] = sum over r of rows_in[r][c] for an fp32 matrix [n_rows, ncols] (row pitch ncols),
 * added in a fixed order (reproducible); written as fp32 (out_f32), rounded to `dtype`
 * (out_cast), or both.  It is stage 2 of the backward -- the fixed-order sum the reference's
 * backward declaration calls for (csrc/layernorm.h:24-32) -- opened to callers that hold several
 * [dgamma | dbeta] buffers of their own: one per micro-batch, or one per row chunk of a batch
 * that is streamed through the device. */
int fln_sum_rows_f32(const float* rows_in, int64_t n_rows, int64_t ncols, float* out_f32,
                     void* out_cast, int dtype, void* stream);

/* One-pass forward with NVFP4-style block-scaled 4-bit output (the second block-scaled input
 * format of Blackwell's tensor cores): e2m1 elements, one e4m3 scale per 16 consecutive
 * elements of a row, one fp32 scale S for the whole tensor, supplied by the caller (delayed
 * scaling: typically 448 * 6 / amax of the previous step; amax_out reports this call's max|y|).
 *   block_scale[r, c / 16] = e4m3(max|y| of the block * S / 6)      round to nearest even, saturating
 *   q element              = e2m1(y * S / float(block_scale))        round to nearest even, saturating at 6
 *   y ~ e2m1(q) * float(block_scale) / S
 *   q            [rows, cols / 2] bytes: element 2 i in the low nibble, 2 i + 1 in the high one
 *   block_scale  [rows, cols / 16] bytes (e4m3), required
 *   tensor_scale_in  one fp32 on the device, required
 * cols must be a multiple of 16; other rules as fln_norm_forward_fp8.  No counterpart in the
 * reference. */
int fln_norm_forward_nvfp4(int kind, const void* x, const void* residual, const void* gamma,
                           const void* beta, void* q, unsigned char* block_scale, void* sum_out,
                           float* mean, float* rstd, const float* tensor_scale_in, float* amax_out,
                           int64_t rows, int64_t cols, int io_dtype, float eps, void* stream);

/* Fused dropout -> residual add -> LayerNorm / RMSNorm forward: the step in front of the
 * normalization in a pre-norm block, in one pass.
 *   d = dropout(x, p): kept elements times 1 / (1 - p'), rounded to the I/O type
 *   s = d + residual (rounded to the I/O type, written to sum_out; residual may be NULL)
 *   y = norm(s) * gamma + beta        (same conventions as fln_norm_forward)
 * The mask comes from Philox4x32-10 and is a pure function of (seed, offset, element index):
 * one 128-bit output per group of 8 consecutive elements of the flattened matrix, 16 bits per
 * element, counter = {group lo, group hi, offset lo, offset hi}, key = {seed lo, seed hi}; an
 * element is kept iff its 16 bits >= round(p * 65536), so the drop probability is
 * p' = round(p * 65536) / 65536 and 0 <= p < 1.
 *   keep_bits  [rows * cols / 8] bytes or NULL: bit j of byte g = element 8 g + j was kept
 * cols must be a multiple of 8 and at most 16384, every pointer 16-byte aligned, otherwise
 * FLN_ERR_UNSUPPORTED.  The gradient of the block is fln_norm_backward on (dy, s) -- its dx is
 * the gradient of s and of the residual -- followed by fln_dropout_backward for x.
 * No counterpart in the reference. */
int fln_dropout_add_norm_forward(int kind, const void* x, const void* residual, const void* gamma,
                                 const void* beta, void* y, void* sum_out, float* mean, float* rstd,
                                 unsigned char* keep_bits, int64_t rows, int64_t cols, int dtype,
                                 float eps, float p, unsigned long long seed, unsigned long long offset,
                                 void* stream);

/* d_x = d_sum / (1 - p') where the element was kept, 0 where it was dropped.  The mask is read
 * from keep_bits (as fln_dropout_add_norm_forward wrote it) or, with keep_bits == NULL,
 * regenerated from (p, seed, offset).  d_x may be d_sum.  No counterpart in the reference. */
int fln_dropout_backward(const void* d_sum, const unsigned char* keep_bits, void* d_x, int64_t rows,
                         int64_t cols, int dtype, float p, unsigned long long seed,
                         unsigned long long offset, void* stream);

/* ----------------------------------------------------------------------------------
 * CUDA-graph launch path for latency-bound shapes
 * -------------------------------------------------------------------------------- */

/* Record any sequence of fln_* launches once and replay it with one graph launch.
 *   fln_graph_begin   creates a private stream and starts capturing on it
 *   fln_graph_stream  the stream to pass to the fln_* calls being recorded
 *   fln_graph_end     ends the capture and instantiates the graph
 *   fln_graph_launch  replays on `stream`; pointers and sizes are those recorded
 *   fln_graph_destroy releases everything (also valid after a failed end)
 * The reference launches eagerly on the legacy stream only
 * (csrc/layernorm_cuda_kernel.cu:171,199); it has no counterpart. */
typedef struct fln_graph fln_graph;
int fln_graph_begin(fln_graph** out);
void* fln_graph_stream(fln_graph* g);
int fln_graph_end(fln_graph* g);
int fln_graph_launch(fln_graph* g, void* stream);
int fln_graph_destroy(fln_graph* g);

/* ----------------------------------------------------------------------------------
 * Host-side helpers
 * -------------------------------------------------------------------------------- */

/* Closed-form byte estimate of a forward+backward call; same formula as
 * get_memory_usage (csrc/layernorm_cuda.cpp:144-164). */
int64_t fln_get_memory_usage(int batch_size, int hidden_size, int use_mixed_precision);

/* Writes newline-separated advisory text into buf (always NUL-terminated) and returns the
 * length that was needed.  Same messages as get_performance_hints
 * (csrc/layernorm_cuda.cpp:167-195) but the SM count is queried, not assumed. */
int fln_get_performance_hints(int batch_size, int hidden_size, char* buf, size_t buf_len);

/* How a forward / backward call of this shape is launched on the current device. */
typedef struct {
  int generic;       /* 1: looping fallback kernel (row too long or ragged for registers) */
  int vec_elems;     /* elements per vector load (1 = scalar path)                        */
  int vecs_per_thread;
  int threads_per_row;
  int threads_per_cta;
  int rows_per_cta;
  int64_t grid;      /* CTAs launched                                                     */
  int sm_count;
  int pipelined;     /* 1: the persistent bulk-async (TMA) pipeline serves this shape; the  */
                     /* fields above then describe its plan (a row count that is no        */
                     /* multiple of rows_per_cta: the plan of all but the last few rows,   */
                     /* which the register kernels take)                                   */
  int stages;        /* shared-memory stages of that pipeline (0 otherwise)                */
  int vector_bytes;  /* bytes per vector access: 16, or 8 / 4 in the odd-K plans           */
} fln_launch_info;
int fln_describe_launch(int backward, int64_t rows, int64_t cols, int dtype, int aligned16,
                        fln_launch_info* out);

/* Tuning hook: force vectors-per-thread (1,2,4,8) and threads-per-row (power of two,
 * 8..1024) for subsequent launches of this process; 0 restores automatic selection.
 * Combinations that cannot hold a row fall back to automatic selection. */
void fln_set_plan_override(int vecs_per_thread, int threads_per_row);

/* Tuning hook: which kernel family serves aligned problems.  0 = automatic (the persistent
 * bulk-async pipeline once every CTA streams several tiles, register-resident kernels
 * otherwise), 1 = register-resident kernels only, 2 = the pipeline whenever the row fits,
 * 3 = like 2 but dgamma / dbeta are reduced by a second kernel instead of in the tail of the
 * backward launch.  Query fln_backward_workspace_bytes again after changing it. */
void fln_set_path_override(int mode);

/* The persistent backward kernels size their grids to fill every SM exactly and split the rows
 * statically, so a kernel of somebody else that holds an SM while one of them launches (a
 * communication kernel overlapped with the step, for instance) delays the CTAs that could not
 * start, and with them the whole launch.  This leaves `sms` SMs out of those grids (default 0).
 * The persistent forward hands its tiles out on demand and always uses every SM.
 * Query fln_backward_workspace_bytes again after changing it.  No counterpart in the reference. */
void fln_set_sm_reserve(int sms);

/* Diagnostic, host only (no GPU needed): checks the launch planner of the pipelined kernels
 * over a grid of shapes and returns the number of plans that violate its invariants (0 = fine).
 * No counterpart in the reference. */
int fln_planner_selftest(void);

/* Tuning hook: stages (tiles in flight) per CTA of the pipelined kernels; 0 = automatic (about
 * 96 KB in flight per SM), >= 2 forces that many where they fit.  Query
 * fln_backward_workspace_bytes again after changing it.  No counterpart in the reference. */
void fln_set_stage_override(int stages);

/* Reads and clears the device status word of the current device (synchronizes the device).
 * 0 = no kernel reported a problem; otherwise a sum of
 *   1  a pipelined kernel gave up waiting for a bulk copy (its outputs are incomplete),
 *   2  the backward's grid barrier gave up waiting for the other CTAs (dgamma / dbeta of that
 *      launch are stale; dx is complete),
 *   4  the forward's tile counter did not add up at the end of a launch (two launches shared a
 *      counter pair: more than 1024 pipelined forward launches in flight at once);
 * -1 = the status could not be read.  Every exit path of the kernels -- the ones that gave up
 * included -- leaves the grid barrier's word and the tile counter ready for the next launch or
 * graph replay.  The reference has no error reporting on its launch path
 * (csrc/layernorm_cuda_kernel.cu:171,199). */
int fln_device_status(void);

/* Every wait inside a kernel (for a bulk copy, at the grid barrier) gives up after about this
 * many nanoseconds (counted in SM cycles at 2 per nanosecond, so up to 1.5 times longer at low
 * clocks) and reports through fln_device_status().  Default 1e9 (one second; 0 restores it).
 * Process-wide; launches recorded into a CUDA graph keep the limit they were recorded with.
 * Tests lower it to make a wait run out quickly.  No counterpart in the reference. */
int fln_set_wait_limit_ns(unsigned long long ns);

/* Test hook, off by default, current device: bit 0 -- CTA 0 of a pipelined kernel arms the
 * barrier of its first tile without issuing the copy, so its wait runs out (status 1);
 * bit 1 -- the backward's grid barrier expects one CTA more than the grid has, so every CTA's
 * wait runs out (status 2).  Nothing faults and nothing spins without bound: the kernels
 * return through their ordinary give-up paths.  No counterpart in the reference. */
int fln_set_test_fault(int bits);

#ifdef __cplusplus
}
#endif
#endif /* FLN_B200_H */
