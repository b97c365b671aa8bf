/*
 * fln_oracle.c -- CPU restatement of the reference's normalization path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product imports, links or runs this file; it is
 * the checker used by tests/, by __graft_entry__.smoke() and by the cpu_baseline leg of
 * bench.py.  Plain C, no dependencies, built by oracle/Makefile into
 * oracle/_build/libfln_oracle.so and called through ctypes (oracle/oracle.py).
 *
 * Reference = JonSnow1807/Fused-LayerNorm-CUDA-Operator; paths below are relative to its root.
 *
 * Two flavours are provided:
 *  (1) oracle_*   the algorithm of the reference (two-pass mean / variance, rsqrt, affine,
 *                 optional GELU) evaluated with double accumulators, so that it is a
 *                 "truth" the fp32 kernels can be compared against at the stated tolerances
 *                 (1e-5 abs/rel fp32, 1 ulp bf16, 1 code step fp8).
 *  (2) ref_g2_*   a literal restatement of the shipped CUDA kernel, including its fp32
 *                 accumulators and the order in which its threads, warps and the block add
 *                 their partial sums.  It is what gets pinned against outputs of the real
 *                 reference kernel run on a B200 (tests/golden/ref_g2_b200.npz).
 *
 * Parity pins: tests/test_oracle_golden.py checks (1) against fixtures generated from
 * torch's CPU layer_norm / native_layer_norm_backward / rms_norm / gelu / float8 cast (the
 * semantic oracle the reference's own tests use, tests/test_layernorm.py:47-178) and (2)
 * against the reference kernel's own outputs.
 */
#define _GNU_SOURCE
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

enum { T_F32 = 0, T_BF16 = 1, T_F16 = 2 };
enum { KIND_LN = 0, KIND_RMS = 1 };
enum { ACT_NONE = 0, ACT_GELU_TANH = 1, ACT_GELU_ERF = 2 };

/* ------------------------------------------------------------------ scalar conversions */
static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static float bf16_to_f(uint16_t h) { return u2f((uint32_t)h << 16); }
static uint16_t f_to_bf16(float f) { /* round to nearest even */
  uint32_t u = f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}
static float f16_to_f(uint16_t h) {
  uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
  if (e == 0) {
    if (m == 0) return u2f(s);
    float v = ldexpf((float)m, -24);
    return s ? -v : v;
  }
  if (e == 31) return u2f(s | 0x7f800000u | (m << 13));
  return u2f(s | ((e + 112u) << 23) | (m << 13));
}
static uint16_t f_to_f16(float f) { /* round to nearest even, overflow -> inf */
  uint32_t u = f2u(f), s = (u >> 16) & 0x8000u;
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(s | 0x7e00u);
  if (a >= 0x47800000u) return (uint16_t)(s | 0x7c00u); /* >= 65536 -> inf (65520 rounds up below) */
  if (a < 0x33000000u) return (uint16_t)s;              /* < 2^-25 -> 0 */
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u;
  int shift = e >= -14 ? 13 : (13 + (-14 - e));
  uint32_t q = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) q++;
  uint32_t he = e >= -14 ? (uint32_t)(e + 15) : 0u;
  /* q carries the implicit bit when normal */
  uint32_t out = e >= -14 ? ((he << 10) + (q - 0x400u)) : q;
  if (out >= 0x7c00u) out = 0x7c00u;
  return (uint16_t)(s | out);
}
/* fp8 e4m3fn (bias 7, 3 mantissa bits, max 448, subnormal step 2^-9), saturating,
 * round to nearest even; NaN -> 0x7f | sign */
static uint8_t f_to_e4m3_sat(float f) {
  uint32_t u = f2u(f);
  uint8_t s = (uint8_t)((u >> 24) & 0x80u);
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint8_t)(s | 0x7f);
  float x = u2f(a);
  if (x >= 448.0f) return (uint8_t)(s | 0x7e);
  if (x == 0.0f) return s;
  int e;
  frexpf(x, &e);                      /* x = m 2^e, m in [0.5,1): leading bit has weight 2^(e-1) */
  int le = e - 1 < -6 ? -6 : e - 1;   /* subnormals share the spacing of the binade of 2^-6 */
  float ulp = ldexpf(1.0f, le - 3);
  float v = nearbyintf(x / ulp) * ulp; /* both scalings exact; default mode = nearest even */
  if (v == 0.0f) return s;
  frexpf(v, &e);
  le = e - 1;
  if (le < -6) return (uint8_t)(s | (uint32_t)(v / ldexpf(1.0f, -9)));
  uint32_t m = (uint32_t)(v / ldexpf(1.0f, le - 3)) - 8u;
  return (uint8_t)(s | ((uint32_t)(le + 7) << 3) | m);
}

static double load_el(const void* p, int64_t i, int dt) {
  switch (dt) {
    case T_F32: return (double)((const float*)p)[i];
    case T_BF16: return (double)bf16_to_f(((const uint16_t*)p)[i]);
    default: return (double)f16_to_f(((const uint16_t*)p)[i]);
  }
}
static float round_to(float v, int dt) { /* value after a round trip through dt */
  switch (dt) {
    case T_F32: return v;
    case T_BF16: return bf16_to_f(f_to_bf16(v));
    default: return f16_to_f(f_to_f16(v));
  }
}
static void store_el(void* p, int64_t i, int dt, float v) {
  switch (dt) {
    case T_F32: ((float*)p)[i] = v; break;
    case T_BF16: ((uint16_t*)p)[i] = f_to_bf16(v); break;
    default: ((uint16_t*)p)[i] = f_to_f16(v); break;
  }
}

API void oracle_convert_from_f32(const float* src, void* dst, int64_t n, int dt) {
  for (int64_t i = 0; i < n; ++i) store_el(dst, i, dt, src[i]);
}
API void oracle_convert_to_f32(const void* src, float* dst, int64_t n, int dt) {
  for (int64_t i = 0; i < n; ++i) dst[i] = (float)load_el(src, i, dt);
}
API void oracle_e4m3_encode(const float* src, uint8_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = f_to_e4m3_sat(src[i]);
}

/* GELU, tanh form: the reference's gelu() (csrc/layernorm_cuda_kernel.cu:31-36). */
static double gelu_tanh(double v) {
  const double s = sqrt(2.0 / M_PI), a = 0.044715;
  return 0.5 * v * (1.0 + tanh(s * (v + a * v * v * v)));
}
/* GELU, exact form (what torch's default F.gelu computes). */
static double gelu_erf(double v) { return 0.5 * v * (1.0 + erf(v * M_SQRT1_2)); }

/* ------------------------------------------------------------------ (1) truth oracle */

/*
 * Forward.  Follows layernorm_kernel (csrc/layernorm_cuda_kernel.cu:39-92): mean
 * (:58-67), variance about the mean (:70-81), normalize + affine (:85-91), optional GELU
 * (layernorm_gelu_kernel :141-147); mean/rstd outputs as layernorm_forward_kernel_optimized
 * writes them (csrc/layernorm_cuda_kernel_optimized.cu:119-122).  gamma and beta are
 * applied independently when present.  With residual != NULL, s = x + residual is first
 * rounded to io_dt (what an unfused add produces) and written to sum_out.
 * y32 (optional) receives the fp32 value before the final rounding to out_dt.
 */
API void oracle_norm_forward(int kind, const void* x, const void* residual, const void* gamma,
                             const void* beta, void* y, float* y32, void* sum_out, float* mean,
                             float* rstd, int64_t rows, int64_t cols, int io_dt, int out_dt,
                             double eps, int act) {
  double* s = (double*)malloc(sizeof(double) * (size_t)cols);
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t base = r * cols;
    for (int64_t j = 0; j < cols; ++j) {
      double v = load_el(x, base + j, io_dt);
      if (residual) {
        float sum = round_to((float)(v + load_el(residual, base + j, io_dt)), io_dt);
        if (sum_out) store_el(sum_out, base + j, io_dt, sum);
        v = (double)sum;
      }
      s[j] = v;
    }
    double mu = 0.0, var = 0.0;
    if (kind == KIND_LN) {
      for (int64_t j = 0; j < cols; ++j) mu += s[j];
      mu /= (double)cols;
      for (int64_t j = 0; j < cols; ++j) var += (s[j] - mu) * (s[j] - mu);
    } else {
      for (int64_t j = 0; j < cols; ++j) var += s[j] * s[j];
    }
    var /= (double)cols;
    const double rs = 1.0 / sqrt(var + eps);
    if (mean && kind == KIND_LN) mean[r] = (float)mu;
    if (rstd) rstd[r] = (float)rs;
    for (int64_t j = 0; j < cols; ++j) {
      double v = (s[j] - mu) * rs;
      if (gamma) v *= load_el(gamma, j, io_dt);
      if (beta) v += load_el(beta, j, io_dt);
      if (act == ACT_GELU_TANH) v = gelu_tanh(v);
      else if (act == ACT_GELU_ERF) v = gelu_erf(v);
      if (y32) y32[base + j] = (float)v;
      if (y) store_el(y, base + j, out_dt, (float)v);
    }
  }
  free(s);
}

/*
 * Backward from saved statistics.  The reference declares this operation
 * (csrc/layernorm.h:24-32; argument list csrc/layernorm_cuda.cpp:97-141) without a kernel;
 * the math is the derivative of the forward above, which is what its tests check against
 * torch autograd (tests/test_layernorm.py:128-178):
 *   xhat = (x - mean) rstd, g = dy gamma,
 *   dx = rstd (g - mean_j g - xhat mean_j(g xhat)) [+ dres_in], dgamma = sum_i dy xhat,
 *   dbeta = sum_i dy.   RMSNorm: mean = 0 and the mean_j g term is absent.
 * dgamma64/dbeta64 (optional, [cols]) receive the double sums; abs64 (optional, [2*cols])
 * receives sum_i |dy xhat| and sum_i |dy|, the scale against which a cancelling sum has to
 * be judged.
 */
API void oracle_norm_backward(int kind, const void* dy, const void* x, const float* mean,
                              const float* rstd, const void* gamma, const void* dres_in,
                              void* dx, float* dx32, void* dgamma, void* dbeta, double* dgamma64,
                              double* dbeta64, double* abs64, int64_t rows, int64_t cols, int dt) {
  double* ag = (double*)calloc((size_t)cols, sizeof(double));
  double* ab = (double*)calloc((size_t)cols, sizeof(double));
  double* aag = (double*)calloc((size_t)cols, sizeof(double));
  double* aab = (double*)calloc((size_t)cols, sizeof(double));
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t base = r * cols;
    const double mu = kind == KIND_LN ? (double)mean[r] : 0.0, rs = (double)rstd[r];
    double s1 = 0.0, s2 = 0.0;
    for (int64_t j = 0; j < cols; ++j) {
      double d = load_el(dy, base + j, dt);
      double g = d * (gamma ? load_el(gamma, j, dt) : 1.0);
      double xh = (load_el(x, base + j, dt) - mu) * rs;
      s1 += g * xh;
      s2 += g;
      ag[j] += d * xh;
      ab[j] += d;
      aag[j] += fabs(d * xh);
      aab[j] += fabs(d);
    }
    const double c1 = s1 / (double)cols, c2 = kind == KIND_LN ? s2 / (double)cols : 0.0;
    if (dx || dx32) {
      for (int64_t j = 0; j < cols; ++j) {
        double d = load_el(dy, base + j, dt);
        double g = d * (gamma ? load_el(gamma, j, dt) : 1.0);
        double xh = (load_el(x, base + j, dt) - mu) * rs;
        double o = rs * (g - c2 - xh * c1);
        if (dres_in) o += load_el(dres_in, base + j, dt);
        if (dx32) dx32[base + j] = (float)o;
        if (dx) store_el(dx, base + j, dt, (float)o);
      }
    }
  }
  for (int64_t j = 0; j < cols; ++j) {
    if (dgamma) store_el(dgamma, j, dt, (float)ag[j]);
    if (dbeta && kind == KIND_LN) store_el(dbeta, j, dt, (float)ab[j]);
    if (dgamma64) dgamma64[j] = ag[j];
    if (dbeta64) dbeta64[j] = ab[j];
    if (abs64) { abs64[j] = aag[j]; abs64[cols + j] = aab[j]; }
  }
  free(ag); free(ab); free(aag); free(aab);
}

/*
 * Per-tensor fp8 quantization of an fp32 tensor: amax = max |y|, scale = 448 / amax in fp32
 * (1 when amax == 0), q = e4m3(sat(y * scale)).  No counterpart in the reference; this is
 * the torch composition y.abs().max(), 448/amax, (y*scale).to(float8_e4m3fn).
 */
API void oracle_quant_fp8(const float* y32, int64_t n, float* amax_out, float* scale_out, uint8_t* q) {
  float amax = 0.0f;
  for (int64_t i = 0; i < n; ++i) { float a = fabsf(y32[i]); if (a > amax) amax = a; }
  float scale = amax > 0.0f ? 448.0f / amax : 1.0f;
  if (amax_out) *amax_out = amax;
  if (scale_out) *scale_out = scale;
  if (q) for (int64_t i = 0; i < n; ++i) q[i] = f_to_e4m3_sat(y32[i] * scale);
}

/* ------------------------------------------------------------------ (2) literal G2 restatement */

/* warpReduceSum (csrc/layernorm_cuda_kernel.cu:7-12): xor-butterfly over 32 lanes; every
 * lane ends with the same value because fp32 addition is commutative. */
static void warp_reduce(float* v /*32*/) {
  for (int mask = 16; mask > 0; mask >>= 1) {
    float t[32];
    for (int l = 0; l < 32; ++l) t[l] = v[l] + v[l ^ mask];
    memcpy(v, t, sizeof(t));
  }
}
/* blockReduceSum (csrc/layernorm_cuda_kernel.cu:14-28): per-warp butterfly, lane 0 of each
 * warp to shared memory, then warp 0 reduces the per-warp values (missing warps = 0). */
static float block_reduce(const float* part, int threads) {
  float shared[32];
  int nw = threads / 32;
  for (int w = 0; w < nw; ++w) {
    float v[32];
    memcpy(v, part + w * 32, sizeof(v));
    warp_reduce(v);
    shared[w] = v[0];
  }
  float v[32];
  for (int l = 0; l < 32; ++l) v[l] = l < nw ? shared[l] : 0.0f;
  warp_reduce(v);
  return v[0];
}

/*
 * layernorm_kernel<float> / layernorm_gelu_kernel<float> as shipped
 * (csrc/layernorm_cuda_kernel.cu:39-92, 95-148) with the launcher's block size
 * (:163-165): fp32 everywhere, thread t sums elements t, t+T, ...; `diff*diff` is
 * accumulated with a fused multiply-add, as nvcc contracts it; the affine is applied only
 * when both gamma and beta are given (:87).  rsqrtf is evaluated as 1/sqrt in fp32 (the
 * device intrinsic may differ from that by 2 ulp).
 */
API void ref_g2_layernorm_f32(const float* x, const float* gamma, const float* beta, float* y,
                              int64_t rows, int N, float eps, int gelu) {
  int threads = 256;
  if (N >= 1024) threads = 512;
  if (N >= 4096) threads = 1024;
  float part[1024];
  const float sc = sqrtf(2.0f / (float)M_PI), a = 0.044715f;
  for (int64_t r = 0; r < rows; ++r) {
    const float* X = x + r * (int64_t)N;
    float* Y = y + r * (int64_t)N;
    for (int t = 0; t < threads; ++t) {
      float s = 0.0f;
      for (int i = t; i < N; i += threads) s += X[i];
      part[t] = s;
    }
    const float mean = block_reduce(part, threads) / (float)N;
    for (int t = 0; t < threads; ++t) {
      float s = 0.0f;
      for (int i = t; i < N; i += threads) { float d = X[i] - mean; s = fmaf(d, d, s); }
      part[t] = s;
    }
    const float rstd = 1.0f / sqrtf(block_reduce(part, threads) / (float)N + eps);
    for (int i = 0; i < N; ++i) {
      float v = (X[i] - mean) * rstd;
      if (gamma && beta) v = fmaf(v, gamma[i], beta[i]);
      if (gelu) {
        float v3 = v * v * v;
        v = 0.5f * v * (1.0f + tanhf(sc * (v + a * v3)));
      }
      Y[i] = v;
    }
  }
}

/* ------------------------------------------------------------------ dropout (counter-based) */

/*
 * Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3",
 * SC'11), restated from the published algorithm: ten rounds of
 *   (hi0, lo0) = M0 * c0, (hi1, lo1) = M1 * c2,  c' = {hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0}
 * with the key bumped by the Weyl constants after every round.  The reference project has no
 * dropout; this is the generator behind fln_dropout_add_norm_forward, pinned by the published
 * known-answer vectors in tests/test_oracle_golden.py.
 */
API void oracle_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
  uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3], k0 = key[0], k1 = key[1];
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1, n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1,
                   n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* keep bits of `groups` groups of 8 elements: group g uses counter {g lo, g hi, offset lo,
 * offset hi}, key {seed lo, seed hi}; element j keeps iff its 16 bits (word j / 2, half j % 2)
 * are >= threshold. */
API void oracle_dropout_keep_bits(uint64_t seed, uint64_t offset, uint32_t threshold, int64_t groups, uint8_t* bits) {
  const uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
  for (int64_t g = 0; g < groups; ++g) {
    const uint32_t ctr[4] = {(uint32_t)g, (uint32_t)((uint64_t)g >> 32), (uint32_t)offset, (uint32_t)(offset >> 32)};
    uint32_t w[4];
    oracle_philox4x32_10(ctr, key, w);
    uint8_t m = 0;
    for (int j = 0; j < 8; ++j) {
      const uint32_t v = (w[j >> 1] >> (16 * (j & 1))) & 0xffffu;
      if (threshold == 0 || v >= threshold) m |= (uint8_t)(1u << j);
    }
    bits[g] = m;
  }
}

/* out[i] = round_to_dt(x[i] * scale) where bit i is set, 0 elsewhere (forward and backward of
 * dropout are the same map) */
API void oracle_dropout_apply(const void* x, const uint8_t* bits, void* out, int64_t n, int dt, float scale) {
  for (int64_t i = 0; i < n; ++i) {
    const int keep = (bits[i >> 3] >> (i & 7)) & 1;
    store_el(out, i, dt, keep ? (float)load_el(x, i, dt) * scale : 0.0f);
  }
}

/* ------------------------------------------------------------------ NVFP4-style quantizer */

/* e4m3 code -> value (finite codes) */
static float e4m3_to_f(uint8_t c) {
  const int sign = c >> 7, e = (c >> 3) & 15, m = c & 7;
  const float v = e == 0 ? ldexpf((float)m, -9) : ldexpf((float)(8 + m), e - 10);
  return sign ? -v : v;
}
/* e2m1: magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6 (codes 0..7), sign in bit 3; round to nearest,
 * ties to the even code, saturating at 6; NaN gives +6 like the hardware conversion. */
static uint8_t f_to_e2m1_sat(float v) {
  static const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  if (v != v) return 7;
  const uint8_t sign = signbit(v) ? 8 : 0;
  const float a = fabsf(v);
  int code = 7;
  for (int c = 0; c < 7; ++c) {
    const float mid = 0.5f * (mag[c] + mag[c + 1]);
    if (a < mid || (a == mid && (c & 1) == 0)) { code = c; break; }
  }
  return (uint8_t)(sign | code);
}
API float oracle_e2m1_decode(uint8_t c) {
  static const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  return (c & 8) ? -mag[c & 7] : mag[c & 7];
}
API float oracle_e4m3_decode(uint8_t c) { return e4m3_to_f(c); }

/*
 * y32 [rows, cols] -> q [rows, cols / 2] (element 2 i in the low nibble), block_scale
 * [rows, cols / 16] e4m3.  tensor scale S (fp32):  b = e4m3(block max * S / 6),
 * q = e2m1(y * (S / float(b))), all in fp32 with one rounding per operation, as
 * fln_norm_forward_nvfp4 states it.  With scales_in != NULL those block scales are used
 * instead of being derived (and copied to block_scale).
 */
API void oracle_quant_nvfp4(const float* y32, int64_t rows, int64_t cols, float S, const uint8_t* scales_in,
                            uint8_t* q, uint8_t* block_scale) {
  const int64_t nb = cols / 16;
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t b = 0; b < nb; ++b) {
      const float* y = y32 + r * cols + b * 16;
      float bm = 0.f;
      for (int i = 0; i < 16; ++i) bm = fmaxf(bm, fabsf(y[i]));
      uint8_t sb;
      if (scales_in) {
        sb = scales_in[r * nb + b];
      } else {
        volatile float t = bm * S;
        volatile float d = t * (1.0f / 6.0f);
        sb = f_to_e4m3_sat(d);
      }
      block_scale[r * nb + b] = sb;
      const float fb = e4m3_to_f(sb);
      const float inv = fb > 0.f ? S / fb : 0.f;
      for (int i = 0; i < 16; i += 2) {
        volatile float a0 = y[i] * inv, a1 = y[i + 1] * inv;
        q[(r * cols + b * 16 + i) / 2] = (uint8_t)(f_to_e2m1_sat(a0) | (f_to_e2m1_sat(a1) << 4));
      }
    }
  }
}
