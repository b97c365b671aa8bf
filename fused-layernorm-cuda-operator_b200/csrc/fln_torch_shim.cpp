// fused_layernorm_cuda: thin PyTorch extension over the C ABI of libfln_b200.so.
//
// It does three things and no arithmetic: validate tensors (device, layout, dtype, shapes),
// allocate outputs / scratch through torch's caching allocator, and launch on torch's
// current stream of the input's device.  Everything is exported twice:
//   * as torch.library operators  fused_layernorm::*  (schemas below; CUDA implementations
//     here, fake and autograd registrations in fused_layernorm/ops.py) so that torch.compile
//     can trace them;
//   * as plain pybind functions with the reference's names and argument names:
//     layernorm / layernorm_gelu (csrc/bindings.cpp:19-44 of the reference) and forward /
//     backward / get_memory_usage / get_performance_hints / __version__ / __cuda_version__
//     (csrc/layernorm_cuda.cpp:49-238 of the reference).
// Error behaviour follows the reference's intended one (csrc/layernorm_cuda.cpp:44-46,56-71):
// TORCH_CHECK -> RuntimeError; unsupported dtypes -> NotImplementedError like its
// AT_DISPATCH macro.  There is no CPU path.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/EmptyTensor.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/autograd.h>
#include <torch/extension.h>
#include <torch/library.h>

#include <array>
#include <optional>
#include <string>
#include <tuple>
#include <vector>

#include "fln_b200.h"

namespace {

using at::Tensor;
using OptTensor = std::optional<Tensor>;

int dtype_code(const Tensor& t, const char* op) {
  switch (t.scalar_type()) {
    case at::kFloat:
      return FLN_F32;
    case at::kBFloat16:
      return FLN_BF16;
    case at::kHalf:
      return FLN_F16;
    default:
      TORCH_CHECK_NOT_IMPLEMENTED(false, "\"", op, "\" not implemented for '", toString(t.scalar_type()), "'");
  }
  return -1;
}

void check_status(int st, const char* what) {
  TORCH_CHECK(st == FLN_OK, what, ": ", fln_status_string(st), " (status ", st, ")");
}

// input must be a CUDA matrix; returns it contiguous
Tensor check_matrix(const Tensor& t, const char* name) {
  TORCH_CHECK(t.device().is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.dim() == 2, "Input must be 2D (batch_size, hidden_size)");
  return t.contiguous();
}

// optional [cols] parameter on the same device and of the same dtype as x
const void* param_ptr(const OptTensor& p, const Tensor& x, const char* name, Tensor& keep) {
  if (!p.has_value() || !p->defined()) return nullptr;
  TORCH_CHECK(p->device().is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(p->device() == x.device(), name, " and input must be on the same device");
  TORCH_CHECK(p->dim() == 1, name, " must be 1D");
  TORCH_CHECK(p->size(0) == x.size(1), name, " size must match hidden dimension");
  TORCH_CHECK(p->scalar_type() == x.scalar_type(), name, " and input must have the same dtype");
  keep = p->contiguous();
  return keep.data_ptr();
}

Tensor check_like(const Tensor& t, const Tensor& x, const char* name) {
  TORCH_CHECK(t.device() == x.device(), name, " and input must be on the same device");
  TORCH_CHECK(t.sizes() == x.sizes(), name, " shape must match input shape");
  TORCH_CHECK(t.scalar_type() == x.scalar_type(), name, " and input must have the same dtype");
  return t.contiguous();
}

Tensor check_stat(const Tensor& t, const Tensor& x, const char* name) {
  TORCH_CHECK(t.device() == x.device(), name, " and input must be on the same device");
  TORCH_CHECK(t.scalar_type() == at::kFloat, name, " must be float32");
  TORCH_CHECK(t.numel() == x.size(0), name, " must have one entry per row");
  return t.contiguous();
}

// Outputs and scratch straight from the caching allocator.  (at::empty / at::empty_like go
// through the dispatcher first: 1.27 instead of 0.87 us per tensor, a tenth of a whole call at
// the latency-bound shapes.)
Tensor new_cuda(at::IntArrayRef sizes, at::ScalarType dtype, const Tensor& on_device_of) {
  return Tensor(at::detail::empty_cuda(sizes, dtype, on_device_of.device(), std::nullopt));
}
Tensor new_like(const Tensor& x) { return new_cuda(x.sizes(), x.scalar_type(), x); }

// makes x's device current for the launch; nothing to undo in the usual case that it already is
struct DeviceOf {
  std::optional<c10::cuda::CUDAGuard> guard;
  explicit DeviceOf(const Tensor& x) {
    if (c10::cuda::current_device() != x.device().index()) guard.emplace(x.device());
  }
};

void* stream_of(const Tensor& x) { return at::cuda::getCurrentCUDAStream(x.get_device()).stream(); }

int act_code(const std::string& approximate) {
  if (approximate == "tanh") return FLN_ACT_GELU_TANH;
  if (approximate == "none" || approximate == "erf") return FLN_ACT_GELU_ERF;
  TORCH_CHECK(false, "approximate must be 'tanh' or 'none', got '", approximate, "'");
  return 0;
}

// ---------------------------------------------------------------------------------------
// forward family
// ---------------------------------------------------------------------------------------
struct FwdOut {
  Tensor y, sum, mean, rstd;
};

FwdOut norm_forward(int kind, const Tensor& input, const OptTensor& residual, const OptTensor& gamma,
                    const OptTensor& beta, double eps, int act, bool want_stats, const char* op) {
  Tensor x = check_matrix(input, "input");
  const int dt = dtype_code(x, op);
  DeviceOf guard(x);
  Tensor gk, bk, rk;
  const void* g = param_ptr(gamma, x, "Gamma", gk);
  const void* b = param_ptr(beta, x, "Beta", bk);
  FwdOut o;
  const void* r = nullptr;
  void* s = nullptr;
  if (residual.has_value() && residual->defined()) {
    rk = check_like(*residual, x, "residual");
    r = rk.data_ptr();
    o.sum = new_like(x);
    s = o.sum.data_ptr();
  }
  o.y = new_like(x);
  float* mean = nullptr;
  float* rstd = nullptr;
  if (want_stats) {
    if (kind == FLN_LAYERNORM) {
      o.mean = new_cuda({x.size(0)}, at::kFloat, x);
      mean = o.mean.data_ptr<float>();
    }
    o.rstd = new_cuda({x.size(0)}, at::kFloat, x);
    rstd = o.rstd.data_ptr<float>();
  }
  check_status(fln_norm_forward(kind, x.data_ptr(), r, g, b, o.y.data_ptr(), s, mean, rstd, x.size(0), x.size(1), dt,
                                dt, (float)eps, act, stream_of(x)),
               op);
  return o;
}

// G2 entry points (reference csrc/bindings.cpp:19-39): output only
Tensor layernorm(const Tensor& input, const OptTensor& gamma, const OptTensor& beta, double epsilon) {
  return norm_forward(FLN_LAYERNORM, input, std::nullopt, gamma, beta, epsilon, FLN_ACT_NONE, false, "layernorm").y;
}
Tensor layernorm_gelu(const Tensor& input, const OptTensor& gamma, const OptTensor& beta, double epsilon,
                      std::string approximate) {
  return norm_forward(FLN_LAYERNORM, input, std::nullopt, gamma, beta, epsilon, act_code(approximate), false,
                      "layernorm_gelu")
      .y;
}
// G1 forward (reference csrc/layernorm_cuda.cpp:49-94): [output, mean, rstd]
std::tuple<Tensor, Tensor, Tensor> layernorm_fwd(const Tensor& input, const OptTensor& gamma, const OptTensor& beta,
                                                 double epsilon) {
  FwdOut o = norm_forward(FLN_LAYERNORM, input, std::nullopt, gamma, beta, epsilon, FLN_ACT_NONE, true, "layernorm");
  return {o.y, o.mean, o.rstd};
}
std::tuple<Tensor, Tensor> rmsnorm_fwd(const Tensor& input, const OptTensor& gamma, double epsilon) {
  FwdOut o = norm_forward(FLN_RMSNORM, input, std::nullopt, gamma, std::nullopt, epsilon, FLN_ACT_NONE, true, "rmsnorm");
  return {o.y, o.rstd};
}
std::tuple<Tensor, Tensor, Tensor, Tensor> add_layernorm_fwd(const Tensor& input, const Tensor& residual,
                                                             const OptTensor& gamma, const OptTensor& beta,
                                                             double epsilon) {
  FwdOut o = norm_forward(FLN_LAYERNORM, input, residual, gamma, beta, epsilon, FLN_ACT_NONE, true, "add_layernorm");
  return {o.y, o.sum, o.mean, o.rstd};
}
std::tuple<Tensor, Tensor, Tensor> add_rmsnorm_fwd(const Tensor& input, const Tensor& residual, const OptTensor& gamma,
                                                   double epsilon) {
  FwdOut o = norm_forward(FLN_RMSNORM, input, residual, gamma, std::nullopt, epsilon, FLN_ACT_NONE, true, "add_rmsnorm");
  return {o.y, o.sum, o.rstd};
}

// fp8-e4m3 output with a per-tensor scale computed on the device: (q, sum, scale, mean, rstd)
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> norm_fp8(int64_t kind, const Tensor& input, const OptTensor& residual,
                                                            const OptTensor& gamma, const OptTensor& beta,
                                                            double epsilon) {
  TORCH_CHECK(kind == FLN_LAYERNORM || kind == FLN_RMSNORM, "kind must be 0 (layernorm) or 1 (rmsnorm)");
  Tensor x = check_matrix(input, "input");
  const int dt = dtype_code(x, "norm_fp8");
  DeviceOf guard(x);
  Tensor gk, bk, rk, sum, mean;
  const void* g = param_ptr(gamma, x, "Gamma", gk);
  const void* b = param_ptr(beta, x, "Beta", bk);
  TORCH_CHECK(!(kind == FLN_RMSNORM && b != nullptr), "rmsnorm takes no beta");
  const void* r = nullptr;
  void* s = nullptr;
  if (residual.has_value() && residual->defined()) {
    rk = check_like(*residual, x, "residual");
    r = rk.data_ptr();
    sum = new_like(x);
    s = sum.data_ptr();
  } else {
    sum = new_cuda({0}, x.scalar_type(), x);
  }
  Tensor q = new_cuda(x.sizes(), at::kFloat8_e4m3fn, x);
  Tensor rstd = new_cuda({x.size(0)}, at::kFloat, x);
  mean = kind == FLN_LAYERNORM ? new_cuda({x.size(0)}, at::kFloat, x) : new_cuda({0}, at::kFloat, x);
  Tensor amax_scale = new_cuda({2}, at::kFloat, x);
  float* as = amax_scale.data_ptr<float>();
  check_status(fln_norm_forward_fp8((int)kind, x.data_ptr(), r, g, b, q.data_ptr(), s,
                                    kind == FLN_LAYERNORM ? mean.data_ptr<float>() : nullptr, rstd.data_ptr<float>(), as,
                                    as + 1, x.size(0), x.size(1), dt, (float)epsilon, stream_of(x)),
               "norm_fp8");
  return {q, sum, amax_scale.slice(0, 1, 2), mean, rstd};
}

// One-pass fp8-e4m3 output: with `scale_in` (one fp32) the caller's scale is used (delayed
// scaling), without it every row gets its own scale.  Returns (q, sum, row_scale, amax);
// row_scale is empty in the delayed form, amax is max|y| of this call in both.
std::tuple<Tensor, Tensor, Tensor, Tensor> norm_fp8_scaled(int64_t kind, const Tensor& input, const OptTensor& residual,
                                                           const OptTensor& gamma, const OptTensor& beta,
                                                           const OptTensor& scale_in, double epsilon) {
  TORCH_CHECK(kind == FLN_LAYERNORM || kind == FLN_RMSNORM, "kind must be 0 (layernorm) or 1 (rmsnorm)");
  Tensor x = check_matrix(input, "input");
  const int dt = dtype_code(x, "norm_fp8_scaled");
  DeviceOf guard(x);
  Tensor gk, bk, rk, sum, sk;
  const void* g = param_ptr(gamma, x, "Gamma", gk);
  const void* b = param_ptr(beta, x, "Beta", bk);
  TORCH_CHECK(!(kind == FLN_RMSNORM && b != nullptr), "rmsnorm takes no beta");
  const void* r = nullptr;
  void* s = nullptr;
  if (residual.has_value() && residual->defined()) {
    rk = check_like(*residual, x, "residual");
    r = rk.data_ptr();
    sum = new_like(x);
    s = sum.data_ptr();
  } else {
    sum = new_cuda({0}, x.scalar_type(), x);
  }
  Tensor q = new_cuda(x.sizes(), at::kFloat8_e4m3fn, x);
  Tensor amax = new_cuda({1}, at::kFloat, x);
  const bool delayed = scale_in.has_value() && scale_in->defined();
  if (delayed) {
    TORCH_CHECK(scale_in->is_cuda() && scale_in->device() == x.device() && scale_in->scalar_type() == at::kFloat &&
                    scale_in->numel() == 1,
                "scale must be one float32 on the input's device");
    sk = scale_in->contiguous();
    check_status(fln_norm_forward_fp8_delayed((int)kind, x.data_ptr(), r, g, b, q.data_ptr(), s, nullptr, nullptr,
                                              sk.data_ptr<float>(), amax.data_ptr<float>(), x.size(0), x.size(1), dt,
                                              (float)epsilon, stream_of(x)),
                 "norm_fp8_scaled");
    return {q, sum, new_cuda({0}, at::kFloat, x), amax};
  }
  Tensor row_scale = new_cuda({x.size(0)}, at::kFloat, x);
  check_status(fln_norm_forward_fp8_rowwise((int)kind, x.data_ptr(), r, g, b, q.data_ptr(), s, nullptr, nullptr,
                                            row_scale.data_ptr<float>(), amax.data_ptr<float>(), x.size(0), x.size(1),
                                            dt, (float)epsilon, stream_of(x)),
               "norm_fp8_scaled");
  return {q, sum, row_scale, amax};
}

// One-pass MXFP8 output: (q e4m3, sum, E8M0 scale bytes [rows, cols / 32] as uint8, amax)
std::tuple<Tensor, Tensor, Tensor, Tensor> norm_mxfp8(int64_t kind, const Tensor& input, const OptTensor& residual,
                                                      const OptTensor& gamma, const OptTensor& beta, double epsilon) {
  TORCH_CHECK(kind == FLN_LAYERNORM || kind == FLN_RMSNORM, "kind must be 0 (layernorm) or 1 (rmsnorm)");
  Tensor x = check_matrix(input, "input");
  TORCH_CHECK(x.size(1) % 32 == 0, "mxfp8 output needs a row length that is a multiple of 32");
  const int dt = dtype_code(x, "norm_mxfp8");
  DeviceOf guard(x);
  Tensor gk, bk, rk, sum;
  const void* g = param_ptr(gamma, x, "Gamma", gk);
  const void* b = param_ptr(beta, x, "Beta", bk);
  TORCH_CHECK(!(kind == FLN_RMSNORM && b != nullptr), "rmsnorm takes no beta");
  const void* r = nullptr;
  void* s = nullptr;
  if (residual.has_value() && residual->defined()) {
    rk = check_like(*residual, x, "residual");
    r = rk.data_ptr();
    sum = new_like(x);
    s = sum.data_ptr();
  } else {
    sum = new_cuda({0}, x.scalar_type(), x);
  }
  Tensor q = new_cuda(x.sizes(), at::kFloat8_e4m3fn, x);
  Tensor scales = new_cuda({x.size(0), x.size(1) / 32}, at::kByte, x);
  Tensor amax = new_cuda({1}, at::kFloat, x);
  check_status(fln_norm_forward_mxfp8((int)kind, x.data_ptr(), r, g, b, q.data_ptr(), scales.data_ptr<uint8_t>(), s,
                                      nullptr, nullptr, amax.data_ptr<float>(), x.size(0), x.size(1), dt,
                                      (float)epsilon, stream_of(x)),
               "norm_mxfp8");
  return {q, sum, scales, amax};
}

// ---------------------------------------------------------------------------------------
// backward family
// ---------------------------------------------------------------------------------------
struct BwdOut {
  Tensor dx, dgamma, dbeta, dgb_f32;
};

BwdOut norm_backward(int kind, const Tensor& grad_output, const Tensor& input, const OptTensor& mean_o,
                     const Tensor& rstd_t, const OptTensor& gamma, const OptTensor& dres_in, bool want_dx,
                     bool want_dgamma, bool want_dbeta, bool want_f32, const char* op) {
  Tensor x = check_matrix(input, "input");
  TORCH_CHECK(grad_output.device().is_cuda(), "grad_output must be a CUDA tensor");
  TORCH_CHECK(grad_output.sizes() == x.sizes(), "grad_output shape must match input shape");
  const int dt = dtype_code(x, op);
  DeviceOf guard(x);
  Tensor dy = check_like(grad_output, x, "grad_output");
  Tensor rstd = check_stat(rstd_t, x, "rstd");
  Tensor mean, gk, dk;
  const float* mean_p = nullptr;
  if (kind == FLN_LAYERNORM) {
    TORCH_CHECK(mean_o.has_value() && mean_o->defined(), "mean is required");
    mean = check_stat(*mean_o, x, "mean");
    mean_p = mean.data_ptr<float>();
  }
  const void* g = param_ptr(gamma, x, "Gamma", gk);
  const void* dr = nullptr;
  if (dres_in.has_value() && dres_in->defined()) {
    dk = check_like(*dres_in, x, "dres_in");
    dr = dk.data_ptr();
    want_dx = true;
  }
  const int64_t rows = x.size(0), cols = x.size(1);
  BwdOut o;
  if (want_dx) o.dx = new_like(x);
  if (want_dgamma) o.dgamma = new_cuda({cols}, x.scalar_type(), x);
  if (want_dbeta && kind == FLN_LAYERNORM) o.dbeta = new_cuda({cols}, x.scalar_type(), x);
  if (want_f32) o.dgb_f32 = new_cuda({(kind == FLN_LAYERNORM ? 2 : 1) * cols}, at::kFloat, x);
  Tensor ws;
  size_t ws_bytes = 0;
  if (o.dgamma.defined() || o.dbeta.defined() || o.dgb_f32.defined()) {
    ws_bytes = fln_backward_workspace_bytes(rows, cols, dt);
    if (ws_bytes > 0) ws = new_cuda({(int64_t)ws_bytes}, at::kByte, x);
  }
  check_status(fln_norm_backward(kind, dy.data_ptr(), x.data_ptr(), mean_p, rstd.data_ptr<float>(), g, dr,
                                 o.dx.defined() ? o.dx.data_ptr() : nullptr,
                                 o.dgamma.defined() ? o.dgamma.data_ptr() : nullptr,
                                 o.dbeta.defined() ? o.dbeta.data_ptr() : nullptr,
                                 o.dgb_f32.defined() ? o.dgb_f32.data_ptr<float>() : nullptr,
                                 ws.defined() ? ws.data_ptr() : nullptr, ws_bytes, rows, cols, dt, stream_of(x)),
               op);
  return o;
}

Tensor or_empty(const Tensor& t, const Tensor& like) { return t.defined() ? t : new_cuda({0}, like.scalar_type(), like); }

// operator forms: masked-off gradients come back as empty (0-element) tensors
std::tuple<Tensor, Tensor, Tensor> layernorm_bwd(const Tensor& grad_output, const Tensor& input, const Tensor& mean,
                                                 const Tensor& rstd, const OptTensor& gamma, const OptTensor& dres_in,
                                                 bool need_dx, bool need_dgamma, bool need_dbeta) {
  BwdOut o = norm_backward(FLN_LAYERNORM, grad_output, input, mean, rstd, gamma, dres_in, need_dx, need_dgamma,
                           need_dbeta, false, "layernorm_backward");
  return {or_empty(o.dx, input), or_empty(o.dgamma, input), or_empty(o.dbeta, input)};
}
std::tuple<Tensor, Tensor> rmsnorm_bwd(const Tensor& grad_output, const Tensor& input, const Tensor& rstd,
                                       const OptTensor& gamma, const OptTensor& dres_in, bool need_dx,
                                       bool need_dgamma) {
  BwdOut o = norm_backward(FLN_RMSNORM, grad_output, input, std::nullopt, rstd, gamma, dres_in, need_dx, need_dgamma,
                           false, false, "rmsnorm_backward");
  return {or_empty(o.dx, input), or_empty(o.dgamma, input)};
}
// (dx, fp32 [dgamma | dbeta]) -- the buffer a row-sharded job all-reduces before rounding
std::tuple<Tensor, Tensor> layernorm_bwd_f32(const Tensor& grad_output, const Tensor& input, const Tensor& mean,
                                             const Tensor& rstd, const OptTensor& gamma) {
  BwdOut o = norm_backward(FLN_LAYERNORM, grad_output, input, mean, rstd, gamma, std::nullopt, true, false, false, true,
                           "layernorm_backward");
  return {o.dx, o.dgb_f32};
}
Tensor cast_from_f32(const Tensor& src, at::ScalarType dtype) {
  TORCH_CHECK(src.device().is_cuda() && src.scalar_type() == at::kFloat, "src must be a CUDA float32 tensor");
  DeviceOf guard(src);
  Tensor s = src.contiguous();
  Tensor out = new_cuda(s.sizes(), dtype, s);
  check_status(fln_cast_from_f32(s.data_ptr<float>(), out.data_ptr(), s.numel(), dtype_code(out, "cast_from_f32"),
                                 stream_of(s)),
               "cast_from_f32");
  return out;
}

// G1 backward (reference csrc/layernorm_cuda.cpp:97-141): [grad_input, grad_gamma, grad_beta],
// undefined (None) where output_mask is false or the parameter is absent
std::vector<OptTensor> backward_g1(const Tensor& grad_output, const Tensor& input, const Tensor& mean,
                                   const Tensor& rstd, const OptTensor& gamma, const OptTensor& beta,
                                   std::array<bool, 3> output_mask) {
  const bool has_g = gamma.has_value() && gamma->defined();
  const bool has_b = beta.has_value() && beta->defined();
  BwdOut o = norm_backward(FLN_LAYERNORM, grad_output, input, mean, rstd, gamma, std::nullopt, output_mask[0],
                           output_mask[1] && has_g, output_mask[2] && has_b, false, "layernorm_backward");
  auto opt = [](const Tensor& t) -> OptTensor { return t.defined() ? OptTensor(t) : std::nullopt; };
  return {opt(o.dx), opt(o.dgamma), opt(o.dbeta)};
}

// LayerNorm with its autograd node in C++: what the module calls in eager mode.  The same
// forward / backward as above without a trip through Python in the backward pass (a Python
// autograd.Function costs ~25 us per training step more than torch's native LayerNorm at the
// latency-bound shapes).
struct LayerNormAutograd : public torch::autograd::Function<LayerNormAutograd> {
  static Tensor forward(torch::autograd::AutogradContext* ctx, const Tensor& input, const OptTensor& gamma,
                        const OptTensor& beta, double epsilon) {
    at::AutoDispatchBelowADInplaceOrView guard;
    auto t = layernorm_fwd(input, gamma, beta, epsilon);
    const bool has_g = gamma.has_value() && gamma->defined();
    const bool has_b = beta.has_value() && beta->defined();
    ctx->save_for_backward({input, has_g ? *gamma : Tensor(), std::get<1>(t), std::get<2>(t)});
    // needs_input_grad counts only the tensor arguments that are present
    ctx->saved_data["i_g"] = has_g ? (int64_t)1 : (int64_t)-1;
    ctx->saved_data["i_b"] = has_b ? (int64_t)(has_g ? 2 : 1) : (int64_t)-1;
    return std::get<0>(t);
  }
  static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx,
                                               torch::autograd::tensor_list grad_outputs) {
    auto saved = ctx->get_saved_variables();
    const Tensor& input = saved[0];
    const Tensor& gamma = saved[1];
    const int64_t i_g = ctx->saved_data["i_g"].toInt(), i_b = ctx->saved_data["i_b"].toInt();
    const bool need_dx = ctx->needs_input_grad(0);
    const bool need_dg = i_g >= 0 && ctx->needs_input_grad((size_t)i_g);
    const bool need_db = i_b >= 0 && ctx->needs_input_grad((size_t)i_b);
    BwdOut o = norm_backward(FLN_LAYERNORM, grad_outputs[0], input, saved[2], saved[3],
                             gamma.defined() ? OptTensor(gamma) : std::nullopt, std::nullopt, need_dx, need_dg, need_db,
                             false, "layernorm_backward");
    return {o.dx, o.dgamma, o.dbeta, Tensor()};
  }
};
Tensor layernorm_autograd(const Tensor& input, const OptTensor& gamma, const OptTensor& beta, double epsilon) {
  return LayerNormAutograd::apply(input, gamma, beta, epsilon);
}

// The same for RMSNorm and for the fused residual-add forms: outputs (y, sum); sum is an empty
// tensor without a residual.  The gradient that arrives for `sum` (the residual stream of a
// pre-norm block) goes into the backward kernel as its incoming residual gradient, and the one
// dx that comes out is the gradient of both `input` and `residual`.
struct NormAutograd : public torch::autograd::Function<NormAutograd> {
  static torch::autograd::tensor_list forward(torch::autograd::AutogradContext* ctx, int64_t kind, const Tensor& input,
                                              const OptTensor& residual, const OptTensor& gamma, const OptTensor& beta,
                                              double epsilon) {
    at::AutoDispatchBelowADInplaceOrView guard;
    TORCH_CHECK(kind == FLN_LAYERNORM || kind == FLN_RMSNORM, "kind must be 0 (layernorm) or 1 (rmsnorm)");
    TORCH_CHECK(!(kind == FLN_RMSNORM && beta.has_value() && beta->defined()), "rmsnorm takes no beta");
    const bool has_r = residual.has_value() && residual->defined();
    FwdOut o = norm_forward((int)kind, input, residual, gamma, beta, epsilon, FLN_ACT_NONE, true,
                            kind == FLN_LAYERNORM ? "add_layernorm" : "add_rmsnorm");
    const bool has_g = gamma.has_value() && gamma->defined();
    const bool has_b = beta.has_value() && beta->defined();
    // the normalized tensor is the sum when there is a residual
    ctx->save_for_backward({has_r ? o.sum : input, has_g ? *gamma : Tensor(),
                            kind == FLN_LAYERNORM ? o.mean : Tensor(), o.rstd});
    ctx->saved_data["kind"] = kind;
    ctx->saved_data["has_r"] = has_r;
    // needs_input_grad counts only the tensor arguments that are present
    int64_t next = 1;
    ctx->saved_data["i_res"] = has_r ? next++ : (int64_t)-1;
    ctx->saved_data["i_g"] = has_g ? next++ : (int64_t)-1;
    ctx->saved_data["i_b"] = has_b ? next++ : (int64_t)-1;
    return {o.y, has_r ? o.sum : new_cuda({0}, input.scalar_type(), input)};
  }
  static torch::autograd::tensor_list backward(torch::autograd::AutogradContext* ctx,
                                               torch::autograd::tensor_list grads) {
    auto saved = ctx->get_saved_variables();
    const int kind = (int)ctx->saved_data["kind"].toInt();
    const bool has_r = ctx->saved_data["has_r"].toBool();
    const int64_t i_res = ctx->saved_data["i_res"].toInt(), i_g = ctx->saved_data["i_g"].toInt(),
                  i_b = ctx->saved_data["i_b"].toInt();
    const Tensor& s = saved[0];
    const Tensor& gamma = saved[1];
    const bool need_dx = ctx->needs_input_grad(0) || (i_res >= 0 && ctx->needs_input_grad((size_t)i_res));
    const bool need_dg = i_g >= 0 && ctx->needs_input_grad((size_t)i_g);
    const bool need_db = i_b >= 0 && ctx->needs_input_grad((size_t)i_b);
    Tensor dy = grads[0].defined() ? grads[0] : at::zeros_like(s);
    OptTensor dres = (has_r && grads[1].defined()) ? OptTensor(grads[1]) : std::nullopt;
    BwdOut o = norm_backward(kind, dy, s, kind == FLN_LAYERNORM ? OptTensor(saved[2]) : std::nullopt, saved[3],
                             gamma.defined() ? OptTensor(gamma) : std::nullopt, dres, need_dx, need_dg, need_db, false,
                             kind == FLN_LAYERNORM ? "layernorm_backward" : "rmsnorm_backward");
    return {Tensor(), o.dx, has_r ? o.dx : Tensor(), o.dgamma, o.dbeta, Tensor()};
  }
};
std::vector<Tensor> norm_autograd(int64_t kind, const Tensor& input, const OptTensor& residual, const OptTensor& gamma,
                                  const OptTensor& beta, double epsilon) {
  return NormAutograd::apply(kind, input, residual, gamma, beta, epsilon);
}

int64_t get_memory_usage(int batch_size, int hidden_size, bool use_mixed_precision) {
  return fln_get_memory_usage(batch_size, hidden_size, use_mixed_precision ? 1 : 0);
}
std::string get_performance_hints(int batch_size, int hidden_size) {
  char buf[1024];
  fln_get_performance_hints(batch_size, hidden_size, buf, sizeof(buf));
  return std::string(buf);
}

}  // namespace

TORCH_LIBRARY(fused_layernorm, m) {
  m.def("layernorm(Tensor input, Tensor? gamma, Tensor? beta, float epsilon) -> Tensor");
  m.def("layernorm_gelu(Tensor input, Tensor? gamma, Tensor? beta, float epsilon, str approximate) -> Tensor");
  m.def("layernorm_fwd(Tensor input, Tensor? gamma, Tensor? beta, float epsilon) -> (Tensor, Tensor, Tensor)");
  m.def("rmsnorm_fwd(Tensor input, Tensor? gamma, float epsilon) -> (Tensor, Tensor)");
  m.def("add_layernorm_fwd(Tensor input, Tensor residual, Tensor? gamma, Tensor? beta, float epsilon) -> (Tensor, Tensor, Tensor, Tensor)");
  m.def("add_rmsnorm_fwd(Tensor input, Tensor residual, Tensor? gamma, float epsilon) -> (Tensor, Tensor, Tensor)");
  m.def("norm_fp8(int kind, Tensor input, Tensor? residual, Tensor? gamma, Tensor? beta, float epsilon) -> (Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("norm_fp8_scaled(int kind, Tensor input, Tensor? residual, Tensor? gamma, Tensor? beta, Tensor? scale_in, float epsilon) -> (Tensor, Tensor, Tensor, Tensor)");
  m.def("norm_mxfp8(int kind, Tensor input, Tensor? residual, Tensor? gamma, Tensor? beta, float epsilon) -> (Tensor, Tensor, Tensor, Tensor)");
  m.def("layernorm_bwd(Tensor grad_output, Tensor input, Tensor mean, Tensor rstd, Tensor? gamma, Tensor? dres_in, bool need_dx, bool need_dgamma, bool need_dbeta) -> (Tensor, Tensor, Tensor)");
  m.def("rmsnorm_bwd(Tensor grad_output, Tensor input, Tensor rstd, Tensor? gamma, Tensor? dres_in, bool need_dx, bool need_dgamma) -> (Tensor, Tensor)");
  m.def("layernorm_bwd_f32(Tensor grad_output, Tensor input, Tensor mean, Tensor rstd, Tensor? gamma) -> (Tensor, Tensor)");
  m.def("cast_from_f32(Tensor src, ScalarType dtype) -> Tensor");
}

TORCH_LIBRARY_IMPL(fused_layernorm, CUDA, m) {
  m.impl("layernorm", &layernorm);
  m.impl("layernorm_gelu", &layernorm_gelu);
  m.impl("layernorm_fwd", &layernorm_fwd);
  m.impl("rmsnorm_fwd", &rmsnorm_fwd);
  m.impl("add_layernorm_fwd", &add_layernorm_fwd);
  m.impl("add_rmsnorm_fwd", &add_rmsnorm_fwd);
  m.impl("norm_fp8", &norm_fp8);
  m.impl("norm_fp8_scaled", &norm_fp8_scaled);
  m.impl("norm_mxfp8", &norm_mxfp8);
  m.impl("layernorm_bwd", &layernorm_bwd);
  m.impl("rmsnorm_bwd", &rmsnorm_bwd);
  m.impl("layernorm_bwd_f32", &layernorm_bwd_f32);
  m.impl("cast_from_f32", &cast_from_f32);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "Fused LayerNorm / RMSNorm for B200 (sm_100a): PyTorch front end of libfln_b200";
  namespace py = pybind11;

  // G2: positional like the reference, plus names, None for gamma/beta and an `eps` alias
  m.def(
      "layernorm",
      [](const Tensor& input, const OptTensor& gamma, const OptTensor& beta, double epsilon, std::optional<double> eps) {
        return layernorm(input, gamma, beta, eps.value_or(epsilon));
      },
      "LayerNorm forward", py::arg("input"), py::arg("gamma") = py::none(), py::arg("beta") = py::none(),
      py::arg("epsilon") = 1e-5, py::kw_only(), py::arg("eps") = py::none());
  m.def(
      "layernorm_gelu",
      [](const Tensor& input, const OptTensor& gamma, const OptTensor& beta, double epsilon, std::optional<double> eps,
         std::string approximate) { return layernorm_gelu(input, gamma, beta, eps.value_or(epsilon), approximate); },
      "LayerNorm + GELU (approximate='tanh' is the reference's formula, 'none' the exact erf form)",
      py::arg("input"), py::arg("gamma") = py::none(), py::arg("beta") = py::none(), py::arg("epsilon") = 1e-5,
      py::kw_only(), py::arg("eps") = py::none(), py::arg("approximate") = "tanh");

  // G1
  m.def(
      "forward",
      [](const Tensor& input, const OptTensor& gamma, const OptTensor& beta, double epsilon) {
        auto t = layernorm_fwd(input, gamma, beta, epsilon);
        return std::vector<Tensor>{std::get<0>(t), std::get<1>(t), std::get<2>(t)};
      },
      "LayerNorm forward (CUDA)", py::arg("input"), py::arg("gamma") = py::none(), py::arg("beta") = py::none(),
      py::arg("epsilon") = 1e-5);
  m.def("layernorm_autograd", &layernorm_autograd,
        "LayerNorm forward that records a C++ autograd node (dx, dgamma, dbeta from the fused backward)",
        py::arg("input"), py::arg("gamma") = py::none(), py::arg("beta") = py::none(), py::arg("epsilon") = 1e-5);
  m.def("norm_autograd", &norm_autograd,
        "(y, sum) of LayerNorm (kind 0) / RMSNorm (kind 1) with optional fused residual add, recording a C++ autograd "
        "node; a gradient arriving for sum is added into dx inside the backward kernel",
        py::arg("kind"), py::arg("input"), py::arg("residual") = py::none(), py::arg("gamma") = py::none(),
        py::arg("beta") = py::none(), py::arg("epsilon") = 1e-5);
  m.def("backward", &backward_g1, "LayerNorm backward (CUDA)", py::arg("grad_output"), py::arg("input"),
        py::arg("mean"), py::arg("rstd"), py::arg("gamma") = py::none(), py::arg("beta") = py::none(),
        py::arg("output_mask") = std::array<bool, 3>{true, true, true});
  m.def("get_memory_usage", &get_memory_usage, "Estimate memory usage", py::arg("batch_size"), py::arg("hidden_size"),
        py::arg("use_mixed_precision") = false);
  m.def("get_performance_hints", &get_performance_hints, "Get performance optimization hints", py::arg("batch_size"),
        py::arg("hidden_size"));

  // additions
  m.def("rmsnorm_fwd", &rmsnorm_fwd, py::arg("input"), py::arg("gamma") = py::none(), py::arg("epsilon") = 1e-6);
  m.def(
      "rmsnorm",
      [](const Tensor& input, const OptTensor& gamma, double epsilon) {
        return norm_forward(FLN_RMSNORM, input, std::nullopt, gamma, std::nullopt, epsilon, FLN_ACT_NONE, false,
                            "rmsnorm")
            .y;
      },
      py::arg("input"), py::arg("gamma") = py::none(), py::arg("epsilon") = 1e-6);
  m.def("add_layernorm_fwd", &add_layernorm_fwd, py::arg("input"), py::arg("residual"), py::arg("gamma") = py::none(),
        py::arg("beta") = py::none(), py::arg("epsilon") = 1e-5);
  m.def("add_rmsnorm_fwd", &add_rmsnorm_fwd, py::arg("input"), py::arg("residual"), py::arg("gamma") = py::none(),
        py::arg("epsilon") = 1e-6);
  m.def(
      "add_layernorm",
      [](const Tensor& input, const Tensor& residual, const OptTensor& gamma, const OptTensor& beta, double epsilon) {
        FwdOut o = norm_forward(FLN_LAYERNORM, input, residual, gamma, beta, epsilon, FLN_ACT_NONE, false,
                                "add_layernorm");
        return std::make_tuple(o.y, o.sum);
      },
      py::arg("input"), py::arg("residual"), py::arg("gamma") = py::none(), py::arg("beta") = py::none(),
      py::arg("epsilon") = 1e-5);
  m.def(
      "add_rmsnorm",
      [](const Tensor& input, const Tensor& residual, const OptTensor& gamma, double epsilon) {
        FwdOut o = norm_forward(FLN_RMSNORM, input, residual, gamma, std::nullopt, epsilon, FLN_ACT_NONE, false,
                                "add_rmsnorm");
        return std::make_tuple(o.y, o.sum);
      },
      py::arg("input"), py::arg("residual"), py::arg("gamma") = py::none(), py::arg("epsilon") = 1e-6);
  m.def(
      "add_rmsnorm_fp8",
      [](const Tensor& input, const OptTensor& residual, const OptTensor& gamma, double epsilon) {
        auto t = norm_fp8(FLN_RMSNORM, input, residual, gamma, std::nullopt, epsilon);
        return std::make_tuple(std::get<0>(t), std::get<1>(t), std::get<2>(t));
      },
      "(q fp8-e4m3, residual sum, scale = 448 / amax)", py::arg("input"), py::arg("residual") = py::none(),
      py::arg("gamma") = py::none(), py::arg("epsilon") = 1e-6);
  m.def("norm_mxfp8", &norm_mxfp8, py::arg("kind"), py::arg("input"), py::arg("residual") = py::none(),
        py::arg("gamma") = py::none(), py::arg("beta") = py::none(), py::arg("epsilon") = 1e-5);
  m.def("norm_fp8_scaled", &norm_fp8_scaled, py::arg("kind"), py::arg("input"), py::arg("residual") = py::none(),
        py::arg("gamma") = py::none(), py::arg("beta") = py::none(), py::arg("scale_in") = py::none(),
        py::arg("epsilon") = 1e-5);
  m.def("norm_fp8", &norm_fp8, py::arg("kind"), py::arg("input"), py::arg("residual") = py::none(),
        py::arg("gamma") = py::none(), py::arg("beta") = py::none(), py::arg("epsilon") = 1e-5);
  m.def("layernorm_bwd", &layernorm_bwd, py::arg("grad_output"), py::arg("input"), py::arg("mean"), py::arg("rstd"),
        py::arg("gamma") = py::none(), py::arg("dres_in") = py::none(), py::arg("need_dx") = true,
        py::arg("need_dgamma") = true, py::arg("need_dbeta") = true);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("grad_output"), py::arg("input"), py::arg("rstd"),
        py::arg("gamma") = py::none(), py::arg("dres_in") = py::none(), py::arg("need_dx") = true,
        py::arg("need_dgamma") = true);
  m.def("layernorm_bwd_f32", &layernorm_bwd_f32, py::arg("grad_output"), py::arg("input"), py::arg("mean"),
        py::arg("rstd"), py::arg("gamma") = py::none());
  m.def("device_status", []() { return fln_device_status(); },
        "read and clear the device status word (0 = no kernel reported a problem)");

  m.attr("__version__") = fln_version();
  m.attr("__cuda_version__") = fln_cuda_runtime_version();
  m.attr("DEFAULT_EPSILON") = 1e-5f;       // csrc/layernorm.h:61-63 of the reference
  m.attr("MAX_GRID_SIZE") = 65535;
  m.attr("PREFERRED_BLOCK_SIZE") = 256;
}
