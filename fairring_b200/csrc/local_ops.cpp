#include "local_ops.h"

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <cmath>
#include <optional>
#include <tuple>

#include "kernels/local_kernels.h"

namespace fairring {

namespace {
void checkFlat(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), name,
              " must be a contiguous fp32 CUDA tensor");
}

// One AdamW step over flat buffers, in place.  `step` counts from 1.
void adamwFlat(at::Tensor p, at::Tensor g, at::Tensor m, at::Tensor v, double lr, double beta1,
               double beta2, double eps, double weight_decay, int64_t step, double grad_scale,
               c10::optional<at::Tensor> shadow) {
  checkFlat(p, "param");
  checkFlat(g, "grad");
  checkFlat(m, "exp_avg");
  checkFlat(v, "exp_avg_sq");
  TORCH_CHECK(g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel(),
              "flat buffers must have the same length");
  TORCH_CHECK(step >= 1, "step counts from 1");
  void* shadow_ptr = nullptr;
  if (shadow.has_value() && shadow->defined()) {
    TORCH_CHECK(shadow->is_cuda() && shadow->scalar_type() == at::kBFloat16 &&
                    shadow->is_contiguous() && shadow->numel() == p.numel(),
                "shadow must be a contiguous bf16 CUDA tensor as long as param");
    shadow_ptr = shadow->data_ptr();
  }
  c10::cuda::CUDAGuard guard(p.device());
  AdamWArgs a;
  a.lr = (float)lr;
  a.beta1 = (float)beta1;
  a.beta2 = (float)beta2;
  a.eps = (float)eps;
  a.weight_decay = (float)weight_decay;
  a.step_size = (float)(lr / (1.0 - std::pow(beta1, (double)step)));
  a.inv_sqrt_bias2 = (float)(1.0 / std::sqrt(1.0 - std::pow(beta2, (double)step)));
  a.grad_scale = (float)grad_scale;
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  cudaError_t e = launchAdamWFlat(p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(),
                                  v.data_ptr<float>(), shadow_ptr, p.numel(), a, sms,
                                  c10::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "adamw_flat launch failed: ", cudaGetErrorString(e));
}

// dst (fp32) = or += src (bf16); both contiguous, same length.
void bf16GradToF32(at::Tensor dst, at::Tensor src, bool accumulate) {
  TORCH_CHECK(dst.is_cuda() && dst.scalar_type() == at::kFloat && dst.is_contiguous(),
              "dst must be a contiguous fp32 CUDA tensor");
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kBFloat16 && src.is_contiguous() &&
                  src.numel() == dst.numel(),
              "src must be a contiguous bf16 CUDA tensor as long as dst");
  c10::cuda::CUDAGuard guard(dst.device());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  cudaError_t e = launchBf16GradToF32(dst.data_ptr<float>(), src.data_ptr(), dst.numel(), accumulate,
                                      sms, c10::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "bf16_grad_to_f32 launch failed: ", cudaGetErrorString(e));
}

// Sum of squares of a flat fp32 buffer, as a 1-element device tensor.
at::Tensor sumSq(at::Tensor x) {
  checkFlat(x, "input");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::zeros({1}, x.options());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  cudaError_t e = launchSumSq(x.data_ptr<float>(), x.numel(), out.data_ptr<float>(), sms,
                              c10::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "sumsq launch failed: ", cudaGetErrorString(e));
  return out;
}

// y, mean, rstd = layer_norm(x); y in `out_dtype` (fp32 or bf16).
std::tuple<at::Tensor, at::Tensor, at::Tensor> layerNormForward(at::Tensor x, at::Tensor gamma,
                                                                at::Tensor beta, double eps,
                                                                at::ScalarType out_dtype) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() >= 1, "x must be a contiguous CUDA tensor");
  TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16, "x must be fp32 or bf16");
  TORCH_CHECK(out_dtype == at::kFloat || out_dtype == at::kBFloat16, "output must be fp32 or bf16");
  const int64_t cols = x.size(-1);
  const int64_t rows = x.numel() / std::max<int64_t>(cols, 1);
  TORCH_CHECK(gamma.is_cuda() && beta.is_cuda() && gamma.scalar_type() == at::kFloat &&
                  beta.scalar_type() == at::kFloat && gamma.is_contiguous() && beta.is_contiguous() &&
                  gamma.numel() == cols && beta.numel() == cols,
              "weight and bias must be contiguous fp32 CUDA vectors of the row length");
  TORCH_CHECK(cols % 8 == 0 && cols <= 8192, "row length must be a multiple of 8, at most 8192");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty(x.sizes(), x.options().dtype(out_dtype));
  at::Tensor mean = at::empty({rows}, x.options().dtype(at::kFloat));
  at::Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  cudaError_t e = launchLayerNormForward(
      x.data_ptr(), x.scalar_type() == at::kBFloat16, gamma.data_ptr<float>(), beta.data_ptr<float>(),
      y.data_ptr(), out_dtype == at::kBFloat16, mean.data_ptr<float>(), rstd.data_ptr<float>(), rows,
      (int)cols, (float)eps, sms, c10::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "layer_norm forward launch failed: ", cudaGetErrorString(e));
  return std::make_tuple(y, mean, rstd);
}

// dx, dgamma, dbeta
std::tuple<at::Tensor, at::Tensor, at::Tensor> layerNormBackward(at::Tensor dy, at::Tensor x,
                                                                 at::Tensor gamma, at::Tensor mean,
                                                                 at::Tensor rstd) {
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && x.is_contiguous() && dy.sizes() == x.sizes(),
              "dy and x must be contiguous and equally shaped");
  TORCH_CHECK(dy.scalar_type() == at::kFloat || dy.scalar_type() == at::kBFloat16, "dy must be fp32 or bf16");
  const int64_t cols = x.size(-1);
  const int64_t rows = x.numel() / std::max<int64_t>(cols, 1);
  c10::cuda::CUDAGuard guard(x.device());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  at::Tensor dx = at::empty_like(x);
  at::Tensor dgamma = at::empty({cols}, gamma.options());
  at::Tensor dbeta = at::empty({cols}, gamma.options());
  at::Tensor partial = at::empty({(int64_t)layerNormBackwardBlocks(rows, sms), 2, cols}, gamma.options());
  cudaError_t e = launchLayerNormBackward(
      dy.data_ptr(), dy.scalar_type() == at::kBFloat16, x.data_ptr(), x.scalar_type() == at::kBFloat16,
      gamma.data_ptr<float>(), mean.data_ptr<float>(), rstd.data_ptr<float>(), dx.data_ptr(),
      partial.data_ptr<float>(), dgamma.data_ptr<float>(), dbeta.data_ptr<float>(), rows, (int)cols, sms,
      c10::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "layer_norm backward launch failed: ", cudaGetErrorString(e));
  return std::make_tuple(dx, dgamma, dbeta);
}

// xnew, y, mean, rstd = x + branch, layer_norm(x + branch); x fp32, branch fp32 or bf16.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> addLayerNormForward(
    at::Tensor x, at::Tensor branch, at::Tensor gamma, at::Tensor beta, double eps,
    at::ScalarType out_dtype) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == at::kFloat && x.dim() >= 1,
              "x must be a contiguous fp32 CUDA tensor");
  TORCH_CHECK(branch.is_cuda() && branch.is_contiguous() && branch.sizes() == x.sizes() &&
                  (branch.scalar_type() == at::kFloat || branch.scalar_type() == at::kBFloat16),
              "branch must be contiguous, shaped like x, fp32 or bf16");
  TORCH_CHECK(out_dtype == at::kFloat || out_dtype == at::kBFloat16, "output must be fp32 or bf16");
  const int64_t cols = x.size(-1);
  const int64_t rows = x.numel() / std::max<int64_t>(cols, 1);
  TORCH_CHECK(gamma.is_cuda() && beta.is_cuda() && gamma.scalar_type() == at::kFloat &&
                  beta.scalar_type() == at::kFloat && gamma.is_contiguous() && beta.is_contiguous() &&
                  gamma.numel() == cols && beta.numel() == cols,
              "weight and bias must be contiguous fp32 CUDA vectors of the row length");
  TORCH_CHECK(cols % 8 == 0 && cols <= 8192, "row length must be a multiple of 8, at most 8192");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor xnew = at::empty_like(x);
  at::Tensor y = at::empty(x.sizes(), x.options().dtype(out_dtype));
  at::Tensor mean = at::empty({rows}, x.options());
  at::Tensor rstd = at::empty({rows}, x.options());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  cudaError_t e = launchAddLayerNormForward(
      x.data_ptr<float>(), branch.data_ptr(), branch.scalar_type() == at::kBFloat16, gamma.data_ptr<float>(),
      beta.data_ptr<float>(), xnew.data_ptr<float>(), y.data_ptr(), out_dtype == at::kBFloat16,
      mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, (int)cols, (float)eps, sms,
      c10::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "add_layer_norm forward launch failed: ", cudaGetErrorString(e));
  return std::make_tuple(xnew, y, mean, rstd);
}

// dx (fp32), dx in bf16 (or an undefined tensor), dgamma, dbeta.  `gres`: the
// gradient that reaches xnew along the residual path, or nothing.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> addLayerNormBackward(
    at::Tensor dy, at::Tensor xnew, at::Tensor gamma, at::Tensor mean, at::Tensor rstd,
    std::optional<at::Tensor> gres, bool want_bf16) {
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && xnew.is_contiguous() && dy.sizes() == xnew.sizes() &&
                  xnew.scalar_type() == at::kFloat,
              "dy and xnew must be contiguous and equally shaped, xnew fp32");
  TORCH_CHECK(dy.scalar_type() == at::kFloat || dy.scalar_type() == at::kBFloat16, "dy must be fp32 or bf16");
  const float* gres_ptr = nullptr;
  if (gres.has_value() && gres->defined()) {
    TORCH_CHECK(gres->is_cuda() && gres->is_contiguous() && gres->scalar_type() == at::kFloat &&
                    gres->sizes() == xnew.sizes(),
                "the residual gradient must be contiguous fp32, shaped like xnew");
    gres_ptr = gres->data_ptr<float>();
  }
  const int64_t cols = xnew.size(-1);
  const int64_t rows = xnew.numel() / std::max<int64_t>(cols, 1);
  c10::cuda::CUDAGuard guard(xnew.device());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  at::Tensor dx = at::empty_like(xnew);
  at::Tensor dbr;
  if (want_bf16) dbr = at::empty(xnew.sizes(), xnew.options().dtype(at::kBFloat16));
  at::Tensor dgamma = at::empty({cols}, gamma.options());
  at::Tensor dbeta = at::empty({cols}, gamma.options());
  at::Tensor partial = at::empty({(int64_t)layerNormBackwardBlocks(rows, sms), 2, cols}, gamma.options());
  cudaError_t e = launchAddLayerNormBackward(
      dy.data_ptr(), dy.scalar_type() == at::kBFloat16, xnew.data_ptr<float>(), gres_ptr,
      gamma.data_ptr<float>(), mean.data_ptr<float>(), rstd.data_ptr<float>(), dx.data_ptr<float>(),
      want_bf16 ? dbr.data_ptr() : nullptr, partial.data_ptr<float>(), dgamma.data_ptr<float>(),
      dbeta.data_ptr<float>(), rows, (int)cols, sms, c10::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "add_layer_norm backward launch failed: ", cudaGetErrorString(e));
  return std::make_tuple(dx, dbr, dgamma, dbeta);
}

// (per-row loss, per-row log-sum-exp) of logits [rows, vocab] against targets [rows].
std::tuple<at::Tensor, at::Tensor> crossEntropyForward(at::Tensor logits, at::Tensor targets) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous(),
              "logits must be a contiguous 2-D CUDA tensor");
  TORCH_CHECK(logits.scalar_type() == at::kFloat || logits.scalar_type() == at::kBFloat16,
              "logits must be fp32 or bf16");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous() &&
                  targets.numel() == logits.size(0),
              "targets must be a contiguous int64 CUDA vector with one entry per row");
  TORCH_CHECK(logits.size(1) % 8 == 0, "the vocabulary size must be a multiple of 8");
  c10::cuda::CUDAGuard guard(logits.device());
  auto fopt = logits.options().dtype(at::kFloat);
  at::Tensor loss = at::empty({logits.size(0)}, fopt), lse = at::empty({logits.size(0)}, fopt);
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  cudaError_t e = launchCrossEntropyForward(logits.data_ptr(), logits.scalar_type() == at::kBFloat16,
                                            targets.data_ptr<int64_t>(), loss.data_ptr<float>(),
                                            lse.data_ptr<float>(), logits.size(0), (int)logits.size(1), sms,
                                            c10::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "cross_entropy forward launch failed: ", cudaGetErrorString(e));
  return std::make_tuple(loss, lse);
}

// Overwrites logits with d(loss)/d(logits) * upstream * scale.
void crossEntropyBackward(at::Tensor logits, at::Tensor targets, at::Tensor lse, at::Tensor upstream,
                          double scale) {
  TORCH_CHECK(upstream.is_cuda() && upstream.scalar_type() == at::kFloat && upstream.numel() == 1,
              "upstream must be a one-element fp32 CUDA tensor");
  c10::cuda::CUDAGuard guard(logits.device());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  cudaError_t e = launchCrossEntropyBackward(
      logits.data_ptr(), logits.scalar_type() == at::kBFloat16, targets.data_ptr<int64_t>(),
      lse.data_ptr<float>(), upstream.data_ptr<float>(), (float)scale, logits.size(0), (int)logits.size(1),
      sms, c10::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "cross_entropy backward launch failed: ", cudaGetErrorString(e));
}
}  // namespace

uint64_t localLaunchCount() { return localLaunchCountImpl(); }

void bindLocalOps(pybind11::module_& m) {
  namespace py = pybind11;
  m.def("adamw_flat_", &adamwFlat, py::arg("param"), py::arg("grad"), py::arg("exp_avg"),
        py::arg("exp_avg_sq"), py::arg("lr"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"),
        py::arg("weight_decay"), py::arg("step"), py::arg("grad_scale") = 1.0,
        py::arg("shadow") = py::none());
  m.def("bf16_grad_to_f32_", &bf16GradToF32, py::arg("dst"), py::arg("src"),
        py::arg("accumulate") = false);
  m.def("sumsq", &sumSq, py::arg("x"));
  m.def("cross_entropy_fwd", &crossEntropyForward, py::arg("logits"), py::arg("targets"));
  m.def("cross_entropy_bwd_", &crossEntropyBackward, py::arg("logits"), py::arg("targets"),
        py::arg("lse"), py::arg("upstream"), py::arg("scale"));
  m.def("add_layer_norm_fwd", &addLayerNormForward, py::arg("x"), py::arg("branch"), py::arg("weight"),
        py::arg("bias"), py::arg("eps"), py::arg("out_dtype"));
  m.def("add_layer_norm_bwd", &addLayerNormBackward, py::arg("dy"), py::arg("xnew"), py::arg("weight"),
        py::arg("mean"), py::arg("rstd"), py::arg("gres"), py::arg("want_bf16"));
  m.def("layer_norm_fwd", &layerNormForward, py::arg("x"), py::arg("weight"), py::arg("bias"),
        py::arg("eps"), py::arg("out_dtype"));
  m.def("layer_norm_bwd", &layerNormBackward, py::arg("dy"), py::arg("x"), py::arg("weight"),
        py::arg("mean"), py::arg("rstd"));
}

}  // namespace fairring
