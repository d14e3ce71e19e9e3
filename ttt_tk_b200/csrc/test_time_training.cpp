// PyTorch extension module `test_time_training`: the reference's operator boundary
// (test_time_training.cpp:24-104 of the reference: `ttt_forward`, `ttt_backward`, same positional
// arguments, both return `Out`) as a thin shim over the C ABI of libttt_mlp_b200.so.
//
// The checks are those of the reference's launchers (kernels/ttt/ttt.cu:621-630,
// kernels/ttt_backward/ttt.cu:1507-1760), made on every call and extended to the tensors the
// reference leaves unchecked; failures raise like TORCH_CHECK does.  Like the reference the
// calls block until the result is ready (kernels/ttt/ttt.cu:714-715); pass
// TTT_B200_ASYNC=1 in the environment for stream-ordered, non-blocking calls.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdlib>
#include <vector>

#include "../../include/ttt_mlp_b200.h"

namespace {

bool async_calls() {
  static const bool v = [] {
    const char* e = std::getenv("TTT_B200_ASYNC");
    return e && e[0] == '1';
  }();
  return v;
}

void check_tensor(const torch::Tensor& t, const char* name, at::ScalarType dtype, const torch::Tensor& like,
                  std::vector<int64_t> shape) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.device() == like.device(), name, " must be on the same device as XQ");
  TORCH_CHECK(t.scalar_type() == dtype, name, " has the wrong dtype");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.sizes() == at::IntArrayRef(shape), name, " has the wrong shape");
}

void check_eta(const torch::Tensor& t, const char* name, const torch::Tensor& like, int64_t B, int64_t H,
               int64_t NC) {
  TORCH_CHECK(t.is_cuda() && t.device() == like.device(), name, " must be a CUDA tensor on XQ's device");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " has the wrong dtype");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  const bool r4 = t.dim() == 4 && t.size(0) == B && t.size(1) == H && t.size(2) == NC && t.size(3) == 64;
  const bool r5 = t.dim() == 5 && t.size(0) == B && t.size(1) == H && t.size(2) == NC && t.size(3) == 64 &&
                  t.size(4) == 1;
  TORCH_CHECK(r4 || r5, name, " must have shape [B, H, NC, 64] or [B, H, NC, 64, 1]");
}

struct Dims {
  int64_t B, H, NC, n;
};

Dims dims_of(const torch::Tensor& XQ, const torch::Tensor& W1_checkpoints, int cgs) {
  TORCH_CHECK(XQ.dim() == 5, "XQ must be 5-D [B, H, NC, 64, 64]");
  TORCH_CHECK(XQ.size(4) == 64, "head dimension must be 64");
  TORCH_CHECK(XQ.size(3) == 64, "mini-batch size must be 64");
  TORCH_CHECK(XQ.size(2) >= 1, "need at least one mini-batch");
  TORCH_CHECK(cgs >= 1, "checkpoint_group_size must be >= 1");
  Dims d{XQ.size(0), XQ.size(1), XQ.size(2), (XQ.size(2) + cgs - 1) / cgs};
  TORCH_CHECK(W1_checkpoints.dim() == 5 && W1_checkpoints.size(2) == d.n,
              "checkpoint tensors must hold ceil(NC / checkpoint_group_size) states");
  return d;
}

}  // namespace

torch::Tensor ttt_forward(const torch::Tensor XQ, const torch::Tensor XK, const torch::Tensor XV,
                          const torch::Tensor last_eta, const torch::Tensor ttt_norm_weight,
                          const torch::Tensor ttt_norm_bias, const torch::Tensor W1, const torch::Tensor b1,
                          const torch::Tensor W2, const torch::Tensor b2, const torch::Tensor W1_checkpoints,
                          const torch::Tensor b1_checkpoints, const torch::Tensor W2_checkpoints,
                          const torch::Tensor b2_checkpoints, const torch::Tensor Out,
                          const int checkpoint_group_size) {
  const Dims d = dims_of(XQ, W1_checkpoints, checkpoint_group_size);
  const auto bf = at::kBFloat16, f32 = at::kFloat;
  const std::vector<int64_t> tok{d.B, d.H, d.NC, 64, 64};
  check_tensor(XQ, "XQ", bf, XQ, tok);
  check_tensor(XK, "XK", bf, XQ, tok);
  check_tensor(XV, "XV", bf, XQ, tok);
  check_eta(last_eta, "last_eta", XQ, d.B, d.H, d.NC);
  check_tensor(ttt_norm_weight, "ttt_norm_weight", f32, XQ, {1, d.H, 1, 64});
  check_tensor(ttt_norm_bias, "ttt_norm_bias", f32, XQ, {1, d.H, 1, 64});
  check_tensor(W1, "W1", f32, XQ, {d.B, d.H, 64, 256});
  check_tensor(b1, "b1", f32, XQ, {d.B, d.H, 1, 256});
  check_tensor(W2, "W2", f32, XQ, {d.B, d.H, 256, 64});
  check_tensor(b2, "b2", f32, XQ, {d.B, d.H, 1, 64});
  check_tensor(W1_checkpoints, "W1_checkpoints", f32, XQ, {d.B, d.H, d.n, 64, 256});
  check_tensor(b1_checkpoints, "b1_checkpoints", f32, XQ, {d.B, d.H, d.n, 1, 256});
  check_tensor(W2_checkpoints, "W2_checkpoints", f32, XQ, {d.B, d.H, d.n, 256, 64});
  check_tensor(b2_checkpoints, "b2_checkpoints", f32, XQ, {d.B, d.H, d.n, 1, 64});
  check_tensor(Out, "Out", bf, XQ, tok);

  const c10::cuda::CUDAGuard guard(XQ.device());
  ttt_b200_fwd_args a = {};
  a.XQ = XQ.data_ptr();
  a.XK = XK.data_ptr();
  a.XV = XV.data_ptr();
  a.last_eta = last_eta.data_ptr();
  a.ttt_norm_weight = ttt_norm_weight.data_ptr<float>();
  a.ttt_norm_bias = ttt_norm_bias.data_ptr<float>();
  a.W1 = W1.data_ptr<float>();
  a.b1 = b1.data_ptr<float>();
  a.W2 = W2.data_ptr<float>();
  a.b2 = b2.data_ptr<float>();
  a.W1_checkpoints = W1_checkpoints.data_ptr<float>();
  a.b1_checkpoints = b1_checkpoints.data_ptr<float>();
  a.W2_checkpoints = W2_checkpoints.data_ptr<float>();
  a.b2_checkpoints = b2_checkpoints.data_ptr<float>();
  a.Out = Out.data_ptr();
  a.B = static_cast<int32_t>(d.B);
  a.H = static_cast<int32_t>(d.H);
  a.NC = static_cast<int32_t>(d.NC);
  a.checkpoint_group_size = checkpoint_group_size;
  a.num_checkpoints = static_cast<int32_t>(d.n);
  a.flags = async_calls() ? 0u : TTT_B200_FLAG_SYNC;
  const int rc = ttt_b200_forward(&a, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "ttt_forward failed (code ", rc, "): ", ttt_b200_last_error());
  return Out;
}

torch::Tensor ttt_backward(
    const torch::Tensor XQ, const torch::Tensor XK, const torch::Tensor XV, const torch::Tensor last_eta,
    const torch::Tensor ttt_norm_weight, const torch::Tensor ttt_norm_bias, const torch::Tensor W1_checkpoints,
    const torch::Tensor b1_checkpoints, const torch::Tensor W2_checkpoints, const torch::Tensor b2_checkpoints,
    const torch::Tensor Out, const torch::Tensor W1_init_group, const torch::Tensor b1_init_group,
    const torch::Tensor W2_init_group, const torch::Tensor b2_init_group, const torch::Tensor x_hat_ln_group,
    const torch::Tensor std_ln_group, const torch::Tensor X2_group, const torch::Tensor Z1_group,
    const torch::Tensor Z1_bar_group, const torch::Tensor X2_bar_group, const torch::Tensor grad_l_wrt_Z2_group,
    const torch::Tensor grad_l_wrt_Z1_group, const torch::Tensor x_hat_fused_group,
    const torch::Tensor grad_x_hat_fused_group, const torch::Tensor grad_output_fused_group,
    const torch::Tensor std_fused_group, const torch::Tensor grad_L_W1_last, const torch::Tensor grad_L_b1_last,
    const torch::Tensor grad_L_W2_last, const torch::Tensor grad_L_b2_last,
    const torch::Tensor grad_L_XQW_mini_batch, const torch::Tensor grad_L_ttt_norm_weight,
    const torch::Tensor grad_L_ttt_norm_bias, const torch::Tensor grad_L_W1_init,
    const torch::Tensor grad_L_b1_init, const torch::Tensor grad_L_W2_init, const torch::Tensor grad_L_b2_init,
    const torch::Tensor grad_L_last_eta, const torch::Tensor grad_L_XQ, const torch::Tensor grad_L_XK,
    const torch::Tensor grad_L_XV, const int checkpoint_group_size) {
  const Dims d = dims_of(XQ, W1_checkpoints, checkpoint_group_size);
  const auto bf = at::kBFloat16, f32 = at::kFloat;
  const int64_t g = checkpoint_group_size;
  const std::vector<int64_t> tok{d.B, d.H, d.NC, 64, 64};
  check_tensor(XQ, "XQ", bf, XQ, tok);
  check_tensor(XK, "XK", bf, XQ, tok);
  check_tensor(XV, "XV", bf, XQ, tok);
  check_eta(last_eta, "last_eta", XQ, d.B, d.H, d.NC);
  check_tensor(ttt_norm_weight, "ttt_norm_weight", f32, XQ, {1, d.H, 1, 64});
  check_tensor(ttt_norm_bias, "ttt_norm_bias", f32, XQ, {1, d.H, 1, 64});
  check_tensor(W1_checkpoints, "W1_checkpoints", f32, XQ, {d.B, d.H, d.n, 64, 256});
  check_tensor(b1_checkpoints, "b1_checkpoints", f32, XQ, {d.B, d.H, d.n, 1, 256});
  check_tensor(W2_checkpoints, "W2_checkpoints", f32, XQ, {d.B, d.H, d.n, 256, 64});
  check_tensor(b2_checkpoints, "b2_checkpoints", f32, XQ, {d.B, d.H, d.n, 1, 64});
  check_tensor(Out, "Out", bf, XQ, tok);
  check_tensor(W1_init_group, "W1_init_group", f32, XQ, {d.B, d.H, g, 64, 256});
  check_tensor(b1_init_group, "b1_init_group", f32, XQ, {d.B, d.H, g, 1, 256});
  check_tensor(W2_init_group, "W2_init_group", f32, XQ, {d.B, d.H, g, 256, 64});
  check_tensor(b2_init_group, "b2_init_group", f32, XQ, {d.B, d.H, g, 1, 64});
  check_tensor(x_hat_ln_group, "x_hat_ln_group", bf, XQ, {d.B, d.H, g, 64, 64});
  check_tensor(std_ln_group, "std_ln_group", f32, XQ, {d.B, d.H, g, 64, 1});
  check_tensor(X2_group, "X2_group", bf, XQ, {d.B, d.H, g, 64, 256});
  check_tensor(Z1_group, "Z1_group", bf, XQ, {d.B, d.H, g, 64, 256});
  check_tensor(Z1_bar_group, "Z1_bar_group", bf, XQ, {d.B, d.H, g, 64, 256});
  check_tensor(X2_bar_group, "X2_bar_group", bf, XQ, {d.B, d.H, g, 64, 256});
  check_tensor(grad_l_wrt_Z2_group, "grad_l_wrt_Z2_group", bf, XQ, {d.B, d.H, g, 64, 64});
  check_tensor(grad_l_wrt_Z1_group, "grad_l_wrt_Z1_group", bf, XQ, {d.B, d.H, g, 64, 256});
  check_tensor(x_hat_fused_group, "x_hat_fused_group", bf, XQ, {d.B, d.H, g, 64, 64});
  check_tensor(grad_x_hat_fused_group, "grad_x_hat_fused_group", bf, XQ, {d.B, d.H, g, 64, 64});
  check_tensor(grad_output_fused_group, "grad_output_fused_group", bf, XQ, {d.B, d.H, g, 64, 64});
  check_tensor(std_fused_group, "std_fused_group", f32, XQ, {d.B, d.H, g, 64, 1});
  check_tensor(grad_L_W1_last, "grad_L_W1_last", f32, XQ, {d.B, d.H, 64, 256});
  check_tensor(grad_L_b1_last, "grad_L_b1_last", f32, XQ, {d.B, d.H, 1, 256});
  check_tensor(grad_L_W2_last, "grad_L_W2_last", f32, XQ, {d.B, d.H, 256, 64});
  check_tensor(grad_L_b2_last, "grad_L_b2_last", f32, XQ, {d.B, d.H, 1, 64});
  check_tensor(grad_L_XQW_mini_batch, "grad_L_XQW_mini_batch", bf, XQ, tok);
  check_tensor(grad_L_ttt_norm_weight, "grad_L_ttt_norm_weight", f32, XQ, {d.B, d.H, 1, 64});
  check_tensor(grad_L_ttt_norm_bias, "grad_L_ttt_norm_bias", f32, XQ, {d.B, d.H, 1, 64});
  check_tensor(grad_L_W1_init, "grad_L_W1_init", f32, XQ, {d.B, d.H, 64, 256});
  check_tensor(grad_L_b1_init, "grad_L_b1_init", f32, XQ, {d.B, d.H, 1, 256});
  check_tensor(grad_L_W2_init, "grad_L_W2_init", f32, XQ, {d.B, d.H, 256, 64});
  check_tensor(grad_L_b2_init, "grad_L_b2_init", f32, XQ, {d.B, d.H, 1, 64});
  check_eta(grad_L_last_eta, "grad_L_last_eta", XQ, d.B, d.H, d.NC);
  check_tensor(grad_L_XQ, "grad_L_XQ", bf, XQ, tok);
  check_tensor(grad_L_XK, "grad_L_XK", bf, XQ, tok);
  check_tensor(grad_L_XV, "grad_L_XV", bf, XQ, tok);

  const c10::cuda::CUDAGuard guard(XQ.device());
  ttt_b200_bwd_args a = {};
  a.XQ = XQ.data_ptr();
  a.XK = XK.data_ptr();
  a.XV = XV.data_ptr();
  a.last_eta = last_eta.data_ptr();
  a.ttt_norm_weight = ttt_norm_weight.data_ptr<float>();
  a.ttt_norm_bias = ttt_norm_bias.data_ptr<float>();
  a.W1_checkpoints = W1_checkpoints.data_ptr<float>();
  a.b1_checkpoints = b1_checkpoints.data_ptr<float>();
  a.W2_checkpoints = W2_checkpoints.data_ptr<float>();
  a.b2_checkpoints = b2_checkpoints.data_ptr<float>();
  a.Out = Out.data_ptr();
  a.W1_init_group = W1_init_group.data_ptr<float>();
  a.b1_init_group = b1_init_group.data_ptr<float>();
  a.W2_init_group = W2_init_group.data_ptr<float>();
  a.b2_init_group = b2_init_group.data_ptr<float>();
  a.x_hat_ln_group = x_hat_ln_group.data_ptr();
  a.std_ln_group = std_ln_group.data_ptr<float>();
  a.X2_group = X2_group.data_ptr();
  a.Z1_group = Z1_group.data_ptr();
  a.Z1_bar_group = Z1_bar_group.data_ptr();
  a.X2_bar_group = X2_bar_group.data_ptr();
  a.grad_l_wrt_Z2_group = grad_l_wrt_Z2_group.data_ptr();
  a.grad_l_wrt_Z1_group = grad_l_wrt_Z1_group.data_ptr();
  a.x_hat_fused_group = x_hat_fused_group.data_ptr();
  a.grad_x_hat_fused_group = grad_x_hat_fused_group.data_ptr();
  a.grad_output_fused_group = grad_output_fused_group.data_ptr();
  a.std_fused_group = std_fused_group.data_ptr<float>();
  a.grad_L_W1_last = grad_L_W1_last.data_ptr<float>();
  a.grad_L_b1_last = grad_L_b1_last.data_ptr<float>();
  a.grad_L_W2_last = grad_L_W2_last.data_ptr<float>();
  a.grad_L_b2_last = grad_L_b2_last.data_ptr<float>();
  a.grad_L_XQW_mini_batch = grad_L_XQW_mini_batch.data_ptr();
  a.grad_L_ttt_norm_weight = grad_L_ttt_norm_weight.data_ptr<float>();
  a.grad_L_ttt_norm_bias = grad_L_ttt_norm_bias.data_ptr<float>();
  a.grad_L_W1_init = grad_L_W1_init.data_ptr<float>();
  a.grad_L_b1_init = grad_L_b1_init.data_ptr<float>();
  a.grad_L_W2_init = grad_L_W2_init.data_ptr<float>();
  a.grad_L_b2_init = grad_L_b2_init.data_ptr<float>();
  a.grad_L_last_eta = grad_L_last_eta.data_ptr();
  a.grad_L_XQ = grad_L_XQ.data_ptr();
  a.grad_L_XK = grad_L_XK.data_ptr();
  a.grad_L_XV = grad_L_XV.data_ptr();
  a.B = static_cast<int32_t>(d.B);
  a.H = static_cast<int32_t>(d.H);
  a.NC = static_cast<int32_t>(d.NC);
  a.checkpoint_group_size = checkpoint_group_size;
  a.num_checkpoints = static_cast<int32_t>(d.n);
  a.flags = async_calls() ? 0u : TTT_B200_FLAG_SYNC;
  const int rc = ttt_b200_backward(&a, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "ttt_backward failed (code ", rc, "): ", ttt_b200_last_error());
  return Out;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "Test Time Training Kernels (B200 / sm_100a)";
  m.def("ttt_forward", &ttt_forward, "TTT Forward.");
  m.def("ttt_backward", &ttt_backward, "TTT Backward.");
}
