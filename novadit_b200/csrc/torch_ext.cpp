// pybind11 module `novadit_cuda`: the thin PyTorch layer over the C ABI.
//
// It exports the same 15 functions, with the same argument meaning, return values and error
// behaviour (TORCH_CHECK -> RuntimeError), as the reference's csrc/bindings.cpp:85-116, so
// novadit/ops/*.py of the reference can import this module unchanged. Each function validates its
// tensors the way the reference's entry points do, allocates the outputs with the input's options,
// and calls one entry point of include/novadit_b200.h on torch's current CUDA stream. There is
// no kernel code and no fallback here. One function is added: the one-pass backward
// (`fused_adaln_backward` / `fused_adarmsnorm_backward`).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "novadit_b200.h"

namespace {

#define ND_CHECK_INPUT(x)                                       \
  TORCH_CHECK((x).is_cuda(), #x " must be a CUDA tensor");      \
  TORCH_CHECK((x).is_contiguous(), #x " must be contiguous")

int dtype_id(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kHalf: return ND_F16;
    case at::kBFloat16: return ND_BF16;
    case at::kFloat: return ND_F32;
    default: return -1;
  }
}

void check_status(int status, const char* what) {
  TORCH_CHECK(status == ND_OK, what, " failed: ", nd_status_string(status),
              status == ND_ERR_LAUNCH ? " (" : "",
              status == ND_ERR_LAUNCH ? cudaGetErrorString(static_cast<cudaError_t>(nd_last_cuda_error())) : "",
              status == ND_ERR_LAUNCH ? ")" : "");
}

void* current_stream(const at::Tensor& t) {
  return static_cast<void*>(c10::cuda::getCurrentCUDAStream(t.get_device()).stream());
}

// csrc/ops/adaln_kernel.cu:863-889 and csrc/ops/adarmsnorm_kernel.cu (same rules)
void check_norm_inputs(const at::Tensor& x, const at::Tensor& scale, const at::Tensor& shift) {
  ND_CHECK_INPUT(x);
  ND_CHECK_INPUT(scale);
  ND_CHECK_INPUT(shift);
  TORCH_CHECK(x.dim() == 3, "x must have shape [B, S, H]");
  TORCH_CHECK(scale.dim() == 2 || scale.dim() == 3, "scale must have shape [B, H] or [B, 1, H]");
  TORCH_CHECK(shift.dim() == 2 || shift.dim() == 3, "shift must have shape [B, H] or [B, 1, H]");
  TORCH_CHECK(x.scalar_type() == scale.scalar_type(), "x and scale must have the same dtype");
  TORCH_CHECK(x.scalar_type() == shift.scalar_type(), "x and shift must have the same dtype");
  TORCH_CHECK(x.size(0) == scale.size(0), "scale batch dimension must match x");
  TORCH_CHECK(x.size(0) == shift.size(0), "shift batch dimension must match x");
  TORCH_CHECK(scale.size(-1) == x.size(-1), "scale hidden dimension must match x");
  TORCH_CHECK(shift.size(-1) == x.size(-1), "shift hidden dimension must match x");
  if (scale.dim() == 3) TORCH_CHECK(scale.size(1) == 1, "3D scale must have shape [B, 1, H]");
  if (shift.dim() == 3) TORCH_CHECK(shift.size(1) == 1, "3D shift must have shape [B, 1, H]");
  TORCH_CHECK(dtype_id(x) >= 0, "only fp16/bf16/fp32 tensors are supported");
}

void check_stat(const at::Tensor& stat, const at::Tensor& x, const char* name) {
  TORCH_CHECK(stat.is_cuda() && stat.is_contiguous(), name, " must be a contiguous CUDA tensor");
  TORCH_CHECK(stat.scalar_type() == at::kFloat, name, " must have dtype float32");
  TORCH_CHECK(stat.dim() == 2 && stat.size(0) == x.size(0) && stat.size(1) == x.size(1), name,
              " must have shape [B, S]");
  TORCH_CHECK(stat.device() == x.device(), "all backward tensors must be on the same device");
}

// csrc/ops/adaln_kernel.cu:891-951
void check_norm_backward(const at::Tensor& dy, const at::Tensor& x, const at::Tensor* scale) {
  ND_CHECK_INPUT(dy);
  ND_CHECK_INPUT(x);
  TORCH_CHECK(dy.dim() == 3, "dy must have shape [B, S, H]");
  TORCH_CHECK(x.dim() == 3, "x must have shape [B, S, H]");
  TORCH_CHECK(dy.sizes() == x.sizes(), "dy and x must have the same shape");
  TORCH_CHECK(dy.scalar_type() == x.scalar_type(), "dy and x must have the same dtype");
  TORCH_CHECK(dy.device() == x.device(), "all backward tensors must be on the same device");
  TORCH_CHECK(dtype_id(x) >= 0, "only fp16/bf16/fp32 tensors are supported");
  if (scale != nullptr) {
    ND_CHECK_INPUT(*scale);
    TORCH_CHECK(scale->dim() == 2 || scale->dim() == 3, "scale must have shape [B, H] or [B, 1, H]");
    TORCH_CHECK(scale->scalar_type() == x.scalar_type(), "scale and x must have the same dtype");
    TORCH_CHECK(scale->size(0) == x.size(0), "scale batch dimension must match x");
    TORCH_CHECK(scale->size(-1) == x.size(-1), "scale hidden dimension must match x");
    if (scale->dim() == 3) TORCH_CHECK(scale->size(1) == 1, "3D scale must have shape [B, 1, H]");
    TORCH_CHECK(scale->device() == x.device(), "all backward tensors must be on the same device");
  }
}

at::Tensor dparam_workspace(const at::Tensor& x, size_t* bytes) {
  const int64_t rows = x.size(0) * x.size(1);
  *bytes = nd_norm_dparam_ws_bytes(rows, 0, x.size(1), x.size(2));
  return at::empty({static_cast<int64_t>(*bytes)}, x.options().dtype(at::kByte));
}

// ------------------------------------------------------------------ norm forward
std::vector<at::Tensor> norm_forward(bool rms, bool stats, const at::Tensor& x, const at::Tensor& scale,
                                     const at::Tensor& shift, double eps) {
  check_norm_inputs(x, scale, shift);
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t B = x.size(0), S = x.size(1), H = x.size(2);
  at::Tensor scale_c = scale.reshape({B, H}).contiguous();
  at::Tensor shift_c = shift.reshape({B, H}).contiguous();
  at::Tensor y = at::empty_like(x);
  auto stat_opts = x.options().dtype(at::kFloat).requires_grad(false);
  at::Tensor mean, invstd;
  if (stats) {
    if (!rms) mean = at::empty({B, S}, stat_opts);
    invstd = at::empty({B, S}, stat_opts);
  }
  int st;
  if (rms) {
    st = nd_adarms_fwd(dtype_id(x), x.data_ptr(), scale_c.data_ptr(), shift_c.data_ptr(), y.data_ptr(),
                       stats ? invstd.data_ptr<float>() : nullptr, B * S, 0, S, H, static_cast<float>(eps),
                       current_stream(x));
  } else {
    st = nd_adaln_fwd(dtype_id(x), x.data_ptr(), scale_c.data_ptr(), shift_c.data_ptr(), y.data_ptr(),
                      stats ? mean.data_ptr<float>() : nullptr, stats ? invstd.data_ptr<float>() : nullptr, B * S,
                      0, S, H, static_cast<float>(eps), current_stream(x));
  }
  check_status(st, rms ? "fused_adarmsnorm_forward" : "fused_adaln_forward");
  if (!stats) return {y};
  if (rms) return {y, scale_c, invstd};
  return {y, scale_c, mean, invstd};
}

std::vector<at::Tensor> fused_adaln_forward(const at::Tensor& x, const at::Tensor& scale, const at::Tensor& shift,
                                            double eps) {
  return norm_forward(false, true, x, scale, shift, eps);
}
at::Tensor fused_adaln_forward_inference(const at::Tensor& x, const at::Tensor& scale, const at::Tensor& shift,
                                         double eps) {
  return norm_forward(false, false, x, scale, shift, eps)[0];
}
std::vector<at::Tensor> fused_adarmsnorm_forward(const at::Tensor& x, const at::Tensor& scale,
                                                 const at::Tensor& shift, double eps) {
  return norm_forward(true, true, x, scale, shift, eps);
}
at::Tensor fused_adarmsnorm_forward_inference(const at::Tensor& x, const at::Tensor& scale,
                                              const at::Tensor& shift, double eps) {
  return norm_forward(true, false, x, scale, shift, eps)[0];
}

// ------------------------------------------------------------------ norm backward
// mode: 1 = dx, 2 = dparam, 3 = both in one pass. Returns {dx} / {dscale, dshift} / {dx, dscale, dshift}.
std::vector<at::Tensor> norm_backward(bool rms, int mode, const at::Tensor& dy, const at::Tensor& x,
                                      const at::Tensor* scale, const at::Tensor* mean, const at::Tensor& invstd) {
  check_norm_backward(dy, x, scale);
  if (mean != nullptr) check_stat(*mean, x, "mean");
  check_stat(invstd, x, rms ? "inv_rms" : "invstd");
  if (mean != nullptr) TORCH_CHECK(invstd.sizes() == mean->sizes(), "invstd must have the same shape as mean");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t B = x.size(0), S = x.size(1), H = x.size(2);
  at::Tensor scale_c;
  if (scale != nullptr) scale_c = scale->reshape({B, H}).contiguous();
  at::Tensor dx, dscale, dshift, ws;
  size_t ws_bytes = 0;
  if (mode & 1) dx = at::empty_like(x);
  if (mode & 2) {
    auto grad_opts = x.options().dtype(at::kFloat).requires_grad(false);
    dscale = at::empty({B, H}, grad_opts);
    dshift = at::empty({B, H}, grad_opts);
    ws = dparam_workspace(x, &ws_bytes);
  }
  const int dt = dtype_id(x);
  void* stream = current_stream(x);
  const float* mean_p = mean != nullptr ? mean->data_ptr<float>() : nullptr;
  const float* inv_p = invstd.data_ptr<float>();
  int st;
  if (rms) {
    if (mode == 1)
      st = nd_adarms_bwd_dx(dt, dy.data_ptr(), x.data_ptr(), scale_c.data_ptr(), inv_p, dx.data_ptr(), B * S, 0, S, H,
                            stream);
    else if (mode == 2)
      st = nd_adarms_bwd_dparam(dt, dy.data_ptr(), x.data_ptr(), inv_p, dscale.data_ptr<float>(),
                                dshift.data_ptr<float>(), B * S, 0, S, H, ws.data_ptr(), ws_bytes, stream);
    else
      st = nd_adarms_bwd(dt, dy.data_ptr(), x.data_ptr(), scale_c.data_ptr(), inv_p, dx.data_ptr(),
                         dscale.data_ptr<float>(), dshift.data_ptr<float>(), B * S, 0, S, H, ws.data_ptr(), ws_bytes,
                         stream);
  } else {
    if (mode == 1)
      st = nd_adaln_bwd_dx(dt, dy.data_ptr(), x.data_ptr(), scale_c.data_ptr(), mean_p, inv_p, dx.data_ptr(), B * S, 0,
                           S, H, stream);
    else if (mode == 2)
      st = nd_adaln_bwd_dparam(dt, dy.data_ptr(), x.data_ptr(), mean_p, inv_p, dscale.data_ptr<float>(),
                               dshift.data_ptr<float>(), B * S, 0, S, H, ws.data_ptr(), ws_bytes, stream);
    else
      st = nd_adaln_bwd(dt, dy.data_ptr(), x.data_ptr(), scale_c.data_ptr(), mean_p, inv_p, dx.data_ptr(),
                        dscale.data_ptr<float>(), dshift.data_ptr<float>(), B * S, 0, S, H, ws.data_ptr(), ws_bytes,
                        stream);
  }
  check_status(st, rms ? "fused_adarmsnorm_backward" : "fused_adaln_backward");
  if (mode == 1) return {dx};
  if (mode == 2) return {dscale, dshift};
  return {dx, dscale, dshift};
}

at::Tensor fused_adaln_backward_dx(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& scale,
                                   const at::Tensor& mean, const at::Tensor& invstd) {
  return norm_backward(false, 1, dy, x, &scale, &mean, invstd)[0];
}
std::vector<at::Tensor> fused_adaln_backward_dparam(const at::Tensor& dy, const at::Tensor& x,
                                                    const at::Tensor& mean, const at::Tensor& invstd) {
  return norm_backward(false, 2, dy, x, nullptr, &mean, invstd);
}
std::vector<at::Tensor> fused_adaln_backward(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& scale,
                                             const at::Tensor& mean, const at::Tensor& invstd) {
  return norm_backward(false, 3, dy, x, &scale, &mean, invstd);
}
at::Tensor fused_adarmsnorm_backward_dx(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& scale,
                                        const at::Tensor& inv_rms) {
  return norm_backward(true, 1, dy, x, &scale, nullptr, inv_rms)[0];
}
std::vector<at::Tensor> fused_adarmsnorm_backward_dparam(const at::Tensor& dy, const at::Tensor& x,
                                                         const at::Tensor& inv_rms) {
  return norm_backward(true, 2, dy, x, nullptr, nullptr, inv_rms);
}
std::vector<at::Tensor> fused_adarmsnorm_backward(const at::Tensor& dy, const at::Tensor& x,
                                                  const at::Tensor& scale, const at::Tensor& inv_rms) {
  return norm_backward(true, 3, dy, x, &scale, nullptr, inv_rms);
}

// ------------------------------------------------------------------ gate-act
// csrc/ops/gate_act_kernel.cu:520-525
void check_gate_act_inputs(const at::Tensor& z) {
  ND_CHECK_INPUT(z);
  TORCH_CHECK(z.dim() == 3, "z must have shape [B, S, 2*I]");
  TORCH_CHECK(z.size(2) % 2 == 0, "z last dim must be even (2 * intermediate_size)");
}

at::Tensor fused_gate_act_forward(const at::Tensor& x, int64_t act_id) {
  check_gate_act_inputs(x);
  TORCH_CHECK(act_id == 0 || act_id == 1, "act_id must be 0 (SiLU) or 1 (GELU), got ", act_id);
  TORCH_CHECK(dtype_id(x) >= 0, "fused_gate_act_forward only supports fp32/fp16/bf16 tensors");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t I = x.size(2) / 2;
  at::Tensor y = at::empty({x.size(0), x.size(1), I}, x.options());
  check_status(nd_gate_act_fwd(dtype_id(x), static_cast<int>(act_id), x.data_ptr(), y.data_ptr(),
                               x.size(0) * x.size(1), I, current_stream(x)),
               "fused_gate_act_forward");
  return y;
}

at::Tensor fused_gate_act_backward(const at::Tensor& dy, const at::Tensor& x, int64_t act_id) {
  check_gate_act_inputs(x);
  TORCH_CHECK(act_id == 0 || act_id == 1, "act_id must be 0 (SiLU) or 1 (GELU), got ", act_id);
  TORCH_CHECK(dtype_id(x) >= 0, "fused_gate_act_backward only supports fp32/fp16/bf16 tensors");
  TORCH_CHECK(dy.is_cuda(), "dy must be a CUDA tensor");
  TORCH_CHECK(dy.dim() == 3 && dy.size(0) == x.size(0) && dy.size(1) == x.size(1) && dy.size(2) * 2 == x.size(2),
              "dy must have shape [B, S, I]");
  TORCH_CHECK(dy.scalar_type() == x.scalar_type(), "dy and x must have the same dtype");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor dy_c = dy.contiguous();  // the reference makes dy contiguous itself (gate_act_kernel.cu:740,796)
  at::Tensor dz = at::empty_like(x);
  check_status(nd_gate_act_bwd(dtype_id(x), static_cast<int>(act_id), dy_c.data_ptr(), x.data_ptr(), dz.data_ptr(),
                               x.size(0) * x.size(1), x.size(2) / 2, current_stream(x)),
               "fused_gate_act_backward");
  return dz;
}

// Activation backward of FC1's pre-activation z [B, S, 2I] = [gate | value] (no counterpart in the reference's
// extension: its autograd Function does this step in eager PyTorch, novadit/ops/fc1_bias_act.py:255-270).
at::Tensor fused_gate_act_backward_gate_first(const at::Tensor& dy, const at::Tensor& z, int64_t act_id) {
  check_gate_act_inputs(z);
  TORCH_CHECK(act_id == 0 || act_id == 1, "act_id must be 0 (SiLU) or 1 (GELU), got ", act_id);
  TORCH_CHECK(dtype_id(z) >= 0, "fused_gate_act_backward_gate_first only supports fp32/fp16/bf16 tensors");
  TORCH_CHECK(dy.is_cuda(), "dy must be a CUDA tensor");
  TORCH_CHECK(dy.dim() == 3 && dy.size(0) == z.size(0) && dy.size(1) == z.size(1) && dy.size(2) * 2 == z.size(2),
              "dy must have shape [B, S, I]");
  TORCH_CHECK(dy.scalar_type() == z.scalar_type(), "dy and z must have the same dtype");
  c10::cuda::CUDAGuard guard(z.device());
  at::Tensor dy_c = dy.contiguous();
  at::Tensor dz = at::empty_like(z);
  check_status(nd_gate_act_bwd_gate_first(dtype_id(z), static_cast<int>(act_id), dy_c.data_ptr(), z.data_ptr(),
                                          dz.data_ptr(), z.size(0) * z.size(1), z.size(2) / 2, current_stream(z)),
               "fused_gate_act_backward_gate_first");
  return dz;
}

at::Tensor fused_geglu_forward(const at::Tensor& z) { return fused_gate_act_forward(z, ND_ACT_GELU); }
at::Tensor fused_geglu_backward(const at::Tensor& dy, const at::Tensor& z) {
  return fused_gate_act_backward(dy, z, ND_ACT_GELU);
}

// ------------------------------------------------------------------ FC1
// csrc/ops/fc1_bias_act_kernel.cu:14-50. `layout`: 2 = rows interleaved (gate0, value0, ...), which is what the
// reference's Python passes to fused_fc1_bias_act_forward; 1 = [gate block | value block] (the nn.Linear weight
// as stored, no re-layout copy); 0 = no gating, y = act(z).
at::Tensor fc1_forward(const at::Tensor& x, const at::Tensor& weight, c10::optional<at::Tensor> bias, int64_t act_id,
                       int layout) {
  TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor");
  TORCH_CHECK(weight.is_cuda(), "weight must be a CUDA tensor");
  TORCH_CHECK(x.is_contiguous(), "x must be contiguous");
  TORCH_CHECK(weight.is_contiguous(), "weight must be contiguous");
  TORCH_CHECK(x.dim() == 3, "x must have shape [batch, seq, hidden]");
  TORCH_CHECK(weight.dim() == 2, "weight must have shape [2 * intermediate, hidden]");
  TORCH_CHECK(layout == 0 || weight.size(0) % 2 == 0, "weight.size(0) must be even");
  TORCH_CHECK(weight.size(1) == x.size(2), "weight hidden dimension must match x.size(2)");
  TORCH_CHECK(x.scalar_type() == weight.scalar_type(), "x and weight must have the same dtype");
  TORCH_CHECK(x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16,
              "fused_fc1_bias_act_forward supports fp16 and bf16 inputs");
  TORCH_CHECK(act_id == 0 || act_id == 1, "act_id must be 0 (SiLU) or 1 (GELU)");
  const void* bias_p = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda(), "bias must be a CUDA tensor");
    TORCH_CHECK(bias->is_contiguous(), "bias must be contiguous");
    TORCH_CHECK(bias->dim() == 1, "bias must have shape [2 * intermediate]");
    TORCH_CHECK(bias->size(0) == weight.size(0), "bias.size(0) must match weight.size(0)");
    TORCH_CHECK(bias->scalar_type() == x.scalar_type(), "bias dtype must match x dtype");
    bias_p = bias->data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t n = weight.size(0);
  const int64_t n_out = layout == 0 ? n : n / 2;
  at::Tensor y = at::empty({x.size(0), x.size(1), n_out}, x.options());
  check_status(nd_fc1_fwd(dtype_id(x), dtype_id(x), static_cast<int>(act_id), layout, x.data_ptr(), weight.data_ptr(),
                          bias_p, 1.0f, nullptr, y.data_ptr(), x.size(0) * x.size(1), x.size(2), n, nullptr,
                          current_stream(x)),
               "fused_fc1_bias_act_forward");
  return y;
}

at::Tensor fused_fc1_bias_act_forward(const at::Tensor& x, const at::Tensor& weight, c10::optional<at::Tensor> bias,
                                      int64_t act_id) {
  return fc1_forward(x, weight, bias, act_id, 2);
}
at::Tensor fused_fc1_bias_act_forward_stacked(const at::Tensor& x, const at::Tensor& weight,
                                              c10::optional<at::Tensor> bias, int64_t act_id) {
  return fc1_forward(x, weight, bias, act_id, 1);
}
at::Tensor fused_fc1_bias_act_forward_plain(const at::Tensor& x, const at::Tensor& weight,
                                            c10::optional<at::Tensor> bias, int64_t act_id) {
  return fc1_forward(x, weight, bias, act_id, 0);
}

// dz [B, S, 2I] from x [B, S, H], the FC1 weight [2I, H] (rows [gate | value]), its bias and dy [B, S, I]: the
// recomputation of z and the activation backward of novadit/ops/fc1_bias_act.py:255-270 in one tcgen05 launch.
at::Tensor fused_fc1_bias_act_backward_dz(const at::Tensor& x, const at::Tensor& weight, c10::optional<at::Tensor> bias,
                                          const at::Tensor& dy, int64_t act_id) {
  TORCH_CHECK(x.is_cuda() && weight.is_cuda() && dy.is_cuda(), "x, weight and dy must be CUDA tensors");
  TORCH_CHECK(x.dim() == 3 && weight.dim() == 2 && weight.size(1) == x.size(2) && weight.size(0) % 2 == 0,
              "x must be [batch, seq, hidden] and weight [2 * intermediate, hidden]");
  TORCH_CHECK(dy.dim() == 3 && dy.size(0) == x.size(0) && dy.size(1) == x.size(1) && dy.size(2) * 2 == weight.size(0),
              "dy must have shape [batch, seq, intermediate]");
  TORCH_CHECK(x.scalar_type() == weight.scalar_type() && x.scalar_type() == dy.scalar_type(), "x, weight, dy: one dtype");
  TORCH_CHECK(x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16, "fp16 and bf16 only");
  TORCH_CHECK(act_id == 0 || act_id == 1, "act_id must be 0 (SiLU) or 1 (GELU)");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor xc = x.contiguous(), wc = weight.contiguous(), dyc = dy.contiguous(), bc;
  const void* bias_p = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->numel() == weight.size(0) && bias->scalar_type() == x.scalar_type(),
                "bias must be a CUDA tensor of 2 * intermediate elements with x's dtype");
    bc = bias->contiguous();
    bias_p = bc.data_ptr();
  }
  at::Tensor dz = at::empty({x.size(0), x.size(1), weight.size(0)}, x.options());
  check_status(nd_fc1_bwd_dz(dtype_id(x), static_cast<int>(act_id), xc.data_ptr(), wc.data_ptr(), bias_p, dyc.data_ptr(),
                             dz.data_ptr(), x.size(0) * x.size(1), x.size(2), weight.size(0), nullptr, current_stream(x)),
               "fused_fc1_bias_act_backward_dz");
  return dz;
}

// The same launch returning dbias [2I] as well (dz summed over the tokens inside the epilogue, a second small launch
// adds the per-warp partials): the `dz_flat.sum(dim=0)` of novadit/ops/fc1_bias_act.py:279 without reading dz again.
std::vector<at::Tensor> fused_fc1_bias_act_backward_dz_dbias(const at::Tensor& x, const at::Tensor& weight,
                                                             c10::optional<at::Tensor> bias, const at::Tensor& dy,
                                                             int64_t act_id) {
  TORCH_CHECK(x.is_cuda() && weight.is_cuda() && dy.is_cuda(), "x, weight and dy must be CUDA tensors");
  TORCH_CHECK(x.dim() == 3 && weight.dim() == 2 && weight.size(1) == x.size(2) && weight.size(0) % 2 == 0,
              "x must be [batch, seq, hidden] and weight [2 * intermediate, hidden]");
  TORCH_CHECK(dy.dim() == 3 && dy.size(0) == x.size(0) && dy.size(1) == x.size(1) && dy.size(2) * 2 == weight.size(0),
              "dy must have shape [batch, seq, intermediate]");
  TORCH_CHECK(x.scalar_type() == weight.scalar_type() && x.scalar_type() == dy.scalar_type(), "x, weight, dy: one dtype");
  TORCH_CHECK(x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16, "fp16 and bf16 only");
  TORCH_CHECK(act_id == 0 || act_id == 1, "act_id must be 0 (SiLU) or 1 (GELU)");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor xc = x.contiguous(), wc = weight.contiguous(), dyc = dy.contiguous(), bc;
  const void* bias_p = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->numel() == weight.size(0) && bias->scalar_type() == x.scalar_type(),
                "bias must be a CUDA tensor of 2 * intermediate elements with x's dtype");
    bc = bias->contiguous();
    bias_p = bc.data_ptr();
  }
  const int64_t m = x.size(0) * x.size(1), n = weight.size(0);
  at::Tensor dz = at::empty({x.size(0), x.size(1), n}, x.options());
  at::Tensor dbias = at::empty({n}, x.options());
  const int64_t ws_bytes = static_cast<int64_t>(nd_fc1_bwd_dbias_ws_bytes(m, n));
  at::Tensor ws = at::empty({ws_bytes > 16 ? ws_bytes : 16}, x.options().dtype(at::kByte));
  check_status(nd_fc1_bwd_dz_dbias(dtype_id(x), static_cast<int>(act_id), xc.data_ptr(), wc.data_ptr(), bias_p,
                                   dyc.data_ptr(), dz.data_ptr(), dbias.data_ptr(), ws.data_ptr(), ws.numel(), m,
                                   x.size(2), n, nullptr, current_stream(x)),
               "fused_fc1_bias_act_backward_dz_dbias");
  return {dz, dbias};
}

// dx = dz @ weight for dz [B, S, 2I] and the FC1 weight [2I, H]: the job of the reference's CuTe-DSL backward-dx
// kernel (csrc/cute_dsl/fc1_bias_act/fc1_bias_act.py:996-1913 behind novadit/ops/fc1_bias_act.py:288-326), on the
// tcgen05 GEMM that reads the weight in place as an MN-major operand (the reference copies and transposes both
// weight halves per call, :309-315).
at::Tensor fused_fc1_bias_act_backward_dx(const at::Tensor& dz, const at::Tensor& weight) {
  TORCH_CHECK(dz.is_cuda() && weight.is_cuda(), "dz and weight must be CUDA tensors");
  TORCH_CHECK(dz.dim() == 3, "dz must have shape [batch, seq, 2 * intermediate]");
  TORCH_CHECK(weight.dim() == 2 && weight.size(0) == dz.size(2), "weight must have shape [2 * intermediate, hidden]");
  TORCH_CHECK(dz.scalar_type() == weight.scalar_type(), "dz and weight must have the same dtype");
  TORCH_CHECK(dz.scalar_type() == at::kHalf || dz.scalar_type() == at::kBFloat16,
              "fused_fc1_bias_act_backward_dx supports fp16 and bf16 inputs");
  c10::cuda::CUDAGuard guard(dz.device());
  at::Tensor dzc = dz.contiguous(), wc = weight.contiguous();
  at::Tensor dx = at::empty({dz.size(0), dz.size(1), weight.size(1)}, dz.options());
  at::Tensor ws = at::empty({static_cast<int64_t>(nd_fc1_bwd_gemm_ws_bytes())}, dz.options().dtype(at::kByte));
  check_status(nd_fc1_bwd_gemm(dtype_id(dz), 0, dzc.data_ptr(), wc.data_ptr(), dx.data_ptr(), dz.size(0) * dz.size(1),
                               weight.size(1), dz.size(2), ws.data_ptr(), ws.numel(), nullptr, current_stream(dz)),
               "fused_fc1_bias_act_backward_dx");
  return dx;
}

// dW [2I, H] = dz^T @ x for dz [B, S, 2I] and x [B, S, H] (novadit/ops/fc1_bias_act.py:276), both read in place
at::Tensor fused_fc1_bias_act_backward_dw(const at::Tensor& dz, const at::Tensor& x) {
  TORCH_CHECK(dz.is_cuda() && x.is_cuda(), "dz and x must be CUDA tensors");
  TORCH_CHECK(dz.dim() == 3 && x.dim() == 3 && dz.size(0) == x.size(0) && dz.size(1) == x.size(1),
              "dz [batch, seq, 2 * intermediate] and x [batch, seq, hidden]");
  TORCH_CHECK(dz.scalar_type() == x.scalar_type(), "dz and x must have the same dtype");
  TORCH_CHECK(dz.scalar_type() == at::kHalf || dz.scalar_type() == at::kBFloat16,
              "fused_fc1_bias_act_backward_dw supports fp16 and bf16 inputs");
  c10::cuda::CUDAGuard guard(dz.device());
  at::Tensor dzc = dz.contiguous(), xc = x.contiguous();
  at::Tensor dw = at::empty({dz.size(2), x.size(2)}, dz.options());
  at::Tensor ws = at::empty({static_cast<int64_t>(nd_fc1_bwd_gemm_ws_bytes())}, dz.options().dtype(at::kByte));
  check_status(nd_fc1_bwd_gemm(dtype_id(dz), 1, dzc.data_ptr(), xc.data_ptr(), dw.data_ptr(), dz.size(2), x.size(2),
                               dz.size(0) * dz.size(1), ws.data_ptr(), ws.numel(), nullptr, current_stream(dz)),
               "fused_fc1_bias_act_backward_dw");
  return dw;
}

// dbias [2I] = sum of dz [B, S, 2I] over batch and sequence (novadit/ops/fc1_bias_act.py:279), fp32 accumulation
at::Tensor fused_fc1_bias_act_backward_dbias(const at::Tensor& dz) {
  TORCH_CHECK(dz.is_cuda() && dz.dim() == 3, "dz must be a CUDA tensor of shape [batch, seq, 2 * intermediate]");
  TORCH_CHECK(dz.scalar_type() == at::kHalf || dz.scalar_type() == at::kBFloat16,
              "fused_fc1_bias_act_backward_dbias supports fp16 and bf16 inputs");
  c10::cuda::CUDAGuard guard(dz.device());
  at::Tensor dzc = dz.contiguous();
  const int64_t cols = dz.size(2);
  at::Tensor ws = at::empty({static_cast<int64_t>(nd_colsum_ws_bytes(cols))}, dz.options().dtype(at::kByte));
  at::Tensor out = at::empty({cols}, dz.options());
  check_status(nd_colsum(dtype_id(dz), dzc.data_ptr(), dz.size(0) * dz.size(1), cols, out.data_ptr(), ws.data_ptr(),
                         ws.numel(), current_stream(dz)),
               "fused_fc1_bias_act_backward_dbias");
  return out;
}

// ------------------------------------------------------------------ row operators next to the path
// The reference binds these two names (csrc/bindings.cpp:91-96) to kernels that raise
// (csrc/ops/qkv_pack_kernel.cu:5-10, csrc/ops/residual_kernel.cu:3-8); here they run.
std::vector<at::Tensor> fused_qkv_pack_forward(const at::Tensor& qkv, int64_t num_heads, int64_t head_dim) {
  TORCH_CHECK(qkv.is_cuda(), "qkv must be a CUDA tensor");
  TORCH_CHECK(qkv.dim() == 3, "qkv must have shape [B, S, 3 * num_heads * head_dim]");
  TORCH_CHECK(num_heads > 0 && head_dim > 0, "num_heads and head_dim must be positive");
  const int64_t hidden = num_heads * head_dim;
  TORCH_CHECK(qkv.size(2) == 3 * hidden, "Expected last dim ", 3 * hidden, ", got ", qkv.size(2));
  TORCH_CHECK(dtype_id(qkv) >= 0, "fused_qkv_pack_forward only supports fp32/fp16/bf16 tensors");
  c10::cuda::CUDAGuard guard(qkv.device());
  at::Tensor src = qkv.contiguous();
  std::vector<at::Tensor> out;
  for (int i = 0; i < 3; ++i) out.push_back(at::empty({qkv.size(0), qkv.size(1), num_heads, head_dim}, qkv.options()));
  check_status(nd_qkv_pack_fwd(dtype_id(qkv), src.data_ptr(), out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                               qkv.size(0) * qkv.size(1), hidden, current_stream(qkv)),
               "fused_qkv_pack_forward");
  return out;
}

// backward of the pack: dq, dk, dv [B, S, heads, head_dim] -> dqkv [B, S, 3 * hidden] (added; not in the reference)
at::Tensor fused_qkv_pack_backward(const at::Tensor& dq, const at::Tensor& dk, const at::Tensor& dv) {
  TORCH_CHECK(dq.is_cuda() && dk.is_cuda() && dv.is_cuda(), "dq, dk, dv must be CUDA tensors");
  TORCH_CHECK(dq.dim() == 4 && dq.sizes() == dk.sizes() && dq.sizes() == dv.sizes(),
              "dq, dk, dv must have the same shape [B, S, num_heads, head_dim]");
  TORCH_CHECK(dq.scalar_type() == dk.scalar_type() && dq.scalar_type() == dv.scalar_type(), "dq, dk, dv must have one dtype");
  TORCH_CHECK(dtype_id(dq) >= 0, "fused_qkv_pack_backward only supports fp32/fp16/bf16 tensors");
  c10::cuda::CUDAGuard guard(dq.device());
  at::Tensor q = dq.contiguous(), k = dk.contiguous(), v = dv.contiguous();
  const int64_t hidden = dq.size(2) * dq.size(3);
  at::Tensor dqkv = at::empty({dq.size(0), dq.size(1), 3 * hidden}, dq.options());
  check_status(nd_qkv_pack_bwd(dtype_id(dq), q.data_ptr(), k.data_ptr(), v.data_ptr(), dqkv.data_ptr(),
                               dq.size(0) * dq.size(1), hidden, current_stream(dq)),
               "fused_qkv_pack_backward");
  return dqkv;
}

at::Tensor fused_out_residual_forward(const at::Tensor& x, const at::Tensor& residual, c10::optional<at::Tensor> bias) {
  TORCH_CHECK(x.is_cuda() && residual.is_cuda(), "x and residual must be CUDA tensors");
  TORCH_CHECK(x.dim() == 3, "x must have shape [B, S, H]");
  TORCH_CHECK(residual.sizes() == x.sizes(), "residual must have the same shape as x");
  TORCH_CHECK(residual.scalar_type() == x.scalar_type(), "x and residual must have the same dtype");
  TORCH_CHECK(dtype_id(x) >= 0, "fused_out_residual_forward only supports fp32/fp16/bf16 tensors");
  const void* bias_p = nullptr;
  at::Tensor bias_c;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda(), "bias must be a CUDA tensor");
    TORCH_CHECK(bias->numel() == x.size(2), "bias must have H elements");
    TORCH_CHECK(bias->scalar_type() == x.scalar_type(), "bias dtype must match x dtype");
    bias_c = bias->contiguous();
    bias_p = bias_c.data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor xc = x.contiguous(), rc = residual.contiguous();
  at::Tensor y = at::empty_like(xc);
  check_status(nd_out_residual_fwd(dtype_id(x), xc.data_ptr(), rc.data_ptr(), bias_p, y.data_ptr(),
                                   x.size(0) * x.size(1), x.size(2), current_stream(x)),
               "fused_out_residual_forward");
  return y;
}

// ------------------------------------------------------------------ added operators (no counterpart in the reference)
// Every function below validates and allocates like the ones above; they exist so that the Python operators of
// novadit_b200.ops reach the C ABI through this module (checks, device guard, torch's stream) and never around it.

void check_gate(const at::Tensor& gate, const at::Tensor& x) {
  ND_CHECK_INPUT(gate);
  TORCH_CHECK(gate.dim() == 2 && gate.size(0) == x.size(0) && gate.size(1) == x.size(2), "gate must have shape [B, H]");
  TORCH_CHECK(gate.scalar_type() == x.scalar_type(), "gate and x must have the same dtype");
  TORCH_CHECK(gate.device() == x.device(), "gate must be on x's device");
}

void check_same(const at::Tensor& t, const at::Tensor& x, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous(), name, " must be a contiguous CUDA tensor");
  TORCH_CHECK(t.sizes() == x.sizes() && t.scalar_type() == x.scalar_type() && t.device() == x.device(), name,
              " must have x's shape, dtype and device");
}

// x_new = x + gate * branch (gate optional) and its norm in one pass -> [x_new, y, scale[B,H], mean, invstd] (AdaLN)
// or [x_new, y, scale[B,H], inv_rms] (AdaRMSNorm)
std::vector<at::Tensor> residual_norm_forward(bool rms, const at::Tensor& x, const at::Tensor& branch,
                                              c10::optional<at::Tensor> gate, const at::Tensor& scale,
                                              const at::Tensor& shift, double eps) {
  check_norm_inputs(x, scale, shift);
  check_same(branch, x, "branch");
  const void* gate_p = nullptr;
  if (gate.has_value() && gate->defined()) {
    check_gate(*gate, x);
    gate_p = gate->data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t B = x.size(0), S = x.size(1), H = x.size(2);
  at::Tensor scale_c = scale.reshape({B, H}).contiguous(), shift_c = shift.reshape({B, H}).contiguous();
  at::Tensor x_new = at::empty_like(x), y = at::empty_like(x);
  auto stat_opts = x.options().dtype(at::kFloat).requires_grad(false);
  at::Tensor invstd = at::empty({B, S}, stat_opts), mean;
  int st;
  if (rms) {
    st = nd_adarms_fwd_residual(dtype_id(x), x.data_ptr(), branch.data_ptr(), gate_p, scale_c.data_ptr(), shift_c.data_ptr(),
                                x_new.data_ptr(), y.data_ptr(), invstd.data_ptr<float>(), B * S, 0, S, H,
                                static_cast<float>(eps), current_stream(x));
  } else {
    mean = at::empty({B, S}, stat_opts);
    st = nd_adaln_fwd_residual(dtype_id(x), x.data_ptr(), branch.data_ptr(), gate_p, scale_c.data_ptr(), shift_c.data_ptr(),
                               x_new.data_ptr(), y.data_ptr(), mean.data_ptr<float>(), invstd.data_ptr<float>(), B * S, 0,
                               S, H, static_cast<float>(eps), current_stream(x));
  }
  check_status(st, rms ? "fused_residual_adarmsnorm_forward" : "fused_residual_adaln_forward");
  if (rms) return {x_new, y, scale_c, invstd};
  return {x_new, y, scale_c, mean, invstd};
}
std::vector<at::Tensor> fused_residual_adaln_forward(const at::Tensor& x, const at::Tensor& branch,
                                                     c10::optional<at::Tensor> gate, const at::Tensor& scale,
                                                     const at::Tensor& shift, double eps) {
  return residual_norm_forward(false, x, branch, gate, scale, shift, eps);
}
std::vector<at::Tensor> fused_residual_adarmsnorm_forward(const at::Tensor& x, const at::Tensor& branch,
                                                          c10::optional<at::Tensor> gate, const at::Tensor& scale,
                                                          const at::Tensor& shift, double eps) {
  return residual_norm_forward(true, x, branch, gate, scale, shift, eps);
}

constexpr int64_t kGatedTileRows = 8;

at::Tensor fused_gated_residual_forward(const at::Tensor& x, const at::Tensor& branch, const at::Tensor& gate) {
  ND_CHECK_INPUT(x);
  TORCH_CHECK(x.dim() == 3 && dtype_id(x) >= 0, "x must be a [B, S, H] fp32/fp16/bf16 tensor");
  check_same(branch, x, "branch");
  check_gate(gate, x);
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty_like(x);
  check_status(nd_gated_residual_fwd(dtype_id(x), x.data_ptr(), branch.data_ptr(), gate.data_ptr(), y.data_ptr(),
                                     x.size(0) * x.size(1), 0, x.size(1), x.size(2), current_stream(x)),
               "fused_gated_residual_forward");
  return y;
}

// backward of y = x + gate * branch for the incoming gradient dy, optionally with a second gradient `dres` of y added
// first: -> [dsum (= dy when there is no dres), dbranch, dgate [B, H] fp32]
std::vector<at::Tensor> fused_gated_residual_backward(const at::Tensor& dy, c10::optional<at::Tensor> dres,
                                                      const at::Tensor& branch, const at::Tensor& gate) {
  ND_CHECK_INPUT(dy);
  TORCH_CHECK(dy.dim() == 3 && dtype_id(dy) >= 0, "dy must be a [B, S, H] fp32/fp16/bf16 tensor");
  check_same(branch, dy, "branch");
  check_gate(gate, dy);
  const bool add = dres.has_value() && dres->defined();
  if (add) check_same(*dres, dy, "dres");
  c10::cuda::CUDAGuard guard(dy.device());
  const int64_t B = dy.size(0), S = dy.size(1), H = dy.size(2);
  const int64_t tiles = (S + kGatedTileRows - 1) / kGatedTileRows;
  at::Tensor part = at::empty({B, tiles, H}, dy.options().dtype(at::kFloat));
  at::Tensor dbranch = at::empty_like(dy), dsum = add ? at::empty_like(dy) : dy;
  int st;
  if (add) {
    st = nd_gated_residual_bwd_add(dtype_id(dy), dy.data_ptr(), dres->data_ptr(), branch.data_ptr(), gate.data_ptr(),
                                   dsum.data_ptr(), dbranch.data_ptr(), part.data_ptr<float>(), B * S, 0, S, H,
                                   kGatedTileRows, current_stream(dy));
  } else {
    st = nd_gated_residual_bwd(dtype_id(dy), dy.data_ptr(), branch.data_ptr(), gate.data_ptr(), dbranch.data_ptr(),
                               part.data_ptr<float>(), B * S, 0, S, H, kGatedTileRows, current_stream(dy));
  }
  check_status(st, "fused_gated_residual_backward");
  return {dsum, dbranch, part.sum(1)};  // the tiles of a sample, summed in one fixed order
}

// AdaLN / AdaRMSNorm forward with FP8 e4m3 output under a caller-given scale (delayed scaling): -> [q, scale[B,H],
// mean, invstd] / [q, scale[B,H], inv_rms]; `amax` (optional device float) receives max(amax, max |y|)
std::vector<at::Tensor> norm_forward_e4m3(bool rms, const at::Tensor& x, const at::Tensor& scale, const at::Tensor& shift,
                                          double eps, const at::Tensor& q_scale, c10::optional<at::Tensor> amax) {
  check_norm_inputs(x, scale, shift);
  TORCH_CHECK(q_scale.is_cuda() && q_scale.scalar_type() == at::kFloat && q_scale.numel() == 1 &&
                  q_scale.device() == x.device(), "q_scale must be one float32 on x's device");
  float* amax_p = nullptr;
  if (amax.has_value() && amax->defined()) {
    TORCH_CHECK(amax->is_cuda() && amax->scalar_type() == at::kFloat && amax->numel() == 1 && amax->device() == x.device(),
                "amax must be one float32 on x's device");
    amax_p = amax->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t B = x.size(0), S = x.size(1), H = x.size(2);
  at::Tensor scale_c = scale.reshape({B, H}).contiguous(), shift_c = shift.reshape({B, H}).contiguous();
  at::Tensor q = at::empty(x.sizes(), x.options().dtype(at::kFloat8_e4m3fn));
  auto stat_opts = x.options().dtype(at::kFloat).requires_grad(false);
  at::Tensor invstd = at::empty({B, S}, stat_opts), mean;
  int st;
  if (rms) {
    st = nd_adarms_fwd_e4m3(dtype_id(x), x.data_ptr(), scale_c.data_ptr(), shift_c.data_ptr(), q.data_ptr(),
                            invstd.data_ptr<float>(), q_scale.data_ptr<float>(), amax_p, B * S, 0, S, H,
                            static_cast<float>(eps), current_stream(x));
  } else {
    mean = at::empty({B, S}, stat_opts);
    st = nd_adaln_fwd_e4m3(dtype_id(x), x.data_ptr(), scale_c.data_ptr(), shift_c.data_ptr(), q.data_ptr(),
                           mean.data_ptr<float>(), invstd.data_ptr<float>(), q_scale.data_ptr<float>(), amax_p, B * S, 0, S,
                           H, static_cast<float>(eps), current_stream(x));
  }
  check_status(st, rms ? "fused_adarmsnorm_forward_e4m3" : "fused_adaln_forward_e4m3");
  if (rms) return {q, scale_c, invstd};
  return {q, scale_c, mean, invstd};
}
std::vector<at::Tensor> fused_adaln_forward_e4m3(const at::Tensor& x, const at::Tensor& scale, const at::Tensor& shift,
                                                 double eps, const at::Tensor& q_scale, c10::optional<at::Tensor> amax) {
  return norm_forward_e4m3(false, x, scale, shift, eps, q_scale, amax);
}
std::vector<at::Tensor> fused_adarmsnorm_forward_e4m3(const at::Tensor& x, const at::Tensor& scale, const at::Tensor& shift,
                                                      double eps, const at::Tensor& q_scale, c10::optional<at::Tensor> amax) {
  return norm_forward_e4m3(true, x, scale, shift, eps, q_scale, amax);
}

// per-tensor amax scaling to e4m3 on the device: -> [q, scale (one float32: amax / 448)]
std::vector<at::Tensor> quantize_e4m3(const at::Tensor& x) {
  ND_CHECK_INPUT(x);
  TORCH_CHECK(dtype_id(x) >= 0, "quantize_e4m3 supports fp32/fp16/bf16 tensors");
  c10::cuda::CUDAGuard guard(x.device());
  auto f32 = x.options().dtype(at::kFloat);
  at::Tensor ws = at::empty({static_cast<int64_t>(nd_amax_ws_bytes())}, x.options().dtype(at::kByte));  // per call: no sharing across streams
  at::Tensor amax = at::empty({1}, f32), scale = at::empty({1}, f32);
  at::Tensor q = at::empty(x.sizes(), x.options().dtype(at::kFloat8_e4m3fn));
  check_status(nd_amax(dtype_id(x), x.data_ptr(), x.numel(), amax.data_ptr<float>(), ws.data_ptr(), ws.numel(),
                       current_stream(x)), "quantize_e4m3 (amax)");
  check_status(nd_quant_e4m3(dtype_id(x), x.data_ptr(), x.numel(), amax.data_ptr<float>(), q.data_ptr(),
                             scale.data_ptr<float>(), current_stream(x)), "quantize_e4m3");
  return {q, scale};
}

// FC1 on e4m3 operands: x_q [B, S, H], w_q [N, H] (rows [gate | value] when gated), bias (16-bit, optional),
// scales = two device floats (x's and w's de-quantisation scales) -> y in `out_bf16 ? bf16 : fp16`
at::Tensor fused_fc1_bias_act_forward_fp8(const at::Tensor& x_q, const at::Tensor& w_q, c10::optional<at::Tensor> bias,
                                          const at::Tensor& scales, int64_t act_id, bool gated, bool out_bf16) {
  ND_CHECK_INPUT(x_q);
  ND_CHECK_INPUT(w_q);
  TORCH_CHECK(x_q.scalar_type() == at::kFloat8_e4m3fn && w_q.scalar_type() == at::kFloat8_e4m3fn, "x_q and w_q must be e4m3");
  TORCH_CHECK(x_q.dim() == 3 && w_q.dim() == 2 && w_q.size(1) == x_q.size(2), "x_q [B, S, H] and w_q [N, H]");
  TORCH_CHECK(!gated || w_q.size(0) % 2 == 0, "weight.size(0) must be even");
  TORCH_CHECK(scales.is_cuda() && scales.scalar_type() == at::kFloat && scales.numel() == 2 && scales.is_contiguous() &&
                  scales.device() == x_q.device(), "scales must be two float32 on x's device");
  TORCH_CHECK(act_id == 0 || act_id == 1, "act_id must be 0 (SiLU) or 1 (GELU)");
  const auto out_t = out_bf16 ? at::kBFloat16 : at::kHalf;
  const void* bias_p = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->is_contiguous() && bias->numel() == w_q.size(0) && bias->scalar_type() == out_t,
                "bias must be a contiguous CUDA tensor of weight.size(0) elements in the output dtype");
    bias_p = bias->data_ptr();
  }
  c10::cuda::CUDAGuard guard(x_q.device());
  const int64_t n = w_q.size(0), n_out = gated ? n / 2 : n;
  at::Tensor y = at::empty({x_q.size(0), x_q.size(1), n_out}, x_q.options().dtype(out_t));
  check_status(nd_fc1_fwd(ND_E4M3, out_bf16 ? ND_BF16 : ND_F16, static_cast<int>(act_id), gated ? 1 : 0, x_q.data_ptr(),
                          w_q.data_ptr(), bias_p, 1.0f, scales.data_ptr<float>(), y.data_ptr(), x_q.size(0) * x_q.size(1),
                          x_q.size(2), n, nullptr, current_stream(x_q)),
               "fused_fc1_bias_act_forward_fp8");
  return y;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("fused_fc1_bias_act_backward_dw", &fused_fc1_bias_act_backward_dw, "dW [2I, H] = dz^T @ x on the tcgen05 path");
  m.def("fused_fc1_bias_act_backward_dbias", &fused_fc1_bias_act_backward_dbias, "dbias [2I] = sum of dz over the tokens");
  m.def("fused_residual_adaln_forward", &fused_residual_adaln_forward,
        "x + gate * branch and its AdaLN in one pass -> [x_new, y, scale[B,H], mean, invstd]");
  m.def("fused_residual_adarmsnorm_forward", &fused_residual_adarmsnorm_forward,
        "x + gate * branch and its AdaRMSNorm in one pass -> [x_new, y, scale[B,H], inv_rms]");
  m.def("fused_gated_residual_forward", &fused_gated_residual_forward, "y = x + gate[b] * branch");
  m.def("fused_gated_residual_backward", &fused_gated_residual_backward,
        "(dy [+ dres]) -> [dsum, dbranch, dgate[B,H] fp32]");
  m.def("fused_adaln_forward_e4m3", &fused_adaln_forward_e4m3, "AdaLN forward with e4m3 output -> [q, scale, mean, invstd]");
  m.def("fused_adarmsnorm_forward_e4m3", &fused_adarmsnorm_forward_e4m3, "AdaRMSNorm forward with e4m3 output -> [q, scale, inv_rms]");
  m.def("quantize_e4m3", &quantize_e4m3, "per-tensor amax scaling to e4m3 -> [q, scale]");
  m.def("fused_fc1_bias_act_forward_fp8", &fused_fc1_bias_act_forward_fp8, "FC1 + bias + activation on e4m3 operands");
  m.def("fused_adaln_forward", &fused_adaln_forward, "fused AdaLN forward -> [y, scale[B,H], mean, invstd]");
  m.def("fused_adaln_forward_inference", &fused_adaln_forward_inference, "fused AdaLN forward, y only");
  m.def("fused_adaln_backward_dx", &fused_adaln_backward_dx, "fused AdaLN backward dx");
  m.def("fused_adaln_backward_dparam", &fused_adaln_backward_dparam, "fused AdaLN backward -> [dscale, dshift] fp32");
  m.def("fused_adaln_backward", &fused_adaln_backward, "one-pass AdaLN backward -> [dx, dscale, dshift]");
  m.def("fused_qkv_pack_forward", &fused_qkv_pack_forward, "qkv [B,S,3H] -> [q, k, v], each [B,S,heads,head_dim]");
  m.def("fused_qkv_pack_backward", &fused_qkv_pack_backward, "dq, dk, dv [B,S,heads,head_dim] -> dqkv [B,S,3H]");
  m.def("fused_out_residual_forward", &fused_out_residual_forward, "y = x + residual (+ bias)");
  m.def("fused_geglu_forward", &fused_geglu_forward, "fused GeGLU forward (GELU-gated, tanh approx)");
  m.def("fused_geglu_backward", &fused_geglu_backward, "fused GeGLU backward");
  m.def("fused_gate_act_forward", &fused_gate_act_forward, "fused gate-act forward (act_id: 0=SiLU, 1=GELU)");
  m.def("fused_gate_act_backward", &fused_gate_act_backward, "fused gate-act backward (act_id: 0=SiLU, 1=GELU)");
  m.def("fused_gate_act_backward_gate_first", &fused_gate_act_backward_gate_first,
        "gate-act backward for rows [gate | value] (FC1 pre-activation)");
  m.def("fused_adarmsnorm_forward", &fused_adarmsnorm_forward, "fused AdaRMSNorm forward -> [y, scale, inv_rms]");
  m.def("fused_adarmsnorm_forward_inference", &fused_adarmsnorm_forward_inference, "fused AdaRMSNorm forward, y only");
  m.def("fused_adarmsnorm_backward_dx", &fused_adarmsnorm_backward_dx, "fused AdaRMSNorm backward dx");
  m.def("fused_adarmsnorm_backward_dparam", &fused_adarmsnorm_backward_dparam,
        "fused AdaRMSNorm backward -> [dscale, dshift] fp32");
  m.def("fused_adarmsnorm_backward", &fused_adarmsnorm_backward, "one-pass AdaRMSNorm backward -> [dx, dscale, dshift]");
  m.def("fused_fc1_bias_act_forward", &fused_fc1_bias_act_forward,
        "fused FC1 + bias + gated activation; weight/bias rows interleaved (gate0, value0, ...)");
  m.def("fused_fc1_bias_act_forward_stacked", &fused_fc1_bias_act_forward_stacked,
        "fused FC1 + bias + gated activation; weight rows [gate block | value block]");
  m.def("fused_fc1_bias_act_backward_dz", &fused_fc1_bias_act_backward_dz,
        "dz of the gated FC1 with z recomputed inside the kernel");
  m.def("fused_fc1_bias_act_backward_dz_dbias", &fused_fc1_bias_act_backward_dz_dbias,
        "[dz, dbias] of the gated FC1: z recomputed and dz summed over the tokens inside one kernel");
  m.def("fused_fc1_bias_act_backward_dx", &fused_fc1_bias_act_backward_dx, "dx = dz @ weight on the tcgen05 GEMM");
  m.def("fused_fc1_bias_act_forward_plain", &fused_fc1_bias_act_forward_plain,
        "fused FC1 + bias + activation without gating, y = act(x W^T + b)");
}
