// Thin torch operator layer over the C ABI in include/bfly.h.
//
// Registers the operators the reference registers in csrc/butterfly.cpp:127-131
// (torch_butterfly::butterfly_multiply_fw / _bw / butterfly_multiply) with the same
// argument meaning and the same argument checks (csrc/butterfly.cpp:34-43, 72-83), plus
// native operators for the base-4 product that the reference only has as PyTorch code
// (torch_butterfly/multiply_base4.py:7-41) and torch_butterfly::cuda_version
// (csrc/version.cpp:14-23).  Everything below this file is plain pointers and sizes.
//
// CUDA tensors only: there is no CPU implementation behind these operators, and they
// raise instead of falling back when handed a CPU tensor.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/script.h>

#include <cstdlib>
#include <tuple>

#include "../../include/bfly.h"

namespace {

using torch::Tensor;

#define BFLY_CHECK_CUDA(x) \
  TORCH_CHECK((x).device().is_cuda(), #x " must be a CUDA tensor: the B200 butterfly library has no CPU path")
#define BFLY_CHECK_SAME_DEVICE(x, y) \
  TORCH_CHECK((x).device() == (y).device(), #x " and " #y " must be on the same device")
#define BFLY_CHECK_DIM(x, d) TORCH_CHECK((x).dim() == (d), #x " must have dimension " #d)

void check_status(int rc, const char* what) {
  TORCH_CHECK(rc == BFLY_OK, what, " failed: ", bfly_strerror(rc), " (status ", rc, ")");
}

int dtype_code(const Tensor& t, const char* what) {
  if (t.scalar_type() == at::kFloat) return BFLY_F32;
  if (t.scalar_type() == at::kComplexFloat) return BFLY_C64;
  TORCH_CHECK(false, what, " not implemented for '", toString(t.scalar_type()), "'");
  return -1;
}

// Borrowed tensors are never mutated; lazily-conjugated or strided views are materialised.
Tensor dense_twiddle(const Tensor& t) { return t.resolve_conj().contiguous(); }
Tensor rows_view(const Tensor& t) {
  Tensor r = t.resolve_conj();
  if (r.size(2) > 1 && r.stride(2) != 1) r = r.contiguous();
  if (r.size(2) <= 1 && r.stride(2) != 1) r = r.contiguous();
  return r;
}

// Shared by the plain operator and the autograd node: with `snapshots` the forward also writes
// the activations the backward starts its phases from (bfly_fw_*_saving).
Tensor fw_impl(const Tensor& twiddle, const Tensor& input, bool increasing_stride,
               c10::optional<int64_t> output_size, Tensor* snapshots) {
  BFLY_CHECK_CUDA(twiddle); BFLY_CHECK_CUDA(input); BFLY_CHECK_SAME_DEVICE(twiddle, input);
  BFLY_CHECK_DIM(twiddle, 6); BFLY_CHECK_DIM(input, 3);
  const int64_t batch = input.size(0), nstacks = input.size(1), input_size = input.size(2);
  const int64_t nblocks = twiddle.size(1), log_n = twiddle.size(2);
  TORCH_CHECK(log_n >= 1 && log_n <= 24, "butterfly_multiply_fw: n must be a power of 2 (2 <= n <= 2^24)");
  const int64_t n = (int64_t)1 << log_n;
  TORCH_CHECK(twiddle.sizes() == torch::IntArrayRef({nstacks, nblocks, log_n, n / 2, 2, 2}),
              "twiddle must have shape (nstacks, nblocks, log_n, n / 2, 2, 2)");
  const int64_t out_size = output_size.has_value() ? output_size.value() : n;
  TORCH_CHECK(out_size <= n, "butterfly_multiply_fw: output_size must be <= n");
  TORCH_CHECK(out_size >= 0, "butterfly_multiply_fw: output_size must be >= 0");
  TORCH_CHECK(twiddle.scalar_type() == input.scalar_type(), "twiddle and input must have the same dtype");
  const int dt = dtype_code(input, "butterfly_multiply_fw_cuda");
  c10::cuda::CUDAGuard guard(input.device());
  const Tensor tw = dense_twiddle(twiddle);
  const Tensor x = rows_view(input);
  Tensor output = torch::empty({batch, nstacks, n}, input.options());
  auto stream = at::cuda::getCurrentCUDAStream();
  int rc;
  if (snapshots) {
    const int64_t ws_bytes = bfly_bw_workspace_bytes(dt, (int)batch, (int)nstacks, (int)log_n, (int)nblocks);
    TORCH_CHECK(ws_bytes >= 0, "butterfly_multiply failed: ", bfly_strerror((int)ws_bytes));
    *snapshots = torch::empty({ws_bytes}, input.options().dtype(at::kByte));
    void* sp = ws_bytes ? snapshots->data_ptr() : nullptr;
    if (dt == BFLY_F32) {
      rc = bfly_fw_f32_saving(tw.data_ptr<float>(), x.data_ptr<float>(), x.stride(0), x.stride(1),
                              output.data_ptr<float>(), (int)batch, (int)nstacks, (int)log_n, (int)nblocks,
                              (int)input_size, (int)out_size, increasing_stride, sp, (size_t)ws_bytes, stream.stream());
    } else {
      rc = bfly_fw_c64_saving(tw.data_ptr(), x.data_ptr(), x.stride(0), x.stride(1), output.data_ptr(), (int)batch,
                              (int)nstacks, (int)log_n, (int)nblocks, (int)input_size, (int)out_size,
                              increasing_stride, sp, (size_t)ws_bytes, stream.stream());
    }
  } else {
    // optional scratch of the forward (room for the re-ordered twiddles of its fastest kernel)
    const int64_t fws = bfly_fw_workspace_bytes(dt, (int)batch, (int)nstacks, (int)log_n, (int)nblocks);
    TORCH_CHECK(fws >= 0, "butterfly_multiply_fw failed: ", bfly_strerror((int)fws));
    Tensor ws;
    if (fws > 0) ws = torch::empty({fws}, input.options().dtype(at::kByte));
    void* wp = fws > 0 ? ws.data_ptr() : nullptr;
    if (dt == BFLY_F32) {
      rc = bfly_fw_f32(tw.data_ptr<float>(), x.data_ptr<float>(), x.stride(0), x.stride(1),
                       output.data_ptr<float>(), (int)batch, (int)nstacks, (int)log_n, (int)nblocks,
                       (int)input_size, (int)out_size, increasing_stride, wp, (size_t)fws, stream.stream());
    } else {
      rc = bfly_fw_c64(tw.data_ptr(), x.data_ptr(), x.stride(0), x.stride(1), output.data_ptr(), (int)batch,
                       (int)nstacks, (int)log_n, (int)nblocks, (int)input_size, (int)out_size,
                       increasing_stride, wp, (size_t)fws, stream.stream());
    }
  }
  check_status(rc, "butterfly_multiply_fw");
  return out_size < n ? output.slice(2, 0, out_size) : output;
}

Tensor butterfly_multiply_fw(const Tensor& twiddle, const Tensor& input, bool increasing_stride,
                             c10::optional<int64_t> output_size) {
  return fw_impl(twiddle, input, increasing_stride, output_size, nullptr);
}

// `snapshots`: what the matching fw_impl call saved (then the backward skips its own forward
// pass over the first phases), or null.
std::tuple<Tensor, Tensor> bw_impl(const Tensor& twiddle, const Tensor& input, const Tensor& grad,
                                   bool increasing_stride, const Tensor* snapshots) {
  BFLY_CHECK_CUDA(twiddle); BFLY_CHECK_CUDA(input); BFLY_CHECK_CUDA(grad);
  BFLY_CHECK_SAME_DEVICE(twiddle, input); BFLY_CHECK_SAME_DEVICE(input, grad);
  BFLY_CHECK_DIM(twiddle, 6); BFLY_CHECK_DIM(input, 3); BFLY_CHECK_DIM(grad, 3);
  const int64_t batch = input.size(0), nstacks = input.size(1), input_size = input.size(2);
  const int64_t nblocks = twiddle.size(1), log_n = twiddle.size(2);
  TORCH_CHECK(log_n >= 1 && log_n <= 24, "butterfly_multiply_bw: n must be a power of 2 (2 <= n <= 2^24)");
  const int64_t n = (int64_t)1 << log_n;
  const int64_t out_size = grad.size(2);
  TORCH_CHECK(twiddle.sizes() == torch::IntArrayRef({nstacks, nblocks, log_n, n / 2, 2, 2}),
              "twiddle must have shape (nstacks, nblocks, log_n, n / 2, 2, 2)");
  TORCH_CHECK(grad.sizes() == torch::IntArrayRef({batch, nstacks, out_size}),
              "grad must have shape (batch_size, nstacks, output_size)");
  TORCH_CHECK(out_size <= n, "butterfly_multiply_bw: output_size must be <= n");
  TORCH_CHECK(twiddle.scalar_type() == input.scalar_type() && grad.scalar_type() == input.scalar_type(),
              "twiddle, input and grad must have the same dtype");
  const int dt = dtype_code(input, "butterfly_multiply_bw_cuda");
  c10::cuda::CUDAGuard guard(input.device());
  const Tensor tw = dense_twiddle(twiddle);
  const Tensor x = rows_view(input);
  const Tensor g = rows_view(grad);
  Tensor d_twiddle = torch::empty_like(tw);
  Tensor d_input = torch::empty({batch, nstacks, std::max(input_size, n)}, input.options());
  const int64_t ws_bytes = bfly_bw_workspace_bytes(dt, (int)batch, (int)nstacks, (int)log_n, (int)nblocks);
  TORCH_CHECK(ws_bytes >= 0, "butterfly_multiply_bw failed: ", bfly_strerror((int)ws_bytes));
  const bool saved = snapshots && snapshots->defined() && snapshots->numel() >= ws_bytes;
  Tensor ws = saved ? *snapshots : torch::empty({ws_bytes}, input.options().dtype(at::kByte));
  auto stream = at::cuda::getCurrentCUDAStream();
  int rc;
  if (saved && dt == BFLY_F32) {
    rc = bfly_bw_f32_saved(tw.data_ptr<float>(), x.data_ptr<float>(), x.stride(0), x.stride(1), g.data_ptr<float>(),
                           g.stride(0), g.stride(1), d_twiddle.data_ptr<float>(), d_input.data_ptr<float>(),
                           (int)batch, (int)nstacks, (int)log_n, (int)nblocks, (int)input_size, (int)out_size,
                           increasing_stride, ws_bytes ? ws.data_ptr() : nullptr, (size_t)ws_bytes, stream.stream());
  } else if (saved) {
    rc = bfly_bw_c64_saved(tw.data_ptr(), x.data_ptr(), x.stride(0), x.stride(1), g.data_ptr(), g.stride(0),
                           g.stride(1), d_twiddle.data_ptr(), d_input.data_ptr(), (int)batch, (int)nstacks,
                           (int)log_n, (int)nblocks, (int)input_size, (int)out_size, increasing_stride,
                           ws_bytes ? ws.data_ptr() : nullptr, (size_t)ws_bytes, stream.stream());
  } else if (dt == BFLY_F32) {
    rc = bfly_bw_f32(tw.data_ptr<float>(), x.data_ptr<float>(), x.stride(0), x.stride(1), g.data_ptr<float>(),
                     g.stride(0), g.stride(1), d_twiddle.data_ptr<float>(), d_input.data_ptr<float>(), (int)batch,
                     (int)nstacks, (int)log_n, (int)nblocks, (int)input_size, (int)out_size, increasing_stride,
                     ws_bytes ? ws.data_ptr() : nullptr, (size_t)ws_bytes, stream.stream());
  } else {
    rc = bfly_bw_c64(tw.data_ptr(), x.data_ptr(), x.stride(0), x.stride(1), g.data_ptr(), g.stride(0), g.stride(1),
                     d_twiddle.data_ptr(), d_input.data_ptr(), (int)batch, (int)nstacks, (int)log_n, (int)nblocks,
                     (int)input_size, (int)out_size, increasing_stride, ws_bytes ? ws.data_ptr() : nullptr,
                     (size_t)ws_bytes, stream.stream());
  }
  check_status(rc, "butterfly_multiply_bw");
  if (input_size < n) d_input = d_input.slice(2, 0, input_size);
  return std::make_tuple(d_twiddle, d_input);
}

std::tuple<Tensor, Tensor> butterfly_multiply_bw(const Tensor& twiddle, const Tensor& input, const Tensor& grad,
                                                 bool increasing_stride) {
  return bw_impl(twiddle, input, grad, increasing_stride, nullptr);
}

// The autograd node may keep the forward's phase-boundary activations for its backward (the
// reference recomputes them, csrc/butterfly.cpp:99-118): that removes one forward-sized pass from
// every training step at the price of holding (phases - 1) activation-sized buffers per call
// between forward and backward.  On by default while those buffers stay under 1 GiB per call;
// the library option "autograd_save" (environment BFLY_AUTOGRAD_SAVE at load time, or
// bfly_set_option) = 0 always recomputes, = 1 always saves.
bool autograd_saves(int64_t snapshot_bytes) {
  int v = -1;
  if (bfly_get_option("autograd_save", &v) == BFLY_OK && v >= 0) return v != 0;
  return snapshot_bytes > 0 && snapshot_bytes <= ((int64_t)1 << 30);
}

using torch::autograd::AutogradContext;
using torch::autograd::variable_list;

// Same contract as the reference's autograd node (csrc/butterfly.cpp:99-118): saves
// {twiddle, input} and the direction flag, returns {d_twiddle, d_input, none, none}.
class ButterflyMultiply : public torch::autograd::Function<ButterflyMultiply> {
 public:
  // `wants_grad`: a gradient can be asked for later.  The caller decides it, because inside
  // apply() gradient mode is always off while parameters still report requires_grad: a forward
  // under torch.no_grad() must not pay for snapshots nobody will read.
  static Tensor forward(AutogradContext* ctx, Tensor twiddle, Tensor input, bool increasing_stride,
                        c10::optional<int64_t> output_size, bool wants_grad) {
    ctx->saved_data["increasing_stride"] = increasing_stride;
    bool save = false;
    if (wants_grad && twiddle.is_cuda() && input.is_cuda() && twiddle.dim() == 6 && input.dim() == 3 &&
        (input.scalar_type() == at::kFloat || input.scalar_type() == at::kComplexFloat)) {
      const int64_t ws = bfly_bw_workspace_bytes(input.scalar_type() == at::kFloat ? BFLY_F32 : BFLY_C64,
                                                 (int)input.size(0), (int)input.size(1), (int)twiddle.size(2),
                                                 (int)twiddle.size(1));
      save = ws > 0 && autograd_saves(ws);
    }
    if (!save) {
      ctx->save_for_backward({twiddle, input});
      return butterfly_multiply_fw(twiddle, input, increasing_stride, output_size);
    }
    Tensor snapshots;
    Tensor out = fw_impl(twiddle, input, increasing_stride, output_size, &snapshots);
    ctx->save_for_backward({twiddle, input, snapshots});
    return out;
  }
  static variable_list backward(AutogradContext* ctx, variable_list grad_output) {
    auto saved = ctx->get_saved_variables();
    auto result = bw_impl(saved[0], saved[1], grad_output[0], ctx->saved_data["increasing_stride"].toBool(),
                          saved.size() > 2 ? &saved[2] : nullptr);
    return {std::get<0>(result), std::get<1>(result), Tensor(), Tensor(), Tensor()};
  }
};

Tensor butterfly_multiply(const Tensor& twiddle, const Tensor& input, bool increasing_stride,
                          c10::optional<int64_t> output_size) {
  const bool wants_grad = at::GradMode::is_enabled() && (twiddle.requires_grad() || input.requires_grad());
  return ButterflyMultiply::apply(twiddle, input, increasing_stride, output_size, wants_grad);
}

// ---------------------------------------------------------------- fused linear layer (float32)

// Butterfly as a linear layer without the PyTorch glue of the reference's module
// (torch_butterfly/butterfly.py:152-169): input (batch, in_size) shared by the stacks, output the
// first out_size columns of the stacks' outputs side by side, bias added in the kernel.
Tensor butterfly_linear_fw(const Tensor& twiddle, const Tensor& input, const c10::optional<Tensor>& bias,
                           bool increasing_stride, int64_t out_size) {
  BFLY_CHECK_CUDA(twiddle); BFLY_CHECK_CUDA(input); BFLY_CHECK_SAME_DEVICE(twiddle, input);
  BFLY_CHECK_DIM(twiddle, 6); BFLY_CHECK_DIM(input, 2);
  TORCH_CHECK(input.scalar_type() == at::kFloat && twiddle.scalar_type() == at::kFloat,
              "butterfly_linear_fw: float32 only");
  const int64_t batch = input.size(0), input_size = input.size(1);
  const int64_t nstacks = twiddle.size(0), nblocks = twiddle.size(1), log_n = twiddle.size(2);
  TORCH_CHECK(log_n >= 1 && log_n <= 24, "butterfly_linear_fw: n must be a power of 2 (2 <= n <= 2^24)");
  const int64_t n = (int64_t)1 << log_n;
  TORCH_CHECK(twiddle.sizes() == torch::IntArrayRef({nstacks, nblocks, log_n, n / 2, 2, 2}),
              "twiddle must have shape (nstacks, nblocks, log_n, n / 2, 2, 2)");
  TORCH_CHECK(out_size >= 0 && out_size <= nstacks * n, "butterfly_linear_fw: out_size must be <= nstacks * n");
  const float* bp = nullptr;
  Tensor b;
  if (bias.has_value() && bias->defined()) {
    BFLY_CHECK_CUDA((*bias)); BFLY_CHECK_SAME_DEVICE((*bias), input);
    TORCH_CHECK(bias->scalar_type() == at::kFloat && bias->dim() == 1 && bias->size(0) >= out_size,
                "bias must be a float32 vector of at least out_size entries");
    b = bias->contiguous();
    bp = b.data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(input.device());
  const Tensor tw = dense_twiddle(twiddle);
  Tensor x = input.stride(1) == 1 || input.size(1) <= 1 ? input : input.contiguous();
  if (x.size(1) <= 1 && x.stride(1) != 1) x = x.contiguous();
  Tensor output = torch::empty({batch, nstacks * n}, input.options());
  const int64_t fws = bfly_fw_workspace_bytes(BFLY_F32, (int)batch, (int)nstacks, (int)log_n, (int)nblocks);
  TORCH_CHECK(fws >= 0, "butterfly_linear_fw failed: ", bfly_strerror((int)fws));
  Tensor ws;
  if (fws > 0) ws = torch::empty({fws}, input.options().dtype(at::kByte));
  auto stream = at::cuda::getCurrentCUDAStream();
  const int rc = bfly_linear_fw_f32(tw.data_ptr<float>(), x.data_ptr<float>(), x.stride(0), output.data_ptr<float>(), bp,
                                    (int)batch, (int)nstacks, (int)log_n, (int)nblocks, (int)input_size, (int)out_size,
                                    increasing_stride, fws > 0 ? ws.data_ptr() : nullptr, (size_t)fws, stream.stream());
  check_status(rc, "butterfly_linear_fw");
  return out_size < nstacks * n ? output.slice(1, 0, out_size) : output;
}

// (d_twiddle, d_input (batch, in_size), d_bias (out_size) or an undefined tensor)
std::tuple<Tensor, Tensor, Tensor> butterfly_linear_bw(const Tensor& twiddle, const Tensor& input, const Tensor& grad,
                                                        bool increasing_stride, bool need_bias) {
  BFLY_CHECK_CUDA(twiddle); BFLY_CHECK_CUDA(input); BFLY_CHECK_CUDA(grad);
  BFLY_CHECK_SAME_DEVICE(twiddle, input); BFLY_CHECK_SAME_DEVICE(input, grad);
  BFLY_CHECK_DIM(twiddle, 6); BFLY_CHECK_DIM(input, 2); BFLY_CHECK_DIM(grad, 2);
  TORCH_CHECK(input.scalar_type() == at::kFloat && twiddle.scalar_type() == at::kFloat && grad.scalar_type() == at::kFloat,
              "butterfly_linear_bw: float32 only");
  const int64_t batch = input.size(0), input_size = input.size(1), out_size = grad.size(1);
  const int64_t nstacks = twiddle.size(0), nblocks = twiddle.size(1), log_n = twiddle.size(2);
  const int64_t n = (int64_t)1 << log_n;
  TORCH_CHECK(grad.size(0) == batch && out_size <= nstacks * n, "grad must have shape (batch_size, out_size <= nstacks * n)");
  c10::cuda::CUDAGuard guard(input.device());
  const Tensor tw = dense_twiddle(twiddle);
  const Tensor x = input.contiguous();
  const Tensor g = grad.contiguous();
  auto stream = at::cuda::getCurrentCUDAStream();
  if (out_size == nstacks * n) {
    const int64_t wsb = bfly_linear_bw_workspace_bytes((int)batch, (int)nstacks, (int)log_n, (int)nblocks);
    if (wsb >= 0) {
      Tensor d_twiddle = torch::empty_like(tw);
      Tensor d_input = torch::empty({batch, input_size}, input.options());
      Tensor d_bias = need_bias ? torch::empty({out_size}, input.options()) : Tensor();
      Tensor ws = torch::empty({std::max<int64_t>(wsb, 16)}, input.options().dtype(at::kByte));
      const int rc = bfly_linear_bw_f32(tw.data_ptr<float>(), x.data_ptr<float>(), x.stride(0), g.data_ptr<float>(), g.stride(0),
                                        d_twiddle.data_ptr<float>(), d_input.data_ptr<float>(), d_input.stride(0),
                                        need_bias ? d_bias.data_ptr<float>() : nullptr, (int)batch, (int)nstacks, (int)log_n,
                                        (int)nblocks, (int)input_size, (int)out_size, increasing_stride, ws.data_ptr(),
                                        (size_t)ws.numel(), stream.stream());
      if (rc == BFLY_OK) return std::make_tuple(d_twiddle, d_input, d_bias);
      if (rc != BFLY_E_UNSUPPORTED) check_status(rc, "butterfly_linear_bw");
    }
  }
  // unfused composition: the operator on the expanded input, then the reductions autograd would run
  Tensor gp = g;
  if (out_size < nstacks * n) gp = torch::constant_pad_nd(g, {0, nstacks * n - out_size});
  auto r = bw_impl(tw, x.unsqueeze(1).expand({batch, nstacks, input_size}), gp.view({batch, nstacks, n}), increasing_stride,
                   nullptr);
  return std::make_tuple(std::get<0>(r), std::get<1>(r).sum(1), need_bias ? g.sum(0) : Tensor());
}

class ButterflyLinear : public torch::autograd::Function<ButterflyLinear> {
 public:
  static Tensor forward(AutogradContext* ctx, Tensor twiddle, Tensor input, c10::optional<Tensor> bias, bool increasing_stride,
                        int64_t out_size) {
    ctx->saved_data["increasing_stride"] = increasing_stride;
    ctx->saved_data["has_bias"] = bias.has_value() && bias->defined();
    ctx->save_for_backward({twiddle, input});
    return butterfly_linear_fw(twiddle, input, bias, increasing_stride, out_size);
  }
  static variable_list backward(AutogradContext* ctx, variable_list grad_output) {
    auto saved = ctx->get_saved_variables();
    auto r = butterfly_linear_bw(saved[0], saved[1], grad_output[0], ctx->saved_data["increasing_stride"].toBool(),
                                 ctx->saved_data["has_bias"].toBool());
    return {std::get<0>(r), std::get<1>(r), std::get<2>(r), Tensor(), Tensor()};
  }
};

Tensor butterfly_linear(const Tensor& twiddle, const Tensor& input, const c10::optional<Tensor>& bias, bool increasing_stride,
                        int64_t out_size) {
  return ButterflyLinear::apply(twiddle, input, bias, increasing_stride, out_size);
}

// ---------------------------------------------------------------- base-4

struct Base4Shape {
  int64_t batch, nstacks, input_size, nblocks, log_n, n;
};

Base4Shape base4_shape(const Tensor& twiddle4, const Tensor& twiddle2, const Tensor& input, const char* what) {
  BFLY_CHECK_CUDA(twiddle4); BFLY_CHECK_CUDA(twiddle2); BFLY_CHECK_CUDA(input);
  BFLY_CHECK_SAME_DEVICE(twiddle4, input); BFLY_CHECK_SAME_DEVICE(twiddle2, input);
  BFLY_CHECK_DIM(twiddle4, 6); BFLY_CHECK_DIM(twiddle2, 6); BFLY_CHECK_DIM(input, 3);
  Base4Shape s;
  s.batch = input.size(0); s.nstacks = input.size(1); s.input_size = input.size(2);
  s.nblocks = twiddle4.size(1);
  s.log_n = twiddle4.size(2) * 2 + twiddle2.size(2);
  TORCH_CHECK(s.log_n >= 1 && s.log_n <= 24 && twiddle2.size(2) <= 1, what, ": n must be a power of 2");
  s.n = (int64_t)1 << s.log_n;
  if (s.log_n / 2 > 0)
    TORCH_CHECK(twiddle4.sizes() == torch::IntArrayRef({s.nstacks, s.nblocks, s.log_n / 2, s.n / 4, 4, 4}),
                "twiddle4 must have shape (nstacks, nblocks, log_n / 2, n / 4, 4, 4)");
  if (s.log_n % 2 == 1)
    TORCH_CHECK(twiddle2.sizes() == torch::IntArrayRef({s.nstacks, s.nblocks, 1, s.n / 2, 2, 2}),
                "twiddle2 must have shape (nstacks, nblocks, 1, n / 2, 2, 2)");
  TORCH_CHECK((input.scalar_type() == at::kFloat || input.scalar_type() == at::kComplexFloat) &&
                  twiddle4.scalar_type() == input.scalar_type() && twiddle2.scalar_type() == input.scalar_type(),
              what, " not implemented for '", toString(input.scalar_type()), "' (float32 and complex64 only, one dtype)");
  return s;
}

Tensor butterfly_multiply_base4_fw(const Tensor& twiddle4, const Tensor& twiddle2, const Tensor& input,
                                   bool increasing_stride, c10::optional<int64_t> output_size) {
  const Base4Shape s = base4_shape(twiddle4, twiddle2, input, "butterfly_multiply_base4_fw");
  const int64_t out_size = output_size.has_value() ? output_size.value() : s.n;
  TORCH_CHECK(out_size <= s.n && out_size >= 0, "butterfly_multiply_base4_fw: output_size must be <= n");
  c10::cuda::CUDAGuard guard(input.device());
  const Tensor t4 = dense_twiddle(twiddle4), t2 = dense_twiddle(twiddle2);
  const Tensor x = rows_view(input);
  Tensor output = torch::empty({s.batch, s.nstacks, s.n}, input.options());
  auto stream = at::cuda::getCurrentCUDAStream();
  int rc;
  if (input.scalar_type() == at::kFloat) {
    rc = bfly4_fw_f32(t4.numel() ? t4.data_ptr<float>() : nullptr, t2.numel() ? t2.data_ptr<float>() : nullptr,
                      x.data_ptr<float>(), x.stride(0), x.stride(1), output.data_ptr<float>(), (int)s.batch,
                      (int)s.nstacks, (int)s.log_n, (int)s.nblocks, (int)s.input_size, (int)out_size,
                      increasing_stride, stream.stream());
  } else {
    rc = bfly4_fw_c64(t4.numel() ? t4.data_ptr() : nullptr, t2.numel() ? t2.data_ptr() : nullptr, x.data_ptr(),
                      x.stride(0), x.stride(1), output.data_ptr(), (int)s.batch, (int)s.nstacks, (int)s.log_n,
                      (int)s.nblocks, (int)s.input_size, (int)out_size, increasing_stride, stream.stream());
  }
  check_status(rc, "butterfly_multiply_base4_fw");
  return out_size < s.n ? output.slice(2, 0, out_size) : output;
}

std::tuple<Tensor, Tensor, Tensor> butterfly_multiply_base4_bw(const Tensor& twiddle4, const Tensor& twiddle2,
                                                               const Tensor& input, const Tensor& grad,
                                                               bool increasing_stride) {
  const Base4Shape s = base4_shape(twiddle4, twiddle2, input, "butterfly_multiply_base4_bw");
  BFLY_CHECK_CUDA(grad); BFLY_CHECK_SAME_DEVICE(input, grad); BFLY_CHECK_DIM(grad, 3);
  const int64_t out_size = grad.size(2);
  TORCH_CHECK(grad.sizes() == torch::IntArrayRef({s.batch, s.nstacks, out_size}) && out_size <= s.n,
              "grad must have shape (batch_size, nstacks, output_size) with output_size <= n");
  TORCH_CHECK(grad.scalar_type() == input.scalar_type(), "grad must have the dtype of input");
  c10::cuda::CUDAGuard guard(input.device());
  const Tensor t4 = dense_twiddle(twiddle4), t2 = dense_twiddle(twiddle2);
  const Tensor x = rows_view(input), g = rows_view(grad);
  Tensor d4 = torch::empty_like(t4), d2 = torch::empty_like(t2);
  Tensor d_input = torch::empty({s.batch, s.nstacks, std::max(s.input_size, s.n)}, input.options());
  const bool real = input.scalar_type() == at::kFloat;
  const int64_t ws_bytes = bfly4_bw_workspace_bytes(real ? BFLY_F32 : BFLY_C64, (int)s.batch, (int)s.nstacks, (int)s.log_n,
                                                    (int)s.nblocks);
  TORCH_CHECK(ws_bytes >= 0, "butterfly_multiply_base4_bw failed: ", bfly_strerror((int)ws_bytes));
  Tensor ws = torch::empty({ws_bytes}, input.options().dtype(at::kByte));
  auto stream = at::cuda::getCurrentCUDAStream();
  int rc;
  if (real) {
    rc = bfly4_bw_f32(t4.numel() ? t4.data_ptr<float>() : nullptr, t2.numel() ? t2.data_ptr<float>() : nullptr,
                      x.data_ptr<float>(), x.stride(0), x.stride(1), g.data_ptr<float>(), g.stride(0), g.stride(1),
                      d4.numel() ? d4.data_ptr<float>() : nullptr, d2.numel() ? d2.data_ptr<float>() : nullptr,
                      d_input.data_ptr<float>(), (int)s.batch, (int)s.nstacks, (int)s.log_n, (int)s.nblocks,
                      (int)s.input_size, (int)out_size, increasing_stride, ws_bytes ? ws.data_ptr() : nullptr,
                      (size_t)ws_bytes, stream.stream());
  } else {
    rc = bfly4_bw_c64(t4.numel() ? t4.data_ptr() : nullptr, t2.numel() ? t2.data_ptr() : nullptr, x.data_ptr(),
                      x.stride(0), x.stride(1), g.data_ptr(), g.stride(0), g.stride(1),
                      d4.numel() ? d4.data_ptr() : nullptr, d2.numel() ? d2.data_ptr() : nullptr, d_input.data_ptr(),
                      (int)s.batch, (int)s.nstacks, (int)s.log_n, (int)s.nblocks, (int)s.input_size, (int)out_size,
                      increasing_stride, ws_bytes ? ws.data_ptr() : nullptr, (size_t)ws_bytes, stream.stream());
  }
  check_status(rc, "butterfly_multiply_base4_bw");
  if (s.input_size < s.n) d_input = d_input.slice(2, 0, s.input_size);
  return std::make_tuple(d4, d2, d_input);
}

class ButterflyMultiplyBase4 : public torch::autograd::Function<ButterflyMultiplyBase4> {
 public:
  static Tensor forward(AutogradContext* ctx, Tensor twiddle4, Tensor twiddle2, Tensor input, bool increasing_stride,
                        c10::optional<int64_t> output_size) {
    ctx->saved_data["increasing_stride"] = increasing_stride;
    ctx->save_for_backward({twiddle4, twiddle2, input});
    return butterfly_multiply_base4_fw(twiddle4, twiddle2, input, increasing_stride, output_size);
  }
  static variable_list backward(AutogradContext* ctx, variable_list grad_output) {
    auto saved = ctx->get_saved_variables();
    auto r = butterfly_multiply_base4_bw(saved[0], saved[1], saved[2], grad_output[0],
                                         ctx->saved_data["increasing_stride"].toBool());
    return {std::get<0>(r), std::get<1>(r), std::get<2>(r), Tensor(), Tensor()};
  }
};

Tensor butterfly_multiply_base4(const Tensor& twiddle4, const Tensor& twiddle2, const Tensor& input,
                                bool increasing_stride, c10::optional<int64_t> output_size) {
  return ButterflyMultiplyBase4::apply(twiddle4, twiddle2, input, increasing_stride, output_size);
}

// ---------------------------------------------------------------- forward with glue operators
//
// One launch for  [Real2Complex] [gather] butterfly [diagonal] [gather] [real part]  -- the modules
// that surround a Butterfly in the reference's exact transforms (torch_butterfly/special.py,
// permutation.py:65-75, complex_utils.py:100-142, diagonal.py:11-38).  Returns None
// when the rows do not fit a tile (the caller then runs the operators one by one).
c10::optional<Tensor> butterfly_multiply_glue_fw(const Tensor& twiddle, const Tensor& input, bool increasing_stride,
                                  const c10::optional<Tensor>& in_perm, const c10::optional<Tensor>& out_diag,
                                  const c10::optional<Tensor>& out_perm, bool out_real) {
  BFLY_CHECK_CUDA(twiddle); BFLY_CHECK_CUDA(input); BFLY_CHECK_SAME_DEVICE(twiddle, input);
  BFLY_CHECK_DIM(twiddle, 6); BFLY_CHECK_DIM(input, 3);
  const int64_t batch = input.size(0), nstacks = input.size(1), input_size = input.size(2);
  const int64_t nblocks = twiddle.size(1), log_n = twiddle.size(2);
  TORCH_CHECK(log_n >= 1 && log_n <= 24, "butterfly_multiply_glue_fw: n must be a power of 2 (2 <= n <= 2^24)");
  const int64_t n = (int64_t)1 << log_n;
  TORCH_CHECK(twiddle.sizes() == torch::IntArrayRef({nstacks, nblocks, log_n, n / 2, 2, 2}),
              "twiddle must have shape (nstacks, nblocks, log_n, n / 2, 2, 2)");
  TORCH_CHECK(input_size <= n, "butterfly_multiply_glue_fw: input_size must be <= n");
  const bool cplx = twiddle.scalar_type() == at::kComplexFloat;
  TORCH_CHECK(cplx || twiddle.scalar_type() == at::kFloat, "butterfly_multiply_glue_fw: float32 or complex64 twiddle expected");
  const bool x_real = cplx && input.scalar_type() == at::kFloat;
  TORCH_CHECK(x_real || input.scalar_type() == twiddle.scalar_type(), "input must have the dtype of twiddle (or float32 for a complex twiddle)");
  TORCH_CHECK(!out_real || cplx, "out_real needs a complex twiddle");
  auto index_vec = [&](const c10::optional<Tensor>& t, const char* name) -> Tensor {
    if (!t.has_value() || !t->defined()) return Tensor();
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->dim() == 1 && t->size(0) == n, name,
                " must be an int32 CUDA vector of n entries");
    return t->contiguous();
  };
  c10::cuda::CUDAGuard guard(input.device());
  const Tensor ip = index_vec(in_perm, "in_perm"), op = index_vec(out_perm, "out_perm");
  Tensor od;
  if (out_diag.has_value() && out_diag->defined()) {
    TORCH_CHECK(out_diag->is_cuda() && out_diag->scalar_type() == twiddle.scalar_type() && out_diag->dim() == 1 &&
                    out_diag->size(0) == n, "out_diag must be a CUDA vector of n entries with the dtype of twiddle");
    od = out_diag->resolve_conj().contiguous();
  }
  TORCH_CHECK(!ip.defined() || input_size == n, "in_perm needs input_size == n");
  const Tensor tw = dense_twiddle(twiddle);
  const Tensor x = rows_view(input);
  Tensor output = torch::empty({batch, nstacks, n}, input.options().dtype(out_real ? at::kFloat : twiddle.scalar_type()));
  auto stream = at::cuda::getCurrentCUDAStream();
  int rc;
  if (cplx) {
    rc = bfly_fw_glue_c64(tw.data_ptr(), x.data_ptr(), x_real, x.stride(0), x.stride(1), output.data_ptr(), out_real,
                          ip.defined() ? ip.data_ptr<int32_t>() : nullptr, od.defined() ? od.data_ptr() : nullptr,
                          op.defined() ? op.data_ptr<int32_t>() : nullptr, (int)batch, (int)nstacks, (int)log_n, (int)nblocks,
                          (int)input_size, (int)n, increasing_stride, stream.stream());
  } else {
    rc = bfly_fw_glue_f32(tw.data_ptr<float>(), x.data_ptr<float>(), x.stride(0), x.stride(1), output.data_ptr<float>(),
                          ip.defined() ? ip.data_ptr<int32_t>() : nullptr, od.defined() ? od.data_ptr<float>() : nullptr,
                          op.defined() ? op.data_ptr<int32_t>() : nullptr, (int)batch, (int)nstacks, (int)log_n, (int)nblocks,
                          (int)input_size, (int)n, increasing_stride, stream.stream());
  }
  if (rc == BFLY_E_UNSUPPORTED) return c10::nullopt;
  check_status(rc, "butterfly_multiply_glue_fw");
  return output;
}

// ---------------------------------------------------------------- unitary twiddle synthesis
//
// (..., 4) float32 angles -> (..., 2, 2) complex64 blocks and back, one kernel each, in place of
// the cos / sin / stack chain of the reference's ButterflyUnitary.forward
// (torch_butterfly/butterfly.py:271-280) and autograd's backward of that chain.
Tensor unitary_twiddle_fw(const Tensor& angles) {
  BFLY_CHECK_CUDA(angles);
  TORCH_CHECK(angles.scalar_type() == at::kFloat && angles.dim() >= 1 && angles.size(-1) == 4,
              "unitary_twiddle: angles must be float32 with last dimension 4 (phi, alpha, psi, chi)");
  c10::cuda::CUDAGuard guard(angles.device());
  const Tensor a = angles.contiguous();
  auto shape = a.sizes().vec();
  shape.back() = 2;
  shape.push_back(2);
  Tensor tw = torch::empty(shape, a.options().dtype(at::kComplexFloat));
  check_status(bfly_unitary_twiddle_fw(a.data_ptr<float>(), tw.data_ptr(), a.numel() / 4, at::cuda::getCurrentCUDAStream().stream()),
               "unitary_twiddle");
  return tw;
}

Tensor unitary_twiddle_bw(const Tensor& angles, const Tensor& grad) {
  BFLY_CHECK_CUDA(angles); BFLY_CHECK_CUDA(grad); BFLY_CHECK_SAME_DEVICE(angles, grad);
  TORCH_CHECK(angles.scalar_type() == at::kFloat && grad.scalar_type() == at::kComplexFloat &&
                  grad.numel() == angles.numel() && angles.dim() >= 1 && angles.size(-1) == 4,
              "unitary_twiddle_bw: angles (..., 4) float32 and grad (..., 2, 2) complex64 expected");
  c10::cuda::CUDAGuard guard(angles.device());
  const Tensor a = angles.contiguous(), g = grad.resolve_conj().contiguous();
  Tensor d = torch::empty_like(a);
  check_status(bfly_unitary_twiddle_bw(a.data_ptr<float>(), g.data_ptr(), d.data_ptr<float>(), a.numel() / 4,
                                       at::cuda::getCurrentCUDAStream().stream()),
               "unitary_twiddle_bw");
  return d;
}

class UnitaryTwiddle : public torch::autograd::Function<UnitaryTwiddle> {
 public:
  static Tensor forward(AutogradContext* ctx, Tensor angles) {
    ctx->save_for_backward({angles});
    return unitary_twiddle_fw(angles);
  }
  static variable_list backward(AutogradContext* ctx, variable_list grad_output) {
    return {unitary_twiddle_bw(ctx->get_saved_variables()[0], grad_output[0])};
  }
};

Tensor unitary_twiddle(const Tensor& angles) { return UnitaryTwiddle::apply(angles); }

// The reference's import-time check (torch_butterfly/__init__.py:13-31) compares this
// with torch.version.cuda, so report the CUDA runtime torch itself runs on.
int64_t cuda_version() { return at::detail::getCUDAHooks().versionCUDART(); }

int64_t launch_count() { return bfly_launch_count(); }

}  // namespace

TORCH_LIBRARY(torch_butterfly, m) {
  m.def("butterfly_multiply_fw(Tensor twiddle, Tensor input, bool increasing_stride, int? output_size=None) -> Tensor",
        butterfly_multiply_fw);
  m.def("butterfly_multiply_bw(Tensor twiddle, Tensor input, Tensor grad, bool increasing_stride) -> (Tensor, Tensor)",
        butterfly_multiply_bw);
  m.def("butterfly_multiply(Tensor twiddle, Tensor input, bool increasing_stride, int? output_size=None) -> Tensor",
        butterfly_multiply);
  m.def("butterfly_linear_fw(Tensor twiddle, Tensor input, Tensor? bias, bool increasing_stride, int out_size) -> Tensor",
        butterfly_linear_fw);
  m.def("butterfly_linear_bw(Tensor twiddle, Tensor input, Tensor grad, bool increasing_stride, bool need_bias) -> (Tensor, Tensor, Tensor)",
        butterfly_linear_bw);
  m.def("butterfly_linear(Tensor twiddle, Tensor input, Tensor? bias, bool increasing_stride, int out_size) -> Tensor",
        butterfly_linear);
  m.def("butterfly_multiply_glue_fw(Tensor twiddle, Tensor input, bool increasing_stride, Tensor? in_perm, Tensor? out_diag, Tensor? out_perm, bool out_real) -> Tensor?",
        butterfly_multiply_glue_fw);
  m.def("unitary_twiddle_fw(Tensor angles) -> Tensor", unitary_twiddle_fw);
  m.def("unitary_twiddle_bw(Tensor angles, Tensor grad) -> Tensor", unitary_twiddle_bw);
  m.def("unitary_twiddle(Tensor angles) -> Tensor", unitary_twiddle);
  m.def("butterfly_multiply_base4_fw(Tensor twiddle4, Tensor twiddle2, Tensor input, bool increasing_stride, int? output_size=None) -> Tensor",
        butterfly_multiply_base4_fw);
  m.def("butterfly_multiply_base4_bw(Tensor twiddle4, Tensor twiddle2, Tensor input, Tensor grad, bool increasing_stride) -> (Tensor, Tensor, Tensor)",
        butterfly_multiply_base4_bw);
  m.def("butterfly_multiply_base4(Tensor twiddle4, Tensor twiddle2, Tensor input, bool increasing_stride, int? output_size=None) -> Tensor",
        butterfly_multiply_base4);
#ifndef BFLY_SEPARATE_VERSION_LIB
  m.def("cuda_version() -> int", cuda_version);
#endif
  m.def("b200_launch_count() -> int", launch_count);
}
