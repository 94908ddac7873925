// Test infrastructure, not product code.
//
// Exposes the reference implementation's per-device entry points
// (csrc/cpu/butterfly_cpu.h:6-15 and, when built with -DREF_WITH_CUDA,
// csrc/cuda/butterfly_cuda.h:6-15) under the operator namespace
// `torch_butterfly_ref`, so that the unmodified reference kernels can be loaded
// into the same process as this repository's `torch_butterfly` operators (an
// operator namespace can only be defined once per process).  The reference
// sources themselves are compiled where they lie; nothing of them is copied.
#include <torch/library.h>
#include <torch/extension.h>
#include <tuple>

torch::Tensor butterfly_multiply_fw_cpu(const torch::Tensor twiddle, const torch::Tensor input,
                                        bool increasing_stride, int output_size);
std::tuple<torch::Tensor, torch::Tensor> butterfly_multiply_bw_cpu(const torch::Tensor twiddle,
                                                                   const torch::Tensor input,
                                                                   const torch::Tensor grad,
                                                                   bool increasing_stride);
#ifdef REF_WITH_CUDA
torch::Tensor butterfly_multiply_fw_cuda(const torch::Tensor twiddle, const torch::Tensor input,
                                         bool increasing_stride, int output_size);
std::tuple<torch::Tensor, torch::Tensor> butterfly_multiply_bw_cuda(const torch::Tensor twiddle,
                                                                    const torch::Tensor input,
                                                                    const torch::Tensor grad,
                                                                    bool increasing_stride);
#endif

static torch::Tensor ref_fw(const torch::Tensor& twiddle, const torch::Tensor& input,
                            bool increasing_stride, int64_t output_size) {
#ifdef REF_WITH_CUDA
  if (input.is_cuda()) return butterfly_multiply_fw_cuda(twiddle, input, increasing_stride, (int)output_size);
#endif
  TORCH_CHECK(!input.is_cuda(), "reference library built without its CUDA kernels");
  return butterfly_multiply_fw_cpu(twiddle, input, increasing_stride, (int)output_size);
}

static std::tuple<torch::Tensor, torch::Tensor> ref_bw(const torch::Tensor& twiddle,
                                                       const torch::Tensor& input,
                                                       const torch::Tensor& grad,
                                                       bool increasing_stride) {
#ifdef REF_WITH_CUDA
  if (input.is_cuda()) return butterfly_multiply_bw_cuda(twiddle, input, grad, increasing_stride);
#endif
  TORCH_CHECK(!input.is_cuda(), "reference library built without its CUDA kernels");
  return butterfly_multiply_bw_cpu(twiddle, input, grad, increasing_stride);
}

TORCH_LIBRARY(torch_butterfly_ref, m) {
  m.def("butterfly_multiply_fw(Tensor twiddle, Tensor input, bool increasing_stride, int output_size) -> Tensor", ref_fw);
  m.def("butterfly_multiply_bw(Tensor twiddle, Tensor input, Tensor grad, bool increasing_stride) -> (Tensor, Tensor)", ref_bw);
}
