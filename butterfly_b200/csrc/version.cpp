// `torch_butterfly::cuda_version`, kept in a library of its own (`_version.so`) because
// the reference package loads `_version` before `_butterfly`
// (torch_butterfly/__init__.py:8-11) and refuses to import when the value disagrees with
// torch.version.cuda (torch_butterfly/__init__.py:13-31).  Replaces csrc/version.cpp:14-23.
// It reports the CUDA runtime that torch itself runs on, not the toolkit this file was
// compiled with, because that is what the check is meant to establish.
#include <ATen/detail/CUDAHooksInterface.h>
#include <torch/library.h>

static int64_t cuda_version() { return at::detail::getCUDAHooks().versionCUDART(); }

TORCH_LIBRARY_FRAGMENT(torch_butterfly, m) { m.def("cuda_version() -> int", cuda_version); }
