// Test infrastructure, not product code.
//
// Force-included (`nvcc -include`) ahead of the reference's
// csrc/cuda/butterfly_cuda.cu so that the file compiles UNMODIFIED against
// torch 2.x: its private dispatch macro (butterfly_cuda.cu:9-22) names an ATen
// internal that was removed, `AT_PRIVATE_CASE_TYPE`.  It is supplied here with
// its old meaning.
#pragma once
#include <ATen/Dispatch.h>
#include <c10/core/ScalarType.h>

#ifndef AT_PRIVATE_CASE_TYPE
#define AT_PRIVATE_CASE_TYPE(NAME, enum_type, type, ...) \
  case enum_type: {                                      \
    using scalar_t = type;                               \
    return __VA_ARGS__();                                \
  }
#endif
