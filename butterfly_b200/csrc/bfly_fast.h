// Entry points of the translation units that hold the shape-specialised kernels; called by the
// executor in bfly_kernels.cu.
#pragma once
#include <cuda_runtime.h>

#include <cuda.h>

#include "bfly_bw3.h"
#include "bfly_fw2.h"

namespace bfly {

// Launch the packed-pair forward kernel (after the small kernel that re-orders the twiddles into
// p.packed).  Returns BFLY_OK, a negative status, or kFw2Declined when a tensor cannot be
// described to the TMA unit (the caller then runs the generic kernel).
// `ctas_per_sm`: 1 or 2 (rows per thread up to 14 or 7).  `err`: device address of the flag that a
// kernel whose bounded wait ran out raises.  `launches`: kernels launched.
int fw2_launch(const Fw2Params& p, int ctas_per_sm, int sms, cudaStream_t stream, int* err, int* launches);

// out[b, f] += bias[f], f < len, on a (B, width) matrix with row pitch `pitch` (elements).
int bias_add_launch(float* out, const float* bias, int64_t B, int len, int64_t pitch, int sms, cudaStream_t stream);

// Launch the packed-pair backward phase kernel.  The three descriptors (activation in, gradient
// in, gradient out) describe boxes of kBw3Rows rows of the phase's panel (bfly_tma.h).
int bw3_launch(const Bw3Params& p, const CUtensorMap& mx, const CUtensorMap& mg, const CUtensorMap& mo, cudaStream_t stream,
               int* err);

// Adds to the count that bfly_launch_count reports (kernels launched by the other translation units).
void count_launches(int n);

}  // namespace bfly
