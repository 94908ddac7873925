// CUDA side of the small operators of bfly_glue.h and their C entry points.  Its own translation
// unit of libbfly_b200.so.
#include <cuda_runtime.h>

#include "../../include/bfly.h"
#include "bfly_fast.h"
#include "bfly_glue.h"

namespace bfly {

// One thread per 2x2 block: a 16-byte load of the angles, two 16-byte stores of the entries
// (forward); two 16-byte loads of the gradient, one 16-byte store (backward).  Grid-stride.
__global__ void __launch_bounds__(256) bfly_unitary_fw_kernel(const float4* __restrict__ angles, float4* __restrict__ tw, int64_t nblk) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nblk; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 a4 = angles[i];
    const float a[4] = {a4.x, a4.y, a4.z, a4.w};
    float t[8];
    unitary_block_fw(a, t);
    tw[2 * i] = make_float4(t[0], t[1], t[2], t[3]);
    tw[2 * i + 1] = make_float4(t[4], t[5], t[6], t[7]);
  }
}

__global__ void __launch_bounds__(256) bfly_unitary_bw_kernel(const float4* __restrict__ angles, const float4* __restrict__ g,
                                                                float4* __restrict__ d, int64_t nblk) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nblk; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 a4 = angles[i], g0 = g[2 * i], g1 = g[2 * i + 1];
    const float a[4] = {a4.x, a4.y, a4.z, a4.w};
    const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    float o[4];
    unitary_block_bw(a, gg, o);
    d[i] = make_float4(o[0], o[1], o[2], o[3]);
  }
}

static int glue_grid(int64_t items, int threads) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  const int64_t want = (items + threads - 1) / threads;
  const int64_t cap = (int64_t)sms * 8;
  return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}

}  // namespace bfly

using namespace bfly;

extern "C" {

int bfly_unitary_twiddle_fw(const float* angles, void* twiddle, int64_t nblocks2x2, void* stream) {
  if (nblocks2x2 < 0) return BFLY_E_ARG;
  if (nblocks2x2 == 0) return BFLY_OK;
  if (!angles || !twiddle) return BFLY_E_ARG;
  if (((uintptr_t)angles | (uintptr_t)twiddle) & 15u) return BFLY_E_ALIGN;
  const int grid = glue_grid(nblocks2x2, 256);
  if (grid < 0) return BFLY_E_NODEVICE;
  bfly_unitary_fw_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const float4*)angles, (float4*)twiddle, nblocks2x2);
  if (cudaGetLastError() != cudaSuccess) return BFLY_E_CUDA;
  count_launches(1);
  return BFLY_OK;
}

int bfly_unitary_twiddle_bw(const float* angles, const void* d_twiddle, float* d_angles, int64_t nblocks2x2, void* stream) {
  if (nblocks2x2 < 0) return BFLY_E_ARG;
  if (nblocks2x2 == 0) return BFLY_OK;
  if (!angles || !d_twiddle || !d_angles) return BFLY_E_ARG;
  if (((uintptr_t)angles | (uintptr_t)d_twiddle | (uintptr_t)d_angles) & 15u) return BFLY_E_ALIGN;
  const int grid = glue_grid(nblocks2x2, 256);
  if (grid < 0) return BFLY_E_NODEVICE;
  bfly_unitary_bw_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const float4*)angles, (const float4*)d_twiddle, (float4*)d_angles,
                                                                  nblocks2x2);
  if (cudaGetLastError() != cudaSuccess) return BFLY_E_CUDA;
  count_launches(1);
  return BFLY_OK;
}

}  // extern "C"
