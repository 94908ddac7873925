// Tensor-memory-accelerator (TMA) path for tile loads and stores.
//
// A tile row in shared memory is a run of 16-byte chunks whose index bits [0,3) are XORed with
// bits [3,6) (bfly_types.h, swz): in byte addresses, bits [4,7) ^= bits [7,10).  That is the
// 128-byte swizzle mode of the TMA unit, so one cp.async.bulk.tensor instruction issued by one
// thread moves a whole R-row tile between global memory and the swizzled tile: no per-thread
// address arithmetic, no registers, zero fill and clipping at the tensor's edges for free.
//
// A (B, S, cols) float tensor with row stride sB and stack stride sS is described as a rank-5
// tensor of 32-float column blocks (128 bytes, the swizzle span):
//     dim0  32 floats inside a column block
//     dim1  column blocks inside one 2^pbe-column group          (stride 128 bytes)
//     dim2  2^pbe-column groups of a row                          (stride 4 << pbe bytes)
//     dim3  stacks                                                (stride 4 * sS bytes)
//     dim4  rows                                                  (stride 4 * sB bytes)
// and a panel (bfly_types.h, Panel) with segments of 2^lseg columns at stride 2^pb is the box
// (32, 2^(lseg-5), 2^(logC-lseg), 1, R) of it: the box lands in shared memory in the order
// row, segment, column -- the tile layout -- with the swizzle applied by the hardware.
// Complex tensors are described as float tensors of twice the width.
//
// The shared-memory tile must start on a 1024-byte boundary (the swizzle uses address bits).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <mutex>

#include "bfly_types.h"

namespace bfly {

// ---------------------------------------------------------------- host: descriptor construction

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled, looked up through the runtime (the library does not link libcuda).
inline EncodeTiledFn tma_encoder() {
  static std::once_flag once;
  static EncodeTiledFn fn = nullptr;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  });
  return fn;
}

// Geometry shared by all tensors of a launch: panel, rows per tile, floats per element.
// A panel whose first column is pbase (in floats) starts at column block
// (pbase mod 2^pbe) / 32 of group pbase >> pbe (the kernels compute these two coordinates).
struct TmaGeom {
  int lseg, pw, pbe;  // in floats: log2 segment length, log2 segments per panel, log2 group length
  int R;              // rows per box
  bool ok;
};

inline TmaGeom tma_geometry(const Panel& pn, int log_n, int R, int floats_per_elem) {
  const int fl = floats_per_elem == 2 ? 1 : 0;
  TmaGeom g;
  g.lseg = pn.lseg + fl;
  g.pw = pn.logC - pn.lseg;
  g.pbe = (g.pw == 0 ? log_n : pn.pb) + fl;
  g.R = R;
  // segments of at least one column block; box extents of at most 256 per dimension; tile rows
  // of whole 1024-byte swizzle periods (the hardware swizzles on address bits, the tile layout
  // on the position inside the row: they agree when every row starts a new period)
  g.ok = g.lseg >= 5 && g.lseg - 5 <= 8 && g.pw <= 8 && R >= 1 && R <= 256 && g.pbe >= g.lseg &&
         pn.logC + fl >= 8;
  return g;
}

// Describe tensor `ptr` ((B, S, cols) elements of floats_per_elem floats, element strides sB, sS)
// for boxes of geometry g.  Returns false when the tensor cannot be described (alignment, ragged
// width); the caller then uses the per-thread copy routines.
inline bool tma_describe(CUtensorMap* map, const TmaGeom& g, const void* ptr, int64_t sB, int64_t sS, int cols,
                         int B, int S, int floats_per_elem) {
  EncodeTiledFn enc = tma_encoder();
  if (!enc || !g.ok || !ptr || B < 1) return false;
  const int64_t f = floats_per_elem;
  const int64_t colsf = (int64_t)cols * f, sBf = sB * f, sSf = sS * f;
  if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0 || sBf % 4 != 0 || sBf <= 0) return false;
  if (colsf < 32 || colsf % 32 != 0) return false;
  const bool stacks = S > 1 && sSf != 0;
  if (stacks && (sSf % 4 != 0 || sSf < 0)) return false;
  int64_t d1, d2;
  if (colsf >= ((int64_t)1 << g.pbe)) {
    if (colsf % ((int64_t)1 << g.pbe) != 0) return false;
    d1 = ((int64_t)1 << g.pbe) >> 5;
    d2 = colsf >> g.pbe;
  } else {
    if (g.pw != 0) return false;  // a strided panel of a row shorter than one group
    d1 = colsf >> 5;
    d2 = 1;
  }
  const cuuint64_t dims[5] = {32, (cuuint64_t)d1, (cuuint64_t)d2, (cuuint64_t)(stacks ? S : 1), (cuuint64_t)B};
  const cuuint64_t strides[4] = {128, (cuuint64_t)4 << g.pbe, (cuuint64_t)((stacks ? sSf : sBf) * 4),
                                 (cuuint64_t)(sBf * 4)};
  const cuuint32_t box[5] = {32, (cuuint32_t)1 << (g.lseg - 5), (cuuint32_t)1 << g.pw, 1, (cuuint32_t)g.R};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < 4; ++i)
    if (strides[i] % 16 != 0 || strides[i] >= ((cuuint64_t)1 << 40)) return false;
  const CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}

// ---------------------------------------------------------------- device: issue and wait

#if defined(__CUDACC__)

constexpr int kTmaSpinLimit = 1 << 22;  // bounded wait: try_wait itself blocks for a while per call

__device__ __forceinline__ uint32_t tma_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Wait for the phase with the given parity; false if the bound ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < kTmaSpinLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_load_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c1, int c2,
                                              int stack, int row) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(c1), "r"(c2), "r"(stack), "r"(row) : "memory");
}
__device__ __forceinline__ void tma_store_tile(const CUtensorMap* map, uint32_t src, int c1, int c2, int stack,
                                               int row) {
  asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
               ::"l"(map), "r"(src), "r"(0), "r"(c1), "r"(c2), "r"(stack), "r"(row) : "memory");
}
// the same box added (float32) onto what global memory holds
__device__ __forceinline__ void tma_reduce_add_tile(const CUtensorMap* map, uint32_t src, int c1, int c2, int stack,
                                                    int row) {
  asm volatile("cp.reduce.async.bulk.tensor.5d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
               ::"l"(map), "r"(src), "r"(0), "r"(c1), "r"(c2), "r"(stack), "r"(row) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all committed stores have finished READING shared memory (the tile may be overwritten)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all committed stores are complete
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

#endif  // __CUDACC__

}  // namespace bfly
