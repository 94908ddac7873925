// CUDA side of the packed-pair forward kernel (bfly_fw2.h): the __global__ kernel, its TMA
// descriptors and its launcher.  Compiled as its own translation unit of libbfly_b200.so.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <mutex>

#include "bfly_fw2.h"
#include "bfly_fast.h"
#include "bfly_tma.h"

namespace bfly {

struct Fw2Maps {
  CUtensorMap in, out, snap[kFw2MaxSnap];
};

// Rank-4 view of a (B, S, cols) float tensor for boxes of one 512-column chunk x rows:
//   dim0 32 floats of a column block, dim1 column blocks of a row, dim2 stacks, dim3 rows.
// The box (32, 16, 1, rows) lands in shared memory as rows of 2 KB with the 128-byte swizzle.
static bool fw2_describe(CUtensorMap* map, const void* ptr, int64_t sB, int64_t sS, int cols, int B, int S, int rows) {
  EncodeTiledFn enc = tma_encoder();
  if (!enc || !ptr || B < 1 || rows < 1 || rows > 256) return false;
  if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0 || sB <= 0 || sB % 4 != 0) return false;
  if (cols < 32 || cols % 32 != 0) return false;
  const bool stacks = S > 1 && sS != 0;
  if (stacks && (sS < 0 || sS % 4 != 0)) return false;
  const cuuint64_t dims[4] = {32, (cuuint64_t)(cols / 32), (cuuint64_t)(stacks ? S : 1), (cuuint64_t)B};
  const cuuint64_t strides[3] = {128, (cuuint64_t)((stacks ? sS : sB) * 4), (cuuint64_t)(sB * 4)};
  const cuuint32_t box[4] = {32, 16, 1, (cuuint32_t)rows};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < 3; ++i)
    if (strides[i] % 16 != 0 || strides[i] >= ((cuuint64_t)1 << 40)) return false;
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same view of the 4096-column panels of wider rows (Fw2Params::view): dim1 runs over the
// panel's 128 column blocks (`blk_stride` floats apart), dim2 over the panels (`panel_stride`).
static bool fw2_describe_view(CUtensorMap* map, const void* ptr, int64_t sB, int64_t blk_stride, int64_t panel_stride,
                              int npanels, int B, int rows) {
  EncodeTiledFn enc = tma_encoder();
  if (!enc || !ptr || B < 1 || rows < 1 || rows > 256) return false;
  if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0 || sB <= 0 || sB % 4 != 0) return false;
  const cuuint64_t dims[4] = {32, 128, (cuuint64_t)npanels, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)(blk_stride * 4), (cuuint64_t)(panel_stride * 4), (cuuint64_t)(sB * 4)};
  const cuuint32_t box[4] = {32, 16, 1, (cuuint32_t)rows};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < 3; ++i)
    if (strides[i] % 16 != 0 || strides[i] >= ((cuuint64_t)1 << 40)) return false;
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

__device__ __forceinline__ void tma_load_box4(uint32_t dst, const CUtensorMap* map, uint32_t bar, int blk, int stack, int row) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(blk), "r"(stack), "r"(row) : "memory");
}
__device__ __forceinline__ void tma_store_box4(const CUtensorMap* map, uint32_t src, int blk, int stack, int row) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(map), "r"(src), "r"(0), "r"(blk), "r"(stack), "r"(row) : "memory");
}

// A warp owns the box (its 512-column chunk) x (its Rw rows) of every tile: it loads the box
// (lane 0 issues the bulk tensor copy, all lanes wait on the warp's mbarrier), runs the groups --
// with a warp barrier between windows inside the chunk and a CTA barrier around the windows
// that reach across chunks -- and stores the box.  Every wait is bounded; a warp whose wait runs
// out raises the CTA's give-up flag, which all warps read after the next CTA barrier.
// THREADS = 512 (CTAS = 1): rows of 8192 columns, sixteen warps with one 512-column chunk each.
template <int CTAS, int THREADS>
__global__ void __launch_bounds__(THREADS, CTAS)
bfly_fw2_kernel(const __grid_constant__ Fw2Params p, const __grid_constant__ Fw2Maps maps, int* __restrict__ err) {
  extern __shared__ __align__(1024) unsigned char smem[];
  float* tile = reinterpret_cast<float*>(smem);
  const uint32_t smem0 = tma_smem(smem);
  const uint32_t tile_bytes = (uint32_t)fw2_tile_bytes(p);
  volatile int* give_up = reinterpret_cast<volatile int*>(smem + tile_bytes + (THREADS / 32) * 8);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if ((smem0 & 1023u) != 0) {  // the hardware swizzle works on address bits
    if (tid == 0) atomicExch(err, 2);
    return;
  }
  const int Rw = p.Rw;
  const int cbits = p.log_n - 9;                 // log2 chunks per row
  const int chunk = warp & ((1 << cbits) - 1);
  const int rg = warp >> cbits;                  // row group of the warp
  const uint32_t box_bytes = (uint32_t)Rw * 2048u;
  const uint32_t mybox = smem0 + (uint32_t)((chunk * p.R + rg * Rw) << 11);
  const uint32_t mybar = smem0 + tile_bytes + (uint32_t)warp * 8u;
  if (lane == 0) {
    mbar_init(mybar, 1);
    fence_async_smem();
  }
  if (tid == 0) *give_up = 0;
  __syncthreads();

  const int64_t ntiles = fw2_num_tiles(p);
  const bool store_chunk = chunk * 512 < p.out_cols;  // chunks right of the output are not written
  auto issue_load = [&](int64_t t) {
    const int stack = (int)(t % p.S);
    const int row0 = (int)(t / p.S) * p.R + rg * Rw;
    mbar_expect_tx(mybar, box_bytes);
    tma_load_box4(mybox, &maps.in, mybar, chunk * 16, p.x_stack ? stack : 0, row0);
  };
  // Bias epilogue: every lane adds bias[stack * n + column] to its 16 columns of each row of the
  // warp's box (16-byte accesses; the swizzle moves whole 16-byte chunks).
  auto add_bias = [&](int stack) {
    const int col0 = chunk * 512 + lane * 16;
    const int flat0 = stack * (1 << p.log_n) + col0;
    float4 b[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int f = flat0 + 4 * k;
      b[k] = make_float4(f + 0 < p.bias_len ? __ldg(p.bias + f + 0) : 0.f, f + 1 < p.bias_len ? __ldg(p.bias + f + 1) : 0.f,
                         f + 2 < p.bias_len ? __ldg(p.bias + f + 2) : 0.f, f + 3 < p.bias_len ? __ldg(p.bias + f + 3) : 0.f);
    }
    for (int i = 0; i < Rw; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float4* q = reinterpret_cast<float4*>(tile + fw2_tile_index(p.R, rg * Rw + i, col0 + 4 * k));
        float4 v = *q;
        v.x += b[k].x; v.y += b[k].y; v.z += b[k].z; v.w += b[k].w;
        *q = v;
      }
    }
  };
  // store the warp's box; `local`: only this warp wrote it since the last CTA barrier
  auto store_box = [&](const CUtensorMap* map, bool local, int stack, int row0, bool wanted, bool with_bias) -> bool {
    fence_async_smem();  // the box is read by the TMA unit next
    if (local) {
      __syncwarp();
    } else {
      __syncthreads();
      if (*give_up) return false;
    }
    if (with_bias) {  // the box is complete and this warp's alone
      add_bias(stack);
      fence_async_smem();
      __syncwarp();
    }
    if (lane == 0 && wanted) {
      tma_store_box4(map, mybox, chunk * 16, (map == &maps.out && !p.out_stack) ? 0 : stack, row0);
      tma_store_commit();
      tma_store_wait_read();  // the box may be overwritten
    }
    __syncwarp();
    return true;
  };
  uint32_t parity = 0;
  if (lane == 0 && blockIdx.x < ntiles) issue_load(blockIdx.x);

  // With one CTA per SM there are registers for two sets of twiddles: the set of the next group
  // (of the next tile, after the last group) is fetched while the current group computes.  TA/TB
  // trade places every group; `flip` says which one is current.
  constexpr bool kPrefetch = (CTAS == 1 && THREADS == 256);
  f2 TA[48], TB[kPrefetch ? 48 : 1];
  bool flip = false;
  if (kPrefetch && blockIdx.x < ntiles) fw2_fetch_tw(p, p.g[0], (int)(blockIdx.x % p.S), tid, TA);

  for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int stack = (int)(t % p.S);
    const int row0 = (int)(t / p.S) * p.R + rg * Rw;
    const bool ok = mbar_wait(mybar, parity);
    parity ^= 1;
    if (!__all_sync(0xffffffffu, ok)) {
      if (lane == 0) {
        *give_up = 1;
        atomicExch(err, 1);
      }
      if (!p.cta_syncs) break;  // no other warp waits for this one
    }
    bool alive = true;
    for (int gi = 0; gi < p.ngroups && alive; ++gi) {
      const Fw2Group& g = p.g[gi];
      if (g.sync == 2) {
        __syncthreads();
        if (*give_up) { alive = false; break; }
      } else if (g.sync == 1) {
        __syncwarp();
      }
      if constexpr (kPrefetch) {
        // what comes next: the following group of this tile, or group 0 of the CTA's next tile
        const bool more = gi + 1 < p.ngroups;
        const int64_t tn = more ? t : t + gridDim.x;
        const Fw2Group& gn = p.g[more ? gi + 1 : 0];
        const int stack_n = (int)(tn % p.S);
        if (!flip) {
          if (tn < ntiles) fw2_fetch_tw(p, gn, stack_n, tid, TB);
          fw2_group_dispatch<true>(p, g, tile, tid, TA);
        } else {
          if (tn < ntiles) fw2_fetch_tw(p, gn, stack_n, tid, TA);
          fw2_group_dispatch<true>(p, g, tile, tid, TB);
        }
        flip = !flip;
      } else {
        fw2_fetch_tw(p, g, stack, tid, TA);
        fw2_group_dispatch<false>(p, g, tile, tid, TA);
      }
      if (g.emit) alive = store_box(&maps.snap[g.emit - 1], g.local != 0, stack, row0, true, false);  // snapshots are full width
    }
    if (!alive) break;
    if (p.has_out) {
      if (!store_box(&maps.out, p.g[p.ngroups - 1].local != 0, stack, row0, store_chunk, p.bias != nullptr)) break;
    } else if (!p.g[p.ngroups - 1].local) {
      __syncthreads();  // other warps still read this box in the last group
      if (*give_up) break;
    }
    if (lane == 0 && t + gridDim.x < ntiles) issue_load(t + gridDim.x);
  }
  if (lane == 0) tma_store_wait_all();
}

// ------------------------------------------------------------------ launcher

// Re-orders the twiddles of the launch into the per-thread order the kernel loads (fw2_pack_entry).
__global__ void __launch_bounds__(256) bfly_fw2_pack_kernel(const __grid_constant__ Fw2Params p) {
  const int64_t n = fw2_pack_entries(p);
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
    float q[4];
    const int U = (1 << p.log_n) / 16;
    const int stack = (int)(e / p.packed_stack);
    const uint32_t r = (uint32_t)(e % p.packed_stack);
    int gi = 0;
    while (gi + 1 < p.ngroups && p.g[gi + 1].pk_off <= r) ++gi;
    const uint32_t w = r - p.g[gi].pk_off;
    fw2_pack_entry(p, p.g[gi], stack, (int)(w % (uint32_t)U), (int)(w / (uint32_t)U) >> 3, (int)(w / (uint32_t)U) & 7, q);
    reinterpret_cast<float4*>(p.packed)[e] = make_float4(q[0], q[1], q[2], q[3]);
  }
}

// out[b, f] += bias[f] for f < len on a (B, width) matrix with row pitch `pitch`: the bias of a
// fused linear layer when the forward ran on a kernel without the bias epilogue.
__global__ void __launch_bounds__(256) bfly_bias_kernel(float* __restrict__ out, const float* __restrict__ bias, int64_t B,
                                                         int len, int64_t pitch) {
  const int64_t total = B * len;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / len;
    const int f = (int)(e - r * len);
    out[r * pitch + f] += __ldg(bias + f);
  }
}
int bias_add_launch(float* out, const float* bias, int64_t B, int len, int64_t pitch, int sms, cudaStream_t stream) {
  if (B <= 0 || len <= 0) return BFLY_OK;
  const int64_t blocks = std::min<int64_t>((B * len + 255) / 256, (int64_t)sms * 8);
  bfly_bias_kernel<<<(int)blocks, 256, 0, stream>>>(out, bias, B, len, pitch);
  return cudaGetLastError() == cudaSuccess ? BFLY_OK : BFLY_E_CUDA;
}

template <int CTAS, int THREADS>
static int fw2_launch_ctas(const Fw2Params& p, const Fw2Maps& maps, int grid, size_t smem, cudaStream_t stream, int* err) {
  static std::mutex mu;
  static bool attr_done[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BFLY_E_NODEVICE;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (!attr_done[dev]) {
      if (cudaFuncSetAttribute(bfly_fw2_kernel<CTAS, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (CTAS == 1 ? 227 : 113) * 1024) != cudaSuccess ||
          cudaFuncSetAttribute(bfly_fw2_kernel<CTAS, THREADS>, cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared) != cudaSuccess) {
        cudaGetLastError();
        return BFLY_E_CUDA;
      }
      attr_done[dev] = true;
    }
  }
  bfly_fw2_kernel<CTAS, THREADS><<<grid, THREADS, smem, stream>>>(p, maps, err);
  return cudaGetLastError() == cudaSuccess ? BFLY_OK : BFLY_E_CUDA;
}

int fw2_launch(const Fw2Params& p_in, int ctas_per_sm, int sms, cudaStream_t stream, int* err, int* launches) {
  Fw2Params p = p_in;
  const int n = 1 << p.log_n;
  Fw2Maps maps;
  std::memset(&maps, 0, sizeof(maps));
  const int xc = std::min(p.x_cols, n);
  if (!p.packed || reinterpret_cast<uintptr_t>(p.packed) % 16 != 0) return kFw2Declined;
  if (p.view) {
    // panels of wider rows: contiguous panels follow each other, strided ones interleave block by block
    const bool contig = p.panel.lseg == p.panel.logC;
    const int64_t blk = contig ? 32 : ((int64_t)1 << p.panel.pb), pan = contig ? n : 32;
    if (!contig && p.panel.lseg != 5) return kFw2Declined;
    if (p.bias) return kFw2Declined;
    if (!fw2_describe_view(&maps.in, p.x, p.x_sB, blk, pan, p.S, p.B, p.Rw)) return kFw2Declined;
    p.x_stack = 1;
    p.has_out = p.out != nullptr;
    p.out_cols = n;
    if (p.has_out && !fw2_describe_view(&maps.out, p.out, p.out_sB, blk, pan, p.S, p.B, p.Rw)) return kFw2Declined;
    p.out_stack = 1;
    for (int i = 0; i < kFw2MaxSnap; ++i)
      if (p.snap[i] && !fw2_describe_view(&maps.snap[i], p.snap[i], p.view_row, blk, pan, p.S, p.B, p.Rw)) return kFw2Declined;
  } else {
  if (!fw2_describe(&maps.in, p.x, p.x_sB, p.x_sS, xc, p.B, p.S, p.Rw)) return kFw2Declined;
  p.x_stack = (p.S > 1 && p.x_sS != 0) ? 1 : 0;
  p.has_out = p.out != nullptr;
  if (p.has_out) {
    if (!fw2_describe(&maps.out, p.out, p.out_sB, p.out_sS, p.out_cols, p.B, p.S, p.Rw)) return kFw2Declined;
    p.out_stack = (p.S > 1 && p.out_sS != 0) ? 1 : 0;
  } else {
    p.out_cols = n;
  }
  for (int i = 0; i < kFw2MaxSnap; ++i)
    if (p.snap[i] && !fw2_describe(&maps.snap[i], p.snap[i], (int64_t)p.S * n, n, n, p.B, p.S, p.Rw)) return kFw2Declined;
  }
  const size_t smem = fw2_smem_bytes(p);
  if (smem > (size_t)(ctas_per_sm == 1 ? 227 : 113) * 1024) return kFw2Declined;
  const int64_t entries = fw2_pack_entries(p);
  bfly_fw2_pack_kernel<<<(int)std::min<int64_t>((entries + 255) / 256, 4 * sms), 256, 0, stream>>>(p);
  if (cudaGetLastError() != cudaSuccess) return BFLY_E_CUDA;
  const int grid = (int)std::min<int64_t>(fw2_num_tiles(p), (int64_t)ctas_per_sm * sms);
  const int rc = fw2_threads(p) == kFw2WideThreads ? fw2_launch_ctas<1, kFw2WideThreads>(p, maps, grid, smem, stream, err)
                 : ctas_per_sm == 1              ? fw2_launch_ctas<1, kFw2Threads>(p, maps, grid, smem, stream, err)
                                                 : fw2_launch_ctas<2, kFw2Threads>(p, maps, grid, smem, stream, err);
  if (rc == BFLY_OK && launches) *launches = 2;
  return rc;
}

}  // namespace bfly
