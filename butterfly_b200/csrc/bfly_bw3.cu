// CUDA side of the packed-pair backward phase kernel (bfly_bw3.h).  Its own translation unit of
// libbfly_b200.so.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "bfly_bw3.h"
#include "bfly_fast.h"
#include "bfly_tma.h"

namespace bfly {


// One CTA = 128 threads = one 1024-column panel x one stack x a slice of the rows.  Tile traffic
// goes through the TMA unit (thread 0 issues one bulk tensor load per tile and one bulk tensor
// store per batch; two mbarriers: the gradient tile is needed only after the forward steps).
// Every wait is bounded; a CTA whose wait runs out raises the flag and stops.
__global__ void __launch_bounds__(kBw3Threads, 2)
bfly_bw3_kernel(const __grid_constant__ Bw3Params p, const __grid_constant__ CUtensorMap map_x,
                const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_o, int* __restrict__ err) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const BwParams<float>& q = p.b;
  float* sm = reinterpret_cast<float*>(smem);
  const uint32_t sm0 = tma_smem(smem);
  uint32_t* meta = reinterpret_cast<uint32_t*>(smem + bw3_tile_bytes(p));
  uint32_t* tmem_slot = meta + (size_t)q.nsg * kBw3Threads * 4 + 8;
  const uint32_t bar = tma_smem(tmem_slot + 2), bar_g = bar + 8;
  const int tid = threadIdx.x, warp = tid >> 5;
  if ((sm0 & 1023u) != 0) {  // the hardware swizzle works on address bits
    if (tid == 0) atomicExch(err, 2);
    return;
  }
  int pbase, stack, row_begin, row_end;
  bw_cta_coords(q, blockIdx.x, pbase, stack, row_begin, row_end);

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sm_addr(tmem_slot)), "r"(kBw3TmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    mbar_init(bar, 1);
    mbar_init(bar_g, 1);
    fence_async_smem();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  Acc3Tmem acc;
  acc.taddr = tmem_base + ((uint32_t)(32 * warp) << 16);  // lane = thread index (4 warps x 32 lanes)

  bw3_init(p, acc, meta, stack, pbase, tid);

  const uint32_t tile_bytes = (uint32_t)kBw3TileBytes;
  const uint32_t smX = sm0, smG = sm0 + (uint32_t)q.nsg * tile_bytes;
  const int sx = q.tma_sx ? stack : 0, sg_ = q.tma_sg ? stack : 0, so = q.tma_so ? stack : 0;
  const int pbf = pbase * q.tma_f;
  const int c1 = (pbf & ((1 << q.tma_pbe) - 1)) >> 5, c2 = pbf >> q.tma_pbe;
  auto issue_load_x = [&](int row0) {
    mbar_expect_tx(bar, tile_bytes);
    tma_load_tile(smX, &map_x, bar, c1, c2, sx, row0);
  };
  auto issue_load_g = [&](int row0) {
    mbar_expect_tx(bar_g, tile_bytes);
    tma_load_tile(smG, &map_g, bar_g, c1, c2, sg_, row0);
  };
  uint32_t parity = 0;
  if (tid == 0 && row_begin < row_end) {
    issue_load_x(row_begin);
    issue_load_g(row_begin);
  }
  __syncthreads();  // the unit-position table is complete
  float tr[32], ar[32];  // tensor-memory fetch buffers (operands of the step that comes next, when prefetching)
  if (kBw3Prefetch) bw3_prefetch(p, acc, 0, tr, ar);
  if (kBw3PrefetchTw) acc.ld32(bw3_step_sg(q.nsg, 0) * 64, tr);
  const int nsteps = bw3_num_steps(q.nsg);
  // bias gradient of a fused linear layer: this thread's 8 columns of the panel, summed over the
  // rows of the incoming gradient
  float db[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  bool gave_up = false;  // a bounded wait ran out: stop, and keep the partial sums out of d_twiddle

  for (int row0 = row_begin; row0 < row_end; row0 += kBw3Rows) {
    {
      const bool ok = mbar_wait(bar, parity);
      if (__syncthreads_or(!ok)) {  // uniform decision: give up on this CTA's rows
        if (tid == 0) atomicExch(err, 1);
        gave_up = true;
        break;
      }
    }
    int step = 0;
    for (; step + 1 < q.nsg; ++step) {
      bw3_step(p, acc, meta, step, sm, tid, tr, ar);
      __syncthreads();
    }
    {  // the gradient tile has had the forward steps to arrive
      const bool ok = mbar_wait(bar_g, parity);
      parity ^= 1;
      if (__syncthreads_or(!ok)) {
        if (tid == 0) atomicExch(err, 1);
        gave_up = true;
        break;
      }
    }
    if (q.dbias) {  // column sums of the gradient tile as it arrived (16-byte chunks 2 tid, 2 tid + 1 of every row)
#pragma unroll
      for (int r = 0; r < kBw3Rows; ++r)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int l = 8 * tid + 4 * h;
          const float4 v = *reinterpret_cast<const float4*>(sm + (size_t)(q.nsg * kBw3Rows + r) * 1024 + swz<2>(l));
          db[4 * h + 0] += v.x; db[4 * h + 1] += v.y; db[4 * h + 2] += v.z; db[4 * h + 3] += v.w;
        }
    }
    for (; step < nsteps; ++step) {
      bw3_step(p, acc, meta, step, sm, tid, tr, ar);
      if (step + 1 == nsteps) fence_async_smem();  // the gradient tile is read by the TMA unit next
      __syncthreads();
    }
    if (tid == 0) {
      const bool more = row0 + kBw3Rows < row_end;
      if (more) issue_load_x(row0 + kBw3Rows);  // the snapshot tiles are free already
      if (q.gout_reduce) tma_reduce_add_tile(&map_o, smG, c1, c2, so, row0);
      else tma_store_tile(&map_o, smG, c1, c2, so, row0);
      tma_store_commit();
      if (more) {
        tma_store_wait_read();  // the gradient tile is free again
        issue_load_g(row0 + kBw3Rows);
      }
    }
  }
  if (tid == 0) tma_store_wait_all();
  if (kBw3Prefetch || kBw3PrefetchTw) acc.wait_ld();  // the fetch issued by the last step
  if (!gave_up) bw3_flush(p, acc, stack, pbase, tid);
  if (!gave_up && q.dbias) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int flat = stack * (1 << q.log_n) + q.panel.col(pbase, 8 * tid + e);
      if (flat < q.dbias_len) atomicAdd(q.dbias + flat, db[e]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kBw3TmemCols) : "memory");
  }
}


int bw3_launch(const Bw3Params& p, const CUtensorMap& mx, const CUtensorMap& mg, const CUtensorMap& mo, cudaStream_t stream,
               int* err) {
  static std::mutex mu;
  static bool attr_done[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BFLY_E_NODEVICE;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (!attr_done[dev]) {
      if (cudaFuncSetAttribute(bfly_bw3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 113 * 1024) != cudaSuccess ||
          cudaFuncSetAttribute(bfly_bw3_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared) != cudaSuccess) {
        cudaGetLastError();
        return BFLY_E_CUDA;
      }
      attr_done[dev] = true;
    }
  }
  const size_t smem = bw3_smem_bytes(p) + 32;  // TMEM slot, two mbarriers
  if (smem > 113 * 1024) return BFLY_E_UNSUPPORTED;
  bfly_bw3_kernel<<<bw_num_ctas(p.b), kBw3Threads, smem, stream>>>(p, mx, mg, mo, err);
  return cudaGetLastError() == cudaSuccess ? BFLY_OK : BFLY_E_CUDA;
}

}  // namespace bfly
