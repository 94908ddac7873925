// CUDA kernels (sm_100a) and C ABI of the butterfly multiply library.
//
// Two kernel families:
//  * bfly_fw_kernel: a CTA owns R whole batch rows in shared memory and runs every stage of
//    the product on them in one launch.  Stages are grouped into register windows of up to
//    4 bits: a thread pulls the 16 elements of its unit and the group's twiddles into
//    registers, runs the group's stages register-to-register, and writes the elements back
//    in place (one shared-memory round trip per group, twiddles amortised over the R rows).
//  * bfly_bw_kernel: twiddle-stationary backward.  A CTA owns a column panel that is closed
//    under the stages of one phase, keeps the twiddles AND the twiddle-gradient
//    accumulators of those stages in registers for its whole life, and streams batches of
//    rows through shared memory (forward recompute into per-sub-group snapshots, then the
//    reverse sweep).  The accumulators are added to d_twiddle once, at the end.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <tuple>
#include <vector>

#include "../../include/bfly.h"
#include "bfly_core.h"
#include "bfly_bw2.h"
#include "bfly_driver.h"
#include "bfly_fast.h"
#include "bfly_tma.h"

namespace bfly {

constexpr int kThreads = 256;

// KMAX: widest register window compiled in (it sets the register budget: windows of up to 3
// bits fit 128 registers and two CTAs per SM, 4-bit windows need one CTA per SM).
// LOGC: compile-time log2 of the tile width, 0 = read from the parameters.
template <typename T, int KMAX> struct FwOcc {
  static constexpr int kMinBlocks = (sizeof(T) == 4 ? (KMAX <= 3 ? 2 : 1) : (KMAX <= 2 ? 2 : 1));
};

// Set when a bounded wait inside a kernel ran out (the kernel then stops early and its output
// is invalid); read and cleared by bfly_device_error().
__device__ int g_device_error = 0;

// Self-test of the give-up protocol: a wait on an mbarrier whose bytes never arrive (nothing is
// ever copied to it), bounded by `limit` polls; when the bound runs out the warp raises the flag
// exactly as the kernels do and returns.  One warp, no global memory touched but the flag.
__global__ void bfly_wait_selftest_kernel(int limit) {
  __shared__ __align__(8) unsigned long long slot;
  const uint32_t bar = tma_smem(&slot);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    fence_async_smem();
    mbar_expect_tx(bar, 16);  // the arrival is counted, the 16 bytes never come
  }
  __syncwarp();
  bool ok = false;
  for (int i = 0; i < limit && !ok; ++i) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done) : "r"(bar), "r"(0u) : "memory");
    ok = done != 0;
  }
  if (!__all_sync(0xffffffffu, ok) && threadIdx.x == 0) atomicExch(&g_device_error, 1);
}

// Device address of the flag on the current device (looked up once per device).
static int device_error_ptr(int** out) {
  static std::mutex mu;
  static int* cache[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BFLY_E_NODEVICE;
  std::lock_guard<std::mutex> lk(mu);
  if (!cache[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_error) != cudaSuccess || !p) {
      cudaGetLastError();
      return BFLY_E_CUDA;
    }
    cache[dev] = static_cast<int*>(p);
  }
  *out = cache[dev];
  return BFLY_OK;
}

// TMA descriptors of a forward launch (bfly_tma.h): input, output, snapshots.
struct FwMaps {
  CUtensorMap in, out, snap[8];
};

// Tile traffic goes through the TMA unit when every tensor of the launch can be described to
// it (p.tma): thread 0 issues one bulk tensor load per tile and one bulk tensor store per
// output, everybody waits on an mbarrier.  Otherwise every thread copies 16-byte chunks.
// GLUE: the instance also runs the glue operators of FwParams::glue (a separate instance, so that
// the plain product keeps its register budget).
template <typename T, int KMAX, int LOGC, int ROWS, bool TMA, bool GLUE>
__global__ void __launch_bounds__(kThreads, (FwOcc<T, KMAX>::kMinBlocks))
bfly_fw_kernel(const __grid_constant__ FwParams<T> p, const __grid_constant__ FwMaps maps) {
  extern __shared__ __align__(16) unsigned char smem_dyn[];
  // the swizzle of the TMA unit works on address bits: the tile starts on a 1024-byte boundary
  unsigned char* smem_raw = smem_dyn + ((1024u - (tma_smem(smem_dyn) & 1023u)) & 1023u);
  T* sm = reinterpret_cast<T*>(smem_raw);
  uint16_t* tab = reinterpret_cast<uint16_t*>(smem_raw + fw_tile_bytes(p));
  const uint32_t bar = tma_smem(smem_raw + fw_smem_bytes(p, kThreads));  // tile and table sizes are multiples of 16
  const int tid = threadIdx.x;
  const int64_t ntiles = fw_num_tiles(p);
  const int64_t n = (int64_t)1 << p.log_n;
  fw_build_table<T>(p, tab, tid, kThreads);  // read only by the thread that wrote it
  if constexpr (TMA) {
    if (tid == 0) {
      mbar_init(bar, 1);
      fence_async_smem();
    }
    __syncthreads();
  }
  const uint32_t tile_bytes = (uint32_t)fw_tile_bytes(p);
  auto coords = [&](int64_t tile, int& row0, int& stack, int& c1, int& c2) {
    int pbase;
    fw_tile_coords(p, tile, row0, stack, pbase);
    const int pbf = pbase * p.tma_f;
    c1 = (pbf & ((1 << p.tma_pbe) - 1)) >> 5;
    c2 = pbf >> p.tma_pbe;
  };
  auto issue_load = [&](int64_t tile) {
    int row0, stack, c1, c2;
    coords(tile, row0, stack, c1, c2);
    mbar_expect_tx(bar, tile_bytes);
    tma_load_tile(tma_smem(sm), &maps.in, bar, c1, c2, p.tma_sx ? stack : 0, row0);
  };
  // gather (and scale) inside every row of the tile, staged through registers; rows are independent,
  // so one barrier between a row's reads and its writes is enough
  auto permute_rows = [&](const int32_t* perm, const T* diag) {
    uint32_t plan[kGlueSlots];
    T v[kGlueSlots];
    const int cnt = tile_permute_plan<T>(p.panel.logC, perm, p.glue.colbit, tid, kThreads, plan);
    for (int r = 0; r < p.R; ++r) {
      tile_permute_read<T>(sm, r, p.panel.logC, diag, plan, cnt, v);
      __syncthreads();
      tile_permute_write<T>(sm, r, p.panel.logC, plan, cnt, v);
    }
    __syncthreads();
  };
  uint32_t parity = 0;
  if (TMA && tid == 0 && blockIdx.x < ntiles) issue_load(blockIdx.x);

  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    int row0, stack, pbase;
    fw_tile_coords(p, tile, row0, stack, pbase);
    if constexpr (TMA) {
      const bool ok = mbar_wait(bar, parity);
      parity ^= 1;
      if (__syncthreads_or(!ok)) {  // uniform decision: give up on this CTA's tiles
        if (tid == 0) atomicExch(&g_device_error, 1);
        break;
      }
    } else {
      if (GLUE && p.glue.x_real) tile_load_real(p.glue.x_real, p.x_sB, p.x_sS, p.x_cols, p.B, stack, row0, p.R, p.panel.logC, sm, tid, kThreads);
      else tile_load_auto<T>(p.x, p.x_sB, p.x_sS, p.x_cols, p.B, stack, row0, p.R, p.panel, pbase, p.vec_in != 0, sm, tid, kThreads);
      tile_load_wait();
      __syncthreads();
    }
    if constexpr (GLUE) {
      if (p.glue.any_in()) permute_rows(p.glue.in_perm, nullptr);
    }
    for (int g = 0; g < p.ngroups; ++g) {
      fw_group_dispatch<T, KMAX, LOGC, ROWS>(p, g, sm, tab, p.R, stack, pbase, tid, kThreads);
      const bool last = (g + 1 == p.ngroups);
      const int emit = p.g[g].emit;
      if (TMA && (emit || (last && p.out))) fence_async_smem();  // the tile is read by the TMA unit next
      __syncthreads();
      if (emit) {
        if constexpr (TMA) {
          if (tid == 0) {
            int r0_, st_, c1, c2;
            coords(tile, r0_, st_, c1, c2);
            tma_store_tile(&maps.snap[emit - 1], tma_smem(sm), c1, c2, stack, row0);
            tma_store_commit();
            if (!last) tma_store_wait_read();  // the next group rewrites the tile
          }
          if (!last) __syncthreads();
        } else {
          tile_store_auto<T>(p.snap[emit - 1], (int64_t)p.S * n, n, (int)n, p.B, stack, row0, p.R, p.panel, pbase, true, sm, tid, kThreads);
          __syncthreads();
        }
      }
    }
    if constexpr (GLUE) {
      if (p.glue.any_out()) {  // the diagonal and the gather of the result, on the finished tile
        if (p.glue.out_perm) {
          permute_rows(p.glue.out_perm, p.glue.out_diag);
        } else {
          tile_scale_rows<T>(sm, p.R, p.panel.logC, p.glue.out_diag, tid, kThreads);
          __syncthreads();
        }
        if constexpr (TMA) {
          fence_async_smem();  // the tile is read by the TMA unit next
          __syncthreads();
        }
      }
    }
    if constexpr (TMA) {
      if (tid == 0) {
        if (p.out) {
          int r0_, st_, c1, c2;
          coords(tile, r0_, st_, c1, c2);
          tma_store_tile(&maps.out, tma_smem(sm), c1, c2, p.tma_so ? stack : 0, row0);
          tma_store_commit();
        }
        if (tile + gridDim.x < ntiles) {
          tma_store_wait_read();  // the tile is free again
          issue_load(tile + gridDim.x);
        }
      }
    } else if (GLUE && p.glue.out_real) {
      tile_store_real(p.glue.out_real, p.out_sB, p.out_sS, p.out_cols, p.B, stack, row0, p.R, p.panel.logC, sm, tid, kThreads);
      __syncthreads();
    } else if (p.out) {
      tile_store_auto<T>(p.out, p.out_sB, p.out_sS, p.out_cols, p.B, stack, row0, p.R, p.panel, pbase, p.vec_out != 0, sm, tid, kThreads);
      __syncthreads();
    }
  }
  if (TMA && tid == 0) tma_store_wait_all();
}

// LOGC / RB: compile-time panel width (log2) and rows per batch, 0 = read from the parameters.
// Phases of at most three sub-groups keep little enough state for two CTAs per SM.
template <typename T, int KW, int NSG> struct BwOcc {
  static constexpr int kMinBlocks = (sizeof(T) == 4 && KW == 2 && NSG <= 3) ? 2 : 1;
};

// Tile traffic goes through the TMA unit when the three tensors can be described to it (p.tma),
// as in the second-generation kernel below; otherwise every thread copies 16-byte chunks.
template <typename T, int KW, int NSG, int LOGC, int RB>
__global__ void __launch_bounds__(kThreads, (BwOcc<T, KW, NSG>::kMinBlocks))
bfly_bw_kernel(const __grid_constant__ BwParams<T> p, const __grid_constant__ CUtensorMap map_x,
               const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_o) {
  extern __shared__ __align__(16) unsigned char smem_dyn[];
  unsigned char* smem_raw = smem_dyn + ((1024u - (tma_smem(smem_dyn) & 1023u)) & 1023u);
  T* smX = reinterpret_cast<T*>(smem_raw);
  const int C = 1 << p.panel.logC;
  T* smG = smX + (size_t)p.nsg * p.Rb * C;
  const uint32_t bar = tma_smem(smG + (size_t)p.Rb * C), bar_g = bar + 8;  // after the tiles (16-byte multiples)
  const int tid = threadIdx.x;
  int pbase, stack, row_begin, row_end;
  bw_cta_coords(p, blockIdx.x, pbase, stack, row_begin, row_end);
  if (p.tma) {
    if (tid == 0) {
      mbar_init(bar, 1);
      mbar_init(bar_g, 1);
      fence_async_smem();
    }
    __syncthreads();
  }
  BwState<T, KW, NSG> st;
  bw_load_state<T, KW, NSG>(p, st, stack, pbase, tid, kThreads);
  const uint32_t tile_bytes = (uint32_t)((size_t)p.Rb * C * sizeof(T));
  const int pbf = pbase * p.tma_f;
  const int c1 = (pbf & ((1 << p.tma_pbe) - 1)) >> 5, c2 = pbf >> p.tma_pbe;
  auto issue_load_x = [&](int row0) {
    mbar_expect_tx(bar, tile_bytes);
    tma_load_tile(tma_smem(smX), &map_x, bar, c1, c2, p.tma_sx ? stack : 0, row0);
  };
  auto issue_load_g = [&](int row0) {
    mbar_expect_tx(bar_g, tile_bytes);
    tma_load_tile(tma_smem(smG), &map_g, bar_g, c1, c2, p.tma_sg ? stack : 0, row0);
  };
  uint32_t parity = 0;
  bool gave_up = false;  // a bounded wait ran out: the partial sums stay out of d_twiddle
  if (p.tma && tid == 0 && row_begin < row_end) {
    issue_load_x(row_begin);
    issue_load_g(row_begin);
  }
  for (int row0 = row_begin; row0 < row_end; row0 += p.Rb) {
    const int R = p.Rb;
    if (p.tma) {
      const bool ok = mbar_wait(bar, parity) && mbar_wait(bar_g, parity);
      parity ^= 1;
      if (__syncthreads_or(!ok)) {  // uniform decision: give up on this CTA's rows
        if (tid == 0) atomicExch(&g_device_error, 1);
        gave_up = true;
        break;
      }
    } else {
      tile_load_auto<T>(p.xin, p.xin_sB, p.xin_sS, p.xin_cols, row_end, stack, row0, R, p.panel, pbase, p.vec_x != 0, smX, tid, kThreads);
      tile_load_auto<T>(p.gin, p.gin_sB, p.gin_sS, p.gin_cols, row_end, stack, row0, R, p.panel, pbase, p.vec_g != 0, smG, tid, kThreads);
      tile_load_wait();
      __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < NSG - 1; ++j) {
      if (j + 1 < p.nsg) {
        bw_sg_step<T, KW, NSG, LOGC, RB, true>(p, st, j, stack, smX, smG, R, tid, kThreads);
        __syncthreads();
      }
    }
#pragma unroll
    for (int j = NSG - 1; j >= 0; --j) {
      if (j < p.nsg) {
        bw_sg_step<T, KW, NSG, LOGC, RB, false>(p, st, j, stack, smX, smG, R, tid, kThreads);
        if (p.tma && j == 0) fence_async_smem();  // the gradient tile is read by the TMA unit next
        __syncthreads();
      }
    }
    if (p.tma) {
      if (tid == 0) {
        const bool more = row0 + p.Rb < row_end;
        if (more) issue_load_x(row0 + p.Rb);  // the snapshot tiles are free already
        tma_store_tile(&map_o, tma_smem(smG), c1, c2, p.tma_so ? stack : 0, row0);
        tma_store_commit();
        if (more) {
          tma_store_wait_read();  // the gradient tile is free again
          issue_load_g(row0 + p.Rb);
        }
      }
    } else {
      tile_store_auto<T>(p.gout, p.gout_sB, p.gout_sS, p.gout_cols, row_end, stack, row0, R, p.panel, pbase, p.vec_o != 0, smG, tid, kThreads);
      __syncthreads();
    }
  }
  if (p.tma && tid == 0) tma_store_wait_all();
  if (!gave_up) bw_flush_state<T, KW, NSG>(p, st, stack, pbase, tid, kThreads);
}

// Second-generation backward phase (bfly_bw2.h): accumulators in tensor memory, four-row
// batches, two CTAs per SM.  Each CTA allocates 256 TMEM columns (two CTAs fill the SM's 512):
// a thread owns the lane (32 * (warp % 4) + lane-in-warp) and, within it, the 128-column range
// picked by warp / 4: 64 columns of accumulators and 64 of twiddles (4 sub-groups x 16).
constexpr int kBw2TmemCols = 256;

// Tile traffic goes through the TMA unit when the three tensors can be described to it
// (p.tma; bfly_tma.h): thread 0 issues one bulk tensor load per tile and one bulk tensor store
// per batch, everybody waits on an mbarrier.  Otherwise every thread copies 16-byte chunks.
template <typename T, int KW, int LOGC>
__global__ void __launch_bounds__(kThreads, 2)
bfly_bw2_kernel(const __grid_constant__ BwParams<T> p, const __grid_constant__ CUtensorMap map_x,
                const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_o) {
  extern __shared__ __align__(16) unsigned char smem_dyn[];
  // the swizzle of the TMA unit works on address bits: tiles start on a 1024-byte boundary
  unsigned char* smem_raw = smem_dyn + ((1024u - (tma_smem(smem_dyn) & 1023u)) & 1023u);
  T* smX = reinterpret_cast<T*>(smem_raw);
  const int C = 1 << p.panel.logC;
  T* smG = smX + (size_t)p.nsg * kBw2Rows * C;
  uint32_t* meta = reinterpret_cast<uint32_t*>(smem_raw + bw2_tile_bytes(p));
  uint32_t* tmem_slot = meta + (size_t)p.nsg * kBw2Meta * kThreads;
  // two mbarriers (8-byte aligned: the tables before them are multiples of 16 bytes): one for the
  // activation tile, one for the gradient tile, which is needed only after the forward steps
  const uint32_t bar = tma_smem(tmem_slot + 2), bar_g = bar + 8;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  int pbase, stack, row_begin, row_end;
  bw_cta_coords(p, blockIdx.x, pbase, stack, row_begin, row_end);

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sm_addr(tmem_slot)), "r"(kBw2TmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (p.tma && tid == 0) {
    mbar_init(bar, 1);
    mbar_init(bar_g, 1);
    fence_async_smem();
  }
  bw2_build_meta<T, KW>(p, meta, pbase, tid, kThreads);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  AccStore<T, KW> accs;
  accs.taddr = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)((warp >> 2) * 128);

  bw2_init<T, KW>(p, accs, meta, stack, tid, kThreads);

  const uint32_t tile_bytes = (uint32_t)(kBw2Rows * C * sizeof(T));
  const int sx = p.tma_sx ? stack : 0, sg_ = p.tma_sg ? stack : 0, so = p.tma_so ? stack : 0;
  // the panel's first column block in the rank-5 view of a row (bfly_tma.h)
  const int pbf = pbase * p.tma_f;
  const int c1 = (pbf & ((1 << p.tma_pbe) - 1)) >> 5, c2 = pbf >> p.tma_pbe;
  auto issue_load_x = [&](int row0) {
    mbar_expect_tx(bar, tile_bytes);
    tma_load_tile(tma_smem(smX), &map_x, bar, c1, c2, sx, row0);
  };
  auto issue_load_g = [&](int row0) {
    mbar_expect_tx(bar_g, tile_bytes);
    tma_load_tile(tma_smem(smG), &map_g, bar_g, c1, c2, sg_, row0);
  };
  uint32_t parity = 0;
  bool gave_up = false;  // a bounded wait ran out: the partial sums stay out of d_twiddle
  if (p.tma && tid == 0 && row_begin < row_end) {
    issue_load_x(row_begin);
    issue_load_g(row_begin);
  }

  for (int row0 = row_begin; row0 < row_end; row0 += kBw2Rows) {
    if (p.tma) {
      const bool ok = mbar_wait(bar, parity);
      parity ^= 1;
      if (__syncthreads_or(!ok)) {  // uniform decision: give up on this CTA's rows
        if (tid == 0) atomicExch(&g_device_error, 1);
        gave_up = true;
        break;
      }
    } else {
      tile_load_auto<T>(p.xin, p.xin_sB, p.xin_sS, p.xin_cols, row_end, stack, row0, kBw2Rows, p.panel, pbase, p.vec_x != 0, smX, tid, kThreads);
      tile_load_auto<T>(p.gin, p.gin_sB, p.gin_sS, p.gin_cols, row_end, stack, row0, kBw2Rows, p.panel, pbase, p.vec_g != 0, smG, tid, kThreads);
      tile_load_wait();
      __syncthreads();
    }
    for (int j = 0; j + 1 < p.nsg; ++j) {
      bw2_fw_step<T, KW, LOGC>(p, accs, meta, j, smX, smG, tid, kThreads);
      __syncthreads();
    }
    if (p.tma) {  // the gradient tile has had the forward steps to arrive
      const bool ok = mbar_wait(bar_g, parity ^ 1);
      if (__syncthreads_or(!ok)) {
        if (tid == 0) atomicExch(&g_device_error, 1);
        gave_up = true;
        break;
      }
    }
    for (int j = p.nsg - 1; j >= 0; --j) {
      bw2_bw_step<T, KW, LOGC>(p, accs, meta, j, smX, smG, tid, kThreads);
      if (p.tma && j == 0) fence_async_smem();  // the gradient tile is read by the TMA unit next
      __syncthreads();
    }
    if (p.tma) {
      if (tid == 0) {
        const bool more = row0 + kBw2Rows < row_end;
        if (more) issue_load_x(row0 + kBw2Rows);  // the snapshot tiles are free already
        tma_store_tile(&map_o, tma_smem(smG), c1, c2, so, row0);
        tma_store_commit();
        if (more) {
          tma_store_wait_read();  // the gradient tile is free again
          issue_load_g(row0 + kBw2Rows);
        }
      }
    } else {
      tile_store_auto<T>(p.gout, p.gout_sB, p.gout_sS, p.gout_cols, row_end, stack, row0, kBw2Rows, p.panel, pbase, p.vec_o != 0, smG, tid, kThreads);
      __syncthreads();
    }
  }
  if (p.tma && tid == 0) tma_store_wait_all();
  if (!gave_up) bw2_flush<T, KW>(p, accs, meta, stack, tid, kThreads);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kBw2TmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ launch side

static std::atomic<int64_t> g_launches{0};
void count_launches(int n) { g_launches.fetch_add(n); }

// Optional per-launch timing (bfly_profile_*): while enabled, every kernel launch is
// bracketed by a pair of CUDA events on the launching stream.
enum KernelId : int { kKernFw = 0, kKernBw = 1, kKernFw2 = 2, kKernBw2 = 3, kKernBw3 = 4, kNumKernelIds = 5 };
struct ProfileRec { int id; cudaEvent_t a, b; };
static std::mutex g_prof_mu;
static bool g_prof_on = false;
static std::vector<ProfileRec> g_prof;

struct ProfileScope {
  cudaStream_t stream;
  bool on = false;
  ProfileRec rec{};
  ProfileScope(int id, cudaStream_t s) : stream(s) {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    if (!g_prof_on) return;
    if (cudaEventCreate(&rec.a) != cudaSuccess) return;
    if (cudaEventCreate(&rec.b) != cudaSuccess) { cudaEventDestroy(rec.a); return; }
    rec.id = id;
    on = true;
    cudaEventRecord(rec.a, stream);
  }
  ~ProfileScope() {
    if (!on) return;
    cudaEventRecord(rec.b, stream);
    std::lock_guard<std::mutex> lk(g_prof_mu);
    g_prof.push_back(rec);
  }
};

struct DeviceInfo {
  int sms = 0;
  bool ok = false;
};

static int device_info(DeviceInfo& out) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BFLY_E_NODEVICE;
  std::lock_guard<std::mutex> lk(mu);
  if (!cache[dev].ok) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      return BFLY_E_NODEVICE;
    cache[dev].sms = sms;
    cache[dev].ok = true;
  }
  out = cache[dev];
  return BFLY_OK;
}

// Function attributes of a kernel instance are set once per (instance, device), and again only
// when a launch needs more dynamic shared memory than any before it: the launch path only looks
// the pair up.
template <typename K>
static int set_smem(K kernel, size_t bytes) {
  struct Entry { const void* fn; int dev; size_t bytes; };
  static std::mutex mu;
  static std::vector<Entry> done;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return BFLY_E_NODEVICE;
  const void* fn = reinterpret_cast<const void*>(kernel);
  std::lock_guard<std::mutex> lk(mu);
  Entry* e = nullptr;
  for (auto& k : done)
    if (k.fn == fn && k.dev == dev) e = &k;
  if (e && e->bytes >= bytes) return BFLY_OK;
  if (bytes > 48 * 1024) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) {
      cudaGetLastError();
      return BFLY_E_CUDA;
    }
  }
  if (!e) {
    // ask for the largest shared-memory carve-out so that two CTAs of up to 113 KB share an SM
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess) {
      cudaGetLastError();
      return BFLY_E_CUDA;
    }
    done.push_back(Entry{fn, dev, bytes});
  } else {
    e->bytes = bytes;
  }
  return BFLY_OK;
}

struct CudaExec {
  cudaStream_t stream;
  DeviceInfo dev;
  int num_sms() const { return dev.sms; }
  int threads() const { return kThreads; }
  static bool use_tma() { return options().tma != 0; }
  bool has_bw2(size_t /*elem_size*/, int kw) const { return options().bw_v2 != 0 && kw == 2; }

  template <typename T, int KW, int LOGC> int launch_bw2(const BwParams<T>& p_in) {
    BwParams<T> p = p_in;
    const size_t smem = bw2_smem_bytes(p, kThreads) + 32 + 1024;  // TMEM slot, two mbarriers, alignment slack
    int rc = set_smem(bfly_bw2_kernel<T, KW, LOGC>, smem);
    if (rc) return rc;
    // describe the three tensors to the TMA unit when they qualify; else per-thread copies
    CUtensorMap mx, mg, mo;
    describe_bw(p, kBw2Rows, mx, mg, mo);
    {
      ProfileScope prof(kKernBw2, stream);
      bfly_bw2_kernel<T, KW, LOGC><<<bw_num_ctas(p), kThreads, smem, stream>>>(p, mx, mg, mo);
    }
    g_launches.fetch_add(1);
    return cudaGetLastError() == cudaSuccess ? BFLY_OK : BFLY_E_CUDA;
  }

  template <typename T, int KMAX, int LOGC, int ROWS> int launch_fw(const FwParams<T>& p_in) {
    FwParams<T> p = p_in;
    const size_t smem = fw_smem_bytes(p, kThreads) + 16 + 1024;  // mbarrier, alignment slack
    // the TMA variant exists for the instances with a compile-time tile shape (the generic
    // instances have no registers to spare for it)
    constexpr bool kTmaInstance = LOGC > 0;
    const bool glue = p.glue.in_perm || p.glue.out_perm || p.glue.out_diag || p.glue.x_real || p.glue.out_real;
    int rc = glue ? set_smem(bfly_fw_kernel<T, KMAX, LOGC, ROWS, false, true>, smem)
                  : set_smem(bfly_fw_kernel<T, KMAX, LOGC, ROWS, false, false>, smem);
    if constexpr (kTmaInstance) {
      if (rc == BFLY_OK)
        rc = glue ? set_smem(bfly_fw_kernel<T, KMAX, LOGC, ROWS, true, true>, smem)
                  : set_smem(bfly_fw_kernel<T, KMAX, LOGC, ROWS, true, false>, smem);
    }
    if (rc) return rc;
    const int64_t ntiles = fw_num_tiles(p);
    const int grid = (int)std::min<int64_t>(ntiles, (int64_t)dev.sms * FwOcc<T, KMAX>::kMinBlocks);
    // describe the tensors to the TMA unit when all of them qualify; else per-thread copies
    FwMaps maps;
    std::memset(&maps, 0, sizeof(maps));
    constexpr int F = (int)(sizeof(T) / 4);
    const int64_t n = (int64_t)1 << p.log_n;
    const TmaGeom geo = tma_geometry(p.panel, p.log_n, p.R, F);
    bool tma = kTmaInstance && use_tma() && geo.ok && !p.glue.x_real && !p.glue.out_real && p.vec_in && (!p.out || p.vec_out) &&
               tma_describe(&maps.in, geo, p.x, p.x_sB, p.x_sS, p.x_cols, p.B, p.S, F) &&
               (!p.out || tma_describe(&maps.out, geo, p.out, p.out_sB, p.out_sS, p.out_cols, p.B, p.S, F));
    for (int i = 0; tma && i < 8; ++i)
      if (p.snap[i]) tma = tma_describe(&maps.snap[i], geo, p.snap[i], (int64_t)p.S * n, n, (int)n, p.B, p.S, F);
    p.tma = tma ? 1 : 0;
    p.tma_sx = (p.S > 1 && p.x_sS != 0); p.tma_so = (p.S > 1 && p.out_sS != 0);
    p.tma_pbe = geo.pbe; p.tma_f = F;
    {
      ProfileScope prof(kKernFw, stream);
      bool launched = false;
      if constexpr (kTmaInstance) {
        if (tma) {
          if (glue) bfly_fw_kernel<T, KMAX, LOGC, ROWS, true, true><<<grid, kThreads, smem, stream>>>(p, maps);
          else bfly_fw_kernel<T, KMAX, LOGC, ROWS, true, false><<<grid, kThreads, smem, stream>>>(p, maps);
          launched = true;
        }
      }
      if (!launched) {
        if (glue) bfly_fw_kernel<T, KMAX, LOGC, ROWS, false, true><<<grid, kThreads, smem, stream>>>(p, maps);
        else bfly_fw_kernel<T, KMAX, LOGC, ROWS, false, false><<<grid, kThreads, smem, stream>>>(p, maps);
      }
    }
    g_launches.fetch_add(1);
    return cudaGetLastError() == cudaSuccess ? BFLY_OK : BFLY_E_CUDA;
  }
  // Instances with the tile shape fixed at compile time exist for the shapes the row planner
  // picks for n = 4096 and n = 1024 float rows and n = 2048 complex rows at two CTAs per SM;
  // everything else runs the generic instance.
  template <typename T, int KMAX> int launch_fw_shape(const FwParams<T>& p) {
    if constexpr (sizeof(T) == 4 && KMAX == KernelCfg<T>::kFwKmaxTwoCtas) {
      if (p.panel.logC == 12 && p.R == 6) return launch_fw<T, KMAX, 12, 6>(p);
      if (p.panel.logC == 10 && p.R == 16) return launch_fw<T, KMAX, 10, 16>(p);
    }
    if constexpr (sizeof(T) == 8 && KMAX == KernelCfg<T>::kFwKmaxTwoCtas) {
      if (p.panel.logC == 11 && p.R == 6) return launch_fw<T, KMAX, 11, 6>(p);  // 2048 complex columns
    }
    return launch_fw<T, KMAX, 0, 0>(p);
  }
  int run_fw2(const Fw2Params& p, int ctas_per_sm) {
    int* err = nullptr;
    int rc = device_error_ptr(&err);
    if (rc) return rc;
    int launches = 0;
    {
      ProfileScope prof(kKernFw2, stream);
      rc = fw2_launch(p, ctas_per_sm, dev.sms, stream, err, &launches);
    }
    if (rc == BFLY_OK) g_launches.fetch_add(launches);
    return rc;
  }
  bool can_run_bw3(const Bw3Params& p_in) {
    Bw3Params p = p_in;
    CUtensorMap mx, mg, mo;
    describe_bw(p.b, kBw3Rows, mx, mg, mo);
    return p.b.tma != 0;
  }
  int run_bw3(const Bw3Params& p_in) {
    Bw3Params p = p_in;
    CUtensorMap mx, mg, mo;
    describe_bw(p.b, kBw3Rows, mx, mg, mo);
    if (!p.b.tma) return kFw2Declined;
    int* err = nullptr;
    int rc = device_error_ptr(&err);
    if (rc) return rc;
    {
      ProfileScope prof(kKernBw3, stream);
      rc = bw3_launch(p, mx, mg, mo, stream, err);
    }
    if (rc == BFLY_OK) g_launches.fetch_add(1);
    return rc;
  }
  template <typename T> int run_fw(const FwParams<T>& p) {
    int kmax = 1;
    for (int g = 0; g < p.ngroups; ++g) kmax = std::max<int>(kmax, p.g[g].K);
    if (kmax <= KernelCfg<T>::kFwKmaxTwoCtas) return launch_fw_shape<T, KernelCfg<T>::kFwKmaxTwoCtas>(p);
    return launch_fw_shape<T, KernelCfg<T>::kFwKmaxOneCta>(p);
  }

  // Describe the three tensors of a backward phase to the TMA unit; p.tma says whether all qualify.
  template <typename T> void describe_bw(BwParams<T>& p, int rows, CUtensorMap& mx, CUtensorMap& mg, CUtensorMap& mo) {
    std::memset(&mx, 0, sizeof(mx)); std::memset(&mg, 0, sizeof(mg)); std::memset(&mo, 0, sizeof(mo));
    constexpr int F = (int)(sizeof(T) / 4);
    const TmaGeom geo = tma_geometry(p.panel, p.log_n, rows, F);
    p.tma = 0;
    if (use_tma() && geo.ok && p.vec_x && p.vec_g && p.vec_o && p.B >= rows &&
        tma_describe(&mx, geo, p.xin, p.xin_sB, p.xin_sS, p.xin_cols, p.B, p.S, F) &&
        tma_describe(&mg, geo, p.gin, p.gin_sB, p.gin_sS, p.gin_cols, p.B, p.S, F) &&
        tma_describe(&mo, geo, p.gout, p.gout_sB, p.gout_sS, p.gout_cols, p.B, p.S, F)) {
      p.tma = 1;
      p.tma_sx = (p.S > 1 && p.xin_sS != 0); p.tma_sg = (p.S > 1 && p.gin_sS != 0); p.tma_so = (p.S > 1 && p.gout_sS != 0);
      p.tma_pbe = geo.pbe; p.tma_f = F;
    }
  }

  template <typename T, int KW, int NSG, int LOGC, int RB> int launch_bw(const BwParams<T>& p_in) {
    BwParams<T> p = p_in;
    const size_t smem = ((size_t)(p.nsg + 1) * p.Rb * sizeof(T) << p.panel.logC) + 16 + 1024;  // two mbarriers, alignment slack
    int rc = set_smem(bfly_bw_kernel<T, KW, NSG, LOGC, RB>, smem);
    if (rc) return rc;
    CUtensorMap mx, mg, mo;
    describe_bw(p, p.Rb, mx, mg, mo);
    {
      ProfileScope prof(kKernBw, stream);
      bfly_bw_kernel<T, KW, NSG, LOGC, RB><<<bw_num_ctas(p), kThreads, smem, stream>>>(p, mx, mg, mo);
    }
    g_launches.fetch_add(1);
    return cudaGetLastError() == cudaSuccess ? BFLY_OK : BFLY_E_CUDA;
  }
  // Instances with the panel shape fixed at compile time cover full 1024-column float panels
  // (512-column complex panels) with the batch heights the planner picks; the rest is generic.
  int run_bw(const BwParams<float>& p, int KW) {
    if (p.v2 && KW == 2) return p.panel.logC == 10 ? launch_bw2<float, 2, 10>(p) : launch_bw2<float, 2, 0>(p);
    if (KW == 2) {
      if (p.panel.logC == 10) {
        if (p.nsg >= 4 && p.Rb == 8) return launch_bw<float, 2, 5, 10, 8>(p);
        if (p.nsg == 3 && p.Rb == 12) return launch_bw<float, 2, 3, 10, 12>(p);
        if (p.nsg <= 3 && p.Rb == 4) return launch_bw<float, 2, 3, 10, 4>(p);
        if (p.nsg <= 2 && p.Rb == 16) return launch_bw<float, 2, 3, 10, 16>(p);
      }
      return p.nsg <= 3 ? launch_bw<float, 2, 3, 0, 0>(p) : launch_bw<float, 2, 5, 0, 0>(p);
    }
    return launch_bw<float, 1, 10, 0, 0>(p);
  }
  int run_bw(const BwParams<cf>& p, int KW) {
    if (p.v2 && KW == 2 && p.nsg <= 2) return p.panel.logC == 10 ? launch_bw2<cf, 2, 10>(p) : launch_bw2<cf, 2, 0>(p);
    if (KW == 2) return p.nsg <= 2 ? launch_bw<cf, 2, 2, 0, 0>(p) : BFLY_E_UNSUPPORTED;  // radix-4 factors, narrow panels
    if (KW != 1) return BFLY_E_UNSUPPORTED;
    if (p.panel.logC == 9) {
      if (p.nsg >= 9 && p.Rb == 4) return launch_bw<cf, 1, 10, 9, 4>(p);
      if (p.nsg <= 2 && p.Rb == 16) return launch_bw<cf, 1, 5, 9, 16>(p);
    }
    return p.nsg <= 5 ? launch_bw<cf, 1, 5, 0, 0>(p) : launch_bw<cf, 1, 10, 0, 0>(p);
  }
  int add_bias(float* out, const float* bias, int64_t B, int len, int64_t pitch) {
    const int rc = bias_add_launch(out, bias, B, len, pitch, dev.sms, stream);
    if (rc == BFLY_OK) g_launches.fetch_add(1);
    return rc;
  }
  int zero(void* ptr, size_t bytes) {
    if (bytes == 0) return BFLY_OK;
    return cudaMemsetAsync(ptr, 0, bytes, stream) == cudaSuccess ? BFLY_OK : BFLY_E_CUDA;
  }
  int zero2d(void* ptr, size_t pitch, size_t width, size_t rows) {
    if (width == 0 || rows == 0) return BFLY_OK;
    return cudaMemset2DAsync(ptr, pitch, 0, width, rows, stream) == cudaSuccess ? BFLY_OK : BFLY_E_CUDA;
  }
};

static int make_exec(void* stream, CudaExec& ex) {
  ex.stream = static_cast<cudaStream_t>(stream);
  return device_info(ex.dev);
}

template <typename T>
static int fw_entry(bool base4, const void* tw2, const void* tw4, const void* x, int64_t x_sB, int64_t x_sS,
                    void* out, int B, int S, int log_n, int nblocks, int in_size, int out_size, int inc,
                    void* stream, void* ws = nullptr, size_t ws_bytes = 0) {
  CudaExec ex;
  int rc = make_exec(stream, ex);
  if (rc) return rc;
  Problem q{B, S, log_n, nblocks, in_size, out_size, inc != 0, base4};
  return drive_fw<T>(ex, q, static_cast<const T*>(tw2), static_cast<const T*>(tw4), static_cast<const T*>(x),
                     x_sB, x_sS, static_cast<T*>(out), ws, ws_bytes);
}

template <typename T>
static int fw_glue_entry(const void* tw, const void* x, int x_is_real, int64_t x_sB, int64_t x_sS, void* out, int out_is_real,
                         const int32_t* in_perm, const void* out_diag, const int32_t* out_perm, int B, int S, int log_n,
                         int nblocks, int in_size, int out_size, int inc, void* stream) {
  CudaExec ex;
  int rc = make_exec(stream, ex);
  if (rc) return rc;
  Problem q{B, S, log_n, nblocks, in_size, out_size, inc != 0, false};
  FwGlue<T> glue{};
  glue.in_perm = in_perm;
  glue.out_perm = out_perm;
  glue.out_diag = static_cast<const T*>(out_diag);
  if (x_is_real) glue.x_real = static_cast<const float*>(x);
  if (out_is_real) glue.out_real = static_cast<float*>(out);
  if (((uintptr_t)in_perm | (uintptr_t)out_perm) & 3u) return BFLY_E_ALIGN;
  return drive_fw_glue<T>(ex, q, static_cast<const T*>(tw), x_is_real ? nullptr : static_cast<const T*>(x), x_sB, x_sS,
                          out_is_real ? nullptr : static_cast<T*>(out), glue);
}

template <typename T>
static int fw_saving_entry(const void* tw2, const void* x, int64_t x_sB, int64_t x_sS, void* out, int B, int S,
                           int log_n, int nblocks, int in_size, int out_size, int inc, void* ws, size_t ws_bytes,
                           void* stream) {
  CudaExec ex;
  int rc = make_exec(stream, ex);
  if (rc) return rc;
  Problem q{B, S, log_n, nblocks, in_size, out_size, inc != 0, false};
  return drive_fw_saving<T>(ex, q, static_cast<const T*>(tw2), static_cast<const T*>(nullptr),
                            static_cast<const T*>(x), x_sB, x_sS, static_cast<T*>(out), ws, ws_bytes);
}

template <typename T>
static int bw_entry(bool base4, const void* tw2, const void* tw4, const void* x, int64_t x_sB, int64_t x_sS,
                    const void* grad, int64_t g_sB, int64_t g_sS, void* d2, void* d4, void* dx, int B, int S,
                    int log_n, int nblocks, int in_size, int out_size, int inc, void* ws, size_t ws_bytes,
                    void* stream, bool snapshots_ready = false) {
  CudaExec ex;
  int rc = make_exec(stream, ex);
  if (rc) return rc;
  Problem q{B, S, log_n, nblocks, in_size, out_size, inc != 0, base4};
  return drive_bw<T>(ex, q, static_cast<const T*>(tw2), static_cast<const T*>(tw4), static_cast<const T*>(x),
                     x_sB, x_sS, static_cast<const T*>(grad), g_sB, g_sS, static_cast<T*>(d2),
                     static_cast<T*>(d4), static_cast<T*>(dx), ws, ws_bytes, snapshots_ready);
}

template <typename T>
static int64_t ws_for(const Problem& q0) {
  // the phase plan depends on the direction of the first block: report the larger need
  int64_t best = 0;
  for (int inc = 0; inc < 2; ++inc) {
    Problem q = q0;
    q.inc = inc != 0;
    BwLayout<T> lay;
    const int rc = plan_bw<T>(q, lay);
    if (rc) return rc;
    best = std::max<int64_t>(best, (int64_t)lay.ws_bytes);
  }
  return best;
}

static int64_t ws_entry(bool base4, int dtype, int B, int S, int log_n, int nblocks) {
  Problem q{B, S, log_n, nblocks, 1, 1, true, base4};
  int rc = check_problem(q);
  if (rc) return rc;
  if (dtype == BFLY_F32) return ws_for<float>(q);
  if (dtype == BFLY_C64) return ws_for<cf>(q);
  return BFLY_E_UNSUPPORTED;
}

// ------------------------------------------------------------------ no-allocation backward
//
// Scratch for bfly_bw_f32_noalloc: part of the library image, resident on every GPU that
// loads it.  In host code the name below is only a handle; the address the kernels need is
// looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[BFLY_NOALLOC_SCRATCH_BYTES];

static int noalloc_scratch_ptr(void** out) {
  static std::mutex mu;
  static void* cache[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return BFLY_E_NODEVICE;
  std::lock_guard<std::mutex> lk(mu);
  if (!cache[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) {
      cudaGetLastError();
      return BFLY_E_CUDA;
    }
    cache[dev] = p;
  }
  *out = cache[dev];
  return BFLY_OK;
}

}  // namespace bfly

using namespace bfly;

extern "C" {

const char* bfly_strerror(int status) {
  switch (status) {
    case BFLY_OK: return "success";
    case BFLY_E_ARG: return "invalid argument (sizes inconsistent or null pointer)";
    case BFLY_E_UNSUPPORTED: return "shape not supported by the B200 butterfly kernels";
    case BFLY_E_ALIGN: return "twiddle pointer must be 16-byte aligned";
    case BFLY_E_WORKSPACE: return "workspace missing, misaligned or too small";
    case BFLY_E_CUDA: return "CUDA runtime call or kernel launch failed";
    case BFLY_E_NODEVICE: return "no usable CUDA device";
    case BFLY_E_TOOLARGE: return "problem needs more scratch than the built-in buffer of the no-allocation entry point holds";
    default: return "unknown status";
  }
}

int bfly_version(void) { return 200; }
int bfly_set_option(const char* name, int value) { return set_option(name, value); }
int bfly_get_option(const char* name, int* value) { return get_option(name, value); }
int bfly_cuda_version(void) { return CUDA_VERSION; }
int64_t bfly_launch_count(void) { return g_launches.load(); }

int bfly_selftest_bounded_wait(int polls, void* stream) {
  if (polls < 1 || polls > (1 << 20)) return BFLY_E_ARG;
  bfly::bfly_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(polls);
  if (cudaGetLastError() != cudaSuccess) return BFLY_E_CUDA;
  g_launches.fetch_add(1);
  return BFLY_OK;
}

int bfly_device_error_async(int* host_flag, void* stream) {
  if (!host_flag) return BFLY_E_ARG;
  return cudaMemcpyFromSymbolAsync(host_flag, bfly::g_device_error, sizeof(int), 0, cudaMemcpyDeviceToHost,
                                   (cudaStream_t)stream) == cudaSuccess ? BFLY_OK : BFLY_E_CUDA;
}

int bfly_device_error(void) {
  int flag = 0;
  const int zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return BFLY_E_CUDA;
  if (cudaMemcpyFromSymbol(&flag, bfly::g_device_error, sizeof(int)) != cudaSuccess) return BFLY_E_CUDA;
  if (flag && cudaMemcpyToSymbol(bfly::g_device_error, &zero, sizeof(int)) != cudaSuccess) return BFLY_E_CUDA;
  return flag > 0 ? flag : (flag != 0);
}

void bfly_profile_enable(int on) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  g_prof_on = on != 0;
}

int bfly_profile_collect(int64_t* launches, double* total_ms, int n_ids) {
  std::vector<ProfileRec> recs;
  {
    std::lock_guard<std::mutex> lk(g_prof_mu);
    recs.swap(g_prof);
  }
  for (int i = 0; i < n_ids; ++i) { launches[i] = 0; total_ms[i] = 0.0; }
  int rc = BFLY_OK;
  for (auto& r : recs) {
    float ms = 0.f;
    if (cudaEventSynchronize(r.b) != cudaSuccess || cudaEventElapsedTime(&ms, r.a, r.b) != cudaSuccess) {
      rc = BFLY_E_CUDA;
    } else if (r.id >= 0 && r.id < n_ids) {
      launches[r.id] += 1;
      total_ms[r.id] += ms;
    }
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
  }
  return rc;
}

int64_t bfly_fw_workspace_bytes(int dtype, int batch, int nstacks, int log_n, int nblocks) {
  Problem q{batch, nstacks, log_n, nblocks, 1, 1, true, false};
  const int rc = check_problem(q);
  if (rc) return rc;
  if (dtype == BFLY_F32) return (int64_t)fw_workspace_bytes<float>(q);
  if (dtype == BFLY_C64) return (int64_t)fw_workspace_bytes<cf>(q);
  return BFLY_E_UNSUPPORTED;
}
int bfly_fw_glue_f32(const float* twiddle, const float* x, int64_t x_sB, int64_t x_sS, float* out, const int32_t* in_perm,
                     const float* out_diag, const int32_t* out_perm, int batch, int nstacks, int log_n, int nblocks,
                     int input_size, int output_size, int increasing_stride, void* stream) {
  return fw_glue_entry<float>(twiddle, x, 0, x_sB, x_sS, out, 0, in_perm, out_diag, out_perm, batch, nstacks, log_n, nblocks,
                              input_size, output_size, increasing_stride, stream);
}
int bfly_fw_glue_c64(const void* twiddle, const void* x, int x_is_real, int64_t x_sB, int64_t x_sS, void* out, int out_is_real,
                     const int32_t* in_perm, const void* out_diag, const int32_t* out_perm, int batch, int nstacks, int log_n,
                     int nblocks, int input_size, int output_size, int increasing_stride, void* stream) {
  return fw_glue_entry<cf>(twiddle, x, x_is_real, x_sB, x_sS, out, out_is_real, in_perm, out_diag, out_perm, batch, nstacks,
                           log_n, nblocks, input_size, output_size, increasing_stride, stream);
}
int bfly_fw_f32(const float* twiddle, const float* x, int64_t x_sB, int64_t x_sS, float* out, int batch,
                int nstacks, int log_n, int nblocks, int input_size, int output_size, int increasing_stride,
                void* workspace, size_t workspace_bytes, void* stream) {
  return fw_entry<float>(false, twiddle, nullptr, x, x_sB, x_sS, out, batch, nstacks, log_n, nblocks,
                         input_size, output_size, increasing_stride, stream, workspace, workspace_bytes);
}
int bfly_fw_c64(const void* twiddle, const void* x, int64_t x_sB, int64_t x_sS, void* out, int batch,
                int nstacks, int log_n, int nblocks, int input_size, int output_size, int increasing_stride,
                void* workspace, size_t workspace_bytes, void* stream) {
  return fw_entry<cf>(false, twiddle, nullptr, x, x_sB, x_sS, out, batch, nstacks, log_n, nblocks, input_size,
                      output_size, increasing_stride, stream, workspace, workspace_bytes);
}
int64_t bfly_bw_workspace_bytes(int dtype, int batch, int nstacks, int log_n, int nblocks) {
  return ws_entry(false, dtype, batch, nstacks, log_n, nblocks);
}
int bfly_bw_f32(const float* twiddle, const float* x, int64_t x_sB, int64_t x_sS, const float* grad,
                int64_t g_sB, int64_t g_sS, float* d_twiddle, float* d_x, int batch, int nstacks, int log_n,
                int nblocks, int input_size, int output_size, int increasing_stride, void* workspace,
                size_t workspace_bytes, void* stream) {
  return bw_entry<float>(false, twiddle, nullptr, x, x_sB, x_sS, grad, g_sB, g_sS, d_twiddle, nullptr, d_x,
                         batch, nstacks, log_n, nblocks, input_size, output_size, increasing_stride, workspace,
                         workspace_bytes, stream);
}
int bfly_bw_c64(const void* twiddle, const void* x, int64_t x_sB, int64_t x_sS, const void* grad, int64_t g_sB,
                int64_t g_sS, void* d_twiddle, void* d_x, int batch, int nstacks, int log_n, int nblocks,
                int input_size, int output_size, int increasing_stride, void* workspace, size_t workspace_bytes,
                void* stream) {
  return bw_entry<cf>(false, twiddle, nullptr, x, x_sB, x_sS, grad, g_sB, g_sS, d_twiddle, nullptr, d_x, batch,
                      nstacks, log_n, nblocks, input_size, output_size, increasing_stride, workspace,
                      workspace_bytes, stream);
}
int bfly_linear_fw_f32(const float* twiddle, const float* x, int64_t x_sB, float* out, const float* bias, int batch,
                       int nstacks, int log_n, int nblocks, int input_size, int output_size, int increasing_stride,
                       void* workspace, size_t workspace_bytes, void* stream) {
  CudaExec ex;
  int rc = make_exec(stream, ex);
  if (rc) return rc;
  Problem q{batch, nstacks, log_n, nblocks, input_size, 1 << log_n, increasing_stride != 0, false};
  return drive_linear_fw(ex, q, twiddle, x, x_sB, out, bias, output_size, workspace, workspace_bytes);
}
int64_t bfly_linear_bw_workspace_bytes(int batch, int nstacks, int log_n, int nblocks) {
  Problem q{batch, nstacks, log_n, nblocks, 1, 1, true, false};
  int rc = check_problem(q);
  if (rc) return rc;
  int64_t best = 0;
  for (int inc = 0; inc < 2; ++inc) {
    q.inc = inc != 0;
    LinearBwLayout L;
    rc = plan_linear_bw(q, L);
    if (rc) return rc;
    best = std::max<int64_t>(best, (int64_t)L.ws_bytes);
  }
  return best;
}
int bfly_linear_bw_f32(const float* twiddle, const float* x, int64_t x_sB, const float* grad, int64_t g_sB, float* d_twiddle,
                       float* d_input, int64_t d_input_sB, float* d_bias, int batch, int nstacks, int log_n, int nblocks,
                       int input_size, int output_size, int increasing_stride, void* workspace, size_t workspace_bytes,
                       void* stream) {
  CudaExec ex;
  int rc = make_exec(stream, ex);
  if (rc) return rc;
  Problem q{batch, nstacks, log_n, nblocks, input_size, 1 << log_n, increasing_stride != 0, false};
  return drive_linear_bw(ex, q, twiddle, x, x_sB, grad, g_sB, d_twiddle, d_input, d_input_sB, d_bias, output_size, workspace,
                         workspace_bytes);
}
int bfly_fw_f32_saving(const float* twiddle, const float* x, int64_t x_sB, int64_t x_sS, float* out, int batch,
                       int nstacks, int log_n, int nblocks, int input_size, int output_size, int increasing_stride,
                       void* snapshots, size_t snapshot_bytes, void* stream) {
  return fw_saving_entry<float>(twiddle, x, x_sB, x_sS, out, batch, nstacks, log_n, nblocks, input_size, output_size,
                                increasing_stride, snapshots, snapshot_bytes, stream);
}
int bfly_fw_c64_saving(const void* twiddle, const void* x, int64_t x_sB, int64_t x_sS, void* out, int batch,
                       int nstacks, int log_n, int nblocks, int input_size, int output_size, int increasing_stride,
                       void* snapshots, size_t snapshot_bytes, void* stream) {
  return fw_saving_entry<cf>(twiddle, x, x_sB, x_sS, out, batch, nstacks, log_n, nblocks, input_size, output_size,
                             increasing_stride, snapshots, snapshot_bytes, stream);
}
int bfly_bw_f32_saved(const float* twiddle, const float* x, int64_t x_sB, int64_t x_sS, const float* grad,
                      int64_t g_sB, int64_t g_sS, float* d_twiddle, float* d_x, int batch, int nstacks, int log_n,
                      int nblocks, int input_size, int output_size, int increasing_stride, void* snapshots,
                      size_t snapshot_bytes, void* stream) {
  return bw_entry<float>(false, twiddle, nullptr, x, x_sB, x_sS, grad, g_sB, g_sS, d_twiddle, nullptr, d_x, batch,
                         nstacks, log_n, nblocks, input_size, output_size, increasing_stride, snapshots,
                         snapshot_bytes, stream, true);
}
int bfly_bw_c64_saved(const void* twiddle, const void* x, int64_t x_sB, int64_t x_sS, const void* grad, int64_t g_sB,
                      int64_t g_sS, void* d_twiddle, void* d_x, int batch, int nstacks, int log_n, int nblocks,
                      int input_size, int output_size, int increasing_stride, void* snapshots, size_t snapshot_bytes,
                      void* stream) {
  return bw_entry<cf>(false, twiddle, nullptr, x, x_sB, x_sS, grad, g_sB, g_sS, d_twiddle, nullptr, d_x, batch,
                      nstacks, log_n, nblocks, input_size, output_size, increasing_stride, snapshots, snapshot_bytes,
                      stream, true);
}
int bfly_bw_f32_noalloc(const float* twiddle, const float* x, int64_t x_sB, int64_t x_sS, const float* grad,
                        int64_t g_sB, int64_t g_sS, float* d_twiddle, float* d_x, int batch, int nstacks, int log_n,
                        int nblocks, int input_size, int output_size, int increasing_stride, void* stream) {
  // how much scratch this very call needs (direction known here, unlike the workspace query)
  Problem q{batch, nstacks, log_n, nblocks, input_size, output_size, increasing_stride != 0, false};
  int rc = check_problem(q);
  if (rc) return rc;
  BwLayout<float> lay;
  rc = plan_bw<float>(q, lay);
  if (rc) return rc;
  if (lay.ws_bytes > (size_t)BFLY_NOALLOC_SCRATCH_BYTES) return BFLY_E_TOOLARGE;
  void* scratch = nullptr;
  if (lay.ws_bytes > 0) {
    rc = noalloc_scratch_ptr(&scratch);
    if (rc) return rc;
  }
  return bw_entry<float>(false, twiddle, nullptr, x, x_sB, x_sS, grad, g_sB, g_sS, d_twiddle, nullptr, d_x,
                         batch, nstacks, log_n, nblocks, input_size, output_size, increasing_stride, scratch,
                         lay.ws_bytes, stream);
}
int bfly4_fw_f32(const float* twiddle4, const float* twiddle2, const float* x, int64_t x_sB, int64_t x_sS,
                 float* out, int batch, int nstacks, int log_n, int nblocks, int input_size, int output_size,
                 int increasing_stride, void* stream) {
  return fw_entry<float>(true, twiddle2, twiddle4, x, x_sB, x_sS, out, batch, nstacks, log_n, nblocks,
                         input_size, output_size, increasing_stride, stream);
}
int bfly4_fw_c64(const void* twiddle4, const void* twiddle2, const void* x, int64_t x_sB, int64_t x_sS, void* out,
                 int batch, int nstacks, int log_n, int nblocks, int input_size, int output_size,
                 int increasing_stride, void* stream) {
  return fw_entry<cf>(true, twiddle2, twiddle4, x, x_sB, x_sS, out, batch, nstacks, log_n, nblocks, input_size,
                      output_size, increasing_stride, stream);
}
int bfly4_bw_c64(const void* twiddle4, const void* twiddle2, const void* x, int64_t x_sB, int64_t x_sS,
                 const void* grad, int64_t g_sB, int64_t g_sS, void* d_twiddle4, void* d_twiddle2, void* d_x,
                 int batch, int nstacks, int log_n, int nblocks, int input_size, int output_size,
                 int increasing_stride, void* workspace, size_t workspace_bytes, void* stream) {
  return bw_entry<cf>(true, twiddle2, twiddle4, x, x_sB, x_sS, grad, g_sB, g_sS, d_twiddle2, d_twiddle4, d_x, batch,
                      nstacks, log_n, nblocks, input_size, output_size, increasing_stride, workspace,
                      workspace_bytes, stream);
}
int64_t bfly4_bw_workspace_bytes(int dtype, int batch, int nstacks, int log_n, int nblocks) {
  return ws_entry(true, dtype, batch, nstacks, log_n, nblocks);
}
int bfly4_bw_f32(const float* twiddle4, const float* twiddle2, const float* x, int64_t x_sB, int64_t x_sS,
                 const float* grad, int64_t g_sB, int64_t g_sS, float* d_twiddle4, float* d_twiddle2, float* d_x,
                 int batch, int nstacks, int log_n, int nblocks, int input_size, int output_size,
                 int increasing_stride, void* workspace, size_t workspace_bytes, void* stream) {
  return bw_entry<float>(true, twiddle2, twiddle4, x, x_sB, x_sS, grad, g_sB, g_sS, d_twiddle2, d_twiddle4, d_x,
                         batch, nstacks, log_n, nblocks, input_size, output_size, increasing_stride, workspace,
                         workspace_bytes, stream);
}

}  // extern "C"
