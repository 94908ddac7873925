// Test helper, not product code: runs the CUDA kernels' per-thread tile routines on the
// host, one simulated thread at a time, behind the same driver that plans the GPU
// launches.  It exists to check planning and index arithmetic on a machine without a
// GPU; the shipped library never falls back to it.
//
// Build: g++ -O2 -std=c++17 -fPIC -shared -I butterfly_b200/csrc tests/emul/bfly_emul.cpp -o tests/emul/libbfly_emul.so
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "bfly_core.h"
#include "bfly_driver.h"

using namespace bfly;

namespace {

struct EmulExec {
  int sms = 7;       // odd on purpose: exercises ragged row slices
  int threads = 64;  // simulated block size (any power of two)
  int num_sms() const { return sms; }

  template <typename T> int run_fw(const FwParams<T>& p) {
    const int C = 1 << p.panel.logC;
    std::vector<T> sm((size_t)p.R * C);
    const int64_t ntiles = fw_num_tiles(p);
    const int64_t n = (int64_t)1 << p.log_n;
    for (int64_t tile = 0; tile < ntiles; ++tile) {
      int row0, stack, pbase;
      fw_tile_coords(p, tile, row0, stack, pbase);
      for (int tid = 0; tid < threads; ++tid)
        tile_load<T>(p.x, p.x_sB, p.x_sS, p.x_cols, p.B, stack, row0, p.R, p.panel, pbase, p.vec_in != 0, sm.data(), tid, threads);
      for (int g = 0; g < p.ngroups; ++g) {
        for (int tid = 0; tid < threads; ++tid)
          fw_group_dispatch<T>(p, p.g[g], sm.data(), p.R, stack, pbase, tid, threads);
        if (p.g[g].emit)
          for (int tid = 0; tid < threads; ++tid)
            tile_store<T>(p.snap[p.g[g].emit - 1], (int64_t)p.S * n, n, (int)n, p.B, stack, row0, p.R, p.panel, pbase, true, sm.data(), tid, threads);
      }
      if (p.out)
        for (int tid = 0; tid < threads; ++tid)
          tile_store<T>(p.out, p.out_sB, p.out_sS, p.out_cols, p.B, stack, row0, p.R, p.panel, pbase, p.vec_out != 0, sm.data(), tid, threads);
    }
    return BFLY_OK;
  }

  template <typename T, int KW> int run_bw_kw(const BwParams<T>& p) {
    constexpr int NSG = kMaxSg;
    const int C = 1 << p.panel.logC;
    // the device kernel uses exactly one thread per unit (or a power-of-two multiple)
    int nthr = threads;
    const int U = C >> KW;
    if (U > nthr) nthr = U;
    std::vector<T> smX((size_t)p.nsg * p.Rb * C), smG((size_t)p.Rb * C);
    std::vector<BwState<T, KW, NSG>> st(nthr);
    const int nctas = bw_num_ctas(p);
    for (int cta = 0; cta < nctas; ++cta) {
      int pbase, stack, rb, re;
      bw_cta_coords(p, cta, pbase, stack, rb, re);
      for (int tid = 0; tid < nthr; ++tid) bw_load_state<T, KW, NSG>(p, st[tid], stack, pbase, tid, nthr);
      for (int row0 = rb; row0 < re; row0 += p.Rb) {
        const int R = p.Rb;
        for (int tid = 0; tid < nthr; ++tid) {
          tile_load<T>(p.xin, p.xin_sB, p.xin_sS, p.xin_cols, re, stack, row0, R, p.panel, pbase, p.vec_x != 0, smX.data(), tid, nthr);
          tile_load<T>(p.gin, p.gin_sB, p.gin_sS, p.gin_cols, re, stack, row0, R, p.panel, pbase, p.vec_g != 0, smG.data(), tid, nthr);
        }
        for (int j = 0; j + 1 < p.nsg; ++j)
          for (int tid = 0; tid < nthr; ++tid) bw_sg_forward<T, KW, NSG>(p, st[tid], j, smX.data(), R, tid, nthr);
        for (int j = p.nsg - 1; j >= 0; --j)
          for (int tid = 0; tid < nthr; ++tid) bw_sg_backward<T, KW, NSG>(p, st[tid], j, smX.data(), smG.data(), R, tid, nthr);
        for (int tid = 0; tid < nthr; ++tid)
          tile_store<T>(p.gout, p.gout_sB, p.gout_sS, p.gout_cols, re, stack, row0, R, p.panel, pbase, p.vec_o != 0, smG.data(), tid, nthr);
      }
      for (int tid = 0; tid < nthr; ++tid) bw_flush_state<T, KW, NSG>(p, st[tid], stack, pbase, tid, nthr);
    }
    return BFLY_OK;
  }
  template <typename T> int run_bw(const BwParams<T>& p, int KW) {
    return KW == 2 ? run_bw_kw<T, 2>(p) : run_bw_kw<T, 1>(p);
  }
  int zero(void* ptr, size_t bytes) { std::memset(ptr, 0, bytes); return BFLY_OK; }
  int zero2d(void* ptr, size_t pitch, size_t width, size_t rows) {
    for (size_t r = 0; r < rows; ++r) std::memset(static_cast<char*>(ptr) + r * pitch, 0, width);
    return BFLY_OK;
  }
};

template <typename T>
int emul_fw(const void* tw2, const void* tw4, const void* x, int64_t x_sB, int64_t x_sS, void* out, Problem q, int threads) {
  EmulExec ex; ex.threads = threads;
  return drive_fw<T>(ex, q, (const T*)tw2, (const T*)tw4, (const T*)x, x_sB, x_sS, (T*)out);
}
template <typename T>
int emul_bw(const void* tw2, const void* tw4, const void* x, int64_t x_sB, int64_t x_sS, const void* g, int64_t g_sB, int64_t g_sS,
            void* d2, void* d4, void* dx, Problem q, int threads, int sms) {
  EmulExec ex; ex.threads = threads; ex.sms = sms;
  BwLayout<T> lay;
  int rc = check_problem(q);
  if (rc) return rc;
  rc = plan_bw<T>(q, lay);
  if (rc) return rc;
  std::vector<char> ws(lay.ws_bytes + 256);
  void* wsp = (void*)(((uintptr_t)ws.data() + 255) / 256 * 256);
  return drive_bw<T>(ex, q, (const T*)tw2, (const T*)tw4, (const T*)x, x_sB, x_sS, (const T*)g, g_sB, g_sS, (T*)d2, (T*)d4, (T*)dx, wsp, lay.ws_bytes);
}

}  // namespace

extern "C" {
// dtype: 0 float32, 1 complex64.  base4: tw2 = twiddle2, tw4 = twiddle4; else tw2 = twiddle.
int bfly_emul_fw(int dtype, int base4, const void* tw2, const void* tw4, const void* x, int64_t x_sB, int64_t x_sS, void* out,
                 int B, int S, int log_n, int nblocks, int in_size, int out_size, int inc, int threads) {
  Problem q{B, S, log_n, nblocks, in_size, out_size, inc != 0, base4 != 0};
  return dtype == 0 ? emul_fw<float>(tw2, tw4, x, x_sB, x_sS, out, q, threads) : emul_fw<cf>(tw2, tw4, x, x_sB, x_sS, out, q, threads);
}
int bfly_emul_bw(int dtype, int base4, const void* tw2, const void* tw4, const void* x, int64_t x_sB, int64_t x_sS, const void* g,
                 int64_t g_sB, int64_t g_sS, void* d2, void* d4, void* dx, int B, int S, int log_n, int nblocks, int in_size,
                 int out_size, int inc, int threads, int sms) {
  Problem q{B, S, log_n, nblocks, in_size, out_size, inc != 0, base4 != 0};
  return dtype == 0 ? emul_bw<float>(tw2, tw4, x, x_sB, x_sS, g, g_sB, g_sS, d2, d4, dx, q, threads, sms)
                    : emul_bw<cf>(tw2, tw4, x, x_sB, x_sS, g, g_sB, g_sS, d2, d4, dx, q, threads, sms);
}
// number of backward phases and workspace bytes the planner chooses (for tests of the planner)
int bfly_emul_bw_plan(int dtype, int base4, int B, int S, int log_n, int nblocks, int inc, int64_t* ws_bytes) {
  Problem q{B, S, log_n, nblocks, 1 << log_n, 1 << log_n, inc != 0, base4 != 0};
  int rc;
  size_t ws = 0; int nph = 0;
  if (dtype == 0) { BwLayout<float> l; rc = plan_bw<float>(q, l); ws = l.ws_bytes; nph = (int)l.phases.size(); }
  else { BwLayout<cf> l; rc = plan_bw<cf>(q, l); ws = l.ws_bytes; nph = (int)l.phases.size(); }
  if (rc) return rc;
  *ws_bytes = (int64_t)ws;
  return nph;
}
}
