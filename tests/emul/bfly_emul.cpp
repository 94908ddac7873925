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
#include "bfly_bw2.h"
#include "bfly_bw3.h"
#include "bfly_driver.h"
#include "bfly_glue.h"

using namespace bfly;

namespace {

long g_fw2_calls = 0;  // launches the emulator ran through the packed-pair forward path
long g_bw3_calls = 0;  // ... and through the packed-pair backward phase path

struct EmulExec {
  int sms = 7;       // odd on purpose: exercises ragged row slices
  int threads_ = 64;  // simulated block size (any power of two)
  int num_sms() const { return sms; }
  int threads() const { return threads_; }
  bool bw2 = true;   // exercise the second-generation backward where the driver selects it
  bool has_bw2(size_t /*elem_size*/, int kw) const { return bw2 && kw == 2; }

  // packed-pair forward kernel: boxes copied by plain loops, groups run thread by thread in plan
  // order (a valid schedule of the device kernel's barriers)
  bool fw2 = true;
  int run_fw2(const Fw2Params& p_in, int /*ctas_per_sm*/) {
    if (!fw2) return kFw2Declined;
    Fw2Params p = p_in;
    const int n = 1 << p.log_n;
    if (p.view && ((p.panel.lseg != p.panel.logC && p.panel.lseg != 5) || p.bias)) return kFw2Declined;
    if (p.x_cols % 32 != 0 && p.x_cols < n) return kFw2Declined;  // what the TMA descriptors would refuse
    if (p.out && p.out_cols % 32 != 0) return kFw2Declined;
    p.has_out = p.out != nullptr;
    if (!p.has_out) p.out_cols = n;
    ++g_fw2_calls;
    for (int64_t e = 0; e < fw2_pack_entries(p); ++e) fw2_pack_one(p, e);  // the re-ordering kernel
    std::vector<float> tile((size_t)p.R * n);
    const int64_t ntiles = fw2_num_tiles(p);
    auto box_copy = [&](bool load, const float* src, float* dst, int64_t sB, int64_t sS, int cols, int stack, int row0) {
      for (int r = 0; r < p.R; ++r)
        for (int c = 0; c < n; ++c) {
          float& t = tile[fw2_tile_index(p.R, r, c)];
          const int row = row0 + r;
          const bool in = row < p.B && c < cols;
          // a panel view addresses (panel, local column) -> real column of the one real stack
          const int64_t at = p.view ? (int64_t)row * sB + fw2_view_col(p, stack, c) : (int64_t)row * sB + (int64_t)stack * sS + c;
          if (load) t = in ? src[at] : 0.f;
          else if (in) dst[at] = t;
        }
    };
    for (int64_t t = 0; t < ntiles; ++t) {
      const int stack = (int)(t % p.S), row0 = (int)(t / p.S) * p.R;
      box_copy(true, p.x, nullptr, p.x_sB, p.x_sS, std::min(p.x_cols, n), stack, row0);
      for (int gi = 0; gi < p.ngroups; ++gi) {
        for (int tid = 0; tid < fw2_threads(p); ++tid) {
          f2 T[48];
          fw2_fetch_tw(p, p.g[gi], stack, tid, T);
          if (tid & 1) fw2_group_dispatch<true>(p, p.g[gi], tile.data(), tid, T);  // both row-loop forms
          else fw2_group_dispatch<false>(p, p.g[gi], tile.data(), tid, T);
        }
        if (p.g[gi].emit) box_copy(false, nullptr, p.snap[p.g[gi].emit - 1], p.view ? (int64_t)p.view_row : (int64_t)p.S * n, n, n, stack, row0);
      }
      if (p.has_out && p.bias)  // the store epilogue of the device kernel
        for (int r = 0; r < p.R; ++r)
          for (int c = 0; c < n; ++c)
            if (stack * n + c < p.bias_len) tile[fw2_tile_index(p.R, r, c)] += p.bias[stack * n + c];
      if (p.has_out) box_copy(false, nullptr, p.out, p.out_sB, p.out_sS, p.out_cols, stack, row0);
    }
    return BFLY_OK;
  }

  // packed-pair backward phase: the device kernel's steps, thread by thread, accumulators in a heap array
  bool bw3 = true;
  bool can_run_bw3(const Bw3Params& p) const {
    const BwParams<float>& q = p.b;
    // what the TMA descriptors would refuse: widths that are not whole 32-column blocks, and, for
    // panels made of strided segments, rows that are not whole groups of segments
    if (!bw3 || !q.vec_x || !q.vec_g || !q.vec_o || q.xin_cols % 32 || q.gin_cols % 32 || q.gout_cols % 32) return false;
    if (q.panel.lseg != q.panel.logC) {
      const int grp = 1 << q.panel.pb;
      for (int cols : {q.xin_cols, q.gin_cols, q.gout_cols})
        if (cols % grp != 0 && cols >= grp) return false; else if (cols < grp) return false;
    }
    return true;
  }
  int run_bw3(const Bw3Params& p) {
    if (!can_run_bw3(p)) return kFw2Declined;
    const BwParams<float>& q = p.b;
    ++g_bw3_calls;
    const int C = 1024, nthr = kBw3Threads;
    std::vector<float> smem((size_t)(q.nsg + 1) * kBw3Rows * C);
    float* smX = smem.data();
    float* smG = smem.data() + (size_t)q.nsg * kBw3Rows * C;
    std::vector<uint32_t> meta((size_t)q.nsg * nthr * 4 + 8);
    std::vector<float> accmem((size_t)nthr * kBw3MaxSg * 64);
    std::vector<float> pf((size_t)nthr * 64);  // per-thread fetch buffers (twiddles, accumulators of the next step)
    const int nctas = bw_num_ctas(q);
    for (int cta = 0; cta < nctas; ++cta) {
      int pbase, stack, rb, re;
      bw_cta_coords(q, cta, pbase, stack, rb, re);
      std::vector<Acc3Host> accs(nthr);
      for (int tid = 0; tid < nthr; ++tid) {
        accs[tid].mem = accmem.data() + (size_t)tid * kBw3MaxSg * 64;
        bw3_init(p, accs[tid], meta.data(), stack, pbase, tid);
        bw3_prefetch(p, accs[tid], 0, pf.data() + (size_t)tid * 64, pf.data() + (size_t)tid * 64 + 32);
      }
      for (int row0 = rb; row0 < re; row0 += kBw3Rows) {
        for (int tid = 0; tid < nthr; ++tid) {
          tile_load_auto<float>(q.xin, q.xin_sB, q.xin_sS, q.xin_cols, q.B, stack, row0, kBw3Rows, q.panel, pbase, true, smX, tid, nthr);
          tile_load_auto<float>(q.gin, q.gin_sB, q.gin_sS, q.gin_cols, q.B, stack, row0, kBw3Rows, q.panel, pbase, true, smG, tid, nthr);
        }
        if (q.dbias)  // column sums of the gradient tile as it arrived
          for (int r = 0; r < kBw3Rows; ++r)
            for (int l = 0; l < C; ++l) {
              const int flat = stack * (1 << q.log_n) + q.panel.col(pbase, l);
              if (flat < q.dbias_len) q.dbias[flat] += smG[r * C + swz<2>(l)];
            }
        for (int step = 0; step < bw3_num_steps(q.nsg); ++step)
          for (int tid = 0; tid < nthr; ++tid)
            bw3_step(p, accs[tid], meta.data(), step, smem.data(), tid, pf.data() + (size_t)tid * 64, pf.data() + (size_t)tid * 64 + 32);
        if (q.gout_reduce) {  // the device kernel's reduce-add store
          for (int r = 0; r < kBw3Rows && row0 + r < q.B; ++r)
            for (int l = 0; l < C; ++l) {
              const int col = q.panel.col(pbase, l);
              if (col < q.gout_cols) q.gout[(int64_t)(row0 + r) * q.gout_sB + (int64_t)stack * q.gout_sS + col] += smG[r * C + swz<2>(l)];
            }
        } else {
          for (int tid = 0; tid < nthr; ++tid)
            tile_store_auto<float>(q.gout, q.gout_sB, q.gout_sS, q.gout_cols, q.B, stack, row0, kBw3Rows, q.panel, pbase, true, smG, tid, nthr);
        }
      }
      for (int tid = 0; tid < nthr; ++tid) bw3_flush(p, accs[tid], stack, pbase, tid);
    }
    return BFLY_OK;
  }

  template <typename T> int run_fw(const FwParams<T>& p) {
    const int C = 1 << p.panel.logC;
    std::vector<T> sm((size_t)p.R * C);
    std::vector<uint16_t> tab((size_t)p.ngroups * p.tab_slots * threads_ + 1);
    for (int tid = 0; tid < threads_; ++tid) fw_build_table<T>(p, tab.data(), tid, threads_);
    const int64_t ntiles = fw_num_tiles(p);
    const int64_t n = (int64_t)1 << p.log_n;
    for (int64_t tile = 0; tile < ntiles; ++tile) {
      int row0, stack, pbase;
      fw_tile_coords(p, tile, row0, stack, pbase);
      for (int tid = 0; tid < threads_; ++tid) {
        if (p.glue.x_real) tile_load_real(p.glue.x_real, p.x_sB, p.x_sS, p.x_cols, p.B, stack, row0, p.R, p.panel.logC, sm.data(), tid, threads_);
        else tile_load_auto<T>(p.x, p.x_sB, p.x_sS, p.x_cols, p.B, stack, row0, p.R, p.panel, pbase, p.vec_in != 0, sm.data(), tid, threads_);
      }
      // the kernel's gather pass: every thread reads, barrier, every thread writes
      auto permute_rows = [&](const int32_t* perm, const T* diag) {
        const int slots = (C + threads_ - 1) / threads_;
        std::vector<T> v((size_t)threads_ * slots);
        std::vector<uint32_t> plan((size_t)threads_ * slots);
        std::vector<int> cnt(threads_);
        for (int tid = 0; tid < threads_; ++tid)
          cnt[tid] = tile_permute_plan<T>(p.panel.logC, perm, p.glue.colbit, tid, threads_, plan.data() + (size_t)tid * slots);
        for (int r = 0; r < p.R; ++r) {
          for (int tid = 0; tid < threads_; ++tid)
            tile_permute_read<T>(sm.data(), r, p.panel.logC, diag, plan.data() + (size_t)tid * slots, cnt[tid], v.data() + (size_t)tid * slots);
          for (int tid = 0; tid < threads_; ++tid)
            tile_permute_write<T>(sm.data(), r, p.panel.logC, plan.data() + (size_t)tid * slots, cnt[tid], v.data() + (size_t)tid * slots);
        }
      };
      if (p.glue.any_in()) permute_rows(p.glue.in_perm, nullptr);
      for (int g = 0; g < p.ngroups; ++g) {
        for (int tid = 0; tid < threads_; ++tid)
          fw_group_dispatch<T, 4, 0, 0>(p, g, sm.data(), tab.data(), p.R, stack, pbase, tid, threads_);
        if (p.g[g].emit)
          for (int tid = 0; tid < threads_; ++tid)
            tile_store_auto<T>(p.snap[p.g[g].emit - 1], (int64_t)p.S * n, n, (int)n, p.B, stack, row0, p.R, p.panel, pbase, true, sm.data(), tid, threads_);
      }
      if (p.glue.any_out()) {
        if (p.glue.out_perm) permute_rows(p.glue.out_perm, p.glue.out_diag);
        else for (int tid = 0; tid < threads_; ++tid) tile_scale_rows<T>(sm.data(), p.R, p.panel.logC, p.glue.out_diag, tid, threads_);
      }
      if (p.glue.out_real)
        for (int tid = 0; tid < threads_; ++tid)
          tile_store_real(p.glue.out_real, p.out_sB, p.out_sS, p.out_cols, p.B, stack, row0, p.R, p.panel.logC, sm.data(), tid, threads_);
      else if (p.out)
        for (int tid = 0; tid < threads_; ++tid)
          tile_store_auto<T>(p.out, p.out_sB, p.out_sS, p.out_cols, p.B, stack, row0, p.R, p.panel, pbase, p.vec_out != 0, sm.data(), tid, threads_);
    }
    return BFLY_OK;
  }

  // second-generation backward: same step routines as the device kernel, accumulators in a heap array
  template <typename T, int KW> int run_bw2(const BwParams<T>& p) {
    constexpr int N = BwTwn<KW>::value;
    const int C = 1 << p.panel.logC;
    const int nthr = C >> KW;
    // one buffer, as on the device: nsg snapshot tiles followed by the gradient tile
    std::vector<T> smem((size_t)(p.nsg + 1) * kBw2Rows * C);
    struct View { T* ptr; T* data() const { return ptr; } };
    const View smX{smem.data()}, smG{smem.data() + (size_t)p.nsg * kBw2Rows * C};
    std::vector<uint32_t> meta((size_t)p.nsg * kBw2Meta * nthr);
    std::vector<T> accmem((size_t)nthr * 2 * kMaxSg * N);
    const int nctas = bw_num_ctas(p);
    for (int cta = 0; cta < nctas; ++cta) {
      int pbase, stack, rb, re;
      bw_cta_coords(p, cta, pbase, stack, rb, re);
      std::vector<AccStore<T, KW>> accs(nthr);
      for (int tid = 0; tid < nthr; ++tid) {
        accs[tid].mem = accmem.data() + (size_t)tid * 2 * kMaxSg * N;
        bw2_build_meta<T, KW>(p, meta.data(), pbase, tid, nthr);
      }
      for (int tid = 0; tid < nthr; ++tid) bw2_init<T, KW>(p, accs[tid], meta.data(), stack, tid, nthr);
      for (int row0 = rb; row0 < re; row0 += kBw2Rows) {
        for (int tid = 0; tid < nthr; ++tid) {
          tile_load_auto<T>(p.xin, p.xin_sB, p.xin_sS, p.xin_cols, re, stack, row0, kBw2Rows, p.panel, pbase, p.vec_x != 0, smX.data(), tid, nthr);
          tile_load_auto<T>(p.gin, p.gin_sB, p.gin_sS, p.gin_cols, re, stack, row0, kBw2Rows, p.panel, pbase, p.vec_g != 0, smG.data(), tid, nthr);
        }
        for (int j = 0; j + 1 < p.nsg; ++j)
          for (int tid = 0; tid < nthr; ++tid)
            bw2_fw_step<T, KW, 0>(p, accs[tid], meta.data(), j, smX.data(), smG.data(), tid, nthr);
        for (int j = p.nsg - 1; j >= 0; --j)
          for (int tid = 0; tid < nthr; ++tid)
            bw2_bw_step<T, KW, 0>(p, accs[tid], meta.data(), j, smX.data(), smG.data(), tid, nthr);
        for (int tid = 0; tid < nthr; ++tid)
          tile_store_auto<T>(p.gout, p.gout_sB, p.gout_sS, p.gout_cols, re, stack, row0, kBw2Rows, p.panel, pbase, p.vec_o != 0, smG.data(), tid, nthr);
      }
      for (int tid = 0; tid < nthr; ++tid) bw2_flush<T, KW>(p, accs[tid], meta.data(), stack, tid, nthr);
    }
    return BFLY_OK;
  }

  template <typename T, int KW> int run_bw_kw(const BwParams<T>& p) {
    if (p.v2) return run_bw2<T, KW>(p);
    constexpr int NSG = kMaxSg;
    const int C = 1 << p.panel.logC;
    // the device kernel uses exactly one thread per unit (or a power-of-two multiple)
    int nthr = threads_;
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
          tile_load_auto<T>(p.xin, p.xin_sB, p.xin_sS, p.xin_cols, re, stack, row0, R, p.panel, pbase, p.vec_x != 0, smX.data(), tid, nthr);
          tile_load_auto<T>(p.gin, p.gin_sB, p.gin_sS, p.gin_cols, re, stack, row0, R, p.panel, pbase, p.vec_g != 0, smG.data(), tid, nthr);
        }
        for (int j = 0; j + 1 < p.nsg; ++j)
          for (int tid = 0; tid < nthr; ++tid) bw_sg_step<T, KW, NSG, 0, 0, true>(p, st[tid], j, stack, smX.data(), smG.data(), R, tid, nthr);
        for (int j = p.nsg - 1; j >= 0; --j)
          for (int tid = 0; tid < nthr; ++tid) bw_sg_step<T, KW, NSG, 0, 0, false>(p, st[tid], j, stack, smX.data(), smG.data(), R, tid, nthr);
        for (int tid = 0; tid < nthr; ++tid)
          tile_store_auto<T>(p.gout, p.gout_sB, p.gout_sS, p.gout_cols, re, stack, row0, R, p.panel, pbase, p.vec_o != 0, smG.data(), tid, nthr);
      }
      for (int tid = 0; tid < nthr; ++tid) bw_flush_state<T, KW, NSG>(p, st[tid], stack, pbase, tid, nthr);
    }
    return BFLY_OK;
  }
  template <typename T> int run_bw(const BwParams<T>& p, int KW) {
    return KW == 2 ? run_bw_kw<T, 2>(p) : run_bw_kw<T, 1>(p);
  }
  int add_bias(float* out, const float* bias, int64_t B, int len, int64_t pitch) {
    for (int64_t b = 0; b < B; ++b)
      for (int f = 0; f < len; ++f) out[b * pitch + f] += bias[f];
    return BFLY_OK;
  }
  int zero(void* ptr, size_t bytes) { std::memset(ptr, 0, bytes); return BFLY_OK; }
  int zero2d(void* ptr, size_t pitch, size_t width, size_t rows) {
    for (size_t r = 0; r < rows; ++r) std::memset(static_cast<char*>(ptr) + r * pitch, 0, width);
    return BFLY_OK;
  }
};

template <typename T>
int emul_fw(const void* tw2, const void* tw4, const void* x, int64_t x_sB, int64_t x_sS, void* out, Problem q, int threads) {
  EmulExec ex; ex.threads_ = threads;
  std::vector<char> ws(fw_workspace_bytes<T>(q) + 256);
  void* wsp = (void*)(((uintptr_t)ws.data() + 255) / 256 * 256);
  return drive_fw<T>(ex, q, (const T*)tw2, (const T*)tw4, (const T*)x, x_sB, x_sS, (T*)out, wsp, fw_workspace_bytes<T>(q));
}
template <typename T>
int emul_bw(const void* tw2, const void* tw4, const void* x, int64_t x_sB, int64_t x_sS, const void* g, int64_t g_sB, int64_t g_sS,
            void* d2, void* d4, void* dx, Problem q, int threads, int sms) {
  EmulExec ex; ex.threads_ = threads; ex.sms = sms;
  BwLayout<T> lay;
  int rc = check_problem(q);
  if (rc) return rc;
  rc = plan_bw<T>(q, lay);
  if (rc) return rc;
  std::vector<char> ws(lay.ws_bytes + 256);
  void* wsp = (void*)(((uintptr_t)ws.data() + 255) / 256 * 256);
  return drive_bw<T>(ex, q, (const T*)tw2, (const T*)tw4, (const T*)x, x_sB, x_sS, (const T*)g, g_sB, g_sS, (T*)d2, (T*)d4, (T*)dx, wsp, lay.ws_bytes);
}

// forward that saves the phase-boundary activations, then the backward that starts from them
template <typename T>
int emul_fw_bw_saved(const void* tw2, const void* x, int64_t x_sB, int64_t x_sS, void* out, const void* g, int64_t g_sB,
                     int64_t g_sS, void* d2, void* dx, Problem q, int threads, int sms) {
  EmulExec ex; ex.threads_ = threads; ex.sms = sms;
  BwLayout<T> lay;
  int rc = check_problem(q);
  if (rc) return rc;
  rc = plan_bw<T>(q, lay);
  if (rc) return rc;
  std::vector<char> ws(lay.ws_bytes + 256);
  void* wsp = (void*)(((uintptr_t)ws.data() + 255) / 256 * 256);
  rc = drive_fw_saving<T>(ex, q, (const T*)tw2, (const T*)nullptr, (const T*)x, x_sB, x_sS, (T*)out, wsp, lay.ws_bytes);
  if (rc) return rc;
  return drive_bw<T>(ex, q, (const T*)tw2, (const T*)nullptr, (const T*)x, x_sB, x_sS, (const T*)g, g_sB, g_sS, (T*)d2,
                     (T*)nullptr, (T*)dx, wsp, lay.ws_bytes, true);
}

}  // namespace

// Worst shared-memory bank-conflict degree (1 = conflict-free) of the accesses a 256-thread CTA
// makes to one tile row: per group / sub-group, per warp, per element of the unit.  An access of
// `bytes` per lane is served in phases of 128/bytes lanes; the degree of a phase is the largest
// number of distinct 4-byte words that fall into one of the 32 banks.
static int conflict_degree(const std::vector<long>& byte_addr, int bytes) {
  const int lanes_per_phase = 128 / bytes;
  int worst = 1;
  for (size_t p0 = 0; p0 < byte_addr.size(); p0 += lanes_per_phase) {
    std::vector<std::vector<long>> bank(32);
    for (size_t i = p0; i < p0 + lanes_per_phase && i < byte_addr.size(); ++i)
      for (int w = 0; w < bytes / 4; ++w) {
        const long word = byte_addr[i] / 4 + w;
        auto& b = bank[word % 32];
        if (std::find(b.begin(), b.end(), word) == b.end()) b.push_back(word);
      }
    for (auto& b : bank) worst = std::max<int>(worst, (int)b.size());
  }
  return worst;
}

template <typename T>
static int window_conflicts(int logC, int lbit, int K, bool vec, const uint8_t* ubit, int nubits, const uint16_t* d) {
  const int nthr = 256, C = 1 << logC, U = C >> K;
  if (U < 32) return 1;  // tiny rows: several rows share a warp, not analysed
  int worst = 1;
  const int V = Vec16<T>::N, E = 1 << K;
  for (int warp = 0; warp < std::min(nthr, U) / 32; ++warp)
    for (int m = 0; m < (vec ? E / V : E); ++m) {
      std::vector<long> addr;
      for (int lane = 0; lane < 32; ++lane) {
        const int u = warp * 32 + lane;
        const int a0 = swzT<T>(deposit_unit(u, ubit, nubits));
        addr.push_back((long)(a0 ^ d[vec ? m * V : m]) * (long)sizeof(T));
      }
      worst = std::max(worst, conflict_degree(addr, vec ? 16 : (int)sizeof(T)));
    }
  return worst;
}

template <typename T>
static int max_conflicts(const Problem& q, int kmax) {
  const std::vector<Stage> st = problem_stages(q);
  int worst = 1;
  std::vector<FwGroup> groups;
  const Panel pn = full_row_panel(q.log_n);
  if (!plan_fw_groups(st, 0, (int)st.size(), {}, pn, Vec16<T>::LOG, kmax, groups)) return -1;
  for (auto& g : groups) worst = std::max(worst, window_conflicts<T>(pn.logC, g.lbit, g.K, g.vec != 0, g.ubit, g.nubits, g.d));
  BwLayout<T> lay;
  if (plan_bw<T>(q, lay) != BFLY_OK) return -1;
  for (auto& ph : lay.phases)
    for (int j = 0; j < ph.nsg; ++j) {
      const BwSg& sg = ph.sg[j];
      const int width = sg.radix == 4 ? 2 : lay.kw;
      worst = std::max(worst, window_conflicts<T>(ph.panel.logC, sg.lbit, width, sg.vec != 0, sg.ubit, sg.nubits, sg.d));
    }
  return worst;
}

extern "C" {
// the per-block arithmetic of the unitary twiddle kernels (bfly_glue.h), looped on the host
void bfly_emul_unitary_fw(const float* angles, float* tw, int64_t blocks) {
  for (int64_t i = 0; i < blocks; ++i) unitary_block_fw(angles + 4 * i, tw + 8 * i);
}
void bfly_emul_unitary_bw(const float* angles, const float* g, float* d, int64_t blocks) {
  for (int64_t i = 0; i < blocks; ++i) unitary_block_bw(angles + 4 * i, g + 8 * i, d + 4 * i);
}
long bfly_emul_fw2_calls(void) { return g_fw2_calls; }
long bfly_emul_bw3_calls(void) { return g_bw3_calls; }
// the library's development switches (bfly_driver.h) for this emulator instance
int bfly_emul_set_option(const char* name, int value) { return set_option(name, value); }
int bfly_emul_get_option(const char* name) { int v = -1; get_option(name, &v); return v; }
int bfly_emul_max_conflicts(int dtype, int base4, int log_n, int nblocks, int inc, int kmax) {
  Problem q{4, 1, log_n, nblocks, 1 << log_n, 1 << log_n, inc != 0, base4 != 0};
  return dtype == 0 ? max_conflicts<float>(q, kmax) : max_conflicts<cf>(q, kmax);
}
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
int bfly_emul_fw_bw_saved(int dtype, const void* tw, const void* x, int64_t x_sB, int64_t x_sS, void* out, const void* g,
                          int64_t g_sB, int64_t g_sS, void* d_tw, void* dx, int B, int S, int log_n, int nblocks, int in_size,
                          int out_size, int inc, int threads, int sms) {
  Problem q{B, S, log_n, nblocks, in_size, out_size, inc != 0, false};
  return dtype == 0 ? emul_fw_bw_saved<float>(tw, x, x_sB, x_sS, out, g, g_sB, g_sS, d_tw, dx, q, threads, sms)
                    : emul_fw_bw_saved<cf>(tw, x, x_sB, x_sS, out, g, g_sB, g_sS, d_tw, dx, q, threads, sms);
}
// fused linear layer: forward into out (B, S * n), backward with d_input summed over the stacks and d_bias
int bfly_emul_linear_fw(const void* tw, const void* x, int64_t x_sB, void* out, const void* bias, int B, int S, int log_n,
                        int nblocks, int in_size, int out_total, int inc) {
  EmulExec ex; ex.threads_ = 256;
  Problem q{B, S, log_n, nblocks, in_size, 1 << log_n, inc != 0, false};
  std::vector<char> ws(fw_workspace_bytes<float>(q) + 256);
  void* wsp = (void*)(((uintptr_t)ws.data() + 255) / 256 * 256);
  return drive_linear_fw(ex, q, (const float*)tw, (const float*)x, x_sB, (float*)out, (const float*)bias, out_total, wsp,
                         fw_workspace_bytes<float>(q));
}
int bfly_emul_linear_bw(const void* tw, const void* x, int64_t x_sB, const void* g, int64_t g_sB, void* d_tw, void* d_in,
                        int64_t din_sB, void* d_bias, int B, int S, int log_n, int nblocks, int in_size, int out_total, int inc,
                        int sms) {
  EmulExec ex; ex.threads_ = 256; ex.sms = sms;
  Problem q{B, S, log_n, nblocks, in_size, 1 << log_n, inc != 0, false};
  LinearBwLayout L;
  int rc = check_problem(q);
  if (rc) return rc;
  rc = plan_linear_bw(q, L);
  if (rc) return rc;
  std::vector<char> ws(L.ws_bytes + 256);
  void* wsp = (void*)(((uintptr_t)ws.data() + 255) / 256 * 256);
  return drive_linear_bw(ex, q, (const float*)tw, (const float*)x, x_sB, (const float*)g, g_sB, (float*)d_tw, (float*)d_in,
                         din_sB, (float*)d_bias, out_total, wsp, L.ws_bytes);
}
// the forward with glue operators (drive_fw_glue); dtype 0 float32, 1 complex64
int bfly_emul_fw_glue(int dtype, const void* tw, const void* x, int x_is_real, int64_t x_sB, int64_t x_sS, void* out, int out_is_real,
                      const int32_t* in_perm, const void* out_diag, const int32_t* out_perm, int B, int S, int log_n, int nblocks,
                      int in_size, int out_size, int inc, int threads) {
  EmulExec ex; ex.threads_ = threads;
  Problem q{B, S, log_n, nblocks, in_size, out_size, inc != 0, false};
  if (dtype == 0) {
    FwGlue<float> g{};
    g.in_perm = in_perm; g.out_perm = out_perm; g.out_diag = (const float*)out_diag;
    return drive_fw_glue<float>(ex, q, (const float*)tw, (const float*)x, x_sB, x_sS, (float*)out, g);
  }
  FwGlue<cf> g{};
  g.in_perm = in_perm; g.out_perm = out_perm; g.out_diag = (const cf*)out_diag;
  if (x_is_real) g.x_real = (const float*)x;
  if (out_is_real) g.out_real = (float*)out;
  return drive_fw_glue<cf>(ex, q, (const cf*)tw, x_is_real ? nullptr : (const cf*)x, x_sB, x_sS, out_is_real ? nullptr : (cf*)out, g);
}
// number of backward phases and workspace bytes the planner chooses (for tests of the planner)
int bfly_emul_bw_plan(int dtype, int base4, int B, int S, int log_n, int nblocks, int inc, int64_t* ws_bytes) {
  Problem q{B, S, log_n, nblocks, 1 << log_n, 1 << log_n, inc != 0, base4 != 0};
  int rc = check_problem(q);
  if (rc) return rc;
  size_t ws = 0; int nph = 0;
  if (dtype == 0) { BwLayout<float> l; rc = plan_bw<float>(q, l); ws = l.ws_bytes; nph = (int)l.phases.size(); }
  else { BwLayout<cf> l; rc = plan_bw<cf>(q, l); ws = l.ws_bytes; nph = (int)l.phases.size(); }
  if (rc) return rc;
  *ws_bytes = (int64_t)ws;
  return nph;
}
}
