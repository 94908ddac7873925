// Host driver shared by the CUDA library and the test-suite's host emulator: validates
// arguments, plans the launches and hands filled parameter blocks to an executor.
//
// Executor concept (E):
//   int  num_sms() const;
//   bool has_bw2(size_t elem_size, int kw) const;          // second-generation backward kernel available
//   int  threads() const;                                  // threads per CTA of its kernels
//   int  run_fw(const FwParams<T>&);                       // one forward launch
//   int  run_fw2(const Fw2Params&, int ctas_per_sm);       // twiddle re-ordering + one launch of the packed-pair
//                                                          // forward kernel (kFw2Declined: not available for these tensors)
//   int  run_bw(const BwParams<T>&, int KW);               // one backward-phase launch
//   int  run_bw3(const Bw3Params&);                        // one launch of the packed-pair backward phase kernel
//                                                          // (kFw2Declined: not available for these tensors)
//   bool can_run_bw3(const Bw3Params&);                    // would run_bw3 accept these tensors?
//   int  zero(void* ptr, size_t bytes);                    // async memset
//   int  zero2d(void* ptr, size_t pitch_bytes, size_t width_bytes, size_t rows);
//   int  add_bias(float* out, const float* bias, int64_t B, int len, int64_t pitch);   // out[b, f] += bias[f], f < len
#pragma once
#include <cstdlib>
#include <cstring>

#include "bfly_bw3.h"
#include "bfly_fw2.h"
#include "bfly_plan.h"

namespace bfly {

// Development and test switches.  They are read from the environment once, when first used
// (BFLY_TMA, BFLY_BW_V2, BFLY_FW2, BFLY_FW_KMAX, BFLY_FW_ROWS, BFLY_FW_LOGCMAX, BFLY_BW_ROWS,
// BFLY_BW_MAXSG, BFLY_AUTOGRAD_SAVE), and can be changed afterwards with set_option() (C ABI: bfly_set_option); the
// launch path itself never touches the environment.  -1 = not set (planner's default).
struct Options {
  int tma = 1;          // tile traffic through the TMA unit where tensors qualify
  int bw_v2 = 1;        // second-generation backward phase kernel
  int bw3 = 1;          // packed-pair backward phase kernel
  int fw2 = 1;          // packed-pair forward kernel
  int fw2_ctas = -1;    // packed-pair forward kernel: CTAs per SM (1 or 2; default 2)
  int fw_kmax = -1;     // generic forward: widest register window
  int fw_rows = -1;     // generic forward: rows per tile
  int fw_logcmax = -1;  // generic forward: widest panel (log2 columns) of a pass
  int bw_rows = -1;     // backward: rows per batch
  int bw_maxsg = -1;    // backward: sub-groups per phase
  int bw_c64_kw2 = 1;   // complex64 radix-2 backward on 2-stage sub-groups (tensor-memory kernel) for n >= 1024
  int bw3_min_rows = 100;  // fewest rows per CTA for which a plain backward phase takes the packed-pair kernel
  int autograd_save = -1;  // torch autograd operator: keep the forward's snapshots for the backward
};
struct OptionName { const char* name; const char* env; int Options::*field; };
inline const OptionName* option_names(int* count) {
  static const OptionName names[] = {
      {"tma", "BFLY_TMA", &Options::tma},           {"bw_v2", "BFLY_BW_V2", &Options::bw_v2},
      {"bw3", "BFLY_BW3", &Options::bw3},
      {"fw2", "BFLY_FW2", &Options::fw2},           {"fw_kmax", "BFLY_FW_KMAX", &Options::fw_kmax},
      {"fw2_ctas", "BFLY_FW2_CTAS", &Options::fw2_ctas},
      {"fw_rows", "BFLY_FW_ROWS", &Options::fw_rows}, {"fw_logcmax", "BFLY_FW_LOGCMAX", &Options::fw_logcmax},
      {"bw_rows", "BFLY_BW_ROWS", &Options::bw_rows}, {"bw_maxsg", "BFLY_BW_MAXSG", &Options::bw_maxsg},
      {"bw_c64_kw2", "BFLY_BW_C64_KW2", &Options::bw_c64_kw2},
      {"bw3_min_rows", "BFLY_BW3_MIN_ROWS", &Options::bw3_min_rows},
      {"autograd_save", "BFLY_AUTOGRAD_SAVE", &Options::autograd_save},
  };
  *count = (int)(sizeof(names) / sizeof(names[0]));
  return names;
}
inline Options& options() {
  static Options opt = [] {
    Options o;
    int cnt = 0;
    const OptionName* names = option_names(&cnt);
    for (int i = 0; i < cnt; ++i)
      if (const char* e = std::getenv(names[i].env)) o.*(names[i].field) = std::atoi(e);
    return o;
  }();
  return opt;
}
inline int set_option(const char* name, int value) {
  int cnt = 0;
  const OptionName* names = option_names(&cnt);
  for (int i = 0; name && i < cnt; ++i)
    if (std::strcmp(names[i].name, name) == 0) {
      options().*(names[i].field) = value;
      return BFLY_OK;
    }
  return BFLY_E_ARG;
}
inline int get_option(const char* name, int* value) {
  int cnt = 0;
  const OptionName* names = option_names(&cnt);
  for (int i = 0; name && value && i < cnt; ++i)
    if (std::strcmp(names[i].name, name) == 0) {
      *value = options().*(names[i].field);
      return BFLY_OK;
    }
  return BFLY_E_ARG;
}

template <typename T> struct KernelCfg;
template <> struct KernelCfg<float> {
  static constexpr int kFwKmaxTwoCtas = 3;  // widest window that still fits two CTAs per SM
  static constexpr int kFwKmaxOneCta = 4;   // widest window at one CTA per SM
  static constexpr int kThreads = 256;
  static int bw_kw(int log_n, bool /*base4*/) { return log_n >= 2 ? 2 : 1; }
  static int bw_max_sg(int kw) {
    if (kw != 2) return 10;
    const int v = options().bw_maxsg;  // experiments: other phase lengths
    if (v >= 1 && v <= 5) return v;
    return 4;  // 8 stages per phase: twiddles and accumulators of 4 sub-groups fill a thread's 128 TMEM columns
  }
};
template <> struct KernelCfg<cf> {
  static constexpr int kFwKmaxTwoCtas = 2;
  static constexpr int kFwKmaxOneCta = 3;
  static constexpr int kThreads = 256;
  // one-stage sub-groups for radix-2 products; a radix-4 factor needs the 2-bit window, and the
  // 16 complex accumulators per sub-group leave room for two sub-groups per phase
  // Full panels of 1024 complex columns (n >= 1024) also take the 2-bit window for radix-2 products:
  // phases of two 2-stage sub-groups on the kernel that keeps twiddles and accumulators in tensor
  // memory (4 stages per phase, two CTAs per SM) measure faster than 10 one-stage sub-groups.
  static int bw_kw(int log_n, bool base4) {
    if (base4 && log_n >= 2) return 2;
    return (log_n >= 10 && options().bw_v2 != 0 && options().bw_c64_kw2 != 0) ? 2 : 1;
  }
  static int bw_max_sg(int kw) { return kw == 2 ? 2 : 10; }
};

// Launch shape of the forward kernel.  The defaults (two CTAs per SM, windows of up to 3 bits
// for float / 2 for complex; for float radix-4 products 4-bit windows, which hold two radix-4
// stages, at one CTA per SM) can be overridden for experiments with the options fw_kmax (window
// bits) and fw_rows (rows per tile).
struct FwTuning { int kmax, ctas_per_sm, max_rows; };
template <typename T> inline FwTuning fw_tuning(bool base4) {
  FwTuning t{KernelCfg<T>::kFwKmaxTwoCtas, 2, 16};
  if (base4 && sizeof(T) == 4) t.kmax = KernelCfg<T>::kFwKmaxOneCta;
  const int k = options().fw_kmax;
  if (k >= 1 && k <= KernelCfg<T>::kFwKmaxOneCta) t.kmax = k;
  if (t.kmax > KernelCfg<T>::kFwKmaxTwoCtas) t.ctas_per_sm = 1;
  const int r = options().fw_rows;
  if (r >= 1 && r <= 64) t.max_rows = r;
  return t;
}

// The packed-pair forward kernel steps aside when it is switched off or when a switch asks for
// something only the generic forward kernel does (per-thread tile copies, forced panels or tile
// shapes).
inline bool fw2_enabled() {
  const Options& o = options();
  return o.fw2 != 0 && o.tma != 0 && o.fw_logcmax < 0 && o.fw_kmax < 0 && o.fw_rows < 0;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
template <typename T> inline bool vec_ok(const void* p, int64_t sB, int64_t sS) {
  return aligned16(p) && (sB * (int64_t)sizeof(T)) % 16 == 0 && (sS * (int64_t)sizeof(T)) % 16 == 0;
}

struct Problem {
  int B, S, log_n, nblocks, in_size, out_size;
  bool inc, base4;
};

inline void twiddle_stack_sizes(const Problem& q, int64_t out[2]);
inline int check_problem(const Problem& q) {
  if (q.B < 0 || q.S < 1 || q.log_n < 1 || q.log_n > 24 || q.nblocks < 1) return BFLY_E_ARG;
  if (q.in_size < 0 || q.out_size < 0 || q.out_size > (1 << q.log_n)) return BFLY_E_ARG;
  // The kernels address a stage's twiddles with 32-bit element offsets inside one stack (and the
  // re-ordered copy of the packed-pair forward, twice as many floats, the same way): a stack of
  // 2^31 twiddle elements or more (8 GB of float32 per stack) is refused rather than wrapped.
  int64_t per_stack[2];
  twiddle_stack_sizes(q, per_stack);
  if (per_stack[0] >= ((int64_t)1 << 31) || per_stack[1] >= ((int64_t)1 << 31)) return BFLY_E_UNSUPPORTED;
  return BFLY_OK;
}

inline std::vector<Stage> problem_stages(const Problem& q) {
  return q.base4 ? make_stages_r4(q.log_n, q.nblocks, q.inc) : make_stages_r2(q.log_n, q.nblocks, q.inc);
}
// elements per stack of the radix-2 (`which` 0) and radix-4 (`which` 1) twiddle tensors
inline void twiddle_stack_sizes(const Problem& q, int64_t out[2]) {
  const int64_t n = (int64_t)1 << q.log_n;
  if (q.base4) {
    out[0] = (int64_t)q.nblocks * (q.log_n % 2) * (n / 2) * 4;
    out[1] = (int64_t)q.nblocks * (q.log_n / 2) * (n / 4) * 16;
  } else {
    out[0] = (int64_t)q.nblocks * q.log_n * (n / 2) * 4;
    out[1] = 0;
  }
}

// Widest panel (log2 columns) of a forward pass: 16 KB rows (4096 floats, 2048 complex).  Rows up
// to that width run in one pass; wider rows would leave too few rows per tile to amortise the
// twiddle fetches (and beyond 227 KB would not fit at all), so they run as several passes over
// panels, which measures 1.3x (n = 8192) to 2.7x (n = 16384) faster than one pass with 3 or 1
// rows per tile.  The option fw_logcmax forces narrower panels (tests run the multi-pass path at small n).
template <typename T> inline int fw_pass_logc(int log_n) {
  int lc = sizeof(T) == 4 ? 12 : 11;
  if (log_n < lc) lc = log_n;
  const int v = options().fw_logcmax;
  if (v >= 3 && v < lc) lc = v;
  return lc;
}

// Stages [t0, t1) through the packed-pair forward kernel (bfly_fw2.h).  Returns kFw2Declined when
// the shape, the stage list or the tensors do not qualify.
template <typename E>
int drive_fw2(E& ex, const Problem& q, const std::vector<Stage>& st, int t0, int t1, const std::vector<int>& cuts,
              float* const* snaps, const float* tw2, const float* x, int64_t x_sB, int64_t x_sS, int x_cols, float* out,
              int64_t out_sB, int64_t out_sS, int out_cols, void* pack_ws, size_t pack_bytes, const float* bias = nullptr,
              int bias_len = 0) {
  if (q.base4 || !tw2 || !pack_ws || !fw2_enabled()) return kFw2Declined;
  std::vector<Fw2Group> groups;
  if (!plan_fw2_groups(st, t0, t1, cuts, q.log_n, groups)) return kFw2Declined;
  if ((int)cuts.size() > kFw2MaxSnap) return kFw2Declined;
  Fw2Params p;
  std::memset(&p, 0, sizeof(p));
  int64_t stk[2];
  twiddle_stack_sizes(q, stk);
  p.tw = tw2; p.tw_stack = stk[0];
  p.B = q.B; p.S = q.S; p.log_n = q.log_n;
  // rows of 8192 columns: one 512-thread CTA per SM with a 7-row tile (224 KB), the whole product in one launch
  const bool wide = q.log_n == kFw2WideLogN;
  const int ctas = (wide || options().fw2_ctas == 1) ? 1 : 2;
  p.threads = wide ? kFw2WideThreads : kFw2Threads;
  p.P = p.threads / ((1 << q.log_n) / 16);
  p.Rw = fw2_rows_per_thread(q.B, q.S, p.P, ctas * ex.num_sms(), (ctas == 1 && !wide) ? 14 : 7);
  p.R = p.P * p.Rw;
  p.packed = static_cast<float*>(pack_ws);
  p.packed_stack = (int64_t)groups.back().pk_off + (int64_t)groups.back().nst * 8 * ((1 << q.log_n) / 16);
  if ((size_t)p.packed_stack * q.S * 16 > pack_bytes) return kFw2Declined;
  p.x = x; p.x_sB = x_sB; p.x_sS = x_sS; p.x_cols = x_cols;
  p.out = out; p.out_sB = out_sB; p.out_sS = out_sS; p.out_cols = out_cols;
  p.bias = bias; p.bias_len = bias_len;
  for (int i = 0; i < kFw2MaxSnap; ++i) p.snap[i] = (snaps && i < (int)cuts.size()) ? snaps[i] : nullptr;
  p.ngroups = (int)groups.size();
  for (int g = 0; g < p.ngroups; ++g) {
    p.g[g] = groups[g];
    if (groups[g].sync == 2 || (groups[g].emit && !groups[g].local)) p.cta_syncs = 1;
  }
  if (!groups.back().local) p.cta_syncs = 1;
  return ex.run_fw2(p, ctas);
}

// Rows wider than 4096 floats on the packed-pair kernel: the stages are cut into passes whose bits
// fit a panel of 4096 columns that the kernel sees as a row of its own -- the low 12 bits
// (contiguous panels), or the top 7 bits with 32-column blocks (bits 0-4) riding along -- one
// launch per pass, in place on `work` between the first read of x and the last write.  One real
// stack, full-width input.  Returns kFw2Declined when the shape or the stage list does not fit.
struct Fw2Pass { int t0, t1; Panel panel; };
inline std::vector<Fw2Pass> plan_fw2_passes(const std::vector<Stage>& st, int t0, int t1, int log_n) {
  std::vector<Fw2Pass> out;
  const int top = log_n - 7;  // lowest bit of the strided panel
  int t = t0;
  while (t < t1) {
    if (st[t].radix != 2) return {};
    bool low = st[t].bit <= 11, high = st[t].bit >= top;
    if (!low && !high) return {};
    int e = t + 1;
    while (e < t1 && st[e].radix == 2) {
      const bool l2 = low && st[e].bit <= 11, h2 = high && st[e].bit >= top;
      if (!l2 && !h2) break;
      low = l2; high = h2;
      ++e;
    }
    Fw2Pass ps;
    ps.t0 = t; ps.t1 = e;
    ps.panel = low ? Panel{12, 12, 12, log_n - 12} : Panel{12, 5, top, log_n - 12};
    out.push_back(ps);
    t = e;
  }
  return out;
}

template <typename E>
int drive_fw2_view(E& ex, const Problem& q, const std::vector<Stage>& st, int t0, int t1, const std::vector<int>& cuts,
                   float* const* snaps, const float* tw2, const float* x, int64_t x_sB, int x_cols, float* out, int64_t out_sB,
                   float* scratch, int64_t scratch_sB, void* pack_ws, size_t pack_bytes) {
  if (q.base4 || !tw2 || !pack_ws || !fw2_enabled() || q.S != 1 || q.log_n <= kFw2MaxLogN || q.log_n > 19) return kFw2Declined;
  const int64_t n = (int64_t)1 << q.log_n;
  if (x_cols < n || (int)cuts.size() > kFw2MaxSnap) return kFw2Declined;
  const std::vector<Fw2Pass> passes = plan_fw2_passes(st, t0, t1, q.log_n);
  if (passes.empty()) return kFw2Declined;
  float* work = out; int64_t work_sB = out_sB;
  if (!work) { work = scratch; work_sB = scratch_sB; }
  if (passes.size() > 1 && !work) return kFw2Declined;
  // plan everything before the first launch: a pass that does not fit must not leave half a product behind
  std::vector<Fw2Params> launches;
  for (size_t pi = 0; pi < passes.size(); ++pi) {
    const Fw2Pass& ps = passes[pi];
    std::vector<Stage> local(st);
    for (int k = ps.t0; k < ps.t1; ++k) {
      const int b = st[k].bit;
      local[k].bit = b < ps.panel.lseg ? b : b - ps.panel.pb + ps.panel.lseg;
      if (local[k].bit < 0 || local[k].bit > 11) return kFw2Declined;
    }
    std::vector<Fw2Group> groups;
    if (!plan_fw2_groups(local, ps.t0, ps.t1, cuts, 12, groups)) return kFw2Declined;
    Fw2Params p;
    std::memset(&p, 0, sizeof(p));
    int64_t stk[2];
    twiddle_stack_sizes(q, stk);
    p.tw = tw2; p.tw_stack = stk[0];
    p.view = 1; p.view_row = (int)n; p.panel = ps.panel;
    p.B = q.B; p.S = 1 << ps.panel.npanels_log; p.log_n = 12;
    const int ctas = options().fw2_ctas == 1 ? 1 : 2;
    p.P = 1;
    p.Rw = fw2_rows_per_thread(q.B, p.S, p.P, ctas * ex.num_sms(), ctas == 1 ? 14 : 7);
    p.R = p.P * p.Rw;
    p.packed = static_cast<float*>(pack_ws);
    p.packed_stack = (int64_t)groups.back().pk_off + (int64_t)groups.back().nst * 8 * (4096 / 16);
    if ((size_t)p.packed_stack * p.S * 16 > pack_bytes) return kFw2Declined;
    const bool first = pi == 0, last = pi + 1 == passes.size();
    p.x = first ? x : work; p.x_sB = first ? x_sB : work_sB; p.x_sS = 0; p.x_cols = 4096;
    p.out = last ? out : work; p.out_sB = last ? out_sB : work_sB; p.out_sS = 0; p.out_cols = 4096;
    for (int i = 0; i < kFw2MaxSnap; ++i) p.snap[i] = (snaps && i < (int)cuts.size()) ? snaps[i] : nullptr;
    p.ngroups = (int)groups.size();
    for (int g = 0; g < p.ngroups; ++g) {
      p.g[g] = groups[g];
      if (groups[g].sync == 2 || (groups[g].emit && !groups[g].local)) p.cta_syncs = 1;
    }
    if (!groups.back().local) p.cta_syncs = 1;
    launches.push_back(p);
  }
  const int ctas = options().fw2_ctas == 1 ? 1 : 2;
  for (size_t pi = 0; pi < launches.size(); ++pi) {
    const int rc = ex.run_fw2(launches[pi], ctas);
    if (rc == kFw2Declined) return pi == 0 ? kFw2Declined : BFLY_E_UNSUPPORTED;
    if (rc != BFLY_OK) return rc;
  }
  return BFLY_OK;
}

// Run stages [t0, t1) of the product with the row-owner forward kernel.  `cuts` lists the
// stage indices after which a snapshot is written (slot i -> snaps[i]); `out` may be null when
// only snapshots are wanted.  Rows that fit one SM's shared memory run in one pass; wider rows
// in several passes over panels, in place on `out` (or on `scratch`, a (B, S, n) buffer with
// the given strides, when `out` is null).
template <typename T, typename E>
int drive_fw_range(E& ex, const Problem& q, const std::vector<Stage>& st, int t0, int t1,
                   const std::vector<int>& cuts, T* const* snaps, const T* tw2, const T* tw4, const T* x,
                   int64_t x_sB, int64_t x_sS, int x_cols, T* out, int64_t out_sB, int64_t out_sS,
                   int out_cols, T* scratch = nullptr, int64_t scratch_sB = 0, int64_t scratch_sS = 0,
                   void* pack_ws = nullptr, size_t pack_bytes = 0, const FwGlue<T>* glue = nullptr) {
  if (q.B == 0 || t1 <= t0) return BFLY_OK;
  if (glue) {
    // glue operators work on tiles that hold whole rows, one gather slot per thread and column group
    if (fw_pass_logc<T>(q.log_n) < q.log_n || ((1 << q.log_n) > kGlueSlots * ex.threads())) return BFLY_E_UNSUPPORTED;
    if (sizeof(T) == 4 && (glue->x_real || glue->out_real)) return BFLY_E_ARG;
  }
  if constexpr (sizeof(T) == 4) {
   if (!glue) {
    // float rows of 512 .. 4096 columns: the packed-pair kernel, when the tensors qualify
    const int rc2 = drive_fw2(ex, q, st, t0, t1, cuts, snaps, tw2, x, x_sB, x_sS, x_cols, out, out_sB, out_sS, out_cols,
                              pack_ws, pack_bytes);
    if (rc2 != kFw2Declined) return rc2;
    // rows wider than the kernel's tile: its panel view, pass by pass
    const int rc3 = drive_fw2_view(ex, q, st, t0, t1, cuts, snaps, tw2, x, x_sB, x_cols, out, out_sB, scratch, scratch_sB,
                                   pack_ws, pack_bytes);
    if (rc3 != kFw2Declined) return rc3;
   }
  }
  const int lc = fw_pass_logc<T>(q.log_n);
  if (((int64_t)sizeof(T) << lc) > kSmemMax) return BFLY_E_UNSUPPORTED;
  std::vector<FwPass> passes;
  if (lc >= q.log_n) passes.push_back(FwPass{t0, t1, full_row_panel(q.log_n)});
  else passes = plan_fw_passes(st, t0, t1, q.log_n, lc);
  if (passes.empty()) return BFLY_E_UNSUPPORTED;
  const FwTuning tune = fw_tuning<T>(q.base4);
  int64_t stk[2];
  twiddle_stack_sizes(q, stk);
  const int64_t n = (int64_t)1 << q.log_n;
  // the buffer the passes work on between the first read of x and the last write
  T* work = out; int64_t work_sB = out_sB, work_sS = out_sS;
  if (!work) { work = scratch; work_sB = scratch_sB; work_sS = scratch_sS; }
  bool first = true;
  for (size_t pi = 0; pi < passes.size(); ++pi) {
    const FwPass& ps = passes[pi];
    const Panel pn = ps.panel;
    std::vector<FwGroup> groups;
    if (!plan_fw_groups(st, ps.t0, ps.t1, cuts, pn, Vec16<T>::LOG, tune.kmax, groups))
      return BFLY_E_UNSUPPORTED;
    size_t g0 = 0;
    while (g0 < groups.size()) {
      const size_t g1 = std::min(groups.size(), g0 + (size_t)kMaxFwGroups);
      const bool last = (g1 == groups.size()) && (pi + 1 == passes.size());
      FwParams<T> p;
      std::memset(&p, 0, sizeof(p));
      p.tw[0] = tw2; p.tw[1] = tw4; p.tw_stack[0] = stk[0]; p.tw_stack[1] = stk[1];
      if (first) {
        p.x = x; p.x_sB = x_sB; p.x_sS = x_sS; p.x_cols = x_cols;
        if (glue) { p.glue.in_perm = glue->in_perm; p.glue.x_real = glue->x_real; }
        if (glue) glue_column_bits(pn.logC, p.glue.colbit);
      } else {  // continue in place from the full-width rows written by the previous launch
        if (!work) return BFLY_E_UNSUPPORTED;
        p.x = work; p.x_sB = work_sB; p.x_sS = work_sS; p.x_cols = (int)n;
      }
      if (last) {
        p.out = out; p.out_sB = out_sB; p.out_sS = out_sS; p.out_cols = out_cols;
        if (glue) { p.glue.out_perm = glue->out_perm; p.glue.out_diag = glue->out_diag; p.glue.out_real = glue->out_real; }
        if (glue) glue_column_bits(pn.logC, p.glue.colbit);
      } else {
        if (!work) return BFLY_E_UNSUPPORTED;
        p.out = work; p.out_sB = work_sB; p.out_sS = work_sS; p.out_cols = (int)n;
      }
      for (int i = 0; i < kMaxSnap; ++i) p.snap[i] = (snaps && i < (int)cuts.size()) ? snaps[i] : nullptr;
      p.B = q.B; p.S = q.S; p.log_n = q.log_n;
      p.R = fw_rows_per_tile<T>(pn.logC, q.B, tune.ctas_per_sm, tune.max_rows);
      p.vec_in = p.x ? vec_ok<T>(p.x, p.x_sB, p.x_sS) : 0;
      p.vec_out = p.out ? vec_ok<T>(p.out, p.out_sB, p.out_sS) : 1;
      p.panel = pn;
      p.ngroups = (int)(g1 - g0);
      p.tab_slots = 1;
      for (size_t g = g0; g < g1; ++g) {
        p.g[g - g0] = groups[g];
        const int U = (1 << pn.logC) >> groups[g].K;
        p.tab_slots = std::max(p.tab_slots, U / ex.threads());
      }
      // the unit table follows the tile in shared memory when it is small; give it room
      {
        const size_t budget = tune.ctas_per_sm <= 1 ? (size_t)kSmemMax : (size_t)(228 * 1024) / tune.ctas_per_sm - 1024 - 2048;
        const size_t tab = (size_t)p.ngroups * p.tab_slots * ex.threads() * sizeof(uint16_t);
        const size_t row_bytes = sizeof(T) << pn.logC;
        p.use_table = tab <= 16 * 1024 && row_bytes + tab <= budget;
        if (p.use_table)
          while (p.R > 1 && (size_t)p.R * row_bytes + tab > budget) --p.R;
      }
      const int rc = ex.run_fw(p);
      if (rc != BFLY_OK) return rc;
      g0 = g1;
      first = false;
    }
  }
  return BFLY_OK;
}

template <typename T, typename E>
int drive_fw(E& ex, const Problem& q, const T* tw2, const T* tw4, const T* x, int64_t x_sB, int64_t x_sS,
             T* out, void* ws = nullptr, size_t ws_bytes = 0) {
  int rc = check_problem(q);
  if (rc != BFLY_OK) return rc;
  if (q.B == 0) return BFLY_OK;
  if (!x || !out || (!tw2 && !tw4)) return BFLY_E_ARG;
  if ((tw2 && !aligned16(tw2)) || (tw4 && !aligned16(tw4))) return BFLY_E_ALIGN;
  const std::vector<Stage> st = problem_stages(q);
  const int64_t n = (int64_t)1 << q.log_n;
  if (ws && !aligned16(ws)) ws = nullptr;  // optional scratch: without it the generic kernel runs
  return drive_fw_range<T>(ex, q, st, 0, (int)st.size(), {}, nullptr, tw2, tw4, x, x_sB, x_sS, q.in_size,
                           out, (int64_t)q.S * n, n, q.out_size, (T*)nullptr, 0, 0, ws, ws ? ws_bytes : 0);
}

// The forward with glue operators folded into its launch (FwGlue).  x / out are null when
// glue.x_real / glue.out_real carry the rows; strides count elements of whichever is used.  A
// product of more than kMaxFwGroups stage groups runs as several launches: the intermediate rows
// then need `out` (complex), so a real output of such a product is not supported.
template <typename T, typename E>
int drive_fw_glue(E& ex, const Problem& q, const T* tw2, const T* x, int64_t x_sB, int64_t x_sS, T* out,
                  const FwGlue<T>& glue) {
  int rc = check_problem(q);
  if (rc != BFLY_OK) return rc;
  if (q.base4) return BFLY_E_UNSUPPORTED;
  if (q.B == 0) return BFLY_OK;
  if ((!x && !glue.x_real) || (!out && !glue.out_real) || !tw2) return BFLY_E_ARG;
  if ((x && glue.x_real) || (out && glue.out_real)) return BFLY_E_ARG;
  if (!aligned16(tw2)) return BFLY_E_ALIGN;
  if (glue.in_perm && q.in_size != (1 << q.log_n)) return BFLY_E_ARG;  // the gather addresses whole rows
  if ((glue.out_perm || glue.out_diag) && q.out_size != (1 << q.log_n)) return BFLY_E_ARG;
  const std::vector<Stage> st = problem_stages(q);
  const int64_t n = (int64_t)1 << q.log_n;
  return drive_fw_range<T>(ex, q, st, 0, (int)st.size(), {}, nullptr, tw2, (const T*)nullptr, x, x_sB, x_sS, q.in_size,
                           out, (int64_t)q.S * n, n, q.out_size, (T*)nullptr, 0, 0, nullptr, 0, &glue);
}

// Scratch the forward can use (0 = none needed): room for the re-ordered twiddles of the
// packed-pair kernel.  The forward also runs without it, on the generic kernel.
template <typename T> inline size_t fw_workspace_bytes(const Problem& q) {
  if (sizeof(T) != 4 || q.base4) return 0;
  return fw2_packed_bytes(q.S, q.log_n, q.nblocks);
}

template <typename T> struct BwLayout;
template <typename T> int plan_bw(const Problem& q, BwLayout<T>& lay);

template <typename T> struct BwLayout {
  std::vector<BwPhase> phases;
  int kw;
  size_t ws_bytes;    // snapshot planes, then the forward's scratch (fw_workspace_bytes)
  size_t pack_off, pack_bytes;
  // more phases than one forward launch can write snapshots for: the backward then runs in
  // chunks of kMaxSnap phases, each with its own forward pass from the input
  bool chunked;
};

template <typename T>
int plan_bw(const Problem& q, BwLayout<T>& lay) {
  const std::vector<Stage> st = problem_stages(q);
  lay.kw = KernelCfg<T>::bw_kw(q.log_n, q.base4);
  int logCmax = 0;
  while ((1 << logCmax) < (KernelCfg<T>::kThreads << lay.kw)) ++logCmax;
  lay.phases = plan_bw_phases(st, q.log_n, logCmax, lay.kw, KernelCfg<T>::bw_max_sg(lay.kw), Vec16<T>::LOG);
  if (lay.phases.empty()) return BFLY_E_UNSUPPORTED;
  lay.chunked = (int)lay.phases.size() - 1 > kMaxSnap;
  const size_t plane = (size_t)q.B * q.S * sizeof(T) << q.log_n;
  // chunked: kMaxSnap snapshots plus one plane the forward passes of the later chunks work on
  const size_t planes = lay.chunked ? (size_t)kMaxSnap + 1 : lay.phases.size() - 1;
  lay.pack_off = planes * ((plane + 255) / 256 * 256);
  // the forward pass over the earlier phases may use the packed-pair kernel: room for its twiddles
  lay.pack_bytes = planes > 0 ? (fw_workspace_bytes<T>(q) + 255) / 256 * 256 : 0;
  lay.ws_bytes = lay.pack_off + lay.pack_bytes;
  return BFLY_OK;
}

// Forward that also writes, into ws, the phase-boundary activations the backward of the same
// problem starts from (the layout drive_bw expects when it is told the snapshots are ready).
template <typename T, typename E>
int drive_fw_saving(E& ex, const Problem& q, const T* tw2, const T* tw4, const T* x, int64_t x_sB, int64_t x_sS,
                    T* out, void* ws, size_t ws_bytes) {
  int rc = check_problem(q);
  if (rc != BFLY_OK) return rc;
  if (q.B == 0) return BFLY_OK;
  if (!x || !out || (!tw2 && !tw4)) return BFLY_E_ARG;
  if ((tw2 && !aligned16(tw2)) || (tw4 && !aligned16(tw4))) return BFLY_E_ALIGN;
  BwLayout<T> lay;
  rc = plan_bw<T>(q, lay);
  if (rc != BFLY_OK) return rc;
  if (lay.ws_bytes > 0 && (!ws || ws_bytes < lay.ws_bytes || !aligned16(ws))) return BFLY_E_WORKSPACE;
  const std::vector<Stage> st = problem_stages(q);
  const int64_t n = (int64_t)1 << q.log_n;
  const int nph = (int)lay.phases.size();
  const size_t plane = ((size_t)q.B * q.S * sizeof(T) << q.log_n);
  const size_t plane_pad = (plane + 255) / 256 * 256;
  T* snaps[kMaxSnap] = {nullptr};
  std::vector<int> cuts;
  if (!lay.chunked) {  // a chunked backward recomputes its snapshots chunk by chunk: nothing to save
    for (int ph = 1; ph < nph; ++ph) {
      snaps[ph - 1] = reinterpret_cast<T*>(static_cast<char*>(ws) + (size_t)(ph - 1) * plane_pad);
      cuts.push_back(lay.phases[ph].t0);
    }
  }
  void* pack_ws = lay.pack_bytes ? static_cast<char*>(ws) + lay.pack_off : nullptr;
  return drive_fw_range<T>(ex, q, st, 0, (int)st.size(), cuts, snaps, tw2, tw4, x, x_sB, x_sS, q.in_size, out,
                           (int64_t)q.S * n, n, q.out_size, (T*)nullptr, 0, 0, pack_ws, lay.pack_bytes);
}

// Backward of the whole product.  d_x is (B, S, max(in_size, n)) contiguous and doubles as
// the gradient buffer between phases; d_tw2 / d_tw4 are overwritten.
template <typename T, typename E>
int drive_bw(E& ex, const Problem& q, const T* tw2, const T* tw4, const T* x, int64_t x_sB, int64_t x_sS,
             const T* grad, int64_t g_sB, int64_t g_sS, T* d_tw2, T* d_tw4, T* d_x, void* ws,
             size_t ws_bytes, bool snapshots_ready = false) {
  int rc = check_problem(q);
  if (rc != BFLY_OK) return rc;
  int64_t stk[2];
  twiddle_stack_sizes(q, stk);
  if ((stk[0] && (!tw2 || !d_tw2)) || (stk[1] && (!tw4 || !d_tw4))) return BFLY_E_ARG;
  if ((tw2 && !aligned16(tw2)) || (tw4 && !aligned16(tw4))) return BFLY_E_ALIGN;
  if ((d_tw2 && !aligned16(d_tw2)) || (d_tw4 && !aligned16(d_tw4))) return BFLY_E_ALIGN;  // 16-byte vector reductions
  if (stk[0]) { rc = ex.zero(d_tw2, (size_t)q.S * stk[0] * sizeof(T)); if (rc) return rc; }
  if (stk[1]) { rc = ex.zero(d_tw4, (size_t)q.S * stk[1] * sizeof(T)); if (rc) return rc; }
  if (q.B == 0) return BFLY_OK;
  if (!x || !grad || !d_x) return BFLY_E_ARG;
  BwLayout<T> lay;
  rc = plan_bw<T>(q, lay);
  if (rc != BFLY_OK) return rc;
  if (lay.ws_bytes > 0 && (!ws || ws_bytes < lay.ws_bytes || !aligned16(ws))) return BFLY_E_WORKSPACE;
  const std::vector<Stage> st = problem_stages(q);
  const int64_t n = (int64_t)1 << q.log_n;
  const int nph = (int)lay.phases.size();
  const size_t plane = ((size_t)q.B * q.S * sizeof(T) << q.log_n);
  const size_t plane_pad = (plane + 255) / 256 * 256;
  const int64_t DX = std::max<int64_t>(q.in_size, n);
  if (lay.chunked) snapshots_ready = false;
  // Phases run last to first.  Normally one forward launch writes every phase-boundary activation
  // and all phases follow; a product with more phases than snapshot slots runs in chunks of
  // kMaxSnap phases, each preceded by its own forward pass from the input.
  for (int pb = nph; pb > 0;) {
  const int pa = lay.chunked ? std::max(0, pb - kMaxSnap) : 0;
  const int first = std::max(pa, 1);  // phase 0 enters with x itself
  T* snaps[kMaxSnap] = {nullptr};
  std::vector<int> cuts;
  for (int ph = first; ph < pb; ++ph) {
    snaps[ph - first] = reinterpret_cast<T*>(static_cast<char*>(ws) + (size_t)(ph - first) * plane_pad);
    cuts.push_back(lay.phases[ph].t0);
  }
  if (!cuts.empty() && !snapshots_ready) {
    // the forward pass of a product with wide rows (several launches over panels) works in place
    // on d_x while no phase has written it yet, afterwards on the spare plane of the workspace
    T* scratch = d_x;
    int64_t scr_sB = (int64_t)q.S * DX, scr_sS = DX;
    if (pb != nph) {
      scratch = reinterpret_cast<T*>(static_cast<char*>(ws) + (size_t)kMaxSnap * plane_pad);
      scr_sB = (int64_t)q.S * n; scr_sS = n;
    }
    void* pack_ws = lay.pack_bytes ? static_cast<char*>(ws) + lay.pack_off : nullptr;
    rc = drive_fw_range<T>(ex, q, st, 0, lay.phases[pb - 1].t0, cuts, snaps, tw2, tw4, x, x_sB, x_sS, q.in_size,
                           (T*)nullptr, 0, 0, 0, scratch, scr_sB, scr_sS, pack_ws, lay.pack_bytes);
    if (rc != BFLY_OK) return rc;
  }
  for (int ph = pb - 1; ph >= pa; --ph) {
    const BwPhase& P = lay.phases[ph];
    BwParams<T> p;
    std::memset(&p, 0, sizeof(p));
    p.tw[0] = tw2; p.tw[1] = tw4; p.dtw[0] = d_tw2; p.dtw[1] = d_tw4;
    p.tw_stack[0] = stk[0]; p.tw_stack[1] = stk[1];
    if (ph == 0) { p.xin = x; p.xin_sB = x_sB; p.xin_sS = x_sS; p.xin_cols = q.in_size; }
    else { p.xin = snaps[ph - first]; p.xin_sB = (int64_t)q.S * n; p.xin_sS = n; p.xin_cols = (int)n; }
    if (ph == nph - 1) { p.gin = grad; p.gin_sB = g_sB; p.gin_sS = g_sS; p.gin_cols = q.out_size; }
    else { p.gin = d_x; p.gin_sB = (int64_t)q.S * DX; p.gin_sS = DX; p.gin_cols = (int)n; }
    p.gout = d_x; p.gout_sB = (int64_t)q.S * DX; p.gout_sS = DX;
    p.gout_cols = (ph == 0) ? (int)std::min<int64_t>(q.in_size, n) : (int)n;
    p.B = q.B; p.S = q.S; p.log_n = q.log_n;
    p.panel = P.panel;
    p.nsg = P.nsg;
    for (int j = 0; j < P.nsg; ++j) {
      p.sg[j] = P.sg[j];
      bw2_assign_kase(p.sg[j], lay.kw);
    }
    if constexpr (sizeof(T) == 4) {
      // float radix-2 phases on full 1024-column panels: the packed-pair kernel, when the tensors qualify
      const Options& o = options();
      if (o.bw3 != 0 && o.tma != 0 && o.bw_rows < 0 && o.bw_v2 != 0 && lay.kw == 2 && q.B >= kBw3Rows) {
        Bw3Params p3;
        std::memset(&p3, 0, sizeof(p3));
        p3.b = p;
        if (bw3_plan(p3.b, p3.sg)) {
          BwParams<float>& b = p3.b;
          b.Rb = kBw3Rows;
          b.xin_cols = (int)std::min<int64_t>(b.xin_cols, n);  // input columns beyond n are never read
          const int groups3 = (1 << P.panel.npanels_log) * q.S;
          int nsl = std::max(1, 2 * ex.num_sms() / groups3);
          int rows3 = (q.B + nsl - 1) / nsl;
          rows3 = (rows3 + kBw3Rows - 1) / kBw3Rows * kBw3Rows;
          b.rows_per_cta = rows3;
          b.nslices = (q.B + rows3 - 1) / rows3;
          b.vec_x = vec_ok<T>(b.xin, b.xin_sB, b.xin_sS);
          b.vec_g = vec_ok<T>(b.gin, b.gin_sB, b.gin_sS);
          b.vec_o = vec_ok<T>(b.gout, b.gout_sB, b.gout_sS);
          // Its per-CTA set-up (pairing the twiddles into tensor memory) is amortised over the CTA's
          // rows: with few rows per CTA the scalar tensor-memory kernel is faster (measured: the
          // packed-pair kernel 4-5 % faster at 222 rows per CTA, equal at 111, 6-13 % slower at 56 and 28).
          const int rc3 = rows3 >= o.bw3_min_rows ? ex.run_bw3(p3) : kFw2Declined;
          if (rc3 == BFLY_OK) continue;
          if (rc3 != kFw2Declined) return rc3;
        }
      }
    }
    const size_t row_bytes = (size_t)(P.nsg + 1) * sizeof(T) << P.panel.logC;
    const int U = (1 << P.panel.logC) >> lay.kw;
    // second-generation kernel: full panels (one unit per thread), four-row batches, two CTAs per SM
    const size_t v2_bytes = 4 * row_bytes + (size_t)P.nsg * 6 * KernelCfg<T>::kThreads * sizeof(uint32_t) + 32 + 1024;
    p.v2 = ex.has_bw2(sizeof(T), lay.kw) && P.nsg <= 4 && U == KernelCfg<T>::kThreads && v2_bytes <= (size_t)(228 * 1024) / 2 - 1024 &&
           q.B >= 4;
    int Rb = (int)(kSmemMax / row_bytes);
    {
      const int v = options().bw_rows;  // experiments: rows per batch
      if (v >= 1 && v < Rb) Rb = v;
    }
    if (Rb > 16) Rb = 16;
    if (Rb < 1) return BFLY_E_UNSUPPORTED;
    if (Rb >= 4) Rb &= ~3;       // batch heights in multiples of four: the kernels keep four rows in flight
    else if (Rb > 2) Rb &= ~1;
    // rows that run in parallel inside a CTA when the panel has fewer units than threads
    const int par = U >= KernelCfg<T>::kThreads ? 1 : KernelCfg<T>::kThreads / std::max(U, 1);
    if (Rb < par && (size_t)par * row_bytes <= (size_t)kSmemMax) Rb = par;
    if (Rb > q.B && q.B < 8) Rb = std::max(q.B, 1);  // tiny batches; otherwise rows past the batch are zero rows
    if (p.v2) Rb = 4;
    p.Rb = Rb;
    const int groups = (1 << P.panel.npanels_log) * q.S;
    int nslices = std::max(1, (p.v2 ? 2 : 1) * ex.num_sms() / groups);
    int rows = (q.B + nslices - 1) / nslices;
    rows = (rows + Rb - 1) / Rb * Rb;
    nslices = (q.B + rows - 1) / rows;
    p.rows_per_cta = rows;
    p.nslices = nslices;
    p.vec_x = vec_ok<T>(p.xin, p.xin_sB, p.xin_sS);
    p.vec_g = vec_ok<T>(p.gin, p.gin_sB, p.gin_sS);
    p.vec_o = vec_ok<T>(p.gout, p.gout_sB, p.gout_sS);
    rc = ex.run_bw(p, lay.kw);
    if (rc != BFLY_OK) return rc;
  }
  pb = pa;
  }
  if (q.in_size > n) {
    rc = ex.zero2d(d_x + n, (size_t)DX * sizeof(T), (size_t)(q.in_size - n) * sizeof(T), (size_t)q.B * q.S);
    if (rc != BFLY_OK) return rc;
  }
  return BFLY_OK;
}

// ------------------------------------------------------------------ fused linear layer (float32)
//
// Butterfly as a linear layer (torch_butterfly/butterfly.py:152-169 of the reference): every stack
// multiplies the same input row (B, in); the outputs of the stacks side by side form (B, S * n), of
// which the first out_total columns are the layer's output, plus a bias.  Fused here:
//   forward   the bias is added in the forward kernel's store epilogue (no extra pass over the output);
//   backward  the input gradient is summed over the stacks by the last phase's store (a float32
//             reduce-add of its tiles into (B, in)), and the bias gradient (column sums of grad)
//             is accumulated by the first phase while it holds the gradient tiles.
// The backward runs only when every phase qualifies for the packed-pair kernel; otherwise it returns
// BFLY_E_UNSUPPORTED before touching any output, and the caller composes the unfused operators.

template <typename E>
int drive_linear_fw(E& ex, const Problem& q, const float* tw, const float* x, int64_t x_sB, float* out, const float* bias,
                    int out_total, void* ws, size_t ws_bytes) {
  int rc = check_problem(q);
  if (rc != BFLY_OK) return rc;
  if (q.base4 || out_total < 0 || out_total > ((int64_t)q.S << q.log_n)) return BFLY_E_ARG;
  if (q.B == 0) return BFLY_OK;
  if (!x || !out || !tw) return BFLY_E_ARG;
  if (!aligned16(tw)) return BFLY_E_ALIGN;
  const std::vector<Stage> st = problem_stages(q);
  const int64_t n = (int64_t)1 << q.log_n;
  if (ws && !aligned16(ws)) ws = nullptr;
  // the packed-pair kernel adds the bias itself; any other route adds it afterwards
  bool fused_bias = false;
  if (bias) {
    const int rc2 = drive_fw2(ex, q, st, 0, (int)st.size(), {}, (float* const*)nullptr, tw, x, x_sB, 0, q.in_size, out,
                              (int64_t)q.S * n, n, (int)n, ws, ws ? ws_bytes : 0, bias, out_total);
    if (rc2 == BFLY_OK) return BFLY_OK;
    if (rc2 != kFw2Declined) return rc2;
  }
  rc = drive_fw_range<float>(ex, q, st, 0, (int)st.size(), {}, nullptr, tw, (const float*)nullptr, x, x_sB, 0, q.in_size, out,
                             (int64_t)q.S * n, n, (int)n, (float*)nullptr, 0, 0, ws, ws ? ws_bytes : 0);
  if (rc != BFLY_OK || !bias || fused_bias) return rc;
  return ex.add_bias(out, bias, q.B, out_total, (int64_t)q.S * n);
}

struct LinearBwLayout {
  BwLayout<float> lay;
  size_t gbuf_off, ws_bytes;  // the gradient plane between phases follows the backward's own scratch
};
inline int plan_linear_bw(const Problem& q, LinearBwLayout& L) {
  const int rc = plan_bw<float>(q, L.lay);
  if (rc != BFLY_OK) return rc;
  const size_t plane = ((size_t)q.B * q.S * sizeof(float) << q.log_n);
  L.gbuf_off = L.lay.ws_bytes;
  L.ws_bytes = L.lay.ws_bytes + (plane + 255) / 256 * 256;
  return BFLY_OK;
}

template <typename E>
int drive_linear_bw(E& ex, const Problem& q, const float* tw, const float* x, int64_t x_sB, const float* grad, int64_t g_sB,
                    float* d_tw, float* d_in, int64_t din_sB, float* d_bias, int out_total, void* ws, size_t ws_bytes) {
  int rc = check_problem(q);
  if (rc != BFLY_OK) return rc;
  const int64_t n = (int64_t)1 << q.log_n;
  const Options& o = options();
  // the fused route: all stacks full, every tensor describable to the TMA unit, every phase on the
  // packed-pair kernel
  if (q.base4 || out_total != q.S * n || q.in_size > n || q.in_size % 32 != 0 || q.B < kBw3Rows) return BFLY_E_UNSUPPORTED;
  if (o.bw3 == 0 || o.tma == 0 || o.bw_rows >= 0 || o.bw_v2 == 0 || !fw2_enabled()) return BFLY_E_UNSUPPORTED;
  if (!tw || !d_tw || !x || !grad || !d_in || !ws) return BFLY_E_ARG;
  if (!aligned16(tw) || !aligned16(d_tw)) return BFLY_E_ALIGN;
  if (!vec_ok<float>(x, x_sB, 0) || !vec_ok<float>(grad, g_sB, n) || !vec_ok<float>(d_in, din_sB, 0) || !aligned16(ws))
    return BFLY_E_UNSUPPORTED;
  LinearBwLayout L;
  rc = plan_linear_bw(q, L);
  if (rc != BFLY_OK) return rc;
  if (ws_bytes < L.ws_bytes) return BFLY_E_WORKSPACE;
  const BwLayout<float>& lay = L.lay;
  const int nph = (int)lay.phases.size();
  if (lay.chunked || lay.kw != 2) return BFLY_E_UNSUPPORTED;
  int64_t stk[2];
  twiddle_stack_sizes(q, stk);
  const std::vector<Stage> st = problem_stages(q);
  std::vector<Bw3Params> launches((size_t)nph);
  const size_t plane = ((size_t)q.B * q.S * sizeof(float) << q.log_n);
  const size_t plane_pad = (plane + 255) / 256 * 256;
  float* gbuf = reinterpret_cast<float*>(static_cast<char*>(ws) + L.gbuf_off);
  float* snaps[kMaxSnap] = {nullptr};
  std::vector<int> cuts;
  for (int ph = 1; ph < nph; ++ph) {
    snaps[ph - 1] = reinterpret_cast<float*>(static_cast<char*>(ws) + (size_t)(ph - 1) * plane_pad);
    cuts.push_back(lay.phases[ph].t0);
  }
  for (int ph = 0; ph < nph; ++ph) {
    const BwPhase& P = lay.phases[ph];
    Bw3Params& p3 = launches[ph];
    std::memset(&p3, 0, sizeof(p3));
    BwParams<float>& b = p3.b;
    b.tw[0] = tw; b.dtw[0] = d_tw; b.tw_stack[0] = stk[0];
    if (ph == 0) { b.xin = x; b.xin_sB = x_sB; b.xin_sS = 0; b.xin_cols = q.in_size; }
    else { b.xin = snaps[ph - 1]; b.xin_sB = (int64_t)q.S * n; b.xin_sS = n; b.xin_cols = (int)n; }
    if (ph == nph - 1) { b.gin = grad; b.gin_sB = g_sB; b.gin_sS = n; b.gin_cols = (int)n; }
    else { b.gin = gbuf; b.gin_sB = (int64_t)q.S * n; b.gin_sS = n; b.gin_cols = (int)n; }
    if (ph == 0) { b.gout = d_in; b.gout_sB = din_sB; b.gout_sS = 0; b.gout_cols = q.in_size; b.gout_reduce = 1; }
    else { b.gout = gbuf; b.gout_sB = (int64_t)q.S * n; b.gout_sS = n; b.gout_cols = (int)n; }
    if (ph == nph - 1 && d_bias) { b.dbias = d_bias; b.dbias_len = out_total; }
    b.B = q.B; b.S = q.S; b.log_n = q.log_n;
    b.panel = P.panel;
    b.nsg = P.nsg;
    for (int j = 0; j < P.nsg; ++j) b.sg[j] = P.sg[j];
    if (!bw3_plan(b, p3.sg)) return BFLY_E_UNSUPPORTED;
    b.Rb = kBw3Rows;
    const int groups3 = (1 << P.panel.npanels_log) * q.S;
    const int nsl = std::max(1, 2 * ex.num_sms() / groups3);
    int rows3 = (q.B + nsl - 1) / nsl;
    rows3 = (rows3 + kBw3Rows - 1) / kBw3Rows * kBw3Rows;
    b.rows_per_cta = rows3;
    b.nslices = (q.B + rows3 - 1) / rows3;
    b.vec_x = b.vec_g = b.vec_o = 1;
    if (!ex.can_run_bw3(p3)) return BFLY_E_UNSUPPORTED;  // a tensor of this phase cannot be described to the TMA unit
  }
  // nothing has been written so far; from here on every step must succeed
  rc = ex.zero(d_tw, (size_t)q.S * stk[0] * sizeof(float));
  if (rc) return rc;
  rc = ex.zero2d(d_in, (size_t)din_sB * sizeof(float), (size_t)q.in_size * sizeof(float), (size_t)q.B);
  if (rc) return rc;
  if (d_bias) { rc = ex.zero(d_bias, (size_t)out_total * sizeof(float)); if (rc) return rc; }
  if (!cuts.empty()) {
    void* pack_ws = lay.pack_bytes ? static_cast<char*>(ws) + lay.pack_off : nullptr;
    rc = drive_fw_range<float>(ex, q, st, 0, lay.phases[nph - 1].t0, cuts, snaps, tw, (const float*)nullptr, x, x_sB, 0,
                               q.in_size, (float*)nullptr, 0, 0, 0, gbuf, (int64_t)q.S * n, n, pack_ws, lay.pack_bytes);
    if (rc != BFLY_OK) return rc;
  }
  for (int ph = nph - 1; ph >= 0; --ph) {
    rc = ex.run_bw3(launches[ph]);
    if (rc != BFLY_OK) return rc == kFw2Declined ? BFLY_E_UNSUPPORTED : rc;
  }
  return BFLY_OK;
}

}  // namespace bfly
