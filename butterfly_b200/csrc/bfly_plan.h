// Host-side planning for the butterfly multiply kernels: turns (log_n, nblocks,
// increasing_stride) into the ordered list of sparse factors ("stages"), cuts that list
// into register-window groups for the forward kernel and into twiddle-stationary phases
// for the backward kernel, and fills the kernel parameter blocks.  Pure host C++ (no CUDA
// types) so the same code drives the GPU launches and the test-suite's host emulator.
#pragma once
#include <algorithm>
#include <cstring>
#include <vector>

#include "bfly_types.h"

namespace bfly {

struct Stage {
  int radix;        // 2 or 4
  int bit;          // lowest bit the factor acts on (radix 4 covers bit, bit+1)
  int which;        // twiddle tensor: 0 = (S,nblocks,log_n,n/2,2,2) or twiddle2, 1 = twiddle4
  uint32_t tw_off;  // element offset of this factor's twiddles inside one stack
};

// Factor order of the radix-2 product: block b runs strides 1,2,..,n/2 when
// (increasing_stride XOR b odd), else n/2,..,1  (csrc/cpu/butterfly_cpu.cpp:33-37).
inline std::vector<Stage> make_stages_r2(int log_n, int nblocks, bool inc) {
  std::vector<Stage> st;
  const uint32_t per = (uint32_t)((1u << log_n) / 2) * 4;
  for (int b = 0; b < nblocks; ++b) {
    const bool cur = inc != (b % 2 != 0);
    for (int idx = 0; idx < log_n; ++idx)
      st.push_back(Stage{2, cur ? idx : log_n - 1 - idx, 0, (uint32_t)(b * log_n + idx) * per});
  }
  return st;
}

// Factor order of the base-4 product: per block log_n/2 radix-4 factors on bit pairs
// (0,1),(2,3),.. (increasing) or from the top down (decreasing), then one radix-2 factor
// on the top bit (increasing) or bit 0 (decreasing) when log_n is odd
// (torch_butterfly/multiply_base4.py:23-40).
inline std::vector<Stage> make_stages_r4(int log_n, int nblocks, bool inc) {
  std::vector<Stage> st;
  const int h = log_n / 2, odd = log_n % 2;
  const uint32_t n = 1u << log_n;
  for (int b = 0; b < nblocks; ++b) {
    const bool cur = inc != (b % 2 != 0);
    for (int idx = 0; idx < h; ++idx)
      st.push_back(Stage{4, cur ? 2 * idx : log_n - 2 - 2 * idx, 1, (uint32_t)(b * h + idx) * (n / 4) * 16});
    if (odd) st.push_back(Stage{2, cur ? log_n - 1 : 0, 0, (uint32_t)b * (n / 2) * 4});
  }
  return st;
}

// Order the non-window local bits of a tile row so that the lane bits of a warp (the first
// five unit-index bits; four for 8-byte elements, where a wavefront is half a warp) hit
// different banks under swz<VB>.  The bank of element l is decided by bits [0, VB+3) of
// swz(l): bits below VB are l's own, bit p in [VB, VB+3) is l[p] ^ l[p+3].  So a non-window
// bit below VB+3 is a good lane bit as it is, and a bank bit p >= VB that lies inside the
// window is replaced by bit p+3, which the swizzle folds onto it.  Windows that start at bit
// 0 are read with 16-byte accesses instead (`vec`): there the natural order is conflict-free.
inline int choose_unit_bits(int logC, int lbit, int K, int vb, bool vec, uint8_t* ubit) {
  std::vector<int> order;
  std::vector<bool> used(32, false);
  auto in_window = [&](int b) { return b >= lbit && b < lbit + K; };
  if (!vec) {
    for (int p = 0; p < vb + 3 && p < logC; ++p) {
      int cand = -1;
      if (!in_window(p)) cand = p;
      else if (p >= vb && p + 3 < logC && !in_window(p + 3)) cand = p + 3;
      if (cand >= 0 && !used[cand]) { order.push_back(cand); used[cand] = true; }
    }
  }
  for (int b = 0; b < logC; ++b)
    if (!in_window(b) && !used[b]) { order.push_back(b); used[b] = true; }
  for (size_t j = 0; j < order.size() && j < (size_t)kMaxUnitBits; ++j) ubit[j] = (uint8_t)order[j];
  return (int)order.size();
}

// Shared memory the planners may fill per CTA: the 227 KB a CTA can opt into on sm_100, less 2 KB
// that the kernels keep for alignment slack (tiles start on a 1024-byte boundary), barriers and slots.
constexpr int kSmemMax = 227 * 1024 - 2048;
constexpr int kMaxSnap = 8;

inline Panel full_row_panel(int log_n) { return Panel{log_n, log_n, log_n, 0}; }

// ------------------------------------------------------------------ forward groups

// Cut stages [t0, t1) into register-window groups of at most kmax bits.  A group never
// crosses a change of radix or direction, nor a stage index listed in `cuts` (a snapshot
// is emitted after the group that ends at cuts[i], into slot i).
inline bool plan_fw_groups(const std::vector<Stage>& st, int t0, int t1, const std::vector<int>& cuts,
                           const Panel& pn, int vb, int kmax, std::vector<FwGroup>& out) {
  auto local_bit = [&](int gb) { return gb < pn.lseg ? gb : gb - pn.pb + pn.lseg; };
  int t = t0;
  while (t < t1) {
    // maximal run: same radix, bits moving by +-step, no cut inside
    const int radix = st[t].radix, step = radix == 4 ? 2 : 1;
    int e = t + 1;
    int dir = 0;
    auto is_cut = [&](int idx) { return std::find(cuts.begin(), cuts.end(), idx) != cuts.end(); };
    while (e < t1 && !is_cut(e) && st[e].radix == radix && st[e].which == st[t].which) {
      const int d = st[e].bit - st[e - 1].bit;
      if (d != step && d != -step) break;
      if (dir == 0) dir = d; else if (d != dir) break;
      ++e;
    }
    const int run = e - t;
    const int per = kmax / step;  // stages per group
    if (per < 1) return false;
    const int ng = (run + per - 1) / per;
    int done = 0;
    for (int gi = 0; gi < ng; ++gi) {
      const int cnt = run / ng + (gi < run % ng ? 1 : 0);
      FwGroup g;
      std::memset(&g, 0, sizeof(g));
      const int first = t + done, last = first + cnt - 1;
      const int lo = std::min(st[first].bit, st[last].bit);
      g.K = (uint8_t)(cnt * step);
      g.lbit = (uint8_t)local_bit(lo);
      const bool dec = (cnt > 1 && st[last].bit < st[first].bit);
      g.pattern = (uint8_t)(radix == 4 ? (dec ? kR4Dec : kR4Inc) : (dec ? kR2Dec : kR2Inc));
      g.which = (uint8_t)st[first].which;
      for (int s = 0; s < cnt; ++s) g.tw_off[s] = st[first + s].tw_off;
      g.vec = (uint8_t)(g.lbit == 0 && (1 << g.K) >= (1 << vb) && pn.lseg >= g.K);
      g.nubits = (uint8_t)choose_unit_bits(pn.logC, g.lbit, g.K, vb, g.vec != 0, g.ubit);
      for (int m = 0; m < (1 << g.K); ++m) g.d[m] = (uint16_t)swz_rt(m << g.lbit, vb);
      for (size_t ci = 0; ci < cuts.size(); ++ci)
        if (cuts[ci] == last + 1) g.emit = (uint8_t)(ci + 1);
      out.push_back(g);
      done += cnt;
    }
    t = e;
  }
  return true;
}

// Rows per forward tile: as many as fit the shared memory one CTA may use when `ctas` CTAs
// share an SM (1 KB per CTA is reserved by the system), capped by max_rows and the batch.
template <typename T>
inline int fw_rows_per_tile(int logC, int B, int ctas, int max_rows) {
  const int row_bytes = (int)sizeof(T) << logC;
  const int budget = ctas <= 1 ? kSmemMax : (228 * 1024) / ctas - 1024 - 2048;
  int R = budget / row_bytes;
  if (R < 1) R = kSmemMax / row_bytes;  // a row that only fits alone: one CTA per SM after all
  if (R > max_rows) R = max_rows;
  if (R > B) R = B;
  return R;
}

// ------------------------------------------------------------------ forward passes
//
// A product whose rows do not fit one SM's shared memory runs as several launches ("passes")
// of the forward kernel, each on panels of at most 2^logCmax columns: a pass is a run of
// consecutive stages whose bits all lie below logCmax (contiguous panels) or inside a bit range
// [lo, hi] narrow enough to leave segments of consecutive columns (strided panels: global bits
// [0, w) and [lo, hi]).  The passes work in place on a full-width buffer.
struct FwPass {
  int t0, t1;
  Panel panel;
};

inline std::vector<FwPass> plan_fw_passes(const std::vector<Stage>& st, int t0, int t1, int log_n, int logCmax) {
  std::vector<FwPass> passes;
  const int lc = std::min(logCmax, log_n);
  auto stage_hi = [&](const Stage& s) { return s.bit + (s.radix == 4 ? 1 : 0); };
  auto feasible = [&](int lo, int hi) {
    if (hi + 1 <= lc) return true;
    return (hi - lo + 1) + std::min(5, lo) <= lc;  // keep 32 consecutive columns per segment when the bits allow
  };
  int t = t0;
  while (t < t1) {
    int lo = st[t].bit, hi = stage_hi(st[t]);
    if (!feasible(lo, hi)) return {};
    int e = t + 1;
    while (e < t1) {
      const int nlo = std::min(lo, st[e].bit), nhi = std::max(hi, stage_hi(st[e]));
      if (!feasible(nlo, nhi)) break;
      lo = nlo; hi = nhi;
      ++e;
    }
    FwPass ps;
    ps.t0 = t; ps.t1 = e;
    if (hi + 1 <= lc) {
      ps.panel = Panel{lc, lc, lc, log_n - lc};
    } else {
      const int pw = hi - lo + 1;
      const int w = std::min(lc - pw, lo);
      ps.panel = Panel{pw + w, w, lo, log_n - pw - w};
    }
    passes.push_back(ps);
    t = e;
  }
  return passes;
}

// ------------------------------------------------------------------ backward phases

// Code variant that the second-generation backward kernel runs for a sub-group (bfly_bw2.h).
inline void bw2_assign_kase(BwSg& sg, int KW) {
  // pattern numbering of bw_pattern() in bfly_core.h
  int pat = KW == 1 ? 0 : (sg.radix == 4 ? 6 : (sg.nst == 2 ? sg.q[0] * 2 + sg.q[1] : 4 + sg.q[0]));
  sg.swap12 = 0;
  if (!sg.vec && KW == 2 && (pat == 2 || pat == 3 || pat == 5)) {
    pat = pat == 2 ? 1 : (pat == 3 ? 0 : 4);
    sg.swap12 = 1;
  }
  sg.kase = (uint8_t)(2 * pat + (sg.vec ? 1 : 0));
}


struct BwPhase {
  int t0, t1;   // stages [t0, t1)
  Panel panel;
  int nsg;
  BwSg sg[kMaxSg];
};

// Cut the stage list into phases.  A phase is a run of consecutive stages whose bits fit a
// panel of at most 2^logCmax columns: either all below logCmax (contiguous panel), or
// within a bit range narrow enough to leave 2^wmin consecutive columns per segment.
// Inside a phase, sub-groups are windows of KW bits holding up to KW radix-2 stages (or one
// radix-4 stage when KW == 2).
inline std::vector<BwPhase> plan_bw_phases(const std::vector<Stage>& st, int log_n, int logCmax, int KW,
                                           int max_sg, int vb) {
  std::vector<BwPhase> phases;
  const int L = (int)st.size();
  const int lc = std::min(logCmax, log_n);
  auto stage_hi = [&](const Stage& s) { return s.bit + (s.radix == 4 ? 1 : 0); };
  // strided panels keep at least KW phase bits so that every window fits inside them
  auto eff_pw = [&](int lo, int hi) { return std::max(hi - lo + 1, std::min(KW, hi + 1)); };
  auto feasible = [&](int lo, int hi) {
    if (hi + 1 <= lc) return true;
    const int pw = eff_pw(lo, hi);
    const int lo_eff = hi - pw + 1;
    return pw + std::min(5, lo_eff) <= lc;  // keep 32 consecutive columns per segment when the bits allow
  };
  int t = 0;
  while (t < L) {
    // ---- grow the phase sub-group by sub-group
    int lo = st[t].bit, hi = stage_hi(st[t]);
    int nsg = 0;
    int e = t;
    struct SgTmp { int first, cnt, wlo; };
    std::vector<SgTmp> sgs;
    while (e < L && nsg < max_sg) {
      // next sub-group starting at stage e
      int cnt = 1;
      int wlo = st[e].bit, whi = stage_hi(st[e]);
      if (st[e].radix == 2) {
        while (cnt < KW && e + cnt < L && st[e + cnt].radix == 2 && st[e + cnt].which == st[e].which) {
          const int b = st[e + cnt].bit;
          const int nlo = std::min(wlo, b), nhi = std::max(whi, b);
          if (nhi - nlo + 1 > KW) break;
          // keep two-bit windows on even bits: a window starting at bit 1 cannot be made
          // bank-conflict free (bank bits 0 and 1 have no substitute)
          if (nhi != nlo && (nlo & 1)) break;
          wlo = nlo; whi = nhi;
          ++cnt;
        }
      } else if (KW < 2) {
        return {};  // radix-4 needs a 2-bit window
      }
      const int nlo = std::min(lo, wlo), nhi = std::max(hi, whi);
      if (!feasible(nlo, nhi)) break;
      lo = nlo; hi = nhi;
      sgs.push_back(SgTmp{e, cnt, wlo});
      e += cnt;
      ++nsg;
    }
    if (sgs.empty()) return {};  // a single stage does not fit: caller reports unsupported
    BwPhase ph;
    std::memset(&ph, 0, sizeof(ph));
    ph.t0 = t; ph.t1 = e; ph.nsg = nsg;
    int lo_eff = 0;
    if (hi + 1 <= lc) {
      ph.panel = Panel{lc, lc, lc, log_n - lc};
    } else {
      const int pw = eff_pw(lo, hi);
      lo_eff = hi - pw + 1;
      const int w = std::min(lc - pw, lo_eff);
      ph.panel = Panel{pw + w, w, lo_eff, log_n - pw - w};
    }
    const bool strided = ph.panel.lseg != ph.panel.logC;
    auto local_bit = [&](int gb) { return gb < ph.panel.lseg ? gb : gb - ph.panel.pb + ph.panel.lseg; };
    for (int j = 0; j < nsg; ++j) {
      BwSg& sg = ph.sg[j];
      const SgTmp& s = sgs[j];
      sg.radix = (uint8_t)st[s.first].radix;
      sg.which = (uint8_t)st[s.first].which;
      sg.nst = (uint8_t)s.cnt;
      const int width = (sg.radix == 4) ? 2 : KW;
      // lowest global bit of the window: the window must end at or below the top bit the panel
      // is closed under, and (strided panels) stay inside the phase bits
      const int top = strided ? hi : ph.panel.logC - 1;
      const int wg = std::min(s.wlo, top - width + 1);
      const int wl = local_bit(wg);
      sg.lbit = (uint8_t)wl;
      for (int k = 0; k < s.cnt; ++k) {
        sg.q[k] = (uint8_t)(st[s.first + k].bit - wg);
        sg.tw_off[k] = st[s.first + k].tw_off;
      }
      sg.vec = (uint8_t)(wl == 0 && (1 << width) >= (1 << vb) && ph.panel.lseg >= width);
      sg.nubits = (uint8_t)choose_unit_bits(ph.panel.logC, wl, width, vb, sg.vec != 0, sg.ubit);
      for (int m = 0; m < (1 << width); ++m) sg.d[m] = (uint16_t)swz_rt(m << wl, vb);
    }
    phases.push_back(ph);
    t = e;
  }
  return phases;
}

}  // namespace bfly
