// Packed-pair forward kernel for float32 radix-2 products on rows of 512 .. 8192 columns (256-thread
// CTAs, two per SM, up to 4096 columns; one 512-thread CTA per SM for 8192), and, panel by panel, on
// wider rows.
//
// A thread owns 16 elements of a row: the 8 values of a three-bit register window, each with
// its right-hand neighbour (column bit 0), held as 8 two-float registers.  A butterfly stage on
// a window bit is then 16 packed multiply-adds (fma.rn.f32x2) on operands that sit side by side
// in shared memory (8-byte or 16-byte accesses), with the two columns' twiddles packed the same
// way; a stage on bit 0 itself works inside the pairs.  Up to three stages run register to
// register between two trips to shared memory ("group").
//
// The tile is stored in chunks of 512 columns -- what the 32 lanes of a warp cover -- and a warp
// owns one chunk of a run of rows (its "box"): it loads and stores the box with its own bulk
// tensor copies, and every group whose window lies below bit 9 needs only a warp-level
// barrier.  A CTA-wide barrier remains around the groups on bits 9 and up.
//
// Host/device header: the planner and the per-thread routines compile as plain C++ too, so the
// test-suite's emulator runs them thread by thread on the CPU.
#pragma once
#include <vector>

#include "bfly_core.h"
#include "bfly_plan.h"

namespace bfly {

constexpr int kFw2Threads = 256;
constexpr int kFw2MaxGroups = 48;
constexpr int kFw2MaxSnap = 8;
constexpr int kFw2MinLogN = 9, kFw2MaxLogN = 12;
// rows of 8192 columns run on one 512-thread CTA per SM (16 warps, one 512-column chunk each)
constexpr int kFw2WideLogN = 13, kFw2WideThreads = 512;
constexpr int kFw2Declined = 1;  // run_fw2: the launch does not qualify, use the generic kernel

// ---------------------------------------------------------------- packed pairs
//
// On the device a pair lives in one 64-bit register from the shared-memory load to the store
// (inline PTX on .b64 operands), and the twiddles arrive already paired from a re-ordered copy
// of the twiddle tensor: packing two floats inside the kernel costs two register moves per
// packed instruction, because the assembler re-does the pack at every use.
#if defined(__CUDA_ARCH__)
typedef unsigned long long f2;
__device__ __forceinline__ f2 mk2(float a, float b) {
  f2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ f2 swap2(f2 v) {
  float a, b;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
  return mk2(b, a);
}
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) {
  f2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f2 mul2(f2 a, f2 b) {
  f2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
template <int IMM> __device__ __forceinline__ void sm_ld8(smaddr_t a, f2& v) {
  asm volatile("ld.shared.b64 %0, [%1+%2];" : "=l"(v) : "r"(a), "n"(IMM) : "memory");
}
template <int IMM> __device__ __forceinline__ void sm_st8(smaddr_t a, const f2& v) {
  asm volatile("st.shared.b64 [%0+%1], %2;" ::"r"(a), "n"(IMM), "l"(v) : "memory");
}
template <int IMM> __device__ __forceinline__ void sm_ld16p(smaddr_t a, f2& v0, f2& v1) {
  asm volatile("ld.shared.v2.b64 {%0, %1}, [%2+%3];" : "=l"(v0), "=l"(v1) : "r"(a), "n"(IMM) : "memory");
}
template <int IMM> __device__ __forceinline__ void sm_st16p(smaddr_t a, const f2& v0, const f2& v1) {
  asm volatile("st.shared.v2.b64 [%0+%1], {%2, %3};" ::"r"(a), "n"(IMM), "l"(v0), "l"(v1) : "memory");
}
#else
struct f2 { float x, y; };
inline f2 mk2(float a, float b) { return f2{a, b}; }
inline f2 swap2(f2 v) { return f2{v.y, v.x}; }
inline f2 fma2(f2 a, f2 b, f2 c) { return f2{fma_(a.x, b.x, c.x), fma_(a.y, b.y, c.y)}; }
inline f2 mul2(f2 a, f2 b) { return f2{mul_(a.x, b.x), mul_(a.y, b.y)}; }
template <int IMM> inline void sm_ld8(smaddr_t a, f2& v) { v = *reinterpret_cast<const f2*>(a + IMM); }
template <int IMM> inline void sm_st8(smaddr_t a, const f2& v) { *reinterpret_cast<f2*>(a + IMM) = v; }
template <int IMM> inline void sm_ld16p(smaddr_t a, f2& v0, f2& v1) {
  v0 = reinterpret_cast<const f2*>(a + IMM)[0]; v1 = reinterpret_cast<const f2*>(a + IMM)[1];
}
template <int IMM> inline void sm_st16p(smaddr_t a, const f2& v0, const f2& v1) {
  reinterpret_cast<f2*>(a + IMM)[0] = v0; reinterpret_cast<f2*>(a + IMM)[1] = v1;
}
#endif

// ---------------------------------------------------------------- plan

// Stage kinds of a group: 0..2 = radix-2 stage on window bit b + kind; 3 = on column bit 0 (inside
// the packed pairs; contiguous windows only).  The kernel is instantiated for the stage-kind
// sequences the planner emits (monotone runs of up to three stages):
//   X(id, number of stages, kind of stage 0, 1, 2)
#define BFLY_FW2_VARIANTS(X) \
  X(0, 1, 0, 0, 0) X(1, 1, 1, 0, 0) X(2, 1, 2, 0, 0)                   \
  X(3, 2, 0, 1, 0) X(4, 2, 1, 2, 0) X(5, 2, 1, 0, 0) X(6, 2, 2, 1, 0) \
  X(7, 3, 0, 1, 2) X(8, 3, 2, 1, 0)                                   \
  X(9, 1, 3, 0, 0) X(10, 2, 3, 0, 0) X(11, 2, 0, 3, 0) X(12, 3, 3, 0, 1) X(13, 3, 1, 0, 3)
constexpr int kFw2FirstPairVariant = 9;  // variants from here on contain a bit-0 stage

inline int fw2_variant_id(int nst, const int* kind) {
  const int k0 = kind[0], k1 = nst > 1 ? kind[1] : 0, k2 = nst > 2 ? kind[2] : 0;
#define BFLY_X(ID, N, A, B, C) if (nst == N && k0 == A && k1 == B && k2 == C) return ID;
  BFLY_FW2_VARIANTS(BFLY_X)
#undef BFLY_X
  return -1;
}

// kind of stage s of a variant
BFLY_HD int fw2_variant_kind(int variant, int s) {
  switch (variant) {
#define BFLY_X(ID, N, A, B, C) case ID: return s == 0 ? A : (s == 1 ? B : C);
    BFLY_FW2_VARIANTS(BFLY_X)
#undef BFLY_X
    default: return 0;
  }
}

struct Fw2Group {
  uint8_t b;        // lowest column bit of the register window (1 for contiguous windows)
  uint8_t contig;   // window = bits 1..3: the thread's 16 elements are 16 consecutive columns
  uint8_t nst;      // stages in the group
  uint8_t variant;  // index into BFLY_FW2_VARIANTS
  uint8_t sync;     // barrier before the group: 0 none, 1 warp, 2 CTA
  uint8_t emit;     // 1 + snapshot slot written after the group, 0 = none
  uint8_t local;    // the window lies inside a warp's 512-column chunk
  uint8_t pad_;
  uint32_t tw_off[3];  // element offset of each stage's twiddles inside one stack
  uint32_t pk_off;     // offset (16-byte entries) of the group's packed twiddles inside one stack
};

struct Fw2Params {
  const float* tw;
  int64_t tw_stack;  // twiddle elements per stack
  // the twiddles re-ordered for the kernel (fw2_pack_entry): per stack and group, entry
  // (s * 8 + j) * U + u holds the j-th 16 bytes of stage s for the thread with unit index u
  float* packed;
  int64_t packed_stack;  // 16-byte entries per stack
  int B, S, log_n;
  int Rw;            // rows of a warp's box = rows a thread processes per group
  int P;             // row groups per tile (256 threads / (n/16) threads per row)
  int R;             // rows per tile = P * Rw
  int cta_syncs;     // the plan contains CTA-wide barriers
  int x_stack, out_stack;  // the input / output descriptor has a stack dimension
  int has_out;
  int out_cols;      // columns of the output that exist (chunks beyond are not stored)
  // the tensors themselves (the device kernel reaches them through TMA descriptors; the host
  // emulator through these)
  const float* x; int64_t x_sB, x_sS; int x_cols;
  float* out; int64_t out_sB, out_sS;
  float* snap[kFw2MaxSnap];
  // optional bias added to the output before it is stored: bias[stack * n + column] for flat
  // output positions below bias_len (the output buffer is then one (B, S * n) matrix)
  const float* bias;
  int bias_len;
  // Panel view (rows wider than 4096 columns, one real stack): the launch's S "stacks" are the
  // column panels of `panel` (4096 columns each: contiguous, or 32-column blocks at a power-of-two
  // stride), log_n = 12 and the stage bits are panel-local.  Tensors are then addressed as
  // row * sB + fw2_view_col(panel index, local column); snapshots are rows of view_row floats.
  int view;
  int view_row;
  Panel panel;
  int threads;       // threads per CTA: 0 = 256; 512 for rows of 8192 columns (one CTA per SM)
  int ngroups;
  Fw2Group g[kFw2MaxGroups];
};

// Real column of local column c of panel pi in a panel view.
BFLY_HD int fw2_view_col(const Fw2Params& p, int pi, int c) { return p.panel.col(p.panel.base(pi), c); }

// Cut stages [t0, t1) (radix 2 only) into groups.  `cuts`: stage indices after which a snapshot
// is written (slot i).  Returns false when the range does not qualify.
inline bool plan_fw2_groups(const std::vector<Stage>& st, int t0, int t1, const std::vector<int>& cuts, int log_n,
                            std::vector<Fw2Group>& out) {
  if (log_n < kFw2MinLogN || log_n > kFw2WideLogN) return false;
  for (int t = t0; t < t1; ++t)
    if (st[t].radix != 2 || st[t].which != 0) return false;
  auto is_cut = [&](int idx) { return std::find(cuts.begin(), cuts.end(), idx) != cuts.end(); };
  int t = t0;
  while (t < t1) {
    int e = t + 1, dir = 0;
    while (e < t1 && e - t < 3 && !is_cut(e)) {
      const int d = st[e].bit - st[e - 1].bit;
      if (d != 1 && d != -1) break;
      if (dir == 0) dir = d; else if (d != dir) break;
      ++e;
    }
    Fw2Group g;
    std::memset(&g, 0, sizeof(g));
    g.nst = (uint8_t)(e - t);
    int lo = st[t].bit, hi = st[t].bit;
    for (int k = t; k < e; ++k) { lo = std::min(lo, st[k].bit); hi = std::max(hi, st[k].bit); }
    int kind[3] = {0, 0, 0};
    if (hi <= 3 && (lo >= 1 || hi <= 2)) {
      g.contig = 1; g.b = 1;
      for (int k = t; k < e; ++k) kind[k - t] = st[k].bit == 0 ? 3 : st[k].bit - 1;
    } else if (lo >= 2) {
      g.contig = 0;
      g.b = (uint8_t)std::min(lo, log_n - 3);
      for (int k = t; k < e; ++k) kind[k - t] = st[k].bit - g.b;
    } else {
      // bits (1,2,3,4)-straddling runs cannot happen with runs of three; a run like (0,1,2,3)
      // neither.  What is left (lo < 2 with hi > 3) does not occur.
      return false;
    }
    const int vid = fw2_variant_id(g.nst, kind);
    if (vid < 0) return false;
    g.variant = (uint8_t)vid;
    g.local = (uint8_t)(g.contig || g.b + 2 < 9);
    for (int k = t; k < e; ++k) g.tw_off[k - t] = st[k].tw_off;
    for (size_t ci = 0; ci < cuts.size(); ++ci)
      if (cuts[ci] == e) g.emit = (uint8_t)(ci + 1);
    out.push_back(g);
    t = e;
  }
  // packed twiddles: 8 entries of 16 bytes per stage and thread, groups one after the other
  {
    uint32_t off = 0;
    const uint32_t U = (uint32_t)((1 << log_n) / 16);
    for (auto& g : out) { g.pk_off = off; off += (uint32_t)g.nst * 8u * U; }
  }
  // barriers: none between groups with the same window (a thread re-reads what it wrote), a warp
  // barrier between windows inside a warp's chunk, a CTA barrier otherwise.  A snapshot store
  // after a CTA-wide group reads boxes that other warps go on writing: CTA barrier after it.
  for (size_t i = 0; i < out.size(); ++i) {
    Fw2Group& g = out[i];
    if (i == 0) { g.sync = g.local ? 0 : 2; continue; }
    const Fw2Group& q = out[i - 1];
    if (q.contig == g.contig && q.b == g.b) g.sync = (q.emit && !q.local) ? 2 : 0;
    else g.sync = (q.local && g.local) ? 1 : 2;
  }
  return !out.empty() && out.size() <= (size_t)kFw2MaxGroups;
}

// Rows per thread and group.  Each row of a thread is 16 KB of the tile: up to `rw_max` rows fit
// (14 with one CTA per SM, 7 with two); fewer rows spread a small batch over more CTAs.  Among the
// candidates the one with the least work on the busiest CTA wins (rows plus a fixed cost per tile
// for the twiddle fetches of its groups).
inline int fw2_rows_per_thread(int B, int S, int P, int grid_max, int rw_max) {
  int best = 1;
  double best_cost = 1e30;
  for (int rw = rw_max; rw >= 1; --rw) {
    const int64_t tiles = (int64_t)((B + P * rw - 1) / (P * rw)) * S;
    const int64_t per_cta = (tiles + grid_max - 1) / grid_max;
    const double cost = (double)per_cta * (rw + 2.0);
    if (cost < best_cost - 1e-9) { best_cost = cost; best = rw; }
  }
  return best;
}

// ---------------------------------------------------------------- per-thread routines

// Float index of (row r of the tile, column c) in the tile: chunk-major, rows of a chunk 512
// floats apart, 128-byte swizzle inside a row chunk.
BFLY_HD int fw2_tile_index(int R, int r, int c) { return ((((c >> 9) * R) + r) << 9) + swz<2>(c & 511); }

// Column of the first element (window bits and bit 0 zero) of the thread with unit index u: the
// unit index fills the other column bits from the bottom up.
BFLY_HD int fw2_unit_col(const Fw2Group& g, int u) {
  const int b = g.contig ? 1 : g.b;
  return g.contig ? (u << 4) : (((u & ((1 << (b - 1)) - 1)) << 1) | ((u >> (b - 1)) << (b + 3)));
}

// Entry j (0..7) of stage s of group g for unit u: the 16 bytes the kernel loads into two packed
// registers.  A stage on a window bit pairs the twiddle blocks of two neighbouring columns
// (blocks i0 and i0 + 1): entry 2*pp holds (t00, t00', t01, t01'), entry 2*pp + 1 holds
// (t10, t10', t11, t11') of register pair pp.  A stage on bit 0 works inside a register: entry k
// holds (t00, t11, t01, t10) of the block of register k.
BFLY_HD void fw2_pack_entry(const Fw2Params& p, const Fw2Group& g, int stack, int u, int s, int j, float* out4) {
  const int b = g.contig ? 1 : g.b;
  const int c0 = p.view ? fw2_view_col(p, stack, fw2_unit_col(g, u)) : fw2_unit_col(g, u);
  const int kind = fw2_variant_kind(g.variant, s);
  const float* twp = p.tw + (p.view ? (int64_t)0 : (int64_t)stack * p.tw_stack) + g.tw_off[s];
  if (kind < 3) {
    const int pp = j >> 1, half = j & 1;
    const int m0 = ((pp >> kind) << (kind + 1)) | (pp & ((1 << kind) - 1));
    // in a panel view the local column and the local stage bit translate to the real ones first
    const int col = p.view ? fw2_view_col(p, stack, fw2_unit_col(g, u) | (m0 << b)) : (c0 | (m0 << b));
    const int q = p.view ? p.panel.global_bit(b + kind) : b + kind;
    const int i0 = ((col >> (q + 1)) << q) | (col & ((1 << q) - 1));  // column bit q deleted
    const float* A = twp + (size_t)i0 * 4;
    out4[0] = A[2 * half]; out4[1] = A[4 + 2 * half]; out4[2] = A[2 * half + 1]; out4[3] = A[4 + 2 * half + 1];
  } else {
    const float* A = twp + (size_t)((c0 >> 1) + j) * 4;
    out4[0] = A[0]; out4[1] = A[3]; out4[2] = A[1]; out4[3] = A[2];
  }
}
BFLY_HD int64_t fw2_pack_entries(const Fw2Params& p) { return p.packed_stack * p.S; }
// Fill packed entry e (0 .. fw2_pack_entries) of the launch: e -> (stack, group, stage, j, u).
BFLY_HD void fw2_pack_one(const Fw2Params& p, int64_t e) {
  const int U = (1 << p.log_n) / 16;
  const int stack = (int)(e / p.packed_stack);
  const uint32_t r = (uint32_t)(e % p.packed_stack);
  int gi = 0;
  while (gi + 1 < p.ngroups && p.g[gi + 1].pk_off <= r) ++gi;
  const uint32_t q = r - p.g[gi].pk_off;
  const int u = (int)(q % (uint32_t)U), sj = (int)(q / (uint32_t)U);
  fw2_pack_entry(p, p.g[gi], stack, u, sj >> 3, sj & 7, p.packed + e * 4);
}

// The thread's packed twiddles of one stage: 8 entries of 16 bytes, U entries apart.
BFLY_HD void fw2_load_tw(f2* T, const float* __restrict__ src, int U) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
#if defined(__CUDA_ARCH__)
    const ulonglong2 q = __ldg(reinterpret_cast<const ulonglong2*>(src) + (size_t)j * U);
    T[2 * j] = q.x; T[2 * j + 1] = q.y;
#else
    const float* q = src + (size_t)j * U * 4;
    T[2 * j] = mk2(q[0], q[1]); T[2 * j + 1] = mk2(q[2], q[3]);
#endif
  }
}

// One stage on the 8 packed registers.  Arithmetic per output as Ops<float>::madd2: the own
// coefficient's product is fused onto the rounded product of the partner's.
template <int KS>
BFLY_HD void fw2_apply(f2* v, const f2* T) {
  // all partner products first, then the fused multiply-adds: eight independent operations in
  // flight between a product and the instruction that consumes it
  f2 q[8];
  if constexpr (KS < 3) {
#pragma unroll
    for (int pp = 0; pp < 4; ++pp) {
      const int m0 = ((pp >> KS) << (KS + 1)) | (pp & ((1 << KS) - 1));
      const int m1 = m0 | (1 << KS);
      q[m0] = mul2(T[pp * 4 + 1], v[m1]);
      q[m1] = mul2(T[pp * 4 + 2], v[m0]);
    }
#pragma unroll
    for (int pp = 0; pp < 4; ++pp) {
      const int m0 = ((pp >> KS) << (KS + 1)) | (pp & ((1 << KS) - 1));
      const int m1 = m0 | (1 << KS);
      v[m0] = fma2(T[pp * 4 + 0], v[m0], q[m0]);
      v[m1] = fma2(T[pp * 4 + 3], v[m1], q[m1]);
    }
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) q[k] = mul2(T[k * 2 + 1], swap2(v[k]));
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = fma2(T[k * 2 + 0], v[k], q[k]);
  }
}

template <bool CONTIG, int IMM>
BFLY_HD void fw2_row_ld(const smaddr_t* a, f2* v) {
  if constexpr (CONTIG) {
#pragma unroll
    for (int k = 0; k < 4; ++k) sm_ld16p<IMM>(a[k], v[2 * k], v[2 * k + 1]);
  } else {
#pragma unroll
    for (int m = 0; m < 8; ++m) sm_ld8<IMM>(a[m], v[m]);
  }
}
template <bool CONTIG, int IMM>
BFLY_HD void fw2_row_st(const smaddr_t* a, const f2* v) {
  if constexpr (CONTIG) {
#pragma unroll
    for (int k = 0; k < 4; ++k) sm_st16p<IMM>(a[k], v[2 * k], v[2 * k + 1]);
  } else {
#pragma unroll
    for (int m = 0; m < 8; ++m) sm_st8<IMM>(a[m], v[m]);
  }
}

template <int NST, int K0, int K1, int K2>
BFLY_HD void fw2_stages(f2* v, const f2* T) {
  fw2_apply<K0>(v, T);
  if constexpr (NST > 1) fw2_apply<K1>(v, T + 16);
  if constexpr (NST > 2) fw2_apply<K2>(v, T + 32);
}

// The thread's packed twiddles of group g (nst * 8 entries of 16 bytes) into T[48].
BFLY_HD void fw2_fetch_tw(const Fw2Params& p, const Fw2Group& g, int stack, int tid, f2* T) {
  const int U = (1 << p.log_n) / 16;
  const float* pk = p.packed + ((int64_t)stack * p.packed_stack + g.pk_off + (tid & (U - 1))) * 4;
  fw2_load_tw(T, pk, U);
  if (g.nst > 1) fw2_load_tw(T + 16, pk + (size_t)8 * U * 4, U);
  if (g.nst > 2) fw2_load_tw(T + 32, pk + (size_t)16 * U * 4, U);
}

// One group applied in place to the thread's rows (p.Rw of them, 2 KB apart in the tile); T holds
// the thread's packed twiddles of the group.  PIPE: the next row's loads are issued before the
// current row's arithmetic (needs registers for two rows).
template <int NST, int K0, int K1, int K2, bool CONTIG, bool PIPE>
BFLY_HD void fw2_group_rows(const Fw2Params& p, const Fw2Group& g, float* tile, int tid, const f2* T) {
  const int nub = p.log_n - 4;  // bits of the unit index: 16 columns per thread
  const int u = tid & ((1 << nub) - 1);
  const int rg = tid >> nub;
  const int Rw = p.Rw;
  const int b = CONTIG ? 1 : g.b;
  const int c0 = fw2_unit_col(g, u);
  constexpr int NA = CONTIG ? 4 : 8;
  smaddr_t a[NA];
  const smaddr_t base = sm_addr(tile);
#pragma unroll
  for (int m = 0; m < NA; ++m) {
    const int col = CONTIG ? c0 + 4 * m : (c0 | (m << b));
    a[m] = base + (smaddr_t)fw2_tile_index(p.R, rg * Rw, col) * 4u;
  }
  // two rows per trip: the second row is an immediate offset, the addresses advance once per trip
  int i = 0;
  if constexpr (PIPE) {
    f2 v0[8], v1[8];
    fw2_row_ld<CONTIG, 0>(a, v0);
#pragma unroll 1
    for (; i + 2 <= Rw; i += 2) {
      fw2_row_ld<CONTIG, 2048>(a, v1);
      fw2_stages<NST, K0, K1, K2>(v0, T);
      fw2_row_st<CONTIG, 0>(a, v0);
      if (i + 2 < Rw) fw2_row_ld<CONTIG, 4096>(a, v0);
      fw2_stages<NST, K0, K1, K2>(v1, T);
      fw2_row_st<CONTIG, 2048>(a, v1);
#pragma unroll
      for (int m = 0; m < NA; ++m) a[m] += 4096u;
    }
    if (i < Rw) {
      fw2_stages<NST, K0, K1, K2>(v0, T);
      fw2_row_st<CONTIG, 0>(a, v0);
    }
  } else {
#pragma unroll 1
    for (; i + 2 <= Rw; i += 2) {
      f2 v0[8], v1[8];
      fw2_row_ld<CONTIG, 0>(a, v0);
      fw2_stages<NST, K0, K1, K2>(v0, T);
      fw2_row_st<CONTIG, 0>(a, v0);
      fw2_row_ld<CONTIG, 2048>(a, v1);
      fw2_stages<NST, K0, K1, K2>(v1, T);
      fw2_row_st<CONTIG, 2048>(a, v1);
#pragma unroll
      for (int m = 0; m < NA; ++m) a[m] += 4096u;
    }
    if (i < Rw) {
      f2 v0[8];
      fw2_row_ld<CONTIG, 0>(a, v0);
      fw2_stages<NST, K0, K1, K2>(v0, T);
      fw2_row_st<CONTIG, 0>(a, v0);
    }
  }
}

// Run group g for one thread: dispatch on the (uniform) variant.
template <bool PIPE>
BFLY_HD void fw2_group_dispatch(const Fw2Params& p, const Fw2Group& g, float* tile, int tid, const f2* T) {
  switch (g.variant) {
#define BFLY_X(ID, N, A, B, C)                                                          \
  case ID:                                                                              \
    if constexpr (ID >= kFw2FirstPairVariant) {                                         \
      fw2_group_rows<N, A, B, C, true, PIPE>(p, g, tile, tid, T);                       \
    } else {                                                                            \
      if (g.contig) fw2_group_rows<N, A, B, C, true, PIPE>(p, g, tile, tid, T);         \
      else fw2_group_rows<N, A, B, C, false, PIPE>(p, g, tile, tid, T);                 \
    }                                                                                   \
    break;
    BFLY_FW2_VARIANTS(BFLY_X)
#undef BFLY_X
    default: break;
  }
}

BFLY_HD int64_t fw2_num_tiles(const Fw2Params& p) { return (int64_t)((p.B + p.R - 1) / p.R) * p.S; }
BFLY_HD size_t fw2_tile_bytes(const Fw2Params& p) { return ((size_t)p.R * sizeof(float)) << p.log_n; }
// the tile, then one mbarrier per warp and the give-up flag
BFLY_HD int fw2_threads(const Fw2Params& p) { return p.threads > 0 ? p.threads : kFw2Threads; }
BFLY_HD size_t fw2_smem_bytes(const Fw2Params& p) { return fw2_tile_bytes(p) + (size_t)(fw2_threads(p) / 32) * 8 + 16; }
// bytes of the re-ordered twiddle copy (same size as the twiddle tensor): 0 when the shape does
// not take this kernel.  Rows wider than 4096 columns (one stack, up to 2^19) run pass by pass on
// panels; a pass holds at most 24 stages (the low 12 bits at the end of one block and the start of
// the next) and re-uses the space.
inline size_t fw2_packed_bytes(int S, int log_n, int nblocks) {
  const size_t whole = (size_t)S * nblocks * log_n * ((size_t)8 << log_n);
  const size_t passes = (log_n > kFw2MaxLogN && log_n <= 19 && S == 1) ? (size_t)24 * ((size_t)8 << log_n) : 0;
  if (log_n == kFw2WideLogN) return whole > passes ? whole : passes;  // one launch, or the panel passes as a fallback
  if (passes) return passes;
  if (log_n < kFw2MinLogN || log_n > kFw2MaxLogN) return 0;
  return whole;
}

}  // namespace bfly
