// Backward phase, packed-pair generation (float32, radix-2 sub-groups, panels of 1024 columns).
//
// Same twiddle-stationary scheme as bfly_bw2.h -- a CTA owns a column panel and a slice of the
// rows, keeps the twiddles and the twiddle-gradient accumulators of the phase's sub-groups in
// tensor memory for its whole life, and streams batches of rows through shared memory -- with
// the arithmetic done on pairs of neighbouring columns:
//
//  * a thread's unit is 8 elements of a row: the 4 values of a two-bit window, each with its
//    right-hand neighbour (column bit 0), held as 4 two-float registers that move between shared
//    memory and registers with 8-byte accesses (16-byte ones when the window is bits 0 and 1).
//    A butterfly stage, its transpose and the gradient outer products are packed instructions
//    (fma.rn.f32x2): half the floating-point issue slots of the scalar kernel;
//  * the twiddles and accumulators are stored in tensor memory already paired the way the
//    packed instructions want them (the two columns' coefficients side by side), 32 + 32
//    columns per sub-group, fetched with one 32-column tcgen05.ld each per step;
//  * 128 threads per CTA (one unit per thread: 1024 columns), two CTAs per SM, five rows per
//    batch, all of them in flight per thread.
//
// Host/device header: the per-thread routines compile as plain C++ for the test emulator.
#pragma once
#include "bfly_bw2.h"
#include "bfly_fw2.h"

namespace bfly {


constexpr int kBw3Threads = 128;
constexpr int kBw3Rows = 5;       // rows per batch
constexpr int kBw3MaxSg = 4;
constexpr int kBw3TmemCols = 256; // per CTA: 4 sub-groups x (32 twiddle + 32 accumulator columns) per thread
#ifndef BFLY_BW3_PREFETCH
#define BFLY_BW3_PREFETCH 0
#endif
// 1: a step requests the tensor-memory operands of the step after it before it ends (their latency
// overlaps the barrier; costs 64 registers that stay live across steps); 0: every step fetches its own
constexpr bool kBw3Prefetch = BFLY_BW3_PREFETCH != 0;
#ifndef BFLY_BW3_PREFETCH_TW
#define BFLY_BW3_PREFETCH_TW 0
#endif
// 1: a step requests only the twiddles of the step after it (32 registers live across the barrier;
// measured: no gain over 0)
constexpr bool kBw3PrefetchTw = BFLY_BW3_PREFETCH_TW != 0 && !kBw3Prefetch;

// Stage kinds on the 4 packed registers (register index m = two window bits):
//   0 / 1: radix-2 stage between registers that differ in register bit 0 / 1
//   2:     radix-2 stage on column bit 0, inside every pair
struct Bw3Sg {
  uint8_t nst;        // stages in the sub-group (1 or 2)
  uint8_t kind[2];
  uint8_t contig;     // the window is column bits 0 and 1: the unit is 8 consecutive columns
  uint8_t lbit;       // lowest local bit of the window (strided kind; >= 2)
  uint8_t gbit[2];    // global column bit of register bit 0 / 1
  uint8_t pad_;
  uint8_t ubit[8];    // local bit positions fed by the 7 bits of the unit index
  uint32_t d[4];      // byte offset pattern of register m inside a tile row: address = a0 ^ d[m]
  uint32_t tw_off[2]; // element offset of each stage's twiddles inside one stack
  uint8_t sbit[2];    // global column bit each stage acts on
  uint8_t pad2_[2];
};

struct Bw3Params {
  BwParams<float> b;   // tensors, panel, row slices, TMA switches (sub-group table unused)
  Bw3Sg sg[kBw3MaxSg];
};

// Lane bits for conflict-free 8-byte accesses under the 128-byte swizzle: half a warp (16 lanes,
// 128 bytes) must cover the 32 banks once.  Bank bit p (1..4) of a float index is the index's own
// bit p, XORed for p >= 2 with bit p + 3; a bank bit the window occupies is represented by its
// partner.  The remaining free bits follow in ascending order.
inline void bw3_choose_unit_bits(int lbit, bool contig, uint8_t* ubit) {
  bool used[10] = {false};
  auto in_window = [&](int b) { return contig ? b <= 2 : (b == 0 || b == lbit || b == lbit + 1); };
  int cnt = 0;
  if (contig) {
    // 16-byte accesses: 8 lanes cover the 8 chunk slots of a 128-byte line: float bits 3, 4 and
    // (through the swizzle, onto float bit 2) bit 5
    for (int b : {3, 4, 5}) { ubit[cnt++] = (uint8_t)b; used[b] = true; }
  } else {
    for (int p = 1; p <= 4; ++p) {
      int c = -1;
      if (!in_window(p)) c = p;
      else if (p >= 2 && !in_window(p + 3)) c = p + 3;
      if (c >= 0 && !used[c]) { ubit[cnt++] = (uint8_t)c; used[c] = true; }
    }
  }
  // a free bit whose bank partner is already a lane bit must not join the first four
  for (int b = 1; b < 10 && cnt < 7; ++b)
    if (!in_window(b) && !used[b]) { ubit[cnt++] = (uint8_t)b; used[b] = true; }
}

// Fill the packed-pair view of a phase's sub-groups.  False when the phase does not qualify
// (radix-4 factors, windows off the even bits, panels other than 1024 columns).
inline bool bw3_plan(const BwParams<float>& p, Bw3Sg* out) {
  if (p.panel.logC != 10 || p.nsg < 1 || p.nsg > kBw3MaxSg) return false;
  for (int j = 0; j < p.nsg; ++j) {
    const BwSg& s = p.sg[j];
    Bw3Sg& o = out[j];
    std::memset(&o, 0, sizeof(o));
    if (s.radix != 2 || s.nst < 1 || s.nst > 2 || s.lbit == 1) return false;  // (a window on local bits 1, 2 has no 8-byte pairing)
    o.nst = s.nst;
    o.contig = s.lbit == 0;
    o.lbit = s.lbit;
    if (!o.contig && s.lbit + 1 > 9) return false;
    const int rb0 = o.contig ? 1 : s.lbit, rb1 = o.contig ? 2 : s.lbit + 1;  // local bits of register bits 0, 1
    o.gbit[0] = (uint8_t)p.panel.global_bit(rb0);
    o.gbit[1] = (uint8_t)p.panel.global_bit(rb1);
    if (p.panel.global_bit(0) != 0 || p.panel.lseg < 5) return false;
    for (int k = 0; k < s.nst; ++k) {
      const int wb = s.q[k];  // window bit of the stage: local bit lbit + wb
      o.kind[k] = (uint8_t)(o.contig ? (wb == 0 ? 2 : 0) : wb);
      o.sbit[k] = (uint8_t)p.panel.global_bit(s.lbit + wb);
      o.tw_off[k] = s.tw_off[k];
    }
    bw3_choose_unit_bits(s.lbit, o.contig != 0, o.ubit);
    for (int m = 0; m < 4; ++m) {
      const int l = o.contig ? 4 * m : (((m & 1) << rb0) | ((m >> 1) << rb1));
      o.d[m] = (uint32_t)swz<2>(l) * 4u;
    }
  }
  return true;
}

// Local column (window bits and bit 0 zero) of unit u.
BFLY_HD int bw3_unit_local(const Bw3Sg& s, int u) {
  int l = 0;
#pragma unroll 1
  for (int j = 0; j < 7; ++j) l |= ((u >> j) & 1) << s.ubit[j];
  return l;
}
// Global column of register m (its left element) of the unit whose first global column is col0.
BFLY_HD int bw3_reg_col(const Bw3Sg& s, int col0, int m) {
  return col0 | ((m & 1) << s.gbit[0]) | ((m >> 1) << s.gbit[1]);
}

// The 16 twiddle floats of stage k for one thread, in the order they sit in tensor memory, and
// the global element offset each comes from (the accumulators go back the same way).
//   stage between registers: per register pair pp, (t00, t00', t01, t01', t10, t10', t11, t11')
//     with ' = the right-hand column (twiddle block i0 + 1);
//   stage inside the pairs: per register, (t00, t11, t01, t10) of the register's block.
BFLY_HD void bw3_tw_offsets(const Bw3Sg& s, int k, int col0, uint32_t* off16) {
  const int kind = s.kind[k], q = s.sbit[k];
  if (kind < 2) {
    for (int pp = 0; pp < 2; ++pp) {
      const int m0 = kind == 0 ? (pp << 1) : pp;
      const int col = bw3_reg_col(s, col0, m0);
      const uint32_t i0 = (uint32_t)delete_bit(col, q);
      for (int e = 0; e < 4; ++e) {
        off16[pp * 8 + 2 * e] = s.tw_off[k] + i0 * 4u + (uint32_t)e;
        off16[pp * 8 + 2 * e + 1] = s.tw_off[k] + (i0 + 1u) * 4u + (uint32_t)e;
      }
    }
  } else {
    for (int m = 0; m < 4; ++m) {
      const uint32_t i = (uint32_t)(bw3_reg_col(s, col0, m) >> 1);
      const uint32_t base = s.tw_off[k] + i * 4u;
      off16[m * 4 + 0] = base + 0; off16[m * 4 + 1] = base + 3; off16[m * 4 + 2] = base + 1; off16[m * 4 + 3] = base + 2;
    }
  }
}

// ---------------------------------------------------------------- tensor-memory store (32 columns)
// (the step routines are templates on the store: Acc3Tmem on the device, Acc3Host in the emulator)
#if defined(__CUDACC__)
struct Acc3Tmem {
  uint32_t taddr;  // lane << 16 | first column of this thread
  // sub-group j: twiddles at column 64 j, accumulators at 64 j + 32
  __device__ __forceinline__ void ld32(int col, float* r) const {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]),
          "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]), "=f"(r[16]),
          "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]), "=f"(r[24]),
          "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
        : "r"(taddr + (uint32_t)col) : "memory");
  }
  __device__ __forceinline__ void st32(int col, const float* r) const {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr + (uint32_t)col), "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]),
          "f"(r[7]), "f"(r[8]), "f"(r[9]), "f"(r[10]), "f"(r[11]), "f"(r[12]), "f"(r[13]), "f"(r[14]), "f"(r[15]),
          "f"(r[16]), "f"(r[17]), "f"(r[18]), "f"(r[19]), "f"(r[20]), "f"(r[21]), "f"(r[22]), "f"(r[23]), "f"(r[24]),
          "f"(r[25]), "f"(r[26]), "f"(r[27]), "f"(r[28]), "f"(r[29]), "f"(r[30]), "f"(r[31]) : "memory");
  }
  __device__ __forceinline__ void wait_ld() const { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
  __device__ __forceinline__ void wait_st() const { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
};
#endif
struct Acc3Host {
  float* mem;  // kBw3MaxSg * 64 floats
  void ld32(int col, float* r) const { for (int e = 0; e < 32; ++e) r[e] = mem[col + e]; }
  void st32(int col, const float* r) const { for (int e = 0; e < 32; ++e) mem[col + e] = r[e]; }
  void wait_ld() const {}
  void wait_st() const {}
};

// (volatile on the device: the reads of registers that a tcgen05.ld fills must stay behind the
// tcgen05.wait::ld that precedes this call)
BFLY_HD void bw3_pack16(const float* r, f2* T) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#if defined(__CUDA_ARCH__)
    asm volatile("mov.b64 %0, {%1, %2};" : "=l"(T[i]) : "f"(r[2 * i]), "f"(r[2 * i + 1]));
#else
    T[i] = mk2(r[2 * i], r[2 * i + 1]);
#endif
  }
}
BFLY_HD void bw3_unpack16(const f2* T, float* r) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#if defined(__CUDA_ARCH__)
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r[2 * i]), "=f"(r[2 * i + 1]) : "l"(T[i]));
#else
    r[2 * i] = T[i].x; r[2 * i + 1] = T[i].y;
#endif
  }
}

// ---------------------------------------------------------------- arithmetic on the units of a batch
//
// v[r][m]: packed register m of the unit in row r.  Every routine works on all rows of the batch
// at once and is written operation by operation across the rows (all partner products, then all
// fused multiply-adds), so that consecutive instructions are independent: the warps are few
// (two per scheduler) and each has to cover the arithmetic latency with its own instructions.
constexpr int kBw3R = kBw3Rows;

template <int KIND>
BFLY_HD void bw3_stage_fw(f2 (*v)[4], const f2* T) {
  f2 q[kBw3R][4];
  if constexpr (KIND < 2) {
#pragma unroll
    for (int pp = 0; pp < 2; ++pp) {
      const int m0 = KIND == 0 ? (pp << 1) : pp, m1 = m0 | (1 << KIND);
#pragma unroll
      for (int r = 0; r < kBw3R; ++r) {
        q[r][m0] = mul2(T[pp * 4 + 1], v[r][m1]);
        q[r][m1] = mul2(T[pp * 4 + 2], v[r][m0]);
      }
    }
#pragma unroll
    for (int pp = 0; pp < 2; ++pp) {
      const int m0 = KIND == 0 ? (pp << 1) : pp, m1 = m0 | (1 << KIND);
#pragma unroll
      for (int r = 0; r < kBw3R; ++r) {
        v[r][m0] = fma2(T[pp * 4 + 0], v[r][m0], q[r][m0]);
        v[r][m1] = fma2(T[pp * 4 + 3], v[r][m1], q[r][m1]);
      }
    }
  } else {
#pragma unroll
    for (int m = 0; m < 4; ++m)
#pragma unroll
      for (int r = 0; r < kBw3R; ++r) q[r][m] = mul2(T[m * 2 + 1], swap2(v[r][m]));
#pragma unroll
    for (int m = 0; m < 4; ++m)
#pragma unroll
      for (int r = 0; r < kBw3R; ++r) v[r][m] = fma2(T[m * 2 + 0], v[r][m], q[r][m]);
  }
}
// acc += g (x) x ; g <- T^T g     (x: the stage's input), all rows
template <int KIND>
BFLY_HD void bw3_stage_bw(f2 (*g)[4], const f2 (*x)[4], const f2* T, f2* A) {
  f2 q[kBw3R][4];
  if constexpr (KIND < 2) {
#pragma unroll
    for (int pp = 0; pp < 2; ++pp) {
      const int m0 = KIND == 0 ? (pp << 1) : pp, m1 = m0 | (1 << KIND);
#pragma unroll
      for (int r = 0; r < kBw3R; ++r) {
        q[r][m0] = mul2(T[pp * 4 + 2], g[r][m1]);
        q[r][m1] = mul2(T[pp * 4 + 1], g[r][m0]);
      }
    }
#pragma unroll
    for (int r = 0; r < kBw3R; ++r)
#pragma unroll
      for (int pp = 0; pp < 2; ++pp) {
        const int m0 = KIND == 0 ? (pp << 1) : pp, m1 = m0 | (1 << KIND);
        A[pp * 4 + 0] = fma2(g[r][m0], x[r][m0], A[pp * 4 + 0]);
        A[pp * 4 + 1] = fma2(g[r][m0], x[r][m1], A[pp * 4 + 1]);
        A[pp * 4 + 2] = fma2(g[r][m1], x[r][m0], A[pp * 4 + 2]);
        A[pp * 4 + 3] = fma2(g[r][m1], x[r][m1], A[pp * 4 + 3]);
      }
#pragma unroll
    for (int pp = 0; pp < 2; ++pp) {
      const int m0 = KIND == 0 ? (pp << 1) : pp, m1 = m0 | (1 << KIND);
#pragma unroll
      for (int r = 0; r < kBw3R; ++r) {
        g[r][m0] = fma2(T[pp * 4 + 0], g[r][m0], q[r][m0]);
        g[r][m1] = fma2(T[pp * 4 + 3], g[r][m1], q[r][m1]);
      }
    }
  } else {
#pragma unroll
    for (int m = 0; m < 4; ++m)
#pragma unroll
      for (int r = 0; r < kBw3R; ++r) q[r][m] = swap2(mul2(T[m * 2 + 1], g[r][m]));
#pragma unroll
    for (int r = 0; r < kBw3R; ++r)
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        A[m * 2 + 0] = fma2(g[r][m], x[r][m], A[m * 2 + 0]);          // (a00, a11)
        A[m * 2 + 1] = fma2(g[r][m], swap2(x[r][m]), A[m * 2 + 1]);   // (a01, a10)
      }
#pragma unroll
    for (int m = 0; m < 4; ++m)
#pragma unroll
      for (int r = 0; r < kBw3R; ++r) g[r][m] = fma2(T[m * 2 + 0], g[r][m], q[r][m]);
  }
}

template <bool CONTIG, int IMM>
BFLY_HD void bw3_unit_ld(const smaddr_t* a, f2* v) {
  if constexpr (CONTIG) {
    sm_ld16p<IMM>(a[0], v[0], v[1]);
    sm_ld16p<IMM>(a[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int m = 0; m < 4; ++m) sm_ld8<IMM>(a[m], v[m]);
  }
}
template <bool CONTIG, int IMM>
BFLY_HD void bw3_unit_st(const smaddr_t* a, const f2* v) {
  if constexpr (CONTIG) {
    sm_st16p<IMM>(a[0], v[0], v[1]);
    sm_st16p<IMM>(a[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int m = 0; m < 4; ++m) sm_st8<IMM>(a[m], v[m]);
  }
}

constexpr int kBw3RowBytes = 4096;                       // 1024 floats
constexpr int kBw3TileBytes = kBw3Rows * kBw3RowBytes;   // one snapshot tile of a batch

// Forward recompute of sub-group j over the batch: snapshot tile j -> tile j + 1.
// `ready` runs after the shared-memory loads have been issued and before the arithmetic: it waits
// for the step's tensor-memory operands and packs them into T (and A), so that the two latencies
// overlap instead of following each other.
template <int NST, int KA, int KB, bool CONTIG, typename READY>
BFLY_HD void bw3_fw_rows(const smaddr_t* a, const f2* T, READY&& ready) {
  f2 v[kBw3Rows][4];
  static_for<0, kBw3Rows>([&](auto rc) {
    constexpr int r = decltype(rc)::value;
    bw3_unit_ld<CONTIG, r * kBw3RowBytes>(a, v[r]);
  });
  ready();
  bw3_stage_fw<KA>(v, T);
  if constexpr (NST > 1) bw3_stage_fw<KB>(v, T + 8);
  static_for<0, kBw3Rows>([&](auto rc) {
    constexpr int r = decltype(rc)::value;
    bw3_unit_st<CONTIG, kBw3TileBytes + r * kBw3RowBytes>(a, v[r]);
  });
}
// Reverse step of sub-group j over the batch: a = addresses in snapshot tile j, ag = in the gradient tile.
template <int NST, int KA, int KB, bool CONTIG, typename READY>
BFLY_HD void bw3_bw_rows(const smaddr_t* a, const smaddr_t* ag, const f2* T, f2* A, READY&& ready) {
  f2 x[kBw3Rows][4], g[kBw3Rows][4];
  static_for<0, kBw3Rows>([&](auto rc) {
    constexpr int r = decltype(rc)::value;
    bw3_unit_ld<CONTIG, r * kBw3RowBytes>(a, x[r]);
    bw3_unit_ld<CONTIG, r * kBw3RowBytes>(ag, g[r]);
  });
  ready();
  if constexpr (NST > 1) {
    f2 x1[kBw3Rows][4];
#pragma unroll
    for (int r = 0; r < kBw3Rows; ++r)
#pragma unroll
      for (int m = 0; m < 4; ++m) x1[r][m] = x[r][m];
    bw3_stage_fw<KA>(x1, T);
    bw3_stage_bw<KB>(g, x1, T + 8, A + 8);
  }
  bw3_stage_bw<KA>(g, x, T, A);
  static_for<0, kBw3Rows>([&](auto rc) {
    constexpr int r = decltype(rc)::value;
    bw3_unit_st<CONTIG, r * kBw3RowBytes>(ag, g[r]);
  });
}

// Code variant of a sub-group: one stage of kind k -> k; two stages (ka, kb) -> 3 + 3 ka + kb.
BFLY_HD int bw3_variant(const Bw3Sg& s) { return s.nst == 1 ? s.kind[0] : 3 + 3 * s.kind[0] + s.kind[1]; }

#define BFLY_BW3_VARIANTS(X)                                                                     \
  X(0, 1, 0, 0) X(1, 1, 1, 0) X(2, 1, 2, 0)                                                      \
  X(3, 2, 0, 0) X(4, 2, 0, 1) X(5, 2, 0, 2) X(6, 2, 1, 0) X(7, 2, 1, 1) X(8, 2, 1, 2)            \
  X(9, 2, 2, 0) X(10, 2, 2, 1) X(11, 2, 2, 2)

// Shared-memory addresses of the thread's unit in row 0 of tile `tile`.  o[m]: byte offset of
// register m inside a tile row (one 16-byte entry of the unit table per sub-group and thread; a
// contiguous unit uses entries 0 and 1: its two 16-byte chunks).
BFLY_HD void bw3_addresses(smaddr_t tile0, const uint32_t* o, int tile, smaddr_t* a) {
  const smaddr_t base = tile0 + (smaddr_t)(tile * kBw3TileBytes);
#pragma unroll
  for (int m = 0; m < 4; ++m) a[m] = base + o[m];
}
BFLY_HD void bw3_load_offsets(const uint32_t* meta, int j, int tid, uint32_t* o) {
#if defined(__CUDA_ARCH__)
  const uint4 q = reinterpret_cast<const uint4*>(meta)[j * kBw3Threads + tid];
  o[0] = q.x; o[1] = q.y; o[2] = q.z; o[3] = q.w;
#else
  for (int m = 0; m < 4; ++m) o[m] = meta[(j * kBw3Threads + tid) * 4 + m];
#endif
}
// Per-step dispatch word kept behind the unit table: variant | contig << 8.
BFLY_HD uint32_t* bw3_step_table(uint32_t* meta, int nsg) { return meta + (size_t)nsg * kBw3Threads * 4; }

// A batch runs 2 nsg - 1 steps: forward recompute of sub-groups 0 .. nsg - 2, then the reverse
// steps of sub-groups nsg - 1 .. 0.  Step s works on sub-group bw3_step_sg(s).
BFLY_HD int bw3_num_steps(int nsg) { return 2 * nsg - 1; }
BFLY_HD bool bw3_step_is_bw(int nsg, int s) { return s >= nsg - 1; }
BFLY_HD int bw3_step_sg(int nsg, int s) { return s < nsg - 1 ? s : 2 * nsg - 2 - s; }

// Issue the tensor-memory loads a step needs (twiddles; accumulators for a reverse step) into the
// thread's fetch buffers.  They are consumed by bw3_step after its tcgen05.wait::ld.
template <typename ACC>
BFLY_HD void bw3_prefetch(const Bw3Params& p, const ACC& acc, int step, float* tr, float* ar) {
  const int j = bw3_step_sg(p.b.nsg, step);
  acc.ld32(j * 64, tr);
  if (bw3_step_is_bw(p.b.nsg, step)) acc.ld32(j * 64 + 32, ar);
}

// One step of a batch for one thread; its tensor-memory operands were requested by bw3_prefetch.
// Before it ends the step requests the operands of the step that follows (the first step of the
// next batch after the last one), so that their latency overlaps the barrier.  A block-wide
// barrier must follow.
template <typename ACC>
BFLY_HD void bw3_step(const Bw3Params& p, const ACC& acc, const uint32_t* meta, int step, float* sm, int tid, float* tr,
                      float* ar) {
  const int nsg = p.b.nsg;
  const int j = bw3_step_sg(nsg, step);
  const bool is_bw = bw3_step_is_bw(nsg, step);
  smaddr_t a[4], ag[4];
  uint32_t o[4];
  bw3_load_offsets(meta, j, tid, o);
  bw3_addresses(sm_addr(sm), o, j, a);
  const uint32_t word = bw3_step_table(const_cast<uint32_t*>(meta), nsg)[j];
  const int var = (int)(word & 0xff);
  const bool contig = (word >> 8) != 0;
  if (kBw3PrefetchTw) {
    if (is_bw) acc.ld32(j * 64 + 32, ar);  // the twiddles were requested by the step before
  } else if (!kBw3Prefetch) {
    bw3_prefetch(p, acc, step, tr, ar);
  }
  f2 T[16], A[16];
  const int next = step + 1 < bw3_num_steps(nsg) ? step + 1 : 0;
  // the next step's operands, unless it re-reads the accumulators this step is about to store
  const bool same_acc = is_bw && bw3_step_is_bw(nsg, next) && bw3_step_sg(nsg, next) == j;
  auto ready = [&]() {
    acc.wait_ld();
    bw3_pack16(tr, T);
    bw3_pack16(tr + 16, T + 8);
    if (is_bw) {
      bw3_pack16(ar, A);
      bw3_pack16(ar + 16, A + 8);
    }
    // the fetch buffers are free (T and A hold the packed copies)
    if (kBw3Prefetch && !same_acc) bw3_prefetch(p, acc, next, tr, ar);
    // twiddles of the step that follows: their latency overlaps this step's arithmetic and the barrier
    if (kBw3PrefetchTw) acc.ld32(bw3_step_sg(nsg, next) * 64, tr);
  };
  if (!is_bw) {
    switch (var) {
#define BFLY_X(ID, N, KA, KB)                                             \
  case ID:                                                                \
    if (contig) bw3_fw_rows<N, KA, KB, true>(a, T, ready);                \
    else bw3_fw_rows<N, KA, KB, false>(a, T, ready);                      \
    break;
      BFLY_BW3_VARIANTS(BFLY_X)
#undef BFLY_X
      default: break;
    }
    return;
  }
  bw3_addresses(sm_addr(sm), o, nsg, ag);  // the gradient tile follows the nsg snapshot tiles
  switch (var) {
#define BFLY_X(ID, N, KA, KB)                                             \
  case ID:                                                                \
    if (contig) bw3_bw_rows<N, KA, KB, true>(a, ag, T, A, ready);         \
    else bw3_bw_rows<N, KA, KB, false>(a, ag, T, A, ready);               \
    break;
    BFLY_BW3_VARIANTS(BFLY_X)
#undef BFLY_X
    default: break;
  }
  float out[32];
  bw3_unpack16(A, out);
  bw3_unpack16(A + 8, out + 16);
  acc.wait_st();  // the previous reverse step's store (long finished) before this thread stores again
  acc.st32(j * 64 + 32, out);
  if (kBw3Prefetch && same_acc) {
    acc.wait_st();
    bw3_prefetch(p, acc, next, tr, ar);
  }
}

// Per-CTA set-up of one thread: unit positions into `meta`, twiddles (paired) and zeroed
// accumulators into tensor memory.
template <typename ACC>
BFLY_HD void bw3_init(const Bw3Params& p, const ACC& acc, uint32_t* meta, int stack, int pbase, int tid) {
  const float* twp = p.b.tw[0] + (int64_t)stack * p.b.tw_stack[0];
  for (int j = 0; j < p.b.nsg; ++j) {
    const Bw3Sg& s = p.sg[j];
    const int l0 = bw3_unit_local(s, tid);
    const uint32_t a0 = (uint32_t)swz<2>(l0) * 4u;
    for (int m = 0; m < 4; ++m) meta[(j * kBw3Threads + tid) * 4 + m] = a0 ^ s.d[m];
    if (tid == 0) bw3_step_table(meta, p.b.nsg)[j] = (uint32_t)bw3_variant(s) | ((uint32_t)s.contig << 8);
    const int col0 = p.b.panel.col(pbase, l0);
    float tr[32], z[32];
    for (int k = 0; k < 2; ++k) {
      uint32_t off[16];
      if (k < s.nst) bw3_tw_offsets(s, k, col0, off);
      for (int e = 0; e < 16; ++e) tr[k * 16 + e] = k < s.nst ? twp[off[e]] : 0.f;
    }
    for (int e = 0; e < 32; ++e) z[e] = 0.f;
    acc.st32(j * 64, tr);
    acc.st32(j * 64 + 32, z);
  }
  acc.wait_st();
}

// Add this thread's accumulators to d_twiddle (one 16-byte vector reduction per 2x2 block).
template <typename ACC>
BFLY_HD void bw3_flush(const Bw3Params& p, const ACC& acc, int stack, int pbase, int tid) {
  float* dtw = p.b.dtw[0] + (int64_t)stack * p.b.tw_stack[0];
  for (int j = 0; j < p.b.nsg; ++j) {
    const Bw3Sg& s = p.sg[j];
    const int col0 = p.b.panel.col(pbase, bw3_unit_local(s, tid));
    float ar[32];
    acc.wait_st();
    acc.ld32(j * 64 + 32, ar);
    acc.wait_ld();
    for (int k = 0; k < s.nst; ++k) {
      uint32_t off[16];
      bw3_tw_offsets(s, k, col0, off);
      // regroup into 2x2 blocks: entries whose offsets share a block (offset / 4)
      const float* v = ar + k * 16;
      if (s.kind[k] < 2) {
        for (int pp = 0; pp < 2; ++pp)
          for (int h = 0; h < 2; ++h) {  // left / right column of the pair
            float blk[4];
            for (int e = 0; e < 4; ++e) blk[e] = v[pp * 8 + 2 * e + h];
            atomic_add_block(dtw + (off[pp * 8 + h] & ~3u), blk);
          }
      } else {
        for (int m = 0; m < 4; ++m) {
          const float blk[4] = {v[m * 4 + 0], v[m * 4 + 2], v[m * 4 + 3], v[m * 4 + 1]};
          atomic_add_block(dtw + (off[m * 4] & ~3u), blk);
        }
      }
    }
  }
}

// shared memory of one CTA: (nsg + 1) tiles of five rows, then the unit table (16 bytes per
// sub-group and thread) and the per-sub-group dispatch words
BFLY_HD size_t bw3_tile_bytes(const Bw3Params& p) { return (size_t)(p.b.nsg + 1) * kBw3TileBytes; }
BFLY_HD size_t bw3_smem_bytes(const Bw3Params& p) {
  return bw3_tile_bytes(p) + ((size_t)p.b.nsg * kBw3Threads * 4 + 8) * sizeof(uint32_t);
}

}  // namespace bfly
