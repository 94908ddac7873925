// Backward phase, second generation: the same twiddle-stationary-accumulator scheme as
// bfly_core.h's backward, restructured so that two CTAs share an SM.
//
//  * The twiddles and the gradient accumulators of all sub-groups (up to four) do not live in
//    registers: each thread keeps them in its private slice of TENSOR MEMORY (TMEM, 256 KB per
//    SM on sm_100, otherwise unused by this library) and pulls the 16 twiddles and 16
//    accumulators of the sub-group it is working on into registers with one tcgen05.ld each,
//    pushing the accumulators back with one tcgen05.st.  That cuts the register need to under
//    100 per thread and keeps the twiddles one short hop away (no L2 latency per step).
//  * Sub-group steps are a runtime loop over one generic routine per stage pattern (no
//    per-sub-group code copies): the hot code is a few KB.
//  * A batch is four rows, all in flight per thread (no row loop); the two CTAs of an SM
//    overlap each other's load / barrier / store latencies.
//
// On the host (test emulator) the accumulator store is a plain array.
#pragma once
#include "bfly_core.h"

namespace bfly {

constexpr int kBw2Rows = 4;  // rows per batch
#ifndef BFLY_BW2_UNR
#define BFLY_BW2_UNR 2
#endif
constexpr int kBw2Unr = BFLY_BW2_UNR;  // rows a thread keeps in flight in a reverse step

// ---------------------------------------------------------------- accumulator store
template <typename T, int KW> struct AccStore {
  static constexpr int N = BwTwn<KW>::value;               // accumulators (elements of T) per sub-group
  static constexpr int NF = N * (int)(sizeof(T) / 4);      // 32-bit columns per sub-group
  // a thread's 128 columns: accumulators of sub-group j at j * NF, its twiddles at kTwBase + j * NF
  // (four sub-groups of 16 columns for float, two of 32 for complex)
  static constexpr int kTwBase = 64;
  static_assert(NF <= 32, "a sub-group's accumulators must fit a quarter of the thread's columns");
#if defined(__CUDA_ARCH__)
  uint32_t taddr;  // TMEM address (lane << 16 | column) of this thread's first column
  __device__ __forceinline__ void ld_tw(int j, T* tw) const { ld_at(kTwBase + j * NF, tw); }
  __device__ __forceinline__ void st_tw(int j, const T* tw) const { st_at(kTwBase + j * NF, tw); }
  __device__ __forceinline__ void ld(int j, T* acc) const { ld_at(j * NF, acc); }
  __device__ __forceinline__ void st(int j, const T* acc) const { st_at(j * NF, acc); }
  __device__ __forceinline__ void ld_at(int col, T* acc) const {
    float* r = reinterpret_cast<float*>(acc);
    const uint32_t a = taddr + (uint32_t)col;
    if constexpr (NF == 32) {
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
          "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
          : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]),
            "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]), "=f"(r[16]),
            "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]), "=f"(r[24]),
            "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
          : "r"(a) : "memory");
    } else if constexpr (NF == 16) {
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
          : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]),
            "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15])
          : "r"(a) : "memory");
    } else if constexpr (NF == 8) {
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                   : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7])
                   : "r"(a) : "memory");
    } else {
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]) : "r"(a) : "memory");
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  }
  __device__ __forceinline__ void st_at(int col, const T* acc) const {
    const float* r = reinterpret_cast<const float*>(acc);
    const uint32_t a = taddr + (uint32_t)col;
    if constexpr (NF == 32) {
      asm volatile(
          "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
          "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
          ::"r"(a), "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]), "f"(r[8]), "f"(r[9]),
            "f"(r[10]), "f"(r[11]), "f"(r[12]), "f"(r[13]), "f"(r[14]), "f"(r[15]), "f"(r[16]), "f"(r[17]), "f"(r[18]),
            "f"(r[19]), "f"(r[20]), "f"(r[21]), "f"(r[22]), "f"(r[23]), "f"(r[24]), "f"(r[25]), "f"(r[26]), "f"(r[27]),
            "f"(r[28]), "f"(r[29]), "f"(r[30]), "f"(r[31]) : "memory");
    } else if constexpr (NF == 16) {
      asm volatile(
          "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
          ::"r"(a), "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]), "f"(r[8]), "f"(r[9]),
            "f"(r[10]), "f"(r[11]), "f"(r[12]), "f"(r[13]), "f"(r[14]), "f"(r[15]) : "memory");
    } else if constexpr (NF == 8) {
      asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                   ::"r"(a), "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]) : "memory");
    } else {
      asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};"
                   ::"r"(a), "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]) : "memory");
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
#else
  T* mem;  // 2 * kMaxSg * N elements: accumulators, then twiddles
  void ld(int j, T* acc) const { for (int e = 0; e < N; ++e) acc[e] = mem[j * N + e]; }
  void st(int j, const T* acc) const { for (int e = 0; e < N; ++e) mem[j * N + e] = acc[e]; }
  void ld_tw(int j, T* tw) const { for (int e = 0; e < N; ++e) tw[e] = mem[(kMaxSg + j) * N + e]; }
  void st_tw(int j, const T* tw) const { for (int e = 0; e < N; ++e) mem[(kMaxSg + j) * N + e] = tw[e]; }
#endif
};

// Per-thread, per-sub-group constants kept in shared memory (kBw2Meta 32-bit words per thread
// and sub-group):
//   meta[(j * nthr + tid) * 4 + m], m = 0..3: byte offset, from the start of the first snapshot
//     tile, of element m of the thread's unit in row 0 of snapshot tile j (swizzle applied); a
//     step fetches the four with one 16-byte load;
//   meta[nsg * nthr * 4 + (j * 2 + k) * nthr + tid], k = 0, 1: element offsets of the unit's
//     twiddles (used when the twiddles are fetched and when the accumulators are flushed).
constexpr int kBw2Meta = 6;

template <typename T, int KW>
BFLY_HD void bw2_build_meta(const BwParams<T>& p, uint32_t* meta, int pbase, int tid, int nthr) {
  constexpr int E = 1 << KW;
  constexpr int SZ = (int)sizeof(T);
  const int C = 1 << p.panel.logC;
  uint32_t* tws = meta + (size_t)p.nsg * nthr * 4;
  for (int j = 0; j < p.nsg; ++j) {
    const BwSg& sg = p.sg[j];
    const int lbase = deposit_unit(tid, sg.ubit, sg.nubits);
    const int col0 = p.panel.col(pbase, lbase);
    const int wg = p.panel.global_bit(sg.lbit);
    uint32_t t0 = 0, t1 = 0;
    if (sg.radix == 4) {
      t0 = sg.tw_off[0] + (uint32_t)delete_2bits(col0, wg) * 16u;
    } else {
      t0 = sg.tw_off[0] + (uint32_t)delete_bit(col0, wg + sg.q[0]) * 4u;
      if (KW > 1 && sg.nst > 1) t1 = sg.tw_off[1] + (uint32_t)delete_bit(col0, wg + sg.q[1]) * 4u;
    }
    const int a0 = swzT<T>(lbase);
    for (int m = 0; m < 4; ++m) {
      const int ms = (sg.swap12 && (m == 1 || m == 2)) ? 3 - m : m;  // register m holds element ms
      meta[(j * nthr + tid) * 4 + m] = m < E ? (uint32_t)(((a0 ^ sg.d[ms]) + j * kBw2Rows * C) * SZ) : 0u;
    }
    tws[(j * 2 + 0) * nthr + tid] = t0;
    tws[(j * 2 + 1) * nthr + tid] = t1;
  }
}

// Twiddles of sub-group j for this thread's unit, from global memory (L2).
template <typename T, int KW>
BFLY_HD void bw2_fetch_tw(const BwParams<T>& p, const uint32_t* meta, int j, int stack, int tid, int nthr, T* dst) {
  const BwSg& sg = p.sg[j];
  const uint32_t* tws = meta + (size_t)p.nsg * nthr * 4;
  const T* twp = p.tw[sg.which] + (int64_t)stack * p.tw_stack[sg.which];
  const uint32_t t0 = tws[(j * 2 + 0) * nthr + tid];
  if (sg.radix == 4) {
    if constexpr (KW == 2) load_tw<T, 16>(dst, twp + t0);
  } else {
    const int wg = p.panel.global_bit(sg.lbit);
#pragma unroll
    for (int pp = 0; pp < (1 << (KW - 1)); ++pp) load_tw<T, 4>(dst + pp * 4, twp + t0 + (uint32_t)((pp << wg) * 4));
    if constexpr (KW > 1) {
      if (sg.nst > 1) {
        const uint32_t t1 = tws[(j * 2 + 1) * nthr + tid];
#pragma unroll
        for (int pp = 0; pp < (1 << (KW - 1)); ++pp)
          load_tw<T, 4>(dst + (1 << (KW - 1)) * 4 + pp * 4, twp + t1 + (uint32_t)((pp << wg) * 4));
      }
    }
  }
}

// Load / store the thread's unit of one tile row: a[m] are the addresses of its elements in
// row 0 of the tile (only a[0] is used on the 16-byte path), IMM the row's byte offset.
template <typename T, int KW, bool VEC, int IMM>
BFLY_HD void bw2_unit_ld(const smaddr_t* a, smaddr_t ro, T* v) {
  constexpr int E = 1 << KW;
  constexpr int V = Vec16<T>::N;
  if constexpr (VEC && E >= V) {
#pragma unroll
    for (int h = 0; h < E / V; ++h) sm_ld16<IMM>(a[h * V] + ro, v + h * V);
  } else {
#pragma unroll
    for (int m = 0; m < E; ++m) sm_ld<IMM>(a[m] + ro, v[m]);
  }
}
template <typename T, int KW, bool VEC, int IMM>
BFLY_HD void bw2_unit_st(const smaddr_t* a, smaddr_t ro, const T* v) {
  constexpr int E = 1 << KW;
  constexpr int V = Vec16<T>::N;
  if constexpr (VEC && E >= V) {
#pragma unroll
    for (int h = 0; h < E / V; ++h) sm_st16<IMM>(a[h * V] + ro, v + h * V);
  } else {
#pragma unroll
    for (int m = 0; m < E; ++m) sm_st<IMM>(a[m] + ro, v[m]);
  }
}

// One sub-group step over the four rows of a batch.
//   FORWARD: snapshot j -> stages -> snapshot j+1.   else: accumulate and propagate the gradient.
// o[m]: byte offsets of the unit's elements from the start of the first snapshot tile.
template <typename T, int KW, int LOGC, int PATID, bool VEC, bool FORWARD>
BFLY_HD void bw2_rows(const BwParams<T>& p, int j, const T* tw, T* acc, const uint32_t* o, T* __restrict__ smX,
                      T* __restrict__ smG) {
  constexpr int E = 1 << KW;
  constexpr int SZ = (int)sizeof(T);
  constexpr int R = kBw2Rows;
  constexpr int ROWB = LOGC > 0 ? (SZ << LOGC) : 0;   // compile-time row pitch
  constexpr int TILEB = LOGC > 0 ? R * ROWB : 0;      // compile-time tile pitch
  const int C = LOGC > 0 ? (1 << LOGC) : (1 << p.panel.logC);
  const smaddr_t xb = sm_addr(smX);
  smaddr_t ax[E];
#pragma unroll
  for (int m = 0; m < E; ++m) ax[m] = xb + (smaddr_t)o[m];
  auto rowoff = [&](int r) -> smaddr_t { return LOGC > 0 ? (smaddr_t)0 : (smaddr_t)((size_t)r * C * SZ); };
  if constexpr (FORWARD) {
    const smaddr_t tileoff = LOGC > 0 ? (smaddr_t)0 : (smaddr_t)((size_t)R * C * SZ);
    T v[R][E];
    static_for<0, R>([&](auto rc) {
      constexpr int r = decltype(rc)::value;
      bw2_unit_ld<T, KW, VEC, r * ROWB>(ax, rowoff(r), v[r]);
    });
    static_for<0, R>([&](auto rc) {
      constexpr int r = decltype(rc)::value;
      bw_apply_fw<T, KW, PATID>(v[r], tw);
      bw2_unit_st<T, KW, VEC, TILEB + r * ROWB>(ax, tileoff + rowoff(r), v[r]);
    });
  } else {
    // the gradient tile follows the nsg snapshot tiles
    const smaddr_t gdelta = (smaddr_t)((size_t)(p.nsg - j) * R * C * SZ);
    smaddr_t ag[E];
#pragma unroll
    for (int m = 0; m < E; ++m) ag[m] = ax[m] + gdelta;
    // kBw2Unr rows in flight (x, g and the recomputed intermediate of each are live together)
    static_for<0, R / kBw2Unr>([&](auto hc) {
      constexpr int h = decltype(hc)::value * kBw2Unr;
      T x[kBw2Unr][E], g[kBw2Unr][E];
      static_for<0, kBw2Unr>([&](auto rc) {
        constexpr int r = h + decltype(rc)::value;
        bw2_unit_ld<T, KW, VEC, r * ROWB>(ax, rowoff(r), x[r - h]);
        bw2_unit_ld<T, KW, VEC, r * ROWB>(ag, rowoff(r), g[r - h]);
      });
      static_for<0, kBw2Unr>([&](auto rc) {
        constexpr int r = h + decltype(rc)::value;
        bw_apply_bw<T, KW, PATID>(g[r - h], x[r - h], tw, acc);
        bw2_unit_st<T, KW, VEC, r * ROWB>(ag, rowoff(r), g[r - h]);
      });
    });
  }
  (void)smG;
}

// Code variant of a sub-group (BwSg::kase), resolved on the host by bw2_assign_kase (bfly_plan.h): 2 * pattern +
// vec, pattern as in bw_pattern().  Without 16-byte accesses, the patterns that differ only in
// which window bit comes first share code: the later-bit-first ones (2, 3, 5) run as (1, 0, 4)
// on a unit whose elements 1 and 2 trade places (BwSg::swap12; the element offsets come from a
// table, so the exchange is free), pair and twiddle numbering being the same under the swap.
template <typename T, int KW, int LOGC, bool FORWARD>
BFLY_HD void bw2_step(const BwParams<T>& p, int j, const T* tw, T* acc, const uint32_t* o, T* smX, T* smG) {
  const int kase = p.sg[j].kase;
#define BFLY_BW2_RUN(PAT, VEC) bw2_rows<T, KW, LOGC, PAT, VEC, FORWARD>(p, j, tw, acc, o, smX, smG)
  if constexpr (KW == 1) {
    if (kase & 1) BFLY_BW2_RUN(0, true);
    else BFLY_BW2_RUN(0, false);
  } else {
    if (kase == 2) { BFLY_BW2_RUN(1, false); return; }  // the common case first
    switch (kase) {
      case 0: BFLY_BW2_RUN(0, false); break;
      case 8: BFLY_BW2_RUN(4, false); break;
      case 12: BFLY_BW2_RUN(6, false); break;
      case 1: BFLY_BW2_RUN(0, true); break;
      case 3: BFLY_BW2_RUN(1, true); break;
      case 5: BFLY_BW2_RUN(2, true); break;
      case 7: BFLY_BW2_RUN(3, true); break;
      case 9: BFLY_BW2_RUN(4, true); break;
      case 11: BFLY_BW2_RUN(5, true); break;
      case 13: BFLY_BW2_RUN(6, true); break;
      default: break;
    }
  }
#undef BFLY_BW2_RUN
}

BFLY_HD void bw2_load_offsets(const uint32_t* meta, int j, int tid, int nthr, uint32_t* o) {
#if defined(__CUDA_ARCH__)
  const uint4 q = reinterpret_cast<const uint4*>(meta)[j * nthr + tid];
  o[0] = q.x; o[1] = q.y; o[2] = q.z; o[3] = q.w;
#else
  for (int m = 0; m < 4; ++m) o[m] = meta[(j * nthr + tid) * 4 + m];
#endif
}

// One forward-recompute step (sub-group j, 0 <= j <= nsg-2) of a batch for one thread.  A
// block-wide barrier must follow.
template <typename T, int KW, int LOGC>
BFLY_HD void bw2_fw_step(const BwParams<T>& p, const AccStore<T, KW>& accs, const uint32_t* meta, int j, T* smX,
                         T* smG, int tid, int nthr) {
  constexpr int N = BwTwn<KW>::value;
  T tw[N];
  accs.ld_tw(j, tw);
  uint32_t o[4];
  bw2_load_offsets(meta, j, tid, nthr, o);
  bw2_step<T, KW, LOGC, true>(p, j, tw, (T*)nullptr, o, smX, smG);
}

// One reverse step (sub-group j, nsg-1 >= j >= 0).  A block-wide barrier must follow.
template <typename T, int KW, int LOGC>
BFLY_HD void bw2_bw_step(const BwParams<T>& p, const AccStore<T, KW>& accs, const uint32_t* meta, int j, T* smX,
                         T* smG, int tid, int nthr) {
  constexpr int N = BwTwn<KW>::value;
  T tw[N], acc[N];
  accs.ld_tw(j, tw);
  accs.ld(j, acc);
  uint32_t o[4];
  bw2_load_offsets(meta, j, tid, nthr, o);
  bw2_step<T, KW, LOGC, false>(p, j, tw, acc, o, smX, smG);
  accs.st(j, acc);
}

// Per-thread set-up: zero accumulators, and the twiddles of the thread's unit in every sub-group
// from global memory into the private store (they stay there for the life of the CTA).
template <typename T, int KW>
BFLY_HD void bw2_init(const BwParams<T>& p, const AccStore<T, KW>& accs, const uint32_t* meta, int stack, int tid,
                      int nthr) {
  constexpr int N = BwTwn<KW>::value;
  T z[N];
#pragma unroll
  for (int e = 0; e < N; ++e) z[e] = Ops<T>::zero();
  for (int j = 0; j < p.nsg; ++j) {
    T tw[N];
#pragma unroll
    for (int e = 0; e < N; ++e) tw[e] = Ops<T>::zero();
    bw2_fetch_tw<T, KW>(p, meta, j, stack, tid, nthr, tw);
    accs.st_tw(j, tw);
    accs.st(j, z);
  }
}

// Add this thread's accumulators to d_twiddle.
template <typename T, int KW>
BFLY_HD void bw2_flush(const BwParams<T>& p, const AccStore<T, KW>& accs, const uint32_t* meta, int stack, int tid,
                       int nthr) {
  constexpr int N = BwTwn<KW>::value;
  for (int j = 0; j < p.nsg; ++j) {
    const BwSg& sg = p.sg[j];
    T acc[N];
    accs.ld(j, acc);
    T* dtw = p.dtw[sg.which] + (int64_t)stack * p.tw_stack[sg.which];
    const uint32_t* tws = meta + (size_t)p.nsg * nthr * 4;
    const uint32_t t0 = tws[(j * 2 + 0) * nthr + tid];
    if (sg.radix == 4) {
      if constexpr (KW == 2) {
#pragma unroll
        for (int b = 0; b < 4; ++b) atomic_add_block(dtw + t0 + b * 4, acc + b * 4);
      }
    } else {
      const int wg = p.panel.global_bit(sg.lbit);
      const uint32_t t1 = tws[(j * 2 + 1) * nthr + tid];
#pragma unroll
      for (int s = 0; s < KW; ++s) {
        if (s < sg.nst) {
#pragma unroll
          for (int pp = 0; pp < (1 << (KW - 1)); ++pp)
            atomic_add_block(dtw + (s == 0 ? t0 : t1) + (uint32_t)((pp << wg) * 4), acc + s * (1 << (KW - 1)) * 4 + pp * 4);
        }
      }
    }
  }
}

// shared memory of one CTA: (nsg + 1) tiles of four rows, then the meta table
template <typename T> BFLY_HD size_t bw2_tile_bytes(const BwParams<T>& p) {
  return ((size_t)(p.nsg + 1) * kBw2Rows * sizeof(T)) << p.panel.logC;
}
template <typename T> BFLY_HD size_t bw2_smem_bytes(const BwParams<T>& p, int nthr) {
  return bw2_tile_bytes(p) + (size_t)p.nsg * kBw2Meta * nthr * sizeof(uint32_t);
}

}  // namespace bfly
