// Tile routines of the butterfly multiply kernels, written per thread: every routine
// takes the thread index and does exactly the work one CUDA thread does between two
// block-wide barriers.  The __global__ kernels call them with threadIdx.x; the
// test-suite's host emulator calls them in a loop over all thread indices, which
// checks the whole index arithmetic (panels, unit decomposition, twiddle addressing,
// padding and slicing) on a machine without a GPU.
#pragma once
#include "bfly_types.h"

namespace bfly {

// Scatter the bits of unit index u to the local bit positions listed in ubit.
BFLY_HD int deposit_unit(int u, const uint8_t* ubit, int nubits) {
  int l = 0;
#pragma unroll 1
  for (int j = 0; j < nubits; ++j) l |= ((u >> j) & 1) << ubit[j];
  return l;
}

template <typename T> struct Vec16 {};  // 16-byte global access
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<cf> { static constexpr int N = 2; };

#if defined(__CUDA_ARCH__)
__device__ __forceinline__ void unpack16(const float4& q, float* v) { v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
__device__ __forceinline__ void unpack16(const float4& q, cf* v) { v[0] = cf{q.x, q.y}; v[1] = cf{q.z, q.w}; }
__device__ __forceinline__ float4 pack16(const float* v) { return make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ float4 pack16(const cf* v) { return make_float4(v[0].re, v[0].im, v[1].re, v[1].im); }
#endif

// ------------------------------------------------------------------ tile load / store

// Copy rows [row0, row0+R) x panel columns from global memory into the swizzled tile.
// Columns >= ncols and rows >= B read as zero.
template <typename T>
BFLY_HD void tile_load(const T* __restrict__ src, int64_t sB, int64_t sS, int ncols, int B, int stack,
                       int row0, int R, const Panel& pn, int pbase, bool vec, T* __restrict__ sm,
                       int tid, int nthr) {
  constexpr int SW = SwBits<T>::value;
  constexpr int V = Vec16<T>::N;
  const int logC = pn.logC;
  const int C = 1 << logC;
  if (vec && pn.lseg >= 2 && C >= V) {
    const int per_row = C / V;
    for (int e = tid; e < R * per_row; e += nthr) {
      const int r = e / per_row;
      const int l = (e - r * per_row) * V;
      const int row = row0 + r;
      const int col = pn.col(pbase, l);
      T v[V];
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] = Ops<T>::zero();
      if (row < B) {
        const T* p = src + (int64_t)row * sB + (int64_t)stack * sS + col;
        if (col + V <= ncols) {
#if defined(__CUDA_ARCH__)
          unpack16(*reinterpret_cast<const float4*>(p), v);
#else
          for (int j = 0; j < V; ++j) v[j] = p[j];
#endif
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j)
            if (col + j < ncols) v[j] = p[j];
        }
      }
#pragma unroll
      for (int j = 0; j < V; ++j) sm[r * C + swz<SW>(l + j)] = v[j];
    }
  } else {
    for (int e = tid; e < R * C; e += nthr) {
      const int r = e >> logC;
      const int l = e & (C - 1);
      const int row = row0 + r;
      const int col = pn.col(pbase, l);
      T v = Ops<T>::zero();
      if (row < B && col < ncols) v = src[(int64_t)row * sB + (int64_t)stack * sS + col];
      sm[r * C + swz<SW>(l)] = v;
    }
  }
}

// Copy the tile back to global memory; columns >= ncols and rows >= B are not written.
template <typename T>
BFLY_HD void tile_store(T* __restrict__ dst, int64_t sB, int64_t sS, int ncols, int B, int stack, int row0,
                        int R, const Panel& pn, int pbase, bool vec, const T* __restrict__ sm, int tid,
                        int nthr) {
  constexpr int SW = SwBits<T>::value;
  constexpr int V = Vec16<T>::N;
  const int logC = pn.logC;
  const int C = 1 << logC;
  if (vec && pn.lseg >= 2 && C >= V) {
    const int per_row = C / V;
    for (int e = tid; e < R * per_row; e += nthr) {
      const int r = e / per_row;
      const int l = (e - r * per_row) * V;
      const int row = row0 + r;
      if (row >= B) continue;
      const int col = pn.col(pbase, l);
      if (col >= ncols) continue;
      T v[V];
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] = sm[r * C + swz<SW>(l + j)];
      T* p = dst + (int64_t)row * sB + (int64_t)stack * sS + col;
      if (col + V <= ncols) {
#if defined(__CUDA_ARCH__)
        *reinterpret_cast<float4*>(p) = pack16(v);
#else
        for (int j = 0; j < V; ++j) p[j] = v[j];
#endif
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j)
          if (col + j < ncols) p[j] = v[j];
      }
    }
  } else {
    for (int e = tid; e < R * C; e += nthr) {
      const int r = e >> logC;
      const int l = e & (C - 1);
      const int row = row0 + r;
      const int col = pn.col(pbase, l);
      if (row < B && col < ncols) dst[(int64_t)row * sB + (int64_t)stack * sS + col] = sm[r * C + swz<SW>(l)];
    }
  }
}

// ------------------------------------------------------------------ butterfly stages on a register window

// Radix-2 stage on bit Q of a 2^K-element register window.  tw holds, per pair p,
// (t00, t01, t10, t11).
template <typename T, int K, int Q>
BFLY_HD void r2_stage_fw(T* v, const T* tw) {
#pragma unroll
  for (int p = 0; p < (1 << (K - 1)); ++p) {
    const int m0 = ((p >> Q) << (Q + 1)) | (p & ((1 << Q) - 1));
    const int m1 = m0 | (1 << Q);
    const T x0 = v[m0], x1 = v[m1];
    v[m0] = Ops<T>::madd2(tw[p * 4 + 0], x0, tw[p * 4 + 1], x1);
    v[m1] = Ops<T>::madd2(tw[p * 4 + 3], x1, tw[p * 4 + 2], x0);
  }
}

// Radix-4 stage on bits [Q, Q+2) of the window.  tw holds, per quad p, a row-major 4x4.
template <typename T, int K, int Q>
BFLY_HD void r4_stage_fw(T* v, const T* tw) {
#pragma unroll
  for (int p = 0; p < (1 << (K - 2)); ++p) {
    const int m0 = ((p >> Q) << (Q + 2)) | (p & ((1 << Q) - 1));
    T x[4], y[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = v[m0 | (j << Q)];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      T a = Ops<T>::mul(tw[p * 16 + i * 4 + 0], x[0]);
#pragma unroll
      for (int j = 1; j < 4; ++j) a = Ops<T>::fmadd(a, tw[p * 16 + i * 4 + j], x[j]);
      y[i] = a;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) v[m0 | (i << Q)] = y[i];
  }
}

template <typename T, int N>
BFLY_HD void load_tw(T* dst, const T* __restrict__ src) {
#if defined(__CUDA_ARCH__)
  constexpr int V = Vec16<T>::N;
#pragma unroll
  for (int j = 0; j < N / V; ++j) unpack16(__ldg(reinterpret_cast<const float4*>(src) + j), dst + j * V);
#else
  for (int j = 0; j < N; ++j) dst[j] = src[j];
#endif
}

template <typename T, int K, int PAT, int S>
BFLY_HD void fw_apply_stage(T* v, const T* tw) {
  if constexpr (PAT == kR2Inc) r2_stage_fw<T, K, S>(v, tw);
  if constexpr (PAT == kR2Dec) r2_stage_fw<T, K, K - 1 - S>(v, tw);
  if constexpr (PAT == kR4Inc) r4_stage_fw<T, K, 2 * S>(v, tw);
  if constexpr (PAT == kR4Dec) r4_stage_fw<T, K, K - 2 - 2 * S>(v, tw);
}

// One group of the forward kernel applied in place to the R rows of a tile.
template <typename T, int K, int PAT>
BFLY_HD void fw_group(const FwParams<T>& p, const FwGroup& g, T* __restrict__ sm, int R, int stack,
                      int pbase, int tid, int nthr) {
  constexpr int SW = SwBits<T>::value;
  constexpr int E = 1 << K;
  constexpr bool R4 = (PAT >= 2);
  constexpr int NST = R4 ? K / 2 : K;
  constexpr int PER = R4 ? E * 4 : E * 2;  // twiddle scalars of one stage for one unit
  const Panel& pn = p.panel;
  const int C = 1 << pn.logC;
  const int U = C >> K;
  int u0, ustep, r0, rstep;
  if (U >= nthr) {
    u0 = tid; ustep = nthr; r0 = 0; rstep = 1;
  } else {
    u0 = tid & (U - 1); ustep = U; r0 = tid / U; rstep = nthr / U;
  }
  const int lbit = g.lbit;
  const int wg = pn.global_bit(lbit);
  const T* twbase = p.tw[g.which] + (int64_t)stack * p.tw_stack[g.which];
  for (int u = u0; u < U; u += ustep) {
    const int lbase = deposit_unit(u, g.ubit, g.nubits);
    const int col0 = pn.col(pbase, lbase);
    int addr[E];
#pragma unroll
    for (int m = 0; m < E; ++m) addr[m] = swz<SW>(lbase | (m << lbit));
    T tw[NST * PER];
#pragma unroll
    for (int s = 0; s < NST; ++s) {
      if constexpr (!R4) {
        const int q = (PAT == kR2Inc) ? s : K - 1 - s;
        const int ibase = delete_bit(col0, wg + q);
#pragma unroll
        for (int pp = 0; pp < E / 2; ++pp)
          load_tw<T, 4>(tw + s * PER + pp * 4, twbase + g.tw_off[s] + (int64_t)(ibase + (pp << wg)) * 4);
      } else {
        const int q = (PAT == kR4Inc) ? 2 * s : K - 2 - 2 * s;
        const int ibase = delete_2bits(col0, wg + q);
#pragma unroll
        for (int pp = 0; pp < E / 4; ++pp)
          load_tw<T, 16>(tw + s * PER + pp * 16, twbase + g.tw_off[s] + (int64_t)(ibase + (pp << wg)) * 16);
      }
    }
    for (int r = r0; r < R; r += rstep) {
      T* row = sm + r * C;
      T v[E];
#pragma unroll
      for (int m = 0; m < E; ++m) v[m] = row[addr[m]];
      if constexpr (NST > 0) fw_apply_stage<T, K, PAT, 0>(v, tw + 0 * PER);
      if constexpr (NST > 1) fw_apply_stage<T, K, PAT, 1>(v, tw + 1 * PER);
      if constexpr (NST > 2) fw_apply_stage<T, K, PAT, 2>(v, tw + 2 * PER);
      if constexpr (NST > 3) fw_apply_stage<T, K, PAT, 3>(v, tw + 3 * PER);
#pragma unroll
      for (int m = 0; m < E; ++m) row[addr[m]] = v[m];
    }
  }
}

// Dispatch on the (uniform) window width and pattern of a group.
template <typename T>
BFLY_HD void fw_group_dispatch(const FwParams<T>& p, const FwGroup& g, T* sm, int R, int stack, int pbase,
                               int tid, int nthr) {
  const int K = g.K, pat = g.pattern;
  if (K == 1) { fw_group<T, 1, kR2Inc>(p, g, sm, R, stack, pbase, tid, nthr); return; }
  if (K == 2) {
    if (pat == kR2Inc) fw_group<T, 2, kR2Inc>(p, g, sm, R, stack, pbase, tid, nthr);
    else if (pat == kR2Dec) fw_group<T, 2, kR2Dec>(p, g, sm, R, stack, pbase, tid, nthr);
    else fw_group<T, 2, kR4Inc>(p, g, sm, R, stack, pbase, tid, nthr);
    return;
  }
  if (K == 3) {
    if (pat == kR2Inc) fw_group<T, 3, kR2Inc>(p, g, sm, R, stack, pbase, tid, nthr);
    else fw_group<T, 3, kR2Dec>(p, g, sm, R, stack, pbase, tid, nthr);
    return;
  }
  if constexpr (sizeof(T) == 4) {  // 4-bit windows only for 4-byte elements (register budget)
    if (K == 4) {
      if (pat == kR2Inc) fw_group<T, 4, kR2Inc>(p, g, sm, R, stack, pbase, tid, nthr);
      else if (pat == kR2Dec) fw_group<T, 4, kR2Dec>(p, g, sm, R, stack, pbase, tid, nthr);
      else if (pat == kR4Inc) fw_group<T, 4, kR4Inc>(p, g, sm, R, stack, pbase, tid, nthr);
      else fw_group<T, 4, kR4Dec>(p, g, sm, R, stack, pbase, tid, nthr);
    }
  }
}

// Tile decomposition of the forward kernel: tile -> (row tile, stack, panel).  Stacks of
// one row tile are adjacent so that a stack-broadcast input is re-read from L2.
template <typename T>
BFLY_HD void fw_tile_coords(const FwParams<T>& p, int64_t tile, int& row0, int& stack, int& pbase) {
  const int np = 1 << p.panel.npanels_log;
  const int pi = (int)(tile % np);
  const int64_t t2 = tile / np;
  stack = (int)(t2 % p.S);
  row0 = (int)(t2 / p.S) * p.R;
  pbase = p.panel.base(pi);
}
template <typename T> BFLY_HD int64_t fw_num_tiles(const FwParams<T>& p) {
  return (int64_t)((p.B + p.R - 1) / p.R) * p.S * (1 << p.panel.npanels_log);
}

// ------------------------------------------------------------------ backward phase

// Per-thread state of a backward phase: the twiddles of the thread's unit in every
// sub-group and the matching gradient accumulators.  They live in registers for the
// whole kernel (all loops over them are fully unrolled with constant indices).
// KW = window bits: a unit has 2^KW elements; TWN = twiddle scalars per unit and sub-group.
template <int KW> struct BwTwn { static constexpr int value = (KW == 2) ? 16 : 4; };
template <typename T, int KW, int NSG> struct BwState {
  T tw[NSG][BwTwn<KW>::value];
  T acc[NSG][BwTwn<KW>::value];
};

// Radix-2 stage with a runtime bit offset q on a 2^KW-element window.
template <typename T, int KW>
BFLY_HD void r2_fw_rt(T* v, const T* tw, int q) {
  if constexpr (KW == 1) {
    r2_stage_fw<T, 1, 0>(v, tw);
  } else {
    if (q == 0) r2_stage_fw<T, 2, 0>(v, tw);
    else r2_stage_fw<T, 2, 1>(v, tw);
  }
}

// Backward of a radix-2 stage: acc += g (x) conj(x) ; g <- T^H g
template <typename T, int KW, int Q>
BFLY_HD void r2_bw_q(T* g, const T* x, const T* tw, T* acc) {
#pragma unroll
  for (int p = 0; p < (1 << (KW - 1)); ++p) {
    const int m0 = ((p >> Q) << (Q + 1)) | (p & ((1 << Q) - 1));
    const int m1 = m0 | (1 << Q);
    const T g0 = g[m0], g1 = g[m1], x0 = x[m0], x1 = x[m1];
    acc[p * 4 + 0] = Ops<T>::acc_gxc(acc[p * 4 + 0], g0, x0);
    acc[p * 4 + 1] = Ops<T>::acc_gxc(acc[p * 4 + 1], g0, x1);
    acc[p * 4 + 2] = Ops<T>::acc_gxc(acc[p * 4 + 2], g1, x0);
    acc[p * 4 + 3] = Ops<T>::acc_gxc(acc[p * 4 + 3], g1, x1);
    g[m0] = Ops<T>::madd2c(tw[p * 4 + 0], g0, tw[p * 4 + 2], g1);
    g[m1] = Ops<T>::madd2c(tw[p * 4 + 3], g1, tw[p * 4 + 1], g0);
  }
}
template <typename T, int KW>
BFLY_HD void r2_bw_rt(T* g, const T* x, const T* tw, T* acc, int q) {
  if constexpr (KW == 1) {
    r2_bw_q<T, 1, 0>(g, x, tw, acc);
  } else {
    if (q == 0) r2_bw_q<T, 2, 0>(g, x, tw, acc);
    else r2_bw_q<T, 2, 1>(g, x, tw, acc);
  }
}

// Backward of a radix-4 stage on a 4-element window.
template <typename T>
BFLY_HD void r4_bw4(T* g, const T* x, const T* tw, T* acc) {
  T o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i * 4 + j] = Ops<T>::acc_gxc(acc[i * 4 + j], g[i], x[j]);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    T a = Ops<T>::mulc(tw[0 * 4 + j], g[0]);
#pragma unroll
    for (int i = 1; i < 4; ++i) a = Ops<T>::fmaddc(a, tw[i * 4 + j], g[i]);
    o[j] = a;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) g[j] = o[j];
}

// Unit and row assignment of a thread in the backward kernel (2^KW elements per unit).
struct BwThread {
  int u, r0, rstep;
};
template <int KW> BFLY_HD BwThread bw_thread(int logC, int tid, int nthr) {
  const int U = (1 << logC) >> KW;
  BwThread t;
  if (U >= nthr) {  // the planner guarantees U == nthr here
    t.u = tid; t.r0 = 0; t.rstep = 1;
  } else {
    t.u = tid & (U - 1); t.r0 = tid / U; t.rstep = nthr / U;
  }
  return t;
}

// Visit the twiddle blocks of the thread's unit in sub-group J: calls f(slot, element_offset,
// count) for every contiguous run of `count` twiddle scalars, `slot` being the index into
// the per-thread state array.
template <typename T, int KW, typename F>
BFLY_HD void bw_for_each_tw(const BwParams<T>& p, const BwSg& sg, int u, int stack, int pbase, F&& f) {
  const int lbase = deposit_unit(u, sg.ubit, sg.nubits);
  const int col0 = p.panel.col(pbase, lbase);
  const int wg = p.panel.global_bit(sg.lbit);
  const int64_t sbase = (int64_t)stack * p.tw_stack[sg.which];
  if (sg.radix == 4) {
    if constexpr (KW == 2) {
      const int i = delete_2bits(col0, wg);
      f(0, sbase + sg.tw_off[0] + (int64_t)i * 16, 16);
    }
  } else {
#pragma unroll
    for (int s = 0; s < KW; ++s) {
      if (s < sg.nst) {
        const int i = delete_bit(col0, wg + sg.q[s]);
#pragma unroll
        for (int pp = 0; pp < (1 << (KW - 1)); ++pp)
          f(s * (1 << (KW - 1)) * 4 + pp * 4, sbase + sg.tw_off[s] + (int64_t)(i + (pp << wg)) * 4, 4);
      }
    }
  }
}

template <typename T, int KW, int NSG>
BFLY_HD void bw_load_state(const BwParams<T>& p, BwState<T, KW, NSG>& st, int stack, int pbase, int tid,
                           int nthr) {
  const BwThread th = bw_thread<KW>(p.panel.logC, tid, nthr);
#pragma unroll
  for (int j = 0; j < NSG; ++j) {
#pragma unroll
    for (int e = 0; e < BwTwn<KW>::value; ++e) { st.tw[j][e] = Ops<T>::zero(); st.acc[j][e] = Ops<T>::zero(); }
    if (j < p.nsg) {
      const BwSg& sg = p.sg[j];
      const T* twp = p.tw[sg.which];
      T* dst = st.tw[j];
      bw_for_each_tw<T, KW>(p, sg, th.u, stack, pbase, [&](int slot, int64_t off, int cnt) {
        if (cnt == 16) load_tw<T, 16>(dst + slot, twp + off);
        else load_tw<T, 4>(dst + slot, twp + off);
      });
    }
  }
}

BFLY_HD void atomic_add_el(float* dst, float v) {
#if defined(__CUDA_ARCH__)
  atomicAdd(dst, v);
#else
  *dst += v;
#endif
}
BFLY_HD void atomic_add_el(cf* dst, cf v) {
  atomic_add_el(&dst->re, v.re);
  atomic_add_el(&dst->im, v.im);
}

template <typename T, int KW, int NSG>
BFLY_HD void bw_flush_state(const BwParams<T>& p, const BwState<T, KW, NSG>& st, int stack, int pbase,
                            int tid, int nthr) {
  const BwThread th = bw_thread<KW>(p.panel.logC, tid, nthr);
#pragma unroll
  for (int j = 0; j < NSG; ++j) {
    if (j < p.nsg) {
      const BwSg& sg = p.sg[j];
      T* dtw = p.dtw[sg.which];
      const T* src = st.acc[j];
      bw_for_each_tw<T, KW>(p, sg, th.u, stack, pbase, [&](int slot, int64_t off, int cnt) {
#pragma unroll
        for (int e = 0; e < 16; ++e)
          if (e < cnt) atomic_add_el(dtw + off + e, src[slot + e]);
      });
    }
  }
}

// Forward recompute of sub-group j: reads the thread's unit of every row from snapshot j,
// applies the sub-group's stages, writes snapshot j+1.
template <typename T, int KW, int NSG>
BFLY_HD void bw_sg_forward(const BwParams<T>& p, const BwState<T, KW, NSG>& st, int j, T* __restrict__ smX,
                           int R, int tid, int nthr) {
  constexpr int SW = SwBits<T>::value;
  constexpr int E = 1 << KW;
  const BwSg& sg = p.sg[j];
  const int C = 1 << p.panel.logC;
  const BwThread th = bw_thread<KW>(p.panel.logC, tid, nthr);
  const int lbase = deposit_unit(th.u, sg.ubit, sg.nubits);
  int addr[E];
#pragma unroll
  for (int m = 0; m < E; ++m) addr[m] = swz<SW>(lbase | (m << sg.lbit));
  const T* src = smX + (size_t)j * p.Rb * C;
  T* dst = smX + (size_t)(j + 1) * p.Rb * C;
  for (int r = th.r0; r < R; r += th.rstep) {
    T v[E];
#pragma unroll
    for (int m = 0; m < E; ++m) v[m] = src[r * C + addr[m]];
    if constexpr (KW == 2) {
      if (sg.radix == 4) {
        r4_stage_fw<T, 2, 0>(v, st.tw[j]);
      } else {
        r2_fw_rt<T, 2>(v, st.tw[j], sg.q[0]);
        if (sg.nst > 1) r2_fw_rt<T, 2>(v, st.tw[j] + 8, sg.q[1]);
      }
    } else {
      r2_fw_rt<T, 1>(v, st.tw[j], 0);
    }
#pragma unroll
    for (int m = 0; m < E; ++m) dst[r * C + addr[m]] = v[m];
  }
}

// Backward of sub-group j: reads snapshot j and the gradient tile, accumulates the twiddle
// gradient of the thread's unit and replaces the gradient in place.
template <typename T, int KW, int NSG>
BFLY_HD void bw_sg_backward(const BwParams<T>& p, BwState<T, KW, NSG>& st, int j, const T* __restrict__ smX,
                            T* __restrict__ smG, int R, int tid, int nthr) {
  constexpr int SW = SwBits<T>::value;
  constexpr int E = 1 << KW;
  const BwSg& sg = p.sg[j];
  const int C = 1 << p.panel.logC;
  const BwThread th = bw_thread<KW>(p.panel.logC, tid, nthr);
  const int lbase = deposit_unit(th.u, sg.ubit, sg.nubits);
  int addr[E];
#pragma unroll
  for (int m = 0; m < E; ++m) addr[m] = swz<SW>(lbase | (m << sg.lbit));
  const T* src = smX + (size_t)j * p.Rb * C;
  for (int r = th.r0; r < R; r += th.rstep) {
    T x[E], g[E];
#pragma unroll
    for (int m = 0; m < E; ++m) { x[m] = src[r * C + addr[m]]; g[m] = smG[r * C + addr[m]]; }
    if constexpr (KW == 2) {
      if (sg.radix == 4) {
        r4_bw4<T>(g, x, st.tw[j], st.acc[j]);
      } else if (sg.nst == 1) {
        r2_bw_rt<T, 2>(g, x, st.tw[j], st.acc[j], sg.q[0]);
      } else {
        T x1[E];
#pragma unroll
        for (int m = 0; m < E; ++m) x1[m] = x[m];
        r2_fw_rt<T, 2>(x1, st.tw[j], sg.q[0]);
        r2_bw_rt<T, 2>(g, x1, st.tw[j] + 8, st.acc[j] + 8, sg.q[1]);
        r2_bw_rt<T, 2>(g, x, st.tw[j], st.acc[j], sg.q[0]);
      }
    } else {
      r2_bw_rt<T, 1>(g, x, st.tw[j], st.acc[j], 0);
    }
#pragma unroll
    for (int m = 0; m < E; ++m) smG[r * C + addr[m]] = g[m];
  }
}

// CTA decomposition of the backward kernel: cta -> (panel, stack, row slice).
template <typename T>
BFLY_HD void bw_cta_coords(const BwParams<T>& p, int cta, int& pbase, int& stack, int& row_begin, int& row_end) {
  const int np = 1 << p.panel.npanels_log;
  const int pi = cta % np;
  const int t2 = cta / np;
  stack = t2 % p.S;
  const int slice = t2 / p.S;
  pbase = p.panel.base(pi);
  row_begin = slice * p.rows_per_cta;
  row_end = row_begin + p.rows_per_cta;
  if (row_end > p.B) row_end = p.B;
}
template <typename T> BFLY_HD int bw_num_ctas(const BwParams<T>& p) {
  return (1 << p.panel.npanels_log) * p.S * p.nslices;
}

// The whole per-CTA body of a backward phase between barriers is:
//   load state; for each row batch { load X0,G | sync | sg fwd 0..nsg-2 (sync each) |
//   sg bwd nsg-1..0 (sync each) | store G | sync }; flush state.
// `Sync` is __syncthreads() on the device; the host emulator runs each step for all
// threads before the next.

}  // namespace bfly
