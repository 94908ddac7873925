// Tile routines of the butterfly multiply kernels, written per thread: every routine
// takes the thread index and does exactly the work one CUDA thread does between two
// block-wide barriers.  The __global__ kernels call them with threadIdx.x; the
// test-suite's host emulator calls them in a loop over all thread indices, which
// checks the whole index arithmetic (panels, unit decomposition, twiddle addressing,
// padding and slicing) on a machine without a GPU.
#pragma once
#include <type_traits>

#include "bfly_types.h"

namespace bfly {

// Compile-time loop: f(std::integral_constant<int, J>) for J = 0 .. N-1.
template <int J, int N, typename F>
BFLY_HD void static_for(F&& f) {
  if constexpr (J < N) {
    f(std::integral_constant<int, J>{});
    static_for<J + 1, N>(f);
  }
}

// ------------------------------------------------------------------ shared-memory access
//
// Tile addresses are byte addresses in the shared state space (32-bit on the device, so
// that address arithmetic is one integer add and row offsets fold into the instruction's
// immediate field); on the host they are plain pointers.
#if defined(__CUDA_ARCH__)
typedef uint32_t smaddr_t;
__device__ __forceinline__ smaddr_t sm_addr(const void* p) { return (smaddr_t)__cvta_generic_to_shared(p); }
template <int IMM> __device__ __forceinline__ void sm_ld(smaddr_t a, float& v) {
  asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(a), "n"(IMM) : "memory");
}
template <int IMM> __device__ __forceinline__ void sm_ld(smaddr_t a, cf& v) {
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2+%3];" : "=f"(v.re), "=f"(v.im) : "r"(a), "n"(IMM) : "memory");
}
template <int IMM> __device__ __forceinline__ void sm_st(smaddr_t a, float v) {
  asm volatile("st.shared.f32 [%0+%1], %2;" ::"r"(a), "n"(IMM), "f"(v) : "memory");
}
template <int IMM> __device__ __forceinline__ void sm_st(smaddr_t a, cf v) {
  asm volatile("st.shared.v2.f32 [%0+%1], {%2, %3};" ::"r"(a), "n"(IMM), "f"(v.re), "f"(v.im) : "memory");
}
// 16-byte chunk = 4 floats or 2 complex
template <int IMM> __device__ __forceinline__ void sm_ld16(smaddr_t a, float* v) {
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4+%5];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(a), "n"(IMM) : "memory");
}
template <int IMM> __device__ __forceinline__ void sm_ld16(smaddr_t a, cf* v) {
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4+%5];"
               : "=f"(v[0].re), "=f"(v[0].im), "=f"(v[1].re), "=f"(v[1].im) : "r"(a), "n"(IMM) : "memory");
}
template <int IMM> __device__ __forceinline__ void sm_st16(smaddr_t a, const float* v) {
  asm volatile("st.shared.v4.f32 [%0+%1], {%2, %3, %4, %5};" ::"r"(a), "n"(IMM), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
}
template <int IMM> __device__ __forceinline__ void sm_st16(smaddr_t a, const cf* v) {
  asm volatile("st.shared.v4.f32 [%0+%1], {%2, %3, %4, %5};" ::"r"(a), "n"(IMM), "f"(v[0].re), "f"(v[0].im), "f"(v[1].re), "f"(v[1].im) : "memory");
}
#else
typedef uintptr_t smaddr_t;
inline smaddr_t sm_addr(const void* p) { return (smaddr_t)p; }
template <int IMM, typename T> inline void sm_ld(smaddr_t a, T& v) { v = *reinterpret_cast<const T*>(a + IMM); }
template <int IMM, typename T> inline void sm_st(smaddr_t a, T v) { *reinterpret_cast<T*>(a + IMM) = v; }
template <int IMM, typename T> inline void sm_ld16(smaddr_t a, T* v) {
  for (int i = 0; i < (int)(16 / sizeof(T)); ++i) v[i] = reinterpret_cast<const T*>(a + IMM)[i];
}
template <int IMM, typename T> inline void sm_st16(smaddr_t a, const T* v) {
  for (int i = 0; i < (int)(16 / sizeof(T)); ++i) reinterpret_cast<T*>(a + IMM)[i] = v[i];
}
#endif

#if defined(__CUDA_ARCH__)
__device__ __forceinline__ void unpack16(const float4& q, float* v) { v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
__device__ __forceinline__ void unpack16(const float4& q, cf* v) { v[0] = cf{q.x, q.y}; v[1] = cf{q.z, q.w}; }
#endif

// Scatter the bits of unit index u to the local bit positions listed in ubit.
BFLY_HD int deposit_unit(int u, const uint8_t* ubit, int nubits) {
  int l = 0;
#pragma unroll 1
  for (int j = 0; j < nubits; ++j) l |= ((u >> j) & 1) << ubit[j];
  return l;
}

// ------------------------------------------------------------------ tile load / store

// Generic copy of rows [row0, row0+R) x panel columns from global memory into the swizzled
// tile (any panel, any alignment).  Columns >= ncols and rows >= B read as zero.
template <typename T>
BFLY_HD void tile_load(const T* __restrict__ src, int64_t sB, int64_t sS, int ncols, int B, int stack,
                       int row0, int R, const Panel& pn, int pbase, T* __restrict__ sm, int tid, int nthr) {
  const int logC = pn.logC;
  const int C = 1 << logC;
  for (int e = tid; e < R * C; e += nthr) {
    const int r = e >> logC;
    const int l = e & (C - 1);
    const int row = row0 + r;
    const int col = pn.col(pbase, l);
    T v = Ops<T>::zero();
    if (row < B && col < ncols) v = src[(int64_t)row * sB + (int64_t)stack * sS + col];
    sm[r * C + swzT<T>(l)] = v;
  }
}

// Generic copy of the tile back to global memory; columns >= ncols and rows >= B are not written.
template <typename T>
BFLY_HD void tile_store(T* __restrict__ dst, int64_t sB, int64_t sS, int ncols, int B, int stack, int row0,
                        int R, const Panel& pn, int pbase, const T* __restrict__ sm, int tid, int nthr) {
  const int logC = pn.logC;
  const int C = 1 << logC;
  for (int e = tid; e < R * C; e += nthr) {
    const int r = e >> logC;
    const int l = e & (C - 1);
    const int row = row0 + r;
    const int col = pn.col(pbase, l);
    if (row < B && col < ncols) dst[(int64_t)row * sB + (int64_t)stack * sS + col] = sm[r * C + swzT<T>(l)];
  }
}

// Gather inside a tile row, staged through registers.  A thread owns the columns
// c_k = deposit(tid + k * nthr, colbit); tile_permute_plan packs, per owned column, (source column
// << 16 | own column) once per pass; then for every row all threads read their sources (times
// diag[source] when a diagonal is given), and after a barrier write their own columns.
template <typename T>
BFLY_HD int tile_permute_plan(int logC, const int32_t* __restrict__ perm, const uint8_t* colbit, int tid, int nthr, uint32_t* plan) {
  const int C = 1 << logC;
  int cnt = 0;
#pragma unroll
  for (int k = 0; k < kGlueSlots; ++k) {
    const int i = tid + k * nthr;
    if (i >= C) break;
    const int c = deposit_unit(i, colbit, logC);
    const int src = perm ? perm[c] : c;
    plan[k] = ((uint32_t)src << 16) | (uint32_t)c;
    cnt = k + 1;
  }
  return cnt;
}
template <typename T>
BFLY_HD void tile_permute_read(const T* __restrict__ sm, int r, int logC, const T* __restrict__ diag, const uint32_t* plan, int cnt, T* v) {
  const T* row = sm + ((size_t)r << logC);
#pragma unroll
  for (int k = 0; k < kGlueSlots; ++k) {  // fixed bound: plan and v stay in registers
    if (k >= cnt) break;
    const int src = (int)(plan[k] >> 16);
    T t = row[swzT<T>(src)];
    if (diag) t = Ops<T>::mul(t, diag[src]);
    v[k] = t;
  }
}
template <typename T>
BFLY_HD void tile_permute_write(T* __restrict__ sm, int r, int logC, const uint32_t* plan, int cnt, const T* v) {
  T* row = sm + ((size_t)r << logC);
#pragma unroll
  for (int k = 0; k < kGlueSlots; ++k) {
    if (k >= cnt) break;
    row[swzT<T>((int)(plan[k] & 0xffffu))] = v[k];
  }
}

// Diagonal without a gather: y[c] *= diag[c] in place, 16 bytes at a time; a thread keeps its
// columns' diagonal entries in registers over the rows of the tile.  No barrier needed inside.
template <typename T>
BFLY_HD void tile_scale_rows(T* __restrict__ sm, int R, int logC, const T* __restrict__ diag, int tid, int nthr) {
  constexpr int V = Vec16<T>::N, VL = Vec16<T>::LOG;
  const int C = 1 << logC;
  if (logC < VL) {
    for (int e = tid; e < R * C; e += nthr) {
      const int l = e & (C - 1);
      T* q = sm + (e >> logC) * C + swzT<T>(l);
      *q = Ops<T>::mul(*q, diag[l]);
    }
    return;
  }
  constexpr int kChunks = kGlueSlots / V;  // chunks per thread and row when C / nthr == kGlueSlots
  T d[kChunks][V];
#pragma unroll
  for (int k = 0; k < kChunks; ++k) {
    const int l = (tid + k * nthr) << VL;
    if (l >= C) break;
#pragma unroll
    for (int i = 0; i < V; ++i) d[k][i] = diag[l + i];
  }
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int k = 0; k < kChunks; ++k) {
      const int l = (tid + k * nthr) << VL;
      if (l >= C) break;
      T* q = sm + r * C + swzT<T>(l);  // the swizzle moves whole 16-byte chunks
      T v[V];
      sm_ld16<0>(sm_addr(q), v);
#pragma unroll
      for (int i = 0; i < V; ++i) v[i] = Ops<T>::mul(v[i], d[k][i]);
      sm_st16<0>(sm_addr(q), v);
    }
  }
}

// Column bits for the gather passes (FwGlue::colbit).  The lanes of a warp run over column bits
// 0, 4, 5, 6, 1: bits 4-6 are the ones the tile's swizzle folds into the bank bits, so consecutive
// lanes land in different banks both at their own column and at its bit-reversed image (the common
// gather).  Measured on B200 against lanes on bits 0-4: 0.40 vs 0.48 ms for an FFT of 16384 rows
// of 2048 complex64 with its bit-reversal; candidates chosen by a bank-conflict model of 8-byte
// accesses did worse than either.  Any choice is correct.
inline void glue_column_bits(int logC, uint8_t* colbit) {
  for (int j = 0; j < 16; ++j) colbit[j] = (uint8_t)j;
  if (logC < 7) return;
  const uint8_t lanes[5] = {0, 4, 5, 6, 1};
  int k = 0;
  for (int j = 0; j < 5; ++j) colbit[k++] = lanes[j];
  for (int b = 0; b < logC; ++b)
    if (b != 0 && b != 1 && b != 4 && b != 5 && b != 6) colbit[k++] = (uint8_t)b;
}

// Whole-row tiles of a complex product fed from / written to float32 rows (real part only).
BFLY_HD void tile_load_real(const float* __restrict__ src, int64_t sB, int64_t sS, int ncols, int B, int stack, int row0,
                            int R, int logC, cf* __restrict__ sm, int tid, int nthr) {
  const int C = 1 << logC;
  const bool vec = logC >= 2 && (ncols & 3) == 0 && ((sB | sS) & 3) == 0 && (((uintptr_t)src) & 15u) == 0;
  if (vec) {  // four floats per access: two 16-byte chunks of the complex tile, which the swizzle keeps 2 apart
    const int Q = C >> 2;
    for (int e = tid; e < R * Q; e += nthr) {
      const int r = e / Q, l = (e - r * Q) << 2;
      const int row = row0 + r;
      float f[4] = {0.f, 0.f, 0.f, 0.f};
      if (row < B && l < ncols) {
        const float* q = src + (int64_t)row * sB + (int64_t)stack * sS + l;
#if defined(__CUDA_ARCH__)
        const float4 t = *reinterpret_cast<const float4*>(q);
        f[0] = t.x; f[1] = t.y; f[2] = t.z; f[3] = t.w;
#else
        for (int i = 0; i < 4; ++i) f[i] = q[i];
#endif
      }
      cf* d = sm + r * C;
      const int a = swzT<cf>(l);
      d[a] = cf{f[0], 0.f}; d[a + 1] = cf{f[1], 0.f};
      d[a ^ 2] = cf{f[2], 0.f}; d[(a ^ 2) + 1] = cf{f[3], 0.f};
    }
    return;
  }
  for (int e = tid; e < R * C; e += nthr) {
    const int r = e >> logC, l = e & (C - 1);
    const int row = row0 + r;
    float v = 0.f;
    if (row < B && l < ncols) v = src[(int64_t)row * sB + (int64_t)stack * sS + l];
    sm[r * C + swzT<cf>(l)] = cf{v, 0.f};
  }
}
BFLY_HD void tile_store_real(float* __restrict__ dst, int64_t sB, int64_t sS, int ncols, int B, int stack, int row0, int R,
                             int logC, const cf* __restrict__ sm, int tid, int nthr) {
  const int C = 1 << logC;
  const bool vec = logC >= 2 && (ncols & 3) == 0 && ((sB | sS) & 3) == 0 && (((uintptr_t)dst) & 15u) == 0;
  if (vec) {
    const int Q = C >> 2;
    for (int e = tid; e < R * Q; e += nthr) {
      const int r = e / Q, l = (e - r * Q) << 2;
      const int row = row0 + r;
      if (row >= B || l >= ncols) continue;
      const cf* s_ = sm + r * C;
      const int a = swzT<cf>(l);
      float* q = dst + (int64_t)row * sB + (int64_t)stack * sS + l;
#if defined(__CUDA_ARCH__)
      *reinterpret_cast<float4*>(q) = make_float4(s_[a].re, s_[a + 1].re, s_[a ^ 2].re, s_[(a ^ 2) + 1].re);
#else
      q[0] = s_[a].re; q[1] = s_[a + 1].re; q[2] = s_[a ^ 2].re; q[3] = s_[(a ^ 2) + 1].re;
#endif
    }
    return;
  }
  for (int e = tid; e < R * C; e += nthr) {
    const int r = e >> logC, l = e & (C - 1);
    const int row = row0 + r;
    if (row < B && l < ncols) dst[(int64_t)row * sB + (int64_t)stack * sS + l] = sm[r * C + swzT<cf>(l)].re;
  }
}
// float products have no real / complex conversion; the overloads keep the kernel's code uniform
BFLY_HD void tile_load_real(const float*, int64_t, int64_t, int, int, int, int, int, int, float*, int, int) {}
BFLY_HD void tile_store_real(float*, int64_t, int64_t, int, int, int, int, int, int, const float*, int, int) {}

// 16-byte-chunk variants for aligned tensors and panels whose segments hold whole chunks.
// The swizzle moves whole chunks, so a chunk travels with one 16-byte access on both sides.
// On the device the load is asynchronous (cp.async, zero-filling what lies outside the
// tensor); tile_load_wait() must be called before the barrier that publishes the tile.
// Work split of a chunk copy: a thread owns the same chunk columns in every row it touches,
// so column mapping, range checks and swizzle are computed once per tile.
struct ChunkSplit {
  int nslot, c0, r0, rstep;
};
BFLY_HD ChunkSplit chunk_split(int lpr, int tid, int nthr) {
  ChunkSplit s;
  const int per_row = 1 << lpr;
  if (per_row >= nthr) {
    s.nslot = per_row / nthr; s.c0 = tid; s.r0 = 0; s.rstep = 1;
  } else {
    s.nslot = 1; s.c0 = tid & (per_row - 1); s.r0 = tid >> lpr; s.rstep = nthr >> lpr;
  }
  return s;
}

template <typename T>
BFLY_HD void tile_load_chunks(const T* __restrict__ src, int64_t sB, int64_t sS, int ncols, int B, int stack,
                              int row0, int R, const Panel& pn, int pbase, T* __restrict__ sm, int tid, int nthr) {
  constexpr int V = Vec16<T>::N;
  constexpr int VL = Vec16<T>::LOG;
  const int C = 1 << pn.logC;
  const T* base = src + (int64_t)stack * sS;
  const ChunkSplit cs = chunk_split(pn.logC - VL, tid, nthr);
  for (int s = 0; s < cs.nslot; ++s) {
    const int l = (cs.c0 + s * nthr) << VL;
    const int col = pn.col(pbase, l);
    int vcol = ncols - col;  // elements of this chunk that exist in a row of the tensor
    vcol = vcol < 0 ? 0 : (vcol > V ? V : vcol);
    T* d = sm + swzT<T>(l);
    const T* q0 = base + col;
    for (int r = cs.r0; r < R; r += cs.rstep) {
      const int row = row0 + r;
      const int valid = row < B ? vcol : 0;
      const T* q = valid ? q0 + (int64_t)row * sB : base;
#if defined(__CUDA_ARCH__)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sm_addr(d + r * C)), "l"(q), "r"(valid * (int)sizeof(T)) : "memory");
#else
      for (int i = 0; i < V; ++i) d[r * C + i] = i < valid ? q[i] : Ops<T>::zero();
#endif
    }
  }
}
BFLY_HD void tile_load_wait() {
#if defined(__CUDA_ARCH__)
  asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
#endif
}

template <typename T>
BFLY_HD void tile_store_chunks(T* __restrict__ dst, int64_t sB, int64_t sS, int ncols, int B, int stack, int row0,
                               int R, const Panel& pn, int pbase, const T* __restrict__ sm, int tid, int nthr) {
  constexpr int V = Vec16<T>::N;
  constexpr int VL = Vec16<T>::LOG;
  const int C = 1 << pn.logC;
  T* base = dst + (int64_t)stack * sS;
  const ChunkSplit cs = chunk_split(pn.logC - VL, tid, nthr);
  const int rend = (B - row0) < R ? (B - row0) : R;  // rows of the tile that exist
  for (int s = 0; s < cs.nslot; ++s) {
    const int l = (cs.c0 + s * nthr) << VL;
    const int col = pn.col(pbase, l);
    if (col >= ncols) continue;
    const T* sp = sm + swzT<T>(l);
    T* q0 = base + col;
    if (col + V <= ncols) {
      for (int r = cs.r0; r < rend; r += cs.rstep) {
        T* q = q0 + (int64_t)(row0 + r) * sB;
#if defined(__CUDA_ARCH__)
        *reinterpret_cast<float4*>(q) = *reinterpret_cast<const float4*>(sp + r * C);
#else
        for (int i = 0; i < V; ++i) q[i] = sp[r * C + i];
#endif
      }
    } else {
      for (int r = cs.r0; r < rend; r += cs.rstep)
        for (int i = 0; i < V; ++i)
          if (col + i < ncols) q0[(int64_t)(row0 + r) * sB + i] = sp[r * C + i];
    }
  }
}

// Chunk copies of a tile whose R rows all exist (row0 + R <= B): the common case, written so
// that one 16-byte move costs a handful of instructions (running pointers, no per-row range
// checks; what lies right of the tensor's last column is zero-filled on load, skipped on store).
template <typename T>
BFLY_HD void tile_load_rows(const T* __restrict__ src, int64_t sB, int64_t sS, int ncols, int stack, int row0,
                            int R, const Panel& pn, int pbase, T* __restrict__ sm, int tid, int nthr) {
  constexpr int V = Vec16<T>::N;
  constexpr int VL = Vec16<T>::LOG;
  constexpr int SZ = (int)sizeof(T);
  const int C = 1 << pn.logC;
  const ChunkSplit cs = chunk_split(pn.logC - VL, tid, nthr);
  const T* rowbase = src + (int64_t)stack * sS + (int64_t)(row0 + cs.r0) * sB;
  const int64_t qstep = (int64_t)cs.rstep * sB;
  const int dstep = cs.rstep * C;
  for (int s = 0; s < cs.nslot; ++s) {
    const int l = (cs.c0 + s * nthr) << VL;
    const int col = pn.col(pbase, l);
    int vcol = ncols - col;
    vcol = vcol < 0 ? 0 : (vcol > V ? V : vcol);
    const T* q = vcol ? rowbase + col : rowbase;
    T* d = sm + swzT<T>(l) + cs.r0 * C;
#if defined(__CUDA_ARCH__)
    smaddr_t da = sm_addr(d);
    const int bytes = vcol * SZ;
#pragma unroll 2
    for (int r = cs.r0; r < R; r += cs.rstep) {
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(da), "l"(q), "r"(bytes) : "memory");
      q += qstep;
      da += (smaddr_t)(dstep * SZ);
    }
#else
    for (int r = cs.r0; r < R; r += cs.rstep) {
      for (int i = 0; i < V; ++i) d[i] = i < vcol ? q[i] : Ops<T>::zero();
      q += qstep;
      d += dstep;
    }
#endif
  }
}

template <typename T>
BFLY_HD void tile_store_rows(T* __restrict__ dst, int64_t sB, int64_t sS, int ncols, int stack, int row0, int R,
                             const Panel& pn, int pbase, const T* __restrict__ sm, int tid, int nthr) {
  constexpr int V = Vec16<T>::N;
  constexpr int VL = Vec16<T>::LOG;
  const int C = 1 << pn.logC;
  const ChunkSplit cs = chunk_split(pn.logC - VL, tid, nthr);
  T* rowbase = dst + (int64_t)stack * sS + (int64_t)(row0 + cs.r0) * sB;
  const int64_t qstep = (int64_t)cs.rstep * sB;
  const int dstep = cs.rstep * C;
  for (int s = 0; s < cs.nslot; ++s) {
    const int l = (cs.c0 + s * nthr) << VL;
    const int col = pn.col(pbase, l);
    if (col >= ncols) continue;
    T* q = rowbase + col;
    const T* sp = sm + swzT<T>(l) + cs.r0 * C;
    if (col + V <= ncols) {
#pragma unroll 2
      for (int r = cs.r0; r < R; r += cs.rstep) {
#if defined(__CUDA_ARCH__)
        *reinterpret_cast<float4*>(q) = *reinterpret_cast<const float4*>(sp);
#else
        for (int i = 0; i < V; ++i) q[i] = sp[i];
#endif
        q += qstep;
        sp += dstep;
      }
    } else {
      for (int r = cs.r0; r < R; r += cs.rstep) {
        for (int i = 0; i < V; ++i)
          if (col + i < ncols) q[i] = sp[i];
        q += qstep;
        sp += dstep;
      }
    }
  }
}

template <typename T>
BFLY_HD void tile_load_auto(const T* src, int64_t sB, int64_t sS, int ncols, int B, int stack, int row0, int R,
                            const Panel& pn, int pbase, bool vec, T* sm, int tid, int nthr) {
  if (vec && pn.lseg >= Vec16<T>::LOG) {
    if (row0 + R <= B) tile_load_rows<T>(src, sB, sS, ncols, stack, row0, R, pn, pbase, sm, tid, nthr);
    else tile_load_chunks<T>(src, sB, sS, ncols, B, stack, row0, R, pn, pbase, sm, tid, nthr);
  } else {
    tile_load<T>(src, sB, sS, ncols, B, stack, row0, R, pn, pbase, sm, tid, nthr);
  }
}
template <typename T>
BFLY_HD void tile_store_auto(T* dst, int64_t sB, int64_t sS, int ncols, int B, int stack, int row0, int R,
                             const Panel& pn, int pbase, bool vec, const T* sm, int tid, int nthr) {
  if (vec && pn.lseg >= Vec16<T>::LOG) {
    if (row0 + R <= B) tile_store_rows<T>(dst, sB, sS, ncols, stack, row0, R, pn, pbase, sm, tid, nthr);
    else tile_store_chunks<T>(dst, sB, sS, ncols, B, stack, row0, R, pn, pbase, sm, tid, nthr);
  } else {
    tile_store<T>(dst, sB, sS, ncols, B, stack, row0, R, pn, pbase, sm, tid, nthr);
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
template <typename T, int K, int PAT>
BFLY_HD void fw_apply_all(T* v, const T* tw) {
  constexpr bool R4 = (PAT >= 2);
  constexpr int NST = R4 ? K / 2 : K;
  constexpr int PER = R4 ? (4 << K) : (2 << K);
  if constexpr (NST > 0) fw_apply_stage<T, K, PAT, 0>(v, tw + 0 * PER);
  if constexpr (NST > 1) fw_apply_stage<T, K, PAT, 1>(v, tw + 1 * PER);
  if constexpr (NST > 2) fw_apply_stage<T, K, PAT, 2>(v, tw + 2 * PER);
  if constexpr (NST > 3) fw_apply_stage<T, K, PAT, 3>(v, tw + 3 * PER);
}

// Tile position (with window bits zero) of every unit this thread owns in every group,
// computed once per CTA into shared memory: tab[(g * slots + slot) * nthr + tid].
template <typename T>
BFLY_HD void fw_build_table(const FwParams<T>& p, uint16_t* tab, int tid, int nthr) {
  const int C = 1 << p.panel.logC;
  if (!p.use_table) return;
  for (int g = 0; g < p.ngroups; ++g) {
    const FwGroup& G = p.g[g];
    const int U = C >> G.K;
    for (int slot = 0; slot < p.tab_slots; ++slot) {
      const int u = (U >= nthr) ? tid + slot * nthr : (tid & (U - 1));
      tab[(g * p.tab_slots + slot) * nthr + tid] = (uint16_t)(u < U ? deposit_unit(u, G.ubit, G.nubits) : 0);
    }
  }
}

// One group of the forward kernel applied in place to the R rows of a tile.
//   LOGC > 0 fixes the tile width at compile time (row offsets become immediates).
//   UNR rows are in flight per thread.
//   VEC: the window starts at bit 0, so a unit is a run of 16-byte chunks (vector accesses).
template <typename T, int K, int PAT, int LOGC, int ROWS, int UNR, bool VEC>
BFLY_HD void fw_group(const FwParams<T>& p, int gi, T* __restrict__ sm, const uint16_t* __restrict__ tab, int R,
                      int stack, int pbase, int tid, int nthr) {
  constexpr int E = 1 << K;
  constexpr int V = Vec16<T>::N;
  constexpr int NA = VEC ? E / V : E;  // shared-memory accesses per unit and row
  constexpr bool R4 = (PAT >= 2);
  constexpr int NST = R4 ? K / 2 : K;
  constexpr int PER = R4 ? E * 4 : E * 2;  // twiddle scalars of one stage for one unit
  constexpr int SZ = (int)sizeof(T);
  constexpr int ROWB = LOGC > 0 ? (SZ << LOGC) : 0;  // compile-time row pitch in bytes
  const FwGroup& g = p.g[gi];
  const Panel& pn = p.panel;
  const int C = LOGC > 0 ? (1 << LOGC) : (1 << pn.logC);
  const int U = C >> K;
  int nslot, r0, rstep;
  if (U >= nthr) {
    nslot = U / nthr; r0 = 0; rstep = 1;
  } else {
    nslot = 1; r0 = tid / U; rstep = nthr / U;
  }
  const int wg = pn.global_bit(g.lbit);
  const T* twbase = p.tw[g.which] + (int64_t)stack * p.tw_stack[g.which];
  const smaddr_t sm0 = sm_addr(sm);
  for (int slot = 0; slot < nslot; ++slot) {
    const int lbase = p.use_table ? (int)tab[(gi * p.tab_slots + slot) * nthr + tid]
                                  : deposit_unit(U >= nthr ? tid + slot * nthr : (tid & (U - 1)), g.ubit, g.nubits);
    const int col0 = pn.col(pbase, lbase);
    const int a0 = swzT<T>(lbase);
    T tw[NST * PER];
    // Twiddle index of the unit: its column with one window bit (radix 2; two bits for radix 4)
    // deleted.  The window bits of col0 are all zero, so the result does not depend on which of
    // them goes -- it is the same for every stage of the group -- and the pairs (quads) of a
    // stage lie 2^wg blocks apart.  Addresses are formed as (uniform pointer) + (32-bit index).
    constexpr int DEL = R4 ? 2 : 1;          // window bits a stage removes from the column index
    constexpr int BLK = R4 ? 16 : 4;         // twiddle scalars per pair (quad)
    const uint32_t ib = (uint32_t)((((col0 >> (wg + K)) << (wg + K - DEL)) | (col0 & ((1 << wg) - 1))) * BLK);
#pragma unroll
    for (int s = 0; s < NST; ++s) {
      const uint32_t es = g.tw_off[s] + ib;
#pragma unroll
      for (int pp = 0; pp < (E >> DEL); ++pp)
        load_tw<T, BLK>(tw + s * PER + pp * BLK, (twbase + (size_t)(pp << wg) * BLK) + es);
    }
    // byte offsets of the unit's elements (scalar path) or chunks (vector path) inside a tile row
    int off[NA];
#pragma unroll
    for (int m = 0; m < NA; ++m) off[m] = (a0 ^ g.d[VEC ? m * V : m]) * SZ;
    if (rstep == 1 && ROWS > 0 && LOGC > 0) {
      // the whole tile height is known at compile time: every row offset is an immediate
      if constexpr (ROWS > 0 && LOGC > 0) {
        smaddr_t a[NA];
#pragma unroll
        for (int m = 0; m < NA; ++m) a[m] = sm0 + (smaddr_t)off[m];
        static_for<0, ROWS / UNR>([&](auto ic) {
          constexpr int rr = decltype(ic)::value * UNR;
          T v[UNR][E];
          static_for<0, UNR>([&](auto jc) {
            constexpr int j = decltype(jc)::value;
#pragma unroll
            for (int m = 0; m < NA; ++m) {
              if constexpr (VEC) sm_ld16<(rr + j) * ROWB>(a[m], v[j] + m * V);
              else sm_ld<(rr + j) * ROWB>(a[m], v[j][m]);
            }
          });
          static_for<0, UNR>([&](auto jc) {
            constexpr int j = decltype(jc)::value;
            fw_apply_all<T, K, PAT>(v[j], tw);
#pragma unroll
            for (int m = 0; m < NA; ++m) {
              if constexpr (VEC) sm_st16<(rr + j) * ROWB>(a[m], v[j] + m * V);
              else sm_st<(rr + j) * ROWB>(a[m], v[j][m]);
            }
          });
        });
      }
    } else if (rstep == 1) {
      for (int r = 0; r < R; r += UNR) {
        const smaddr_t rb = sm0 + (smaddr_t)(r * C * SZ);
        smaddr_t a[NA];
#pragma unroll
        for (int m = 0; m < NA; ++m) a[m] = rb + (smaddr_t)off[m];
        T v[UNR][E];
        static_for<0, UNR>([&](auto jc) {
          constexpr int j = decltype(jc)::value;
          if (r + j < R) {
            const smaddr_t ro = LOGC > 0 ? 0 : (smaddr_t)(j * C * SZ);
#pragma unroll
            for (int m = 0; m < NA; ++m) {
              if constexpr (VEC) sm_ld16<j * ROWB>(a[m] + ro, v[j] + m * V);
              else sm_ld<j * ROWB>(a[m] + ro, v[j][m]);
            }
          }
        });
        static_for<0, UNR>([&](auto jc) {
          constexpr int j = decltype(jc)::value;
          if (r + j < R) {
            fw_apply_all<T, K, PAT>(v[j], tw);
            const smaddr_t ro = LOGC > 0 ? 0 : (smaddr_t)(j * C * SZ);
#pragma unroll
            for (int m = 0; m < NA; ++m) {
              if constexpr (VEC) sm_st16<j * ROWB>(a[m] + ro, v[j] + m * V);
              else sm_st<j * ROWB>(a[m] + ro, v[j][m]);
            }
          }
        });
      }
    } else {
      // fewer units than threads: several rows are processed side by side
      for (int r = r0; r < R; r += rstep) {
        const smaddr_t rb = sm0 + (smaddr_t)(r * C * SZ);
        T v[E];
#pragma unroll
        for (int m = 0; m < NA; ++m) {
          if constexpr (VEC) sm_ld16<0>(rb + (smaddr_t)off[m], v + m * V);
          else sm_ld<0>(rb + (smaddr_t)off[m], v[m]);
        }
        fw_apply_all<T, K, PAT>(v, tw);
#pragma unroll
        for (int m = 0; m < NA; ++m) {
          if constexpr (VEC) sm_st16<0>(rb + (smaddr_t)off[m], v + m * V);
          else sm_st<0>(rb + (smaddr_t)off[m], v[m]);
        }
      }
    }
  }
}

template <typename T, int K, int PAT, int LOGC, int ROWS, int UNR>
BFLY_HD void fw_group_v(const FwParams<T>& p, int gi, T* sm, const uint16_t* tab, int R, int stack, int pbase,
                        int tid, int nthr) {
  if constexpr ((1 << K) >= Vec16<T>::N) {
    if (p.g[gi].vec) {
      fw_group<T, K, PAT, LOGC, ROWS, UNR, true>(p, gi, sm, tab, R, stack, pbase, tid, nthr);
      return;
    }
  }
  fw_group<T, K, PAT, LOGC, ROWS, UNR, false>(p, gi, sm, tab, R, stack, pbase, tid, nthr);
}

// Dispatch on the (uniform) window width and pattern of a group.  KMAX is the widest window
// this kernel instance was compiled for (it sets the register budget of the kernel).
template <typename T, int KMAX, int LOGC, int ROWS>
BFLY_HD void fw_group_dispatch(const FwParams<T>& p, int gi, T* sm, const uint16_t* tab, int R, int stack,
                               int pbase, int tid, int nthr) {
  const int K = p.g[gi].K, pat = p.g[gi].pattern;
  constexpr int U2 = 2;
  constexpr int U3 = (sizeof(T) == 4) ? 2 : 1;
  if (K == 1) { fw_group_v<T, 1, kR2Inc, LOGC, ROWS, U2>(p, gi, sm, tab, R, stack, pbase, tid, nthr); return; }
  if (K == 2) {
    if (pat == kR2Inc) fw_group_v<T, 2, kR2Inc, LOGC, ROWS, U2>(p, gi, sm, tab, R, stack, pbase, tid, nthr);
    else if (pat == kR2Dec) fw_group_v<T, 2, kR2Dec, LOGC, ROWS, U2>(p, gi, sm, tab, R, stack, pbase, tid, nthr);
    else fw_group_v<T, 2, kR4Inc, LOGC, ROWS, U2>(p, gi, sm, tab, R, stack, pbase, tid, nthr);
    return;
  }
  if constexpr (KMAX >= 3) {
    if (K == 3) {
      if (pat == kR2Inc) fw_group_v<T, 3, kR2Inc, LOGC, ROWS, U3>(p, gi, sm, tab, R, stack, pbase, tid, nthr);
      else fw_group_v<T, 3, kR2Dec, LOGC, ROWS, U3>(p, gi, sm, tab, R, stack, pbase, tid, nthr);
      return;
    }
  }
  if constexpr (KMAX >= 4 && sizeof(T) == 4) {  // 4-bit windows only for 4-byte elements (register budget)
    if (K == 4) {
      if (pat == kR2Inc) fw_group_v<T, 4, kR2Inc, LOGC, ROWS, 1>(p, gi, sm, tab, R, stack, pbase, tid, nthr);
      else if (pat == kR2Dec) fw_group_v<T, 4, kR2Dec, LOGC, ROWS, 1>(p, gi, sm, tab, R, stack, pbase, tid, nthr);
      else if (pat == kR4Inc) fw_group_v<T, 4, kR4Inc, LOGC, ROWS, 1>(p, gi, sm, tab, R, stack, pbase, tid, nthr);
      else fw_group_v<T, 4, kR4Dec, LOGC, ROWS, 1>(p, gi, sm, tab, R, stack, pbase, tid, nthr);
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
// shared memory of one forward CTA: the tile followed by the unit table
template <typename T> BFLY_HD size_t fw_tile_bytes(const FwParams<T>& p) { return ((size_t)p.R * sizeof(T)) << p.panel.logC; }
template <typename T> BFLY_HD size_t fw_smem_bytes(const FwParams<T>& p, int nthr) {
  return fw_tile_bytes(p) + (p.use_table ? (size_t)p.ngroups * p.tab_slots * nthr * sizeof(uint16_t) : 0);
}

// ------------------------------------------------------------------ backward phase

// Per-thread state of a backward phase: the twiddles of the thread's unit in every
// sub-group, the matching gradient accumulators, and the unit's tile position.  They live
// in registers for the whole kernel (all loops over them are fully unrolled with constant
// indices).  KW = window bits: a unit has 2^KW elements.  The twiddles themselves are not
// kept: they are re-read from L2 (where the whole twiddle tensor stays resident) one
// sub-group step ahead of their use, which frees registers for more rows in flight.
template <int KW> struct BwTwn { static constexpr int value = (KW == 2) ? 16 : 4; };
template <typename T, int KW, int NSG> struct BwState {
  T tw[2][BwTwn<KW>::value];     // twiddles of the sub-group being processed (buffer j & 1) and of
                                 // the next one (the other buffer), fetched one step ahead
  T acc[NSG][BwTwn<KW>::value];  // gradient accumulators of every sub-group of the phase
  int a0[NSG];                   // swizzled tile index of the unit (window bits zero)
  uint32_t twi[NSG][KW];         // element offset of the unit's first twiddle block per stage
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

// Fetch the twiddles of sub-group j (of the thread's unit) into buffer j & 1.
template <typename T, int KW, int NSG>
BFLY_HD void bw_fetch_tw(const BwParams<T>& p, BwState<T, KW, NSG>& st, int j, int stack) {
  const BwSg& sg = p.sg[j];
  const T* twp = p.tw[sg.which] + (int64_t)stack * p.tw_stack[sg.which];
  T* dst = st.tw[j & 1];
  if (sg.radix == 4) {
    if constexpr (KW == 2) load_tw<T, 16>(dst, twp + st.twi[j][0]);
  } else {
    const int wg = p.panel.global_bit(sg.lbit);
#pragma unroll
    for (int s = 0; s < KW; ++s) {
      if (s < sg.nst) {
#pragma unroll
        for (int pp = 0; pp < (1 << (KW - 1)); ++pp)
          load_tw<T, 4>(dst + s * (1 << (KW - 1)) * 4 + pp * 4, twp + st.twi[j][s] + (uint32_t)((pp << wg) * 4));
      }
    }
  }
}

template <typename T, int KW, int NSG>
BFLY_HD void bw_load_state(const BwParams<T>& p, BwState<T, KW, NSG>& st, int stack, int pbase, int tid,
                           int nthr) {
  const BwThread th = bw_thread<KW>(p.panel.logC, tid, nthr);
#pragma unroll
  for (int b = 0; b < 2; ++b)
#pragma unroll
    for (int e = 0; e < BwTwn<KW>::value; ++e) st.tw[b][e] = Ops<T>::zero();
#pragma unroll
  for (int j = 0; j < NSG; ++j) {
#pragma unroll
    for (int e = 0; e < BwTwn<KW>::value; ++e) st.acc[j][e] = Ops<T>::zero();
    st.a0[j] = 0;
#pragma unroll
    for (int s = 0; s < KW; ++s) st.twi[j][s] = 0;
    if (j < p.nsg) {
      const BwSg& sg = p.sg[j];
      const int lbase = deposit_unit(th.u, sg.ubit, sg.nubits);
      st.a0[j] = swzT<T>(lbase);
      const int col0 = p.panel.col(pbase, lbase);
      const int wg = p.panel.global_bit(sg.lbit);
      if (sg.radix == 4) {
        st.twi[j][0] = sg.tw_off[0] + (uint32_t)delete_2bits(col0, wg) * 16u;
      } else {
#pragma unroll
        for (int s = 0; s < KW; ++s)
          if (s < sg.nst) st.twi[j][s] = sg.tw_off[s] + (uint32_t)delete_bit(col0, wg + sg.q[s]) * 4u;
      }
    }
  }
  bw_fetch_tw<T, KW, NSG>(p, st, 0, stack);
}

// Add one 2x2 block (four elements, 16-byte aligned) of accumulators to d_twiddle: one vector
// reduction per 16 bytes instead of one per scalar.
BFLY_HD void atomic_add_block(float* dst, const float* v) {
#if defined(__CUDA_ARCH__)
  asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
#else
  for (int e = 0; e < 4; ++e) dst[e] += v[e];
#endif
}
BFLY_HD void atomic_add_block(cf* dst, const cf* v) {
#if defined(__CUDA_ARCH__)
  asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v[0].re), "f"(v[0].im), "f"(v[1].re), "f"(v[1].im) : "memory");
  asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(dst + 2), "f"(v[2].re), "f"(v[2].im), "f"(v[3].re), "f"(v[3].im) : "memory");
#else
  for (int e = 0; e < 4; ++e) { dst[e].re += v[e].re; dst[e].im += v[e].im; }
#endif
}

template <typename T, int KW, int NSG>
BFLY_HD void bw_flush_state(const BwParams<T>& p, const BwState<T, KW, NSG>& st, int stack, int pbase,
                            int tid, int nthr) {
#pragma unroll
  for (int j = 0; j < NSG; ++j) {
    if (j < p.nsg) {
      const BwSg& sg = p.sg[j];
      T* dtw = p.dtw[sg.which] + (int64_t)stack * p.tw_stack[sg.which];
      if (sg.radix == 4) {
        if constexpr (KW == 2) {
#pragma unroll
          for (int b = 0; b < 4; ++b) atomic_add_block(dtw + st.twi[j][0] + b * 4, st.acc[j] + b * 4);
        }
      } else {
        const int wg = p.panel.global_bit(sg.lbit);
#pragma unroll
        for (int s = 0; s < KW; ++s) {
          if (s < sg.nst) {
#pragma unroll
            for (int pp = 0; pp < (1 << (KW - 1)); ++pp)
              atomic_add_block(dtw + st.twi[j][s] + (uint32_t)((pp << wg) * 4), st.acc[j] + s * (1 << (KW - 1)) * 4 + pp * 4);
          }
        }
      }
    }
  }
}

// Load / store the thread's unit of one tile row (16-byte accesses when the window starts
// at bit 0 and the unit is a whole number of chunks).  IMM is a compile-time byte offset.
template <typename T, int KW, bool VEC, int IMM>
BFLY_HD void bw_unit_ld(smaddr_t rowbase, const int* off, T* v) {
  constexpr int E = 1 << KW;
  constexpr int V = Vec16<T>::N;
  if constexpr (VEC && E >= V) {
#pragma unroll
    for (int h = 0; h < E / V; ++h) sm_ld16<IMM>(rowbase + (smaddr_t)off[h * V], v + h * V);
  } else {
#pragma unroll
    for (int m = 0; m < E; ++m) sm_ld<IMM>(rowbase + (smaddr_t)off[m], v[m]);
  }
}
template <typename T, int KW, bool VEC, int IMM>
BFLY_HD void bw_unit_st(smaddr_t rowbase, const int* off, const T* v) {
  constexpr int E = 1 << KW;
  constexpr int V = Vec16<T>::N;
  if constexpr (VEC && E >= V) {
#pragma unroll
    for (int h = 0; h < E / V; ++h) sm_st16<IMM>(rowbase + (smaddr_t)off[h * V], v + h * V);
  } else {
#pragma unroll
    for (int m = 0; m < E; ++m) sm_st<IMM>(rowbase + (smaddr_t)off[m], v[m]);
  }
}

// Stage pattern of a sub-group, resolved once per sub-group step (not per row):
//   KW == 2, radix 2: two stages on bits (q0, q1) -> q0*2 + q1 ; one stage on bit q -> 4 + q
//   KW == 2, radix 4: 6          KW == 1: 0
BFLY_HD int bw_pattern(const BwSg& sg, int KW) {
  if (KW == 1) return 0;
  if (sg.radix == 4) return 6;
  return sg.nst == 2 ? sg.q[0] * 2 + sg.q[1] : 4 + sg.q[0];
}

template <typename T, int KW, int PATID>
BFLY_HD void bw_apply_fw(T* v, const T* tw) {
  if constexpr (KW == 1) {
    r2_stage_fw<T, 1, 0>(v, tw);
  } else if constexpr (PATID == 6) {
    r4_stage_fw<T, 2, 0>(v, tw);
  } else if constexpr (PATID >= 4) {
    r2_stage_fw<T, 2, PATID - 4>(v, tw);
  } else {
    r2_stage_fw<T, 2, PATID / 2>(v, tw);
    r2_stage_fw<T, 2, PATID % 2>(v, tw + 8);
  }
}
template <typename T, int KW, int PATID>
BFLY_HD void bw_apply_bw(T* g, const T* x, const T* tw, T* acc) {
  if constexpr (KW == 1) {
    r2_bw_q<T, 1, 0>(g, x, tw, acc);
  } else if constexpr (PATID == 6) {
    r4_bw4<T>(g, x, tw, acc);
  } else if constexpr (PATID >= 4) {
    r2_bw_q<T, 2, PATID - 4>(g, x, tw, acc);
  } else {
    T x1[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) x1[m] = x[m];
    r2_stage_fw<T, 2, PATID / 2>(x1, tw);
    r2_bw_q<T, 2, PATID % 2>(g, x1, tw + 8, acc + 8);
    r2_bw_q<T, 2, PATID / 2>(g, x, tw, acc);
  }
}

// Forward recompute of sub-group j over the rows of a batch: reads the thread's unit of every
// row from snapshot j, applies the sub-group's stages, writes snapshot j+1.
// LOGC / RB > 0 fix the panel width and the batch height at compile time.
template <typename T, int KW, int NSG, int LOGC, int RB, int PATID, bool VEC>
BFLY_HD void bw_sg_forward_rows(const BwParams<T>& p, const BwState<T, KW, NSG>& st, int j, T* __restrict__ smX,
                                int R, int tid, int nthr) {
  constexpr int E = 1 << KW;
  constexpr int SZ = (int)sizeof(T);
  constexpr int UNR = (RB > 0 && RB % 4 == 0 && sizeof(T) == 4) ? 4 : 2;  // rows in flight per thread
  constexpr int ROWB = LOGC > 0 ? (SZ << LOGC) : 0;
  const BwSg& sg = p.sg[j];
  const int C = LOGC > 0 ? (1 << LOGC) : (1 << p.panel.logC);
  const int Rb = RB > 0 ? RB : p.Rb;
  const BwThread th = bw_thread<KW>(p.panel.logC, tid, nthr);
  int off[E];
#pragma unroll
  for (int m = 0; m < E; ++m) off[m] = (st.a0[j] ^ sg.d[m]) * SZ;
  const smaddr_t src = sm_addr(smX) + (smaddr_t)(j * Rb * C * SZ);
  const smaddr_t dst = src + (smaddr_t)(Rb * C * SZ);
  if (LOGC > 0 && RB > 0 && th.rstep == 1) {
    if constexpr (LOGC > 0 && RB > 0) {
      // a real loop (not unrolled: the body is reused from the instruction cache) over row
      // pairs; inside the body the second row is an immediate offset
#pragma unroll 1
      for (int rr = 0; rr < RB; rr += UNR) {
        const smaddr_t so = (smaddr_t)(rr * ROWB);
        T v[UNR][E];
        static_for<0, UNR>([&](auto jc) {
          constexpr int jj = decltype(jc)::value;
          bw_unit_ld<T, KW, VEC, jj * ROWB>(src + so, off, v[jj]);
        });
        static_for<0, UNR>([&](auto jc) {
          constexpr int jj = decltype(jc)::value;
          bw_apply_fw<T, KW, PATID>(v[jj], st.tw[j & 1]);
          bw_unit_st<T, KW, VEC, jj * ROWB>(dst + so, off, v[jj]);
        });
      }
    }
  } else {
    for (int r = th.r0; r < R; r += th.rstep) {
      T v[E];
      bw_unit_ld<T, KW, VEC, 0>(src + (smaddr_t)(r * C * SZ), off, v);
      bw_apply_fw<T, KW, PATID>(v, st.tw[j & 1]);
      bw_unit_st<T, KW, VEC, 0>(dst + (smaddr_t)(r * C * SZ), off, v);
    }
  }
}

// Backward of sub-group j over the rows of a batch: reads snapshot j and the gradient tile,
// accumulates the twiddle gradient of the thread's unit and replaces the gradient in place.
template <typename T, int KW, int NSG, int LOGC, int RB, int PATID, bool VEC>
BFLY_HD void bw_sg_backward_rows(const BwParams<T>& p, BwState<T, KW, NSG>& st, int j, const T* __restrict__ smX,
                                 T* __restrict__ smG, int R, int tid, int nthr) {
  constexpr int E = 1 << KW;
  constexpr int SZ = (int)sizeof(T);
  constexpr int UNR = (RB > 0 && RB % 4 == 0 && sizeof(T) == 4) ? 4 : 2;  // rows in flight per thread
  constexpr int ROWB = LOGC > 0 ? (SZ << LOGC) : 0;
  const BwSg& sg = p.sg[j];
  const int C = LOGC > 0 ? (1 << LOGC) : (1 << p.panel.logC);
  const int Rb = RB > 0 ? RB : p.Rb;
  const BwThread th = bw_thread<KW>(p.panel.logC, tid, nthr);
  int off[E];
#pragma unroll
  for (int m = 0; m < E; ++m) off[m] = (st.a0[j] ^ sg.d[m]) * SZ;
  const smaddr_t src = sm_addr(smX) + (smaddr_t)(j * Rb * C * SZ);
  const smaddr_t gb = sm_addr(smG);
  if (LOGC > 0 && RB > 0 && th.rstep == 1) {
    if constexpr (LOGC > 0 && RB > 0) {
#pragma unroll 1
      for (int rr = 0; rr < RB; rr += UNR) {
        const smaddr_t so = (smaddr_t)(rr * ROWB);
        T x[UNR][E], g[UNR][E];
        static_for<0, UNR>([&](auto jc) {
          constexpr int jj = decltype(jc)::value;
          bw_unit_ld<T, KW, VEC, jj * ROWB>(src + so, off, x[jj]);
          bw_unit_ld<T, KW, VEC, jj * ROWB>(gb + so, off, g[jj]);
        });
        static_for<0, UNR>([&](auto jc) {
          constexpr int jj = decltype(jc)::value;
          bw_apply_bw<T, KW, PATID>(g[jj], x[jj], st.tw[j & 1], st.acc[j]);
          bw_unit_st<T, KW, VEC, jj * ROWB>(gb + so, off, g[jj]);
        });
      }
    }
  } else {
    for (int r = th.r0; r < R; r += th.rstep) {
      T x[E], g[E];
      bw_unit_ld<T, KW, VEC, 0>(src + (smaddr_t)(r * C * SZ), off, x);
      bw_unit_ld<T, KW, VEC, 0>(gb + (smaddr_t)(r * C * SZ), off, g);
      bw_apply_bw<T, KW, PATID>(g, x, st.tw[j & 1], st.acc[j]);
      bw_unit_st<T, KW, VEC, 0>(gb + (smaddr_t)(r * C * SZ), off, g);
    }
  }
}

// Resolve the (uniform) stage pattern and access kind of sub-group j, then run the rows.
template <typename T, int KW, int NSG, int LOGC, int RB, bool FORWARD>
BFLY_HD void bw_sg_step(const BwParams<T>& p, BwState<T, KW, NSG>& st, int j, int stack, T* __restrict__ smX,
                        T* __restrict__ smG, int R, int tid, int nthr) {
  const BwSg& sg = p.sg[j];
  // twiddles of the step that follows go into the other buffer while this step computes:
  // forward steps walk j upwards (the last one hands over to the backward of nsg-1),
  // backward steps walk j downwards (j = 0 is followed by the forward of j = 0: same twiddles)
  if (FORWARD) bw_fetch_tw<T, KW, NSG>(p, st, j + 1, stack);
  else if (j > 0) bw_fetch_tw<T, KW, NSG>(p, st, j - 1, stack);
  const int pat = bw_pattern(sg, KW);
  const bool vec = sg.vec != 0;
  auto run = [&](auto pc, auto vc) {
    constexpr int PATID = decltype(pc)::value;
    constexpr bool VEC = decltype(vc)::value;
    if constexpr (FORWARD) bw_sg_forward_rows<T, KW, NSG, LOGC, RB, PATID, VEC>(p, st, j, smX, R, tid, nthr);
    else bw_sg_backward_rows<T, KW, NSG, LOGC, RB, PATID, VEC>(p, st, j, smX, smG, R, tid, nthr);
  };
  auto with_vec = [&](auto pc) {
    if (vec) run(pc, std::true_type{});
    else run(pc, std::false_type{});
  };
  if constexpr (KW == 1) {
    with_vec(std::integral_constant<int, 0>{});
  } else {
    switch (pat) {
      case 0: with_vec(std::integral_constant<int, 0>{}); break;
      case 1: with_vec(std::integral_constant<int, 1>{}); break;
      case 2: with_vec(std::integral_constant<int, 2>{}); break;
      case 3: with_vec(std::integral_constant<int, 3>{}); break;
      case 4: with_vec(std::integral_constant<int, 4>{}); break;
      case 5: with_vec(std::integral_constant<int, 5>{}); break;
      default: with_vec(std::integral_constant<int, 6>{}); break;
    }
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

}  // namespace bfly
