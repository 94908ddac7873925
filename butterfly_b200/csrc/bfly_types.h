// Shared host/device plain-old-data types and arithmetic helpers of the butterfly
// multiply kernels.  This header compiles as CUDA (nvcc) and as plain C++ (g++),
// so the tile routines built on it can be executed thread-by-thread on the host
// by the test-suite's emulator to check their index arithmetic without a GPU.
#pragma once
#include <stdint.h>
#include <math.h>

#include "../../include/bfly.h"  // status codes

#if defined(__CUDACC__)
#define BFLY_HD __host__ __device__ __forceinline__
#else
#define BFLY_HD inline
#endif

namespace bfly {

// ---------------------------------------------------------------- element types

struct cf {  // complex<float>, re/im interleaved exactly like torch.complex64
  float re, im;
};

BFLY_HD float fma_(float a, float b, float c) {
#if defined(__CUDA_ARCH__)
  return __fmaf_rn(a, b, c);
#else
  return fmaf(a, b, c);
#endif
}
BFLY_HD float mul_(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fmul_rn(a, b);
#else
  return a * b;
#endif
}

template <typename T> struct Ops;

// Real arithmetic.  One butterfly output is  y = a*x + b*z  evaluated as
// fma(a, x, rn(b*z)): the product of the partner coefficient is rounded first and
// the own-coefficient product is fused, which is how the reference's CUDA
// expression `t_own * x_own + t_partner * x_partner` (csrc/cuda/butterfly_cuda.cu:256)
// contracts under nvcc's default -fmad=true.
template <> struct Ops<float> {
  static BFLY_HD float zero() { return 0.f; }
  // a*x + b*z
  static BFLY_HD float madd2(float a, float x, float b, float z) { return fma_(a, x, mul_(b, z)); }
  // conj(a)*x + conj(b)*z
  static BFLY_HD float madd2c(float a, float x, float b, float z) { return fma_(a, x, mul_(b, z)); }
  // acc + g*conj(x)
  static BFLY_HD float acc_gxc(float acc, float g, float x) { return fma_(g, x, acc); }
  // acc + a*x
  static BFLY_HD float fmadd(float acc, float a, float x) { return fma_(a, x, acc); }
  static BFLY_HD float mul(float a, float x) { return mul_(a, x); }
  // acc + conj(a)*x
  static BFLY_HD float fmaddc(float acc, float a, float x) { return fma_(a, x, acc); }
  static BFLY_HD float mulc(float a, float x) { return mul_(a, x); }
};

// Complex arithmetic as fused chains (4 FMA-pipe operations per complex multiply-add).
template <> struct Ops<cf> {
  static BFLY_HD cf zero() { return cf{0.f, 0.f}; }
  static BFLY_HD cf mul(cf a, cf x) {
    cf r;
    r.re = fma_(a.re, x.re, -mul_(a.im, x.im));
    r.im = fma_(a.re, x.im, mul_(a.im, x.re));
    return r;
  }
  static BFLY_HD cf fmadd(cf acc, cf a, cf x) {
    cf r;
    r.re = fma_(a.re, x.re, fma_(-a.im, x.im, acc.re));
    r.im = fma_(a.re, x.im, fma_(a.im, x.re, acc.im));
    return r;
  }
  static BFLY_HD cf mulc(cf a, cf x) {  // conj(a)*x
    cf r;
    r.re = fma_(a.re, x.re, mul_(a.im, x.im));
    r.im = fma_(a.re, x.im, -mul_(a.im, x.re));
    return r;
  }
  static BFLY_HD cf fmaddc(cf acc, cf a, cf x) {  // acc + conj(a)*x
    cf r;
    r.re = fma_(a.re, x.re, fma_(a.im, x.im, acc.re));
    r.im = fma_(a.re, x.im, fma_(-a.im, x.re, acc.im));
    return r;
  }
  static BFLY_HD cf madd2(cf a, cf x, cf b, cf z) { return fmadd(mul(b, z), a, x); }
  static BFLY_HD cf madd2c(cf a, cf x, cf b, cf z) { return fmaddc(mulc(b, z), a, x); }
  static BFLY_HD cf acc_gxc(cf acc, cf g, cf x) {  // acc + g*conj(x)
    cf r;
    r.re = fma_(g.re, x.re, fma_(g.im, x.im, acc.re));
    r.im = fma_(g.im, x.re, fma_(-g.re, x.im, acc.im));
    return r;
  }
};

// ---------------------------------------------------------------- bit helpers

// Remove bit `pos` from x (bits above move down by one).
BFLY_HD int delete_bit(int x, int pos) {
  const int low = (1 << pos) - 1;
  return ((x >> 1) & ~low) | (x & low);
}
// Remove bits pos, pos+1 from x.
BFLY_HD int delete_2bits(int x, int pos) {
  const int low = (1 << pos) - 1;
  return ((x >> 2) & ~low) | (x & low);
}
// Insert `nbits` zero bits at position pos.
BFLY_HD int insert_zeros(int x, int pos, int nbits) {
  const int low = (1 << pos) - 1;
  return ((x & ~low) << nbits) | (x & low);
}

// Elements per 16-byte chunk.
template <typename T> struct Vec16 {};
template <> struct Vec16<float> { static constexpr int N = 4; static constexpr int LOG = 2; };
template <> struct Vec16<cf> { static constexpr int N = 2; static constexpr int LOG = 1; };

// Shared-memory placement of local column l of a tile row.  Rows are stored as 16-byte
// chunks (2^VB elements); the low three bits of the chunk index (which select one of the
// eight 16-byte bank groups of a 128-byte wavefront) are XORed with the next three, so whole
// chunks move (16-byte copies stay possible) and every access pattern the kernels use --
// 32 lanes that differ in five chosen bits of l, or 8 lanes reading consecutive chunks --
// is free of bank conflicts.
template <int VB> BFLY_HD int swz(int l) { return l ^ (((l >> (VB + 3)) & 7) << VB); }
template <typename T> BFLY_HD int swzT(int l) { return swz<Vec16<T>::LOG>(l); }
inline int swz_rt(int l, int vb) { return l ^ (((l >> (vb + 3)) & 7) << vb); }

// ---------------------------------------------------------------- descriptors

constexpr int kMaxK = 4;          // widest register window of the forward kernel (2^4 elements/thread)
constexpr int kMaxFwGroups = 40;  // stage groups one forward launch can carry
constexpr int kMaxSg = 10;        // sub-groups of one backward phase
constexpr int kMaxUnitBits = 16;

// Column geometry of a tile ("panel"): 2^logC columns of one batch row, made of
// 2^(logC-lseg) segments of 2^lseg consecutive columns; segment k of panel pi starts at
// global column  base(pi) + k << pb .  A full row is the panel lseg = logC = log_n.
struct Panel {
  int logC;   // log2 columns in the panel
  int lseg;   // log2 segment length (local bits [0,lseg) are global bits [0,lseg))
  int pb;     // global bit that local bit lseg maps to (local bit lseg+j -> global pb+j)
  int npanels_log;  // log2 number of panels per row
  BFLY_HD int pw() const { return logC - lseg; }
  BFLY_HD int base(int pi) const {
    const int mid = pb - lseg;  // global bits [lseg, pb) come from the low bits of pi
    return ((pi & ((1 << mid) - 1)) << lseg) | ((pi >> mid) << (pb + pw()));
  }
  BFLY_HD int col(int pbase, int l) const {
    return pbase + (l & ((1 << lseg) - 1)) + ((l >> lseg) << pb);
  }
  BFLY_HD int global_bit(int lbit) const { return lbit < lseg ? lbit : lbit - lseg + pb; }
};

enum FwPattern : int { kR2Inc = 0, kR2Dec = 1, kR4Inc = 2, kR4Dec = 3 };

// One register-window group of the forward kernel: K consecutive radix-2 stages (or K/2
// radix-4 stages) acting on local bits [lbit, lbit+K).
struct FwGroup {
  uint8_t lbit, K, pattern, which;  // which: twiddle tensor (0 radix-2, 1 radix-4)
  uint8_t nubits;                   // log2(units per tile row) = logC - K
  uint8_t emit;                     // 1 + snapshot slot to write after this group, 0 = none
  uint8_t vec;                      // window starts at bit 0 and spans whole chunks: 16-byte accesses
  uint8_t pad_;
  uint32_t tw_off[kMaxK];           // element offset of each stage's twiddle inside one stack
  uint8_t ubit[kMaxUnitBits];       // local bit position of unit-index bit j
  uint16_t d[1 << kMaxK];           // swz(m << lbit): element m of a unit sits at swz(unit) ^ d[m]
};

// Glue operators folded into a forward launch whose tile holds whole rows (none of them set = the
// plain product).  They replace element-wise and gather operators that would otherwise each make a
// full pass over the rows in device memory:
//   x_real    the input rows are float32 and enter the complex product with zero imaginary part
//   in_perm   row[c] <- row[in_perm[c]] right after the load (n entries)
//   out_diag  y[c] <- y[c] * out_diag[c] after the last factor (n entries) ...
//   out_perm  ... then y[c] <- y[out_perm[c]] (n entries)
//   out_real  only the real parts of the result are written, as float32 rows
// x_real / out_real take the place of FwParams::x / ::out (same strides, counted in floats).
constexpr int kGlueSlots = 16;  // columns per thread of a row in the gather passes
template <typename T> struct FwGlue {
  const int32_t* in_perm;
  const int32_t* out_perm;
  const T* out_diag;
  const float* x_real;
  float* out_real;
  // gather passes: bit j of (thread + k * threads) becomes bit colbit[j] of the column a thread owns,
  // chosen so that the lanes of a warp spread over the shared-memory banks on both sides of a
  // bit-reversal gather (glue_column_bits)
  uint8_t colbit[16];
  BFLY_HD bool any_in() const { return in_perm != nullptr; }
  BFLY_HD bool any_out() const { return out_perm != nullptr || out_diag != nullptr; }
};

template <typename T> struct FwParams {
  const T* tw[2];            // radix-2 / radix-4 twiddle tensors
  int64_t tw_stack[2];       // elements per stack in each
  const T* x;                // input rows
  int64_t x_sB, x_sS;        // element strides (x_sS may be 0)
  int x_cols;                // valid input columns (zero beyond)
  T* out;                    // output rows, or nullptr when only snapshots are wanted
  int64_t out_sB, out_sS;
  int out_cols;              // columns written
  T* snap[8];                // snapshot buffers, (B,S,n) contiguous
  int B, S, log_n;
  int R;                     // rows per tile
  int tab_slots;             // units per thread and group (max over groups)
  int use_table;             // unit positions come from a per-CTA table in shared memory
  int vec_in, vec_out;       // 16-byte global accesses allowed
  // tile traffic through the TMA unit (set by the launcher when every tensor qualifies):
  // tma_s*: the tensor's descriptor has a stack dimension; tma_pbe, tma_f: see bfly_tma.h
  int tma, tma_sx, tma_so, tma_pbe, tma_f;
  Panel panel;
  int ngroups;
  FwGlue<T> glue;
  FwGroup g[kMaxFwGroups];
};

// One sub-group of a backward phase.  With a 2-bit window (KW = 2): up to two radix-2
// stages, or one radix-4 stage, on the 4 elements at local bits [lbit, lbit+2).  With a
// 1-bit window (KW = 1): one radix-2 stage on the 2 elements at local bit lbit.
struct BwSg {
  uint8_t lbit, nst, radix, which;
  uint8_t q[2];                // bit offset of each stage inside the window
  uint8_t nubits, vec;
  uint32_t tw_off[2];
  uint8_t ubit[kMaxUnitBits];
  uint16_t d[4];               // swz(m << lbit)
  // second-generation backward kernel: the code variant that runs this sub-group (bw2_kase) and
  // whether the unit's elements 1 and 2 trade places in the registers for it
  uint8_t kase, swap12, pad_[2];
};

template <typename T> struct BwParams {
  const T* tw[2];
  T* dtw[2];
  int64_t tw_stack[2];
  const T* xin;  int64_t xin_sB, xin_sS;   int xin_cols;   // activation entering the phase
  const T* gin;  int64_t gin_sB, gin_sS;   int gin_cols;   // gradient leaving the phase (zero beyond)
  T* gout;       int64_t gout_sB, gout_sS; int gout_cols;  // gradient entering the phase
  int B, S, log_n;
  int v2;            // run the two-CTAs-per-SM kernel (accumulators in tensor memory, 4-row batches)
  int Rb;            // rows per batch held in shared memory
  int rows_per_cta;  // rows of one row slice (multiple of Rb)
  int nslices;
  int vec_x, vec_g, vec_o;
  // tile traffic through the TMA unit (set by the launcher when all three tensors qualify):
  // tma_s*: the tensor's descriptor has a stack dimension; tma_pbe, tma_f: see bfly_tma.h
  int tma, tma_sx, tma_sg, tma_so, tma_pbe, tma_f;
  // fused linear layer (packed-pair kernel only): add the phase's output into gout instead of
  // storing it (gout then has stack stride 0: the input gradient summed over the stacks), and
  // accumulate the column sums of gin into dbias[stack * n + column] for flat positions < dbias_len
  int gout_reduce;
  T* dbias;
  int dbias_len;
  Panel panel;
  int nsg;
  BwSg sg[kMaxSg];
};

}  // namespace bfly
