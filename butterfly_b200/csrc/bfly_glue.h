// Small operators next to the butterfly multiply, written once for the CUDA kernels and for the
// host emulator of the tests.
//
// Unitary twiddle synthesis.  The reference's ButterflyUnitary layer stores four angles
// (phi, alpha, psi, chi) per 2x2 block and builds the complex block from them with a chain of
// cos / sin / stack operators on every forward call, leaving the chain's backward to autograd
// (torch_butterfly/butterfly.py:271-280):
//     [[ cos(phi) e^{i(alpha+psi)},  sin(phi) e^{i(alpha+chi)} ],
//      [-sin(phi) e^{i(alpha-chi)},  cos(phi) e^{i(alpha-psi)} ]]
// Here one pass reads the 4 angles and writes the 4 complex entries, and one pass turns the
// gradient of the entries (PyTorch's convention for a complex tensor under a real loss:
// dL/dRe + i dL/dIm) into the gradient of the angles.
#pragma once
#include <cmath>
#include <cstdint>

#include "bfly_types.h"

namespace bfly {

struct UnitaryTrig {
  float c, s;            // cos / sin of phi
  float cu, su, cv, sv;  // of u = alpha + psi, v = alpha + chi
  float cw, sw, cz, sz;  // of w = alpha - chi, z = alpha - psi
};

BFLY_HD UnitaryTrig unitary_trig(const float* a) {
  UnitaryTrig t;
  const float phi = a[0], alpha = a[1], psi = a[2], chi = a[3];
#if defined(__CUDA_ARCH__)
  sincosf(phi, &t.s, &t.c);
  sincosf(alpha + psi, &t.su, &t.cu);
  sincosf(alpha + chi, &t.sv, &t.cv);
  sincosf(alpha - chi, &t.sw, &t.cw);
  sincosf(alpha - psi, &t.sz, &t.cz);
#else
  t.s = std::sin(phi); t.c = std::cos(phi);
  t.su = std::sin(alpha + psi); t.cu = std::cos(alpha + psi);
  t.sv = std::sin(alpha + chi); t.cv = std::cos(alpha + chi);
  t.sw = std::sin(alpha - chi); t.cw = std::cos(alpha - chi);
  t.sz = std::sin(alpha - psi); t.cz = std::cos(alpha - psi);
#endif
  return t;
}

// angles[4] -> tw[8] = (A.re, A.im, B.re, B.im, C.re, C.im, D.re, D.im), row-major 2x2 complex
BFLY_HD void unitary_block_fw(const float* a, float* tw) {
  const UnitaryTrig t = unitary_trig(a);
  tw[0] = t.c * t.cu;  tw[1] = t.c * t.su;
  tw[2] = t.s * t.cv;  tw[3] = t.s * t.sv;
  tw[4] = -t.s * t.cw; tw[5] = -t.s * t.sw;
  tw[6] = t.c * t.cz;  tw[7] = t.c * t.sz;
}

// angles[4], g[8] (gradient of the 8 floats above) -> d[4] (gradient of phi, alpha, psi, chi)
BFLY_HD void unitary_block_bw(const float* a, const float* g, float* d) {
  const UnitaryTrig t = unitary_trig(a);
  // radial parts: d/dphi of (c, s, -s, c) times the unit phasors
  const float ra = t.cu * g[0] + t.su * g[1], rb = t.cv * g[2] + t.sv * g[3];
  const float rc = t.cw * g[4] + t.sw * g[5], rd = t.cz * g[6] + t.sz * g[7];
  d[0] = -t.s * ra + t.c * rb - t.c * rc - t.s * rd;
  // angular parts: derivative with respect to each entry's own phase
  const float ta = t.c * (-t.su * g[0] + t.cu * g[1]), tb = t.s * (-t.sv * g[2] + t.cv * g[3]);
  const float tc = -t.s * (-t.sw * g[4] + t.cw * g[5]), td = t.c * (-t.sz * g[6] + t.cz * g[7]);
  d[1] = ta + tb + tc + td;
  d[2] = ta - td;
  d[3] = tb - tc;
}

}  // namespace bfly
