/* Test infrastructure, not product code.
 *
 * CPU oracle for the butterfly multiply: a plain-C restatement of
 *   csrc/cpu/butterfly_cpu.cpp:17-66   (forward)
 *   csrc/cpu/butterfly_cpu.cpp:68-177  (backward)
 *   torch_butterfly/multiply_base4.py:7-41 (base-4 forward; its backward is the adjoint)
 * of the reference, instantiated for float, double, complex-float and
 * complex-double (complex elements are stored re, im interleaved).
 *
 * Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
 * load this library; the shipped CUDA path never does.
 *
 * Build:  gcc -O2 -ffp-contract=off -fPIC -shared bfly_oracle.c -o libbfly_oracle.so
 * (-ffp-contract=off keeps every product separately rounded, as the reference's
 * CPU build does, so float results are bit-identical to the reference CPU op.)
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define R float
#define NC 1
#define FN(x) CAT(x, _f32)
#include "bfly_oracle_impl.h"
#undef R
#undef NC
#undef FN

#define R double
#define NC 1
#define FN(x) CAT(x, _f64)
#include "bfly_oracle_impl.h"
#undef R
#undef NC
#undef FN

#define R float
#define NC 2
#define FN(x) CAT(x, _c64)
#include "bfly_oracle_impl.h"
#undef R
#undef NC
#undef FN

#define R double
#define NC 2
#define FN(x) CAT(x, _c128)
#include "bfly_oracle_impl.h"
#undef R
#undef NC
#undef FN
