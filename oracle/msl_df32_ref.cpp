// msl_df32_ref.cpp -- runs the reference's hand-written df32 kernel `lv_rk4_df32`
// (the DF32_KERNEL text of examples/05_df32_precision.py:27-80: operator
// overloads, rhs, advance, the RK4 loop) on the CPU.  TEST INFRASTRUCTURE ONLY.
//
// The MSL text is not copied into this repository: oracle/build.py takes the
// string out of the example where it lies, writes it under oracle/_ref/ and
// passes its location as PD_DF32_MSL.  The kernel text relies on a prelude the
// reference gets from the external metal-runtime project (type df32 and
// df_add / df_sub / df_mul / df_from_float / df_to_float); that prelude is not
// in the reference tree, so the one below is this oracle's restatement
// (df32_ops.h).  What this build pins is therefore the kernel's structure --
// which operations, in which order, on which constants -- not the prelude's
// arithmetic.
#include <stdint.h>
#include <metal_stdlib>
using namespace metal;

#include "df32_ops.h"
typedef df df32;
static inline df32 df_from_float(float a) { return dfc(a); }
static inline float df_to_float(df32 a) { return a.hi; }

#include PD_DF32_MSL

extern "C" __attribute__((visibility("default")))
void ref_lv_rk4_df32(int64_t n, const float* x0, const float* y0, const float* a, const float* b, const float* c,
                     const float* d, float* xo, float* yo, float dt, uint32_t steps) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) lv_rk4_df32(x0, y0, a, b, c, d, xo, yo, dt, steps, (uint)i);
}
