// msl_ref.cpp -- runs the reference's own emitted RK4 Lotka-Volterra kernel
// (tests/golden/rk4_lotka_volterra.metal: 500 steps, dt = 0.01, one program
// instance per trajectory) on the CPU.  TEST INFRASTRUCTURE ONLY.
//
// The .metal file is not copied: the build passes its location in the
// reference checkout as PD_GOLDEN_RK4 and it is #included from there.  It is
// scalar MSL that is also valid C++ once <metal_stdlib> resolves to the shim
// in oracle/msl_shim/.  Built with -ffp-contract=off so every statement is one
// IEEE binary32 operation, as written.
#include <stdint.h>

#include PD_GOLDEN_RK4

extern "C" __attribute__((visibility("default")))
void ref_rk4_lv_golden(int64_t n, const float* x0, const float* y0, const float* a, const float* b,
                       const float* c, const float* d, float* xo, float* yo) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        uint3 pid = {(uint)i, 0u, 0u};
        palladium_kernel(x0, y0, a, b, c, d, xo, yo, pid);
    }
}
