// msl_gbm_ref.cpp -- runs the reference's hand-written Monte Carlo kernel
// `gbm_paths` (the GBM_MSL text of examples/03_sde_montecarlo.py:34-70: pcg_hash,
// uniform01, Box-Muller, the path loop) on the CPU.  TEST INFRASTRUCTURE ONLY.
//
// The MSL text is not copied into this repository: oracle/build.py takes the
// string out of the example where it lies, writes it under oracle/_ref/ and
// passes its location as PD_GBM_MSL.  It is scalar MSL that is valid C++ once
// <metal_stdlib> resolves to the shim in oracle/msl_shim/; the float math
// functions resolve to the C library's (Metal's own differ by rounding).
#include <stdint.h>

#include PD_GBM_MSL

extern "C" __attribute__((visibility("default")))
void ref_gbm_paths(int64_t n, uint32_t n_steps, float s0, float strike, float drift_dt, float vol_sqdt,
                   float* payoff) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) gbm_paths(payoff, n_steps, s0, strike, drift_dt, vol_sqdt, (uint)i);
}

extern "C" __attribute__((visibility("default")))
void ref_pcg_hash(int64_t n, const uint32_t* in, uint32_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = pcg_hash(in[i]);
}
