// Run-time compiled ensemble kernels (PD_FAMILY_CUSTOM_ODE).
//
// The reference hands its native handler MSL source text plus an entry-point
// name and compiles it on first use, keeping the compiled pipeline for the
// life of the process (native/ffi/palladium_ffi.cpp:44-49,75-84,136-148).  The
// same mechanism here: the caller supplies the right-hand side of an ODE as
// CUDA C statements, the library wraps it in one of its integrator loops,
// compiles the text with NVRTC under the flag set of the requested math mode,
// loads the result with the driver API and caches it by source text.
#ifndef PD_RTC_H_
#define PD_RTC_H_

#include <cstddef>
#include <cstdint>
#include <string>

#include "../../include/palladium_cuda.h"

// Kernel argument block of the generated kernels (the generated source declares
// the same struct; both sides are checked against each other by a size constant).
struct PdOdeArgs {
    const float* in[16];   // dim state arrays, then nparam parameter arrays, each (n) f32
    float* out[16];        // RK4: dim arrays.  BS3(2): t, dim arrays, steps, rejected, real
    long long n;
    unsigned long long* cursor;   // BS3(2): the next unclaimed system (zeroed before the launch)
    int steps;             // RK4 step count
    int max_steps;         // BS3(2) attempt limit
    int refill_every;      // BS3(2): attempts between refill checks
    float h_half, h_full, h_sixth;
    float t1, rtol, atol, dt0, safety, factor_min, factor_max, coeff1, coeff2;
};

struct PdRtcKernel {
    void* function = nullptr;   // CUfunction
    int regs = -1;
    int static_smem = -1;
    int blocks_per_sm = -1;     // at the block size asked for
    char name[64] = {0};
};

// Validates the block (dim, nparam, method, source present).  Never touches a device.
int pd_rtc_check_params(const pd_custom_ode_params* p, char* err, size_t err_cap);

// Compiles the kernel for `arch` ("sm_100a", ...) without loading it; `log`
// receives the compiler's messages.  Needs NVRTC but no device.
int pd_rtc_compile_only(const pd_custom_ode_params* p, int math_mode, const char* arch, std::string* log,
                        char* err, size_t err_cap);

// Compiled + loaded kernel for the current device (cached).  block is used for
// the occupancy figure only.
int pd_rtc_get(const pd_custom_ode_params* p, int math_mode, int device, int block, PdRtcKernel* out, char* err,
               size_t err_cap);

// Launches on `stream` (a cudaStream_t).
int pd_rtc_launch(const PdRtcKernel& k, long long grid, int block, const PdOdeArgs& args, void* stream, char* err,
                  size_t err_cap);

const char* pd_rtc_kernel_name(const pd_custom_ode_params* p);

// Caller-written kernels (PD_FAMILY_SOURCE): the same compile / cache / load path
// on complete CUDA source; the kernel takes one pointer per buffer (inputs, then
// outputs) followed by the three extents of the logical grid.
int pd_rtc_check_source(const pd_source_kernel_params* p, char* err, size_t err_cap);
int pd_rtc_get_source(const pd_source_kernel_params* p, int math_mode, int device, int block, PdRtcKernel* out,
                      char* err, size_t err_cap);
int pd_rtc_launch_source(const PdRtcKernel& k, const int64_t cuda_grid[3], const int64_t block[3],
                         const int64_t logical_grid[3], int n_buffers, void* const* buffers, void* stream, char* err,
                         size_t err_cap);

#endif  // PD_RTC_H_
