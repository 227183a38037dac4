/* palladium_cuda.h -- C ABI of libpalladium_cuda.so, the CUDA (sm_100a) handler
 * that takes the place of the reference's only native component, the XLA-FFI
 * handler `palladium_dispatch` (native/ffi/palladium_ffi.cpp:110-209).
 *
 * The reference handler receives MSL source + entry-point name + grid +
 * threadgroup + math_mode as attributes and a list of argument / result
 * buffers.  Here the kernels are fixed, hand-written CUDA families, so the
 * `msl_source` / `function_name` pair is replaced by a family id and a small
 * parameter struct; everything else (grid, threadgroup, math_mode ordinal,
 * "remaining args" / "remaining rets" as pointer arrays) keeps its meaning.
 *
 * All entry points are plain C: pointers, sizes, ints.  No entry point takes
 * ownership of a caller buffer.  Every function that can fail returns a
 * pd_status and, when `err` is non-NULL, copies a NUL-terminated message into
 * the caller's buffer (the reference returns a malloc'ed message that must be
 * freed with mr_free_error_message, palladium_ffi.cpp:55-63; copying into the
 * caller's buffer avoids a cross-library free).
 */
#ifndef PALLADIUM_CUDA_H_
#define PALLADIUM_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PD_ABI_VERSION 1

#if defined(__GNUC__)
#define PD_API __attribute__((visibility("default")))
#else
#define PD_API
#endif

typedef enum pd_status {
    PD_OK = 0,
    PD_ERR_INVALID_ARGUMENT = 1, /* maps to xla::ffi::Error::InvalidArgument (palladium_ffi.cpp:118-121) */
    PD_ERR_INTERNAL = 2,         /* maps to xla::ffi::Error::Internal (palladium_ffi.cpp:126,139,147,167) */
    PD_ERR_CUDA = 3,             /* a CUDA runtime call failed; message carries cudaGetErrorString */
    PD_ERR_DEVICE_STATUS = 4     /* a kernel's bounded wait ran out (the register-tile stencil waits, with a limit, for its tile copies); see pd_device_status */
} pd_status;

/* MRMathMode ordinals as the reference passes them (src/palladium/ffi.py:38;
 * range check at native/ffi/palladium_ffi.cpp:118-121). */
typedef enum pd_math_mode {
    PD_MATH_SAFE = 0,    /* IEEE op order, no FMA contraction, IEEE div/sqrt, no flush-to-zero */
    PD_MATH_RELAXED = 1, /* FMA contraction allowed, accurate div/sqrt/libm */
    PD_MATH_FAST = 2     /* reassociation + approximate transcendentals + flush-to-zero */
} pd_math_mode;

/* Kernel families: one per reference kernel on the integrator path. */
typedef enum pd_family {
    PD_FAMILY_LV_RK4 = 0,        /* lv_kernel, examples/01_ode_ensembles.py:72-91 */
    PD_FAMILY_VDP_BS32 = 1,      /* vdp_adaptive_kernel, examples/02_adaptive_lockstep.py:69-171 */
    PD_FAMILY_GBM_THREEFRY = 2,  /* pallas_gbm_kernel, examples/03_sde_montecarlo.py:97-119 */
    PD_FAMILY_GRAY_SCOTT = 3,    /* gray_scott_kernel + stepping loop, examples/04_reaction_diffusion.py:61-109 */
    PD_FAMILY_LV_RK4_DF32 = 4,   /* lv_rk4_df32, examples/05_df32_precision.py:27-80 */
    PD_FAMILY_KEPLER_RK4_DF32 = 5, /* same df32 RK4 scheme on the two-body problem */
    PD_FAMILY_THREEFRY_BITS = 6, /* random_bits / uniform / fold_in, src/palladium/emit/rules.py:168-201 */
    PD_FAMILY_GBM_PCG = 7,       /* gbm_paths with pcg_hash, the hand-written kernel GBM_MSL, examples/03_sde_montecarlo.py:34-70 */
    PD_FAMILY_CUSTOM_ODE = 8,    /* a caller-supplied right-hand side, compiled at run time: the counterpart of
                                    handing the handler MSL source + entry-point name, native/ffi/palladium_ffi.cpp:136-148 */
    PD_FAMILY_SOURCE = 9,        /* a complete caller-written kernel: source text + entry-point name, the
                                    attributes of the reference handler itself, native/ffi/palladium_ffi.cpp:110-117 */
    PD_FAMILY_COUNT = 10
} pd_family;

/* ---- per-family parameter blocks (passed by pointer + sizeof) ------------ */

/* in:  x0,y0,a,b,c,d  (N) f32.   out: x,y (N) f32, or one (N,2) f32 array of (x, y) pairs.
 * The three step constants are rounded to f32 from double products exactly as
 * Python folds them: f32(0.5*dt), f32(dt), f32(dt/6). */
typedef struct pd_lv_rk4_params {
    double dt;
    int64_t steps;
} pd_lv_rk4_params;

/* in:  x0,v0,mu (N) f32 [, order (N) i32: the sequence in which the kernel's work
 *      queue hands out the trajectories, a permutation of 0..N-1; results do not
 *      depend on it, run time does (longest first is best); entries outside
 *      [0, N) are skipped].
 * out_layout 0: t,x,v,steps,rejected,real  (6 x (N) f32)   examples/02:173-181
 * out_layout 1: t,x,v,steps,rejected       (5 x (N) f32)   tests/test_08_adaptive.py:33-142
 * out_layout 2: state (N,2) f32, accepted (N) i32, rejected (N) i32
 *               (accepted == the reference's `real` counter). */
typedef struct pd_vdp_bs32_params {
    double t1, rtol, atol, dt0;
    double pcoeff, icoeff, safety, factor_min, factor_max;
    int64_t error_order;
    int64_t max_steps;
    int64_t out_layout;
} pd_vdp_bs32_params;

/* in:  key data (2) u32.   out[0]: (N) f32 payoff (output_kind 0) or terminal
 * price (output_kind 1); optional out[1]: (2) f64 = {sum payoff, sum payoff^2}
 * over this call's paths.  Path i uses RNG stream fold_in(key, path_offset+i). */
/* PD_FAMILY_GBM_PCG takes the same block and no input: path i, step s draws
 * u1 = uniform01(2*c), u2 = uniform01(2*c + 1) with c = (path_offset + i) * steps + s
 * in 32-bit arithmetic (examples/03_sde_montecarlo.py:60-62). */
typedef struct pd_gbm_params {
    double s0, strike, r, sigma, t;
    int64_t steps;
    int64_t path_offset;
    int64_t output_kind;
} pd_gbm_params;

/* in:  u,v (rows_alloc, cols) f32 row-major.   out: u,v same shape.
 * halo == 0: rows_alloc == rows, periodic in both directions (the reference).
 * halo  > 0: a row slab with `halo` ghost rows above and below
 *            (rows_alloc == rows + 2*halo), periodic in columns only; step s
 *            (1-based, steps <= halo) updates rows [s, rows_alloc - s). */
typedef struct pd_gray_scott_params {
    double du, dv, f, k, dt;
    int64_t steps;
    int64_t rows, cols;
    int64_t halo;
} pd_gray_scott_params;

/* in:  x0,y0,a,b,c,d (N) f32.   out: x,y (N) f32 (df32 state rounded to f32).
 * dt is rounded to f32 first, as the reference passes a float scalar. */
typedef struct pd_lv_rk4_df32_params {
    double dt;
    int64_t steps;
} pd_lv_rk4_df32_params;

/* in:  x,y,vx,vy each as (hi, lo): 8 x (N) f32.   out: same 8 arrays.
 * dt and gm are split into df32 (hi, lo) from the doubles given here. */
typedef struct pd_kepler_rk4_df32_params {
    double dt, gm;
    int64_t steps;
} pd_kepler_rk4_df32_params;

/* in:  key data (2) u32 [, data (M) u32 for op 2].
 * op 0: out (N) u32 = random_bits(key, (N,))
 * op 1: out (N) f32 = uniform(key, (N,))
 * op 2: out (M,2) u32 = key_data(fold_in(key, data[m]))
 * op 3: out (G,count) f32, row g = uniform(fold_in(key, g), (count,))
 * op 4: out (N) u32 = pcg_hash(i)   (key is ignored) */
typedef struct pd_threefry_params {
    int64_t op;
    int64_t count;
} pd_threefry_params;

/* An ensemble of independent ODE systems y' = f(t, y, p) whose right-hand side
 * the caller writes as CUDA C statements, the body of
 *     void rhs(float t, const float* y, const float* p, float* dy)
 * (y and dy have `dim` elements, p has `nparam`; pd_math.h's helpers, e.g.
 * pd_powf and the df32 operations, are in scope).  The library wraps it in an
 * integrator loop, compiles the text with NVRTC under the flag set of the math
 * mode (first use of a source text; cached for the process, as the reference
 * caches compiled pipelines by source text, palladium_ffi.cpp:44-49,75-84) and
 * launches one thread per system.
 *   method PD_ODE_RK4:  classic RK4, `steps` steps of `dt`; the arithmetic order
 *     of the Lotka-Volterra family (stage y + f32(dt/2)*k, combine
 *     ((k1 + 2 k2) + 2 k3) + k4, times f32(dt/6)).
 *     in: dim state arrays then nparam parameter arrays, (N) f32.  out: dim arrays.
 *   method PD_ODE_BS32: Bogacki-Shampine 3(2) with the PI controller, counters
 *     and stall semantics of the Van der Pol family.
 *     in: as above.  out: t, dim state arrays, steps, rejected, real, (N) f32.
 *   method PD_ODE_DOPRI5, PD_ODE_TSIT5: the seven-stage 5(4) pairs of Dormand and
 *     Prince and of Tsitouras (the pair the reference's CPU comparison runs,
 *     benchmarks/bench_ensembles.py:88-118) under the same controller, counters
 *     and outputs as PD_ODE_BS32; error_order is 5 for them.
 * Compiler errors in the right-hand side come back as PD_ERR_INVALID_ARGUMENT
 * with the compiler's log in `err`. */
#define PD_ODE_RK4 0
#define PD_ODE_BS32 1
#define PD_ODE_DOPRI5 2
#define PD_ODE_TSIT5 3
#define PD_ODE_MAX_DIM 8
#define PD_ODE_MAX_PARAM 8
typedef struct pd_custom_ode_params {
    const char* rhs_source;   /* NUL-terminated; must stay valid for the call only */
    int64_t dim, nparam, method;
    double dt;                /* RK4 */
    int64_t steps;
    double t1, rtol, atol, dt0;   /* the adaptive methods */
    double pcoeff, icoeff, safety, factor_min, factor_max;
    int64_t error_order;
    int64_t max_steps;
} pd_custom_ode_params;

/* A complete kernel of the caller's, as CUDA C source: what the reference's
 * handler receives as `msl_source` + `function_name` (palladium_ffi.cpp:110-117),
 * compiled on the first use of a (source, name, math mode) and kept for the
 * life of the process (:44-49,75-84).  The kernel must be declared
 *     extern "C" __global__ void <function_name>(T0* b0, ..., Tk* bk,
 *                                                long long gx, long long gy, long long gz)
 * with one pointer per buffer in binding order -- inputs first, then outputs,
 * the order the reference binds them (:128-148) -- followed by the extents of
 * the logical grid.  One thread is launched per grid point, rounded up to whole
 * blocks, so the kernel returns when (PD_THREAD_X, PD_THREAD_Y, PD_THREAD_Z)
 * lies outside (gx, gy, gz); those macros and pd_math.h are in scope.
 * `block` is the threadgroup; (0,0,0) lets the library choose (:158-162).
 * Buffer sizes are the caller's business: none are checked. */
typedef struct pd_source_kernel_params {
    const char* cuda_source;     /* NUL-terminated; must stay valid for the call only */
    const char* function_name;   /* at most 63 bytes */
} pd_source_kernel_params;

/* ---- launch geometry report (the `.explain()` payload) -------------------- */
typedef struct pd_launch_info {
    char kernel_name[64];
    int64_t cuda_grid[3];
    int64_t cuda_block[3];
    int64_t items_per_thread;
    int64_t launches;          /* kernel launches one call performs */
    int64_t scratch_bytes;     /* device scratch the call needs beyond in/out */
    int32_t regs_per_thread;   /* -1 when no CUDA device is present */
    int32_t static_smem_bytes; /* -1 when no CUDA device is present */
    int32_t dynamic_smem_bytes;
    int32_t blocks_per_sm;     /* occupancy; -1 when no CUDA device is present */
} pd_launch_info;

/* ---- row slabs on several GPUs: the halo exchange from inside the kernel ----
 * The reference has no multi-device code; this is the multi-GPU form of its
 * stepping loop (examples/04_reaction_diffusion.py:92-109).  A slab call
 * (pd_launch, PD_FAMILY_GRAY_SCOTT, halo > 0) leaves rows [halo, halo + rows)
 * valid; the neighbours above and below need this slab's first and last `halo`
 * owned rows in their ghost rows before their next call.  pd_gray_scott_slab_push
 * is the same call with the neighbours' OUTPUT fields given as peer device
 * pointers (mapped with pd_peer_open below): the final launch of the call stores
 * the boundary rows to its own output and, from the same registers, to the
 * neighbours' ghost rows, plain stores that travel over NVLink.  Nothing waits
 * inside the kernel: the caller orders "every rank's call has finished" before
 * any rank's next call (one barrier on the host or a one-element all-reduce on
 * the stream), and alternates two output sets so that a neighbour never reads
 * the set being pushed into.
 *   up_*:   fields of the slab that owns the rows above this one; this slab's rows
 *           [halo, 2*halo) land in its rows [halo + up_rows, 2*halo + up_rows).
 *   down_*: fields of the slab below; this slab's rows [rows, rows + halo) land
 *           in its rows [0, halo).
 * Requires rows >= halo.  On one rank (periodic wrap onto itself) the neighbours
 * are the call's own outputs. */
typedef struct pd_gs_neighbours {
    void* up_u;
    void* up_v;
    int64_t up_rows;     /* owned rows of the upper neighbour (its fields have up_rows + 2*halo rows) */
    void* down_u;
    void* down_v;
    int64_t down_rows;
} pd_gs_neighbours;

PD_API int pd_gray_scott_slab_push(const pd_gray_scott_params* params, int math_mode,
                                   const void* u, const void* v, void* uo, void* vo,
                                   const pd_gs_neighbours* neighbours,
                                   void* workspace, size_t workspace_bytes,
                                   void* cuda_stream, char* err, size_t err_cap);

/* Device memory that another process on the same node can map (CUDA IPC):
 * pd_peer_alloc returns a whole allocation, pd_peer_export its 64-byte handle,
 * pd_peer_open maps a handle received from another rank (peer access is enabled
 * on first use), pd_peer_close / pd_peer_free release them. */
#define PD_PEER_HANDLE_BYTES 64
PD_API int pd_peer_alloc(size_t bytes, void** ptr, char* err, size_t err_cap);
PD_API int pd_peer_export(void* ptr, unsigned char handle[PD_PEER_HANDLE_BYTES], char* err, size_t err_cap);
PD_API int pd_peer_open(const unsigned char handle[PD_PEER_HANDLE_BYTES], void** ptr, char* err, size_t err_cap);
PD_API int pd_peer_close(void* ptr, char* err, size_t err_cap);
PD_API int pd_peer_free(void* ptr, char* err, size_t err_cap);

/* Compile a PD_FAMILY_CUSTOM_ODE right-hand side for sm_100a without loading or
 * launching it: needs NVRTC but no CUDA device, so a host can reject a faulty
 * right-hand side where it is defined (the reference raises at trace time,
 * before any dispatch).  `log` receives the compiler's messages. */
PD_API int pd_custom_ode_check(const pd_custom_ode_params* params, size_t params_bytes, int math_mode,
                               char* log, size_t log_cap, char* err, size_t err_cap);

/* The text handed to the compiler for a PD_FAMILY_CUSTOM_ODE call (defines,
 * shared prologue, the right-hand side, the integrator kernel): what the
 * reference's `debug_msl` shows of an emitted kernel
 * (src/palladium/__init__.py:162-190).  `needed` receives the size including the
 * terminating NUL; the text is truncated to out_cap. */
PD_API int pd_custom_ode_source(const pd_custom_ode_params* params, size_t params_bytes, int math_mode,
                                char* out, size_t out_cap, size_t* needed, char* err, size_t err_cap);

/* The same for a PD_FAMILY_SOURCE kernel. */
PD_API int pd_source_kernel_check(const pd_source_kernel_params* params, size_t params_bytes, int math_mode,
                                  char* log, size_t log_cap, char* err, size_t err_cap);

/* ABI version of the loaded library (== PD_ABI_VERSION it was built with). */
PD_API int pd_version(void);

/* Number of CUDA devices visible, or 0 (never fails). */
PD_API int pd_device_count(void);

/* Launch one call of a family on DEVICE buffers, stream-ordered, no host
 * synchronisation.  Replaces the dispatch half of PalladiumDispatch
 * (palladium_ffi.cpp:150-165) for callers that already hold device memory.
 *   grid / block: the reference's grid (padded to 3 dims, ffi.py:167-169) and
 *   threadgroup (0,0,0 = library chooses, palladium_ffi.cpp:158-162).
 *   workspace: optional caller-provided device scratch of at least
 *   pd_launch_info.scratch_bytes; NULL lets the library use its cached pool. */
PD_API int pd_launch(int family, const void* params, size_t params_bytes, int math_mode,
              const int64_t grid[3], const int64_t block[3],
              int n_in, const void* const* in, const size_t* in_bytes,
              int n_out, void* const* out, const size_t* out_bytes,
              void* workspace, size_t workspace_bytes,
              void* cuda_stream, char* err, size_t err_cap);

/* Same call on HOST buffers: uploads the inputs, launches, downloads the
 * outputs and returns when they are in place -- the contract of the reference
 * handler, which is registered on XLA's "cpu" platform and blocks until the
 * outputs are flushed (src/palladium/ffi.py:78; palladium_ffi.cpp:165-188).
 * Thread-safe; device staging buffers come from a per-thread cached pool. */
PD_API int pd_dispatch_host(int family, const void* params, size_t params_bytes, int math_mode,
                     const int64_t grid[3], const int64_t block[3],
                     int n_in, const void* const* in, const size_t* in_bytes,
                     int n_out, void* const* out, const size_t* out_bytes,
                     char* err, size_t err_cap);

/* The same call in two halves, for callers that keep several calls in flight: what
 * BoundKernel.launch() / PendingResult.wait() are in the reference
 * (src/palladium/dispatch.py:129-194; docs/performance.md:35-40 quotes 33 us per
 * dispatch at depth 16 against 136 us for a blocking one).
 * pd_submit_host copies the inputs into page-locked memory of the library -- the
 * caller's arrays may change as soon as it returns --, queues one upload, the
 * kernels and one download on a stream of the call's own and hands back a ticket.
 * pd_wait_host blocks until that call has finished, copies the results into `out`
 * (sizes as submitted) and retires the ticket; with n_out == 0 it only retires it.
 * `out` of pd_submit_host is NULL for that form.  Alternatively it names the result
 * arrays up front: they must be page-locked (an ordinary array would make the
 * submission wait for the kernels) and stay alive until the wait, which is then
 * called with n_out == 0 and copies nothing.
 * `in_on_device` is NULL, or says per input (non-zero) that `in[i]` is device memory
 * already -- inputs uploaded once and used by many calls, the reference's
 * `call.pin(*arrays)` (src/palladium/dispatch.py:230-255); such memory must stay
 * alive and unchanged until the wait.
 * At most 64 calls may be in flight in a process; every ticket must be waited for. */
PD_API int pd_submit_host(int family, const void* params, size_t params_bytes, int math_mode,
                   const int64_t grid[3], const int64_t block[3],
                   int n_in, const void* const* in, const size_t* in_bytes, const int* in_on_device,
                   int n_out, void* const* out, const size_t* out_bytes, uint64_t* ticket,
                   char* err, size_t err_cap);
PD_API int pd_wait_host(uint64_t ticket, int n_out, void* const* out, const size_t* out_bytes,
                 char* err, size_t err_cap);

/* Launch geometry for a call, without launching anything (the native half of
 * MetalCallable.explain, src/palladium/__init__.py:116-128).  Works without a
 * GPU; the register / shared-memory / occupancy fields are then -1. */
PD_API int pd_explain(int family, const void* params, size_t params_bytes, int math_mode,
               const int64_t grid[3], const int64_t block[3],
               pd_launch_info* info, char* err, size_t err_cap);

/* Tuning knobs for experiments (e.g. "lv_items_per_thread", "vdp_variant") and for
 * the host-buffer path: "host_streams" (streams the chunks of a large call rotate
 * over), "host_chunks", "host_copy_threads" (helper threads that stage inputs from
 * ordinary, pageable memory into page-locked buffers for calls of 16 MB and more;
 * 0 leaves such inputs to the driver's own pageable copy).
 * Returns PD_ERR_INVALID_ARGUMENT for an unknown key. */
PD_API int pd_set_tuning(const char* key, int64_t value);
PD_API int pd_get_tuning(const char* key, int64_t* value);

/* The same knobs, overridden for the calling thread only: calls made by this
 * thread see `value`, every other thread keeps the process-wide setting.  This
 * is how one call picks a kernel variant without changing what concurrent
 * callers run (the reference has no counterpart: its only per-call choices are
 * math_mode and threadgroup, src/palladium/__init__.py:222-226).
 * pd_clear_thread_tuning(NULL) drops all of the thread's overrides.
 * pd_get_tuning reports the value the calling thread would use. */
PD_API int pd_set_thread_tuning(const char* key, int64_t value);
PD_API int pd_clear_thread_tuning(const char* key);

/* Roofline denominators measured on the current device: a chain of dependent
 * FP32 FMAs (2 flops each) and a chain of 32-bit integer add/xor/funnel-shift
 * operations, both with enough independent chains per thread to saturate issue.
 * Results in operations per second.  Time is taken with CUDA events. */
PD_API int pd_measure_fp32_fma_peak(double* flops_per_s, char* err, size_t err_cap);
PD_API int pd_measure_int32_alu_peak(double* ops_per_s, char* err, size_t err_cap);

/* Milliseconds the kernels of the most recent pd_launch / pd_dispatch_host
 * call of the calling thread took on the device (CUDA events on the launch
 * stream), or a negative value if timing was not enabled.  Enable with
 * pd_set_tuning("time_kernels", 1); it adds an event pair and a synchronise. */
PD_API double pd_last_kernel_ms(void);

/* The status word of the current device: 0, or the code a kernel recorded when
 * one of its bounded waits ran out (1: a tile copy of the register-tile stencil
 * kernel did not arrive within its limit -- that call's outputs are not valid).
 * No kernel of this library waits on another kernel or another GPU; the only
 * device-side waits are a warp's waits for its own asynchronous tile copies.
 * pd_dispatch_host checks the word itself after its final synchronise and
 * returns PD_ERR_DEVICE_STATUS; after stream-ordered pd_launch calls, read it
 * here once the stream has been synchronised.  `clear` != 0 resets it.
 * No counterpart in the reference, whose dispatch blocks and reports through
 * its status code alone (native/ffi/palladium_ffi.cpp:176-188). */
PD_API int pd_device_status(int* code, int clear, char* err, size_t err_cap);

/* Multi-step Gray-Scott on DEVICE buffers that allocates no device memory.
 * No counterpart in the reference (its stepping loop lets metal-runtime
 * allocate, examples/04_reaction_diffusion.py:92-98): it is for hosts that
 * cannot let this library call cudaMalloc -- a process whose runtime reserved
 * the GPU memory pool up front (XLA with preallocation, which is where the FFI
 * handler runs), or a fixed-budget stepping loop that cannot take the
 * device-wide synchronisation of cudaMalloc / cudaFree.
 *   Same arithmetic, parameters and buffer layout as
 *   pd_launch(PD_FAMILY_GRAY_SCOTT, ...); u, v are inputs, uo, vo outputs, each
 *   (rows + 2*halo) x cols float32.  The ping-pong fields of a call with
 *   steps >= 2 live in a fixed 8 MiB array inside the library image, held by
 *   every GPU the library is used on until the process exits.
 *   Limit: (rows + 2*halo) * cols <= 1 048 576 cells (2^20); larger calls return
 *   PD_ERR_INVALID_ARGUMENT.  All calls on a device share that array: calls
 *   whose kernels overlap on the GPU race on it, so order them on one stream.
 *   Nothing in the array needs clearing between calls.  The first call on a
 *   device resolves the array's address (cudaGetSymbolAddress); make it with
 *   that device current and before beginning any stream capture. */
PD_API int pd_gray_scott_static(const pd_gray_scott_params* params, int math_mode,
                                const void* u, const void* v, void* uo, void* vo,
                                void* cuda_stream, char* err, size_t err_cap);

#ifdef __cplusplus
}
#endif
#endif /* PALLADIUM_CUDA_H_ */
