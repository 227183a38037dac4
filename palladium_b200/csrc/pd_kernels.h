// pd_kernels.h -- argument blocks and per-math-mode launcher tables shared by
// the C-ABI layer (pd_api.cu) and the kernel translation unit (pd_kernels.cu),
// which is compiled once per math mode with a different nvcc flag set:
//   SAFE    -DPD_MODE=0  -fmad=false -prec-div=true  -prec-sqrt=true  -ftz=false
//   RELAXED -DPD_MODE=1  -fmad=true  -prec-div=true  -prec-sqrt=true  -ftz=false
//   FAST    -DPD_MODE=2  -use_fast_math
#ifndef PD_KERNELS_H_
#define PD_KERNELS_H_

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

struct PdLvArgs {
    const float *x0, *y0, *a, *b, *c, *d;
    float *xo, *yo;
    float* state2_out;  // when set, the final state goes here as (N, 2) interleaved pairs instead of xo / yo
    int64_t n;
    int steps;
    float h_half, h_full, h_sixth;
    int packed;   // two trajectories per packed f32x2 operation (kernels with 2 or 4 trajectories per thread)
    float neg_zero;   // -0.0f, as a run-time value (see p_mad in pd_kernels.cu)
};

struct PdVdpArgs {
    const float *x0, *v0, *mu;
    const int32_t* order;  // optional: the sequence in which the queue hands out trajectories (a permutation of 0..n-1)
    // any output pointer may be null
    float *t_out, *x_out, *v_out, *steps_out, *rejected_out, *real_out;
    float *state2_out;
    int32_t *accepted_i32, *rejected_i32;
    unsigned long long* cursor;  // work-queue head (scratch, zeroed by the caller)
    int64_t n;
    int max_steps;
    int refill_every;  // attempts between two refill checks of a warp
    // variant 3 (two passes): pass one suspends what is unfinished after `pass_limit`
    // attempts and files it under a bucket of predicted remaining attempts; pass two
    // resumes the suspended states, longest predicted first.
    int pass_limit;                     // 0: never suspend
    int pass_limits[3];                 // host side: the caps of the suspending passes, ascending, 0 = unused
    int resume;                         // lanes start from suspended states
    const unsigned long long* n_dev;    // queue length in device memory (pass two), or null for n
    unsigned long long* cursor2;        // pass two's queue head
    unsigned long long* n_susp;         // number of suspended trajectories (written between the passes)
    float* susp;                        // 10 arrays of n words: t, dt, x, v, k1x, k1v, prev_pow, rejected, real, iter
    int32_t* bucket_of;                 // bucket of each suspended trajectory, -1 otherwise
    unsigned int* hist;                 // 64 bucket counters
    unsigned int* offsets;              // 64 write positions
    int32_t* order2;                    // pass two's hand-out order
    int compact_every; // variant 2: refill rounds between two block-level compactions
    long long round_limit;  // variant 2: upper bound on rounds (list-scheduling bound), a guard against endless loops
    float t1, rtol, atol, dt0, safety, factor_min, factor_max, coeff1, coeff2;
};

struct PdGbmArgs {
    const uint32_t* key;
    float* out;
    double* block_partials;  // scratch: 2 doubles per block
    int64_t n;
    uint32_t path_offset;
    int steps;
    int output_kind;
    int rng;  // 0 Threefry keyed by `key`, 1 pcg_hash of a running counter
    float s0, strike, drift_dt, vol_sqdt;
};

struct PdGsArgs {
    const float *u, *v;
    float *uo, *vo;
    int rows_alloc, cols;
    int row_lo, row_hi;  // rows updated by this launch: [row_lo, row_hi)
    int periodic_rows;
    float du, dv, f, fk, dt;
    // Row slabs on several GPUs: when `push` is set, output rows [top_lo, top_hi)
    // are also stored to the upper neighbour's fields at row + up_shift, and rows
    // [bot_lo, bot_hi) to the lower neighbour's at row + dn_shift (its ghost rows;
    // peer device memory, plain stores over NVLink).
    int push;
    int top_lo, top_hi, up_shift;
    int bot_lo, bot_hi, dn_shift;
    float *up_u, *up_v, *dn_u, *dn_v;
    // Register-tile kernel: bound on the polls of a tile copy's barrier, the longer bound used once
    // the first has run out (the copy in flight must land before the block may exit), and the word
    // that receives a non-zero code when a wait ran out (device-visible, may be null).
    long long wait_limit, drain_limit;
    int* status;
};

struct PdDfLvArgs {
    const float *x0, *y0, *a, *b, *c, *d;
    float *xo, *yo;
    int64_t n;
    int steps;
    float dt;
};

struct PdKeplerArgs {
    const float* in[8];
    float* out[8];
    int64_t n;
    int steps;
    float dt_hi, dt_lo, gm_hi, gm_lo;
};

struct PdThreefryArgs {
    const uint32_t* key;
    const uint32_t* data;
    void* out;
    int64_t n;      // outputs (op 0/1), data items (op 2), groups (op 3)
    int64_t count;  // draws per group (op 3)
    int op;
};

// One table per math mode.
struct PdModeTable {
    cudaError_t (*lv_rk4)(const PdLvArgs&, int items_per_thread, int block, cudaStream_t);
    cudaError_t (*vdp_bs32)(const PdVdpArgs&, int variant, int grid, int block, cudaStream_t);
    cudaError_t (*gbm)(const PdGbmArgs&, int grid, int block, cudaStream_t);
    cudaError_t (*gray_scott)(const PdGsArgs&, int variant, cudaStream_t);
    // kernel entry used for cudaFuncGetAttributes / occupancy in pd_explain
    const void* (*kernel_ptr)(int family, int variant);
};

const PdModeTable* pd_mode_table_safe();
const PdModeTable* pd_mode_table_relaxed();
const PdModeTable* pd_mode_table_fast();

// Mode-independent kernels (rounding-explicit arithmetic only); they live in
// the SAFE object.
cudaError_t pd_launch_lv_df32(const PdDfLvArgs&, int block, cudaStream_t);
cudaError_t pd_launch_kepler_df32(const PdKeplerArgs&, int block, cudaStream_t);
cudaError_t pd_launch_threefry(const PdThreefryArgs&, int block, cudaStream_t);
cudaError_t pd_launch_gbm_finish(const double* partials, int n_blocks, double* sums, cudaStream_t);
const void* pd_common_kernel_ptr(int family);
cudaError_t pd_launch_fma_chain(float* sink, int iters, int grid, int block, cudaStream_t);
cudaError_t pd_launch_int_chain(uint32_t* sink, int iters, int grid, int block, cudaStream_t);

// Gray-Scott geometry, shared by launcher and explain.
static const int PD_GS_TILE_ROWS = 32;
static const int PD_GS_BLOCK = 128;
#define PD_GS_TB_ROWS 16  /* output rows per block of the temporally blocked kernel */
#ifndef PD_GS_RT_ROWS
#define PD_GS_RT_ROWS 16  /* output rows per warp of the register-tile kernel */
#define PD_GS_RT_WARPS 4  /* warps per block */
#define PD_GS_RT_BLOCKS 2 /* blocks per SM the register budget allows */
#endif
#ifndef PD_GS_RT_GROUP
#define PD_GS_RT_GROUP 2  /* tile rows advanced per straight-line block (1 or 2; tile heights are even) */
#endif

// The stencil's constants from the call's parameters (double on the host, rounded once each).
inline void pd_gs_set_constants(PdGsArgs& a, double du, double dv, double f, double k, double dt) {
    a.du = (float)du; a.dv = (float)dv; a.f = (float)f; a.fk = (float)(f + k); a.dt = (float)dt;
}

// A 2-D tensor map over one row-major float32 field of this GPU (rows x cols), box = box_rows x box_cols,
// out-of-range elements read as zero.  Implemented once, in the C-ABI translation unit.
cudaError_t pd_encode_field_map(CUtensorMap* map, const float* base, int rows, int cols, int box_rows, int box_cols);

#endif  // PD_KERNELS_H_
