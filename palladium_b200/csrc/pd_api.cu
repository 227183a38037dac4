// pd_api.cu -- the C ABI of libpalladium_cuda.so (declared in
// include/palladium_cuda.h).  This file is the CUDA counterpart of the
// reference's XLA-FFI handler (native/ffi/palladium_ffi.cpp): it validates a
// call, picks the launch geometry, owns the little device scratch the kernels
// need, and launches them.  It never owns caller data.
#include "../../include/palladium_cuda.h"
#include "pd_kernels.h"
#include "pd_rtc.h"

#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <map>
#include <mutex>
#include <thread>
#include <string>
#include <vector>

namespace {

// ---------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------
int fail(int code, char* err, size_t cap, const char* fmt, ...) {
    if (err && cap) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, cap, fmt, ap);
        va_end(ap);
    }
    return code;
}
#define PD_CUDA_TRY(expr)                                                                   \
    do {                                                                                    \
        cudaError_t e_ = (expr);                                                            \
        if (e_ != cudaSuccess)                                                              \
            return fail(PD_ERR_CUDA, err, err_cap, "%s failed: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

// ---------------------------------------------------------------------------
// tuning knobs: a fixed table of integers.  Reading one on the launch path is a
// relaxed atomic load (no lock, no string look-up); names are resolved only by
// the setters.  A thread may override a knob for its own calls
// (pd_set_thread_tuning), so a caller can pick a kernel variant without
// changing what other threads of the process run.
// ---------------------------------------------------------------------------
#define PD_KNOBS(X)                                                                                              \
    X(lv_items_per_thread, 0)  /* 0 = choose from N and alignment */                                            \
    X(lv_block, 0)             /* 0 = choose from N */                                                          \
    X(lv_packed, -1)           /* packed f32x2 arithmetic on pairs of trajectories: 1 on, 0 off, -1 by mode */    \
    X(vdp_variant, 2)          /* 0 direct, 1 lane refill, 2 refill + tail compaction, 3 two passes */           \
    X(vdp_block, 128)                                                                                            \
    X(vdp_refill_every, 16)    /* attempts between refill checks (16 measured 3 % faster than 8, 24 no better) */                                             \
    X(vdp_pass_limit, 1000)    /* variant 3: attempts after which pass one suspends a trajectory */             \
    X(vdp_pass_limit2, 0)      /* variant 3: cap of a second suspending pass (0 = none) */                      \
    X(vdp_pass_limit3, 0)      /* variant 3: cap of a third suspending pass (0 = none) */                       \
    X(vdp_compact_every, 16)   /* variant 2: refill rounds between block-level compactions */                   \
    X(vdp_blocks_per_sm, 0)    /* 0 = about 1024 resident threads per SM */                                     \
    X(gbm_block, 256)                                                                                            \
    X(gbm_blocks_per_sm, 0)                                                                                      \
    X(gs_variant, -1)          /* -1 = best for the shape; 0 per cell, 1 vec4 (one step), 2 temporal blocking */ \
    X(gs_fuse, 0)              /* steps fused per launch by variant 2; 0 = the kernel's default */              \
    X(gs_persistent, -1)       /* variant 2: 0 one tile per block, 1 persistent blocks + cp.async, 2 register tiles + TMA, -1 by size */ \
    X(gs_wait_limit, 1 << 22)  /* register-tile kernel: polls of a tile copy's barrier before the warp gives up */ \
    X(df32_block, 128)                                                                                           \
    X(host_streams, 6)         /* streams the chunks of a host-buffer call rotate over (1..8) */                \
    X(host_copy_threads, 4)    /* helper threads that copy ordinary (pageable) host arrays into page-locked staging (0 = none) */ \
    X(host_chunks, -1)         /* chunks of a large host-buffer call (-1 = by size, 0 = ramped sizes) */        \
    X(time_kernels, 0)

enum Knob {
#define X(name, def) K_##name,
    PD_KNOBS(X)
#undef X
    K_COUNT
};
const char* const kKnobNames[K_COUNT] = {
#define X(name, def) #name,
    PD_KNOBS(X)
#undef X
};
std::atomic<int64_t> g_knobs[K_COUNT] = {
#define X(name, def) {def},
    PD_KNOBS(X)
#undef X
};
struct ThreadKnobs { bool set[K_COUNT] = {}; int64_t value[K_COUNT] = {}; };
thread_local ThreadKnobs t_knobs;

int knob_index(const char* key) {
    for (int i = 0; i < K_COUNT; ++i)
        if (strcmp(kKnobNames[i], key) == 0) return i;
    return -1;
}
inline int64_t knob(Knob k) {
    return t_knobs.set[k] ? t_knobs.value[k] : g_knobs[k].load(std::memory_order_relaxed);
}

// ---------------------------------------------------------------------------
// device facts
// ---------------------------------------------------------------------------
struct DeviceFacts { int device = -1; int sms = 148; bool present = false; };
DeviceFacts device_facts() {
    DeviceFacts f;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        cudaGetLastError();
        return f;
    }
    if (cudaGetDevice(&f.device) != cudaSuccess) { cudaGetLastError(); return f; }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, f.device) == cudaSuccess && sms > 0)
        f.sms = sms;
    f.present = true;
    return f;
}

const PdModeTable* mode_table(int math_mode) {
    switch (math_mode) {
        case PD_MATH_SAFE: return pd_mode_table_safe();
        case PD_MATH_RELAXED: return pd_mode_table_relaxed();
        case PD_MATH_FAST: return pd_mode_table_fast();
        default: return nullptr;
    }
}

// ---------------------------------------------------------------------------
// scratch pool: one grow-only device buffer per (device, stream).  Work on one
// stream is ordered, so consecutive calls can share the buffer.
// ---------------------------------------------------------------------------
struct ScratchSlot { void* ptr = nullptr; size_t bytes = 0; };
std::mutex g_scratch_mutex;
std::map<std::pair<int, void*>, ScratchSlot>& scratch_pool() {
    static std::map<std::pair<int, void*>, ScratchSlot> pool;
    return pool;
}
cudaError_t scratch_get(int device, void* stream, size_t bytes, void** out) {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    ScratchSlot& slot = scratch_pool()[std::make_pair(device, stream)];
    if (slot.bytes < bytes) {
        if (slot.ptr) {
            cudaError_t e = cudaFree(slot.ptr);  // synchronises: no kernel still reads it
            if (e != cudaSuccess) return e;
            slot.ptr = nullptr;
            slot.bytes = 0;
        }
        size_t want = bytes < 4096 ? 4096 : bytes;
        cudaError_t e = cudaMalloc(&slot.ptr, want);
        if (e != cudaSuccess) return e;
        slot.bytes = want;
    }
    *out = slot.ptr;
    return cudaSuccess;
}

// ---------------------------------------------------------------------------
// Device status word.  Kernels whose waits are bounded (the register-tile
// stencil waits for its tile copies) record a non-zero code here when a wait
// runs out.  One word per device in pinned, device-mapped host memory: the
// kernel writes it over the bus, the host reads it without a copy once the
// stream has been synchronised.
// ---------------------------------------------------------------------------
const int kMaxStatusDevices = 64;
std::mutex g_status_mutex;
int* g_status_host[kMaxStatusDevices] = {};
int* g_status_dev[kMaxStatusDevices] = {};
cudaError_t status_word(int device, int** host, int** dev) {
    if (device < 0 || device >= kMaxStatusDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!g_status_host[device]) {
        int* h = nullptr;
        cudaError_t e = cudaHostAlloc((void**)&h, 64, cudaHostAllocMapped | cudaHostAllocPortable);
        if (e != cudaSuccess) return e;
        memset(h, 0, 64);
        int* d = nullptr;
        e = cudaHostGetDevicePointer((void**)&d, h, 0);
        if (e != cudaSuccess) { cudaFreeHost(h); return e; }
        g_status_host[device] = h;
        g_status_dev[device] = d;
    }
    if (host) *host = g_status_host[device];
    if (dev) *dev = g_status_dev[device];
    return cudaSuccess;
}

// After a synchronise: a non-zero status word becomes PD_ERR_DEVICE_STATUS and is cleared.
// A device that never ran a kernel with bounded waits has no word and nothing to report.
int check_device_status(int device, char* err, size_t err_cap) {
    if (device < 0 || device >= kMaxStatusDevices) return PD_OK;
    volatile int* word;
    {
        std::lock_guard<std::mutex> lock(g_status_mutex);
        word = g_status_host[device];
    }
    if (!word || *word == 0) return PD_OK;
    const int code = *word;
    *word = 0;
    return fail(PD_ERR_DEVICE_STATUS, err, err_cap,
                "device status %d: %s", code,
                code == 1 ? "a tile copy of the stencil kernel did not arrive within its wait limit; the outputs of the call are not valid"
                          : "a kernel reported a failed bounded wait");
}

thread_local double t_last_kernel_ms = -1.0;

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---------------------------------------------------------------------------
// launch plans: everything pd_explain reports and pd_launch needs
// ---------------------------------------------------------------------------
struct Plan {
    const char* kernel_name = "";
    int64_t grid[3] = {1, 1, 1};
    int64_t block[3] = {1, 1, 1};
    int64_t items = 1;
    int64_t launches = 1;
    int64_t scratch_bytes = 0;
    int variant = 0;
    int64_t dynamic_smem = 0;      // bytes of dynamic shared memory per block (the tiled stencil kernels)
    const void* kernel = nullptr;
    PdRtcKernel rtc;               // run-time compiled families only
};

int requested_block(const int64_t block[3]) {
    if (!block) return 0;
    int64_t b = block[0] * (block[1] > 0 ? block[1] : 1) * (block[2] > 0 ? block[2] : 1);
    return b > 0 ? (int)b : 0;
}

int check_block(int b, char* err, size_t err_cap) {
    if (b < 32 || b > 256 || (b % 32) != 0)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                    "threadgroup of %d threads is not supported: use a multiple of 32 in [32, 256]", b);
    return PD_OK;
}

int occupancy_blocks(const void* kernel, int block, size_t dynamic_smem = 0) {
    int n = 0;
    if (dynamic_smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dynamic_smem) != cudaSuccess)
        cudaGetLastError();
    if (!kernel || cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, block, dynamic_smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

template <class P>
int get_params(const void* params, size_t bytes, const P** out, const char* what, char* err, size_t err_cap) {
    if (!params || bytes != sizeof(P))
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "%s: params block must be %zu bytes, got %zu", what,
                    sizeof(P), params ? bytes : (size_t)0);
    *out = static_cast<const P*>(params);
    return PD_OK;
}

// Trajectories per thread of the fixed-step kernel.  Measured at 2^22 / 100 000 trajectories (ms per
// 1000-step pass; "p" = packed f32x2 arithmetic):
//   SAFE     1: 6.75 / 0.192   2: 6.68 / 0.188   4: 6.73 / 0.258   2p: 6.92 / 0.200   4p: 7.20 / 0.276
//   RELAXED  1: 5.26 / 0.155   2: 5.01 / 0.143   4: 5.31 / 0.200   2p: 4.68 / 0.133   4p: 4.92 / 0.184
//   FAST     1: 3.71 / 0.110   2: 3.56 / 0.102   4: 3.70 / 0.139   2p: 3.60 / 0.106   4p: 3.54 / 0.137
// Below about 512 trajectories per SM a launch is a single partial wave, and more threads win.
int lv_items_for(int64_t n, int sms, bool vec_ok, int math_mode) {
    int64_t forced = knob(K_lv_items_per_thread);
    if (forced == 1 || forced == 2 || forced == 4) return vec_ok ? (int)forced : 1;
    if (!vec_ok) return 1;
    if (math_mode == PD_MATH_FAST && n >= (int64_t)4 * sms * 2048) return 4;
    if (n >= (int64_t)sms * 512) return 2;
    return 1;
}

// Whether the kernel with `items` trajectories per thread computes on packed pairs.
int lv_packed_for(int items, int math_mode) {
    const int64_t forced = knob(K_lv_packed);
    if (items < 2) return 0;
    if (forced == 0 || forced == 1) return (int)forced;
    if (math_mode == PD_MATH_RELAXED) return 1;
    if (math_mode == PD_MATH_FAST) return items == 4 ? 1 : 0;
    return 0;  // SAFE: the exactly rounded packed form is slower than scalar code (table above)
}

int build_plan(int family, const void* params, size_t params_bytes, int math_mode, const int64_t grid[3],
               const int64_t block[3], bool vec_ok, const DeviceFacts& dev, Plan* plan, char* err,
               size_t err_cap) {
    if (math_mode < PD_MATH_SAFE || math_mode > PD_MATH_FAST)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "palladium_dispatch: math_mode out of range");
    if (!grid) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "grid must not be NULL");
    for (int i = 0; i < 3; ++i)
        if (grid[i] < 0) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "grid[%d] is negative", i);
    const PdModeTable* mt = mode_table(math_mode);
    const int req_block = requested_block(block);
    if (req_block && family != PD_FAMILY_SOURCE) {
        int rc = check_block(req_block, err, err_cap);
        if (rc) return rc;
    }
    const int64_t n = grid[0];
    switch (family) {
        case PD_FAMILY_LV_RK4: {
            const pd_lv_rk4_params* p;
            int rc = get_params(params, params_bytes, &p, "lv_rk4", err, err_cap);
            if (rc) return rc;
            if (p->steps < 0 || p->steps > INT32_MAX)
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "lv_rk4: steps out of range");
            const int items = lv_items_for(n, dev.sms, vec_ok, math_mode);
            int b = req_block ? req_block : (int)knob(K_lv_block);
            if (!b) b = (n / items >= (int64_t)dev.sms * 2048) ? 128 : 64;
            plan->kernel_name = items == 4 ? "pd_lv_rk4_kernel<4>" : items == 2 ? "pd_lv_rk4_kernel<2>" : "pd_lv_rk4_kernel<1>";
            plan->items = items;
            plan->block[0] = b;
            plan->grid[0] = ((n + items - 1) / items + b - 1) / b;
            plan->variant = items;
            plan->kernel = mt->kernel_ptr(family, items);
            return PD_OK;
        }
        case PD_FAMILY_VDP_BS32: {
            const pd_vdp_bs32_params* p;
            int rc = get_params(params, params_bytes, &p, "vdp_bs32", err, err_cap);
            if (rc) return rc;
            if (p->max_steps < 0 || p->max_steps > (1 << 24))
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                            "vdp_bs32: max_steps must lie in [0, 2^24] (the reference counts in float32)");
            if (p->out_layout < 0 || p->out_layout > 2)
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "vdp_bs32: out_layout must be 0, 1 or 2");
            if (p->error_order <= 0)
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "vdp_bs32: error_order must be positive");
            const int variant = (int)knob(K_vdp_variant);
            int b = req_block ? req_block : (int)knob(K_vdp_block);
            int variant_used = variant;
            // two passes make sense only when a trajectory can outlast the first one
            if (variant == 3 && p->max_steps <= knob(K_vdp_pass_limit)) variant_used = 2;
            if (variant_used >= 2) b = 256;   // the compaction kernel's shared arrays are sized for 256 threads
            plan->variant = variant_used;
            plan->kernel = mt->kernel_ptr(family, variant);
            plan->block[0] = b;
            if (variant == 0) {
                plan->kernel_name = "pd_vdp_direct_kernel";
                plan->grid[0] = (n + b - 1) / b;
            } else {
                plan->kernel_name = plan->variant >= 2 ? "pd_vdp_compact_kernel" : "pd_vdp_refill_kernel";
                // About 1024 resident threads per SM measured best: enough warps to
                // hide the divide / pow latencies, and few enough threads that each one
                // integrates many trajectories, which evens out the heavy-tailed work.
                int per_sm = (int)knob(K_vdp_blocks_per_sm);
                if (!per_sm) {
                    per_sm = 1024 / b > 0 ? 1024 / b : 1;
                    const int occ = dev.present ? occupancy_blocks(plan->kernel, b) : 0;
                    if (occ > 0 && per_sm > occ) per_sm = occ;
                }
                int64_t g = (int64_t)dev.sms * per_sm;
                const int64_t needed = (n + b - 1) / b;
                if (g > needed) g = needed;
                plan->grid[0] = g > 0 ? g : 1;
                plan->scratch_bytes = 256;
                if (plan->variant == 3) {
                    // header (queue heads, count, bucket counters) + bucket and order per trajectory
                    // + ten words of suspended state per trajectory
                    const int64_t per = ((n + 63) / 64) * 64;
                    plan->scratch_bytes = 1024 + 4 * per * 12;
                    plan->launches = 4;
                }
            }
            return PD_OK;
        }
        case PD_FAMILY_CUSTOM_ODE: {
            const pd_custom_ode_params* p;
            int rc = get_params(params, params_bytes, &p, "custom_ode", err, err_cap);
            if (rc) return rc;
            rc = pd_rtc_check_params(p, err, err_cap);
            if (rc) return rc;
            const int b = req_block ? req_block : 128;
            plan->kernel_name = pd_rtc_kernel_name(p);
            plan->block[0] = b;
            plan->grid[0] = (n + b - 1) / b;
            if (p->method != PD_ODE_RK4) {
                // persistent warps, about 1024 threads per SM (as for the Van der Pol kernel)
                int per_sm = 1024 / b > 0 ? 1024 / b : 1;
                int64_t g = (int64_t)dev.sms * per_sm;
                if (g > plan->grid[0]) g = plan->grid[0];
                plan->grid[0] = g > 0 ? g : 1;
                plan->scratch_bytes = 256;
            }
            if (dev.present) {
                // compiled on the first use of this source text, cached afterwards
                rc = pd_rtc_get(p, math_mode, dev.device, b, &plan->rtc, err, err_cap);
                if (rc) return rc;
            }
            return PD_OK;
        }
        case PD_FAMILY_SOURCE: {
            const pd_source_kernel_params* p;
            int rc = get_params(params, params_bytes, &p, "source kernel", err, err_cap);
            if (rc) return rc;
            rc = pd_rtc_check_source(p, err, err_cap);
            if (rc) return rc;
            // One thread per point of the logical grid, as Metal's dispatchThreads launches
            // them; whole blocks here, the kernel trims the edge itself.
            int64_t b[3];
            if (req_block) {
                for (int i = 0; i < 3; ++i) b[i] = block[i] > 0 ? block[i] : 1;
                if (b[0] * b[1] * b[2] > 1024 || b[2] > 64)
                    return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                                "threadgroup (%lld, %lld, %lld) exceeds 1024 threads (or 64 in z)", (long long)b[0],
                                (long long)b[1], (long long)b[2]);
            } else if (grid[1] <= 1 && grid[2] <= 1) {
                b[0] = 128; b[1] = 1; b[2] = 1;
            } else if (grid[2] <= 1) {
                b[0] = 32; b[1] = 4; b[2] = 1;
            } else {
                b[0] = 32; b[1] = 2; b[2] = 2;
            }
            for (int i = 0; i < 3; ++i) {
                const int64_t g = grid[i] > 0 ? grid[i] : (i == 0 ? 0 : 1);
                plan->block[i] = b[i];
                plan->grid[i] = (g + b[i] - 1) / b[i];
            }
            if (plan->grid[1] > 65535 || plan->grid[2] > 65535)
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                            "grid needs more than 65535 blocks in y or z; put the long axis first");
            plan->kernel_name = p->function_name;
            if (dev.present) {
                rc = pd_rtc_get_source(p, math_mode, dev.device, (int)(b[0] * b[1] * b[2]), &plan->rtc, err, err_cap);
                if (rc) return rc;
            }
            return PD_OK;
        }
        case PD_FAMILY_GBM_PCG:
        case PD_FAMILY_GBM_THREEFRY: {
            const pd_gbm_params* p;
            int rc = get_params(params, params_bytes, &p, "gbm", err, err_cap);
            if (rc) return rc;
            if (p->steps < 0 || p->steps > (1 << 30))
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gbm: steps out of range");
            if (p->path_offset < 0 || p->path_offset + n > ((int64_t)1 << 32))
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                            "gbm_threefry: path indices must fit in 32 bits (fold_in takes a uint32)");
            int b = req_block ? req_block : (int)knob(K_gbm_block);
            plan->kernel_name = family == PD_FAMILY_GBM_PCG ? "pd_gbm_kernel<pcg>" : "pd_gbm_kernel<threefry>";
            plan->kernel = mt->kernel_ptr(family, 0);
            int per_sm = (int)knob(K_gbm_blocks_per_sm);
            if (!per_sm) per_sm = dev.present ? occupancy_blocks(plan->kernel, b) : 0;
            if (per_sm <= 0) per_sm = 2048 / b / 2;
            int64_t g = (int64_t)dev.sms * per_sm;
            const int64_t needed = (n + b - 1) / b;
            if (g > needed) g = needed;
            plan->grid[0] = g > 0 ? g : 1;
            plan->block[0] = b;
            plan->launches = 2;
            plan->scratch_bytes = (int64_t)plan->grid[0] * 2 * sizeof(double);
            return PD_OK;
        }
        case PD_FAMILY_GRAY_SCOTT: {
            const pd_gray_scott_params* p;
            int rc = get_params(params, params_bytes, &p, "gray_scott", err, err_cap);
            if (rc) return rc;
            if (p->rows <= 0 || p->cols <= 0 || p->rows > (1 << 20) || p->cols > (1 << 20))
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gray_scott: rows/cols out of range");
            if (grid[0] != p->rows || grid[1] != p->cols)
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                            "gray_scott: grid (%lld, %lld) does not match rows x cols (%lld, %lld)",
                            (long long)grid[0], (long long)grid[1], (long long)p->rows, (long long)p->cols);
            if (p->steps < 0) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gray_scott: steps is negative");
            if (p->halo < 0) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gray_scott: halo is negative");
            if (p->halo > 0 && p->steps > p->halo)
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                            "gray_scott: a slab with %lld halo rows can advance at most %lld steps per call",
                            (long long)p->halo, (long long)p->halo);
            const int64_t rows_alloc = p->rows + 2 * p->halo;
            if (rows_alloc * p->cols >= ((int64_t)1 << 31))
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gray_scott: more than 2^31 cells per call");
            int variant = (int)knob(K_gs_variant);
            const bool vec_shape = (p->cols % 4 == 0) && p->cols >= 128 && vec_ok;
            // the one-thread-per-cell kernel spreads rows over the second launch dimension, 8 per block
            if ((!vec_shape || variant == 0) && (rows_alloc + 7) / 8 > 65535)
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                            "gray_scott: %lld rows of %lld columns cannot be launched (grids narrower than 128 "
                            "columns, with a column count that is not a multiple of 4, or in unaligned buffers take at "
                            "most 524280 rows)", (long long)rows_alloc, (long long)p->cols);
            if (variant < 0) variant = vec_shape ? (p->steps >= 2 ? 2 : 1) : 0;
            if (variant >= 1 && !vec_shape) variant = 0;
            int fuse = (int)knob(K_gs_fuse);
            if (fuse == 0) fuse = 4;
            fuse = fuse < 2 ? 2 : (fuse > 4 ? 4 : fuse);
            plan->variant = variant;
            int64_t launches = p->steps;
            if (variant == 0) {
                plan->kernel = mt->kernel_ptr(family, 0);
                plan->kernel_name = "pd_gs_cell_kernel";
                plan->block[0] = 32; plan->block[1] = 8;
                plan->grid[0] = (p->cols + 31) / 32;
                plan->grid[1] = (rows_alloc + 7) / 8;
            } else if (variant == 1 || p->steps < 2) {
                plan->variant = vec_shape ? 1 : 0;
                plan->kernel = mt->kernel_ptr(family, 1);
                plan->kernel_name = "pd_gs_vec4_kernel";
                plan->items = 4 * PD_GS_TILE_ROWS;
                plan->block[0] = PD_GS_BLOCK;
                plan->grid[0] = (p->cols / 4 + PD_GS_BLOCK - 1) / PD_GS_BLOCK;
                plan->grid[1] = (rows_alloc + PD_GS_TILE_ROWS - 1) / PD_GS_TILE_ROWS;
            } else {
                const int k = p->steps < fuse ? (int)p->steps : fuse;
                // 0: one tile per block in shared memory; 1: persistent blocks with cp.async prefetch;
                // 2: one tile per warp in registers, tiles fetched by the copy engine (TMA).
                // -1: the register-tile kernel once there are tiles for every resident warp, since
                // a warp works through its tile alone (small grids finish sooner spread over blocks).
                int form = (int)knob(K_gs_persistent);
                const int64_t tiles = ((p->cols + 119) / 120) * ((rows_alloc + PD_GS_RT_ROWS - 1) / PD_GS_RT_ROWS);
                if (form < 0) form = tiles >= (int64_t)dev.sms * 8 ? 2 : 0;
                if (form > 2) form = 2;
                plan->variant = (form == 2 ? 30 : form == 1 ? 20 : 10) + k;  // the kernel of the full-size launches
                plan->kernel = mt->kernel_ptr(family, plan->variant);
                static const char* const names[3][3] = {
                    {"pd_gs_tb_kernel<2>", "pd_gs_tb_kernel<3>", "pd_gs_tb_kernel<4>"},
                    {"pd_gs_tbp_kernel<2>", "pd_gs_tbp_kernel<3>", "pd_gs_tbp_kernel<4>"},
                    {"pd_gs_rt_kernel<2>", "pd_gs_rt_kernel<3>", "pd_gs_rt_kernel<4>"}};
                plan->kernel_name = names[form][k - 2];
                plan->items = 4;  // cells per thread per row
                {
                    // shared memory per block: the block-tile kernels keep two (three when persistent) copies of
                    // a (16 + 2k) x 128 tile of both fields; the register-tile kernel one landing zone per warp
                    const int64_t tile = 2 * (int64_t)(form == 2 ? PD_GS_RT_ROWS + 2 * k : PD_GS_TB_ROWS + 2 * k) * 512;
                    plan->dynamic_smem = form == 2 ? PD_GS_RT_WARPS * tile + 8 * PD_GS_RT_WARPS : (form == 1 ? 3 : 2) * tile;
                }
                if (form == 2) {
                    plan->block[0] = PD_GS_RT_WARPS * 32;
                    int64_t g = (int64_t)dev.sms * PD_GS_RT_BLOCKS;
                    if (g > (tiles + PD_GS_RT_WARPS - 1) / PD_GS_RT_WARPS) g = (tiles + PD_GS_RT_WARPS - 1) / PD_GS_RT_WARPS;
                    plan->grid[0] = g > 0 ? g : 1;
                } else {
                    plan->block[0] = 256;
                    plan->grid[0] = (p->cols + 119) / 120;
                    plan->grid[1] = (rows_alloc + PD_GS_TB_ROWS - 1) / PD_GS_TB_ROWS;
                }
                launches = (p->steps + k - 1) / k;
            }
            plan->launches = launches;
            // Intermediate fields.  A periodic grid ping-pongs between one scratch pair and the
            // caller's output.  A slab never writes an intermediate state into its output: with
            // the in-kernel exchange a neighbour may already have stored the next call's ghost
            // rows there, so three or more launches alternate between two scratch pairs.
            const int64_t pairs = launches < 2 ? 0 : (p->halo > 0 && launches >= 3 ? 2 : 1);
            plan->scratch_bytes = pairs * 2 * rows_alloc * p->cols * (int64_t)sizeof(float);
            return PD_OK;
        }
        case PD_FAMILY_LV_RK4_DF32:
        case PD_FAMILY_KEPLER_RK4_DF32: {
            int64_t steps;
            if (family == PD_FAMILY_LV_RK4_DF32) {
                const pd_lv_rk4_df32_params* p;
                int rc = get_params(params, params_bytes, &p, "lv_rk4_df32", err, err_cap);
                if (rc) return rc;
                steps = p->steps;
                plan->kernel_name = "pd_lv_df32_kernel";
            } else {
                const pd_kepler_rk4_df32_params* p;
                int rc = get_params(params, params_bytes, &p, "kepler_rk4_df32", err, err_cap);
                if (rc) return rc;
                steps = p->steps;
                plan->kernel_name = "pd_kepler_df32_kernel";
            }
            if (steps < 0 || steps > INT32_MAX)
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "df32: steps out of range");
            int b = req_block ? req_block : (int)knob(K_df32_block);
            plan->block[0] = b;
            plan->grid[0] = (n + b - 1) / b;
            plan->kernel = pd_common_kernel_ptr(family);
            return PD_OK;
        }
        case PD_FAMILY_THREEFRY_BITS: {
            const pd_threefry_params* p;
            int rc = get_params(params, params_bytes, &p, "threefry_bits", err, err_cap);
            if (rc) return rc;
            if (p->op < 0 || p->op > 4)
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "threefry_bits: op must be 0..4");
            if (p->op == 3 && p->count <= 0)
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "threefry_bits: count must be positive");
            const int64_t total = p->op == 3 ? n * p->count : n;
            if (total >= ((int64_t)1 << 32))
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "threefry_bits: more than 2^32 draws");
            int b = req_block ? req_block : 256;
            plan->kernel_name = "pd_threefry_kernel";
            plan->block[0] = b;
            plan->grid[0] = (total + b - 1) / b;
            plan->kernel = pd_common_kernel_ptr(family);
            return PD_OK;
        }
        default:
            return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "unknown kernel family %d", family);
    }
}

int check_buffers(const char* what, int n_have, int n_want, const size_t* bytes, const size_t* want_bytes,
                  const void* const* ptrs, char* err, size_t err_cap) {
    if (n_have != n_want)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "kernel takes %d %s arrays, got %d", n_want, what, n_have);
    for (int i = 0; i < n_want; ++i) {
        if (bytes[i] != want_bytes[i])
            return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "%s %d: expected %zu bytes, got %zu", what, i,
                        want_bytes[i], bytes[i]);
        if (want_bytes[i] && !ptrs[i])
            return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "%s %d: NULL pointer", what, i);
        if (!aligned(ptrs[i], 4))
            return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "%s %d: pointer is not 4-byte aligned", what, i);
    }
    return PD_OK;
}

bool all_aligned16(int n_in, const void* const* in, int n_out, void* const* out) {
    for (int i = 0; i < n_in; ++i) if (!aligned(in[i], 16)) return false;
    for (int i = 0; i < n_out; ++i) if (!aligned(out[i], 16)) return false;
    return true;
}

// Expected buffer sizes for a family call.
int expected_sizes(int family, const void* params, const int64_t grid[3], std::vector<size_t>* in,
                   std::vector<size_t>* out, int n_in_given, int n_out_given, char* err, size_t err_cap) {
    const size_t n = (size_t)grid[0];
    switch (family) {
        case PD_FAMILY_LV_RK4:
            in->assign(6, 4 * n);
            if (n_out_given == 1) out->assign(1, 8 * n);   // one (N, 2) array of (x, y) pairs
            else out->assign(2, 4 * n);
            return PD_OK;
        case PD_FAMILY_LV_RK4_DF32:
            in->assign(6, 4 * n); out->assign(2, 4 * n); return PD_OK;
        case PD_FAMILY_VDP_BS32: {
            const pd_vdp_bs32_params* p = static_cast<const pd_vdp_bs32_params*>(params);
            in->assign(n_in_given == 4 ? 4 : 3, 4 * n);   // optional 4th input: the hand-out order, (N) int32
            if (p->out_layout == 0) out->assign(6, 4 * n);
            else if (p->out_layout == 1) out->assign(5, 4 * n);
            else { out->assign(3, 4 * n); (*out)[0] = 8 * n; }
            return PD_OK;
        }
        case PD_FAMILY_GBM_PCG:
        case PD_FAMILY_GBM_THREEFRY:
            if (family == PD_FAMILY_GBM_THREEFRY) in->assign(1, 8); else in->clear();
            out->assign(1, 4 * n);
            if (n_out_given == 2) out->push_back(16);
            return PD_OK;
        case PD_FAMILY_GRAY_SCOTT: {
            const pd_gray_scott_params* p = static_cast<const pd_gray_scott_params*>(params);
            const size_t cells = (size_t)(p->rows + 2 * p->halo) * (size_t)p->cols;
            in->assign(2, 4 * cells); out->assign(2, 4 * cells); return PD_OK;
        }
        case PD_FAMILY_KEPLER_RK4_DF32:
            in->assign(8, 4 * n); out->assign(8, 4 * n); return PD_OK;
        case PD_FAMILY_CUSTOM_ODE: {
            const pd_custom_ode_params* p = static_cast<const pd_custom_ode_params*>(params);
            in->assign((size_t)(p->dim + p->nparam), 4 * n);
            out->assign((size_t)(p->method == PD_ODE_RK4 ? p->dim : p->dim + 4), 4 * n);
            return PD_OK;
        }
        case PD_FAMILY_THREEFRY_BITS: {
            const pd_threefry_params* p = static_cast<const pd_threefry_params*>(params);
            in->assign(1, 8);
            if (p->op == 2) { in->push_back(4 * n); out->assign(1, 8 * n); }
            else if (p->op == 3) out->assign(1, 4 * n * (size_t)p->count);
            else out->assign(1, 4 * n);
            return PD_OK;
        }
        default:
            return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "unknown kernel family %d", family);
    }
}

void split_df32(double v, float* hi, float* lo) {
    *hi = (float)v;
    *lo = (float)(v - (double)*hi);
}

int launch_impl(int family, const void* params, size_t params_bytes, int math_mode, const int64_t grid[3],
                const int64_t block[3], int n_in, const void* const* in, const size_t* in_bytes, int n_out,
                void* const* out, const size_t* out_bytes, void* workspace, size_t workspace_bytes,
                cudaStream_t st, char* err, size_t err_cap, const pd_gs_neighbours* neighbours = nullptr) {
    DeviceFacts dev = device_facts();
    if (!dev.present)
        return fail(PD_ERR_CUDA, err, err_cap,
                    "no CUDA device is available: libpalladium_cuda has no CPU fallback");
    if ((n_in > 0 && (!in || !in_bytes)) || (n_out > 0 && (!out || !out_bytes)))
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "buffer arrays must not be NULL");
    const bool vec_ok = all_aligned16(n_in, in, n_out, out);
    Plan plan;
    int rc = build_plan(family, params, params_bytes, math_mode, grid, block, vec_ok, dev, &plan, err, err_cap);
    if (rc) return rc;
    if (family != PD_FAMILY_SOURCE) {   // a caller-written kernel defines its own buffer sizes
        std::vector<size_t> want_in, want_out;
        rc = expected_sizes(family, params, grid, &want_in, &want_out, n_in, n_out, err, err_cap);
        if (rc) return rc;
        rc = check_buffers("input", n_in, (int)want_in.size(), in_bytes, want_in.data(), in, err, err_cap);
        if (rc) return rc;
        rc = check_buffers("output", n_out, (int)want_out.size(), out_bytes, want_out.data(),
                           const_cast<const void* const*>(out), err, err_cap);
        if (rc) return rc;
    } else {
        if (n_in + n_out > 64)
            return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "source kernel: at most 64 buffers, got %d", n_in + n_out);
        for (int i = 0; i < n_in; ++i)
            if (in_bytes[i] && !in[i]) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "input %d: NULL pointer", i);
        for (int i = 0; i < n_out; ++i)
            if (out_bytes[i] && !out[i]) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "output %d: NULL pointer", i);
    }

    void* scratch = nullptr;
    if (plan.scratch_bytes > 0) {
        if (workspace) {
            if (workspace_bytes < (size_t)plan.scratch_bytes)
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "workspace of %zu bytes is smaller than the %lld needed",
                            workspace_bytes, (long long)plan.scratch_bytes);
            if (!aligned(workspace, 256))
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "workspace must be 256-byte aligned");
            scratch = workspace;
        } else {
            PD_CUDA_TRY(scratch_get(dev.device, (void*)st, (size_t)plan.scratch_bytes, &scratch));
        }
    }

    // Kernel timing synchronises on an event, which a stream that is being captured into a graph cannot do.
    bool timed = knob(K_time_kernels) != 0;
    if (timed) {
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &capturing) != cudaSuccess) cudaGetLastError();
        if (capturing != cudaStreamCaptureStatusNone) timed = false;
    }
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    t_last_kernel_ms = -1.0;
    if (timed) {
        PD_CUDA_TRY(cudaEventCreate(&ev0));
        PD_CUDA_TRY(cudaEventCreate(&ev1));
        PD_CUDA_TRY(cudaEventRecord(ev0, st));
    }

    const PdModeTable* mt = mode_table(math_mode);
    const int64_t n = grid[0];
    const int b = (int)plan.block[0];
    switch (family) {
        case PD_FAMILY_LV_RK4: {
            const pd_lv_rk4_params* p = static_cast<const pd_lv_rk4_params*>(params);
            PdLvArgs a;
            a.x0 = (const float*)in[0]; a.y0 = (const float*)in[1]; a.a = (const float*)in[2];
            a.b = (const float*)in[3]; a.c = (const float*)in[4]; a.d = (const float*)in[5];
            a.state2_out = nullptr;
            if (n_out == 1) {
                if (!aligned(out[0], 8))
                    return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "output 0: (N,2) state must be 8-byte aligned");
                a.state2_out = (float*)out[0]; a.xo = nullptr; a.yo = nullptr;
            } else {
                a.xo = (float*)out[0]; a.yo = (float*)out[1];
            }
            a.n = n; a.steps = (int)p->steps;
            a.h_half = (float)(0.5 * p->dt); a.h_full = (float)p->dt;
            a.h_sixth = (float)(p->dt / 6.0);
            a.packed = lv_packed_for((int)plan.items, math_mode);
            a.neg_zero = -0.0f;
            PD_CUDA_TRY(mt->lv_rk4(a, (int)plan.items, b, st));
            break;
        }
        case PD_FAMILY_VDP_BS32: {
            const pd_vdp_bs32_params* p = static_cast<const pd_vdp_bs32_params*>(params);
            PdVdpArgs a;
            memset(&a, 0, sizeof(a));
            a.x0 = (const float*)in[0]; a.v0 = (const float*)in[1]; a.mu = (const float*)in[2];
            a.order = (n_in == 4 && plan.variant >= 1) ? (const int32_t*)in[3] : nullptr;
            if (p->out_layout == 2) {
                if (!aligned(out[0], 8))
                    return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "output 0: (N,2) state must be 8-byte aligned");
                a.state2_out = (float*)out[0];
                a.accepted_i32 = (int32_t*)out[1];
                a.rejected_i32 = (int32_t*)out[2];
            } else {
                a.t_out = (float*)out[0]; a.x_out = (float*)out[1]; a.v_out = (float*)out[2];
                a.steps_out = (float*)out[3]; a.rejected_out = (float*)out[4];
                if (p->out_layout == 0) a.real_out = (float*)out[5];
            }
            a.n = n; a.max_steps = (int)p->max_steps;
            a.refill_every = (int)knob(K_vdp_refill_every);
            if (a.refill_every < 1) a.refill_every = 1;
            a.t1 = (float)p->t1; a.rtol = (float)p->rtol; a.atol = (float)p->atol; a.dt0 = (float)p->dt0;
            a.safety = (float)p->safety; a.factor_min = (float)p->factor_min; a.factor_max = (float)p->factor_max;
            a.coeff1 = (float)((p->icoeff + p->pcoeff) / (double)p->error_order);
            a.coeff2 = (float)(-p->pcoeff / (double)p->error_order);
            if (plan.variant >= 1) {
                a.cursor = (unsigned long long*)scratch;
                PD_CUDA_TRY(cudaMemsetAsync(scratch, 0, 256, st));
            }
            if (plan.variant == 3) {
                // scratch: [0] queue head of pass one, [8] of pass two, [16] suspended count,
                // [256] 64 bucket counters, [512] 64 write positions, [1024] per-trajectory arrays
                char* base = (char*)scratch;
                const int64_t per = ((n + 63) / 64) * 64;
                a.cursor2 = (unsigned long long*)(base + 8);
                a.n_susp = (unsigned long long*)(base + 16);
                a.hist = (unsigned int*)(base + 256);
                a.offsets = (unsigned int*)(base + 512);
                a.bucket_of = (int32_t*)(base + 1024);
                a.order2 = (int32_t*)(base + 1024 + 4 * per);
                a.susp = (float*)(base + 1024 + 8 * per);
                a.pass_limits[0] = (int)knob(K_vdp_pass_limit);
                a.pass_limits[1] = (int)knob(K_vdp_pass_limit2);
                a.pass_limits[2] = (int)knob(K_vdp_pass_limit3);
                for (int k = 1; k < 3; ++k)   // a cap that does not rise ends the list
                    if (a.pass_limits[k] <= a.pass_limits[k - 1]) { a.pass_limits[k] = 0; if (k == 1) a.pass_limits[2] = 0; }
                PD_CUDA_TRY(cudaMemsetAsync(base, 0, 1024, st));
                PD_CUDA_TRY(cudaMemsetAsync(a.bucket_of, 0xFF, 4 * (size_t)per, st));
            }
            if (plan.variant >= 2) {
                a.compact_every = (int)knob(K_vdp_compact_every);
                if (a.compact_every < 1) a.compact_every = 1;
                // list scheduling: the last lane finishes within (average load + longest job) rounds
                const long long lanes = (long long)plan.grid[0] * b;
                const long long per_job = a.max_steps / a.refill_every + 2;
                a.round_limit = ((n + lanes - 1) / lanes + 2) * per_job + 2LL * a.compact_every;
            }
            PD_CUDA_TRY(mt->vdp_bs32(a, plan.variant, (int)plan.grid[0], b, st));
            break;
        }
        case PD_FAMILY_GBM_PCG:
        case PD_FAMILY_GBM_THREEFRY: {
            const pd_gbm_params* p = static_cast<const pd_gbm_params*>(params);
            PdGbmArgs a;
            a.rng = family == PD_FAMILY_GBM_PCG ? 1 : 0;
            a.key = a.rng == 0 ? (const uint32_t*)in[0] : nullptr;
            a.out = (float*)out[0];
            a.block_partials = (n_out == 2) ? (double*)scratch : nullptr;
            a.n = n; a.path_offset = (uint32_t)p->path_offset; a.steps = (int)p->steps;
            a.output_kind = (int)p->output_kind;
            const double dt = p->t / (double)(p->steps > 0 ? p->steps : 1);
            a.s0 = (float)p->s0; a.strike = (float)p->strike;
            a.drift_dt = (float)((p->r - p->sigma * p->sigma / 2.0) * dt);
            // Threefry kernel: f32(sigma) * sqrt_f32(f32(dt)) (examples/03:100); the hand-written
            // kernel receives np.float32(sigma * np.sqrt(dt)) (examples/03:88).
            a.vol_sqdt = a.rng == 0 ? (float)p->sigma * sqrtf((float)dt) : (float)(p->sigma * sqrt(dt));
            if (n_out == 2 && !aligned(out[1], 8))
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "output 1: float64 sums must be 8-byte aligned");
            PD_CUDA_TRY(mt->gbm(a, (int)plan.grid[0], b, st));
            if (n_out == 2) {
                if (n > 0) PD_CUDA_TRY(pd_launch_gbm_finish((const double*)scratch, (int)plan.grid[0], (double*)out[1], st));
                else PD_CUDA_TRY(cudaMemsetAsync(out[1], 0, 16, st));
            }
            break;
        }
        case PD_FAMILY_GRAY_SCOTT: {
            const pd_gray_scott_params* p = static_cast<const pd_gray_scott_params*>(params);
            const int rows_alloc = (int)(p->rows + 2 * p->halo);
            const size_t field_bytes = (size_t)rows_alloc * (size_t)p->cols * sizeof(float);
            PdGsArgs a = {};
            a.rows_alloc = rows_alloc; a.cols = (int)p->cols;
            a.periodic_rows = p->halo == 0 ? 1 : 0;
            pd_gs_set_constants(a, p->du, p->dv, p->f, p->k, p->dt);
            if (p->steps == 0) {
                PD_CUDA_TRY(cudaMemcpyAsync(out[0], in[0], field_bytes, cudaMemcpyDeviceToDevice, st));
                PD_CUDA_TRY(cudaMemcpyAsync(out[1], in[1], field_bytes, cudaMemcpyDeviceToDevice, st));
                break;
            }
            float* ping_u = (float*)out[0];
            float* ping_v = (float*)out[1];
            float* pong_u = (float*)scratch;
            float* pong_v = scratch ? (float*)((char*)scratch + field_bytes) : nullptr;
            // slabs: a second scratch pair, so that only the final launch touches the output
            const bool slab_pairs = p->halo > 0 && plan.launches >= 3;
            float* pang_u = slab_pairs ? (float*)((char*)scratch + 2 * field_bytes) : nullptr;
            float* pang_v = slab_pairs ? (float*)((char*)scratch + 3 * field_bytes) : nullptr;
            const float* src_u = (const float*)in[0];
            const float* src_v = (const float*)in[1];
            // Fused launches of k steps each (k = 1 for the one-step kernels); the
            // last launch must land in `out`, so an odd launch count starts there.
            const int tb_base = plan.variant >= 32 ? 30 : (plan.variant >= 22 ? 20 : 10);
            const int fuse = plan.variant >= 12 ? plan.variant - tb_base : 1;
            if (tb_base == 30) {
                // bounded waits of the tile copies: about a second of polling before a warp gives up
                // (a copy takes microseconds), then a longer bound for the copy in flight to land
                int* status_dev = nullptr;
                PD_CUDA_TRY(status_word(dev.device, nullptr, &status_dev));
                a.status = status_dev;
                a.wait_limit = knob(K_gs_wait_limit);
                a.drain_limit = (long long)1 << 24;
            }
            bool to_out = (plan.launches % 2) == 1;
            int64_t done = 0;
            while (done < p->steps) {
                const int k = (int)((p->steps - done) < fuse ? (p->steps - done) : fuse);
                a.u = src_u; a.v = src_v;
                const bool last = done + k >= p->steps;
                if (p->halo > 0) {
                    // to_out alternates per launch; here it only picks between the scratch pairs
                    a.uo = last ? ping_u : (slab_pairs && to_out ? pang_u : pong_u);
                    a.vo = last ? ping_v : (slab_pairs && to_out ? pang_v : pong_v);
                } else {
                    a.uo = to_out ? ping_u : pong_u;
                    a.vo = to_out ? ping_v : pong_v;
                }
                if (p->halo == 0) { a.row_lo = 0; a.row_hi = rows_alloc; }
                else { a.row_lo = (int)(done + k); a.row_hi = rows_alloc - (int)(done + k); }
                const int variant = k >= 2 ? tb_base + k : (plan.variant >= 12 ? 1 : plan.variant);
                if (last && neighbours) {
                    // The final launch also feeds the neighbours' ghost rows: from its own
                    // stores when it is a temporally blocked launch, else by a copy kernel.
                    const int h = (int)p->halo, rows = (int)p->rows;
                    a.top_lo = h; a.top_hi = 2 * h; a.up_shift = (int)neighbours->up_rows;
                    a.bot_lo = rows; a.bot_hi = rows + h; a.dn_shift = -rows;
                    a.up_u = (float*)neighbours->up_u; a.up_v = (float*)neighbours->up_v;
                    a.dn_u = (float*)neighbours->down_u; a.dn_v = (float*)neighbours->down_v;
                    a.push = k >= 2 ? 1 : 0;
                }
                PD_CUDA_TRY(mt->gray_scott(a, variant, st));
                if (last && neighbours && !a.push) PD_CUDA_TRY(mt->gray_scott(a, -1, st));
                src_u = a.uo; src_v = a.vo;
                to_out = !to_out;
                done += k;
            }
            break;
        }
        case PD_FAMILY_LV_RK4_DF32: {
            const pd_lv_rk4_df32_params* p = static_cast<const pd_lv_rk4_df32_params*>(params);
            PdDfLvArgs a;
            a.x0 = (const float*)in[0]; a.y0 = (const float*)in[1]; a.a = (const float*)in[2];
            a.b = (const float*)in[3]; a.c = (const float*)in[4]; a.d = (const float*)in[5];
            a.xo = (float*)out[0]; a.yo = (float*)out[1];
            a.n = n; a.steps = (int)p->steps; a.dt = (float)p->dt;
            PD_CUDA_TRY(pd_launch_lv_df32(a, b, st));
            break;
        }
        case PD_FAMILY_KEPLER_RK4_DF32: {
            const pd_kepler_rk4_df32_params* p = static_cast<const pd_kepler_rk4_df32_params*>(params);
            PdKeplerArgs a;
            for (int i = 0; i < 8; ++i) { a.in[i] = (const float*)in[i]; a.out[i] = (float*)out[i]; }
            a.n = n; a.steps = (int)p->steps;
            split_df32(p->dt, &a.dt_hi, &a.dt_lo);
            split_df32(p->gm, &a.gm_hi, &a.gm_lo);
            PD_CUDA_TRY(pd_launch_kepler_df32(a, b, st));
            break;
        }
        case PD_FAMILY_THREEFRY_BITS: {
            const pd_threefry_params* p = static_cast<const pd_threefry_params*>(params);
            PdThreefryArgs a;
            a.key = (const uint32_t*)in[0];
            a.data = p->op == 2 ? (const uint32_t*)in[1] : nullptr;
            a.out = out[0]; a.n = n; a.count = p->count; a.op = (int)p->op;
            PD_CUDA_TRY(pd_launch_threefry(a, b, st));
            break;
        }
        case PD_FAMILY_SOURCE: {
            std::vector<void*> buffers;
            for (int i = 0; i < n_in; ++i) buffers.push_back(const_cast<void*>(in[i]));
            for (int i = 0; i < n_out; ++i) buffers.push_back(out[i]);
            const int64_t logical[3] = {grid[0], grid[1] > 0 ? grid[1] : 1, grid[2] > 0 ? grid[2] : 1};
            rc = pd_rtc_launch_source(plan.rtc, plan.grid, plan.block, logical, (int)buffers.size(), buffers.data(),
                                      (void*)st, err, err_cap);
            if (rc) return rc;
            break;
        }
        case PD_FAMILY_CUSTOM_ODE: {
            const pd_custom_ode_params* p = static_cast<const pd_custom_ode_params*>(params);
            PdOdeArgs a;
            memset(&a, 0, sizeof(a));
            for (int i = 0; i < n_in; ++i) a.in[i] = (const float*)in[i];
            for (int i = 0; i < n_out; ++i) a.out[i] = (float*)out[i];
            a.n = n;
            a.steps = (int)p->steps; a.max_steps = (int)p->max_steps;
            a.h_half = (float)(0.5 * p->dt); a.h_full = (float)p->dt; a.h_sixth = (float)(p->dt / 6.0);
            a.t1 = (float)p->t1; a.rtol = (float)p->rtol; a.atol = (float)p->atol; a.dt0 = (float)p->dt0;
            a.safety = (float)p->safety; a.factor_min = (float)p->factor_min; a.factor_max = (float)p->factor_max;
            if (p->method != PD_ODE_RK4) {
                a.coeff1 = (float)((p->icoeff + p->pcoeff) / (double)p->error_order);
                a.coeff2 = (float)(-p->pcoeff / (double)p->error_order);
                a.cursor = (unsigned long long*)scratch;
                a.refill_every = (int)knob(K_vdp_refill_every);
                if (a.refill_every < 1) a.refill_every = 1;
                PD_CUDA_TRY(cudaMemsetAsync(scratch, 0, 256, st));
            }
            rc = pd_rtc_launch(plan.rtc, plan.grid[0], b, a, (void*)st, err, err_cap);
            if (rc) return rc;
            break;
        }
        default:
            return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "unknown kernel family %d", family);
    }

    if (timed) {
        PD_CUDA_TRY(cudaEventRecord(ev1, st));
        PD_CUDA_TRY(cudaEventSynchronize(ev1));
        float ms = 0.0f;
        PD_CUDA_TRY(cudaEventElapsedTime(&ms, ev0, ev1));
        t_last_kernel_ms = ms;
        cudaEventDestroy(ev0);
        cudaEventDestroy(ev1);
    }
    return PD_OK;
}

// Per-thread staging state for pd_dispatch_host.
const int kHostStreams = 8;   // streams created per staging thread; `host_streams` of them are used
// Copies out of ordinary (pageable) host memory.  The driver moves such memory to the device at 7-15
// GB/s and keeps the calling thread busy meanwhile; a few threads copying slices into page-locked
// staging memory, from which the upload is a true asynchronous DMA, are several times faster.
class CopyPool {
public:
    struct Job { char* dst; const char* src; size_t bytes; };
    // every dst <- src of `copies`, cut into slices shared out among up to `helpers` helper threads and
    // the caller; returns when every byte is copied
    void copy(const std::vector<Job>& copies, int helpers) {
        const size_t kSlice = (size_t)128 << 10;
        size_t total = 0;
        for (const Job& j : copies) total += j.bytes;
        if (helpers <= 0 || total < 4 * kSlice) {
            for (const Job& j : copies) memcpy(j.dst, j.src, j.bytes);
            return;
        }
        std::lock_guard<std::mutex> one_at_a_time(call_mutex_);
        ensure_workers(helpers);
        {
            std::lock_guard<std::mutex> lock(m_);
            jobs_.clear();
            for (const Job& j : copies)
                for (size_t off = 0; off < j.bytes; off += kSlice)
                    jobs_.push_back(Job{j.dst + off, j.src + off, off + kSlice <= j.bytes ? kSlice : j.bytes - off});
            next_ = 0;
            pending_ = (int)jobs_.size();
        }
        cv_work_.notify_all();
        run_jobs();
        std::unique_lock<std::mutex> lock(m_);
        cv_done_.wait(lock, [&] { return pending_ == 0; });
    }

private:
    void ensure_workers(int n) {
        if (n > 16) n = 16;
        while ((int)started_ < n) {
            std::thread([this] { for (;;) { wait_for_work(); run_jobs(); } }).detach();   // lives as long as the process
            ++started_;
        }
    }
    void wait_for_work() {
        std::unique_lock<std::mutex> lock(m_);
        cv_work_.wait(lock, [&] { return next_ < jobs_.size(); });
    }
    void run_jobs() {
        for (;;) {
            Job job;
            {
                std::lock_guard<std::mutex> lock(m_);
                if (next_ >= jobs_.size()) return;
                job = jobs_[next_++];
            }
            memcpy(job.dst, job.src, job.bytes);
            std::lock_guard<std::mutex> lock(m_);
            if (--pending_ == 0) cv_done_.notify_all();
        }
    }
    std::mutex call_mutex_, m_;
    std::condition_variable cv_work_, cv_done_;
    std::vector<Job> jobs_;
    size_t next_ = 0;
    int pending_ = 0;
    unsigned started_ = 0;
};
CopyPool& copy_pool() {
    static CopyPool* pool = new CopyPool();   // never destroyed: its threads may outlive static destruction
    return *pool;
}
bool is_pageable(const void* ptr) {
    cudaPointerAttributes attr;
    const bool yes = cudaPointerGetAttributes(&attr, ptr) == cudaSuccess && attr.type == cudaMemoryTypeUnregistered;
    cudaGetLastError();
    return yes;
}

struct StageBuffer { unsigned char* ptr = nullptr; size_t bytes = 0; cudaEvent_t uploaded = nullptr; bool in_use = false; };

struct HostStaging {
    int device = -1;
    StageBuffer stage[8];                          // page-locked staging for pageable inputs, one per chunk stream
    cudaStream_t stream = nullptr;                 // stream 0, also used for unchunked calls
    cudaStream_t streams[kHostStreams] = {};
    cudaEvent_t broadcast_done = nullptr;
    std::vector<ScratchSlot> slots;
    ~HostStaging() {
        // Device memory is reclaimed when the context goes away; freeing here
        // could run after the runtime has shut down.
    }
};
thread_local HostStaging t_staging;

}  // namespace

// cuTensorMapEncodeTiled through the runtime's driver entry point table (no link against libcuda).
cudaError_t pd_encode_field_map(CUtensorMap* map, const float* base, int rows, int cols, int box_rows, int box_cols) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status) == cudaSuccess &&
            status == cudaDriverEntryPointSuccess)
            encode = reinterpret_cast<EncodeFn>(fn);
        else
            cudaGetLastError();
    });
    if (!encode) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * sizeof(float)};   // bytes between rows; a multiple of 16
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1u, 1u};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

extern "C" {

int pd_version(void) { return PD_ABI_VERSION; }

int pd_device_count(void) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return count;
}

int pd_launch(int family, const void* params, size_t params_bytes, int math_mode, const int64_t grid[3],
              const int64_t block[3], int n_in, const void* const* in, const size_t* in_bytes, int n_out,
              void* const* out, const size_t* out_bytes, void* workspace, size_t workspace_bytes,
              void* cuda_stream, char* err, size_t err_cap) {
    return launch_impl(family, params, params_bytes, math_mode, grid, block, n_in, in, in_bytes, n_out, out,
                       out_bytes, workspace, workspace_bytes, (cudaStream_t)cuda_stream, err, err_cap);
}

int pd_gray_scott_slab_push(const pd_gray_scott_params* params, int math_mode, const void* u, const void* v,
                            void* uo, void* vo, const pd_gs_neighbours* nb, void* workspace, size_t workspace_bytes,
                            void* cuda_stream, char* err, size_t err_cap) {
    if (!params || !nb) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "params and neighbours must not be NULL");
    if (params->halo <= 0)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gray_scott push: the call needs a slab (halo > 0)");
    if (params->steps <= 0)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gray_scott push: steps must be positive");
    if (params->rows < params->halo)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                    "gray_scott push: a slab of %lld rows cannot serve %lld halo rows", (long long)params->rows,
                    (long long)params->halo);
    if (!nb->up_u || !nb->up_v || !nb->down_u || !nb->down_v)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gray_scott push: neighbour pointers must not be NULL");
    if (nb->up_rows < params->halo || nb->down_rows < params->halo)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gray_scott push: neighbour slabs are smaller than the halo");
    if (!aligned(nb->up_u, 16) || !aligned(nb->up_v, 16) || !aligned(nb->down_u, 16) || !aligned(nb->down_v, 16))
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gray_scott push: neighbour fields must be 16-byte aligned");
    const int64_t grid[3] = {params->rows, params->cols, 1};
    const size_t bytes = (size_t)(params->rows + 2 * params->halo) * (size_t)params->cols * sizeof(float);
    const void* in[2] = {u, v};
    void* out[2] = {uo, vo};
    const size_t sizes[2] = {bytes, bytes};
    return launch_impl(PD_FAMILY_GRAY_SCOTT, params, sizeof(*params), math_mode, grid, nullptr, 2, in, sizes, 2, out,
                       sizes, workspace, workspace_bytes, (cudaStream_t)cuda_stream, err, err_cap, nb);
}

int pd_peer_alloc(size_t bytes, void** ptr, char* err, size_t err_cap) {
    if (!ptr || bytes == 0) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "pd_peer_alloc: bad arguments");
    PD_CUDA_TRY(cudaMalloc(ptr, bytes));
    return PD_OK;
}

int pd_peer_export(void* ptr, unsigned char handle[PD_PEER_HANDLE_BYTES], char* err, size_t err_cap) {
    static_assert(sizeof(cudaIpcMemHandle_t) == PD_PEER_HANDLE_BYTES, "IPC handle size");
    if (!ptr || !handle) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "pd_peer_export: bad arguments");
    cudaIpcMemHandle_t h;
    PD_CUDA_TRY(cudaIpcGetMemHandle(&h, ptr));
    memcpy(handle, &h, sizeof h);
    return PD_OK;
}

int pd_peer_open(const unsigned char handle[PD_PEER_HANDLE_BYTES], void** ptr, char* err, size_t err_cap) {
    if (!ptr || !handle) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "pd_peer_open: bad arguments");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    PD_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return PD_OK;
}

int pd_peer_close(void* ptr, char* err, size_t err_cap) {
    if (!ptr) return PD_OK;
    PD_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return PD_OK;
}

int pd_peer_free(void* ptr, char* err, size_t err_cap) {
    if (!ptr) return PD_OK;
    PD_CUDA_TRY(cudaFree(ptr));
    return PD_OK;
}

int pd_dispatch_host(int family, const void* params, size_t params_bytes, int math_mode, const int64_t grid[3],
                     const int64_t block[3], int n_in, const void* const* in, const size_t* in_bytes, int n_out,
                     void* const* out, const size_t* out_bytes, char* err, size_t err_cap) {
    DeviceFacts dev = device_facts();
    if (!dev.present)
        return fail(PD_ERR_CUDA, err, err_cap,
                    "no CUDA device is available: libpalladium_cuda has no CPU fallback");
    if (n_in < 0 || n_out < 0 || n_in > 64 || n_out > 64)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "buffer count out of range");
    if ((n_in > 0 && (!in || !in_bytes)) || (n_out > 0 && (!out || !out_bytes)))
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "buffer arrays must not be NULL");
    HostStaging& hs = t_staging;
    if (hs.device != dev.device) {
        hs.device = dev.device;
        hs.stream = nullptr;
        for (int i = 0; i < kHostStreams; ++i) hs.streams[i] = nullptr;
        hs.broadcast_done = nullptr;
        hs.slots.clear();
        for (StageBuffer& sb : hs.stage) { sb.uploaded = nullptr; sb.in_use = false; }   // events belong to a device
    }
    if (!hs.stream) {
        for (int i = 0; i < kHostStreams; ++i)
            PD_CUDA_TRY(cudaStreamCreateWithFlags(&hs.streams[i], cudaStreamNonBlocking));
        hs.stream = hs.streams[0];
        PD_CUDA_TRY(cudaEventCreateWithFlags(&hs.broadcast_done, cudaEventDisableTiming));
    }
    const int total = n_in + n_out;
    if ((int)hs.slots.size() < total) hs.slots.resize(total);
    std::vector<const void*> d_in(n_in);
    std::vector<void*> d_out(n_out);
    for (int i = 0; i < total; ++i) {
        const size_t bytes = i < n_in ? in_bytes[i] : out_bytes[i - n_in];
        ScratchSlot& slot = hs.slots[i];
        if (slot.bytes < bytes || !slot.ptr) {
            if (slot.ptr) PD_CUDA_TRY(cudaFree(slot.ptr));
            slot.ptr = nullptr; slot.bytes = 0;
            const size_t want = bytes < 256 ? 256 : bytes;
            PD_CUDA_TRY(cudaMalloc(&slot.ptr, want));
            slot.bytes = want;
        }
        if (i < n_in) d_in[i] = slot.ptr; else d_out[i - n_in] = slot.ptr;
    }
    for (int i = 0; i < n_in; ++i)
        if (in_bytes[i] && !in[i]) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "input %d: NULL pointer", i);
    for (int i = 0; i < n_out; ++i)
        if (out_bytes[i] && !out[i]) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "output %d: NULL pointer", i);

    // ---- chunked pipeline for the per-trajectory families ------------------------------
    // Trajectories (paths) are independent, so a large call is cut into chunks
    // that travel round-robin over a few streams (`host_streams`): while chunk c integrates, the
    // inputs of chunk c+1 are uploading and the results of chunk c-1 are
    // downloading.  A buffer whose size is not proportional to the trajectory
    // count (the RNG key) is uploaded once and the chunk streams wait for it.
    const bool per_item_family = family == PD_FAMILY_LV_RK4 || (family == PD_FAMILY_VDP_BS32 && n_in == 3) ||
                                 family == PD_FAMILY_LV_RK4_DF32 || family == PD_FAMILY_KEPLER_RK4_DF32 ||
                                 family == PD_FAMILY_CUSTOM_ODE ||
                                 ((family == PD_FAMILY_GBM_THREEFRY || family == PD_FAMILY_GBM_PCG) && n_out == 1);
    const int64_t n = grid ? grid[0] : 0;
    const int64_t kMinChunked = (int64_t)1 << 18;
    bool chunked = per_item_family && n >= kMinChunked && params && params_bytes <= 256;
    std::vector<size_t> in_item(n_in, 0), out_item(n_out, 0);
    if (chunked) {
        for (int i = 0; i < n_in; ++i)
            if (in_bytes[i] % (size_t)n == 0 && in_bytes[i] / (size_t)n >= 4) in_item[i] = in_bytes[i] / (size_t)n;
        for (int i = 0; i < n_out; ++i) {
            if (out_bytes[i] % (size_t)n == 0 && out_bytes[i] / (size_t)n >= 4) out_item[i] = out_bytes[i] / (size_t)n;
            else chunked = false;
        }
    }
    if (chunked) {
        // Chunk boundaries.  host_chunks > 0: that many equal chunks.  host_chunks == 0:
        // a ramp -- small chunks first and last, large ones between -- so that the
        // upload of the first chunk and the download of the last one, which nothing
        // can hide, are short, while most of the work runs in launches large enough
        // for the kernels' best configuration.
        std::vector<int64_t> bounds;   // chunk c covers [bounds[c], bounds[c + 1])
        {
            int64_t want_chunks = knob(K_host_chunks);
            if (want_chunks < 0) {
                // about 2^17 trajectories per chunk measured best from 2^20 to 2^22 (8 / 16 / 32
                // chunks); beyond that more, larger chunks
                want_chunks = n >> 17;
                if (want_chunks < 8) want_chunks = 8;
                if (want_chunks > 48) want_chunks = 48;
                // An adaptive launch balances its trajectories through a work queue, which a cut into
                // chunks defeats (each chunk ends with its own tail of long trajectories), and its copies
                // are small beside the kernel: measured at 10^6 Van der Pol oscillators, SAFE, 8 / 4 / 2 /
                // 1 chunks: 18.3 / 17.0 / 15.7 / 15.1 ms (BS3(2)); 4.0 / 3.8 / 3.45 / 3.5 ms (Tsit5).
                if (family == PD_FAMILY_VDP_BS32) want_chunks = 1;
                if (family == PD_FAMILY_CUSTOM_ODE &&
                    static_cast<const pd_custom_ode_params*>(params)->method != PD_ODE_RK4)
                    want_chunks = n >= ((int64_t)1 << 19) ? 2 : 1;
            }
            if (want_chunks > 0) {
                int64_t chunk = ((n + want_chunks - 1) / want_chunks + 4095) / 4096 * 4096;  // 16 KiB-aligned slices
                if (chunk < ((int64_t)1 << 16)) chunk = (int64_t)1 << 16;
                for (int64_t lo = 0; lo < n; lo += chunk) bounds.push_back(lo);
            } else {
                static const int ramp64[] = {1, 1, 2, 4, 8, 8, 8, 8, 8, 8, 4, 2, 1, 1};
                static const int ramp32[] = {1, 1, 2, 4, 8, 8, 4, 2, 1, 1};
                static const int ramp16[] = {1, 1, 2, 4, 4, 2, 1, 1};
                const int* ramp = ramp16; int parts = 8, units = 16;
                if (n >= ((int64_t)1 << 22)) { ramp = ramp64; parts = 14; units = 64; }
                else if (n >= ((int64_t)1 << 21)) { ramp = ramp32; parts = 10; units = 32; }
                const int64_t unit = (n / units + 4095) / 4096 * 4096;
                int64_t lo = 0;
                for (int i = 0; i < parts && lo < n; ++i) {
                    bounds.push_back(lo);
                    lo += unit * ramp[i];
                }
            }
            bounds.push_back(n);
        }
        int n_streams = (int)knob(K_host_streams);
        n_streams = n_streams < 1 ? 1 : (n_streams > kHostStreams ? kHostStreams : n_streams);
        // From the first queued copy on, an error must not return before every stream has been
        // drained: queued copies still read and write the caller's host buffers, and the call is
        // blocking by contract.  Errors are recorded in rc and end the loops; the synchronise
        // loop at the end always runs.
        int rc = PD_OK;
        auto cuda_ok = [&](cudaError_t e, const char* what) {
            if (e == cudaSuccess) return true;
            if (rc == PD_OK) rc = fail(PD_ERR_CUDA, err, err_cap, "%s failed: %s", what, cudaGetErrorString(e));
            return false;
        };
        bool any_broadcast = false;
        for (int i = 0; i < n_in && rc == PD_OK; ++i) {
            if (in_item[i] == 0 && in_bytes[i]) {
                cuda_ok(cudaMemcpyAsync(hs.slots[i].ptr, in[i], in_bytes[i], cudaMemcpyHostToDevice, hs.streams[0]),
                        "cudaMemcpyAsync (shared input)");
                any_broadcast = true;
            }
        }
        if (any_broadcast && rc == PD_OK) {
            cuda_ok(cudaEventRecord(hs.broadcast_done, hs.streams[0]), "cudaEventRecord");
            for (int sidx = 1; sidx < n_streams && rc == PD_OK; ++sidx)
                cuda_ok(cudaStreamWaitEvent(hs.streams[sidx], hs.broadcast_done, 0), "cudaStreamWaitEvent");
        }
        unsigned char local_params[256];
        memcpy(local_params, params, params_bytes);
        // A chunk is far below the size at which a launch of its own would trade threads for
        // per-thread parallelism, but several chunks share the GPU at any time: four trajectories
        // per thread measured 2 % faster end to end (3.94 -> 3.85 ms per pass at 2^22) than one.
        // A caller's own setting of the knob, for this thread or process-wide, is left alone.
        const bool chunk_items = family == PD_FAMILY_LV_RK4 && !t_knobs.set[K_lv_items_per_thread] &&
                                 g_knobs[K_lv_items_per_thread].load(std::memory_order_relaxed) == 0;
        if (chunk_items) { t_knobs.set[K_lv_items_per_thread] = true; t_knobs.value[K_lv_items_per_thread] = 4; }
        int c = 0;
        std::vector<const void*> c_in(n_in);
        std::vector<void*> c_out(n_out);
        std::vector<size_t> c_in_bytes(n_in), c_out_bytes(n_out);
        // Inputs in ordinary (pageable) memory go through the stream's page-locked staging buffer,
        // filled by the copy threads: 100 MB of NumPy arrays upload in 13.6 ms through the driver's
        // own pageable path and in a third of that this way, overlapped with the kernels.
        const int copy_helpers = (int)knob(K_host_copy_threads);
        std::vector<char> staged(n_in, 0);
        bool any_staged = false;
        size_t in_total = 0;
        for (int i = 0; i < n_in; ++i) in_total += in_bytes[i];
        // (a call below 16 MB is over before the threads are awake: 6 MB took 824 us with them, 544 without)
        for (int i = 0; i < n_in; ++i)
            if (copy_helpers > 0 && in_total >= ((size_t)16 << 20) && in_item[i] && in_bytes[i] && is_pageable(in[i])) {
                staged[i] = 1;
                any_staged = true;
            }
        for (; c + 1 < (int)bounds.size() && rc == PD_OK; ++c) {
            const int64_t lo = bounds[c];
            const int64_t len = bounds[c + 1] - lo;
            const int sidx = c % n_streams;
            cudaStream_t st = hs.streams[sidx];
            StageBuffer& stage = hs.stage[sidx];
            size_t stage_off = 0;
            std::vector<CopyPool::Job> stage_jobs;
            if (any_staged) {
                size_t need = 0;
                for (int i = 0; i < n_in; ++i)
                    if (staged[i]) need += ((size_t)len * in_item[i] + 255) / 256 * 256;
                if (stage.in_use && !cuda_ok(cudaEventSynchronize(stage.uploaded), "cudaEventSynchronize")) break;
                stage.in_use = false;
                if (stage.bytes < need) {
                    if (stage.ptr) cudaFreeHost(stage.ptr);
                    stage.ptr = nullptr; stage.bytes = 0;
                    if (!cuda_ok(cudaHostAlloc((void**)&stage.ptr, need, cudaHostAllocDefault), "cudaHostAlloc")) break;
                    stage.bytes = need;
                }
                if (!stage.uploaded &&
                    !cuda_ok(cudaEventCreateWithFlags(&stage.uploaded, cudaEventDisableTiming), "cudaEventCreateWithFlags"))
                    break;
            }
            for (int i = 0; i < n_in; ++i) {
                if (in_item[i]) {
                    const size_t off = (size_t)lo * in_item[i];
                    c_in[i] = (const char*)hs.slots[i].ptr + off;
                    c_in_bytes[i] = (size_t)len * in_item[i];
                    if (staged[i]) {
                        stage_jobs.push_back(CopyPool::Job{(char*)stage.ptr + stage_off, (const char*)in[i] + off, c_in_bytes[i]});
                        stage_off += (c_in_bytes[i] + 255) / 256 * 256;
                    }
                } else {
                    c_in[i] = hs.slots[i].ptr;
                    c_in_bytes[i] = in_bytes[i];
                }
            }
            if (!stage_jobs.empty()) copy_pool().copy(stage_jobs, copy_helpers);   // all staged inputs of the chunk at once
            size_t job = 0;
            for (int i = 0; i < n_in && rc == PD_OK; ++i) {
                if (!in_item[i]) continue;
                const size_t off = (size_t)lo * in_item[i];
                const void* src = staged[i] ? (const void*)stage_jobs[job++].dst : (const void*)((const char*)in[i] + off);
                cuda_ok(cudaMemcpyAsync((char*)hs.slots[i].ptr + off, src, c_in_bytes[i], cudaMemcpyHostToDevice, st),
                        "cudaMemcpyAsync (upload)");
            }
            if (rc) break;
            if (any_staged && rc == PD_OK && cuda_ok(cudaEventRecord(stage.uploaded, st), "cudaEventRecord"))
                stage.in_use = true;
            for (int i = 0; i < n_out; ++i) {
                c_out[i] = (char*)hs.slots[n_in + i].ptr + (size_t)lo * out_item[i];
                c_out_bytes[i] = (size_t)len * out_item[i];
            }
            if (family == PD_FAMILY_GBM_THREEFRY || family == PD_FAMILY_GBM_PCG) {
                pd_gbm_params gp;
                memcpy(&gp, params, sizeof(gp));
                gp.path_offset += lo;
                memcpy(local_params, &gp, sizeof(gp));
            }
            if (rc) break;
            const int64_t c_grid[3] = {len, grid[1], grid[2]};
            rc = launch_impl(family, local_params, params_bytes, math_mode, c_grid, block, n_in, c_in.data(),
                             c_in_bytes.data(), n_out, c_out.data(), c_out_bytes.data(), nullptr, 0, st, err, err_cap);
            if (rc) break;
            for (int i = 0; i < n_out && rc == PD_OK; ++i)
                cuda_ok(cudaMemcpyAsync((char*)out[i] + (size_t)lo * out_item[i], c_out[i], c_out_bytes[i],
                                        cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync (download)");
        }
        if (chunk_items) t_knobs.set[K_lv_items_per_thread] = false;
        for (int sidx = 0; sidx < kHostStreams; ++sidx) {
            cudaError_t e = cudaStreamSynchronize(hs.streams[sidx]);
            if (e != cudaSuccess && rc == PD_OK)
                rc = fail(PD_ERR_CUDA, err, err_cap, "cudaStreamSynchronize failed: %s", cudaGetErrorString(e));
        }
        for (int sidx = 0; sidx < kHostStreams; ++sidx) hs.stage[sidx].in_use = false;   // every upload has finished
        if (rc == PD_OK) rc = check_device_status(dev.device, err, err_cap);
        return rc;
    }

    // ---- one upload, one launch sequence, one download --------------------------------
    int rc = PD_OK;
    {
        // large pageable inputs: into page-locked staging by the copy threads, then one DMA each
        const int copy_helpers = (int)knob(K_host_copy_threads);
        StageBuffer& stage = hs.stage[0];
        size_t need = 0;
        std::vector<char> staged(n_in, 0);
        size_t in_total = 0;
        for (int i = 0; i < n_in; ++i) in_total += in_bytes[i];
        for (int i = 0; i < n_in; ++i)
            if (copy_helpers > 0 && in_total >= ((size_t)16 << 20) && in_bytes[i] >= ((size_t)1 << 20) && is_pageable(in[i])) {
                staged[i] = 1;   // smaller calls are quicker through the driver's own pageable copy than after waking the threads
                need += (in_bytes[i] + 255) / 256 * 256;
            }
        if (need > stage.bytes) {
            if (stage.ptr) cudaFreeHost(stage.ptr);
            stage.ptr = nullptr; stage.bytes = 0;
            cudaError_t e = cudaHostAlloc((void**)&stage.ptr, need, cudaHostAllocDefault);
            if (e != cudaSuccess) {
                cudaGetLastError();
                std::fill(staged.begin(), staged.end(), 0);   // no staging memory: the driver's pageable path still works
            } else {
                stage.bytes = need;
            }
        }
        size_t stage_off = 0;
        std::vector<CopyPool::Job> stage_jobs;
        for (int i = 0; i < n_in; ++i)
            if (staged[i]) {
                stage_jobs.push_back(CopyPool::Job{(char*)stage.ptr + stage_off, (const char*)in[i], in_bytes[i]});
                stage_off += (in_bytes[i] + 255) / 256 * 256;
            }
        if (!stage_jobs.empty()) copy_pool().copy(stage_jobs, copy_helpers);
        size_t job = 0;
        for (int i = 0; i < n_in && rc == PD_OK; ++i) {
            if (!in_bytes[i]) continue;
            const void* src = staged[i] ? (const void*)stage_jobs[job++].dst : in[i];
            cudaError_t e = cudaMemcpyAsync(hs.slots[i].ptr, src, in_bytes[i], cudaMemcpyHostToDevice, hs.stream);
            if (e != cudaSuccess) rc = fail(PD_ERR_CUDA, err, err_cap, "cudaMemcpyAsync (upload) failed: %s", cudaGetErrorString(e));
        }
    }
    if (rc == PD_OK)
        rc = launch_impl(family, params, params_bytes, math_mode, grid, block, n_in, d_in.data(), in_bytes, n_out,
                         d_out.data(), out_bytes, nullptr, 0, hs.stream, err, err_cap);
    for (int i = 0; i < n_out && rc == PD_OK; ++i) {
        if (!out_bytes[i]) continue;
        cudaError_t e = cudaMemcpyAsync(out[i], d_out[i], out_bytes[i], cudaMemcpyDeviceToHost, hs.stream);
        if (e != cudaSuccess) rc = fail(PD_ERR_CUDA, err, err_cap, "cudaMemcpyAsync (download) failed: %s", cudaGetErrorString(e));
    }
    // the call is blocking by contract: queued copies still use the caller's buffers, so drain on every path
    cudaError_t e = cudaStreamSynchronize(hs.stream);
    if (e != cudaSuccess && rc == PD_OK)
        rc = fail(PD_ERR_CUDA, err, err_cap, "cudaStreamSynchronize failed: %s", cudaGetErrorString(e));
    if (rc == PD_OK) rc = check_device_status(dev.device, err, err_cap);
    return rc;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Asynchronous host-buffer calls: pd_submit_host / pd_wait_host.
// A slot owns one page-locked host block and one device block (inputs first, then outputs, each
// at a 256-byte offset), a stream and an event.  Submitting packs the inputs into the host block
// -- so the caller may change its arrays as soon as the call returns -- and queues ONE upload,
// the kernels and ONE download on the slot's stream; waiting synchronises the event, copies the
// results out and frees the slot for the next submission.
// ---------------------------------------------------------------------------
namespace {

struct AsyncSlot {
    int device = -1;
    bool busy = false;
    uint64_t ticket = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t done = nullptr;
    unsigned char* host = nullptr;
    unsigned char* dev = nullptr;
    size_t capacity = 0, host_capacity = 0;   // bytes of the device block and of the host block
    size_t out_begin = 0;
    bool direct_out = false;   // the results went straight to arrays the caller named at submission
    std::vector<size_t> out_offset, out_bytes;
};
const int kMaxAsyncSlots = 64;
const size_t kCopyThreadsFromBytes = (size_t)16 << 20;   // calls with at least this much input use the copy threads
std::mutex g_async_mutex;
std::vector<AsyncSlot*>& async_slots() {
    static std::vector<AsyncSlot*> slots;
    return slots;
}
uint64_t g_next_ticket = 1;

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace

extern "C" {

int pd_submit_host(int family, const void* params, size_t params_bytes, int math_mode, const int64_t grid[3],
                   const int64_t block[3], int n_in, const void* const* in, const size_t* in_bytes,
                   const int* in_on_device, int n_out, void* const* out, const size_t* out_bytes, uint64_t* ticket,
                   char* err, size_t err_cap) {
    DeviceFacts dev = device_facts();
    if (!dev.present)
        return fail(PD_ERR_CUDA, err, err_cap, "no CUDA device is available: libpalladium_cuda has no CPU fallback");
    if (!ticket) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "ticket must not be NULL");
    if (n_in < 0 || n_out < 0 || n_in > 64 || n_out > 64)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "buffer count out of range");
    if ((n_in > 0 && (!in || !in_bytes)) || (n_out > 0 && !out_bytes))
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "buffer arrays must not be NULL");
    for (int i = 0; i < n_in; ++i)
        if (in_bytes[i] && !in[i]) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "input %d: NULL pointer", i);
    // Device block: every input that is not on the device already, then the outputs.  Host block:
    // the same inputs at the same offsets (copied there by the copy threads, so that the caller's
    // arrays are free again when this returns and the upload is one asynchronous copy whatever
    // memory they live in), then the outputs unless the caller named page-locked result arrays.
    auto on_device = [&](int i) { return in_on_device && in_on_device[i]; };
    std::vector<size_t> in_offset(n_in), out_offset(n_out);
    size_t total = 0, host_total = 0;
    for (int i = 0; i < n_in; ++i) {
        in_offset[i] = total;
        if (on_device(i) || !in_bytes[i]) continue;
        total += align256(in_bytes[i]);
    }
    host_total = total;
    const size_t out_begin = total, host_out_begin = host_total;
    for (int i = 0; i < n_out; ++i) {
        out_offset[i] = total;
        total += align256(out_bytes[i]);
        if (!out) host_total += align256(out_bytes[i]);
    }
    if (total == 0) total = 256;
    if (host_total == 0) host_total = 256;

    AsyncSlot* slot = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_async_mutex);
        std::vector<AsyncSlot*>& slots = async_slots();
        for (AsyncSlot* s : slots)   // a free slot that is large enough, else any free slot (it grows below)
            if (!s->busy && s->device == dev.device && s->capacity >= total && s->host_capacity >= host_total) { slot = s; break; }
        if (!slot)
            for (AsyncSlot* s : slots)
                if (!s->busy && s->device == dev.device) { slot = s; break; }
        if (!slot) {
            if ((int)slots.size() >= kMaxAsyncSlots)
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                            "%d host-buffer calls are in flight: wait for earlier results before submitting more",
                            kMaxAsyncSlots);
            slot = new AsyncSlot();
            slot->device = dev.device;
            slots.push_back(slot);
        }
        slot->busy = true;
        slot->ticket = g_next_ticket++;
    }
    auto release = [&](int rc) {
        std::lock_guard<std::mutex> lock(g_async_mutex);
        slot->busy = false;
        return rc;
    };
    auto cuda_fail = [&](cudaError_t e, const char* what) {
        cudaGetLastError();
        return release(fail(PD_ERR_CUDA, err, err_cap, "%s failed: %s", what, cudaGetErrorString(e)));
    };
    cudaError_t e;
    if (!slot->stream) {
        if ((e = cudaStreamCreateWithFlags(&slot->stream, cudaStreamNonBlocking)) != cudaSuccess)
            return cuda_fail(e, "cudaStreamCreateWithFlags");
        if ((e = cudaEventCreateWithFlags(&slot->done, cudaEventDisableTiming)) != cudaSuccess)
            return cuda_fail(e, "cudaEventCreateWithFlags");
    }
    // the slot is free, so nothing of an earlier call still uses its blocks
    if (slot->capacity < total) {
        if (slot->dev) { cudaFree(slot->dev); slot->dev = nullptr; }
        slot->capacity = 0;
        const size_t want = total < 65536 ? 65536 : total;
        if ((e = cudaMalloc((void**)&slot->dev, want)) != cudaSuccess) return cuda_fail(e, "cudaMalloc");
        slot->capacity = want;
    }
    if (slot->host_capacity < host_total) {
        if (slot->host) { cudaFreeHost(slot->host); slot->host = nullptr; }
        slot->host_capacity = 0;
        const size_t want = host_total < 65536 ? 65536 : host_total;
        if ((e = cudaHostAlloc((void**)&slot->host, want, cudaHostAllocDefault)) != cudaSuccess)
            return cuda_fail(e, "cudaHostAlloc");
        slot->host_capacity = want;
    }
    // Three regimes, by what was measured (six arrays per call): below 256 KB the arrays are packed
    // by memcpy and go up in one copy (55 us per blocking call); from 16 MB on the copy threads fill
    // the host block (a 100 MB call: 13.6 -> 4.5 ms); in between, waking the threads costs more than
    // they save for a caller that blocks on every call (6 MB: 830 against 475 us), so pageable
    // arrays go straight to the driver, whose copy returns once the source has been staged.
    const bool by_threads = out_begin >= kCopyThreadsFromBytes && knob(K_host_copy_threads) > 0;
    if (out_begin < ((size_t)256 << 10) || by_threads) {
        std::vector<CopyPool::Job> copies;
        for (int i = 0; i < n_in; ++i)
            if (!on_device(i) && in_bytes[i])
                copies.push_back(CopyPool::Job{(char*)slot->host + in_offset[i], (const char*)in[i], in_bytes[i]});
        copy_pool().copy(copies, by_threads ? (int)knob(K_host_copy_threads) : 0);
        if (out_begin) {
            if ((e = cudaMemcpyAsync(slot->dev, slot->host, out_begin, cudaMemcpyHostToDevice, slot->stream)) != cudaSuccess)
                return cuda_fail(e, "cudaMemcpyAsync (upload)");
        }
    } else {
        for (int i = 0; i < n_in; ++i) {
            if (on_device(i) || !in_bytes[i]) continue;
            const void* src = in[i];
            if (!is_pageable(in[i])) {   // page-locked or managed: would be read after this returns
                memcpy(slot->host + in_offset[i], in[i], in_bytes[i]);
                src = slot->host + in_offset[i];
            }
            if ((e = cudaMemcpyAsync(slot->dev + in_offset[i], src, in_bytes[i], cudaMemcpyHostToDevice, slot->stream)) !=
                cudaSuccess) {
                cudaStreamSynchronize(slot->stream);
                return cuda_fail(e, "cudaMemcpyAsync (upload)");
            }
        }
    }
    std::vector<const void*> d_in(n_in);
    std::vector<void*> d_out(n_out);
    for (int i = 0; i < n_in; ++i) d_in[i] = on_device(i) ? in[i] : slot->dev + in_offset[i];
    for (int i = 0; i < n_out; ++i) d_out[i] = slot->dev + out_offset[i];
    int rc = launch_impl(family, params, params_bytes, math_mode, grid, block, n_in, d_in.data(), in_bytes, n_out,
                         d_out.data(), out_bytes, nullptr, 0, slot->stream, err, err_cap);
    if (rc) {
        cudaStreamSynchronize(slot->stream);   // the upload still reads the slot's host block
        return release(rc);
    }
    if (out) {
        // the caller's own (page-locked) result arrays: one download each, nothing to copy at the wait
        for (int i = 0; i < n_out; ++i) {
            if (!out_bytes[i]) continue;
            if (!out[i]) {
                cudaStreamSynchronize(slot->stream);
                return release(fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "output %d: NULL pointer", i));
            }
            if ((e = cudaMemcpyAsync(out[i], slot->dev + out_offset[i], out_bytes[i], cudaMemcpyDeviceToHost,
                                     slot->stream)) != cudaSuccess) {
                cudaStreamSynchronize(slot->stream);
                return cuda_fail(e, "cudaMemcpyAsync (download)");
            }
        }
    } else if (total > out_begin && n_out > 0) {
        // the outputs keep the spacing of the device block: one copy, unpacked at the wait
        if ((e = cudaMemcpyAsync(slot->host + host_out_begin, slot->dev + out_begin, total - out_begin,
                                 cudaMemcpyDeviceToHost, slot->stream)) != cudaSuccess) {
            cudaStreamSynchronize(slot->stream);
            return cuda_fail(e, "cudaMemcpyAsync (download)");
        }
    }
    if ((e = cudaEventRecord(slot->done, slot->stream)) != cudaSuccess) {
        cudaStreamSynchronize(slot->stream);
        return cuda_fail(e, "cudaEventRecord");
    }
    slot->out_begin = out_begin;
    for (size_t& o : out_offset) o = o - out_begin + host_out_begin;   // where each result lies in the host block
    slot->out_offset = out_offset;
    slot->out_bytes.assign(out_bytes, out_bytes + n_out);
    slot->direct_out = out != nullptr;
    *ticket = slot->ticket;
    return PD_OK;
}

int pd_wait_host(uint64_t ticket, int n_out, void* const* out, const size_t* out_bytes, char* err, size_t err_cap) {
    AsyncSlot* slot = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_async_mutex);
        for (AsyncSlot* s : async_slots())
            if (s->busy && s->ticket == ticket) { slot = s; break; }
    }
    if (!slot) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "unknown or already retired ticket");
    auto release = [&](int rc) {
        std::lock_guard<std::mutex> lock(g_async_mutex);
        slot->busy = false;
        return rc;
    };
    cudaError_t e = cudaEventSynchronize(slot->done);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return release(fail(PD_ERR_CUDA, err, err_cap, "cudaEventSynchronize failed: %s", cudaGetErrorString(e)));
    }
    int rc = check_device_status(slot->device, err, err_cap);
    if (rc) return release(rc);
    // a wait with unusable arguments leaves the ticket valid: the caller can wait again
    if (n_out != 0 && slot->direct_out)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                    "the results of this call went to the arrays named at submission; wait with n_out = 0");
    if (n_out != 0) {   // n_out == 0 retires the ticket without collecting anything
        if (n_out != (int)slot->out_bytes.size() || !out || !out_bytes)
            return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "the call produced %d arrays, %d were offered",
                        (int)slot->out_bytes.size(), n_out);
        for (int i = 0; i < n_out; ++i) {
            if (out_bytes[i] != slot->out_bytes[i] || (out_bytes[i] && !out[i]))
                return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "output %d: %zu bytes offered, %zu produced", i,
                            out_bytes[i], slot->out_bytes[i]);
        }
        for (int i = 0; i < n_out; ++i)
            if (out_bytes[i]) memcpy(out[i], slot->host + slot->out_offset[i], out_bytes[i]);
    }
    return release(PD_OK);
}

int pd_explain(int family, const void* params, size_t params_bytes, int math_mode, const int64_t grid[3],
               const int64_t block[3], pd_launch_info* info, char* err, size_t err_cap) {
    if (!info) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "info must not be NULL");
    DeviceFacts dev = device_facts();
    Plan plan;
    int rc = build_plan(family, params, params_bytes, math_mode, grid, block, true, dev, &plan, err, err_cap);
    if (rc) return rc;
    memset(info, 0, sizeof(*info));
    snprintf(info->kernel_name, sizeof(info->kernel_name), "%s", plan.kernel_name);
    for (int i = 0; i < 3; ++i) { info->cuda_grid[i] = plan.grid[i]; info->cuda_block[i] = plan.block[i]; }
    info->items_per_thread = plan.items;
    info->launches = plan.launches;
    info->scratch_bytes = plan.scratch_bytes;
    info->regs_per_thread = -1;
    info->static_smem_bytes = -1;
    info->dynamic_smem_bytes = (int32_t)plan.dynamic_smem;
    info->blocks_per_sm = -1;
    if (dev.present && plan.rtc.function) {
        info->regs_per_thread = plan.rtc.regs;
        info->static_smem_bytes = plan.rtc.static_smem;
        info->blocks_per_sm = plan.rtc.blocks_per_sm;
    }
    if (dev.present && plan.kernel) {
        cudaFuncAttributes attr;
        if (cudaFuncGetAttributes(&attr, plan.kernel) == cudaSuccess) {
            info->regs_per_thread = attr.numRegs;
            info->static_smem_bytes = (int32_t)attr.sharedSizeBytes;
            const int threads = (int)(plan.block[0] * plan.block[1] * plan.block[2]);
            info->blocks_per_sm = occupancy_blocks(plan.kernel, threads, (size_t)plan.dynamic_smem);
        } else {
            cudaGetLastError();
        }
    }
    return PD_OK;
}

int pd_set_tuning(const char* key, int64_t value) {
    const int i = key ? knob_index(key) : -1;
    if (i < 0) return PD_ERR_INVALID_ARGUMENT;
    g_knobs[i].store(value, std::memory_order_relaxed);
    return PD_OK;
}

int pd_get_tuning(const char* key, int64_t* value) {
    const int i = key ? knob_index(key) : -1;
    if (i < 0 || !value) return PD_ERR_INVALID_ARGUMENT;
    *value = knob((Knob)i);
    return PD_OK;
}

int pd_set_thread_tuning(const char* key, int64_t value) {
    const int i = key ? knob_index(key) : -1;
    if (i < 0) return PD_ERR_INVALID_ARGUMENT;
    t_knobs.set[i] = true;
    t_knobs.value[i] = value;
    return PD_OK;
}

int pd_clear_thread_tuning(const char* key) {
    if (!key) {
        t_knobs = ThreadKnobs();
        return PD_OK;
    }
    const int i = knob_index(key);
    if (i < 0) return PD_ERR_INVALID_ARGUMENT;
    t_knobs.set[i] = false;
    return PD_OK;
}

static int measure_chain(bool fp, double* out_rate, char* err, size_t err_cap) {
    if (!out_rate) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "result pointer must not be NULL");
    DeviceFacts dev = device_facts();
    if (!dev.present) return fail(PD_ERR_CUDA, err, err_cap, "no CUDA device is available");
    void* sink = nullptr;
    PD_CUDA_TRY(cudaMalloc(&sink, 256));
    cudaEvent_t e0, e1;
    PD_CUDA_TRY(cudaEventCreate(&e0));
    PD_CUDA_TRY(cudaEventCreate(&e1));
    const int grid = dev.sms * 8, block = 256, iters = 4096;
    double best = 0.0;
    for (int rep = 0; rep < 5; ++rep) {
        PD_CUDA_TRY(cudaEventRecord(e0, 0));
        if (fp) PD_CUDA_TRY(pd_launch_fma_chain((float*)sink, iters, grid, block, 0));
        else PD_CUDA_TRY(pd_launch_int_chain((uint32_t*)sink, iters, grid, block, 0));
        PD_CUDA_TRY(cudaEventRecord(e1, 0));
        PD_CUDA_TRY(cudaEventSynchronize(e1));
        float ms = 0.0f;
        PD_CUDA_TRY(cudaEventElapsedTime(&ms, e0, e1));
        // fp: 8 reps x 8 chains x 2 flops; int: 8 reps x 4 chains x 3 ops
        const double per_thread = fp ? (double)iters * 8 * 8 * 2 : (double)iters * 8 * 4 * 3;
        const double rate = per_thread * (double)grid * block / (ms * 1e-3);
        if (rep > 0 && rate > best) best = rate;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(sink);
    *out_rate = best;
    return PD_OK;
}

int pd_measure_fp32_fma_peak(double* flops_per_s, char* err, size_t err_cap) {
    return measure_chain(true, flops_per_s, err, err_cap);
}
int pd_measure_int32_alu_peak(double* ops_per_s, char* err, size_t err_cap) {
    return measure_chain(false, ops_per_s, err, err_cap);
}

double pd_last_kernel_ms(void) { return t_last_kernel_ms; }

int pd_device_status(int* code, int clear, char* err, size_t err_cap) {
    if (!code) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "code must not be NULL");
    DeviceFacts dev = device_facts();
    if (!dev.present) return fail(PD_ERR_CUDA, err, err_cap, "no CUDA device is available");
    volatile int* word = nullptr;
    if (dev.device >= 0 && dev.device < kMaxStatusDevices) {
        std::lock_guard<std::mutex> lock(g_status_mutex);
        word = g_status_host[dev.device];
    }
    *code = word ? *word : 0;   // no word yet: no kernel with bounded waits has run on this device
    if (word && clear) *word = 0;
    return PD_OK;
}

}  // extern "C"
