// pd_noalloc.cu -- pd_gray_scott_static: multi-step Gray-Scott that allocates
// no device memory.
//
// Some hosts of this library may not (or must not) call cudaMalloc themselves
// or have a plugin do it behind their back: a runtime that reserved the whole
// GPU memory pool at start-up and hands out memory only through its own
// allocator (an XLA / JAX process with preallocation on is the usual case, and
// the FFI handler this library replaces runs inside such a process), or a
// stepping loop with a fixed memory budget in which the implicit device-wide
// synchronisation of cudaMalloc / cudaFree would stall every other stream.
// The regular entry points keep a grow-only scratch pool for the ping-pong
// fields of a multi-step call; this one keeps those fields in a fixed array
// that is part of the library image instead.
//
// Cost and limits, so a caller can decide:
//   * the array is 2 x PD_STATIC_GS_MAX_CELLS floats = 8 MiB, and every GPU on
//     which the library is used holds it from the first use until the process
//     exits, whether or not this entry point is ever called again;
//   * a call may cover at most PD_STATIC_GS_MAX_CELLS cells (1024 x 1024, or
//     any other shape with that many cells including halo rows); larger calls
//     are rejected with PD_ERR_INVALID_ARGUMENT, they are not split;
//   * every call on a device shares the one array, which keeps whatever the
//     previous call left in it.  Nothing in it has to start at zero: each
//     step overwrites the rows it will read next before they are read.  Two
//     calls whose kernels overlap on the GPU (different streams, or different
//     host threads without ordering between them) race on it and corrupt each
//     other's fields; order them on one stream or with events.
//   * the first call on each device looks up the device address of the array
//     (cudaGetSymbolAddress), which makes the CUDA runtime load this module on
//     that device.  Make that first call once, up front, with the device
//     current, and before any stream capture is begun on the stream.
#include "../../include/palladium_cuda.h"
#include "pd_kernels.h"

#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>

#include <mutex>

#define PD_STATIC_GS_MAX_CELLS (1 << 20)

// In host code this name is only a handle for the runtime, never a device
// address: the address is fetched per device below and handed to the kernels.
static __device__ __align__(256) float pd_static_gs_scratch[2 * PD_STATIC_GS_MAX_CELLS];

namespace {

const int kMaxDevices = 64;
std::mutex g_setup_mutex;
float* g_scratch_ptr[kMaxDevices] = {nullptr};

int fail(int code, char* err, size_t cap, const char* fmt, ...) {
    if (err && cap) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, cap, fmt, ap);
        va_end(ap);
    }
    return code;
}

// Once per device, with that device current: resolve the array's device address.
int scratch_for_current_device(float** out, char* err, size_t cap) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess)
        return fail(PD_ERR_CUDA, err, cap, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (device < 0 || device >= kMaxDevices)
        return fail(PD_ERR_INVALID_ARGUMENT, err, cap, "device index %d is outside [0, %d)", device, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[device]) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, pd_static_gs_scratch);
        if (e != cudaSuccess || !ptr)
            return fail(PD_ERR_CUDA, err, cap, "cudaGetSymbolAddress(pd_static_gs_scratch) failed: %s",
                        cudaGetErrorString(e));
        g_scratch_ptr[device] = ptr;
    }
    *out = g_scratch_ptr[device];
    return PD_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int pd_gray_scott_static(const pd_gray_scott_params* p, int math_mode, const void* u, const void* v,
                                    void* uo, void* vo, void* cuda_stream, char* err, size_t err_cap) {
    if (!p) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gray_scott: params must not be NULL");
    const PdModeTable* mt = math_mode == PD_MATH_SAFE ? pd_mode_table_safe()
                          : math_mode == PD_MATH_RELAXED ? pd_mode_table_relaxed()
                          : math_mode == PD_MATH_FAST ? pd_mode_table_fast() : nullptr;
    if (!mt) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "palladium_dispatch: math_mode out of range");
    if (p->rows <= 0 || p->cols <= 0 || p->steps < 0 || p->halo < 0)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gray_scott: rows, cols must be positive; steps, halo non-negative");
    if (p->halo > 0 && p->steps > p->halo)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                    "gray_scott: a slab with %lld halo rows can advance at most %lld steps per call",
                    (long long)p->halo, (long long)p->halo);
    const int64_t rows_alloc = p->rows + 2 * p->halo;
    // the divisions keep the comparison free of overflow for absurd shapes
    if (rows_alloc > PD_STATIC_GS_MAX_CELLS || p->cols > PD_STATIC_GS_MAX_CELLS / rows_alloc)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                    "gray_scott (static scratch): %lld x %lld cells exceed the fixed maximum of %d cells per call; "
                    "use pd_launch, which takes a workspace or allocates one",
                    (long long)rows_alloc, (long long)p->cols, PD_STATIC_GS_MAX_CELLS);
    if (!u || !v || !uo || !vo) return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap, "gray_scott: NULL buffer");
    // Grids narrower than 128 columns (or not a multiple of 4) run the one-thread-per-cell kernel, whose
    // rows are spread over the second launch dimension, 8 per block, at most 65535 blocks.
    if (!((p->cols % 4 == 0) && p->cols >= 128) && (rows_alloc + 7) / 8 > 65535)
        return fail(PD_ERR_INVALID_ARGUMENT, err, err_cap,
                    "gray_scott: %lld rows of %lld columns cannot be launched (grids narrower than 128 columns, or "
                    "with a column count that is not a multiple of 4, take at most 524280 rows)",
                    (long long)rows_alloc, (long long)p->cols);
    const size_t cells = (size_t)rows_alloc * (size_t)p->cols;
    const size_t field_bytes = cells * sizeof(float);
    cudaStream_t st = (cudaStream_t)cuda_stream;

    float* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch, err, err_cap);
    if (rc) return rc;

    if (p->steps == 0) {
        cudaError_t e = cudaMemcpyAsync(uo, u, field_bytes, cudaMemcpyDeviceToDevice, st);
        if (e == cudaSuccess) e = cudaMemcpyAsync(vo, v, field_bytes, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) return fail(PD_ERR_CUDA, err, err_cap, "cudaMemcpyAsync failed: %s", cudaGetErrorString(e));
        return PD_OK;
    }

    PdGsArgs a = {};
    a.rows_alloc = (int)rows_alloc;
    a.cols = (int)p->cols;
    a.periodic_rows = p->halo == 0 ? 1 : 0;
    pd_gs_set_constants(a, p->du, p->dv, p->f, p->k, p->dt);
    const bool vec = (p->cols % 4 == 0) && p->cols >= 128 && aligned16(u) && aligned16(v) && aligned16(uo) && aligned16(vo);
    const int variant = vec ? 1 : 0;

    float* pong_u = scratch;          // 256-byte aligned; the second field starts
    float* pong_v = scratch + cells;  // cells * 4 bytes later (16-byte aligned when cols % 4 == 0)
    const float* src_u = (const float*)u;
    const float* src_v = (const float*)v;
    bool to_out = (p->steps % 2) == 1;  // the last step has to land in the caller's output
    for (int64_t s = 1; s <= p->steps; ++s) {
        a.u = src_u; a.v = src_v;
        a.uo = to_out ? (float*)uo : pong_u;
        a.vo = to_out ? (float*)vo : pong_v;
        if (p->halo == 0) { a.row_lo = 0; a.row_hi = (int)rows_alloc; }
        else { a.row_lo = (int)s; a.row_hi = (int)rows_alloc - (int)s; }
        cudaError_t e = mt->gray_scott(a, variant, st);
        if (e != cudaSuccess) return fail(PD_ERR_CUDA, err, err_cap, "gray_scott launch failed: %s", cudaGetErrorString(e));
        src_u = a.uo; src_v = a.vo;
        to_out = !to_out;
    }
    return PD_OK;
}
