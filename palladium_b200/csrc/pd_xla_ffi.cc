// pd_xla_ffi.cc -- XLA-FFI handler symbol `palladium_cuda_dispatch`.
//
// The counterpart of XLA_FFI_DEFINE_HANDLER_SYMBOL(palladium_dispatch, ...) in
// the reference (native/ffi/palladium_ffi.cpp:197-209).  The attribute list is
// the reference's with `msl_source` / `function_name` replaced by `family` and
// the family's parameter block (`params`, the bytes of the pd_*_params struct);
// grid, threadgroup and math_mode keep their names and meaning, and the buffers
// still arrive as RemainingArgs / RemainingRets, so one handler serves every
// family and any input / output count.
//
// Registered on the "cpu" platform, like the reference's handler
// (src/palladium/ffi.py:78): XLA hands it host buffers and the call blocks until
// the outputs are in place, which is exactly pd_dispatch_host.
//
// This file needs the XLA FFI headers (`jax.ffi.include_dir()`); it is not part
// of the default build and is compiled by palladium_b200/xla_ffi.py only where
// JAX is installed.
#include <cstdint>
#include <cstring>
#include <string>
#include <string_view>
#include <vector>

#include "../../include/palladium_cuda.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

static ffi::Error Dispatch(int64_t family, const void* params, size_t params_bytes, int64_t grid_x, int64_t grid_y,
                           int64_t grid_z, int64_t threadgroup_x, int64_t threadgroup_y, int64_t threadgroup_z,
                           int64_t math_mode, ffi::RemainingArgs args, ffi::RemainingRets rets) {
  std::vector<const void*> in;
  std::vector<size_t> in_bytes;
  std::vector<void*> out;
  std::vector<size_t> out_bytes;
  in.reserve(args.size());
  out.reserve(rets.size());
  for (size_t i = 0; i < args.size(); ++i) {
    auto buf = args.get<ffi::AnyBuffer>(i);
    if (!buf.has_value()) return buf.error();
    in.push_back(buf->untyped_data());
    in_bytes.push_back(buf->size_bytes());
  }
  for (size_t i = 0; i < rets.size(); ++i) {
    auto buf = rets.get<ffi::AnyBuffer>(i);
    if (!buf.has_value()) return buf.error();
    out.push_back((*buf)->untyped_data());
    out_bytes.push_back((*buf)->size_bytes());
  }
  const int64_t grid[3] = {grid_x, grid_y, grid_z};
  const int64_t block[3] = {threadgroup_x, threadgroup_y, threadgroup_z};
  char err[1024] = {0};
  const int rc = pd_dispatch_host(static_cast<int>(family), params, params_bytes, static_cast<int>(math_mode),
                                  grid, block, static_cast<int>(in.size()), in.data(), in_bytes.data(),
                                  static_cast<int>(out.size()), out.data(), out_bytes.data(), err, sizeof err);
  if (rc == PD_ERR_INVALID_ARGUMENT) return ffi::Error::InvalidArgument(err);
  if (rc != PD_OK) return ffi::Error::Internal(err);
  return ffi::Error::Success();
}

static ffi::Error PalladiumCudaDispatch(int64_t family, ffi::Span<const uint8_t> params, int64_t grid_x,
                                        int64_t grid_y, int64_t grid_z, int64_t threadgroup_x,
                                        int64_t threadgroup_y, int64_t threadgroup_z, int64_t math_mode,
                                        ffi::RemainingArgs args, ffi::RemainingRets rets) {
  // The run-time compiled families hold host pointers (source text) in their parameter
  // blocks; attribute bytes must never be read as such pointers.
  if (family == PD_FAMILY_SOURCE || family == PD_FAMILY_CUSTOM_ODE)
    return ffi::Error::InvalidArgument(
        "palladium_cuda_dispatch: this family carries source text; call palladium_cuda_dispatch_source");
  // An attribute span has no alignment guarantee, and the parameter blocks hold int64 / double fields.
  alignas(8) unsigned char aligned_params[256];
  if (params.size() > sizeof aligned_params)
    return ffi::Error::InvalidArgument("palladium_cuda_dispatch: params block is larger than 256 bytes");
  std::memcpy(aligned_params, params.begin(), params.size());
  return Dispatch(family, aligned_params, params.size(), grid_x, grid_y, grid_z, threadgroup_x, threadgroup_y,
                  threadgroup_z, math_mode, args, rets);
}

// The run-time compiled families carry source text, which cannot travel as a
// pointer inside `params`: this handler takes it as string attributes -- for a
// caller-written kernel exactly the reference's `msl_source` / `function_name`
// pair under CUDA names -- and points the parameter block at them.
static ffi::Error PalladiumCudaDispatchSource(std::string_view cuda_source, std::string_view function_name,
                                              int64_t family, ffi::Span<const uint8_t> params, int64_t grid_x,
                                              int64_t grid_y, int64_t grid_z, int64_t threadgroup_x,
                                              int64_t threadgroup_y, int64_t threadgroup_z, int64_t math_mode,
                                              ffi::RemainingArgs args, ffi::RemainingRets rets) {
  const std::string source(cuda_source), name(function_name);  // NUL-terminated copies
  if (family == PD_FAMILY_SOURCE) {
    pd_source_kernel_params p;
    p.cuda_source = source.c_str();
    p.function_name = name.c_str();
    return Dispatch(family, &p, sizeof p, grid_x, grid_y, grid_z, threadgroup_x, threadgroup_y, threadgroup_z,
                    math_mode, args, rets);
  }
  if (family == PD_FAMILY_CUSTOM_ODE) {
    if (params.size() != sizeof(pd_custom_ode_params))
      return ffi::Error::InvalidArgument("palladium_cuda_dispatch_source: params has the wrong size for custom_ode");
    pd_custom_ode_params p;
    std::memcpy(&p, params.begin(), sizeof p);
    p.rhs_source = source.c_str();
    return Dispatch(family, &p, sizeof p, grid_x, grid_y, grid_z, threadgroup_x, threadgroup_y, threadgroup_z,
                    math_mode, args, rets);
  }
  return ffi::Error::InvalidArgument("palladium_cuda_dispatch_source: family takes no source text");
}

XLA_FFI_DEFINE_HANDLER_SYMBOL(palladium_cuda_dispatch_source, PalladiumCudaDispatchSource,
                              ffi::Ffi::Bind()
                                  .Attr<std::string_view>("cuda_source")
                                  .Attr<std::string_view>("function_name")
                                  .Attr<int64_t>("family")
                                  .Attr<ffi::Span<const uint8_t>>("params")
                                  .Attr<int64_t>("grid_x")
                                  .Attr<int64_t>("grid_y")
                                  .Attr<int64_t>("grid_z")
                                  .Attr<int64_t>("threadgroup_x")
                                  .Attr<int64_t>("threadgroup_y")
                                  .Attr<int64_t>("threadgroup_z")
                                  .Attr<int64_t>("math_mode")
                                  .RemainingArgs()
                                  .RemainingRets());

XLA_FFI_DEFINE_HANDLER_SYMBOL(palladium_cuda_dispatch, PalladiumCudaDispatch,
                              ffi::Ffi::Bind()
                                  .Attr<int64_t>("family")
                                  .Attr<ffi::Span<const uint8_t>>("params")
                                  .Attr<int64_t>("grid_x")
                                  .Attr<int64_t>("grid_y")
                                  .Attr<int64_t>("grid_z")
                                  .Attr<int64_t>("threadgroup_x")
                                  .Attr<int64_t>("threadgroup_y")
                                  .Attr<int64_t>("threadgroup_z")
                                  .Attr<int64_t>("math_mode")
                                  .RemainingArgs()
                                  .RemainingRets());
