// Backward of the mixed attention for callers that must not allocate.
//
// Some hosts of this library cannot hand it fresh device memory at call time: a
// serving runtime that carved its whole arena up front and has no spare block for a
// per-call (B, H, T) buffer, a plugin interface that only passes the tensors of
// the operator itself, or code running where a device allocation is forbidden
// because cudaMalloc may synchronise the device and stall every other stream.
// For them the one piece of scratch the backward needs -- delta = rowsum(O * dO),
// one fp32 per (batch, head, row) -- lives in a fixed array inside the library.
//
// The array costs SAF_STATIC_DELTA_FLOATS * 4 bytes (4 MiB) on every GPU that loads
// the library, until the process exits.  All calls on a device share it: two calls
// that overlap on the GPU (different streams) race on it; serialise them.  Nothing
// in it has to start at zero -- every row that is read is written first by the same
// call -- so no clearing pass is needed and the previous call's contents are harmless.
// The array's device address is remembered per device ordinal; a process that calls
// cudaDeviceReset() must not use this entry point on that device afterwards (the
// remembered address belongs to the destroyed context).
#include <atomic>

#include "saf_internal.h"

namespace saf {
namespace {

static __device__ __align__(256) float g_static_delta[SAF_STATIC_DELTA_FLOATS];

constexpr int kMaxDevices = SAF_MAX_DEVICES;
std::atomic<float*> g_delta_addr[kMaxDevices];   // zero-initialised; racing first calls store the same value

// Device address of the scratch array on the current device.  In host code the name
// g_static_delta is only a handle for the runtime, not an address a kernel could use:
// the address is looked up once per device, with that device current.
int static_delta_ptr(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(SAF_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(SAF_ERR_LIMIT, "device ordinal %d beyond %d", dev, kMaxDevices);
  float* addr = g_delta_addr[dev].load(std::memory_order_relaxed);
  if (!addr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_delta);
    if (e != cudaSuccess) return fail(SAF_ERR_CUDA, "cudaGetSymbolAddress(static delta scratch): %s", cudaGetErrorString(e));
    addr = reinterpret_cast<float*>(p);
    g_delta_addr[dev].store(addr, std::memory_order_relaxed);
  }
  *out = addr;
  return SAF_OK;
}

}  // namespace
}  // namespace saf

using namespace saf;

extern "C" int saf_mixed_attn_bwd_static(const SafMixedAttnBwdArgs* args, void* stream) {
  if (!args) return fail(SAF_ERR_INVALID, "null argument struct");
  if (args->struct_size != (int32_t)sizeof(SafMixedAttnBwdArgs))
    return fail(SAF_ERR_INVALID, "SafMixedAttnBwdArgs size mismatch: caller %d, library %d", args->struct_size,
                (int)sizeof(SafMixedAttnBwdArgs));
  const SafMixedAttnArgs& a = args->fwd;
  int rc = validate_mixed_args(&a);       // a malformed struct is reported as such, not as a size limit
  if (rc) return rc;
  // delta is read and written for live heads only: a call that cannot contain one has no size limit
  const bool may_be_live = (mixed_possible_states(a) & (1u << SAF_LIVE)) != 0;
  const int64_t need = (int64_t)a.B * a.H * a.T;
  if (may_be_live && need > (int64_t)SAF_STATIC_DELTA_FLOATS)
    return fail(SAF_ERR_LIMIT,
                "B*H*T = %lld rows exceed the static scratch of %d rows; use saf_mixed_attn_bwd with caller-provided delta",
                (long long)need, (int)SAF_STATIC_DELTA_FLOATS);
  float* scratch = nullptr;
  rc = static_delta_ptr(&scratch);
  if (rc) return rc;
  SafMixedAttnBwdArgs g = *args;
  g.delta.ptr = scratch;
  g.delta.stride[0] = (int64_t)a.H * a.T;
  g.delta.stride[1] = a.T;
  g.delta.stride[2] = 1;
  g.delta.stride[3] = 0;
  return saf_mixed_attn_bwd(&g, stream);
}
