// Internal declarations shared by the translation units of libsaf_b200.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "../../include/saf_b200.h"

namespace saf {

// error text of the calling thread; returns `code` so call sites can `return fail(...)`
int fail(int code, const char* fmt, ...);
void count_launch(int n = 1);
int check_launch(const char* what);   // cudaGetLastError -> SAF_ERR_CUDA

// ---- per-device bookkeeping ---------------------------------------------------
// One process may drive several GPUs: anything that CUDA keeps per device (a kernel's dynamic shared memory
// limit, the SM count) is remembered per device ordinal, never per process.
constexpr int SAF_MAX_DEVICES = 64;

// "has this been done on device d yet?" -- first(d) returns true exactly once per device ordinal (ordinals
// outside [0, SAF_MAX_DEVICES) always return true: the caller then simply repeats its idempotent set-up).
struct PerDeviceOnce {
  std::atomic<bool> done[SAF_MAX_DEVICES];
  bool first(int dev) {
    if (dev < 0 || dev >= SAF_MAX_DEVICES) return true;
    return !done[dev].exchange(true, std::memory_order_acq_rel);
  }
  void forget(int dev) {
    if (dev >= 0 && dev < SAF_MAX_DEVICES) done[dev].store(false, std::memory_order_release);
  }
};

int current_device();        // cudaGetDevice; -1 when it fails
int device_sm_count();       // SM count of the current device, cached per device (148 when the query fails)

// Raises `kernel`'s dynamic shared memory limit to `bytes` on the current device, once per device.
template <typename K>
int ensure_dyn_smem(K kernel, int bytes, PerDeviceOnce& once) {
  const int dev = current_device();
  if (!once.first(dev)) return SAF_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    once.forget(dev);
    return fail(SAF_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  return SAF_OK;
}

// ---- element conversion -----------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

// runtime-typed scalar load (pattern / decomposed buffers may differ from the activation type)
__device__ __forceinline__ float load_rt(const void* base, int64_t idx, int dtype) {
  if (dtype == SAF_F32) return reinterpret_cast<const float*>(base)[idx];
  if (dtype == SAF_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

inline int dtype_size(int dt) { return dt == SAF_F32 ? 4 : 2; }

// argument checks of the mixed-attention entry points, and the head states a call can contain (bit s = state s)
int validate_mixed_args(const SafMixedAttnArgs* a);
uint32_t mixed_possible_states(const SafMixedAttnArgs& a);

// ---- kernels' host launchers (each returns SAF_OK or an error code) ----------
// states_mask: bit s set -> heads in state s are processed by this launch
int launch_generic_fwd(const SafMixedAttnArgs& a, uint32_t states_mask, cudaStream_t st);
int launch_generic_bwd(const SafMixedAttnBwdArgs& a, uint32_t states_mask, cudaStream_t st);
int launch_scan_fwd(const SafMixedAttnArgs& a, cudaStream_t st);                       // state 3 heads
int launch_scan_bwd(const SafMixedAttnBwdArgs& a, cudaStream_t st);                    // state 3 heads: dv
// state 3 heads, forward, on the tensor core (bf16, head_dim a multiple of 64, long T); SAF_ERR_UNSUPPORTED otherwise
int launch_scan_fwd_mma(const SafMixedAttnArgs& a, cudaStream_t st);
// tcgen05 fast path; returns SAF_ERR_UNSUPPORTED when the call does not qualify
// `want`: states still to be served; the launch covers the subset it can and reports it
int launch_flash_fwd_sm100(const SafMixedAttnArgs& a, uint32_t want, uint32_t* handled_states, cudaStream_t st);
// dense-stored frozen heads as a TMA-staged lower-triangular GEMM (bf16 patterns)
int launch_dense_pv_sm100(const SafMixedAttnArgs& a, uint32_t* handled_states, cudaStream_t st);
int launch_flash_bwd_sm100(const SafMixedAttnBwdArgs& a, uint32_t* handled_states, cudaStream_t st);
int launch_gemm_sm100(const SafIndexedLinearArgs& a, cudaStream_t st);
int launch_gemm_generic(const SafIndexedLinearArgs& a, cudaStream_t st);
int launch_gemm_bwd_dx(const SafIndexedLinearArgs& a, const void* dout, int64_t lddo, void* dx, int64_t lddx,
                       const void* bias, cudaStream_t st);
int launch_gemm_bwd_dw(const SafIndexedLinearArgs& a, const void* dout, int64_t lddo, cudaStream_t st);
// tcgen05 versions of the two backward products; SAF_ERR_UNSUPPORTED when the call does not qualify
int launch_gemm_bwd_dx_sm100(const SafIndexedLinearArgs& a, const void* dout, int64_t lddo, void* dx, int64_t lddx,
                             const void* bias, cudaStream_t st);
int launch_gemm_bwd_dw_sm100(const SafIndexedLinearArgs& a, const void* dout, int64_t lddo, cudaStream_t st);
int launch_rope_slabs(void* x, int64_t ld, int M, int n_slabs, int slab, int T, const int32_t* slab_rope,
                      const float* cosT, const float* sinT, int dtype, int inverse, cudaStream_t st);
int launch_layernorm(const void* x, int64_t ldx, const void* w, const void* b, void* out, int64_t ldo, int M, int C,
                     float eps, int dtype, int rms, cudaStream_t st);
int launch_logz(const float* alpha, const float* rho, float* z, int H, int S, int rows, cudaStream_t st);   // rows >= `rows` get 0
int launch_pattern_grad(const SafPatternGradArgs& a, cudaStream_t st);
int launch_attn_stats_sm100(const SafAttnStatsArgs& a, cudaStream_t st);

// TMA descriptor encode through the driver entry point (no link-time libcuda dependency)
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                      CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                      CUtensorMapFloatOOBfill);
TensorMapEncodeFn tensor_map_encoder();
// rank-`rank` bf16 map, 128B swizzle; dims/strides innermost first, strides in BYTES for dims 1..rank-1
int make_tensor_map_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box, bool l2_256);

// a (B, Hn, T, HD) bf16 tensor that TMA can tile: 16-byte aligned base, unit last stride, other strides multiples of 8
bool tma_rows_ok(const SafTensor& t);
// its map with boxes of 128 rows x 64 columns (one 128-byte-swizzled atom), coordinates (column, row, head, batch)
int make_row_tile_map_bf16(CUtensorMap* m, const SafTensor& t, int B, int Hn, int T, int HD);

}  // namespace saf
