// Stand-alone launch of the dense-pattern GEMM (csrc/dense_pv_body.cuh) for calls the mixed launch does not
// take (frozen heads only with in-kernel RoPE requested for the live ones, unsupported live-head layouts, ...).
#include "dense_pv_body.cuh"

namespace saf {
namespace {

template <int HD>
__global__ void __launch_bounds__(DP_THREADS, 1)
dense_pv_kernel(const __grid_constant__ CUtensorMap mapP, const __grid_constant__ CUtensorMap mapV,
                const __grid_constant__ CUtensorMap mapO, const __grid_constant__ DpParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  dense_pv_cta<HD>(mapP, mapV, mapO, p, (int)blockIdx.x, smem);
}

template <int HD>
int dp_launch(const SafMixedAttnArgs& a, cudaStream_t st) {
  CUtensorMap mp_, mv, mo;
  DpParams p;
  int rc = dense_pv_prepare(a, true, false, &mp_, &mv, &mo, &p);
  if (rc) return rc;
  static PerDeviceOnce smem_once;
  if ((rc = ensure_dyn_smem(dense_pv_kernel<HD>, DpCfg<HD>::SMEM_BYTES, smem_once))) return rc;
  dense_pv_kernel<HD><<<dense_pv_slots(p), DP_THREADS, DpCfg<HD>::SMEM_BYTES, st>>>(mp_, mv, mo, p);
  count_launch();
  return check_launch("dense_pv_kernel");
}

}  // namespace

int launch_dense_pv_sm100(const SafMixedAttnArgs& a, uint32_t* handled, cudaStream_t st) {
  *handled = 0;
  if (!dense_pv_eligible(a) || !saf_device_supported()) return SAF_ERR_UNSUPPORTED;
  if (a.force_state >= 0 && a.force_state != SAF_DENSE) return SAF_ERR_UNSUPPORTED;
  if (a.frozen_host) {
    bool any = false;
    for (int h = 0; h < a.H; ++h) any |= a.frozen_host[h] == SAF_DENSE;
    if (!any) return SAF_ERR_UNSUPPORTED;
  }
  const int rc = (a.HD == 64) ? dp_launch<64>(a, st) : dp_launch<128>(a, st);
  if (rc == SAF_OK) *handled = 1u << SAF_DENSE;
  return rc;
}

}  // namespace saf
