// placeholder until the tcgen05 kernel lands
#include "saf_internal.h"
namespace saf {
int launch_flash_fwd_sm100(const SafMixedAttnArgs&, uint32_t* handled, cudaStream_t) {
  *handled = 0;
  return SAF_ERR_UNSUPPORTED;
}
}  // namespace saf
