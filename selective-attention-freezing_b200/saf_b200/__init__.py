"""saf_b200: B200 (sm_100a) implementation of SAF's mixed-attention hot path.

`saf_b200.ops` holds the torch-facing operators (reference signatures), `saf_b200.attention`
the attention-module hook, `kernel` (sibling package) the drop-in import surface;
`saf_b200.trainable_patterns` the parameter gradients of learnable decomposed patterns and
`saf_b200.capture` the freeze controller's attention statistics without the attention capture.
"""
from . import _cabi  # noqa: F401  (raises if the CUDA library is not built)
from .ops import (fused_mixed_attn, frozen_pv, linear_rows, linear_rows2, linear_permuted_cols,  # noqa: F401
                  qkv_projection, decomposed_logz, decomposed_logz_fft, decomp_logits, make_rho_band, fused_attn_usable,
                  frozen_pv_usable, launch_count, BAND_ROWS)
