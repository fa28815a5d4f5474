"""`kernel.fused_attn` import path of the reference (kernel/fused_attn.py), served by libsaf_b200."""
from saf_b200.ops import (fused_mixed_attn, fused_attn_usable, decomposed_logz, decomp_logits,  # noqa: F401
                          make_rho_band, BAND_ROWS)

HAVE_TRITON = True   # "the fused GPU path is available"; nothing here uses Triton
