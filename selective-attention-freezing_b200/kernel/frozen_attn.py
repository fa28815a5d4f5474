"""`kernel.frozen_attn` import path of the reference (kernel/frozen_attn.py), served by libsaf_b200."""
from saf_b200.ops import frozen_pv, frozen_pv_usable  # noqa: F401

HAVE_TRITON = True   # "the fused GPU path is available"; nothing here uses Triton
