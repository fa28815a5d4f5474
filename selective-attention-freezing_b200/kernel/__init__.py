"""Drop-in replacement for the reference's `kernel` package (kernel/__init__.py:14-22).

Same twelve names, same signatures; every operator runs hand-written sm_100a CUDA
through libsaf_b200.so.  `HAVE_TRITON` stays exported (callers gate on it,
nanogpt/bench_downstream_finetune.py:126) and is True when the CUDA library is
loaded, although no Triton is involved.
"""
from .frozen_attn import frozen_pv, frozen_pv_usable, HAVE_TRITON
from .indexed_linear import linear_rows, linear_rows2, linear_permuted_cols
from .fused_attn import (fused_mixed_attn, fused_attn_usable, decomposed_logz,
                         decomp_logits, make_rho_band, BAND_ROWS)

__all__ = ["frozen_pv", "frozen_pv_usable", "HAVE_TRITON",
           "linear_rows", "linear_rows2", "linear_permuted_cols",
           "fused_mixed_attn", "fused_attn_usable", "decomposed_logz",
           "decomp_logits", "make_rho_band", "BAND_ROWS"]
