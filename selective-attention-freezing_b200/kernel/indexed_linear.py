"""`kernel.indexed_linear` import path of the reference (kernel/indexed_linear.py), served by libsaf_b200."""
from saf_b200.ops import linear_rows, linear_rows2, linear_permuted_cols  # noqa: F401
