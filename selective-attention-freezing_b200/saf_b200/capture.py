"""Controller measurement path without the (B, H, T, T) capture.

The reference's FreezeController._measure (nanogpt/dynamic_freeze.py:629-745) turns capture on, lets the eager
attention retain softmax(QK^T) for every layer, and reduces it to three statistics per head: the mean attention
matrix, the centred sum of squares summed over cells (`_centered_batch_reduced_moments` / `_merge_reduced_moments`,
:96-143) and sum p log p (`_negative_entropy_sum`, :146-173).  `AttentionMoments` keeps exactly those for the live
heads of one layer and updates them from q, k alone: one flash forward for the row log-sum-exp, then
`saf_attention_moments`, which recomputes each probability tile on the tensor cores and merges it into the running
mean in place.  Frozen heads need no measurement: their "attention" is the stored pattern (zero variance).

Priors that sample logits also want per-cell statistics of the raw scores (`_last_logits`, nanogpt/model.py:828-831;
merged at nanogpt/dynamic_freeze.py:721-737): `LogitMoments` keeps their running mean and, on request, centred squares,
from the same kernel run on q k^T * sm_scale over the whole square.
"""
import ctypes as C
import math

import torch

from . import ops
from ._cabi import STATS_LOGITS, SafAttnStatsArgs, SafMixedAttnArgs, lib


def _row_lse(q, k, sm_scale):
    """(B, U, T) fp32 log2-domain log-sum-exp of the causal scores, from the mixed-attention forward run with every
    head live (k stands in for v; the output is scratch)."""
    B, U, T, HD = q.shape
    out = torch.empty((B, U, T, HD), device=q.device, dtype=q.dtype)
    lse = torch.empty((B, U, T), device=q.device, dtype=torch.float32)
    live = torch.zeros(U, dtype=torch.int32, device=q.device)
    a, keep = SafMixedAttnArgs(), []
    ops._fill_mixed(a, q, k, k, out, lse, None, None, None, None, live, None, None, None, sm_scale, None, None, keep)
    ops._call(q, lib.saf_mixed_attn_fwd, C.byref(a))
    return lse


@torch.no_grad()
def attention_moments(q, k, mean, count_prev, head_m2, neg_entropy, sm_scale=None):
    """Merge one batch into running statistics, in place.

    q, k (B, U, T, hd) bf16 as the attention sees them (rotated); mean (U, T, T) fp32; head_m2, neg_entropy (U,)
    fp64.  After the call they hold what the reference's Chan merge of
    `_centered_batch_reduced_moments(softmax(causal(q k^T * sm_scale)))` into (count_prev, mean, head_m2) holds,
    and neg_entropy has grown by `_negative_entropy_sum` of the same tensor.  Returns the new count."""
    ops._require_cuda(q, "q")
    B, U, T, HD = q.shape
    assert k.shape == q.shape, "q and k must have the same (B, U, T, hd) shape"
    assert mean.shape == (U, T, T) and mean.dtype == torch.float32 and mean.is_contiguous()
    assert head_m2.dtype == neg_entropy.dtype == torch.float64 and head_m2.numel() == neg_entropy.numel() == U
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(HD)
    lse = _row_lse(q, k, sm_scale)
    a = SafAttnStatsArgs()
    a.struct_size = C.sizeof(SafAttnStatsArgs)
    a.dtype = ops._dt(q)
    a.B, a.U, a.T, a.HD = B, U, T, HD
    a.sm_scale = float(sm_scale)
    a.q, a.k, a.lse = ops._st(q), ops._st(k), ops._st(lse)
    a.mean = mean.data_ptr()
    a.count_prev = int(count_prev)
    a.head_m2, a.neg_entropy = head_m2.data_ptr(), neg_entropy.data_ptr()
    a.status = ops._status_ptr(q.device)
    ops._call(q, lib.saf_attention_moments, C.byref(a))
    return int(count_prev) + B


class AttentionMoments:
    """Running attention statistics of the live heads of one layer (what `_measure` keeps per layer)."""

    def __init__(self, n_heads, T, device):
        self.count = 0
        self.T = T
        self.mean = torch.empty((n_heads, T, T), device=device, dtype=torch.float32)   # written by the first update
        self.head_m2 = torch.zeros(n_heads, device=device, dtype=torch.float64)
        self.neg_entropy = torch.zeros(n_heads, device=device, dtype=torch.float64)

    def update(self, q, k, sm_scale=None):
        self.count = attention_moments(q, k, self.mean, self.count, self.head_m2, self.neg_entropy, sm_scale)
        return self

    def per_head_variance(self):
        """Variance averaged over cells, `att_m2 / max(n-1, 1) / cells` (nanogpt/dynamic_freeze.py:764-768)."""
        cells = self.T * self.T
        return (self.head_m2 / max(self.count - 1, 1) / cells).clamp_min(0).float()

    def mean_forward_kl(self, chunk_rows=1024):
        """E_s mean_i KL(P_s[i] || Pbar[i]) per head from the entropy identity
        (`_mean_forward_kl_from_entropy`, nanogpt/dynamic_freeze.py:176-193)."""
        T = self.T
        sample_term = self.neg_entropy / (self.count * T)
        mean_term = torch.zeros_like(sample_term)
        for r0 in range(0, T, chunk_rows):
            pr = self.mean[:, r0:r0 + chunk_rows]
            pr = pr / pr.sum(-1, keepdim=True).clamp_min(1e-12)
            mean_term += torch.xlogy(pr, pr).sum(dim=(1, 2)).double()
        return (sample_term - mean_term / T).clamp_min(0).float()


@torch.no_grad()
def logit_moments(q, k, mean, count_prev, cell_m2=None, sm_scale=None):
    """Merge one batch of raw scores lg = q k^T * sm_scale (B, U, T, T, nothing masked) into running per-cell
    statistics, in place: mean (U, T, T) fp32 becomes the Chan merge of `lg.mean(0)`; cell_m2 (U, T, T) fp32, when
    given, that of `_centered_batch_moments(lg)` under `_merge_moments` (nanogpt/dynamic_freeze.py:62-93).
    Returns the new count."""
    ops._require_cuda(q, "q")
    B, U, T, HD = q.shape
    assert k.shape == q.shape, "q and k must have the same (B, U, T, hd) shape"
    assert mean.shape == (U, T, T) and mean.dtype == torch.float32 and mean.is_contiguous()
    if cell_m2 is not None:
        assert cell_m2.shape == (U, T, T) and cell_m2.dtype == torch.float32 and cell_m2.is_contiguous()
    a = SafAttnStatsArgs()
    a.struct_size = C.sizeof(SafAttnStatsArgs)
    a.dtype = ops._dt(q)
    a.B, a.U, a.T, a.HD = B, U, T, HD
    a.sm_scale = float(sm_scale if sm_scale is not None else 1.0 / math.sqrt(HD))
    a.q, a.k = ops._st(q), ops._st(k)
    a.mean = mean.data_ptr()
    a.count_prev = int(count_prev)
    a.status = ops._status_ptr(q.device)
    a.quantity = STATS_LOGITS
    a.cell_m2 = cell_m2.data_ptr() if cell_m2 is not None else None
    ops._call(q, lib.saf_attention_moments, C.byref(a))
    return int(count_prev) + B


class LogitMoments:
    """Running per-cell statistics of the raw scores of one layer's heads (`logit_mean` / `logit_m2` of `_measure`)."""

    def __init__(self, n_heads, T, device, with_var=False):
        self.count = 0
        self.T = T
        self.mean = torch.empty((n_heads, T, T), device=device, dtype=torch.float32)   # written by the first update
        self.m2 = torch.empty((n_heads, T, T), device=device, dtype=torch.float32) if with_var else None

    def update(self, q, k, sm_scale=None):
        self.count = logit_moments(q, k, self.mean, self.count, self.m2, sm_scale)
        return self

    def std(self):
        """`(logit_m2 / max(n - 1, 1)).clamp_min(0).sqrt()` (nanogpt/dynamic_freeze.py:787-790)."""
        assert self.m2 is not None, "built without with_var"
        return (self.m2 / max(self.count - 1, 1)).clamp_min(0).sqrt()
