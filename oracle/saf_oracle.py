"""CPU oracle for the SAF mixed-attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain torch CPU arithmetic (fp32 or fp64), what the
reference computes on the path the CUDA library accelerates.  It is the checker
for the parity tests, for ``__graft_entry__.smoke()`` and for the CPU-baseline
leg of ``bench.py``; the product (the ``kernel`` package and the C-ABI library)
never imports it and has no CPU fallback.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the reference
itself (its eager ``CausalSelfAttention`` capture path, its cheap split path,
``kernel/indexed_linear.py`` and the host helpers of ``kernel/fused_attn.py``,
all of which run on CPU) and stores their outputs on seeded inputs under
``tests/golden/``; ``tests/test_oracle_golden.py`` checks every function below
against those vectors.  The GQA ``kvidx`` variant has no test in the reference;
``tests/golden/make_golden_gqa.py`` runs the reference's own Qwen3 hybrid
attention module (its split torch path, qwen/nanogpt/hybrid_prior_attention.py:
586-640) on a random-init HF ``Qwen3Attention`` and stores inputs, intermediate
q/k/v and outputs in ``tests/golden/gqa_vectors.npz``, which pin ``mixed_attn(kvidx=)``
and ``gqa_attention_layer``.

Each function cites the reference file:line it follows (paths are relative to
the reference project root).
"""
import math

import torch

BAND_ROWS = 64          # kernel/fused_attn.py:58


# ---------------------------------------------------------------------------
# error metrics used by every parity test
# ---------------------------------------------------------------------------
def max_abs(a, b):
    return (a.double() - b.double()).abs().max().item() if a.numel() else 0.0


def rel_l2(a, b):
    """||a-b|| / ||b||  (supplement/test_controls.py:40-44 uses the same pair)."""
    if a.numel() == 0:
        return 0.0
    d = (a.double() - b.double()).norm().item()
    n = b.double().norm().item()
    return d / max(n, 1e-30)


# ---------------------------------------------------------------------------
# RoPE                                                    nanogpt/model.py:57-99
# ---------------------------------------------------------------------------
def rope_cache(hd, T, base=10000.0, dtype=torch.float32):
    """cos/sin tables (T, hd) = cat(freqs, freqs); nanogpt/model.py:73-83."""
    inv_freq = 1.0 / (base ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    pos = torch.arange(T, dtype=torch.float32)
    freqs = torch.outer(pos, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x):
    """nanogpt/model.py:57-60."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def apply_rope(x, cos, sin):
    """x: (..., T, hd); cos/sin: (T, hd).  nanogpt/model.py:63-68."""
    return x * cos + rotate_half(x) * sin


# ---------------------------------------------------------------------------
# pattern builders
# ---------------------------------------------------------------------------
def sink_decay_pattern(alpha, rho, T, dtype=torch.float64):
    """P[h,i,j] = a_h [j=0] + (1-a_h) rho_h^(i-j) / Z_i  for j<=i, else 0.

    The structured pattern of the headline benchmark configuration (sink on
    column 0 plus a geometric decay over distance); rows sum to one.  The
    reference can only hold it as a dense state-1 buffer installed through
    ``freeze_heads`` (nanogpt/model.py:705-733)."""
    alpha = torch.as_tensor(alpha, dtype=dtype).reshape(-1)
    rho = torch.as_tensor(rho, dtype=dtype).reshape(-1)
    i = torch.arange(T, dtype=dtype)
    dist = i[:, None] - i[None, :]
    causal = dist >= 0
    out = []
    for a, r in zip(alpha.tolist(), rho.tolist()):
        dec = torch.where(causal, torch.tensor(r, dtype=dtype) ** dist.clamp(min=0), torch.zeros((), dtype=dtype))
        dec /= dec.sum(-1, keepdim=True)
        dec *= (1.0 - a)
        dec[:, 0] += a
        out.append(dec)
    return torch.stack(out)


def freeze_normalise(patterns):
    """tril + row renormalisation applied at install time; nanogpt/model.py:716-719."""
    patterns = patterns.tril()
    return patterns / patterns.sum(-1, keepdim=True).clamp_min(1e-12)


def decomp_logits(alpha, rho, rows=None):
    """L[h,i,j] = alpha[h,j] + rho[h,i-j], -inf for j>i.  kernel/fused_attn.py:83-98."""
    H, S = alpha.shape
    r0, r1 = (0, S) if rows is None else rows
    i = torch.arange(r0, r1)
    j = torch.arange(S)
    dist = i[:, None] - j[None, :]
    lg = alpha[:, None, :] + rho[:, dist.clamp(min=0)]
    return lg.masked_fill(dist < 0, float("-inf"))


def decomposed_logz(alpha, rho, chunk=256):
    """z[h,i] = logsumexp_{j<=i}(alpha[h,j] + rho[h,i-j]).  kernel/fused_attn.py:101-116."""
    H, S = alpha.shape
    z = torch.empty_like(alpha)
    for i0 in range(0, S, chunk):
        i1 = min(i0 + chunk, S)
        z[:, i0:i1] = decomp_logits(alpha, rho, rows=(i0, i1)).logsumexp(-1)
    return z


def make_rho_band(rho):
    """band[h,r,u] = rho[h, r-u+(S-64)], -inf outside [0,S).  kernel/fused_attn.py:65-80."""
    H, S = rho.shape
    assert S % BAND_ROWS == 0
    r = torch.arange(BAND_ROWS)[:, None]
    u = torch.arange(S)[None, :]
    src = r - u + (S - BAND_ROWS)
    band = rho[:, src.clamp(0, S - 1)]
    ninf = torch.full((), float("-inf"), dtype=rho.dtype)
    return torch.where((src >= 0) & (src < S), band, ninf).contiguous()


def decomp_pattern(alpha, rho, z, T):
    """exp(alpha[j] + rho[i-j] - z[i]) on the causal triangle; nanogpt/model.py:796-803,
    kernel/test_fused_attn.py:40-50."""
    lg = decomp_logits(alpha[:, :T], rho[:, :T])
    return torch.exp(lg - z[:, :T, None])


# ---------------------------------------------------------------------------
# mixed attention                     nanogpt/model.py:824-844 (eager oracle),
#                                     kernel/test_fused_attn.py:53-63 (ref())
# ---------------------------------------------------------------------------
def sink_decay_rows(a, r, rows, n_cols, dtype=torch.float64, device=None):
    """Rows `rows` (1-D long tensor) of sink_decay_pattern(a, r) for ONE head, columns [0, n_cols): the
    same formula evaluated without the T x T matrix (what freeze_heads stores for that head, row by row,
    nanogpt/model.py:705-733)."""
    i = rows.to(device=device, dtype=dtype)[:, None]
    j = torch.arange(n_cols, dtype=dtype, device=device)[None, :]
    dist = i - j
    rr = torch.tensor(float(r), dtype=dtype, device=device)
    dec = torch.where(dist >= 0, rr ** dist.clamp(min=0), torch.zeros((), dtype=dtype, device=device))
    dec = dec / dec.sum(-1, keepdim=True) * (1.0 - float(a))
    dec[:, 0] += float(a)
    return dec


def mixed_attn(q, k, v, patt, frozen, hidx=None, pidx=None, sm_scale=None,
               alpha=None, rho=None, z=None, kvidx=None, dtype=torch.float32,
               row_chunk=1024, rows=None, sink_decay=None):
    """Eager mixed attention, one (batch, head) and one row chunk at a time.

    q, k: (B, U, T, hd) compact live heads (or (B, HKV, T, hd) k with kvidx);
    v: (B, H, T, hd) (or (B, HKV, T, hd) with kvidx); frozen: (H,) ints with
    0 = live softmax(q k^T * sm_scale) v, 1 = patt[pidx[h] or h, :T, :T] @ v,
    2 = exp(alpha[j] + rho[i-j] - z[i]) @ v, 3 = the dense pattern
    sink_decay_pattern(a[h], r[h]) @ v with sink_decay = (a, r) per head (a state-1
    head whose stored rows are produced on the fly).  Returns (B, H, T, hd) in `dtype`;
    with rows = 1-D long tensor of query positions, only those rows: (B, H, len(rows), hd).
    Runs on the device of v.  Differentiable w.r.t. q, k, v (autograd gives the backward oracle).
    """
    frozen = [int(x) for x in torch.as_tensor(frozen).tolist()]
    H = len(frozen)
    B, T, hd = v.shape[0], v.shape[2], v.shape[3]
    dev = v.device
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(hd)
    hidx = list(range(H)) if hidx is None else [int(x) for x in torch.as_tensor(hidx).tolist()]
    pidx = list(range(H)) if pidx is None else [int(x) for x in torch.as_tensor(pidx).tolist()]
    kv = None if kvidx is None else [int(x) for x in torch.as_tensor(kvidx).tolist()]
    if rows is None:
        chunks = [torch.arange(i0, min(i0 + row_chunk, T), device=dev) for i0 in range(0, T, row_chunk)]
    else:
        rows = torch.as_tensor(rows, dtype=torch.long, device=dev)
        chunks = [rows[i0:i0 + row_chunk] for i0 in range(0, rows.numel(), row_chunk)]
    outs = []
    for b in range(B):
        per_head = []
        for h in range(H):
            vh = v[b, kv[h] if kv is not None else h].to(dtype)
            acc = []
            for ri in chunks:
                i1 = int(ri.max().item()) + 1          # keys past the chunk's last row are masked for every row
                cols = torch.arange(i1, device=dev)
                if frozen[h] == 0:
                    qh = q[b, hidx[h]].index_select(0, ri).to(dtype)
                    kh = k[b, kv[h] if kv is not None else hidx[h], :i1].to(dtype)
                    s = (qh @ kh.t()) * sm_scale
                    p = s.masked_fill(ri[:, None] < cols[None, :], float("-inf")).softmax(-1)
                elif frozen[h] == 1:
                    p = patt[pidx[h]].index_select(0, ri.to(patt.device))[:, :i1].to(device=dev, dtype=dtype)
                elif frozen[h] == 3:
                    p = sink_decay_rows(float(sink_decay[0][h]), float(sink_decay[1][h]), ri, i1,
                                        dtype=torch.float64, device=dev).to(dtype)
                else:
                    dist = ri[:, None] - cols[None, :]
                    lg = alpha[h, :i1].to(device=dev, dtype=dtype)[None, :] + \
                        rho[h].to(device=dev, dtype=dtype)[dist.clamp(min=0)]
                    lg = lg.masked_fill(dist < 0, float("-inf"))
                    p = torch.exp(lg - z[h].to(device=dev, dtype=dtype).index_select(0, ri)[:, None])
                acc.append(p @ vh[:i1])
            per_head.append(torch.cat(acc, 0))
        outs.append(torch.stack(per_head))
    return torch.stack(outs)


def frozen_pv(patt, v, fz_idx, T, dtype=torch.float32):
    """y[b,f] = patt[fz_idx[f], :T, :T] @ v[b,f].  kernel/test_frozen_attn.py:27-28."""
    fz = torch.as_tensor(fz_idx).long()
    return torch.matmul(patt[fz, :T, :T].to(dtype).unsqueeze(0), v.to(dtype))


def sink_decay_scan(v, alpha, rho, dtype=torch.float64):
    """O(T) form of sink_decay_pattern(alpha, rho) @ v for one head.

    s_i = rho s_{i-1} + v_i ; Z_i = rho Z_{i-1} + 1 ; y_i = a v_0 + (1-a) s_i / Z_i.
    v: (T, hd).  Used to check that the scan identity equals the dense product."""
    T = v.shape[0]
    y = torch.empty(T, v.shape[1], dtype=dtype)
    s = torch.zeros(v.shape[1], dtype=dtype)
    zn = 0.0
    v = v.to(dtype)
    for i in range(T):
        s = rho * s + v[i]
        zn = rho * zn + 1.0
        y[i] = alpha * v[0] + (1.0 - alpha) * s / zn
    return y


# ---------------------------------------------------------------------------
# indexed linear                                     kernel/indexed_linear.py
# ---------------------------------------------------------------------------
def linear_rows(x, weight, bias, rows):
    """F.linear(x, weight[rows], bias[rows]).  kernel/indexed_linear.py:28-38."""
    w = weight[rows]
    b = None if bias is None else bias[rows]
    return torch.nn.functional.linear(x, w, b)


def linear_rows2(x, w1, w2, b1, b2, rows):
    """[x@w1[rows]^T + b1[rows], x@w2[rows]^T + b2[rows]] on the feature dim.
    kernel/indexed_linear.py:86-98."""
    return torch.cat([linear_rows(x, w1, b1, rows), linear_rows(x, w2, b2, rows)], dim=-1)


def linear_permuted_cols(y, weight, bias, cols):
    """F.linear(y, weight[:, cols], bias).  kernel/indexed_linear.py:58-70."""
    return torch.nn.functional.linear(y, weight[:, cols], bias)


# ---------------------------------------------------------------------------
# one attention layer (the module hook)     nanogpt/model.py:1063-1077, 824-844
# ---------------------------------------------------------------------------
def attention_layer(x, wq, wk, wv, wo, frozen, patt, n_head, rope=None, alpha=None, rho=None,
                    z=None, dtype=torch.float32, row_chunk=1024, pidx=None, rows=None, sink_decay=None):
    """Eager capture path of the reference's CausalSelfAttention in dynamic mode:
    full q/k/v projections, RoPE on q,k, softmax for live heads and stored pattern
    for frozen ones, then c_proj.  x: (B,T,C); w*: (C,C) in F.linear layout.
    `frozen`: (H,) ints 0/1/2/3 (see mixed_attn); patt: (H,S,S) or None.  rope = (cos, sin) (T,hd).
    rows = query positions to evaluate (all when None): the result is then (B, len(rows), C)."""
    B, T, C = x.shape
    hd = C // n_head
    x = x.to(dtype)
    q = (x @ wq.to(dtype).t()).view(B, T, n_head, hd).transpose(1, 2)
    k = (x @ wk.to(dtype).t()).view(B, T, n_head, hd).transpose(1, 2)
    v = (x @ wv.to(dtype).t()).view(B, T, n_head, hd).transpose(1, 2)
    if rope is not None:
        cos, sin = rope[0].to(dtype), rope[1].to(dtype)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    y = mixed_attn(q, k, v, patt, frozen, pidx=pidx, alpha=alpha, rho=rho, z=z, dtype=dtype, row_chunk=row_chunk,
                   rows=rows, sink_decay=sink_decay)
    y = y.transpose(1, 2).reshape(B, y.shape[2], C)
    return y @ wo.to(dtype).t()


# ---------------------------------------------------------------------------
# GQA layer (Qwen3-style)      qwen/nanogpt/hybrid_prior_attention.py:530-640
# ---------------------------------------------------------------------------
def rms_norm_heads(x, weight, eps=1e-6):
    """Per-head RMSNorm over the last dim, as the q_norm / k_norm the reference adopts from the HF module
    (hybrid_prior_attention.py:522-523; transformers Qwen3RMSNorm: x * rsqrt(mean(x^2) + eps) * weight,
    statistics in fp32)."""
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return weight * xf.to(x.dtype)


def gqa_attention_layer(x, wq_std, wk, wv, wo, frozen, hidx, pidx, kvidx, patt, cos, sin, sm_scale,
                        q_norm_w=None, k_norm_w=None, eps=1e-6, alpha=None, rho=None, z=None,
                        dtype=torch.float32, row_chunk=1024, rows=None, sink_decay=None):
    """The reference's Qwen3 hybrid attention (hybrid_prior_attention.py:530-584 fused call,
    :586-640 split path; both give the same function): K, V for the HKV raw heads, Q for the live
    ("standard") heads only through the shrunken projection, per-head RMSNorm on q and k when their
    weights are given, RoPE on q and k, query head h reads KV head kvidx[h], frozen heads apply their
    pattern to V[kvidx[h]], then o_proj.  x (B,T,C); wq_std (n_std*hd, C); wk, wv (HKV*hd, C);
    wo (C, H*hd); cos, sin (T, hd)."""
    B, T, C = x.shape
    H = len([int(t) for t in torch.as_tensor(frozen).tolist()])
    hd = wk.shape[0] // (int(torch.as_tensor(kvidx).max().item()) + 1)
    hkv = wk.shape[0] // hd
    n_std = wq_std.shape[0] // hd if wq_std is not None else 0
    x = x.to(dtype)
    k = (x @ wk.to(dtype).t()).view(B, T, hkv, hd)
    v = (x @ wv.to(dtype).t()).view(B, T, hkv, hd).transpose(1, 2)
    if k_norm_w is not None:
        k = rms_norm_heads(k, k_norm_w.to(dtype), eps)
    k = apply_rope(k.transpose(1, 2), cos.to(dtype), sin.to(dtype))
    if n_std:
        q = (x @ wq_std.to(dtype).t()).view(B, T, n_std, hd)
        if q_norm_w is not None:
            q = rms_norm_heads(q, q_norm_w.to(dtype), eps)
        q = apply_rope(q.transpose(1, 2), cos.to(dtype), sin.to(dtype))
    else:
        q = v[:, :0]
    y = mixed_attn(q, k, v, patt, frozen, hidx=hidx, pidx=pidx, kvidx=kvidx, sm_scale=sm_scale, alpha=alpha,
                   rho=rho, z=z, dtype=dtype, row_chunk=row_chunk, rows=rows, sink_decay=sink_decay)
    y = y.transpose(1, 2).reshape(B, y.shape[2], H * hd)
    return y @ wo.to(dtype).t()


# ---------------------------------------------------------------------------
# seeded synthetic inputs of the benchmark configurations
# ---------------------------------------------------------------------------
def frozen_heads_for_layer(n_head, n_frozen, seed, layer):
    """Seeded permutation choice of frozen heads (benchmark configurations 1-4)."""
    g = torch.Generator().manual_seed(seed + layer)
    return sorted(torch.randperm(n_head, generator=g)[:n_frozen].tolist())


def sink_decay_params(n, seed):
    """alpha ~ U(0.05, 0.3), rho ~ U(0.8, 0.99) per frozen head."""
    g = torch.Generator().manual_seed(seed)
    a = 0.05 + 0.25 * torch.rand(n, generator=g, dtype=torch.float64)
    r = 0.8 + 0.19 * torch.rand(n, generator=g, dtype=torch.float64)
    return a, r


# ---------------------------------------------------------------------------
# rest of the transformer block                       nanogpt/model.py:45-54, 1193-1240
# ---------------------------------------------------------------------------
def layer_norm(x, weight, bias=None, eps=1e-5):
    """LayerNorm.forward (nanogpt/model.py:53-54)."""
    return torch.nn.functional.layer_norm(x, weight.shape, weight, bias, eps)


def mlp(x, w_fc, w_proj, b_fc=None, b_proj=None):
    """MLP.forward without dropout (nanogpt/model.py:1202-1207): c_proj(gelu(c_fc(x))), exact (erf) GELU."""
    return torch.nn.functional.linear(torch.nn.functional.gelu(torch.nn.functional.linear(x, w_fc, b_fc)), w_proj, b_proj)


def block(x, ln1_w, ln2_w, attn, w_fc, w_proj):
    """Block.forward (nanogpt/model.py:1237-1240) with `attn` a callable for the attention module."""
    x = x + attn(layer_norm(x, ln1_w))
    return x + mlp(layer_norm(x, ln2_w), w_fc, w_proj)


# ---------------------------------------------------------------------------
# learnable decomposed patterns        supplement/trainable_patterns.py:7-13,
#                                      supplement/trainable_pattern_kernels.py:8-58
# ---------------------------------------------------------------------------
def pattern_dense_reference(value, alpha, rho):
    """dense_reference (supplement/trainable_patterns.py:7-13): softmax over j <= i of alpha_j + rho_{i-j},
    times value.  value (B,H,T,D); alpha, rho (H,S), S >= T."""
    T = value.shape[-2]
    lg = decomp_logits(alpha[:, :T], rho[:, :T])
    return torch.matmul(lg.softmax(-1).to(value.dtype), value)


def pattern_normalisers(alpha, rho, length):
    """normalisers (supplement/trainable_pattern_kernels.py:8-18, 62-66): logsumexp rows below `length`, zero beyond."""
    z = torch.zeros_like(alpha)
    z[:, :length] = decomposed_logz(alpha[:, :length].contiguous(), rho[:, :length].contiguous())
    return z


def pattern_param_grads(value, out, grad, alpha, rho, z, states=None):
    """_parameter_backward (supplement/trainable_pattern_kernels.py:21-58) in closed form:
    dS = P (dO V^T - delta), dalpha_j = sum_{b,i} dS_ij, drho_d = sum_{b,i-j=d} dS_ij for heads in state 2."""
    B, H, T, D = value.shape
    P = decomp_pattern(alpha.double(), rho.double(), z.double(), T)                      # (H,T,T), zero above diagonal
    dP = torch.matmul(grad.double(), value.double().transpose(-1, -2))                   # (B,H,T,T)
    delta = (grad.double() * out.double()).sum(-1, keepdim=True)
    dS = (P[None] * (dP - delta)).sum(0)                                                 # (H,T,T)
    da = torch.zeros_like(alpha, dtype=torch.float64)
    dr = torch.zeros_like(rho, dtype=torch.float64)
    da[:, :T] = dS.sum(1)
    for d in range(T):
        dr[:, d] = torch.diagonal(dS, offset=-d, dim1=1, dim2=2).sum(-1)
    if states is not None:
        keep = (torch.as_tensor(states) == 2).to(da.dtype)[:, None]
        da, dr = da * keep, dr * keep
    return da, dr


# ---------------------------------------------------------------------------
# controller statistics of captured attention        nanogpt/dynamic_freeze.py:96-193, 629-745
# ---------------------------------------------------------------------------
def attention_probs(q, k, sm_scale=None):
    """The tensor the eager capture retains for live heads (nanogpt/model.py:829-835): softmax of the causal scores.
    q, k (B,U,T,hd) -> (B,U,T,T)."""
    T, hd = q.shape[-2], q.shape[-1]
    sc = torch.matmul(q, k.transpose(-1, -2)) * (sm_scale if sm_scale is not None else 1.0 / math.sqrt(hd))
    causal = torch.ones(T, T, dtype=torch.bool).tril()
    return sc.masked_fill(~causal, float("-inf")).softmax(-1)


def centered_batch_reduced_moments(att):
    """_centered_batch_reduced_moments (:96-127): count, mean over samples (H,T,T), centred squares summed per head."""
    bm = att.mean(0)
    return int(att.shape[0]), bm.double(), (att - bm).square().sum(dim=(0, 2, 3)).double()


def merge_reduced_moments(count, mean, head_m2, bn, bm, bm2):
    """_merge_reduced_moments (:130-143): Chan's merge with the M2 kept as one scalar per head."""
    if count == 0:
        return bn, bm.clone(), bm2.clone()
    total = count + bn
    delta = bm - mean
    return total, mean + delta * (bn / total), head_m2 + bm2 + delta.square().sum(dim=(-1, -2)) * (count * bn / total)


def raw_logits(q, k, sm_scale=None):
    """What the eager capture retains as `_last_logits` (nanogpt/model.py:828-831): q k^T / sqrt(hd), nothing masked."""
    return torch.matmul(q, k.transpose(-1, -2)) * (sm_scale if sm_scale is not None else 1.0 / math.sqrt(q.shape[-1]))


def centered_batch_moments(values):
    """_centered_batch_moments (nanogpt/dynamic_freeze.py:62-81): count, mean and centred squares over samples, per cell."""
    bm = values.mean(0)
    return int(values.shape[0]), bm.double(), (values - bm).square().sum(0).double()


def merge_moments(count, mean, m2, bn, bm, bm2):
    """_merge_moments (nanogpt/dynamic_freeze.py:84-93): Chan's merge per cell."""
    if count == 0:
        return bn, bm.clone(), bm2.clone()
    total = count + bn
    delta = bm - mean
    return total, mean + delta * (bn / total), m2 + bm2 + delta.square() * (count * bn / total)


def negative_entropy_sum(att, eps=1e-12):
    """_negative_entropy_sum (:146-173): sum of p log p over samples, rows and columns per head, rows renormalised."""
    pr = att.float()
    pr = pr / pr.sum(-1, keepdim=True).clamp_min(eps)
    return torch.xlogy(pr, pr).sum(dim=(0, 2, 3)).double()


def mean_forward_kl(neg_entropy, mean, n):
    """_mean_forward_kl_from_entropy (:176-193)."""
    T = mean.shape[-1]
    return (neg_entropy / (n * T) - negative_entropy_sum(mean.unsqueeze(0)) / T).clamp_min(0).float()
