"""Attention-module hook: a from-scratch stand-in for the dynamic branch of the reference's
`CausalSelfAttention` (nanogpt/model.py:520-1186, dynamic part :634-1077).

Same public methods (`forward(x, rope)`, `freeze_heads`, `freeze_heads_decomposed`,
`unfreeze_heads`, `set_capture`, `refresh_dynamic_derived_state`), same parameter names
(`q_proj`, `k_proj`, `v_proj`, `c_proj`) and same buffer names / shapes / dtypes (`dyn_frozen`,
`dyn_pattern`, `dyn_decomp`, `dyn_alpha`, `dyn_rho`, `dyn_z`, `dyn_rho_band`), so a reference
checkpoint's attention state loads unchanged.  Additions: `dyn_sd` (H, 2) with the (sink weight,
decay) of heads frozen on a structured pattern, kept as the int32 bit patterns of fp32 numbers so that
casting the module to bf16 cannot round them (read them with `sd_params()`), and `dyn_struct` (H,) bool marking
them; `freeze_heads(..., detect_structured=True)` recognises such patterns (exactness-checked)
and routes them to the O(T) scan instead of the dense product.

Hot path (`_attend_cheap`):
  inference: ONE tensor-core GEMM for [Q(live) | K(live) | V(all)] reading the canonical weights in
             place with RoPE in its epilogue -> fused mixed attention -> c_proj GEMM.
  training : linear_rows2 (live-only Q/K, exact-zero grads for frozen rows, RoPE in its epilogue and the adjoint
             rotation in its backward), v_proj and c_proj through the same indexed GEMMs with every row selected.
The eager capture path (`set_capture(True)`) is the reference's semantic definition
(nanogpt/model.py:824-844) written with torch ops; it exists for measurement by a freeze
controller, never as a fallback of the hot path.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops

BAND_ROWS = ops.BAND_ROWS


def rope_tables(head_dim, seq_len, base=10000.0, device=None):
    """fp32 (T, hd) cos / sin tables, cat(freqs, freqs) layout (nanogpt/model.py:73-83)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    pos = torch.arange(seq_len, dtype=torch.float32)
    freqs = torch.outer(pos, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(device).contiguous(), emb.sin().to(device).contiguous()


def classify_sink_decay(pattern, tol=None):
    """If `pattern` (T, T) equals a * [j=0] + (1-a) r^(i-j) / Z_i on the causal triangle, return (a, r).

    r is read from the ratio of two neighbouring entries, a from the second row, and the pair is
    accepted only if the rebuilt pattern matches every entry to `tol` (default: 8 ulp of the stored
    dtype, at least 1e-6).  Returns None otherwise."""
    T = pattern.shape[-1]
    if T < 3:
        return None
    p = pattern.double()
    if tol is None:
        tol = max(1e-6, 8 * torch.finfo(pattern.dtype).eps)
    i = min(T - 1, 8)
    if p[i, 2].item() <= 0 or p[1, 1].item() <= 0:
        return None
    r = (p[i, 1] / p[i, 2]).item()
    if not (0.0 < r <= 1.0):
        return None
    a = 1.0 - p[1, 1].item() * (1.0 + r)
    if not (-1e-9 <= a < 1.0):
        return None
    a = max(a, 0.0)
    dev = pattern.device
    for i0 in range(0, T, 1024):
        i1 = min(i0 + 1024, T)
        ii = torch.arange(i0, i1, device=dev, dtype=torch.float64)[:, None]
        jj = torch.arange(0, i1, device=dev, dtype=torch.float64)[None, :]
        dist = ii - jj
        zi = (1.0 - r ** (ii + 1.0)) / (1.0 - r) if r < 1.0 else ii + 1.0
        rebuilt = torch.where(dist >= 0, (1.0 - a) * (r ** dist.clamp(min=0)) / zi, torch.zeros((), device=dev, dtype=torch.float64))
        rebuilt[:, 0] += a
        if (rebuilt - p[i0:i1, :i1]).abs().max().item() > tol:
            return None
        if i1 < T and p[i0:i1, i1:].abs().max().item() > tol:
            return None
    return a, r


class SafCausalSelfAttention(nn.Module):

    def __init__(self, config, layer_idx=0):
        super().__init__()
        assert config.n_embd % config.n_head == 0
        self.layer_idx = layer_idx
        self.n_head = config.n_head
        self.n_embd = config.n_embd
        self.head_dim = config.n_embd // config.n_head
        self.dropout = float(getattr(config, "dropout", 0.0))
        self.position_encoding = getattr(config, "position_encoding", "rope")
        bias = bool(getattr(config, "bias", False))
        self.q_proj = nn.Linear(config.n_embd, config.n_embd, bias=bias)
        self.k_proj = nn.Linear(config.n_embd, config.n_embd, bias=bias)
        self.v_proj = nn.Linear(config.n_embd, config.n_embd, bias=bias)
        self.c_proj = nn.Linear(config.n_embd, config.n_embd, bias=bias)
        self.dynamic = True
        self.prior_repr = getattr(config, "rand_attn_prior_repr", "dense")
        self._pattern_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[
            getattr(config, "freeze_pattern_dtype", "float32")]
        H, S = config.n_head, config.block_size
        self.block_size = S
        self.register_buffer("dyn_frozen", torch.zeros(H, dtype=torch.bool))
        self.register_buffer("dyn_struct", torch.zeros(H, dtype=torch.bool))
        self.register_buffer("dyn_sd", torch.zeros(H, 2, dtype=torch.int32))   # fp32 bits, see sd_params()
        if self.prior_repr == "decomposed":
            assert S % BAND_ROWS == 0, (
                f"rand_attn_prior_repr='decomposed' needs block_size divisible by {BAND_ROWS} (got {S})")
            self.register_buffer("dyn_decomp", torch.zeros(H, dtype=torch.bool))
            self.register_buffer("dyn_alpha", torch.zeros(H, S))
            self.register_buffer("dyn_rho", torch.zeros(H, S))
            self.register_buffer("dyn_z", torch.zeros(H, S))
            self.register_buffer("dyn_rho_band", None)
            self.register_buffer("dyn_pattern", None)
        else:
            # the dense (H, S, S) buffer is allocated at the first dense freeze: structured heads
            # never need it (at S = 16384 it would be 6.4 GB per layer in bf16)
            self.register_buffer("dyn_pattern", None)
        self._capture = False
        self._last_attn = None
        self._last_logits = None
        self._capture_logits = True
        self._retain_attention = True
        self._stats = None
        self._logit_stats = None
        self._fz_dirty = True

    # ---- freeze state ---------------------------------------------------------------------
    def set_capture(self, flag, capture_logits=True, retain_attention=True):
        """nanogpt/model.py:690-703."""
        self._capture = bool(flag)
        self._capture_logits = bool(capture_logits)
        self._retain_attention = bool(retain_attention)
        if not flag:
            self._last_attn = None
            self._last_logits = None

    def set_statistics(self, accumulator, logit_accumulator=None):
        """Measurement without the capture: while an accumulator is set (a `saf_b200.capture.AttentionMoments` over
        this layer's live heads, in their compact order), every fused forward merges the attention statistics of
        its live heads into it from the rotated q, k -- what the controller derives from `_last_attn` after
        `set_capture(True)` (nanogpt/dynamic_freeze.py:664-745) -- and the fast path keeps running.  None switches
        it off.  Frozen heads are not measured: their attention is the stored pattern.  `logit_accumulator` (a
        `saf_b200.capture.LogitMoments`) does the same for the raw scores of the live heads, what
        `set_capture(True, capture_logits=True)` retains as `_last_logits` (nanogpt/dynamic_freeze.py:721-737)."""
        self._stats = accumulator
        self._logit_stats = logit_accumulator

    def _measure(self, qu, ku):
        if self._stats is not None:
            self._stats.update(qu, ku)
        if self._logit_stats is not None:
            self._logit_stats.update(qu, ku)

    def sd_params(self):
        """(H, 2) fp32 view of the structured heads' (sink weight, decay)."""
        return self.dyn_sd.view(torch.float32)

    def _set_sd(self, h, a, r):
        self.dyn_sd[h] = torch.tensor([a, r], dtype=torch.float32).view(torch.int32).to(self.dyn_sd.device)

    def _ensure_pattern(self):
        if self.dyn_pattern is None:
            S = self.block_size
            self.dyn_pattern = torch.zeros(self.n_head, S, S, device=self.dyn_frozen.device,
                                           dtype=self._pattern_dtype)

    def freeze_heads(self, head_idx, patterns, detect_structured=False):
        """Freeze heads to fixed (T, T) patterns; tril + row renormalisation as the reference does
        at install time (nanogpt/model.py:705-733)."""
        head_idx = list(head_idx)
        if patterns.ndim != 3 or patterns.size(-2) != patterns.size(-1):
            raise ValueError("frozen patterns must have shape (n_heads, T, T)")
        if patterns.size(0) != len(head_idx):
            raise ValueError("one frozen pattern is required per head index")
        T = patterns.size(-1)
        if T > self.block_size:
            raise ValueError("frozen pattern exceeds the configured block size")
        patterns = patterns.tril()
        patterns = patterns / patterns.sum(-1, keepdim=True).clamp_min(1e-12)
        for j, h in enumerate(head_idx):
            sd = classify_sink_decay(patterns[j]) if detect_structured else None
            self.dyn_frozen[h] = True
            if self.prior_repr == "decomposed":
                self.dyn_decomp[h] = False
            if sd is not None:
                self.dyn_struct[h] = True
                self._set_sd(h, *sd)
                continue
            self.dyn_struct[h] = False
            self._ensure_pattern()
            self.dyn_pattern[h, :T, :T] = patterns[j].to(self.dyn_pattern.device, self.dyn_pattern.dtype)
        self._fz_dirty = True

    def freeze_heads_sink_decay(self, head_idx, alpha, rho):
        """Freeze heads on the structured pattern a[j=0] + (1-a) r^(i-j)/Z_i, stored as two numbers."""
        for h, a, r in zip(list(head_idx), list(alpha), list(rho)):
            a, r = float(a), float(r)
            if not (0.0 <= a < 1.0 and 0.0 <= r <= 1.0):
                raise ValueError("sink weight must lie in [0, 1) and decay in [0, 1]")
            self.dyn_frozen[h] = True
            self.dyn_struct[h] = True
            self._set_sd(h, a, r)
            if self.prior_repr == "decomposed":
                self.dyn_decomp[h] = False
        self._fz_dirty = True

    def freeze_heads_decomposed(self, head_idx, alpha, rho, z=None):
        """nanogpt/model.py:735-764."""
        assert self.prior_repr == "decomposed", \
            "freeze_heads_decomposed requires rand_attn_prior_repr='decomposed'"
        T = alpha.size(-1)
        buf = self.dyn_alpha
        idx = torch.as_tensor(list(head_idx), dtype=torch.long, device=buf.device)
        a32 = alpha.to(buf.device, torch.float32)
        r32 = rho.to(buf.device, torch.float32)
        z32 = ops.decomposed_logz(a32, r32) if z is None else z.to(buf.device, torch.float32)
        self.dyn_frozen[idx] = True
        self.dyn_decomp[idx] = True
        self.dyn_struct[idx] = False
        self.dyn_alpha[idx, :T] = a32.to(buf.dtype)
        self.dyn_rho[idx, :T] = r32.to(buf.dtype)
        self.dyn_z[idx, :T] = z32.to(buf.dtype)
        if self.dyn_rho_band is None:
            self.dyn_rho_band = torch.zeros(self.n_head, BAND_ROWS, self.dyn_rho.size(1), device=buf.device,
                                            dtype=buf.dtype)
        self.dyn_rho_band[idx] = ops.make_rho_band(self.dyn_rho[idx])
        self._fz_dirty = True

    def unfreeze_heads(self, head_idx):
        """nanogpt/model.py:766-772."""
        for h in head_idx:
            self.dyn_frozen[h] = False
            self.dyn_struct[h] = False
            if self.prior_repr == "decomposed":
                self.dyn_decomp[h] = False
        self._fz_dirty = True

    @torch.no_grad()
    def refresh_dynamic_derived_state(self, *, rebuild_rho_band=False):
        """nanogpt/model.py:774-794."""
        if self.prior_repr == "decomposed" and rebuild_rho_band:
            idx = (self.dyn_decomp & self.dyn_frozen).nonzero(as_tuple=True)[0]
            if idx.numel():
                if self.dyn_rho_band is None:
                    self.dyn_rho_band = torch.zeros(self.n_head, BAND_ROWS, self.dyn_rho.size(1),
                                                    device=self.dyn_rho.device, dtype=self.dyn_rho.dtype)
                self.dyn_rho_band[idx] = ops.make_rho_band(self.dyn_rho[idx])
        self._fz_dirty = True
        self._refresh_freeze_cache()

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        # lazy buffers present in a checkpoint are materialised before the parent load (nanogpt/model.py:900-911)
        for name in ("dyn_pattern", "dyn_rho_band"):
            key = prefix + name
            if key in state_dict and getattr(self, name, None) is None:
                setattr(self, name, torch.zeros_like(state_dict[key], device=self.dyn_frozen.device))
        for name in ("dyn_struct", "dyn_sd"):   # absent from reference checkpoints
            key = prefix + name
            if key not in state_dict:
                state_dict[key] = getattr(self, name).clone()
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        self._fz_dirty = True

    def _refresh_freeze_cache(self):
        """Per-freeze-set caches; the only place with host syncs (nanogpt/model.py:846-898)."""
        frozen = self.dyn_frozen
        dev = frozen.device
        fz = frozen.cpu().tolist()
        st = self.dyn_struct.cpu().tolist()
        dec = self.dyn_decomp.cpu().tolist() if self.prior_repr == "decomposed" else [False] * self.n_head
        states = []
        for h in range(self.n_head):
            states.append(0 if not fz[h] else (3 if st[h] else (2 if dec[h] else 1)))
        self._states = states
        self._live = [h for h in range(self.n_head) if states[h] == 0]
        self._n_frozen = self.n_head - len(self._live)
        self._fz_mask_i32 = torch.tensor(states, dtype=torch.int32, device=dev)
        hidx = [0] * self.n_head
        for slot, h in enumerate(self._live):
            hidx[h] = slot
        self._hidx_i32 = torch.tensor(hidx, dtype=torch.int32, device=dev)
        hd = self.head_dim
        if self._live:
            self._uf_cols = (torch.tensor(self._live, device=dev)[:, None] * hd + torch.arange(hd, device=dev)).reshape(-1)
        else:
            self._uf_cols = None
        self._all_rows = torch.arange(self.n_embd, device=dev)
        self._dec_any = 2 in states
        self._sd_any = 3 in states
        sd = self.sd_params()
        self._sd = (sd[:, 0].contiguous(), sd[:, 1].contiguous()) if self._sd_any else None
        self._patt_cast = None      # compact copy of the dense heads' patterns in the activation dtype, built on demand
        self._mask_frozen_only = None   # head states with live heads masked out (training with attention dropout)
        self._fz_dirty = False

    # ---- forward --------------------------------------------------------------------------
    def _rope_f32(self, rope, T, device):
        """fp32 (T, hd) tables from the caller's (1,1,T,hd) cache, or None."""
        if self.position_encoding != "rope":
            return None
        if rope is None:
            raise ValueError("RoPE Q/K requested without a rotary cache")
        cos, sin = rope
        key = (cos.data_ptr(), ops._ver(cos), T)
        if getattr(self, "_rope_key", None) != key:
            self._rope_cache = (cos.reshape(-1, cos.shape[-1])[:T].float().contiguous(),
                                sin.reshape(-1, sin.shape[-1])[:T].float().contiguous())
            self._rope_key = key
        return self._rope_cache

    def _frozen_patterns(self, T):
        """(H, T, T) fp32 patterns of all heads for the eager path (rows of live heads are zero)."""
        dev = self.dyn_frozen.device
        fp = torch.zeros(self.n_head, T, T, device=dev)
        for h, s in enumerate(self._states):
            if s == 1:
                fp[h] = self.dyn_pattern[h, :T, :T].float()
            elif s == 2:
                lg = ops.decomp_logits(self.dyn_alpha[h:h + 1, :T].float(), self.dyn_rho[h:h + 1, :T].float())
                fp[h] = torch.exp(lg - self.dyn_z[h:h + 1, :T].float()[:, :, None])[0]
            elif s == 3:
                a, r = self.sd_params()[h].tolist()
                i = torch.arange(T, device=dev, dtype=torch.float64)
                dist = i[:, None] - i[None, :]
                decay = torch.where(dist >= 0, torch.tensor(r, dtype=torch.float64, device=dev) ** dist.clamp(min=0),
                                    torch.zeros((), dtype=torch.float64, device=dev))
                pat = (1.0 - a) * decay / decay.sum(-1, keepdim=True)
                pat[:, 0] += a
                fp[h] = pat.float()
        return fp

    def _attend_dynamic(self, q, k, v):
        """Eager definition (nanogpt/model.py:824-844)."""
        B, nh, T, hd = q.shape
        scores = (q @ k.transpose(-2, -1)) * (1.0 / math.sqrt(hd))
        if self._capture and self._capture_logits:
            self._last_logits = scores.detach()          # raw, unmasked: for the priors that sample logits
        causal = torch.tril(torch.ones(T, T, dtype=torch.bool, device=q.device))
        att = F.softmax(scores.masked_fill(~causal, float("-inf")), dim=-1)
        if self._n_frozen:
            fp = self._frozen_patterns(T).to(att.dtype).unsqueeze(0)
            att = torch.where(self.dyn_frozen.view(1, nh, 1, 1), fp.expand_as(att), att)
        if self._capture and self._retain_attention:
            self._last_attn = att.detach()
        return att @ v

    def _attend_cheap(self, x, rope=None, residual=None):
        B, T, C = x.shape
        nh, hd = self.n_head, self.head_dim
        rp = self._rope_f32(rope, T, x.device)
        patt, pidx = self.dyn_pattern, None
        dec = (self.dyn_alpha, self.dyn_rho, self.dyn_z) if self._dec_any else (None, None, None)
        act_dt = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
        if act_dt == torch.bfloat16 and patt is not None and patt.dtype != act_dt and 1 in self._states:
            # The kernels multiply the pattern in the activation dtype (the reference casts P to v's dtype in
            # registers, kernel/frozen_attn.py:81).  A compact bf16 copy of the dense heads' planes, made once per
            # freeze set, gives the same products and lets them run on the TMA-fed tensor-core path.
            if self._patt_cast is None:
                dense = [h for h in range(nh) if self._states[h] == 1]
                slot = [0] * nh
                for i, h in enumerate(dense):
                    slot[h] = i
                self._patt_cast = (patt[dense].to(act_dt), torch.tensor(slot, dtype=torch.int32, device=patt.device))
            patt, pidx = self._patt_cast
        nuf = len(self._live)
        if not torch.is_grad_enabled() and act_dt == torch.bfloat16 and (self.dropout == 0.0 or not self.training):
            # inference: one GEMM, canonical weights read in place, RoPE in the epilogue
            w = [m.weight if m.weight.dtype == act_dt else m.weight.to(act_dt) for m in (self.q_proj, self.k_proj, self.v_proj)]
            bs = None
            if self.q_proj.bias is not None:
                bs = [m.bias.to(act_dt) for m in (self.q_proj, self.k_proj, self.v_proj)]
            qkv = ops.qkv_projection(x.to(act_dt), w[0], w[1], w[2], self._live, hd, rope=rp, T=T, biases=bs)
            qkv = qkv.view(B, T, 2 * nuf + nh, hd)
            qu = qkv[:, :, :nuf].transpose(1, 2)
            ku = qkv[:, :, nuf:2 * nuf].transpose(1, 2)
            v = qkv[:, :, 2 * nuf:].transpose(1, 2)
            if nuf:
                self._measure(qu, ku)
            y = ops.fused_mixed_attn(qu, ku, v, patt, self._fz_mask_i32, self._hidx_i32, pidx,
                                     alpha=dec[0], rho=dec[1], z=dec[2], validate=False, sink_decay=self._sd)
            y = y.transpose(1, 2).reshape(B, T, nh * hd)
            cw = self.c_proj.weight if self.c_proj.weight.dtype == act_dt else self.c_proj.weight.to(act_dt)
            cb = None if self.c_proj.bias is None else self.c_proj.bias.to(act_dt)
            if residual is not None and (nh * hd) % 64 == 0:
                return ops.linear_act(y, cw, cb, residual=residual.to(act_dt))   # residual add in the GEMM epilogue
            out = ops.linear_rows(y, cw, cb, self._all_rows)
            return out if residual is None else residual + out
        # training / fp32: live-only Q,K projection with exact-zero frozen rows in the weight gradient; v_proj and
        # c_proj run on the library's own forward / dx / dW GEMMs too (all rows selected)
        v = ops.linear_rows(x, self.v_proj.weight, self.v_proj.bias, self._all_rows).view(B, T, nh, hd).transpose(1, 2)
        if nuf == 0:
            qu = ku = v[:, :0]
        else:
            # rotation fused into the projection's epilogue (adjoint rotation in its backward), so the
            # attention kernels get rotated q, k and take the tensor-core path
            qk = ops.linear_rows2(x, self.q_proj.weight, self.k_proj.weight, self.q_proj.bias, self.k_proj.bias,
                                  self._uf_cols, rope=rp, head_dim=hd).view(B, T, 2, nuf, hd)
            qu, ku = qk[:, :, 0].transpose(1, 2), qk[:, :, 1].transpose(1, 2)
            self._measure(qu.detach(), ku.detach())
        if self.dropout > 0.0 and self.training and nuf:
            # The fused kernels implement no attention dropout.  As in the reference, which leaves its fused path
            # in this case and lets the SDPA half of its split path apply the dropout (nanogpt/model.py:971-974,
            # 1017-1061): live heads go through torch's SDPA with dropout_p, frozen heads through the library
            # (their patterns carry no dropout).  The library call marks the live heads as structured heads with
            # zero parameters -- an O(T) scan whose rows are then overwritten -- so they cost no attention FLOPs.
            if self._mask_frozen_only is None:
                st = self._fz_mask_i32.clone()
                st[st == 0] = 3
                sd = self.sd_params().clone()
                sd[torch.as_tensor(self._live, device=sd.device)] = torch.tensor([0.0, 0.5], device=sd.device)
                self._mask_frozen_only = (st, (sd[:, 0].contiguous(), sd[:, 1].contiguous()))
            st, sd = self._mask_frozen_only
            y = ops.fused_mixed_attn(v[:, :0], v[:, :0], v, patt, st, self._hidx_i32, pidx,
                                     alpha=dec[0], rho=dec[1], z=dec[2], validate=False, sink_decay=sd)
            live = torch.as_tensor(self._live, device=x.device)
            y_live = F.scaled_dot_product_attention(qu, ku, v.index_select(1, live), dropout_p=self.dropout,
                                                    is_causal=True)
            y = y.index_copy(1, live, y_live.to(y.dtype))
        else:
            y = ops.fused_mixed_attn(qu, ku, v, patt, self._fz_mask_i32, self._hidx_i32, pidx,
                                     alpha=dec[0], rho=dec[1], z=dec[2], validate=False, sink_decay=self._sd)
        y = y.transpose(1, 2).reshape(B, T, nh * hd)
        out = ops.linear_rows(y, self.c_proj.weight, self.c_proj.bias, self._all_rows)
        out = F.dropout(out, self.dropout, self.training)                # resid_dropout (nanogpt/model.py:1169)
        return out if residual is None else residual + out

    def forward(self, x, rope=None, residual=None):
        """(B, T, C) -> (B, T, C), output of c_proj included (nanogpt/model.py:1063-1077)."""
        if self._fz_dirty:
            self._refresh_freeze_cache()
        B, T, C = x.shape
        nh, hd = self.n_head, self.head_dim
        if self._capture:
            q = self.q_proj(x).view(B, T, nh, hd).transpose(1, 2)
            k = self.k_proj(x).view(B, T, nh, hd).transpose(1, 2)
            v = self.v_proj(x).view(B, T, nh, hd).transpose(1, 2)
            if self.position_encoding == "rope":
                cos, sin = rope
                cos, sin = cos.reshape(1, 1, -1, hd)[:, :, :T].to(q.dtype), sin.reshape(1, 1, -1, hd)[:, :, :T].to(q.dtype)
                rot = lambda t: torch.cat((-t[..., hd // 2:], t[..., :hd // 2]), dim=-1)   # noqa: E731
                q, k = q * cos + rot(q) * sin, k * cos + rot(k) * sin
            y = self._attend_dynamic(q, k, v).transpose(1, 2).contiguous().view(B, T, nh * hd)
            out = F.dropout(self.c_proj(y), self.dropout, self.training)
            return out if residual is None else residual + out
        if not x.is_cuda:
            raise RuntimeError("SafCausalSelfAttention runs on CUDA only (set_capture(True) gives the eager torch path)")
        return self._attend_cheap(x, rope=rope, residual=residual)
