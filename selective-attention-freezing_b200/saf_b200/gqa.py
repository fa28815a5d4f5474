"""Grouped-query attention with frozen heads, Qwen-shaped: the counterpart of the reference's Qwen3 adapter
(`HybridQwen3Attention`, qwen/nanogpt/hybrid_prior_attention.py:466-640) as a stand-alone module over this
library, plus the block around it (RMSNorm, gated SiLU MLP) and a random-init stack in the shapes of the
grouped-query benchmark configuration.

What the reference does and this module keeps:
  * K and V are projected for the HKV raw heads (query heads of a group share them, so none can be dropped);
    Q is projected for the live ("standard") query heads only.  The reference copies those rows into a shrunken
    `q_proj_std` when it wraps the Hugging Face module (:104-121); here `q_proj` stays canonical and the indexed
    GEMM reads the live heads' rows in place, so a checkpoint's q_proj loads unchanged and (un)freezing a head
    needs no weight surgery;
  * optional per-head RMSNorm on q and k before the rotation (Qwen3 has it, Qwen2.5 does not);
  * RoPE on q and k, query head h reads KV head kvidx[h] = h // (H / HKV), frozen heads apply their pattern to
    V[kvidx[h]]; `fused_mixed_attn(q, k, v, ..., kvidx=)` with compact `pidx` patterns (:575-581);
  * forward only (the reference's grouped-query kernel has no backward, and training raises there too).

bf16 inference without q/k norm is three launches for the attention path: ONE indexed GEMM for
[Q(live) | K(HKV) | V(HKV)] with the rotation of Q and K in its epilogue, the mixed attention, and o_proj with
the residual add in its epilogue.  With q/k norm the normalisation sits between projection and rotation, so
the rotation moves into the attention call (`rope=`).  fp32 runs the same calls on the CUDA-core kernels.
"""
from types import SimpleNamespace

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .attention import rope_tables
from .workloads import WORKLOADS


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.variance_epsilon = eps

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.bfloat16 and not torch.is_grad_enabled() and x.stride(-1) == 1 \
                and x.dim() == 3:
            return ops.rms_norm(x, self.weight, self.variance_epsilon)
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.variance_epsilon)
        return self.weight * xf.to(x.dtype)


class SafGqaAttention(nn.Module):
    """config: hidden_size, num_attention_heads, num_key_value_heads, head_dim, attention_bias (q/k/v bias, as
    Qwen2.5), qk_norm (per-head RMSNorm, as Qwen3), rms_norm_eps, max_position_embeddings."""

    def __init__(self, config, layer_idx=0):
        super().__init__()
        self.layer_idx = layer_idx
        self.hidden = config.hidden_size
        self.n_head = config.num_attention_heads
        self.n_kv = config.num_key_value_heads
        self.head_dim = config.head_dim
        assert self.n_head % self.n_kv == 0
        self.scaling = self.head_dim ** -0.5
        bias = bool(getattr(config, "attention_bias", False))
        self.q_proj = nn.Linear(self.hidden, self.n_head * self.head_dim, bias=bias)
        self.k_proj = nn.Linear(self.hidden, self.n_kv * self.head_dim, bias=bias)
        self.v_proj = nn.Linear(self.hidden, self.n_kv * self.head_dim, bias=bias)
        self.o_proj = nn.Linear(self.n_head * self.head_dim, self.hidden, bias=False)
        if getattr(config, "qk_norm", False):
            eps = getattr(config, "rms_norm_eps", 1e-6)
            self.q_norm, self.k_norm = RMSNorm(self.head_dim, eps), RMSNorm(self.head_dim, eps)
        else:
            self.q_norm = self.k_norm = None
        H = self.n_head
        self.register_buffer("kvidx_i32", (torch.arange(H) // (H // self.n_kv)).to(torch.int32))
        self.register_buffer("frozen_mask_i32", torch.zeros(H, dtype=torch.int32))
        self.register_buffer("hidx_i32", torch.arange(H, dtype=torch.int32))
        self.register_buffer("pidx_i32", torch.zeros(H, dtype=torch.int32))
        self.register_buffer("sd_alpha", torch.zeros(H))
        self.register_buffer("sd_rho", torch.zeros(H))
        self.register_buffer("prior_pattern", None)
        self.register_buffer("dec_alpha", None)
        self.register_buffer("dec_rho", None)
        self.register_buffer("dec_z", None)
        self._live = list(range(H))
        self._rope_key = None

    # ---- freeze state -----------------------------------------------------------------------
    def set_frozen(self, dense=(), patterns=None, decomposed=(), decomp=None, sink_decay=(), sd_params=None):
        """Install the frozen heads of this layer.  dense: heads frozen on stored (T, T) patterns, `patterns`
        (len(dense), S, S) (tril + row renormalisation as the reference applies when it wraps a module, :139-146);
        decomposed: heads on alpha/rho vectors, decomp = (alpha, rho) of shape (H, S) (rows of other heads ignored,
        :124-137); sink_decay: heads on the structured pattern, sd_params = (a, r) per listed head."""
        H = self.n_head
        dev = self.frozen_mask_i32.device
        states = [0] * H
        for h in dense:
            states[h] = 1
        for h in decomposed:
            states[h] = 2
        for h in sink_decay:
            states[h] = 3
        self._live = [h for h in range(H) if states[h] == 0]
        hidx, pidx = [0] * H, [0] * H
        for slot, h in enumerate(self._live):
            hidx[h] = slot
        for slot, h in enumerate(dense):
            pidx[h] = slot
        self.frozen_mask_i32 = torch.tensor(states, dtype=torch.int32, device=dev)
        self.hidx_i32 = torch.tensor(hidx, dtype=torch.int32, device=dev)
        self.pidx_i32 = torch.tensor(pidx, dtype=torch.int32, device=dev)
        if len(dense):
            p = patterns.to(dev).float().tril()
            p = p / p.sum(-1, keepdim=True).clamp_min(torch.finfo(torch.float32).tiny)
            self.prior_pattern = p.to(self.o_proj.weight.dtype).contiguous()
        else:
            self.prior_pattern = None
        if len(decomposed):
            a, r = decomp
            a, r = a.detach().to(dev, torch.float32).contiguous(), r.detach().to(dev, torch.float32).contiguous()
            self.dec_alpha, self.dec_rho, self.dec_z = a, r, ops.decomposed_logz(a, r)
        else:
            self.dec_alpha = self.dec_rho = self.dec_z = None
        sa, sr = torch.zeros(H), torch.zeros(H)
        if len(sink_decay):
            for h, a, r in zip(sink_decay, *sd_params):
                sa[h], sr[h] = float(a), float(r)
        self.sd_alpha, self.sd_rho = sa.to(dev), sr.to(dev)
        self._has_sd = bool(len(sink_decay))

    def _rope(self, cos, sin, T):
        """fp32 (T, hd) tables from the caller's position embeddings ((1, T, hd), (T, hd) or (1, 1, T, hd))."""
        key = (cos.data_ptr(), ops._ver(cos), T)
        if self._rope_key != key:
            hd = cos.shape[-1]
            self._rope_tabs = (cos.reshape(-1, hd)[:T].float().contiguous(), sin.reshape(-1, hd)[:T].float().contiguous())
            self._rope_key = key
        return self._rope_tabs

    def forward(self, hidden_states, position_embeddings, residual=None):
        """(B, T, hidden) -> (B, T, hidden), o_proj included (and `residual` added when given)."""
        if torch.is_grad_enabled() and any(p.requires_grad for p in self.parameters()):
            raise NotImplementedError("grouped-query mixed attention is forward-only (as in the reference)")
        x = hidden_states
        B, T, _ = x.shape
        hd, H, HKV = self.head_dim, self.n_head, self.n_kv
        U = len(self._live)
        cos, sin = self._rope(*position_embeddings, T)
        kw = dict(alpha=self.dec_alpha, rho=self.dec_rho, z=self.dec_z)
        if getattr(self, "_has_sd", False):
            kw["sink_decay"] = (self.sd_alpha, self.sd_rho)
        bs = None
        if self.q_proj.bias is not None:
            bs = [self.q_proj.bias, self.k_proj.bias, self.v_proj.bias]
        fused_rope = self.q_norm is None
        qkv = ops.qkv_projection(x, self.q_proj.weight, self.k_proj.weight, self.v_proj.weight, self._live, hd,
                                 rope=(cos, sin) if fused_rope else None, T=T, biases=bs, grouped=True)
        qkv = qkv.view(B, T, U + 2 * HKV, hd)
        q = qkv[:, :, :U]
        k = qkv[:, :, U:U + HKV]
        v = qkv[:, :, U + HKV:].transpose(1, 2)
        if not fused_rope:
            q, k = self.q_norm(q), self.k_norm(k)
            kw["rope"] = (cos, sin)
        q, k = q.transpose(1, 2), k.transpose(1, 2)
        y = ops.fused_mixed_attn(q, k, v, self.prior_pattern, self.frozen_mask_i32, self.hidx_i32, self.pidx_i32,
                                 sm_scale=self.scaling, validate=False, kvidx=self.kvidx_i32, token_major_out=True, **kw)
        y = y.transpose(1, 2).reshape(B, T, H * hd)
        if x.dtype == torch.bfloat16 and self.hidden % 64 == 0:
            return ops.linear_act(y, self.o_proj.weight, None, residual=residual)
        out = F.linear(y, self.o_proj.weight)
        return out if residual is None else residual + out


class GatedMLP(nn.Module):
    """down_proj(silu(gate_proj(x)) * up_proj(x)), the MLP of Qwen-shaped blocks."""

    def __init__(self, config):
        super().__init__()
        self.gate_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=False)

    def forward(self, x, residual=None):
        if x.is_cuda and x.dtype == torch.bfloat16 and not torch.is_grad_enabled() and \
                self.gate_proj.weight.shape[0] % 128 == 0 and self.down_proj.weight.shape[0] % 64 == 0:
            h = ops.linear_swiglu(x, self.gate_proj.weight, self.up_proj.weight)
            return ops.linear_act(h, self.down_proj.weight, None, residual=residual)
        y = self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))
        return y if residual is None else residual + y


class SafQwenBlock(nn.Module):
    """x + attn(norm(x)); x + mlp(norm(x)) with RMSNorm, grouped-query mixed attention and the gated MLP."""

    def __init__(self, config, layer_idx=0):
        super().__init__()
        eps = getattr(config, "rms_norm_eps", 1e-6)
        self.input_layernorm = RMSNorm(config.hidden_size, eps)
        self.self_attn = SafGqaAttention(config, layer_idx)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps)
        self.mlp = GatedMLP(config)

    def forward(self, x, position_embeddings):
        x = self.self_attn(self.input_layernorm(x), position_embeddings, residual=x)
        return self.mlp(self.post_attention_layernorm(x), residual=x)


def gqa_config(w):
    return SimpleNamespace(hidden_size=w["hidden"], num_attention_heads=w["n_head"], num_key_value_heads=w["n_kv"],
                           head_dim=w["head_dim"], attention_bias=w.get("qkv_bias", False), qk_norm=False,
                           rms_norm_eps=1e-6, intermediate_size=w["mlp"], max_position_embeddings=w["T"])


def build_gqa_stack(name, device, dtype=torch.bfloat16, seed=1337, blocks=False, n_layer=None):
    """Random-init N(0, 0.02^2) stack in the shapes of a grouped-query workload (no checkpoint is needed): one
    SafGqaAttention per layer (blocks=True: the whole block with RMSNorms and the gated MLP), 25 % of the query
    heads of every layer frozen on seeded sink+decay patterns."""
    from .synthetic import frozen_heads_for_layer, sink_decay_params
    w = WORKLOADS[name] if isinstance(name, str) else name
    cfg = gqa_config(w)
    g = torch.Generator().manual_seed(seed)
    layers = []
    for li in range(w["n_layer"] if n_layer is None else n_layer):
        m = SafQwenBlock(cfg, li) if blocks else SafGqaAttention(cfg, li)
        with torch.no_grad():
            for pname, p in m.named_parameters():
                if p.dim() >= 2:
                    p.copy_(torch.randn(p.shape, generator=g) * 0.02)
                elif pname.endswith("bias"):
                    p.copy_(torch.randn(p.shape, generator=g) * 0.02)
        attn = m.self_attn if blocks else m
        fz = frozen_heads_for_layer(w["n_head"], w["n_frozen"], seed, li)
        a, r = sink_decay_params(len(fz), seed + 1000 + li)
        m = m.to(device=device, dtype=dtype).eval()
        attn.set_frozen(sink_decay=fz, sd_params=(a.tolist(), r.tolist()))
        layers.append(m)
    cos, sin = rope_tables(w["head_dim"], w["T"], base=w["rope_base"], device=device)
    return layers, (cos, sin), w


def gqa_stack_forward(layers, rope, x):
    h = x
    for m in layers:
        h = m(h, rope)
    return h


def gqa_stack_flops(w, blocks=False):
    """Algorithmic FLOPs of one pass per sequence: live causal attention, grouped QKV projection, o_proj [, MLP]."""
    H, HKV, hd, T, nf, C, L = w["n_head"], w["n_kv"], w["head_dim"], w["T"], w["n_frozen"], w["hidden"], w["n_layer"]
    U = H - nf
    live = 2 * U * T * T * hd
    qkv = 2 * T * C * (U + 2 * HKV) * hd
    oproj = 2 * T * (H * hd) * C
    mlp = 2 * T * C * 3 * w["mlp"]
    return dict(live=live * L, qkv=qkv * L, oproj=oproj * L, mlp=mlp * L if blocks else 0)
