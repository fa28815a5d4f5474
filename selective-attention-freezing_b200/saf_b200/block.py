"""The transformer block around the attention path: LayerNorm, residuals and the MLP
(Block / MLP / LayerNorm of the reference, nanogpt/model.py:45-54, 1193-1240), with the same parameter names
(`ln_1`, `main_block`, `ln_2`, `mlp.c_fc`, `mlp.c_proj`) so a reference checkpoint's block state loads unchanged.

bf16 inference runs five launches of this library besides the attention path: two LayerNorms, c_fc with the
GELU in its epilogue, c_proj with the residual add in its epilogue, and the attention output projection.  Other
modes (training, fp32) use the torch modules, as the reference does."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .attention import SafCausalSelfAttention


class LayerNorm(nn.Module):
    """LayerNorm with an optional bias (nanogpt/model.py:45-54)."""

    def __init__(self, ndim, bias):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(ndim))
        self.bias = nn.Parameter(torch.zeros(ndim)) if bias else None

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.bfloat16 and not torch.is_grad_enabled():
            return ops.layer_norm(x, self.weight, self.bias, 1e-5)
        return F.layer_norm(x, self.weight.shape, self.weight, self.bias, 1e-5)


class MLP(nn.Module):
    """c_fc -> GELU -> c_proj (nanogpt/model.py:1193-1207); `residual` is added in c_proj's epilogue."""

    def __init__(self, config):
        super().__init__()
        bias = getattr(config, "bias", False)
        self.c_fc = nn.Linear(config.n_embd, 4 * config.n_embd, bias=bias)
        self.gelu = nn.GELU()
        self.c_proj = nn.Linear(4 * config.n_embd, config.n_embd, bias=bias)
        self.dropout = nn.Dropout(getattr(config, "dropout", 0.0))

    def forward(self, x, residual=None):
        fast = x.is_cuda and x.dtype == torch.bfloat16 and not torch.is_grad_enabled() and \
            self.c_fc.weight.dtype == torch.bfloat16 and (not self.training or self.dropout.p == 0.0)
        if fast:
            hdn = ops.linear_act(x, self.c_fc.weight, self.c_fc.bias, act="gelu")
            return ops.linear_act(hdn, self.c_proj.weight, self.c_proj.bias, residual=residual)
        y = self.dropout(self.c_proj(self.gelu(self.c_fc(x))))
        return y if residual is None else residual + y


class SafBlock(nn.Module):
    """x + attn(ln_1(x)); x + mlp(ln_2(x))  (Block.forward, nanogpt/model.py:1237-1240)."""

    def __init__(self, config, layer_idx=0):
        super().__init__()
        bias = getattr(config, "bias", False)
        self.ln_1 = LayerNorm(config.n_embd, bias=bias)
        self.main_block = SafCausalSelfAttention(config, layer_idx=layer_idx)
        self.ln_2 = LayerNorm(config.n_embd, bias=bias)
        self.mlp = MLP(config)

    def forward(self, x, rope=None):
        x = self.main_block(self.ln_1(x), rope=rope, residual=x)     # residual added in c_proj's epilogue
        return self.mlp(self.ln_2(x), residual=x)
