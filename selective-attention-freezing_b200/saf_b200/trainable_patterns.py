"""Learnable decomposed patterns: parameter gradients for alpha and rho of state-2 heads.

Mirror of supplement/trainable_pattern_kernels.py (`normalisers`, `PatternGradient`) and of the
opt-in switch in supplement/trainable_patterns.py (`enable`, `attach_optimizer`).  The frozen path is
unchanged: `fused_mixed_attn` still produces the output and dV; `PatternGradient` adds
    dalpha[h,j] = sum_{b,i} P_ij (dP_ij - delta_i),   drho[h,d] = sum_{b,i-j=d} P_ij (dP_ij - delta_i)
with P = exp(alpha_j + rho_{i-j} - z_i), dP = dO V^T, delta_i = dO_i . O_i, computed by
`saf_pattern_param_grad` without a T x T buffer.  `saf_b200.ops.fused_mixed_attn` applies it by
itself when it is handed alpha / rho that require grad, which is what the reference's patched
dispatch does (supplement/trainable_patterns.py:56-93).
"""
import ctypes as C

import torch
from torch import nn

from . import _cabi
from ._cabi import SafPatternGradArgs, check, lib
from . import ops


@torch.no_grad()
def normalisers(alpha, rho, length):
    """z[h,i] = logsumexp_{j<=i}(alpha[h,j] + rho[h,i-j]) for i < length, 0 beyond
    (supplement/trainable_pattern_kernels.py:62-66).  alpha, rho (H, S); returns (H, S) like alpha."""
    ops._require_cuda(alpha, "alpha")
    H, S = alpha.shape
    a = alpha.detach().float().contiguous()
    r = rho.detach().float().contiguous()
    z = torch.empty_like(a)
    ops._call(a, lib.saf_pattern_normalisers, a.data_ptr(), r.data_ptr(), z.data_ptr(), H, S, int(length))
    return z.to(alpha.dtype)


def pattern_param_grad(grad, out, value, alpha, rho, z, states):
    """(dalpha, drho), both (H, S) fp32-accumulated and returned in alpha's / rho's dtype."""
    B, H, T, HD = value.shape
    S = alpha.shape[1]
    if grad.stride(-1) != 1:
        grad = grad.contiguous()
    if out.stride(-1) != 1:
        out = out.contiguous()
    if value.stride(-1) != 1:
        value = value.contiguous()
    if not (grad.dtype == out.dtype == value.dtype):
        grad, out = grad.to(value.dtype), out.to(value.dtype)
    a32 = alpha.detach().float().contiguous()
    r32 = rho.detach().float().contiguous()
    z32 = z.detach().float().contiguous()
    da = torch.zeros_like(a32)
    dr = torch.zeros_like(r32)
    g = SafPatternGradArgs()
    g.struct_size = C.sizeof(SafPatternGradArgs)
    g.dtype = ops._dt(value)
    g.B, g.H, g.T, g.HD, g.SD = B, H, T, HD, S
    g.force_state = -1
    g.v, g.out, g.dout = ops._st(value), ops._st(out), ops._st(grad)
    g.alpha, g.rho, g.z = a32.data_ptr(), r32.data_ptr(), z32.data_ptr()
    states = states if states.dtype == torch.int32 else states.to(torch.int32)
    g.frozen = states.data_ptr()
    host = ops.host_ints(states)
    keep = None
    if host is not None:
        keep = (C.c_int32 * H)(*host)
        g.frozen_host = keep
    g.dalpha, g.drho = da.data_ptr(), dr.data_ptr()
    delta = torch.empty((B, H, T), device=value.device, dtype=torch.float32)   # scratch of the tensor-core path
    g.delta = delta.data_ptr()
    g.status = ops._status_ptr(value.device)
    ops._call(value, lib.saf_pattern_param_grad, C.byref(g))
    return da.to(alpha.dtype), dr.to(rho.dtype)


class PatternGradient(torch.autograd.Function):
    """Identity on `out` that adds the exact softmax-parameter derivatives
    (supplement/trainable_pattern_kernels.py:69-85): backward returns
    (grad, None, dalpha, drho, None, None)."""

    @staticmethod
    def forward(ctx, out, value, alpha, rho, z, states):
        ctx.save_for_backward(out, value, alpha, rho, z, states)
        return out.view_as(out)

    @staticmethod
    def backward(ctx, grad):
        out, value, alpha, rho, z, states = ctx.saved_tensors
        da, dr = pattern_param_grad(grad, out, value, alpha, rho, z, states)
        return grad, None, da, dr, None, None


# z of the current parameter values, keyed by the parameter object: recomputed when alpha or rho change
_Z_CACHE = {}


def clear_pattern_cache():
    _Z_CACHE.clear()


def current_normalisers(alpha, rho, length):
    """`normalisers`, cached per (alpha, rho) version like the reference's dispatch cache
    (supplement/trainable_patterns.py:66-80).  Optimizers that update parameters without touching the
    version counter must call `clear_pattern_cache()` after each step (`attach_optimizer` does)."""
    key = id(alpha)
    sig = (ops._ver(alpha), ops._ver(rho), int(length), alpha.device)
    hit = _Z_CACHE.get(key)
    if hit is not None and hit[0] is alpha and hit[1] == sig:
        return hit[2]
    z = normalisers(alpha, rho, length)
    _Z_CACHE[key] = (alpha, sig, z)
    return z


def enable(model, optimizer=None):
    """Turn the fitted `dyn_alpha` / `dyn_rho` buffers of every attention module that has decomposed
    heads into parameters (supplement/trainable_patterns.py:17-41).  Works on any module tree whose
    attention modules carry `dyn_decomp`, `dyn_alpha`, `dyn_rho` (saf_b200.attention.SafAttention and
    the reference's CausalSelfAttention both do).  Returns the new parameters."""
    parameters = []
    for attn in model.modules():
        if not hasattr(attn, "dyn_decomp") or not hasattr(attn, "dyn_alpha"):
            continue
        if not bool(attn.dyn_decomp.any().item()):
            continue
        for name in ("dyn_alpha", "dyn_rho"):
            old = getattr(attn, name)
            if isinstance(old, nn.Parameter):
                raise RuntimeError("Pattern parameters were already enabled")
            delattr(attn, name)
            parameter = nn.Parameter(old.detach().clone().float())
            attn.register_parameter(name, parameter)
            parameters.append(parameter)
        attn.register_state_dict_pre_hook(_export_current_buffers)
    if not parameters:
        raise RuntimeError("No fitted patterns to train")
    if optimizer is not None:
        optimizer.add_param_group(dict(params=parameters, weight_decay=0.))
        attach_optimizer(model, optimizer)
    return parameters


def attach_optimizer(model, optimizer):
    """Drop the cached normalisers after every optimizer step (fused optimizers do not reliably bump
    the tensors' version counters, supplement/trainable_patterns.py:44-50)."""
    optimizer.register_step_post_hook(lambda *args: clear_pattern_cache())


@torch.no_grad()
def _export_current_buffers(attn, prefix, keep_vars):
    """Before a state dict is taken, bring the derived buffers in line with the trained parameters
    (supplement/trainable_patterns.py:53-58)."""
    attn.dyn_z.copy_(normalisers(attn.dyn_alpha, attn.dyn_rho, attn.dyn_alpha.shape[1]).to(attn.dyn_z.dtype))
    if getattr(attn, "dyn_rho_band", None) is not None:
        attn.dyn_rho_band.copy_(ops.make_rho_band(attn.dyn_rho.detach()).to(attn.dyn_rho_band.dtype))
