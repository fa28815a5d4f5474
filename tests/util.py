"""Shared builders for the parity tests (seeded inputs in the style of the reference's
kernel/test_fused_attn.py:24-37 and kernel/test_frozen_attn.py:20-24)."""
import torch

from oracle import saf_oracle as O


def make_pattern(nh, S, seed=0, dtype=torch.float32):
    g = torch.Generator(device="cpu").manual_seed(seed)
    p = torch.rand(nh, S, S, generator=g).tril()
    return (p / p.sum(-1, keepdim=True).clamp(min=1e-9)).to(dtype)


def make_decomp(nh, S, seed=0, scale=0.8):
    g = torch.Generator(device="cpu").manual_seed(seed)
    alpha = torch.randn(nh, S, generator=g) * scale
    rho = torch.randn(nh, S, generator=g) * scale
    return alpha, rho, O.decomposed_logz(alpha, rho)


def head_maps(H, frozen_states):
    """hidx for compact q/k (live heads keep their order)."""
    live = [h for h in range(H) if frozen_states[h] == 0]
    hidx = torch.zeros(H, dtype=torch.int32)
    for slot, h in enumerate(live):
        hidx[h] = slot
    return live, hidx


def errs(a, b):
    return O.max_abs(a.float().cpu(), b.float().cpu()), O.rel_l2(a.float().cpu(), b.float().cpu())
