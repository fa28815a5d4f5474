"""GPU parity of the learnable-pattern gradients (normalisers, PatternGradient, fused_mixed_attn with
alpha / rho that require grad) against the CPU oracle and the reference's golden vectors.
The reference has no test for supplement/trainable_pattern_kernels.py; its dense_reference
(supplement/trainable_patterns.py:7-13) with autograd is the definition."""
import os

import numpy as np
import pytest
import torch

from oracle import saf_oracle as O
from tests.util import errs

pytestmark = pytest.mark.gpu

_G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))


def g(name):
    return torch.from_numpy(_G[name])


def _vectors(H, S, seed, slope=0.02):
    gen = torch.Generator().manual_seed(seed)
    al = torch.randn(H, S, generator=gen) * 0.7
    rh = -slope * torch.arange(S).float()[None, :] * torch.rand(H, 1, generator=gen) + 0.3 * torch.randn(H, S, generator=gen)
    return al, rh


def test_normalisers_match_reference_definition():
    from saf_b200.trainable_patterns import normalisers
    al, rh = g("tp_alpha"), g("tp_rho")
    z = normalisers(al.cuda(), rh.cuda(), 40).cpu()
    assert O.max_abs(z, O.pattern_normalisers(al, rh, 40)) <= 2e-6
    assert torch.equal(z[:, 40:], torch.zeros_like(z[:, 40:]))


def test_pattern_gradient_golden_fp32():
    """PatternGradient on the reference's own vectors: gradients equal autograd through dense_reference."""
    from saf_b200.trainable_patterns import normalisers, PatternGradient
    val, al, rh, w, y = [g(n).cuda() for n in ("tp_value", "tp_alpha", "tp_rho", "tp_w", "tp_out")]
    al.requires_grad_(True)
    rh.requires_grad_(True)
    z = normalisers(al, rh, val.shape[-2])
    states = torch.full((al.shape[0],), 2, dtype=torch.int32, device="cuda")
    out = PatternGradient.apply(y.clone().requires_grad_(True), val, al, rh, z, states)
    (out * w).sum().backward()
    assert O.max_abs(al.grad.cpu(), g("tp_dalpha")) <= 2e-5
    assert O.max_abs(rh.grad.cpu(), g("tp_drho")) <= 2e-5


CASES = [
    # B, H, T, hd, S, states
    (2, 4, 300, 64, 320, [2, 0, 2, 1]),
    (1, 3, 1024, 128, 1024, [2, 2, 0]),
    (3, 2, 517, 64, 576, [2, 2]),
    (2, 3, 200, 32, 256, [0, 2, 2]),        # head_dim without a tensor-core kernel
    (1, 2, 2048, 64, 2048, [2, 2]),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: f"B{c[0]}H{c[1]}T{c[2]}d{c[3]}")
def test_fused_mixed_attn_trains_alpha_rho(case, dtype):
    """alpha / rho that require grad get the exact softmax-parameter gradients through fused_mixed_attn;
    v, q, k gradients are unchanged; heads in other states contribute nothing."""
    from kernel import fused_mixed_attn
    B, H, T, hd, S, states = case
    dev = "cuda"
    gen = torch.Generator().manual_seed(T + hd)
    live = [h for h in range(H) if states[h] == 0]
    hidx = [0] * H
    for i, h in enumerate(live):
        hidx[h] = i
    q = torch.randn(B, len(live), T, hd, generator=gen).to(dtype)
    k = torch.randn(B, len(live), T, hd, generator=gen).to(dtype)
    v = torch.randn(B, H, T, hd, generator=gen).to(dtype)
    w = torch.randn(B, H, T, hd, generator=gen)
    patt = torch.rand(H, S, S, generator=gen).tril()
    patt = patt / patt.sum(-1, keepdim=True)
    al, rh = _vectors(H, S, T)
    # oracle in fp64 on the same (rounded) inputs
    z = O.pattern_normalisers(al.double(), rh.double(), T)
    vr = v.double().requires_grad_(True)
    y_ref = O.mixed_attn(q.double(), k.double(), vr, patt.double(), states, hidx=torch.tensor(hidx),
                         alpha=al.double(), rho=rh.double(), z=z)
    da_ref, dr_ref = O.pattern_param_grads(v.double(), y_ref.detach(), w.double(), al.double(), rh.double(), z, states)
    (y_ref * w.double()).sum().backward()

    ad = al.to(dev).requires_grad_(True)
    rd = rh.to(dev).requires_grad_(True)
    vd = v.to(dev).requires_grad_(True)
    y = fused_mixed_attn(q.to(dev), k.to(dev), vd, patt.to(dev).to(dtype), torch.tensor(states, dtype=torch.int32, device=dev),
                         torch.tensor(hidx, dtype=torch.int32, device=dev), alpha=ad, rho=rd)
    fa, fr = errs(y, y_ref)
    (y.float() * w.to(dev)).sum().backward()
    if dtype == torch.float32:
        assert fa <= 2e-5, f"fwd {fa}"
        tol = 2e-4 * max(1.0, da_ref.abs().max().item())
        assert O.max_abs(ad.grad.cpu().double(), da_ref) <= tol
        assert O.max_abs(rd.grad.cpu().double(), dr_ref) <= 2e-4 * max(1.0, dr_ref.abs().max().item())
        assert errs(vd.grad, vr.grad)[0] <= 2e-4
    else:
        assert fa <= 2e-2 and fr <= 1e-2, f"fwd {fa} {fr}"
        # the saved output and dO are bf16: bound by magnitude, and by rel-L2
        for got, ref, name in ((ad.grad, da_ref, "dalpha"), (rd.grad, dr_ref, "drho")):
            a, r = errs(got, ref)
            assert a <= 2e-2 * max(1.0, ref.abs().max().item()) and r <= 2e-2, f"{name} {a} {r}"
    for h in range(H):
        if states[h] != 2:
            assert not ad.grad[h].any() and not rd.grad[h].any()
    assert not ad.grad[:, T:].any() and not rd.grad[:, T:].any()


def test_enable_turns_buffers_into_parameters_and_trains():
    """saf_b200.trainable_patterns.enable on an attention module: dyn_alpha / dyn_rho become parameters,
    a training step changes them, and the state dict carries refreshed normalisers."""
    from saf_b200.attention import SafCausalSelfAttention as SafAttention, rope_tables
    from saf_b200.trainable_patterns import enable, normalisers
    from types import SimpleNamespace
    cfg = SimpleNamespace(n_embd=256, n_head=4, block_size=256, bias=False, dropout=0.0, position_encoding="rope",
                          rand_attn_prior_repr="decomposed", freeze_pattern_dtype="float32")
    attn = SafAttention(cfg).cuda()
    al, rh = _vectors(2, 256, 5)
    attn.freeze_heads_decomposed([1, 3], al.cuda(), rh.cuda())
    opt = torch.optim.SGD([p for p in attn.parameters()], lr=0.1)
    params = enable(attn, opt)
    assert len(params) == 2 and isinstance(attn.dyn_alpha, torch.nn.Parameter)
    x = torch.randn(2, 256, 256, device="cuda")
    cos, sin = rope_tables(64, 256, device="cuda")
    rope = (cos.view(1, 1, 256, -1), sin.view(1, 1, 256, -1))
    before = attn.dyn_alpha.detach().clone()
    attn(x, rope=rope).square().mean().backward()
    assert attn.dyn_alpha.grad is not None and attn.dyn_alpha.grad[1].abs().sum() > 0
    assert not attn.dyn_alpha.grad[0].any()
    opt.step()
    assert not torch.equal(before, attn.dyn_alpha.detach())
    sd = attn.state_dict()
    zz = normalisers(attn.dyn_alpha, attn.dyn_rho, 256)
    assert torch.allclose(sd["dyn_z"][[1, 3]].float(), zz[[1, 3]].float(), atol=1e-5)


@pytest.mark.parametrize("T", [1, 37, 129])
def test_pattern_param_grad_small_and_ragged(T):
    """Tiny and ragged sequences on the tensor-core path (bf16, head_dim 64) against the closed form."""
    from saf_b200.trainable_patterns import normalisers, pattern_param_grad
    B, H, hd, S = 2, 2, 64, 192
    gen = torch.Generator().manual_seed(T)
    v = torch.randn(B, H, T, hd, generator=gen).bfloat16()
    w = torch.randn(B, H, T, hd, generator=gen).bfloat16()
    al, rh = _vectors(H, S, T + 1)
    z = O.pattern_normalisers(al.double(), rh.double(), T)
    y = torch.matmul(O.decomp_pattern(al.double(), rh.double(), z, T)[None], v.double()).bfloat16()
    da_ref, dr_ref = O.pattern_param_grads(v.double(), y.double(), w.double(), al.double(), rh.double(), z)
    states = torch.full((H,), 2, dtype=torch.int32, device="cuda")
    zd = normalisers(al.cuda(), rh.cuda(), T)
    da, dr = pattern_param_grad(w.cuda(), y.cuda(), v.cuda(), al.cuda(), rh.cuda(), zd, states)
    for got, ref in ((da, da_ref), (dr, dr_ref)):
        a, _ = errs(got, ref)
        assert a <= 2e-2 * max(1.0, ref.abs().max().item()), a
    assert not da[:, T:].any() and not dr[:, T:].any()


def test_pattern_param_grad_without_training_heads_is_zero_and_launches_nothing():
    from saf_b200 import launch_count
    from saf_b200.trainable_patterns import pattern_param_grad
    B, H, T, hd, S = 1, 3, 64, 64, 64
    v = torch.randn(B, H, T, hd, device="cuda").bfloat16()
    al, rh = _vectors(H, S, 9)
    states = torch.tensor([0, 1, 3], dtype=torch.int32, device="cuda")
    n0 = launch_count()
    da, dr = pattern_param_grad(v, v, v, al.cuda(), rh.cuda(), torch.zeros(H, S, device="cuda"), states)
    assert launch_count() == n0
    assert not da.any() and not dr.any()
