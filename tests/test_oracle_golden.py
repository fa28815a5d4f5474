"""Pins the CPU oracle to the reference: every oracle function against vectors produced by running the
reference's own code (tests/golden/make_golden.py).  Runs without a GPU."""
import os

import numpy as np
import pytest
import torch

from oracle import saf_oracle as O
from tests.golden import cases

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))


def g(name):
    return torch.from_numpy(G[name])


def oracle_layer(name):
    B, T, C, H, fz, seed, kind = cases.LAYER_CASES[name]
    x, ws = cases.layer_inputs(B, T, C, H, seed)
    patt, _ = cases.layer_patterns(kind, len(fz), T, seed)
    full = torch.zeros(H, T, T)
    full[fz] = O.freeze_normalise(patt)
    states = [1 if h in fz else 0 for h in range(H)]
    rope = O.rope_cache(C // H, T)
    return O.attention_layer(x, *ws, states, full, H, rope=rope), (B, T, C, H, fz, seed, kind)


@pytest.mark.parametrize("name", ["small_sink", "small_rand"])
def test_layer_small_full(name):
    y, _ = oracle_layer(name)
    assert O.max_abs(y, g(f"layer_{name}_eager_full")) <= 2e-6


def test_layer_config0_sample_and_checksums():
    """Benchmark configuration 0, as the reference computes it (fp32, B=2, T=1024, 12 heads, {2,5,8} frozen)."""
    y, _ = oracle_layer("config0")
    s, tot, atot = cases.sample(y, 24, 24)
    assert O.max_abs(s, g("layer_config0_eager_sample")) <= 5e-6
    assert O.max_abs(s, g("layer_config0_cheap_sample")) <= 5e-6
    ref_tot, ref_atot = G["layer_config0_eager_sums"]
    assert abs(atot - ref_atot) / ref_atot <= 1e-5


def test_layer_decomposed():
    name, B, T, C, H, dense, dec, seed = cases.DECOMP_LAYER
    x, ws = cases.layer_inputs(B, T, C, H, seed)
    al, rh = cases.decomp_vectors(len(dec), T, seed + 2)
    patt = torch.zeros(H, T, T)
    patt[dense] = O.freeze_normalise(cases.random_pattern(len(dense), T, seed + 1))
    alpha, rho = torch.zeros(H, T), torch.zeros(H, T)
    alpha[dec], rho[dec] = al, rh
    z = O.decomposed_logz(alpha, rho)
    assert O.max_abs(z[dec], g(f"layer_{name}_z")) <= 2e-6
    states = [0] * H
    for h in dense:
        states[h] = 1
    for h in dec:
        states[h] = 2
    y = O.attention_layer(x, *ws, states, patt, H, rope=O.rope_cache(C // H, T), alpha=alpha, rho=rho, z=z)
    assert O.max_abs(y, g(f"layer_{name}_eager_full")) <= 2e-6


def test_op_helpers():
    H, S = 6, 192
    al, rh = cases.decomp_vectors(H, S, 23)
    assert O.max_abs(O.decomposed_logz(al, rh), g("op_logz")) <= 2e-6
    assert torch.equal(O.decomp_logits(al, rh, rows=(10, 14)), g("op_logits_rows_10_14"))
    assert torch.equal(O.make_rho_band(rh)[:, ::9, ::7], g("op_rho_band_sample"))


def test_op_mixed_forward_backward():
    B, H, T, hd, S = 2, 6, 150, 32, 192
    q, k, v = cases.op_inputs(B, H, T, hd, 21)
    patt = cases.random_pattern(H, S, 22)
    al, rh = cases.decomp_vectors(H, S, 23)
    z = O.decomposed_logz(al, rh)
    states = [0, 1, 2, 0, 1, 0]
    live = [0, 3, 5]
    hidx = torch.tensor([0, 0, 0, 1, 0, 2])
    qq, kk, vv = [t.clone().requires_grad_(True) for t in (q, k, v)]
    y = O.mixed_attn(qq[:, live], kk[:, live], vv, patt, states, hidx=hidx, alpha=al, rho=rh, z=z)
    assert O.max_abs(y, g("op_mixed_y")) <= 2e-6
    w = torch.randn(y.shape, generator=torch.Generator().manual_seed(24))
    (y * w).sum().backward()
    assert O.max_abs(qq.grad, g("op_mixed_dq")) <= 2e-5
    assert O.max_abs(kk.grad, g("op_mixed_dk")) <= 2e-5
    assert O.max_abs(vv.grad, g("op_mixed_dv")) <= 2e-5
    assert O.max_abs(O.frozen_pv(patt, v[:, [0, 3]], [1, 4], T), g("op_frozen_pv")) <= 2e-6


def test_op_rope():
    B, H, T, hd = 2, 6, 150, 32
    q, k, _ = cases.op_inputs(B, H, T, hd, 21)
    cos, sin = O.rope_cache(hd, T)
    assert torch.equal(O.apply_rope(q, cos, sin), g("op_rope_q"))
    assert torch.equal(O.apply_rope(k, cos, sin), g("op_rope_k"))


def test_indexed_linear():
    gen = torch.Generator().manual_seed(25)
    C_, hd2 = 96, 24
    x = torch.randn(3, 17, C_, generator=gen)
    w1, w2 = torch.randn(C_, C_, generator=gen) * 0.1, torch.randn(C_, C_, generator=gen) * 0.1
    b1, b2 = torch.randn(C_, generator=gen) * 0.1, torch.randn(C_, generator=gen) * 0.1
    rows = (torch.tensor([0, 2, 3])[:, None] * hd2 + torch.arange(hd2)).reshape(-1)
    leaves = [t.clone().requires_grad_(True) for t in (x, w1, w2, b1, b2)]
    y = O.linear_rows2(*leaves, rows)
    assert O.max_abs(y, g("lin_rows2_y")) <= 1e-6
    wgt = torch.randn(y.shape, generator=gen)
    (y * wgt).sum().backward()
    for nme, t in zip(("dx", "dw1", "dw2", "db1", "db2"), leaves):
        assert O.max_abs(t.grad, g(f"lin_rows2_{nme}")) <= 2e-5, nme
    dead = (torch.tensor([1])[:, None] * hd2 + torch.arange(hd2)).reshape(-1)
    assert leaves[1].grad[dead].abs().max().item() == 0.0 and g("lin_rows2_dw1")[dead].abs().max().item() == 0.0
    assert O.max_abs(O.linear_rows(x, w1, b1, rows), g("lin_rows_y")) <= 1e-6
    cols = torch.cat([rows, dead])
    leaves = [t.clone().requires_grad_(True) for t in (x, w1, b1)]
    y3 = O.linear_permuted_cols(*leaves, cols)
    assert O.max_abs(y3, g("lin_pcols_y")) <= 1e-6
    wgt = torch.randn(y3.shape, generator=gen)
    (y3 * wgt).sum().backward()
    for nme, t in zip(("dy", "dw", "db"), leaves):
        assert O.max_abs(t.grad, g(f"lin_pcols_{nme}")) <= 2e-5, nme


def test_scan_identity_equals_dense_product():
    a, r = O.sink_decay_params(2, seed=5)
    T = 300
    v = torch.randn(T, 8, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    P = O.sink_decay_pattern(a, r, T)
    for i in range(2):
        assert O.max_abs(O.sink_decay_scan(v, a[i].item(), r[i].item()), P[i] @ v) <= 1e-12
    assert (P.sum(-1) - 1).abs().max().item() <= 1e-12


def test_block_functions_match_reference_modules():
    """layer_norm / mlp of the oracle against the reference's LayerNorm and MLP modules run on the same inputs."""
    t = lambda k: torch.from_numpy(G[k])
    y = O.layer_norm(t("blk_x"), t("blk_ln_w"), t("blk_ln_b"))
    assert O.max_abs(y, t("blk_ln_y")) <= 1e-6
    y = O.mlp(t("blk_x"), t("blk_fc_w"), t("blk_pr_w"), t("blk_fc_b"), t("blk_pr_b"))
    assert O.max_abs(y, t("blk_mlp_y")) <= 1e-6


def test_trainable_pattern_gradients():
    """The closed-form parameter gradients equal autograd through the reference's dense_reference
    (supplement/trainable_patterns.py:7-13), and the restated forward equals its output."""
    val, al, rh, w = g("tp_value"), g("tp_alpha"), g("tp_rho"), g("tp_w")
    T = val.shape[-2]
    y = O.pattern_dense_reference(val, al, rh)
    assert O.max_abs(y, g("tp_out")) <= 2e-6
    z = O.pattern_normalisers(al, rh, T)
    assert torch.equal(z[:, T:], torch.zeros_like(z[:, T:]))
    da, dr = O.pattern_param_grads(val, y, w, al, rh, z)
    assert O.max_abs(da, g("tp_dalpha")) <= 2e-5
    assert O.max_abs(dr, g("tp_drho")) <= 2e-5
    # heads outside state 2 contribute nothing
    da2, dr2 = O.pattern_param_grads(val, y, w, al, rh, z, states=[2, 0, 2])
    assert torch.equal(da2[1], torch.zeros_like(da2[1])) and O.max_abs(da2[0], g("tp_dalpha")[0]) <= 2e-5
    # dV of these heads is the ordinary frozen-head backward: P^T dO
    P = O.decomp_pattern(al, rh, z, T)
    assert O.max_abs(torch.matmul(P.transpose(-1, -2)[None], w), g("tp_dvalue")) <= 2e-5


def test_controller_statistics():
    """Restated capture reductions equal the reference's own (nanogpt/dynamic_freeze.py:96-193) on two merged batches."""
    count, mean, m2 = 0, None, None
    negent = torch.zeros(2, dtype=torch.float64)
    for bi in range(2):
        att = O.attention_probs(g(f"st_q{bi}"), g(f"st_k{bi}"))
        bn, bm, b2 = O.centered_batch_reduced_moments(att)
        count, mean, m2 = O.merge_reduced_moments(count, mean, m2, bn, bm, b2)
        negent += O.negative_entropy_sum(att)
        assert O.max_abs(mean, g(f"st_mean{bi}")) <= 1e-6
        assert O.max_abs(m2, g(f"st_m2_{bi}")) <= 1e-5
        assert O.max_abs(negent, g(f"st_negent{bi}")) <= 1e-4
    assert O.max_abs(O.mean_forward_kl(negent, mean.float(), count), g("st_kl")) <= 1e-5


def test_logit_statistics():
    """Per-cell moments of the raw logits, merged over two batches, equal the reference's _centered_batch_moments /
    _merge_moments (nanogpt/dynamic_freeze.py:62-93, used at :721-727)."""
    count, mean, m2 = 0, None, None
    for bi in range(2):
        lg = O.raw_logits(g(f"st_q{bi}"), g(f"st_k{bi}"))
        bn, bm, b2 = O.centered_batch_moments(lg)
        count, mean, m2 = O.merge_moments(count, mean, m2, bn, bm, b2)
        assert O.max_abs(mean, g(f"lg_mean{bi}")) <= 1e-6
        assert O.max_abs(m2, g(f"lg_m2_{bi}")) <= 1e-5
    assert count == 6


# ---- grouped-query variant: vectors from the reference's own Qwen3 hybrid attention module (split torch path) ----
GQ = np.load(os.path.join(os.path.dirname(__file__), "golden", "gqa_vectors.npz"))


def gq(case, name):
    return torch.from_numpy(GQ[f"gqa_{case}_{name}"])


def gqa_prior(case):
    if case == "dense":
        return dict(patt=gq(case, "patt"))
    return dict(patt=None, alpha=gq(case, "alpha"), rho=gq(case, "rho"), z=gq(case, "z"))


@pytest.mark.parametrize("case", ["dense", "decomp"])
def test_gqa_operator_matches_reference_module(case):
    """mixed_attn(kvidx=) on the exact q, k, v the reference module hands to its fused call, then its o_proj,
    equals the module's own (split torch path) output."""
    pr = gqa_prior(case)
    y = O.mixed_attn(gq(case, "q"), gq(case, "k"), gq(case, "v"), pr.pop("patt"), gq(case, "frozen_mask_i32"),
                     hidx=gq(case, "hidx_i32"), pidx=gq(case, "pidx_i32"), kvidx=gq(case, "kvidx_i32"),
                     sm_scale=float(GQ[f"gqa_{case}_scaling"][0]), **pr)
    B, H, T, hd = y.shape
    out = y.transpose(1, 2).reshape(B, T, H * hd) @ gq(case, "wo").t()
    assert O.max_abs(out, gq(case, "y")) <= 2e-6
    # sampled rows give the same numbers as the full evaluation
    rows = torch.tensor([0, 1, 37, 63, 64, 99])
    pr = gqa_prior(case)
    ys = O.mixed_attn(gq(case, "q"), gq(case, "k"), gq(case, "v"), pr.pop("patt"), gq(case, "frozen_mask_i32"),
                      hidx=gq(case, "hidx_i32"), pidx=gq(case, "pidx_i32"), kvidx=gq(case, "kvidx_i32"),
                      sm_scale=float(GQ[f"gqa_{case}_scaling"][0]), rows=rows, **pr)
    assert O.max_abs(ys, y[:, :, rows]) <= 1e-6


@pytest.mark.parametrize("case", ["dense", "decomp"])
def test_gqa_layer_matches_reference_module(case):
    """The whole layer restated (projections, per-head RMSNorm, RoPE base 1e6, kvidx attention, o_proj)."""
    pr = gqa_prior(case)
    y = O.gqa_attention_layer(gq(case, "x"), gq(case, "wq_std"), gq(case, "wk"), gq(case, "wv"), gq(case, "wo"),
                              gq(case, "frozen_mask_i32"), gq(case, "hidx_i32"), gq(case, "pidx_i32"),
                              gq(case, "kvidx_i32"), pr.pop("patt"), gq(case, "cos"), gq(case, "sin"),
                              float(GQ[f"gqa_{case}_scaling"][0]), q_norm_w=gq(case, "q_norm"),
                              k_norm_w=gq(case, "k_norm"), eps=float(GQ[f"gqa_{case}_eps"][0]), **pr)
    assert O.max_abs(y, gq(case, "y")) <= 3e-6


def test_sampled_rows_and_structured_state_match_full_evaluation():
    """rows= and state 3 (pattern rows produced on the fly) agree with the dense state-1 evaluation that the
    reference-generated layer vectors pin."""
    B, H, T, hd = 1, 4, 150, 16
    gq_ = torch.Generator().manual_seed(5)
    q, k, v = [torch.randn(B, H, T, hd, generator=gq_) for _ in range(3)]
    a, r = O.sink_decay_params(H, 9)
    patt = O.sink_decay_pattern(a, r, T).float()
    full = O.mixed_attn(q, k, v, patt, [0, 1, 0, 1])
    struct = O.mixed_attn(q, k, v, None, [0, 3, 0, 3], sink_decay=(a, r))
    assert O.max_abs(struct, full) <= 1e-6
    rows = torch.tensor([0, 5, 64, 127, 128, 149])
    assert O.max_abs(O.mixed_attn(q, k, v, None, [0, 3, 0, 3], sink_decay=(a, r), rows=rows), full[:, :, rows]) <= 1e-6
