"""Generates tests/golden/*.npz by RUNNING THE REFERENCE (its own Python/torch code on CPU).

    python tests/golden/make_golden.py /path/to/reference

Nothing under tests/ or in the library reads the reference at run time; these vectors are how the
reference's behaviour travels.  What is recorded:
  * layer level: the reference's CausalSelfAttention in dynamic mode (nanogpt/model.py), both the eager
    capture path (_attend_dynamic, :824-844) and the cheap split path (_attend_cheap, :1017-1061), fp32,
    RoPE, on the seeded inputs of tests/golden/cases.py -- including benchmark configuration 0;
  * op level: ref() and decomp_materialize() of kernel/test_fused_attn.py:40-63, ref_fwd() of
    kernel/test_frozen_attn.py:27-28, decomp_logits / decomposed_logz / make_rho_band of
    kernel/fused_attn.py:65-116, linear_rows / linear_rows2 / linear_permuted_cols of
    kernel/indexed_linear.py with their gradients, apply_rotary_pos_emb of nanogpt/model.py:63-68;
  * block level: the reference's LayerNorm and MLP modules (nanogpt/model.py:45-54, 1193-1207) on seeded inputs;
  * learnable patterns: dense_reference of supplement/trainable_patterns.py:7-13 with its autograd gradients;
  * controller statistics: _centered_batch_reduced_moments, _merge_reduced_moments, _negative_entropy_sum and
    _mean_forward_kl_from_entropy of nanogpt/dynamic_freeze.py:96-193 on two seeded batches of softmax attention;
    _centered_batch_moments and _merge_moments (:62-93) on the raw logits of the same batches.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def load_ref(ref_root):
    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, "nanogpt"))
    import model as ref_model  # noqa
    import kernel as ref_kernel  # noqa

    def load_file(name, path):
        spec = importlib.util.spec_from_file_location(name, path)
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        return m
    t_fused = load_file("ref_test_fused", os.path.join(ref_root, "kernel", "test_fused_attn.py"))
    t_frozen = load_file("ref_test_frozen", os.path.join(ref_root, "kernel", "test_frozen_attn.py"))
    return ref_model, ref_kernel, t_fused, t_frozen


def ref_layer(M, B, T, C, H, ws, repr_="dense"):
    cfg = M.GPTConfig(block_size=T, vocab_size=64, n_layer=1, n_head=H, n_embd=C, dropout=0.0, bias=False,
                      position_encoding="rope", rand_attn_dynamic=True, rand_attn_prior_repr=repr_,
                      freeze_pattern_dtype="float32")
    attn = M.CausalSelfAttention(cfg, layer_idx=0)
    with torch.no_grad():
        for lin, w in zip((attn.q_proj, attn.k_proj, attn.v_proj, attn.c_proj), ws):
            lin.weight.copy_(w)
    rope = M.RotaryEmbedding(C // H, T, base=10000.0)(T, torch.float32)
    return attn.eval(), rope


def main(ref_root):
    torch.manual_seed(0)
    torch.set_num_threads(8)
    M, K, TF, TZ = load_ref(ref_root)
    out = {}

    # ---- layer level --------------------------------------------------------------------------
    for name, (B, T, C, H, fz, seed, kind) in cases.LAYER_CASES.items():
        x, ws = cases.layer_inputs(B, T, C, H, seed)
        patt, _ = cases.layer_patterns(kind, len(fz), T, seed)
        attn, rope = ref_layer(M, B, T, C, H, ws)
        attn.freeze_heads(fz, patt)
        with torch.no_grad():
            y_cheap = attn(x, rope=rope)
            attn.set_capture(True)
            y_eager = attn(x, rope=rope)
            attn.set_capture(False)
        s, tot, atot = cases.sample(y_eager, 24, 24)
        out[f"layer_{name}_eager_sample"] = s.numpy()
        out[f"layer_{name}_eager_sums"] = np.array([tot, atot])
        s2, tot2, atot2 = cases.sample(y_cheap, 24, 24)
        out[f"layer_{name}_cheap_sample"] = s2.numpy()
        out[f"layer_{name}_cheap_sums"] = np.array([tot2, atot2])
        if name != "config0":
            out[f"layer_{name}_eager_full"] = y_eager.numpy()
        # the pattern as the reference stored it (after its tril + renormalise)
        ps, pt, pa = cases.sample(attn.dyn_pattern[fz, :T, :T], 24, 24)
        out[f"layer_{name}_stored_pattern_sample"] = ps.numpy()
        print(name, "cheap-vs-eager max|d| =", (y_cheap - y_eager).abs().max().item())

    name, B, T, C, H, dense, dec, seed = cases.DECOMP_LAYER
    x, ws = cases.layer_inputs(B, T, C, H, seed)
    attn, rope = ref_layer(M, B, T, C, H, ws, repr_="decomposed")
    al, rh = cases.decomp_vectors(len(dec), T, seed + 2)
    attn.freeze_heads_decomposed(dec, al, rh)
    attn.freeze_heads(dense, cases.random_pattern(len(dense), T, seed + 1))
    with torch.no_grad():
        attn.set_capture(True)
        y_eager = attn(x, rope=rope)
        attn.set_capture(False)
        y_cheap = attn(x, rope=rope)
    out[f"layer_{name}_eager_full"] = y_eager.numpy()
    out[f"layer_{name}_z"] = attn.dyn_z[dec].numpy()
    print(name, "cheap-vs-eager max|d| =", (y_cheap - y_eager).abs().max().item())

    # ---- op level -----------------------------------------------------------------------------
    B, H, T, hd, S = 2, 6, 150, 32, 192
    q, k, v = cases.op_inputs(B, H, T, hd, 21)
    patt = cases.random_pattern(H, S, 22)
    al, rh = cases.decomp_vectors(H, S, 23)
    z = K.decomposed_logz(al, rh)
    out["op_logz"] = z.numpy()
    out["op_logits_rows_10_14"] = K.decomp_logits(al, rh, rows=(10, 14)).numpy()
    out["op_rho_band_sample"] = K.make_rho_band(rh)[:, ::9, ::7].numpy()
    dense_heads, dec_heads = [1, 4], [2]
    ref_patt = patt.clone()
    ref_patt[dec_heads, :T, :T] = TF.decomp_materialize(al[dec_heads], rh[dec_heads], T, z=z[dec_heads])
    qq, kk, vv = [t.clone().requires_grad_(True) for t in (q, k, v)]
    y = TF.ref(qq, kk, vv, ref_patt, dense_heads + dec_heads, T)
    g = torch.Generator().manual_seed(24)
    w = torch.randn(y.shape, generator=g)
    (y * w).sum().backward()
    out["op_mixed_y"] = y.detach().numpy()
    out["op_mixed_dq"] = qq.grad.numpy()
    out["op_mixed_dk"] = kk.grad.numpy()
    out["op_mixed_dv"] = vv.grad.numpy()
    out["op_frozen_pv"] = TZ.ref_fwd(patt, v[:, [0, 3]], torch.tensor([1, 4]), T).numpy()
    # RoPE
    rope = M.RotaryEmbedding(hd, T, base=10000.0)(T, torch.float32)
    rq, rk = M.apply_rotary_pos_emb(q, k, *rope)
    out["op_rope_q"] = rq.numpy()
    out["op_rope_k"] = rk.numpy()
    # indexed linear (the reference's own autograd Functions, CPU)
    g = torch.Generator().manual_seed(25)
    C_, Hh, hd2 = 96, 4, 24
    x = torch.randn(3, 17, C_, generator=g)
    w1, w2 = torch.randn(C_, C_, generator=g) * 0.1, torch.randn(C_, C_, generator=g) * 0.1
    b1, b2 = torch.randn(C_, generator=g) * 0.1, torch.randn(C_, generator=g) * 0.1
    rows = (torch.tensor([0, 2, 3])[:, None] * hd2 + torch.arange(hd2)).reshape(-1)
    leaves = [t.clone().requires_grad_(True) for t in (x, w1, w2, b1, b2)]
    y2 = K.linear_rows2(*leaves, rows)
    wgt = torch.randn(y2.shape, generator=g)
    (y2 * wgt).sum().backward()
    out["lin_rows2_y"] = y2.detach().numpy()
    for nme, t in zip(("dx", "dw1", "dw2", "db1", "db2"), leaves):
        out[f"lin_rows2_{nme}"] = t.grad.numpy()
    out["lin_rows_y"] = K.linear_rows(x, w1, b1, rows).numpy()
    cols = torch.cat([rows, (torch.tensor([1])[:, None] * hd2 + torch.arange(hd2)).reshape(-1)])
    leaves = [t.clone().requires_grad_(True) for t in (x, w1, b1)]
    y3 = K.linear_permuted_cols(*leaves, cols)
    wgt = torch.randn(y3.shape, generator=g)
    (y3 * wgt).sum().backward()
    out["lin_pcols_y"] = y3.detach().numpy()
    for nme, t in zip(("dy", "dw", "db"), leaves):
        out[f"lin_pcols_{nme}"] = t.grad.numpy()

    # ---- rest of the block: the reference's LayerNorm and MLP modules (nanogpt/model.py:45-54, 1193-1207) ----
    g = torch.Generator().manual_seed(26)
    Cb = 96
    xb = torch.randn(2, 19, Cb, generator=g) * 1.5 + 0.3
    ln = M.LayerNorm(Cb, bias=True)
    cfgb = M.GPTConfig(block_size=32, vocab_size=64, n_layer=1, n_head=4, n_embd=Cb, dropout=0.0, bias=True)
    mlp = M.MLP(cfgb)
    with torch.no_grad():
        ln.weight.copy_(1 + 0.1 * torch.randn(Cb, generator=g))
        ln.bias.copy_(0.1 * torch.randn(Cb, generator=g))
        mlp.c_fc.weight.copy_(torch.randn(4 * Cb, Cb, generator=g) * 0.1)
        mlp.c_fc.bias.copy_(torch.randn(4 * Cb, generator=g) * 0.1)
        mlp.c_proj.weight.copy_(torch.randn(Cb, 4 * Cb, generator=g) * 0.1)
        mlp.c_proj.bias.copy_(torch.randn(Cb, generator=g) * 0.1)
        out["blk_x"] = xb.numpy()
        out["blk_ln_w"], out["blk_ln_b"] = ln.weight.numpy().copy(), ln.bias.numpy().copy()
        out["blk_ln_y"] = ln(xb).numpy()
        out["blk_fc_w"], out["blk_fc_b"] = mlp.c_fc.weight.numpy().copy(), mlp.c_fc.bias.numpy().copy()
        out["blk_pr_w"], out["blk_pr_b"] = mlp.c_proj.weight.numpy().copy(), mlp.c_proj.bias.numpy().copy()
        out["blk_mlp_y"] = mlp.eval()(xb).numpy()

    # ---- learnable decomposed patterns: dense_reference of supplement/trainable_patterns.py:7-13 and its autograd
    # gradients (what supplement/trainable_pattern_kernels.py:21-58 computes without the T x T buffer) ----
    spec = importlib.util.spec_from_file_location("ref_trainable_patterns",
                                                  os.path.join(ref_root, "supplement", "trainable_patterns.py"))
    TP = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(TP)
    g = torch.Generator().manual_seed(27)
    Bt, Ht, Tt, Dt, St = 2, 3, 40, 16, 64
    val = torch.randn(Bt, Ht, Tt, Dt, generator=g).requires_grad_(True)
    al = (torch.randn(Ht, St, generator=g) * 0.7).requires_grad_(True)
    rh = (-0.05 * torch.arange(St).float()[None, :] * torch.rand(Ht, 1, generator=g)
          + 0.3 * torch.randn(Ht, St, generator=g)).requires_grad_(True)
    wt = torch.randn(Bt, Ht, Tt, Dt, generator=g)
    yt = TP.dense_reference(val, al, rh)
    (yt * wt).sum().backward()
    out["tp_value"], out["tp_alpha"], out["tp_rho"], out["tp_w"] = (val.detach().numpy(), al.detach().numpy(),
                                                                      rh.detach().numpy(), wt.numpy())
    out["tp_out"] = yt.detach().numpy()
    out["tp_dvalue"], out["tp_dalpha"], out["tp_drho"] = val.grad.numpy(), al.grad.numpy(), rh.grad.numpy()

    # ---- controller statistics: the reference's own reductions of captured attention
    # (nanogpt/dynamic_freeze.py:96-193) on two seeded batches, merged with its Chan formula ----
    import dynamic_freeze as DF  # noqa: E402  (nanogpt/ is on sys.path)
    g = torch.Generator().manual_seed(28)
    Bs, Us, Ts, Ds = 3, 2, 40, 16
    count, mean, m2 = 0, None, None
    negent = torch.zeros(Us, dtype=torch.float64)
    for bi in range(2):
        qs = torch.randn(Bs, Us, Ts, Ds, generator=g)
        ks = torch.randn(Bs, Us, Ts, Ds, generator=g)
        sc = (qs @ ks.transpose(-1, -2)) / Ds ** 0.5
        att = sc.masked_fill(~torch.ones(Ts, Ts, dtype=torch.bool).tril(), float("-inf")).softmax(-1)
        bn, bm, b2 = DF._centered_batch_reduced_moments(att)
        count, mean, m2 = DF._merge_reduced_moments(count, mean, m2, bn, bm, b2)
        negent += DF._negative_entropy_sum(att)
        out[f"st_q{bi}"], out[f"st_k{bi}"] = qs.numpy(), ks.numpy()
        out[f"st_mean{bi}"], out[f"st_m2_{bi}"], out[f"st_negent{bi}"] = mean.numpy().copy(), m2.numpy().copy(), negent.numpy().copy()
    out["st_kl"] = DF._mean_forward_kl_from_entropy(negent, mean.float(), count).numpy()

    # ---- per-cell statistics of the raw logits (the tensor model.py:828-831 retains as `_last_logits`), reduced with
    # the reference's _centered_batch_moments / _merge_moments as _measure does (nanogpt/dynamic_freeze.py:721-727) ----
    lcount, lmean, lm2 = 0, None, None
    for bi in range(2):
        qs, ks = torch.from_numpy(out[f"st_q{bi}"]), torch.from_numpy(out[f"st_k{bi}"])
        lg = (qs @ ks.transpose(-2, -1)) * (1.0 / Ds ** 0.5)
        lbn, lbm, lb2 = DF._centered_batch_moments(lg)
        lcount, lmean, lm2 = DF._merge_moments(lcount, lmean, lm2, lbn, lbm, lb2)
        out[f"lg_mean{bi}"], out[f"lg_m2_{bi}"] = lmean.numpy().copy(), lm2.numpy().copy()

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB,", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
