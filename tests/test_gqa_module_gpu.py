"""The grouped-query module (Qwen-shaped) on the GPU:
  * on the inputs and weights of the reference's own Qwen3 hybrid attention module (tests/golden/gqa_vectors.npz,
    produced by running that module's split torch path) against that module's outputs, fp32;
  * in bf16 at 12 query / 2 KV heads x 128 against the oracle's restatement of the layer (pinned by those vectors);
  * RMSNorm, the gated-MLP GEMM epilogue and the whole block against plain torch fp32 arithmetic.
Bars: fp32 1e-4 end to end; bf16 max-abs <= 2e-2 and rel-L2 <= 1e-2 against fp32."""
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from oracle import saf_oracle as O
from tests.util import errs

pytestmark = pytest.mark.gpu
GQ = np.load(os.path.join(os.path.dirname(__file__), "golden", "gqa_vectors.npz"))


def gq(case, name):
    return torch.from_numpy(GQ[f"gqa_{case}_{name}"])


@pytest.mark.parametrize("case", ["dense", "decomp"])
def test_module_reproduces_the_reference_qwen3_module(case):
    from saf_b200.gqa import SafGqaAttention
    H, HKV, hd, C, T, S, B = [int(v) for v in GQ["dims"]]
    cfg = SimpleNamespace(hidden_size=C, num_attention_heads=H, num_key_value_heads=HKV, head_dim=hd, attention_bias=False,
                          qk_norm=True, rms_norm_eps=float(GQ[f"gqa_{case}_eps"][0]))
    m = SafGqaAttention(cfg)
    frozen = gq(case, "frozen_mask_i32").tolist()
    live = [h for h in range(H) if frozen[h] == 0]
    fz = [h for h in range(H) if frozen[h] != 0]
    with torch.no_grad():
        m.q_proj.weight.zero_()
        wq_std = gq(case, "wq_std").view(len(live), hd, C)
        for slot, h in enumerate(live):          # the reference keeps only these rows (its shrunken q_proj_std)
            m.q_proj.weight[h * hd:(h + 1) * hd] = wq_std[slot]
        m.k_proj.weight.copy_(gq(case, "wk"))
        m.v_proj.weight.copy_(gq(case, "wv"))
        m.o_proj.weight.copy_(gq(case, "wo"))
        m.q_norm.weight.copy_(gq(case, "q_norm"))
        m.k_norm.weight.copy_(gq(case, "k_norm"))
    m = m.cuda().eval()
    if case == "dense":
        m.set_frozen(dense=fz, patterns=gq(case, "patt"))
    else:
        m.set_frozen(decomposed=fz, decomp=(gq(case, "alpha"), gq(case, "rho")))
    assert abs(m.scaling - float(GQ[f"gqa_{case}_scaling"][0])) < 1e-7
    assert torch.equal(m.kvidx_i32.cpu(), gq(case, "kvidx_i32")) and torch.equal(m.hidx_i32.cpu(), gq(case, "hidx_i32"))
    with torch.inference_mode():
        y = m(gq(case, "x").cuda(), (gq(case, "cos").cuda(), gq(case, "sin").cuda()))
    assert O.max_abs(y.cpu(), gq(case, "y")) <= 1e-4


def test_bf16_layer_at_qwen_shapes_against_the_oracle():
    from saf_b200.gqa import SafGqaAttention
    from saf_b200.attention import rope_tables
    H, HKV, hd, C, T, B = 12, 2, 128, 1536, 1024, 2
    cfg = SimpleNamespace(hidden_size=C, num_attention_heads=H, num_key_value_heads=HKV, head_dim=hd, attention_bias=True,
                          qk_norm=False)
    g = torch.Generator().manual_seed(3)
    m = SafGqaAttention(cfg)
    with torch.no_grad():
        for n, p in m.named_parameters():
            p.copy_(torch.randn(p.shape, generator=g) * (0.02 if p.dim() == 2 else 0.1))
    m = m.cuda().bfloat16().eval()
    dense, sd_heads = [4], [1, 9]
    p = torch.rand(1, T, T, generator=g).tril()
    a, r = O.sink_decay_params(2, 77)
    m.set_frozen(dense=dense, patterns=p, sink_decay=sd_heads, sd_params=(a.tolist(), r.tolist()))
    x = torch.randn(B, T, C, generator=g).bfloat16()
    res = torch.randn(B, T, C, generator=g).bfloat16()
    cos, sin = rope_tables(hd, T, base=1e6, device="cuda")
    with torch.inference_mode():
        y = m(x.cuda(), (cos, sin), residual=res.cuda())
    # oracle on the same bf16-rounded weights; biases enter as an extra input column of ones
    wf = {n: t.detach().float().cpu() for n, t in m.named_parameters()}
    live = m._live
    rows = (torch.tensor(live)[:, None] * hd + torch.arange(hd)).reshape(-1)
    xb = torch.cat([x.float(), torch.ones(B, T, 1)], -1)
    wq = torch.cat([wf["q_proj.weight"][rows], wf["q_proj.bias"][rows, None]], 1)
    wk = torch.cat([wf["k_proj.weight"], wf["k_proj.bias"][:, None]], 1)
    wv = torch.cat([wf["v_proj.weight"], wf["v_proj.bias"][:, None]], 1)
    sd_full = (torch.zeros(H, dtype=torch.float64), torch.zeros(H, dtype=torch.float64))
    for h, aa, rr in zip(sd_heads, a.float().double(), r.float().double()):
        sd_full[0][h], sd_full[1][h] = aa, rr
    oc, os_ = O.rope_cache(hd, T, base=1e6)
    ref = O.gqa_attention_layer(xb, wq, wk, wv, wf["o_proj.weight"], m.frozen_mask_i32.cpu(), m.hidx_i32.cpu(),
                                m.pidx_i32.cpu(), m.kvidx_i32.cpu(), m.prior_pattern.float().cpu(), oc, os_, m.scaling,
                                sink_decay=sd_full) + res.float()
    a_, r_ = errs(y, ref)
    assert a_ <= 2e-2 and r_ <= 1e-2, (a_, r_)


def test_rmsnorm_and_gated_mlp_epilogue():
    from saf_b200 import ops
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(3, 70, 1536, generator=g) * 1.5 + 0.2).bfloat16()
    w = (1 + 0.1 * torch.randn(1536, generator=g)).bfloat16()
    y = ops.rms_norm(x.cuda(), w.cuda(), 1e-6)
    xf = x.float()
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    a, r = errs(y, ref)
    assert r <= 4e-3 and a <= 4e-2      # one bf16 rounding of the result
    # gated MLP: silu(x Wg^T) * (x Wu^T) in one launch, odd tile counts and a ragged last row tile
    # (8300 rows take the CTA-pair tiles)
    for M, C, N in ((300, 256, 384), (1000, 1536, 8960), (8300, 256, 640)):
        xx = torch.randn(M, C, generator=g).bfloat16()
        wg = (torch.randn(N, C, generator=g) * 0.05).bfloat16()
        wu = (torch.randn(N, C, generator=g) * 0.05).bfloat16()
        h = ops.linear_swiglu(xx.cuda(), wg.cuda(), wu.cuda())
        ref = torch.nn.functional.silu(xx.float() @ wg.float().t()) * (xx.float() @ wu.float().t())
        a, r = errs(h, ref)
        assert r <= 6e-3, (M, C, N, r)


def test_whole_block_against_fp32_torch():
    from saf_b200.gqa import build_gqa_stack
    layers, rope, w = build_gqa_stack("tiny_gqa", "cuda", blocks=True, n_layer=1)
    blk = layers[0]
    B, T, C = 2, w["T"], w["hidden"]
    g = torch.Generator().manual_seed(6)
    x = torch.randn(B, T, C, generator=g).bfloat16()
    with torch.inference_mode():
        y = blk(x.cuda(), rope)
    # fp32 restatement of the block on the bf16-rounded weights
    wf = {n: t.detach().float().cpu() for n, t in blk.named_parameters()}
    at = blk.self_attn
    H, hd = at.n_head, at.head_dim

    def rms(t, wt):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * wt
    xf = x.float()
    h1 = rms(xf, wf["input_layernorm.weight"])
    rows = (torch.tensor(at._live)[:, None] * hd + torch.arange(hd)).reshape(-1)
    hb = torch.cat([h1, torch.ones(B, T, 1)], -1)
    wq = torch.cat([wf["self_attn.q_proj.weight"][rows], wf["self_attn.q_proj.bias"][rows, None]], 1)
    wk = torch.cat([wf["self_attn.k_proj.weight"], wf["self_attn.k_proj.bias"][:, None]], 1)
    wv = torch.cat([wf["self_attn.v_proj.weight"], wf["self_attn.v_proj.bias"][:, None]], 1)
    oc, os_ = O.rope_cache(hd, T, base=w["rope_base"])
    attn = O.gqa_attention_layer(hb, wq, wk, wv, wf["self_attn.o_proj.weight"], at.frozen_mask_i32.cpu(),
                                 at.hidx_i32.cpu(), at.pidx_i32.cpu(), at.kvidx_i32.cpu(), None, oc, os_, at.scaling,
                                 sink_decay=(at.sd_alpha.double().cpu(), at.sd_rho.double().cpu()))
    x1 = xf + attn
    h2 = rms(x1, wf["post_attention_layernorm.weight"])
    mlp = (torch.nn.functional.silu(h2 @ wf["mlp.gate_proj.weight"].t()) * (h2 @ wf["mlp.up_proj.weight"].t())) \
        @ wf["mlp.down_proj.weight"].t()
    ref = x1 + mlp
    a, r = errs(y, ref)
    assert r <= 1e-2 and a <= 6e-2, (a, r)     # residual stream of magnitude ~1 carried in bf16


def test_training_is_refused_like_the_reference():
    from saf_b200.gqa import build_gqa_stack
    layers, rope, w = build_gqa_stack("tiny_gqa", "cuda", n_layer=1)
    x = torch.randn(1, w["T"], w["hidden"], device="cuda", dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        layers[0](x, rope)
