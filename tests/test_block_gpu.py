"""GPU parity of the block around the attention path (LayerNorm, MLP with fused GELU / residual epilogues,
whole block) against the CPU oracle in fp32 on the same bf16-rounded inputs (nanogpt/model.py:45-54, 1193-1240)."""
from types import SimpleNamespace

import pytest
import torch

from oracle import saf_oracle as O
from tests.util import errs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(3, 70, 768, True), (2, 33, 2048, False), (1, 9, 200, True), (2, 5, 4096, False)],
                         ids=lambda s: f"M{s[0] * s[1]}C{s[2]}{'b' if s[3] else ''}")
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "fp32"])
def test_layer_norm(shape, dtype):
    from saf_b200 import ops
    B, T, C, has_b = shape
    g = torch.Generator().manual_seed(C + T)
    x = (torch.randn(B, T, C, generator=g) * 2 + 0.5).to(dtype)
    w = (1 + 0.1 * torch.randn(C, generator=g)).to(dtype)
    b = (0.1 * torch.randn(C, generator=g)).to(dtype) if has_b else None
    ref = O.layer_norm(x.float(), w.float(), None if b is None else b.float())
    y = ops.layer_norm(x.cuda(), w.cuda(), None if b is None else b.cuda())
    a, r = errs(y, ref)
    assert (a <= 2e-5 * max(1.0, ref.abs().max().item())) if dtype == torch.float32 else (a <= 3e-2 and r <= 5e-3), f"{a} {r}"


@pytest.mark.parametrize("shape", [(2, 300, 256, False), (1, 1000, 768, True), (2, 130, 1024, False),
                                   (3, 2900, 256, True)],     # 8700 rows: the CTA-pair tiles, ragged last pair
                         ids=lambda s: f"M{s[0] * s[1]}C{s[2]}")
def test_mlp_with_fused_gelu_and_residual(shape):
    from saf_b200 import ops
    B, T, C, bias = shape
    g = torch.Generator().manual_seed(C)
    x = torch.randn(B, T, C, generator=g).bfloat16()
    res = torch.randn(B, T, C, generator=g).bfloat16()
    w_fc = (torch.randn(4 * C, C, generator=g) * 0.05).bfloat16()
    w_pr = (torch.randn(C, 4 * C, generator=g) * 0.02).bfloat16()
    b_fc = (torch.randn(4 * C, generator=g) * 0.1).bfloat16() if bias else None
    b_pr = (torch.randn(C, generator=g) * 0.1).bfloat16() if bias else None
    f = lambda t: None if t is None else t.float()
    hid_ref = torch.nn.functional.gelu(torch.nn.functional.linear(x.float(), w_fc.float(), f(b_fc)))
    hid = ops.linear_act(x.cuda(), w_fc.cuda(), None if b_fc is None else b_fc.cuda(), act="gelu")
    a, r = errs(hid, hid_ref)
    assert r <= 5e-3, f"gelu(c_fc) rel-l2 {r}"
    ref = res.float() + O.mlp(x.float(), w_fc.float(), w_pr.float(), f(b_fc), f(b_pr))
    y = ops.linear_act(hid, w_pr.cuda(), None if b_pr is None else b_pr.cuda(), residual=res.cuda())
    a, r = errs(y, ref)
    assert a <= 3e-2 * max(1.0, ref.abs().max().item()) and r <= 1e-2, f"mlp + residual: max-abs {a} rel-l2 {r}"


def test_whole_block_bf16_inference():
    """x + attn(ln_1 x); x + mlp(ln_2 x) with 25 % of the heads frozen: 8 library launches, no torch compute."""
    from saf_b200 import launch_count
    from saf_b200.block import SafBlock
    from saf_b200.attention import rope_tables
    B, T, C, H = 2, 700, 256, 4
    hd = C // H
    cfg = SimpleNamespace(n_embd=C, n_head=H, block_size=T, bias=False, dropout=0.0, position_encoding="rope",
                          rand_attn_prior_repr="dense", freeze_pattern_dtype="float32")
    torch.manual_seed(3)
    blk = SafBlock(cfg)
    with torch.no_grad():
        for prm in blk.parameters():
            if prm.ndim == 2:
                prm.copy_(torch.randn_like(prm) * 0.05)
            else:
                prm.copy_(1 + 0.1 * torch.randn_like(prm))
    fz = [2]
    a, r = O.sink_decay_params(1, seed=7)
    a, r = a.float().double(), r.float().double()
    blk = blk.cuda().bfloat16().eval()
    blk.main_block.freeze_heads_sink_decay(fz, a.tolist(), r.tolist())
    cos, sin = rope_tables(hd, T, device="cuda")
    rope = (cos.view(1, 1, T, hd), sin.view(1, 1, T, hd))
    x = torch.randn(B, T, C, generator=torch.Generator().manual_seed(1)).bfloat16()
    with torch.inference_mode():
        n0 = launch_count()
        y = blk(x.cuda(), rope=rope)
        assert launch_count() - n0 == 7      # ln_1, qkv, mixed attention, c_proj, ln_2, c_fc+gelu, c_proj+residual
    # oracle in fp32 on the same bf16-rounded weights
    sd = {k: v.float().cpu() for k, v in blk.state_dict().items()}
    patt = torch.zeros(H, T, T)
    patt[fz] = O.sink_decay_pattern(a, r, T).float()
    states = [1 if h in fz else 0 for h in range(H)]
    attn = lambda t: O.attention_layer(t, sd["main_block.q_proj.weight"], sd["main_block.k_proj.weight"],
                                       sd["main_block.v_proj.weight"], sd["main_block.c_proj.weight"], states, patt, H,
                                       rope=O.rope_cache(hd, T))
    ref = O.block(x.float(), sd["ln_1.weight"], sd["ln_2.weight"], attn, sd["mlp.c_fc.weight"], sd["mlp.c_proj.weight"])
    aerr, rerr = errs(y, ref)
    assert aerr <= 6e-2 and rerr <= 1e-2, f"block: max-abs {aerr} rel-l2 {rerr}"


def test_whole_model_last_position_logits():
    """Token ids -> embedding -> blocks -> final LayerNorm -> tied lm_head at the last position
    (GPT.forward for inference, nanogpt/model.py:1373-1416)."""
    from saf_b200.model import SafGPT
    B, T, C, H, L, V = 2, 300, 256, 4, 2, 1000
    hd = C // H
    cfg = SimpleNamespace(n_embd=C, n_head=H, n_layer=L, block_size=T, bias=False, dropout=0.0, position_encoding="rope",
                          rand_attn_prior_repr="dense", freeze_pattern_dtype="float32", vocab_size=V, rope_base=10000.0)
    torch.manual_seed(11)
    m = SafGPT(cfg)
    with torch.no_grad():
        for prm in m.parameters():
            prm.copy_(torch.randn_like(prm) * 0.05 if prm.ndim == 2 else 1 + 0.1 * torch.randn_like(prm))
    m = m.cuda().bfloat16().eval()
    fz = [1]
    a, r = O.sink_decay_params(1, seed=3)
    a, r = a.float().double(), r.float().double()
    for blk in m.transformer.h:
        blk.main_block.freeze_heads_sink_decay(fz, a.tolist(), r.tolist())
    idx = torch.randint(0, V, (B, T), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    with torch.inference_mode():
        logits, _ = m(idx.cuda())
    assert logits.shape == (B, 1, V)
    sd = {k: v.float().cpu() for k, v in m.state_dict().items()}
    patt = torch.zeros(H, T, T)
    patt[fz] = O.sink_decay_pattern(a, r, T).float()
    states = [1 if h in fz else 0 for h in range(H)]
    x = sd["lm_head.weight"][idx.long()]
    for li in range(L):
        pre = f"transformer.h.{li}."
        attn = lambda t, pre=pre: O.attention_layer(t, sd[pre + "main_block.q_proj.weight"], sd[pre + "main_block.k_proj.weight"],
                                                    sd[pre + "main_block.v_proj.weight"], sd[pre + "main_block.c_proj.weight"],
                                                    states, patt, H, rope=O.rope_cache(hd, T))
        x = O.block(x, sd[pre + "ln_1.weight"], sd[pre + "ln_2.weight"], attn, sd[pre + "mlp.c_fc.weight"],
                    sd[pre + "mlp.c_proj.weight"])
    ref = torch.nn.functional.linear(O.layer_norm(x, sd["transformer.ln_f.weight"])[:, -1:, :], sd["lm_head.weight"])
    aerr, rerr = errs(logits, ref)
    assert rerr <= 2e-2, f"logits: max-abs {aerr} rel-l2 {rerr}"
