"""Generates tests/golden/gqa_vectors.npz by RUNNING THE REFERENCE's GQA attention module on CPU.

    python tests/golden/make_golden_gqa.py /path/to/reference

The reference has no unit test for its `kvidx` (grouped-query) variant of the fused operator; its only check is
an in-benchmark comparison against its own split torch path.  This script runs that split path itself:
`make_qwen3_hybrid_class()` of qwen/nanogpt/hybrid_prior_attention.py:466-640 wrapped around a random-init
Hugging Face `Qwen3Attention` (6 query heads on 2 KV heads x 32, RoPE base 1e6), with CPU tensors, so
`fused_attn_usable` is False and the module takes its portable fallback (:586-640: repeat_kv, SDPA for the live
heads, dense P @ V for the pattern heads).  Stored per case:
  * the input, every weight, the rotary tables, the pattern buffers and index maps the module built;
  * q (live heads, normed + rotated), k (raw KV heads, normed + rotated) and v (raw KV heads), produced by
    re-issuing the module's own sub-modules in the order of its forward (:551-571) -- the exact arguments
    the module hands to `fused_mixed_attn(..., kvidx=)`;
  * the module's output (after o_proj).
Cases: dense stored patterns, and the decomposed representation (alpha / rho, state 2).
Nothing under tests/ or in the library reads the reference at run time.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "qwen"))
    sys.path.insert(0, os.path.join(ref_root, "qwen", "nanogpt"))
    import hybrid_prior_attention as HPA
    from transformers import Qwen3Config
    from transformers.models.qwen3 import modeling_qwen3 as Q3

    torch.set_num_threads(8)
    H, HKV, hd, C, T, S, B = 6, 2, 32, 128, 100, 128, 2
    cfg = Qwen3Config(hidden_size=C, num_attention_heads=H, num_key_value_heads=HKV, head_dim=hd,
                      num_hidden_layers=1, intermediate_size=256, vocab_size=128, rope_theta=1e6,
                      max_position_embeddings=512, attention_bias=False)
    cfg._attn_implementation = "sdpa"        # the split path's causal branch (:605-613)
    cls = HPA.make_qwen3_hybrid_class()
    out = {"dims": np.array([H, HKV, hd, C, T, S, B])}
    for case, decomposed in (("dense", False), ("decomp", True)):
        torch.manual_seed(41 if decomposed else 40)
        orig = Q3.Qwen3Attention(cfg, layer_idx=0)
        with torch.no_grad():
            orig.q_norm.weight.copy_(1 + 0.2 * torch.randn(hd))
            orig.k_norm.weight.copy_(1 + 0.2 * torch.randn(hd))
        mask = torch.tensor([0, 1, 0, 0, 1, 0], dtype=torch.bool)
        patt = torch.rand(H, S, S).tril()
        patt = patt / patt.sum(-1, keepdim=True)
        decomp = None
        if decomposed:
            decomp = (torch.randn(H, S) * 0.8, torch.randn(H, S) * 0.8)
        m = cls(orig, None if decomposed else patt, mask, device="cpu", dtype=torch.float32, use_triton=True,
                decomp=decomp).eval()
        x = torch.randn(B, T, C)
        cos, sin = Q3.Qwen3RotaryEmbedding(cfg)(x, torch.arange(T)[None])
        with torch.no_grad():
            y, _ = m(x, (cos, sin), attention_mask=None)
            # the arguments of the module's fused call, from its own sub-modules (forward :551-571)
            k = m.k_norm(m.k_proj(x).view(B, T, HKV, hd)).transpose(1, 2)
            v = m.v_proj(x).view(B, T, HKV, hd).transpose(1, 2)
            q_std = m.q_norm(m.q_proj_std(x).view(B, T, m.n_standard_heads, hd)).transpose(1, 2)
            q_std, k = Q3.apply_rotary_pos_emb(q_std, k, cos, sin)
        assert m.hybrid_calls == 1 and m.triton_calls == 0        # the split torch path ran
        pre = f"gqa_{case}_"
        out[pre + "x"], out[pre + "y"] = x.numpy(), y.numpy()
        out[pre + "q"], out[pre + "k"], out[pre + "v"] = q_std.numpy(), k.numpy(), v.numpy()
        out[pre + "cos"], out[pre + "sin"] = cos[0].numpy(), sin[0].numpy()
        out[pre + "wq_std"], out[pre + "wk"] = m.q_proj_std.weight.detach().numpy(), m.k_proj.weight.detach().numpy()
        out[pre + "wv"], out[pre + "wo"] = m.v_proj.weight.detach().numpy(), m.o_proj.weight.detach().numpy()
        out[pre + "q_norm"], out[pre + "k_norm"] = m.q_norm.weight.detach().numpy(), m.k_norm.weight.detach().numpy()
        out[pre + "eps"] = np.array([m.q_norm.variance_epsilon])
        out[pre + "scaling"] = np.array([m.scaling])
        for nme in ("frozen_mask_i32", "hidx_i32", "pidx_i32", "kvidx_i32"):
            out[pre + nme] = getattr(m, nme).numpy()
        if decomposed:
            out[pre + "alpha"], out[pre + "rho"], out[pre + "z"] = m.dec_alpha.numpy(), m.dec_rho.numpy(), m.dec_z.numpy()
        else:
            out[pre + "patt"] = m.prior_pattern.numpy()
        print(case, "output", tuple(y.shape), "mean |y| =", y.abs().mean().item())
    path = os.path.join(HERE, "gqa_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB,", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden_gqa.py /path/to/reference")
    main(sys.argv[1])
