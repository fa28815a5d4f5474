"""Seeded synthetic stand-ins for the benchmark configurations (no dataset or checkpoint is needed:
the reference's own benches draw random token ids and uniform patterns too,
nanogpt/bench_inference_triton.py:86-111,170-173)."""
from types import SimpleNamespace

import torch

from .attention import SafCausalSelfAttention, rope_tables
from .workloads import WORKLOADS  # noqa: F401  (plain data, importable without the CUDA library)


def frozen_heads_for_layer(n_head, n_frozen, seed, layer):
    g = torch.Generator().manual_seed(seed + layer)
    return sorted(torch.randperm(n_head, generator=g)[:n_frozen].tolist())


def sink_decay_params(n, seed):
    """a ~ U(0.05, 0.3), r ~ U(0.8, 0.99) per frozen head."""
    g = torch.Generator().manual_seed(seed)
    a = 0.05 + 0.25 * torch.rand(n, generator=g, dtype=torch.float64)
    r = 0.8 + 0.19 * torch.rand(n, generator=g, dtype=torch.float64)
    return a, r


def workload_config(w):
    C = w["n_head"] * w["head_dim"]
    return SimpleNamespace(n_embd=C, n_head=w["n_head"], block_size=w["T"], bias=False, dropout=0.0,
                           position_encoding="rope", rand_attn_prior_repr="dense", freeze_pattern_dtype="bfloat16")


def build_attention_layer(w, li, g, seed=1337):
    """Layer `li` of a workload's stack on the CPU in fp32: weights drawn from generator `g` (the stack's
    running generator), frozen heads and their (sink weight, decay) from the layer's own seeds."""
    C = w["n_head"] * w["head_dim"]
    m = SafCausalSelfAttention(workload_config(w), layer_idx=li)
    with torch.no_grad():
        for lin in (m.q_proj, m.k_proj, m.v_proj, m.c_proj):
            lin.weight.copy_(torch.randn(C, C, generator=g) * 0.02)
    fz = w.get("frozen_heads") or frozen_heads_for_layer(w["n_head"], w["n_frozen"], seed, li)
    a, r = sink_decay_params(len(fz), seed + 1000 + li)
    m.freeze_heads_sink_decay(fz, a.tolist(), r.tolist())
    return m


def build_attention_stack(name, device, dtype=None, seed=1337, blocks=False, n_layer=None):
    """The attention+projection stack of a GPT-2-style model: one SafCausalSelfAttention per layer with
    random-init N(0, 0.02^2) weights, 25 % of the heads of every layer frozen on seeded sink+decay patterns.
    blocks=True wraps every layer in its transformer block (LayerNorms, residuals, MLP with 4x expansion);
    n_layer builds only the first layers (same weights as the full stack's)."""
    w = WORKLOADS[name]
    if dtype is None:
        dtype = getattr(torch, w.get("dtype", "bfloat16"))
    if w.get("n_kv") is not None:
        raise ValueError("workload %r is grouped-query: build it with saf_b200.gqa.build_gqa_stack" % name)
    C = w["n_head"] * w["head_dim"]
    cfg = workload_config(w)
    g = torch.Generator().manual_seed(seed)
    layers = []
    for li in range(w["n_layer"] if n_layer is None else n_layer):
        m = build_attention_layer(w, li, g, seed)
        if blocks:
            from .block import SafBlock
            blk = SafBlock(cfg, layer_idx=li)
            blk.main_block = m
            with torch.no_grad():
                blk.mlp.c_fc.weight.copy_(torch.randn(4 * C, C, generator=g) * 0.02)
                blk.mlp.c_proj.weight.copy_(torch.randn(C, 4 * C, generator=g) * 0.02)
            m = blk
        layers.append(m.to(device=device, dtype=dtype).eval())
    cos, sin = rope_tables(w["head_dim"], w["T"], base=w["rope_base"], device=device)
    rope = (cos.view(1, 1, w["T"], -1), sin.view(1, 1, w["T"], -1))
    return layers, rope, w


def stack_forward(layers, rope, x, probe=None):
    """x -> layer_L(...layer_1(x)); `probe(i, fn)` may wrap each layer call (timing)."""
    h = x
    for i, m in enumerate(layers):
        h = m(h, rope=rope) if probe is None else probe(i, m, h, rope)
    return h


def hot_stack_flops(w):
    """Algorithmic FLOPs of one pass per sequence in the batch: live causal attention, indexed QKV GEMM, c_proj."""
    H, hd, T, nf = w["n_head"], w["head_dim"], w["T"], w["n_frozen"]
    U, C = H - nf, H * hd
    live = 2 * U * T * T * hd                     # causal half of 4 T^2 hd
    qkv = 2 * T * C * (2 * U + H) * hd
    oproj = 2 * T * C * C
    mlp = 2 * T * C * 8 * C                       # c_fc and c_proj of the 4x MLP
    return dict(live=live * w["n_layer"], qkv=qkv * w["n_layer"], oproj=oproj * w["n_layer"], mlp=mlp * w["n_layer"])


def per_layer_split(m, rope, x, reps=5):
    """Device time (ms, median of `reps`, CUDA events) of the pieces of one layer's hot path on input x:
    the fused projection, the mixed-attention launch, and -- each launched alone on the same tensors --
    the live heads only and the frozen heads only, then c_proj.  bf16 inference path."""
    from . import ops
    B, T, C = x.shape
    nh, hd = m.n_head, m.head_dim
    if m._fz_dirty:
        m._refresh_freeze_cache()
    live = list(m._live)
    nuf = len(live)
    fz = [h for h in range(nh) if h not in live]
    rp = m._rope_f32(rope, T, x.device)

    def timed(fn):
        for _ in range(2):
            out = fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2], out

    with torch.inference_mode():
        w = [m.q_proj.weight, m.k_proj.weight, m.v_proj.weight]
        t_qkv, qkv = timed(lambda: ops.qkv_projection(x, w[0], w[1], w[2], live, hd, rope=rp, T=T))
        qkv = qkv.view(B, T, 2 * nuf + nh, hd)
        qu, ku = qkv[:, :, :nuf].transpose(1, 2), qkv[:, :, nuf:2 * nuf].transpose(1, 2)
        v = qkv[:, :, 2 * nuf:].transpose(1, 2)
        t_mixed, y = timed(lambda: ops.fused_mixed_attn(qu, ku, v, None, m._fz_mask_i32, m._hidx_i32, validate=False,
                                                        sink_decay=m._sd))
        out = {"qkv_rope_gemm": t_qkv, "mixed_attention": t_mixed}
        if nuf:
            zeros = torch.zeros(nuf, dtype=torch.int32, device=x.device)
            v_live = qkv[:, :, [2 * nuf + h for h in live]].transpose(1, 2)
            out["live_heads_alone"], _ = timed(lambda: ops.fused_mixed_attn(qu, ku, v_live, None, zeros, validate=False))
        if fz:
            sd = m._sd
            idx = torch.tensor(fz, device=x.device)
            v_fz = qkv[:, :, [2 * nuf + h for h in fz]].transpose(1, 2)
            a_fz, r_fz = sd[0][idx].contiguous(), sd[1][idx].contiguous()
            out["frozen_heads_alone"], _ = timed(lambda: ops.frozen_pv(None, v_fz, None, T, sink_decay=(a_fz, r_fz)))
        y2 = y.transpose(1, 2).reshape(B, T, nh * hd)
        out["c_proj_gemm"], _ = timed(lambda: ops.linear_rows(y2, m.c_proj.weight, None, m._all_rows))
    return out


def build_model(name, device, dtype=torch.bfloat16, seed=1337, vocab_size=50257):
    """The whole GPT-2-style model of a workload (random init N(0, 0.02^2), tied embedding), blocks as in
    build_attention_stack(blocks=True)."""
    from .model import SafGPT
    blocks, rope, w = build_attention_stack(name, "cpu", dtype=torch.float32, seed=seed, blocks=True)
    C = w["n_head"] * w["head_dim"]
    cfg = SimpleNamespace(n_embd=C, n_head=w["n_head"], n_layer=w["n_layer"], block_size=w["T"], bias=False, dropout=0.0,
                          position_encoding="rope", rand_attn_prior_repr="dense", freeze_pattern_dtype="bfloat16",
                          vocab_size=vocab_size, rope_base=w["rope_base"])
    m = SafGPT(cfg)
    m.transformer.h = torch.nn.ModuleList(blocks)
    g = torch.Generator().manual_seed(seed + 7)
    with torch.no_grad():
        m.lm_head.weight.copy_(torch.randn(vocab_size, C, generator=g) * 0.02)
    return m.to(device=device, dtype=dtype).eval(), w
