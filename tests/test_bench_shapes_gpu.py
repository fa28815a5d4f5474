"""Parity AT THE BENCHMARK SHAPES: the sequence lengths, head counts and head dimensions the throughput numbers
are quoted on (124M shapes at T=4096 and T=16384, 16 heads x 128 at T=8192 forward and backward, grouped-query
12/2 heads x 128 at T=8192), one sequence (two at T=4096) so the oracle stays cheap.

Two checkers, both the pinned oracle (oracle/saf_oracle.py):
  * every row, every head: the oracle's formulas evaluated with torch fp32 on the device (TF32 off), in row chunks;
  * 64 sampled query rows (first, middle and last tile pairs, tile seams, the ragged tail), all heads and
    columns: the oracle on the CPU in fp64.
Bars: bf16 forward max-abs <= 2e-2 and rel-L2 <= 1e-2 against the fp32 eager result; gradients within the
reference's bf16 gates (kernel/test_fused_attn.py:188-193: max-abs 2e-1) and rel-L2 <= 3.5e-2
(supplement/test_controls.py:188).
"""
import pytest
import torch

from oracle import saf_oracle as O
from tests.util import errs, head_maps

pytestmark = pytest.mark.gpu

FWD_ABS, FWD_REL = 2e-2, 1e-2
BWD_ABS, BWD_REL = 2e-1, 3.5e-2


def sample_rows(T, n=64):
    """Query positions: tile seams of the first, a middle and the last 256-row pair, a spread, and the tail."""
    mid = (T // 2) // 256 * 256
    last = (T - 1) // 256 * 256
    picks = {0, 1, 63, 64, 127, 128, 129, 255, T - 1, T - 2, max(T - 65, 0), max(T - 129, 0)}
    for base in (mid, last):
        for off in (0, 1, 127, 128, 200, 255):
            if base + off < T:
                picks.add(base + off)
    spread = torch.linspace(0, T - 1, n).long().tolist()
    for r in spread:
        if len(picks) >= n:
            break
        picks.add(int(r))
    return torch.tensor(sorted(picks), dtype=torch.long)


def structured_states(H, n_frozen, seed=1337, layer=0):
    fz = O.frozen_heads_for_layer(H, n_frozen, seed, layer)
    return fz, [3 if h in fz else 0 for h in range(H)]


def op_inputs(B, U, HV, HK, T, hd, seed, dev):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, U, T, hd, generator=g).bfloat16()
    k = torch.randn(B, HK, T, hd, generator=g).bfloat16()
    v = torch.randn(B, HV, T, hd, generator=g).bfloat16()
    return q, k, v


def check_forward(y, q, k, v, states, hidx, T, rows=None, **kw):
    """y (device, bf16) against the oracle: all rows in fp32 on the device, sampled rows in fp64 on the CPU."""
    dev = y.device
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        dkw = {n: (t.to(dev) if torch.is_tensor(t) else t) for n, t in kw.items()}
        if "sink_decay" in kw:
            dkw["sink_decay"] = kw["sink_decay"]
        with torch.no_grad():
            full = O.mixed_attn(q.to(dev).float(), k.to(dev).float(), v.to(dev).float(), dkw.pop("patt", None), states,
                                hidx=hidx, **dkw)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    a, r = errs(y, full)
    assert a <= FWD_ABS and r <= FWD_REL, f"all rows: max-abs {a} rel-l2 {r}"
    rows = sample_rows(T) if rows is None else rows
    ckw = dict(kw)
    with torch.no_grad():
        part = O.mixed_attn(q.double(), k.double(), v.double(), ckw.pop("patt", None), states, hidx=hidx, rows=rows,
                            dtype=torch.float64, **ckw)
    a2, r2 = errs(y[:, :, rows.to(dev)], part)
    assert a2 <= FWD_ABS and r2 <= FWD_REL, f"sampled rows (fp64): max-abs {a2} rel-l2 {r2}"
    return a, r


@pytest.mark.parametrize("B,T", [(1, 16384), (2, 4096), (1, 16300)])
def test_124m_shapes_structured_heads(B, T):
    """12 heads x 64, 9 live + 3 sink+decay heads: the mixed launch of the long-context and T=4096 prefill
    workloads (and a ragged length close to 16K)."""
    from kernel import fused_mixed_attn
    dev, H, hd = "cuda", 12, 64
    fz, states = structured_states(H, 3)
    live, hidx = head_maps(H, states)
    q, k, v = op_inputs(B, len(live), H, len(live), T, hd, T + B, dev)
    a, r = O.sink_decay_params(H, 2337)
    a, r = a.float().double(), r.float().double()
    y = fused_mixed_attn(q.to(dev), k.to(dev), v.to(dev), None, torch.tensor(states, dtype=torch.int32, device=dev),
                         hidx.to(dev), sink_decay=(a.float().to(dev), r.float().to(dev)))
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all()
    check_forward(y, q, k, v, states, hidx, T, sink_decay=(a, r))


def _c3_heads(T, S, dev):
    """16 heads x 128 with four frozen heads in all three frozen representations: two sink+decay, one dense
    stored in bf16, one decomposed."""
    H = 16
    states = [0] * H
    states[3], states[9] = 3, 3
    states[6] = 1
    states[12] = 2
    live, hidx = head_maps(H, states)
    g = torch.Generator().manual_seed(77)
    p = torch.rand(1, S, S, generator=g).tril_()
    p /= p.sum(-1, keepdim=True)
    patt = p.bfloat16()                                   # compact: one plane, addressed through pidx
    pidx = torch.zeros(H, dtype=torch.int32)
    alpha, rho = torch.zeros(H, S), torch.zeros(H, S)
    alpha[12] = torch.randn(S, generator=g) * 0.8
    rho[12] = torch.randn(S, generator=g) * 0.8 - 0.002 * torch.arange(S)
    z = torch.zeros(H, S)
    z[12] = O.decomposed_logz(alpha[12:13], rho[12:13])[0]
    a, r = O.sink_decay_params(H, 4337)
    return states, live, hidx, patt, pidx, alpha, rho, z, (a.float().double(), r.float().double())


def test_1b_shape_forward_and_backward():
    """16 heads x 128, T=8192 (the training configuration's attention): forward and all three input gradients
    with live, structured, dense-stored and decomposed heads in one call."""
    from kernel import fused_mixed_attn
    dev, B, T, hd = "cuda", 1, 8192, 128
    states, live, hidx, patt, pidx, alpha, rho, z, sd = _c3_heads(T, T, dev)
    H = len(states)
    q, k, v = op_inputs(B, len(live), H, len(live), T, hd, 8192, dev)
    qd, kd, vd = [t.to(dev).requires_grad_(True) for t in (q, k, v)]
    y = fused_mixed_attn(qd, kd, vd, patt.to(dev), torch.tensor(states, dtype=torch.int32, device=dev), hidx.to(dev),
                         pidx.to(dev), alpha=alpha.to(dev), rho=rho.to(dev), z=z.to(dev),
                         sink_decay=(sd[0].float().to(dev), sd[1].float().to(dev)))
    gw = torch.Generator().manual_seed(7)
    w = torch.randn(B, H, T, hd, generator=gw).bfloat16()
    y.backward(w.to(dev))
    torch.cuda.synchronize()
    check_forward(y.detach(), q, k, v, states, hidx, T, patt=patt.float(), pidx=pidx, alpha=alpha, rho=rho, z=z,
                  sink_decay=sd)
    # backward oracle: autograd through the same formulas, fp32 on the device
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        rq, rk, rv = [t.to(dev).float().requires_grad_(True) for t in (q, k, v)]
        y_ref = O.mixed_attn(rq, rk, rv, patt.float().to(dev), states, hidx=hidx, pidx=pidx, alpha=alpha.to(dev),
                             rho=rho.to(dev), z=z.to(dev), sink_decay=sd)
        y_ref.backward(w.to(dev).float())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    for name, got, want in (("dq", qd.grad, rq.grad), ("dk", kd.grad, rk.grad), ("dv", vd.grad, rv.grad)):
        a, r = errs(got, want)
        assert a <= BWD_ABS and r <= BWD_REL, f"{name}: max-abs {a} rel-l2 {r}"


def test_gqa_shape_forward():
    """12 query heads on 2 KV heads x 128, T=8192: live heads read K/V through kvidx, structured and
    dense-stored frozen heads read the V of their KV group."""
    from kernel import fused_mixed_attn
    dev, B, T, hd, H, HKV = "cuda", 1, 8192, 128, 12, 2
    fz = O.frozen_heads_for_layer(H, 3, 1337, 0)
    states = [0] * H
    states[fz[0]], states[fz[1]], states[fz[2]] = 3, 3, 1
    live, hidx = head_maps(H, states)
    kv = torch.tensor([h * HKV // H for h in range(H)], dtype=torch.int32)
    q, k, v = op_inputs(B, len(live), HKV, HKV, T, hd, 4242, dev)
    g = torch.Generator().manual_seed(78)
    p = torch.rand(1, T, T, generator=g).tril_()
    p /= p.sum(-1, keepdim=True)
    patt = p.bfloat16()
    pidx = torch.zeros(H, dtype=torch.int32)
    a, r = O.sink_decay_params(H, 5337)
    sd = (a.float().double(), r.float().double())
    y = fused_mixed_attn(q.to(dev), k.to(dev), v.to(dev), patt.to(dev),
                         torch.tensor(states, dtype=torch.int32, device=dev), hidx.to(dev), pidx.to(dev),
                         kvidx=kv.to(dev), sink_decay=(sd[0].float().to(dev), sd[1].float().to(dev)))
    torch.cuda.synchronize()
    assert y.is_contiguous() and y.shape == (B, H, T, hd)
    check_forward(y, q, k, v, states, hidx, T, patt=patt.float(), pidx=pidx, kvidx=kv, sink_decay=sd)


@pytest.mark.parametrize("name,B", [("c2", 1), ("c1", 2)])
def test_layer_of_the_benchmark_stack(name, B):
    """Layer 0 of the benchmark's stack exactly as bench.py builds it (indexed QKV GEMM with RoPE, mixed attention,
    c_proj; bf16) against the oracle's eager layer on sampled rows (fp32 on the CPU) and on every row (fp32 torch on
    the device)."""
    from saf_b200 import synthetic
    dev = torch.device("cuda")
    layers, rope, w = synthetic.build_attention_stack(name, dev, n_layer=1)
    m = layers[0]
    T, H, hd = w["T"], w["n_head"], w["head_dim"]
    C = H * hd
    g = torch.Generator().manual_seed(1000)
    x = torch.randn(B, T, C, generator=g).bfloat16()
    with torch.inference_mode():
        y = m(x.to(dev), rope=rope)
    torch.cuda.synchronize()
    ws = [lin.weight.detach().float().cpu() for lin in (m.q_proj, m.k_proj, m.v_proj, m.c_proj)]
    states = list(m._states)
    sd = m.sd_params().double().cpu()
    cos, sin = O.rope_cache(hd, T, base=w["rope_base"])
    rows = sample_rows(T)
    with torch.no_grad():
        ref = O.attention_layer(x.float(), *ws, states, None, H, rope=(cos, sin), rows=rows,
                                sink_decay=(sd[:, 0], sd[:, 1]))
    a, r = errs(y[:, rows.to(dev)], ref)
    assert a <= FWD_ABS and r <= FWD_REL, f"sampled rows: max-abs {a} rel-l2 {r}"
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        with torch.no_grad():
            full = O.attention_layer(x.to(dev).float(), *[t.to(dev) for t in ws], states, None, H,
                                     rope=(cos.to(dev), sin.to(dev)), sink_decay=(sd[:, 0], sd[:, 1]))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    a, r = errs(y, full)
    assert a <= FWD_ABS and r <= FWD_REL, f"all rows: max-abs {a} rel-l2 {r}"


@pytest.mark.parametrize("with_dense", [False, True], ids=["structured", "structured+dense"])
def test_head_dim_96_recipe_shape_forward_and_backward(with_dense):
    """16 heads x 96 at T=8192 (the reference's own ~1B recipe, nanogpt/config/train_gpt_1b_rope.py): the 128-column
    tensor-core kernels with zero-filled tiles, forward and all three input gradients.  With a dense-stored head
    the call takes the one-shot kernel (pattern tiles produced by the softmax warps), without it the persistent one."""
    from kernel import fused_mixed_attn
    dev, B, T, hd, H = "cuda", 1, 8192, 96, 16
    states = [0] * H
    states[2], states[11] = 3, 3
    patt = pidx = None
    if with_dense:
        states[7] = 1
        g = torch.Generator().manual_seed(79)
        p = torch.rand(1, T, T, generator=g).tril_()
        p /= p.sum(-1, keepdim=True)
        patt = p.bfloat16()
        pidx = torch.zeros(H, dtype=torch.int32)
    live, hidx = head_maps(H, states)
    q, k, v = op_inputs(B, len(live), H, len(live), T, hd, 9696, dev)
    a, r = O.sink_decay_params(H, 6337)
    sd = (a.float().double(), r.float().double())
    qd, kd, vd = [t.to(dev).requires_grad_(True) for t in (q, k, v)]
    y = fused_mixed_attn(qd, kd, vd, None if patt is None else patt.to(dev),
                         torch.tensor(states, dtype=torch.int32, device=dev), hidx.to(dev),
                         None if pidx is None else pidx.to(dev), sink_decay=(sd[0].float().to(dev), sd[1].float().to(dev)))
    gw = torch.Generator().manual_seed(7)
    w = torch.randn(B, H, T, hd, generator=gw).bfloat16()
    y.backward(w.to(dev))
    torch.cuda.synchronize()
    kw = dict(sink_decay=sd)
    if with_dense:
        kw.update(patt=patt.float(), pidx=pidx)
    check_forward(y.detach(), q, k, v, states, hidx, T, **kw)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        rq, rk, rv = [t.to(dev).float().requires_grad_(True) for t in (q, k, v)]
        y_ref = O.mixed_attn(rq, rk, rv, None if patt is None else patt.float().to(dev), states, hidx=hidx, pidx=pidx,
                             sink_decay=sd)
        y_ref.backward(w.to(dev).float())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    for name, got, want in (("dq", qd.grad, rq.grad), ("dk", kd.grad, rk.grad), ("dv", vd.grad, rv.grad)):
        a_, r_ = errs(got, want)
        assert a_ <= BWD_ABS and r_ <= BWD_REL, f"{name}: max-abs {a_} rel-l2 {r_}"
