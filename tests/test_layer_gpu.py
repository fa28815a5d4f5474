"""The attention-module hook on the GPU against (a) vectors the reference itself produced for the same
seeded inputs (tests/golden/reference_vectors.npz, incl. benchmark configuration 0) and (b) the oracle.

Tolerances: fp32 end to end < 1e-3 as the reference's own integration test demands
(nanogpt/test_prior_flash.py:125-132; measured here ~1e-5); bf16 max-abs <= 2e-2 and rel-L2 <= 1e-2
against the fp32 eager result."""
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from oracle import saf_oracle as O
from tests.golden import cases
from tests.util import errs

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))


def build(C, H, T, ws, repr_="dense", dtype=torch.float32):
    from saf_b200.attention import SafCausalSelfAttention, rope_tables
    cfg = SimpleNamespace(n_embd=C, n_head=H, block_size=T, bias=False, dropout=0.0, position_encoding="rope",
                          rand_attn_prior_repr=repr_, freeze_pattern_dtype="float32")
    m = SafCausalSelfAttention(cfg)
    with torch.no_grad():
        for lin, w in zip((m.q_proj, m.k_proj, m.v_proj, m.c_proj), ws):
            lin.weight.copy_(w)
    m = m.cuda().to(dtype).eval()
    cos, sin = rope_tables(C // H, T, device="cuda")
    return m, (cos.view(1, 1, T, -1), sin.view(1, 1, T, -1))


@pytest.mark.parametrize("structured", [False, True], ids=["dense", "scan"])
@pytest.mark.parametrize("name", ["config0", "small_sink", "small_rand"])
def test_fp32_layer_matches_reference_vectors(name, structured):
    B, T, C, H, fz, seed, kind = cases.LAYER_CASES[name]
    x, ws = cases.layer_inputs(B, T, C, H, seed)
    patt, _ = cases.layer_patterns(kind, len(fz), T, seed)
    m, rope = build(C, H, T, ws)
    m.freeze_heads(fz, patt.cuda(), detect_structured=structured)
    if structured and kind == "sink_decay":
        assert m.dyn_struct[fz].all() and m.dyn_pattern is None      # recognised, no dense buffer allocated
    if structured and kind == "random":
        assert not m.dyn_struct.any()
    with torch.no_grad():
        y = m(x.cuda(), rope=rope)
    s, tot, atot = cases.sample(y.cpu(), 24, 24)
    ref = torch.from_numpy(G[f"layer_{name}_eager_sample"])
    assert O.max_abs(s, ref) <= 2e-5
    assert abs(atot - G[f"layer_{name}_eager_sums"][1]) / G[f"layer_{name}_eager_sums"][1] <= 1e-5
    if name != "config0":
        assert O.max_abs(y.cpu(), torch.from_numpy(G[f"layer_{name}_eager_full"])) <= 2e-5


def test_fp32_layer_decomposed_matches_reference_vectors():
    name, B, T, C, H, dense, dec, seed = cases.DECOMP_LAYER
    x, ws = cases.layer_inputs(B, T, C, H, seed)
    m, rope = build(C, H, T, ws, repr_="decomposed")
    al, rh = cases.decomp_vectors(len(dec), T, seed + 2)
    m.freeze_heads_decomposed(dec, al.cuda(), rh.cuda())
    m.freeze_heads(dense, cases.random_pattern(len(dense), T, seed + 1).cuda())
    assert O.max_abs(m.dyn_z[dec].cpu(), torch.from_numpy(G[f"layer_{name}_z"])) <= 1e-5
    with torch.no_grad():
        y = m(x.cuda(), rope=rope)
    assert O.max_abs(y.cpu(), torch.from_numpy(G[f"layer_{name}_eager_full"])) <= 2e-5
    # rollback of a freeze
    m.unfreeze_heads(dec)
    with torch.no_grad():
        y2 = m(x.cuda(), rope=rope)
    assert (y2 - y).abs().max().item() > 1e-4


@pytest.mark.parametrize("name", ["config0", "small_sink"])
def test_bf16_inference_path_vs_fp32_reference(name):
    """Tensor-core path: one QKV GEMM with RoPE epilogue + tcgen05 flash + scan + c_proj GEMM."""
    from saf_b200 import launch_count
    B, T, C, H, fz, seed, kind = cases.LAYER_CASES[name]
    x, ws = cases.layer_inputs(B, T, C, H, seed)
    patt, _ = cases.layer_patterns(kind, len(fz), T, seed)
    m, rope = build(C, H, T, ws, dtype=torch.bfloat16)
    m.freeze_heads(fz, patt.cuda(), detect_structured=True)
    xb = x.bfloat16()
    with torch.inference_mode():
        n0 = launch_count()
        y = m(xb.cuda(), rope=rope)
        # head_dim 64: QKV GEMM, one mixed launch (flash + co-scheduled scan), c_proj GEMM.
        # head_dim 32 has no tensor-core kernels: generic GEMM + RoPE pass, generic attention, scan, c_proj GEMM
        assert launch_count() - n0 == (3 if C // H == 64 else 5)
    # fp32 eager result on the same (bf16-rounded) inputs and weights
    full = torch.zeros(H, T, T)
    full[fz] = O.freeze_normalise(patt)
    states = [1 if h in fz else 0 for h in range(H)]
    ref = O.attention_layer(xb.float(), *[w.bfloat16().float() for w in ws], states, full, H,
                            rope=O.rope_cache(C // H, T))
    a, r = errs(y, ref)
    assert a <= 2e-2 and r <= 1e-2, f"max-abs {a} rel-l2 {r}"
    if name == "config0":
        s, _, _ = cases.sample(y.float().cpu(), 24, 24)
        assert O.max_abs(s, torch.from_numpy(G["layer_config0_eager_sample"])) <= 2e-2


def test_training_path_gradients_and_exact_zero_rows():
    """Frozen heads' q/k weight-gradient rows are exactly 0.0, live rows are not
    (nanogpt/test_prior_decomposed.py:117-136); all gradients match the oracle's autograd."""
    B, T, C, H, fz, seed, kind = cases.LAYER_CASES["small_sink"]
    x, ws = cases.layer_inputs(B, T, C, H, seed)
    patt, _ = cases.layer_patterns(kind, len(fz), T, seed)
    m, rope = build(C, H, T, ws)
    m.train()
    m.freeze_heads(fz, patt.cuda(), detect_structured=True)
    xd = x.cuda().requires_grad_(True)
    y = m(xd, rope=rope)
    w = torch.randn(y.shape, generator=torch.Generator().manual_seed(3))
    (y * w.cuda()).sum().backward()
    full = torch.zeros(H, T, T)
    full[fz] = O.freeze_normalise(patt)
    states = [1 if h in fz else 0 for h in range(H)]
    leaves = [t.clone().requires_grad_(True) for t in (x, *ws)]
    yr = O.attention_layer(*leaves, states, full, H, rope=O.rope_cache(C // H, T))
    (yr * w).sum().backward()
    assert O.max_abs(y.detach().cpu(), yr.detach()) <= 2e-5
    got = [xd.grad, m.q_proj.weight.grad, m.k_proj.weight.grad, m.v_proj.weight.grad, m.c_proj.weight.grad]
    for nme, gt, rf in zip(("dx", "dWq", "dWk", "dWv", "dWo"), got, leaves):
        assert O.rel_l2(gt.cpu(), rf.grad) <= 1e-4, nme
    hd = C // H
    for h in range(H):
        rows = slice(h * hd, (h + 1) * hd)
        for wg in (m.q_proj.weight.grad, m.k_proj.weight.grad):
            if h in fz:
                assert wg[rows].abs().max().item() == 0.0
            else:
                assert wg[rows].abs().max().item() > 0.0


def test_capture_path_and_state_dict_round_trip():
    B, T, C, H, fz, seed, kind = cases.LAYER_CASES["small_sink"]
    x, ws = cases.layer_inputs(B, T, C, H, seed)
    patt, _ = cases.layer_patterns(kind, len(fz), T, seed)
    m, rope = build(C, H, T, ws)
    m.freeze_heads(fz, patt.cuda())
    with torch.no_grad():
        y = m(x.cuda(), rope=rope)
        m.set_capture(True)
        ye = m(x.cuda(), rope=rope)
        m.set_capture(False)
    assert (y - ye).abs().max().item() <= 1e-4 and m._last_attn is None
    m2, _ = build(C, H, T, [torch.zeros_like(w) for w in ws])
    m2.load_state_dict(m.state_dict())
    with torch.no_grad():
        y2 = m2(x.cuda(), rope=rope)
    assert torch.equal(y, y2)
    for name in ("dyn_frozen", "dyn_pattern"):
        assert name in m.state_dict()


def test_inference_layer_is_cuda_graph_capturable():
    """The reference captures its prefill in a CUDA graph (nanogpt/bench_checkpoint_prefill.py:89-109): after one
    warm-up call (host copies of the index tensors are cached then) nothing in the path synchronises or allocates
    outside torch's graph pool, and a replay on new input matches the eager call bit for bit."""
    B, T, C, H, fz, seed, kind = cases.LAYER_CASES["config0"]
    x, ws = cases.layer_inputs(B, T, C, H, seed)
    patt, _ = cases.layer_patterns(kind, len(fz), T, seed)
    m, rope = build(C, H, T, ws, dtype=torch.bfloat16)
    m.freeze_heads(fz, patt.cuda(), detect_structured=True)
    static_x = x.bfloat16().cuda()
    with torch.inference_mode():
        y_eager = m(static_x, rope=rope).clone()      # warm-up
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            m(static_x, rope=rope)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_y = m(static_x, rope=rope)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(static_y, y_eager)
        x2 = torch.randn(B, T, C, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
        y2_eager = m(x2, rope=rope).clone()
        static_x.copy_(x2)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(static_y, y2_eager)


@pytest.mark.parametrize("structured", [True, False], ids=["scan", "dense"])
def test_training_step_under_bf16_autocast(structured):
    """fp32 master weights, bf16 autocast (the reference's training mode, supplement/test_controls.py:137-190): the
    forward and every gradient go through the tensor-core kernels (projection with fused RoPE, mixed attention forward
    and backward, dx / dW) and must match the fp32 oracle's autograd within bf16 rel-L2 gates; frozen heads' q/k
    weight-gradient rows stay exactly zero."""
    from saf_b200 import launch_count
    B, T, C, H, fz, seed, kind = cases.LAYER_CASES["config0"]
    x, ws = cases.layer_inputs(B, T, C, H, seed)
    patt, _ = cases.layer_patterns(kind, len(fz), T, seed)
    m, rope = build(C, H, T, ws)
    m.train()
    m.freeze_heads(fz, patt.cuda(), detect_structured=structured)
    xd = x.cuda().requires_grad_(True)
    n0 = launch_count()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = m(xd, rope=rope)
    w = torch.randn(y.shape, generator=torch.Generator().manual_seed(3))
    (y.float() * w.cuda()).sum().backward()
    # forward: v_proj, linear_rows2+RoPE, mixed attention, c_proj | backward: c_proj dx + dW, delta, dK/dV (+ frozen-head
    # roles), dQ, adjoint RoPE, q/k dx + dW, v_proj dx + dW.  The module's fp32-stored dense pattern is used through a
    # compact bf16 copy, so dense heads ride the same launches.  Every GEMM of the layer is the library's own.
    assert launch_count() - n0 == 14
    full = torch.zeros(H, T, T)
    full[fz] = O.freeze_normalise(patt)
    states = [1 if h in fz else 0 for h in range(H)]
    leaves = [t.clone().requires_grad_(True) for t in (x, *ws)]
    yr = O.attention_layer(*leaves, states, full, H, rope=O.rope_cache(C // H, T))
    (yr * w).sum().backward()
    a, r = errs(y, yr.detach())
    assert r <= 1.5e-2, f"forward rel-l2 {r}"
    got = [xd.grad, m.q_proj.weight.grad, m.k_proj.weight.grad, m.v_proj.weight.grad, m.c_proj.weight.grad]
    for nme, gt, rf in zip(("dx", "dWq", "dWk", "dWv", "dWo"), got, leaves):
        assert gt.dtype == torch.float32
        assert O.rel_l2(gt.cpu(), rf.grad) <= 3.5e-2, f"{nme} rel-l2 {O.rel_l2(gt.cpu(), rf.grad)}"
    hd = C // H
    for h in fz:
        rows = slice(h * hd, (h + 1) * hd)
        assert m.q_proj.weight.grad[rows].abs().max().item() == 0.0
        assert m.k_proj.weight.grad[rows].abs().max().item() == 0.0


def test_dropout_is_applied_in_training_and_absent_in_eval():
    """dropout > 0: the reference leaves its fused path while training (nanogpt/model.py:971-974) so that its SDPA
    half applies attention dropout, and always applies the residual dropout (:1169).  Here: eval output equals
    the dropout-free module; train-mode outputs differ from it and from one another; with the seed fixed they
    repeat; frozen heads' Q/K rows still get exactly zero gradient."""
    import copy
    B, T, C, H, fz, seed, kind = cases.LAYER_CASES["small_sink"]
    x, ws = cases.layer_inputs(B, T, C, H, seed)
    patt, _ = cases.layer_patterns(kind, len(fz), T, seed)
    m0, rope = build(C, H, T, ws)
    m0.freeze_heads(fz, patt.cuda(), detect_structured=True)
    m1 = copy.deepcopy(m0)
    m1.dropout = 0.25
    xd = x.cuda()
    m0.eval()
    m1.eval()
    with torch.no_grad():
        y0, y1 = m0(xd, rope=rope), m1(xd, rope=rope)
    assert torch.equal(y0, y1)
    m1.train()
    torch.manual_seed(11)
    ya = m1(xd, rope=rope)
    yb = m1(xd, rope=rope)
    torch.manual_seed(11)
    yc = m1(xd, rope=rope)
    assert not torch.allclose(ya, y0, atol=1e-4) and not torch.allclose(ya, yb, atol=1e-4)
    assert torch.equal(ya, yc)
    assert torch.isfinite(ya).all()
    # same expectation: the mean over many masks approaches the dropout-free output
    acc = torch.zeros_like(y0)
    n = 64
    with torch.no_grad():
        for _ in range(n):
            acc += m1(xd, rope=rope)
    assert O.rel_l2(acc.cpu() / n, y0.cpu()) < 0.25
    ya.square().sum().backward()
    hd = m1.head_dim
    for h in fz:
        assert m1.q_proj.weight.grad[h * hd:(h + 1) * hd].abs().max().item() == 0.0
        assert m1.k_proj.weight.grad[h * hd:(h + 1) * hd].abs().max().item() == 0.0
    assert m1.v_proj.weight.grad.abs().max().item() > 0.0
