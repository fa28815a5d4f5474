"""GPU parity of linear_rows / linear_rows2 / linear_permuted_cols (forward, dx, dW, db) against
the CPU oracle, including the exact-zero gradient rows of unselected heads
(kernel/indexed_linear.py:112-115, nanogpt/test_prior_decomposed.py:117-136)."""
import pytest
import torch

from oracle import saf_oracle as O
from tests.util import errs

pytestmark = pytest.mark.gpu


def head_rows(heads, hd):
    return (torch.tensor(heads)[:, None] * hd + torch.arange(hd)).reshape(-1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("bias", [False, True], ids=["nobias", "bias"])
@pytest.mark.parametrize("shape", [(2, 130, 256, 4, 64, [0, 2, 3]), (1, 515, 768, 12, 64, [0, 1, 3, 4, 6, 7, 9, 10, 11]),
                                   (2, 64, 192, 2, 96, [1])], ids=lambda s: f"T{s[1]}C{s[2]}")
def test_linear_rows2(shape, bias, dtype):
    from kernel import linear_rows2, linear_rows
    B, T, C, H, hd, live = shape
    dev = "cuda"
    g = torch.Generator().manual_seed(T + C)
    x = torch.randn(B, T, C, generator=g).to(dtype)
    w1 = (torch.randn(H * hd, C, generator=g) * 0.05).to(dtype)
    w2 = (torch.randn(H * hd, C, generator=g) * 0.05).to(dtype)
    b1 = (torch.randn(H * hd, generator=g) * 0.1).to(dtype) if bias else None
    b2 = (torch.randn(H * hd, generator=g) * 0.1).to(dtype) if bias else None
    rows = head_rows(live, hd)
    ref_in = [t.float().clone().requires_grad_(True) if t is not None else None for t in (x, w1, w2, b1, b2)]
    y_ref = O.linear_rows2(*ref_in, rows)
    dev_in = [t.clone().to(dev).requires_grad_(True) if t is not None else None for t in (x, w1, w2, b1, b2)]
    y = linear_rows2(*dev_in, rows.to(dev))
    assert y.shape == y_ref.shape
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    a, r = errs(y, y_ref)
    assert a <= tol * max(1.0, y_ref.abs().max().item()), f"fwd {a}"
    if dtype == torch.bfloat16:
        assert r <= 1e-2
    w = torch.randn(y_ref.shape, generator=g)
    (y.float() * w.to(dev)).sum().backward()
    (y_ref * w).sum().backward()
    names = ("dx", "dw1", "dw2", "db1", "db2")
    for n, d, rf in zip(names, dev_in, ref_in):
        if d is None:
            continue
        a, r = errs(d.grad, rf.grad)
        assert r <= (1e-5 if dtype == torch.float32 else 1.5e-2), f"{n} rel-l2 {r}"
    # rows of frozen heads: exactly zero gradient
    dead = [h for h in range(H) if h not in live]
    if dead:
        dr = head_rows(dead, hd).to(dev)
        assert dev_in[1].grad[dr].abs().max().item() == 0.0
        assert dev_in[2].grad[dr].abs().max().item() == 0.0
    # single-weight variant: bit-identical to the matching half of the fused call when both run the same kernel
    # (head widths that are whole 64-row weight blocks); other widths may take different kernels for the two calls
    y1 = linear_rows(dev_in[0].detach(), dev_in[1].detach(), None if b1 is None else dev_in[3].detach(), rows.to(dev))
    if hd % 64 == 0 or dtype == torch.float32:
        assert torch.equal(y1, y[..., : y.shape[-1] // 2])
    else:
        assert errs(y1, y[..., : y.shape[-1] // 2])[1] <= 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_linear_permuted_cols(dtype):
    from kernel import linear_permuted_cols
    dev = "cuda"
    B, T, C, H, hd = 2, 77, 256, 4, 64
    g = torch.Generator().manual_seed(11)
    y_in = torch.randn(B, T, C, generator=g).to(dtype)
    w = (torch.randn(C, C, generator=g) * 0.05).to(dtype)
    b = (torch.randn(C, generator=g) * 0.1).to(dtype)
    cols = torch.cat([head_rows([0, 2, 3], hd), head_rows([1], hd)])
    ref_in = [t.float().clone().requires_grad_(True) for t in (y_in, w, b)]
    o_ref = O.linear_permuted_cols(*ref_in, cols)
    dev_in = [t.clone().to(dev).requires_grad_(True) for t in (y_in, w, b)]
    o = linear_permuted_cols(*dev_in, cols.to(dev))
    a, r = errs(o, o_ref)
    assert r <= (1e-5 if dtype == torch.float32 else 1e-2), f"fwd {r}"
    wgt = torch.randn(o_ref.shape, generator=g)
    (o.float() * wgt.to(dev)).sum().backward()
    (o_ref * wgt).sum().backward()
    for n, d, rf in zip(("dy", "dw", "db"), dev_in, ref_in):
        a, r = errs(d.grad, rf.grad)
        assert r <= (1e-5 if dtype == torch.float32 else 1.5e-2), f"{n} rel-l2 {r}"


def test_gather_is_bit_exact():
    """Selecting rows must not change a single bit: the sliced product equals the same kernel
    run over a physically gathered weight."""
    from kernel import linear_rows
    dev = "cuda"
    g = torch.Generator().manual_seed(3)
    x = torch.randn(300, 256, generator=g).bfloat16().to(dev)
    w = (torch.randn(512, 256, generator=g) * 0.05).bfloat16().to(dev)
    rows = head_rows([1, 4, 6], 64).to(dev)
    y = linear_rows(x, w, None, rows)
    wg = w[rows].contiguous()
    y2 = linear_rows(x, wg, None, torch.arange(wg.shape[0], device=dev))
    assert torch.equal(y, y2)


def test_decomposed_logz_kernel():
    from kernel import decomposed_logz
    g = torch.Generator().manual_seed(9)
    alpha = torch.randn(5, 320, generator=g) * 3
    rho = torch.randn(5, 320, generator=g) * 3
    z_ref = O.decomposed_logz(alpha.double(), rho.double())
    z = decomposed_logz(alpha.cuda(), rho.cuda())
    assert O.max_abs(z.cpu(), z_ref) <= 1e-5


@pytest.mark.parametrize("cfg", [(2, 9000, 768, 12, 64, [0, 1, 3, 4, 6, 7, 9, 10, 11], False),
                                 (2, 1000, 768, 12, 64, [0, 1, 3, 4, 6, 7, 9, 10, 11], True),
                                 (1, 700, 512, 4, 128, [0, 2, 3], False),
                                 (3, 129, 256, 4, 64, [], False),
                                 (1, 1500, 1536, 16, 96, [0, 1, 2, 3, 5, 6, 7, 9, 10, 11, 13, 14], False),
                                 (2, 333, 384, 4, 96, [1, 3], True),
                                 # 8192 rows and more: CTA-pair tiles (ragged last pair, bias, 128- and 96-wide heads)
                                 (3, 3000, 768, 12, 64, [0, 1, 3, 4, 6, 7, 9, 10, 11], True),
                                 (2, 4100, 512, 4, 128, [0, 2, 3], False),
                                 (6, 1500, 768, 8, 96, [0, 1, 2, 3, 5, 6], True)],
                         ids=["c2shape", "bias", "hd128", "allfrozen", "hd96", "hd96bias", "pair-bias", "pair-hd128",
                              "pair-hd96"])
def test_qkv_projection_with_rope_epilogue(cfg):
    """[Q(live) | K(live) | V(all)] in one tensor-core GEMM with the rotation in the epilogue equals
    projection followed by the reference's apply_rotary_pos_emb (nanogpt/model.py:63-68)."""
    from saf_b200 import qkv_projection
    B, T, C, H, hd, live, bias = cfg
    dev = "cuda"
    g = torch.Generator().manual_seed(T + C + hd)
    x = torch.randn(B, T, C, generator=g).bfloat16()
    ws = [(torch.randn(H * hd, C, generator=g) * 0.05).bfloat16() for _ in range(3)]
    bs = [(torch.randn(H * hd, generator=g) * 0.1).bfloat16() for _ in range(3)] if bias else None
    cos, sin = O.rope_cache(hd, T)
    rows = head_rows(live, hd) if live else torch.zeros(0, dtype=torch.long)
    xf = x.float()
    q = O.linear_rows(xf, ws[0].float(), None if bs is None else bs[0].float(), rows).view(B, T, len(live), hd)
    k = O.linear_rows(xf, ws[1].float(), None if bs is None else bs[1].float(), rows).view(B, T, len(live), hd)
    v = torch.nn.functional.linear(xf, ws[2].float(), None if bs is None else bs[2].float())
    q = O.apply_rope(q.transpose(1, 2), cos, sin).transpose(1, 2).reshape(B * T, -1)
    k = O.apply_rope(k.transpose(1, 2), cos, sin).transpose(1, 2).reshape(B * T, -1)
    ref = torch.cat([q, k, v.reshape(B * T, -1)], dim=-1)
    out = qkv_projection(x.to(dev), *[w.to(dev) for w in ws], live, hd, rope=(cos.to(dev), sin.to(dev)), T=T,
                         biases=None if bs is None else [b.to(dev) for b in bs])
    assert out.shape == ref.shape
    a, r = errs(out, ref)
    assert r <= 5e-3 and a <= 2e-2 * max(1.0, ref.abs().max().item()), f"{a} {r}"


@pytest.mark.parametrize("cfg", [(2, 300, 256, 4, 64, [0, 2, 3], torch.float32), (2, 300, 256, 4, 64, [0, 2, 3], torch.bfloat16),
                                 (1, 1100, 1024, 8, 128, [0, 1, 2, 4, 5, 7], torch.bfloat16),
                                 (1, 700, 768, 8, 96, [0, 1, 2, 4, 5, 7], torch.bfloat16),
                                 (2, 40, 96, 3, 32, [0, 2], torch.float32)],
                         ids=lambda c: f"T{c[1]}C{c[2]}hd{c[4]}{'bf16' if c[6] == torch.bfloat16 else 'fp32'}")
def test_linear_rows2_with_fused_rope(cfg):
    """Rotation in the projection's epilogue, adjoint rotation in its backward (training path of the hook)."""
    from kernel import linear_rows2
    B, T, C, H, hd, live, dtype = cfg
    dev = "cuda"
    g = torch.Generator().manual_seed(T + C + hd)
    x = torch.randn(B, T, C, generator=g).to(dtype)
    w1 = (torch.randn(H * hd, C, generator=g) * 0.05).to(dtype)
    w2 = (torch.randn(H * hd, C, generator=g) * 0.05).to(dtype)
    rows = head_rows(live, hd)
    cos, sin = O.rope_cache(hd, T)
    ref_in = [t.float().clone().requires_grad_(True) for t in (x, w1, w2)]
    U = len(live)
    y_lin = O.linear_rows2(ref_in[0], ref_in[1], ref_in[2], None, None, rows).view(B, T, 2 * U, hd)
    y_ref = O.apply_rope(y_lin.transpose(1, 2), cos, sin).transpose(1, 2).reshape(B, T, 2 * U * hd)
    dev_in = [t.clone().to(dev).requires_grad_(True) for t in (x, w1, w2)]
    y = linear_rows2(dev_in[0], dev_in[1], dev_in[2], None, None, rows.to(dev), rope=(cos.to(dev), sin.to(dev)), head_dim=hd)
    a, r = errs(y, y_ref)
    if dtype == torch.float32:
        assert a <= 2e-5 * max(1.0, y_ref.abs().max().item()), f"fwd {a}"
    else:
        assert r <= 1e-2, f"fwd rel-l2 {r}"
    w = torch.randn(y_ref.shape, generator=g)
    (y.float() * w.to(dev)).sum().backward()
    (y_ref * w).sum().backward()
    for n, d, rf in zip(("dx", "dw1", "dw2"), dev_in, ref_in):
        a, r = errs(d.grad, rf.grad)
        assert r <= (1e-5 if dtype == torch.float32 else 1.5e-2), f"{n} rel-l2 {r}"
    dead = [h for h in range(H) if h not in live]
    dr = head_rows(dead, hd).to(dev)
    assert dev_in[1].grad[dr].abs().max().item() == 0.0 and dev_in[2].grad[dr].abs().max().item() == 0.0


def test_backward_products_many_tiles_bf16():
    """dx and dW on the tensor-core kernels across several persistent tiles and ragged edges."""
    from kernel import linear_rows2
    B, T, C, H, hd = 3, 1500, 1096, 16, 128
    live = [0, 1, 2, 3, 5, 6, 7, 8, 10, 11, 13, 14, 15]
    dev = "cuda"
    g = torch.Generator().manual_seed(5)
    x = torch.randn(B, T, C, generator=g).bfloat16()
    w1 = (torch.randn(H * hd, C, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(H * hd, C, generator=g) * 0.05).bfloat16()
    rows = head_rows(live, hd)
    ref_in = [t.float().clone().requires_grad_(True) for t in (x, w1, w2)]
    y_ref = O.linear_rows2(ref_in[0], ref_in[1], ref_in[2], None, None, rows)
    dev_in = [t.clone().to(dev).requires_grad_(True) for t in (x, w1, w2)]
    y = linear_rows2(dev_in[0], dev_in[1], dev_in[2], None, None, rows.to(dev))
    w = torch.randn(y_ref.shape, generator=g).bfloat16().float()
    (y.float() * w.to(dev)).sum().backward()
    (y_ref * w).sum().backward()
    for n, d, rf in zip(("dx", "dw1", "dw2"), dev_in, ref_in):
        a, r = errs(d.grad, rf.grad)
        assert r <= 1.5e-2, f"{n} rel-l2 {r}"
    dead = [h for h in range(H) if h not in live]
    dr = head_rows(dead, hd).to(dev)
    assert dev_in[1].grad[dr].abs().max().item() == 0.0 and dev_in[2].grad[dr].abs().max().item() == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("bias", [False, True])
def test_linear_rows_single_weight_gradients(bias, dtype):
    """linear_rows (one weight) with its three gradients against the reference's own autograd Function: dx, the
    weight gradient with exact zeros in the rows that were not selected, the bias gradient likewise
    (kernel/indexed_linear.py:28-55)."""
    from kernel import linear_rows
    dev = "cuda"
    g = torch.Generator().manual_seed(31)
    x = torch.randn(3, 70, 256, generator=g)
    w = torch.randn(256, 256, generator=g) * 0.05
    b = torch.randn(256, generator=g) * 0.1 if bias else None
    rows = (torch.tensor([0, 2, 3])[:, None] * 64 + torch.arange(64)).reshape(-1)
    ins = [t.to(dtype) for t in (x, w)] + ([b.to(dtype)] if bias else [])
    ref = [t.float().clone().requires_grad_(True) for t in ins]
    y_ref = O.linear_rows(ref[0], ref[1], ref[2] if bias else None, rows)
    gy = torch.randn(y_ref.shape, generator=g)
    (y_ref * gy).sum().backward()
    got = [t.clone().to(dev).requires_grad_(True) for t in ins]
    y = linear_rows(got[0], got[1], got[2] if bias else None, rows.to(dev))
    (y.float() * gy.to(dev)).sum().backward()
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert O.rel_l2(y.float().cpu(), y_ref.detach()) <= tol
    for name, a, r in zip(("dx", "dw", "db"), got, ref):
        assert a.grad is not None, f"{name} was not produced"
        assert O.rel_l2(a.grad.float().cpu(), r.grad) <= tol, name
    unselected = torch.ones(256, dtype=torch.bool)
    unselected[rows] = False
    assert got[1].grad[unselected.to(dev)].abs().max().item() == 0.0
    if bias:
        assert got[2].grad[unselected.to(dev)].abs().max().item() == 0.0


@pytest.mark.parametrize("blocks", [1, 3, 5, 7], ids=lambda k: f"{k}x64cols")
def test_cta_pair_gemm_with_partial_column_tiles(blocks):
    """8192 rows and more take the CTA-pair kernel (256 x 256 tiles, each CTA loads half of the weight tile): output
    widths of 64, 192, 320 and 448 columns leave the last column tile with 1 or 3 of its 4 blocks, so one CTA of the
    pair loads fewer weight blocks than the other (or none); C = 200 ends inside a K step; bias and a ragged last pair."""
    from kernel import linear_rows
    M, C = 8192 + 70, 200
    g = torch.Generator().manual_seed(blocks)
    x = torch.randn(M, C, generator=g).bfloat16()
    w = (torch.randn(1024, C, generator=g) * 0.05).bfloat16()
    b = (torch.randn(1024, generator=g) * 0.1).bfloat16()
    rows = torch.arange(128, 128 + 64 * blocks)
    ref = O.linear_rows(x.float(), w.float(), b.float(), rows)
    y = linear_rows(x.cuda(), w.cuda(), b.cuda(), rows.cuda())
    a, r = errs(y, ref)
    assert r <= 5e-3 and a <= 2e-2 * max(1.0, ref.abs().max().item()), f"{a} {r}"


@pytest.mark.parametrize("cfg", [(16384, 120, 21), (20972, 184, 21), (3000, 120, 21)], ids=lambda c: f"M{c[0]}C{c[1]}b{c[2]}")
def test_column_tiles_with_an_odd_number_of_blocks(cfg):
    """A last column tile of 1 or 3 output blocks between full tiles: the epilogue's two staging buffers must keep
    taking turns across tiles (they once alternated by the block's index inside its tile, and the block stored last
    was overwritten while the TMA store was still reading it: whole 128-row tiles of the last block came out wrong,
    a few per call).  Forward (both kernel forms), dx and dW (C = 320 gives their output an odd block count too)."""
    from kernel import linear_rows
    M, C, nb = cfg
    g = torch.Generator().manual_seed(8)
    rows = torch.arange(64 * nb) + 64
    x = torch.randn(M, C, generator=g).bfloat16().cuda()
    w = (torch.randn(64 * (nb + 4), C, generator=g) * 0.05).bfloat16().cuda()
    ref = torch.nn.functional.linear(x.float(), w.float()[rows.cuda()])
    for _ in range(3):                       # the overwrite was a race: give it more than one chance
        y = linear_rows(x, w, None, rows.cuda()).float()
        rel = ((y - ref).norm() / ref.norm()).item()
        assert rel <= 5e-3 and (y - ref).abs().max().item() <= 0.1, rel
    # backward products with 5 output blocks per row tile (C = 320)
    C2 = 320
    x2 = torch.randn(4096, C2, generator=g).bfloat16()
    w2 = (torch.randn(64 * (nb + 4), C2, generator=g) * 0.05).bfloat16()
    xr, wr = x2.float().requires_grad_(True), w2.float().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr[rows])
    wgt = torch.randn(yr.shape, generator=g).bfloat16().float()
    (yr * wgt).sum().backward()
    xd, wd = x2.cuda().requires_grad_(True), w2.cuda().requires_grad_(True)
    (linear_rows(xd, wd, None, rows.cuda()).float() * wgt.cuda()).sum().backward()
    for name, d, r_ in (("dx", xd.grad, xr.grad), ("dw", wd.grad, wr.grad)):
        a, r = errs(d, r_)
        assert r <= 1.5e-2, f"{name} rel-l2 {r}"
