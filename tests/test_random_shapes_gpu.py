"""Seeded random shapes through the C ABI against the oracle: sizes, head states, tails and flag combinations nobody
wrote down by hand.  (A sweep of this kind found the staging-buffer overwrite in the GEMM epilogues.)"""
import random

import pytest
import torch

from oracle import saf_oracle as O
from tests.test_mixed_attn_gpu import run_case

pytestmark = pytest.mark.gpu


def errs(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return (a - b).abs().max().item(), ((a - b).norm() / b.norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_indexed_linear_random_shapes(seed):
    """Row counts on both sides of the CTA-pair threshold, K ending inside a step, every count of output blocks."""
    from kernel import linear_rows
    rnd = random.Random(seed)
    for i in range(8):
        M = rnd.choice([rnd.randint(1, 2000), rnd.randint(8192, 21000)])
        C = 8 * rnd.randint(8, 200)
        nb = rnd.randint(1, 40)
        rows = torch.arange(64 * nb) + 64 * rnd.randint(0, 3)
        g = torch.Generator().manual_seed(seed * 100 + i)
        x = torch.randn(M, C, generator=g).bfloat16().cuda()
        w = (torch.randn(64 * (nb + 4), C, generator=g) * 0.05).bfloat16().cuda()
        b = (torch.randn(64 * (nb + 4), generator=g) * 0.1).bfloat16().cuda() if i % 2 else None
        y = linear_rows(x, w, b, rows.cuda())
        ref = torch.nn.functional.linear(x.float(), w.float()[rows.cuda()], None if b is None else b.float()[rows.cuda()])
        a, r = errs(y, ref)
        assert r <= 5e-3 and a <= 0.1, f"M{M} C{C} blocks{nb}: {a} {r}"


@pytest.mark.parametrize("seed", [21, 22, 23, 24])
def test_mixed_attention_random_shapes(seed):
    """All four head states in random proportion, odd sequence lengths, strided / compact / rotated inputs, forward
    and backward (run_case holds the tolerances)."""
    rnd = random.Random(seed)
    for i in range(8):
        hd = rnd.choice([64, 64, 128])
        B, H = rnd.randint(1, 3), rnd.randint(2, 8)
        T = rnd.choice([rnd.randint(1, 300), rnd.randint(300, 1200), rnd.randint(1200, 2100)])
        S = ((T + 63) // 64) * 64 + 64 * rnd.randint(0, 2)
        heads = list(range(H))
        rnd.shuffle(heads)
        fz = heads[:rnd.randint(0, H)]
        kinds = [rnd.choice("dcs") for _ in fz]
        dense = [h for h, k in zip(fz, kinds) if k == "d"]
        dec = [h for h, k in zip(fz, kinds) if k == "c"]
        sink = [h for h, k in zip(fz, kinds) if k == "s"]
        dtype = torch.bfloat16 if rnd.random() < 0.8 else torch.float32
        if hd == 128 and dtype == torch.float32 and T > 1200:
            T, S = 700, 704
        run_case(B, H, T, hd, S, dense, dec, dtype=dtype, sink=sink,
                 buf_bf16=(dtype == torch.bfloat16 and rnd.random() < 0.5), strided=rnd.random() < 0.3,
                 compact_patt=rnd.random() < 0.3, rope=rnd.random() < 0.3)


@pytest.mark.parametrize("seed", [31, 32])
def test_structured_scan_random_shapes(seed):
    """Scan of structured heads: widths 64 / 96 / 128, batches from 1 to 33, lengths from 1 to 20000 (register scan,
    chunked scan, tensor-core scan with one and with several chunks), decays up to 0.99995."""
    from kernel import frozen_pv
    rnd = random.Random(seed)
    for i in range(10):
        hd = rnd.choice([64, 128, 96, 64])
        B = rnd.choice([1, 2, 3, 5, 8, 17, 33])
        nf = rnd.randint(1, 6)
        T = rnd.choice([rnd.randint(1, 1100), rnd.randint(1000, 5000), rnd.randint(4000, 20000)])
        if B * nf * T * hd > 3e8:
            B = max(1, int(3e8 / (nf * T * hd)))
        dtype = torch.bfloat16 if rnd.random() < 0.8 else torch.float32
        a, r = O.sink_decay_params(nf, seed=i + T)
        if rnd.random() < 0.3:
            r = r * 0 + rnd.choice([0.5, 0.9, 0.999, 0.99995])
        a, r = a.float(), r.float()
        v = torch.randn(B, nf, T, hd, generator=torch.Generator().manual_seed(seed * 100 + i)).to(dtype)
        y = frozen_pv(None, v.cuda(), None, T, sink_decay=(a.cuda(), r.cuda())).float().cpu()
        assert torch.isfinite(y).all()
        for _ in range(min(2, B * nf)):
            b, f = rnd.randrange(B), rnd.randrange(nf)
            ref = O.sink_decay_scan(v[b, f], a[f].item(), r[f].item())
            d = (y[b, f].double() - ref).abs().max().item()
            rel = ((y[b, f].double() - ref).norm() / ref.norm().clamp_min(1e-9)).item()
            tol_a, tol_r = (2e-2, 1e-2) if dtype == torch.bfloat16 else (5e-5, 1e-5)
            assert d <= tol_a and rel <= tol_r, f"B{B} nf{nf} T{T} hd{hd} {dtype}: {d} {rel}"
