"""GPU parity of frozen_pv (forward and backward) against the CPU oracle; shapes and
tolerances from the reference's kernel/test_frozen_attn.py:65-83 (fp32 1e-5 / 1e-4, bf16 5e-2)."""
import pytest
import torch

from oracle import saf_oracle as O
from tests.util import make_pattern, errs

pytestmark = pytest.mark.gpu

CASES = [
    (2, 12, 1024, 64, 1024, [0, 1, 2]),
    (2, 12, 1024, 64, 1024, [3]),
    (2, 12, 1024, 64, 1024, list(range(12))),
    (2, 12, 700, 64, 1024, [0, 5, 11]),
    (2, 12, 1, 64, 1024, [0, 5, 11]),
    (2, 12, 37, 64, 1024, [0, 5, 11]),
    (1, 16, 2048, 96, 2048, [0, 7, 8, 15]),
    (3, 8, 256, 128, 512, [1, 6]),
    (8, 12, 1024, 64, 1024, [0, 1, 2]),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: f"B{c[0]}nh{c[1]}T{c[2]}d{c[3]}nf{len(c[5])}")
def test_frozen_pv(case, dtype):
    from kernel import frozen_pv
    B, nh, T, hd, S, fz = case
    dev = "cuda"
    patt = make_pattern(nh, S, seed=nh * S + T)
    g = torch.Generator(device="cpu").manual_seed(T * hd + B)
    base = torch.randn(B, len(fz), T, hd, generator=g).to(dtype)
    v_ref = base.float().clone().requires_grad_(True)
    y_ref = O.frozen_pv(patt, v_ref, fz, T)
    v_dev = base.clone().to(dev).requires_grad_(True)
    y = frozen_pv(patt.to(dev), v_dev, torch.tensor(fz, dtype=torch.int32, device=dev), T)
    assert y.shape == (B, len(fz), T, hd) and y.is_contiguous()
    tol_f, tol_b = (1e-5, 1e-4) if dtype == torch.float32 else (2e-2, 5e-2)
    a, r = errs(y, y_ref)
    assert a <= tol_f, f"fwd {a}"
    w = torch.randn(y_ref.shape, generator=g)
    (y.float() * w.to(dev)).sum().backward()
    (y_ref * w).sum().backward()
    a, r = errs(v_dev.grad, v_ref.grad)
    assert a <= tol_b, f"bwd {a}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("shape", [(2, 3, 1024, 64), (1, 4, 2500, 128), (2, 2, 333, 96), (1, 3, 16384, 64),
                                   (1, 2, 5000, 128), (1, 1, 4097, 64), (1, 1, 66000, 64)],   # chunk-parallel scan: ragged, 1-row tail, wider chunks
                         ids=lambda s: f"B{s[0]}nf{s[1]}T{s[2]}d{s[3]}")
def test_frozen_pv_sink_decay_scan(shape, dtype):
    """Structured pattern through the scan == dense product with the materialised pattern
    (fp64 scan recurrence as the long-sequence oracle)."""
    from kernel import frozen_pv
    B, nf, T, hd = shape
    dev = "cuda"
    a, r = O.sink_decay_params(nf, seed=T)
    a, r = a.float(), r.float()
    g = torch.Generator(device="cpu").manual_seed(T + hd)
    base = torch.randn(B, nf, T, hd, generator=g).to(dtype)
    if T <= 4096:
        patt = O.sink_decay_pattern(a.double(), r.double(), T)
        v_ref = base.double().clone().requires_grad_(True)
        y_ref = torch.matmul(patt.unsqueeze(0), v_ref)
    else:
        v_ref = None
        y_ref = torch.stack([torch.stack([O.sink_decay_scan(base[b, f], a[f].item(), r[f].item())
                                          for f in range(nf)]) for b in range(B)])
    v_dev = base.clone().to(dev).requires_grad_(True)
    y = frozen_pv(None, v_dev, None, T, sink_decay=(a.to(dev), r.to(dev)))
    fa, fr = errs(y, y_ref)
    if dtype == torch.float32:
        assert fa <= 2e-5, f"fwd {fa}"
    else:
        assert fa <= 2e-2 and fr <= 1e-2, f"fwd {fa} {fr}"
    if v_ref is None:
        return
    w = torch.randn(y_ref.shape, generator=g, dtype=torch.float64)
    (y.double() * w.to(dev)).sum().backward()
    (y_ref * w).sum().backward()
    ba, br = errs(v_dev.grad, v_ref.grad)
    if dtype == torch.float32:
        assert ba <= 1e-4, f"bwd {ba}"
    else:
        # gradients sum many rows and grow past 16, where one bf16 ulp is already 0.125:
        # bound the absolute error by the output magnitude (2^-7 relative) and keep rel-L2
        assert ba <= 2 ** -7 * max(1.0, v_ref.grad.abs().max().item()) and br <= 1e-2, f"bwd {ba} {br}"


@pytest.mark.parametrize("cfg", [(5, 3, 700, 64), (2, 2, 1024, 128), (3, 2, 1300, 64), (1, 1, 130, 128)],
                         ids=lambda c: f"B{c[0]}nf{c[1]}T{c[2]}hd{c[3]}")
def test_dense_bf16_pattern_on_tensor_core_ignores_upper_triangle(cfg):
    """TMA-staged lower-triangular GEMM: entries above the diagonal of the stored pattern never count
    (Y_i = sum_{j<=i} P_ij V_j, kernel/frozen_attn.py:51-89), batch rows share one pattern tile, ragged T."""
    from kernel import frozen_pv
    from saf_b200 import launch_count
    B, NF, T, hd = cfg
    S = ((T + 63) // 64) * 64 + 64
    g = torch.Generator().manual_seed(T + hd)
    patt = torch.rand(NF + 1, S, S, generator=g)
    patt = patt / patt.tril().sum(-1, keepdim=True).clamp_min(1e-6)     # rows of the lower triangle sum to one
    patt = patt.bfloat16()                                               # upper triangle left non-zero on purpose
    v = torch.randn(B, NF, T, hd, generator=g).bfloat16()
    idx = torch.arange(1, NF + 1, dtype=torch.int32)                     # pattern planes 1..NF
    ref = torch.matmul(patt[1:, :T, :T].float().tril(), v.float())
    n0 = launch_count()
    y = frozen_pv(patt.cuda(), v.cuda(), idx.cuda(), T)
    assert launch_count() - n0 == 1
    a, r = errs(y, ref)
    assert a <= 2e-2 and r <= 1e-2, f"max-abs {a} rel-l2 {r}"
