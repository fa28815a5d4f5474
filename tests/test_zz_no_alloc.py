"""The allocation-free backward entry point, called straight through the C ABI.

Who needs it: a host that cannot give the library fresh device memory per call -- an inference or
training runtime that laid out its whole device arena ahead of time, a plugin boundary that only ever
passes the operator's own tensors, or a call site where allocating could synchronise the GPU.  For them
`saf_mixed_attn_bwd_static` keeps the one scratch buffer of the backward (delta, one fp32 per
batch x head x row) in a fixed 4 MiB array inside the library.

Checks: same dQ/dK/dV as the regular entry point (which gets a torch-allocated delta) on two calls in a
row -- the second call finds the first call's values in the shared array and must not care; sizes past
the limit are refused with a clear message.
Collected last on purpose (file name), so a failure here cannot hide another test's result."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(seed, B=2, H=6, T=333, hd=64, dtype=torch.float32):
    dev = "cuda"
    g = torch.Generator().manual_seed(seed)
    states = [0, 1, 0, 3, 0, 0]
    live = [h for h in range(H) if states[h] == 0]
    hidx = torch.zeros(H, dtype=torch.int32)
    for s, h in enumerate(live):
        hidx[h] = s
    q = torch.randn(B, len(live), T, hd, generator=g).to(dtype).to(dev)
    k = torch.randn(B, len(live), T, hd, generator=g).to(dtype).to(dev)
    v = torch.randn(B, H, T, hd, generator=g).to(dtype).to(dev)
    do = torch.randn(B, H, T, hd, generator=g).to(dtype).to(dev)
    p = torch.rand(H, T, T, generator=g).tril()
    patt = (p / p.sum(-1, keepdim=True)).to(dev)
    sd = (torch.full((H,), 0.2, device=dev), torch.full((H,), 0.9, device=dev))
    frozen = torch.tensor(states, dtype=torch.int32, device=dev)
    return q, k, v, do, patt, frozen, hidx.to(dev), sd


def _backward(entry, q, k, v, do, patt, frozen, hidx, sd, out, lse, with_delta):
    from saf_b200 import _cabi, ops
    B, H, T, hd = v.shape
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.empty_like(v)
    delta = torch.empty(B, H, T, device=v.device) if with_delta else None
    g, keep = _cabi.SafMixedAttnBwdArgs(), []
    g.struct_size = C.sizeof(_cabi.SafMixedAttnBwdArgs)
    ops._fill_mixed(g.fwd, q, k, v, out, lse, patt, None, None, None, frozen, hidx, None, None, hd ** -0.5, None, sd, keep)
    g.dout, g.dq, g.dk, g.dv, g.delta = ops._st(do), ops._st(dq), ops._st(dk), ops._st(dv), ops._st(delta)
    rc = entry(C.byref(g), ops._stream(v))
    return rc, dq, dk, dv


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_static_scratch_backward_matches_regular_entry_twice(dtype):
    from saf_b200 import _cabi, ops
    lib = _cabi.lib
    for seed in (1, 2):                                   # two calls in a row share the static array
        q, k, v, do, patt, frozen, hidx, sd = _problem(seed, dtype=dtype)
        B, H, T, hd = v.shape
        out = torch.empty_like(v)
        lse = torch.empty(B, H, T, device=v.device)
        a, keep = _cabi.SafMixedAttnArgs(), []
        ops._fill_mixed(a, q, k, v, out, lse, patt, None, None, None, frozen, hidx, None, None, hd ** -0.5, None, sd, keep)
        _cabi.check(lib.saf_mixed_attn_fwd(C.byref(a), ops._stream(v)))
        rc, dq0, dk0, dv0 = _backward(lib.saf_mixed_attn_bwd, q, k, v, do, patt, frozen, hidx, sd, out, lse, True)
        _cabi.check(rc)
        # no delta tensor is passed: the scratch is the library's own fixed array
        rc, dq1, dk1, dv1 = _backward(lib.saf_mixed_attn_bwd_static, q, k, v, do, patt, frozen, hidx, sd, out, lse, False)
        _cabi.check(rc)
        torch.cuda.synchronize()
        # same kernels, same inputs: the tolerance of the other backward tests (2e-4 fp32, 2e-1 bf16) is met with zero error
        for name, x, y in (("dq", dq0, dq1), ("dk", dk0, dk1), ("dv", dv0, dv1)):
            err = (x.float() - y.float()).abs().max().item()
            assert err <= (2e-4 if dtype == torch.float32 else 2e-1), f"{name}: {err}"
            assert torch.isfinite(y.float()).all()
        assert dq1.abs().max().item() > 0


def test_static_scratch_rejects_sizes_past_the_limit():
    from saf_b200 import _cabi
    g = _cabi.SafMixedAttnBwdArgs()
    g.struct_size = C.sizeof(_cabi.SafMixedAttnBwdArgs)
    # an otherwise well-formed call (the entry validates its arguments before it looks at the size) with live heads
    g.fwd.struct_size = C.sizeof(_cabi.SafMixedAttnArgs)
    g.fwd.dtype, g.fwd.force_state, g.fwd.HD, g.fwd.U = _cabi.SAF_BF16, -1, 64, 16
    g.fwd.B, g.fwd.H, g.fwd.T = 8, 16, 16384          # 2,097,152 rows > 1,048,576
    word = (C.c_int32 * 16)()
    for t in (g.fwd.q, g.fwd.k, g.fwd.v, g.fwd.out):
        t.ptr = C.cast(word, C.c_void_p)              # never dereferenced: the call is refused on the host
        t.stride[3] = 1
    g.fwd.frozen = C.cast(word, C.c_void_p)
    assert _cabi.lib.saf_mixed_attn_bwd_static(C.byref(g), None) == _cabi.SAF_ERR_LIMIT
    assert "static scratch" in _cabi.last_error()
