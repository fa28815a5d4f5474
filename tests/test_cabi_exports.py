"""CPU-side checks of the C ABI: the library loads without a GPU, exports every symbol the header
declares, its structs have the size the ctypes mirror assumes, and bad arguments are refused with
an error code and a message before anything touches a device."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "saf_b200.h")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(saf_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported():
    from saf_b200 import _cabi
    names = declared_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(_cabi.lib, n), f"{n} declared in include/saf_b200.h but not exported"
    assert set(names) == set(_cabi.EXPORTS)


def test_struct_sizes_match_the_header(tmp_path):
    from saf_b200 import _cabi
    prog = tmp_path / "sz.c"
    prog.write_text('#include <stdio.h>\n#include "saf_b200.h"\nint main(){printf("%zu %zu %zu %zu %zu\\n",'
                    "sizeof(SafTensor),sizeof(SafMixedAttnArgs),sizeof(SafMixedAttnBwdArgs),sizeof(SafFrozenPvArgs),"
                    "sizeof(SafIndexedLinearArgs));return 0;}\n")
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(prog), "-o", str(exe)])
    got = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    want = [C.sizeof(t) for t in (_cabi.SafTensor, _cabi.SafMixedAttnArgs, _cabi.SafMixedAttnBwdArgs,
                                  _cabi.SafFrozenPvArgs, _cabi.SafIndexedLinearArgs)]
    assert got == want


def test_invalid_arguments_are_refused_before_launch():
    from saf_b200 import _cabi
    a = _cabi.SafMixedAttnArgs()
    a.struct_size = 12
    assert _cabi.lib.saf_mixed_attn_fwd(C.byref(a), None) == _cabi.SAF_ERR_INVALID
    assert "size mismatch" in _cabi.last_error()
    a.struct_size = C.sizeof(_cabi.SafMixedAttnArgs)
    a.dtype, a.B, a.H, a.T, a.HD, a.force_state = _cabi.SAF_BF16, 1, 2, 16, 256, -1
    assert _cabi.lib.saf_mixed_attn_fwd(C.byref(a), None) == _cabi.SAF_ERR_UNSUPPORTED
    assert "head_dim" in _cabi.last_error()
    a.HD = 64
    assert _cabi.lib.saf_mixed_attn_fwd(C.byref(a), None) == _cabi.SAF_ERR_INVALID   # null v / out
    assert _cabi.lib.saf_mixed_attn_fwd(None, None) == _cabi.SAF_ERR_INVALID
    p = _cabi.SafFrozenPvArgs()
    assert _cabi.lib.saf_frozen_pv_fwd(C.byref(p), None) == _cabi.SAF_ERR_INVALID
    ln = _cabi.SafIndexedLinearArgs()
    ln.struct_size = C.sizeof(_cabi.SafIndexedLinearArgs)
    ln.dtype, ln.M, ln.C, ln.n_weights, ln.n_slabs, ln.slab = _cabi.SAF_F16, 4, 8, 1, 1, 8
    assert _cabi.lib.saf_indexed_linear_fwd(C.byref(ln), None) == _cabi.SAF_ERR_UNSUPPORTED
    assert _cabi.lib.saf_decomposed_logz(None, None, None, 2, 8, None) == _cabi.SAF_ERR_INVALID
    assert _cabi.lib.saf_decomposed_logz(None, None, None, 0, 8, None) == _cabi.SAF_OK
    assert _cabi.lib.saf_pattern_normalisers(None, None, None, 2, 8, 4, None) == _cabi.SAF_ERR_INVALID
    assert _cabi.lib.saf_pattern_normalisers(None, None, None, 2, 8, 9, None) == _cabi.SAF_ERR_INVALID   # T > S
    assert "T > S" in _cabi.last_error()
    assert _cabi.lib.saf_pattern_param_grad(None, None) == _cabi.SAF_ERR_INVALID
    pg = _cabi.SafPatternGradArgs()
    assert _cabi.lib.saf_pattern_param_grad(C.byref(pg), None) == _cabi.SAF_ERR_INVALID
    assert "size mismatch" in _cabi.last_error()
    pg.struct_size = C.sizeof(_cabi.SafPatternGradArgs)
    pg.dtype, pg.B, pg.H, pg.T, pg.HD, pg.SD, pg.force_state = _cabi.SAF_BF16, 1, 2, 16, 64, 8, -1
    assert _cabi.lib.saf_pattern_param_grad(C.byref(pg), None) == _cabi.SAF_ERR_INVALID    # SD < T
    assert _cabi.lib.saf_attention_moments(None, None) == _cabi.SAF_ERR_INVALID
    st = _cabi.SafAttnStatsArgs()
    assert _cabi.lib.saf_attention_moments(C.byref(st), None) == _cabi.SAF_ERR_INVALID
    st.struct_size = C.sizeof(_cabi.SafAttnStatsArgs)
    st.dtype, st.B, st.U, st.T, st.HD = _cabi.SAF_BF16, 1, 1, 16, 64
    assert _cabi.lib.saf_attention_moments(C.byref(st), None) == _cabi.SAF_ERR_INVALID     # null q / k / mean
    st.T = 0
    assert _cabi.lib.saf_attention_moments(C.byref(st), None) == _cabi.SAF_OK
    pg.force_state = 1
    assert _cabi.lib.saf_pattern_param_grad(C.byref(pg), None) == _cabi.SAF_OK             # no such head trains


def test_operators_refuse_cpu_tensors():
    import torch
    import kernel
    v = torch.zeros(1, 2, 4, 8)
    assert kernel.fused_attn_usable(v) is False and kernel.frozen_pv_usable(v) is False
    with pytest.raises(RuntimeError, match="no CPU path"):
        kernel.fused_mixed_attn(v, v, v, None, torch.zeros(2, dtype=torch.int32))
    assert kernel.HAVE_TRITON and kernel.BAND_ROWS == 64


def test_host_helpers_match_oracle():
    import torch
    import kernel
    from oracle import saf_oracle as O
    g = torch.Generator().manual_seed(1)
    al, rh = torch.randn(3, 128, generator=g), torch.randn(3, 128, generator=g)
    assert torch.equal(kernel.make_rho_band(rh), O.make_rho_band(rh))
    assert torch.equal(kernel.decomp_logits(al, rh, rows=(5, 9)), O.decomp_logits(al, rh, rows=(5, 9)))
    assert O.max_abs(kernel.decomposed_logz(al, rh), O.decomposed_logz(al, rh)) <= 1e-6
    with pytest.raises(AssertionError, match="multiple of 64"):
        kernel.make_rho_band(torch.zeros(2, 100))


def test_slab_decomposition_and_pattern_classifier():
    import torch
    from saf_b200.ops import _slabs_of
    from saf_b200.attention import classify_sink_decay
    from oracle import saf_oracle as O
    rows = (torch.tensor([0, 1, 3, 6])[:, None] * 64 + torch.arange(64)).reshape(-1)
    slab, row0 = _slabs_of(rows)
    assert slab == 64 and row0 == [0, 64, 192, 384]
    slab, row0 = _slabs_of(torch.tensor([5, 6, 7, 20, 21, 22, 40, 41, 42]))
    assert slab == 3 and row0 == [5, 20, 40]
    a, r = O.sink_decay_params(3, seed=2)
    P = O.sink_decay_pattern(a, r, 200)
    for i in range(3):
        got = classify_sink_decay(P[i].float())
        assert got is not None and abs(got[0] - a[i].item()) < 1e-5 and abs(got[1] - r[i].item()) < 1e-5
    rnd = torch.rand(64, 64).tril()
    assert classify_sink_decay(rnd / rnd.sum(-1, keepdim=True)) is None


def test_per_device_bookkeeping_self_check():
    """Kernel attributes and SM counts are remembered per device ordinal (one process may drive several GPUs):
    the library's host-only self-check walks every ordinal, repeats, forgets one and probes out-of-range ones."""
    from saf_b200 import _cabi
    assert _cabi.lib.saf_selftest_per_device_once() == 0


def test_static_backward_validates_before_it_applies_its_limit():
    """A malformed struct is INVALID, not LIMIT; a call that cannot contain a live head has no size limit
    (it is refused later for its null tensors, not for its size)."""
    from saf_b200 import _cabi
    g = _cabi.SafMixedAttnBwdArgs()
    g.struct_size = C.sizeof(_cabi.SafMixedAttnBwdArgs)
    g.fwd.struct_size = 8                                   # wrong inner size, huge dims
    g.fwd.B, g.fwd.H, g.fwd.T, g.fwd.HD = 64, 64, 65536, 64
    assert _cabi.lib.saf_mixed_attn_bwd_static(C.byref(g), None) == _cabi.SAF_ERR_INVALID
    g.fwd.struct_size = C.sizeof(_cabi.SafMixedAttnArgs)
    g.fwd.dtype, g.fwd.force_state, g.fwd.U = _cabi.SAF_BF16, _cabi.SINK_DECAY, 0
    rc = _cabi.lib.saf_mixed_attn_bwd_static(C.byref(g), None)
    assert rc == _cabi.SAF_ERR_INVALID and "non-null" in _cabi.last_error()    # no LIMIT for a frozen-only call
    g.fwd.force_state, g.fwd.U = -1, 4
    dummy = (C.c_int32 * 64)()
    g.fwd.frozen = C.cast(dummy, C.c_void_p)
    g.fwd.v.ptr = g.fwd.out.ptr = g.fwd.q.ptr = g.fwd.k.ptr = C.cast(dummy, C.c_void_p)
    for t in (g.fwd.v, g.fwd.out, g.fwd.q, g.fwd.k):
        t.stride[3] = 1
    assert _cabi.lib.saf_mixed_attn_bwd_static(C.byref(g), None) == _cabi.SAF_ERR_LIMIT


def test_fft_normalisers_match_the_direct_ones_and_differentiate():
    """decomposed_logz_fft (the reference's O(T log T) normaliser, nanogpt/dynamic_freeze.py:330-361) equals the
    direct logsumexp the oracle is pinned on (for logit spreads the transform's fp64 round-off can resolve) and its
    gradient equals the dense one's."""
    import torch
    from oracle import saf_oracle as O
    from saf_b200 import decomposed_logz_fft
    g = torch.Generator().manual_seed(8)
    for scale in (0.8, 3.0):
        alpha = torch.randn(3, 192, generator=g) * scale
        rho = torch.randn(3, 192, generator=g) * scale - 0.02 * torch.arange(192)
        z = decomposed_logz_fft(alpha, rho)
        assert O.max_abs(z, O.decomposed_logz(alpha, rho)) <= 2e-5 * max(1.0, scale)
    a1, r1 = alpha.clone().requires_grad_(True), rho.clone().requires_grad_(True)
    decomposed_logz_fft(a1, r1).sum().backward()
    a2, r2 = alpha.clone().requires_grad_(True), rho.clone().requires_grad_(True)
    O.decomp_logits(a2, r2).logsumexp(-1).sum().backward()
    assert O.max_abs(a1.grad, a2.grad) <= 1e-4 and O.max_abs(r1.grad, r2.grad) <= 1e-4


def test_statistics_entry_accepts_the_shorter_struct_and_refuses_unknown_quantities():
    """SafAttnStatsArgs grew by `quantity` and `cell_m2`: a caller that stops at `status` (the struct as it was)
    is still served, any other size and any unknown quantity are INVALID; empty problems return before a launch."""
    import ctypes as C
    from saf_b200 import _cabi
    a = _cabi.SafAttnStatsArgs()
    full = C.sizeof(_cabi.SafAttnStatsArgs)
    short = _cabi.SafAttnStatsArgs.quantity.offset
    assert short < full
    a.B, a.U, a.T, a.HD = 0, 2, 128, 64            # empty batch: nothing to launch
    for size in (full, short):
        a.struct_size = size
        assert _cabi.lib.saf_attention_moments(C.byref(a), None) == 0
    a.struct_size = full - 4
    assert _cabi.lib.saf_attention_moments(C.byref(a), None) == _cabi.SAF_ERR_INVALID
    a.struct_size = full
    a.quantity = 7
    assert _cabi.lib.saf_attention_moments(C.byref(a), None) == _cabi.SAF_ERR_INVALID
    a.quantity = _cabi.STATS_LOGITS
    assert _cabi.lib.saf_attention_moments(C.byref(a), None) == 0
    # the probe validates its arguments before it looks for a device
    assert _cabi.lib.saf_selftest_mma_rate(0, 16, None, None, None) == _cabi.SAF_ERR_INVALID
    assert _cabi.lib.saf_selftest_mma_rate(0, 0, C.c_void_p(8), None, None) == _cabi.SAF_ERR_INVALID
    assert _cabi.lib.saf_selftest_mma_rate(5000, 16, C.c_void_p(8), None, None) == _cabi.SAF_ERR_INVALID
