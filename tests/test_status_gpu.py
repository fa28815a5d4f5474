"""The device-side error word: every wait inside the kernels is bounded, and a wait that runs out is reported
through an int32 word instead of a hang.  The failure is made by a wait nothing ever satisfies (1 ms limit);
nothing traps and the context stays usable."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_is_reported():
    from saf_b200 import _cabi, ops
    dev = torch.device("cuda")
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    word = torch.zeros(1, dtype=torch.int32, device=dev)
    assert _cabi.lib.saf_selftest_wait_timeout(word.data_ptr(), 1_000_000, stream) == 0
    torch.cuda.synchronize()
    assert word.item() == (6 | (99 << 8))
    # the first error sticks until it is cleared
    assert _cabi.lib.saf_selftest_wait_timeout(word.data_ptr(), 1_000_000, stream) == 0
    torch.cuda.synchronize()
    assert word.item() == (6 | (99 << 8))
    assert _cabi.lib.saf_selftest_wait_timeout(None, 1_000_000, stream) == _cabi.SAF_ERR_INVALID
    assert _cabi.lib.saf_selftest_wait_timeout(word.data_ptr(), 10**12, stream) == _cabi.SAF_ERR_INVALID


def test_operators_hand_the_status_word_to_the_library_and_the_check_raises():
    from saf_b200 import _cabi, ops
    dev = torch.device("cuda")
    # a healthy call leaves the word at zero
    x = torch.randn(256, 128, device=dev, dtype=torch.bfloat16)
    w = torch.randn(128, 128, device=dev, dtype=torch.bfloat16)
    ops.linear_rows(x, w, None, torch.arange(128, device=dev))
    assert ops.device_status(dev) == 0
    # the same word, made to carry a give-up, raises once and is cleared
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    assert _cabi.lib.saf_selftest_wait_timeout(ops._status_ptr(dev), 1_000_000, stream) == 0
    with pytest.raises(_cabi.SafError, match="self-test wait"):
        ops.device_status(dev)
    assert ops.device_status(dev) == 0
    # the context is still usable
    y = ops.linear_rows(x, w, None, torch.arange(128, device=dev))
    assert torch.isfinite(y.float()).all()
    a = SafArgsProbe.mixed(dev)
    assert a.status == ops._status_ptr(dev)


class SafArgsProbe:
    @staticmethod
    def mixed(dev):
        """The argument struct a fused_mixed_attn call fills (without launching anything)."""
        from saf_b200 import _cabi, ops
        v = torch.zeros(1, 2, 64, 64, device=dev, dtype=torch.bfloat16)
        frozen = torch.zeros(2, dtype=torch.int32, device=dev)
        a = _cabi.SafMixedAttnArgs()
        ops._fill_mixed(a, v, v, v, v, None, None, None, None, None, frozen, None, None, None, 0.125, None, None, [])
        return a
