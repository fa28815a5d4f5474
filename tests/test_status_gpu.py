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


def test_mma_rate_probe_reports_the_tensor_pipe_pace():
    """The characterisation probe: a K = 16 step of a 128 x 128 product cannot beat 128 * 128 * 16 / 4096 = 64 cycles
    (nominal dense bf16 rate) and, alone on the SM, stays near it; N = 64 from a TMEM operand halves it."""
    from saf_b200 import _cabi, ops
    dev = torch.device("cuda")
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    cyc = torch.zeros(1, dtype=torch.int64, device=dev)
    reps = 128
    got = {}
    for form in (0, 1, 2):
        assert _cabi.lib.saf_selftest_mma_rate(form, reps, cyc.data_ptr(), ops._status_ptr(dev), stream) == 0
        assert ops.device_status(dev) == 0
        got[form] = cyc.item() / (8.0 * reps)
    assert 60 <= got[0] <= 90 and 60 <= got[1] <= 90, got
    assert 30 <= got[2] <= 50, got
    # with the neighbour warps on tensor memory and arithmetic and bulk copies landing in shared memory the
    # instructions still retire (slower), and nothing runs into a limit
    assert _cabi.lib.saf_selftest_mma_rate(0 + 512 + 1024 + 2048, reps, cyc.data_ptr(), ops._status_ptr(dev), stream) == 0
    assert ops.device_status(dev) == 0
    assert got[0] - 1 <= cyc.item() / (8.0 * reps) <= 400
    assert _cabi.lib.saf_selftest_mma_rate(-1, reps, cyc.data_ptr(), None, stream) == _cabi.SAF_ERR_INVALID
    assert _cabi.lib.saf_selftest_mma_rate(200, reps, cyc.data_ptr(), None, stream) == _cabi.SAF_ERR_INVALID
    assert _cabi.lib.saf_selftest_mma_rate(0, 0, cyc.data_ptr(), None, stream) == _cabi.SAF_ERR_INVALID
