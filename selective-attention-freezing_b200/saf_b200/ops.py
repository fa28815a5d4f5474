"""Torch-facing operators over the C ABI.

These keep the reference's call signatures (kernel/fused_attn.py:650-652,
qwen/kernel/fused_attn.py:667-669, kernel/frozen_attn.py:185,
kernel/indexed_linear.py:125-141) and autograd behaviour: dQ/dK come back in the
compact live-head shape, pattern buffers never receive gradient, unselected
weight rows get exactly-zero gradient.  Torch is used for allocation, autograd
bookkeeping and the current stream only; every FLOP runs in libsaf_b200.
"""
import ctypes as C
import math
import os
import weakref

import torch

from . import _cabi
from ._cabi import (SafTensor, SafMixedAttnArgs, SafMixedAttnBwdArgs, SafFrozenPvArgs, SafIndexedLinearArgs,
                    check, lib)

BAND_ROWS = 64  # kernel/fused_attn.py:58 (kept for callers; these kernels read rho directly)

_DT = {torch.float32: _cabi.SAF_F32, torch.bfloat16: _cabi.SAF_BF16, torch.float16: _cabi.SAF_F16}


def _dt(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError("unsupported dtype %s (float32, bfloat16, float16)" % t.dtype)


def _st(t, nd=None):
    s = SafTensor()
    if t is None:
        s.ptr = None
        return s
    s.ptr = t.data_ptr()
    for i, x in enumerate(t.stride()):
        s.stride[i] = x
    return s


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(t):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _call(t, fn, *args):
    """Run one library entry on tensor t's device and current stream.  The library works on the CURRENT device
    (per-device kernel attributes, SM count, tensor maps), so a tensor that lives on another GPU of this process
    makes its device current for the call."""
    if t.device.index is not None and t.device.index != torch.cuda.current_device():
        with torch.cuda.device(t.device):
            rc = fn(*args, _stream(t))
    else:
        rc = fn(*args, _stream(t))
    check(rc)
    if _CHECK_EVERY_CALL:
        device_status(t.device)


# ---------------------------------------------------------------------------
# device-side error word
# ---------------------------------------------------------------------------
# Every wait inside the kernels is bounded.  A wait that runs out records (kind | where << 8) in an int32 word
# the call was given, stops issuing work, skips its stores and returns.  One word per device, handed to every call.
_STATUS = {}
_CHECK_EVERY_CALL = os.environ.get("SAF_B200_CHECK_STATUS", "0") not in ("", "0")
_DEV_KINDS = {1: "TMA producer wait", 2: "MMA issuer wait", 3: "epilogue wait", 4: "softmax / compute wait",
              5: "scan wait", 6: "self-test wait"}


def _status_ptr(device):
    """Device address of this device's status word (allocated and zeroed at first use; make that first use
    before a CUDA graph capture -- any warm-up call does)."""
    key = torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    w = _STATUS.get(key)
    if w is None:
        w = _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return w.data_ptr()


def device_status(device=None, clear=True):
    """Reads the device's status word (synchronises with that device) and raises SafError if a kernel gave up
    on a wait since the last check; returns 0 otherwise.  Outputs of a call that gave up are undefined.
    Set SAF_B200_CHECK_STATUS=1 to run this check after every library call (debugging; it synchronises)."""
    key = torch.cuda.current_device() if device is None else torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    w = _STATUS.get(key)
    if w is None:
        return 0
    code = int(w.item())
    if code == 0:
        return 0
    if clear:
        w.zero_()
    kind, where = code & 0xff, code >> 8
    raise _cabi.SafError(_cabi.SAF_ERR_CUDA, "a kernel gave up on a bounded wait: %s (site %d, raw 0x%x); the outputs of "
                         "that call are undefined" % (_DEV_KINDS.get(kind, "kind %d" % kind), where, code))


def _require_cuda(t, name):
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor: this package has no CPU path" % name)


def _ver(t):
    """Version counter of a tensor; inference tensors have none (they cannot be modified in place
    outside inference mode either), so they count as version 0."""
    return 0 if t.is_inference() else t._version


# host copies of small device index tensors, refreshed when the tensor changes
_HOST_CACHE = {}


def host_ints(t):
    """Host list of a small device int tensor, cached per tensor object and version.

    One device->host copy per change of the tensor (the reference pays the same
    sync in its cache refresh, nanogpt/model.py:846-858).  The cache entry holds a
    weak reference to the tensor object, so a new tensor that happens to reuse
    the address of a dead one never sees its values.  Returns None while a CUDA
    graph is being captured and the value is not cached yet."""
    if t is None:
        return None
    hit = _HOST_CACHE.get(id(t))
    if hit is not None and hit[0]() is t and hit[1] == _ver(t):
        return hit[2]
    if t.is_cuda and torch.cuda.is_current_stream_capturing():
        return None
    vals = [int(x) for x in t.detach().cpu().tolist()]
    if len(_HOST_CACHE) > 1024:
        for k in [k for k, v in _HOST_CACHE.items() if v[0]() is None]:
            del _HOST_CACHE[k]
        if len(_HOST_CACHE) > 1024:
            _HOST_CACHE.clear()
    _HOST_CACHE[id(t)] = (weakref.ref(t), _ver(t), vals)
    return vals


def launch_count():
    """Kernel launches enqueued by the library in this process."""
    return int(lib.saf_launch_count())


# ---------------------------------------------------------------------------
# host helpers kept from the reference's import surface (pure index algebra)
# ---------------------------------------------------------------------------
def _toeplitz_windows(rho, width, cols=None):
    """W of shape (H, width, S) with W[h, w, u] = rho[h, u - w] (-inf where u < w): row w is rho shifted right
    by w.  Built without index arithmetic: rho is padded with `width - 1` leading -inf values, reversed, and its
    length-S sliding windows (a strided view, `unfold`) are read back to front.  cols = (u0, u1) materialises
    only those columns."""
    H, S = rho.shape
    u0, u1 = (0, S) if cols is None else cols
    pad = rho.new_full((H, width - 1), float("-inf"))
    rev = torch.cat([pad, rho], dim=1).flip(1)               # rev[k] = padded[S + width - 2 - k]
    win = rev.unfold(1, S, 1)                                 # (H, width, S) view: win[h, i, u] = rev[h, i + u]
    return win[:, :, S - u1:S - u0].flip(2)                   # [h, i, u - u0] = padded[width - 1 - i + u] = rho[u - i]


def make_rho_band(rho):
    """(H, S) -> (H, 64, S) with band[h, r, u] = rho[h, r - u + (S - 64)], -inf outside
    (kernel/fused_attn.py:65-80).  The CUDA kernels index rho directly and do not
    consume the band; it is produced for callers that store it as a buffer."""
    H, S = rho.shape
    assert S % BAND_ROWS == 0, \
        f"decomposed prior buffer length {S} must be a multiple of {BAND_ROWS}"
    # band row r, read right to left, is rho shifted by (63 - r): reverse the columns of the shifted copies
    shifted = _toeplitz_windows(rho, BAND_ROWS)               # [h, w, u] = rho[h, u - w]
    return shifted.flip(1).flip(2).contiguous()               # [h, r, u] = rho[h, (S - 1 - u) - (63 - r)]


def decomp_logits(alpha, rho, rows=None):
    """L[h,i,j] = alpha[h,j] + rho[h,i-j], -inf above the diagonal (kernel/fused_attn.py:83-98)."""
    H, S = alpha.shape
    r0, r1 = (0, S) if rows is None else rows
    # column j of the Toeplitz matrix rho[i - j] is rho shifted down by j; the -inf padding of the shifted copies
    # is the causal mask
    shifted = _toeplitz_windows(rho, S, cols=(r0, r1))        # [h, j, i - r0] = rho[h, i - j]
    return alpha[:, None, :] + shifted.transpose(1, 2)


@torch.no_grad()
def decomposed_logz(alpha, rho, chunk=None):
    """z[h,i] = logsumexp_{j<=i}(alpha[h,j] + rho[h,i-j]) (kernel/fused_attn.py:101-116).
    CUDA tensors run the library kernel (one warp per row, fp32); CPU tensors use
    the chunked torch formula so freeze-time code keeps working off-device."""
    if alpha.is_cuda:
        a = alpha.detach().float().contiguous()
        r = rho.detach().float().contiguous()
        z = torch.empty_like(a)
        H, S = a.shape
        _call(a, lib.saf_decomposed_logz, a.data_ptr(), r.data_ptr(), z.data_ptr(), H, S)
        return z.to(alpha.dtype)
    H, S = alpha.shape
    if chunk is None:
        chunk = max(1, int(2 ** 27 // max(H * S, 1)))
    z = torch.empty_like(alpha)
    for i0 in range(0, S, chunk):
        i1 = min(i0 + chunk, S)
        z[:, i0:i1] = decomp_logits(alpha, rho, rows=(i0, i1)).logsumexp(-1)
    return z


def decomposed_logz_fft(alpha, rho):
    """The same row normalisers, z[h,i] = log sum_{j<=i} exp(alpha[h,j]) exp(rho[h,i-j]), as the first T entries of a
    linear convolution computed with FFTs in O(T log T) (nanogpt/dynamic_freeze.py:330-361).  Differentiable in
    alpha and rho (the reference's prior fitter optimises through it); any device.  Both factors are shifted by
    their detached row maxima and the transform runs in fp64: one global shift cannot keep an early prefix, whose
    terms may sit far below a late maximum, above fp32 round-off of the transform.  Like the reference's, it resolves
    prefixes down to about 1e-13 of the largest term; beyond that spread use decomposed_logz."""
    if alpha.ndim != 2 or alpha.shape != rho.shape:
        raise ValueError("alpha and rho must have matching (N, T) shapes")
    T = alpha.shape[1]
    wide = torch.float64
    a_max = alpha.detach().to(wide).amax(dim=-1, keepdim=True)
    r_max = rho.detach().to(wide).amax(dim=-1, keepdim=True)
    ea = torch.exp(alpha.to(wide) - a_max)
    er = torch.exp(rho.to(wide) - r_max)
    n = 1
    while n < 2 * T - 1:                       # zero padding makes the circular product a linear one
        n *= 2
    conv = torch.fft.irfft(torch.fft.rfft(ea, n=n) * torch.fft.rfft(er, n=n), n=n)[..., :T]
    z = torch.log(conv.clamp_min(torch.finfo(wide).tiny)) + a_max + r_max
    return z.to(alpha.dtype)


def fused_attn_usable(q):
    """True when the CUDA library can serve this tensor (kernel/fused_attn.py:61-62)."""
    return bool(q.is_cuda)


def frozen_pv_usable(v):
    """kernel/frozen_attn.py:44-46."""
    return bool(v.is_cuda)


# ---------------------------------------------------------------------------
# fused mixed attention
# ---------------------------------------------------------------------------
def _fill_mixed(a, q, k, v, out, lse, patt, alpha, rho, z, frozen, hidx, pidx, kvidx, sm_scale, rope, sink_decay,
                keep):
    B, Hv, T, HD = v.shape
    H = frozen.numel()
    a.struct_size = C.sizeof(SafMixedAttnArgs)
    a.dtype = _dt(v)
    a.B, a.H, a.T, a.HD = B, H, T, HD
    a.U = q.shape[1] if q is not None else 0
    a.HKV = Hv if kvidx is not None else 0
    a.force_state = -1
    a.status = _status_ptr(v.device)
    a.sm_scale = float(sm_scale)
    a.q, a.k, a.v, a.out = _st(q), _st(k), _st(v), _st(out)
    a.lse = _st(lse)
    if patt is not None:
        a.patt = _st(patt)
        a.S = patt.shape[1]
        a.patt_dtype = _dt(patt)
    if alpha is not None:
        a.alpha, a.rho, a.z = _st(alpha), _st(rho), _st(z)
        a.SD = alpha.shape[1]
        a.dec_dtype = _dt(alpha)
    a.frozen = _ptr(frozen)
    a.hidx = _ptr(hidx)
    a.pidx = _ptr(pidx)
    a.kvidx = _ptr(kvidx)
    hs = host_ints(frozen)
    if hs is not None:
        arr = (C.c_int32 * len(hs))(*hs)
        keep.append(arr)
        a.frozen_host = C.cast(arr, C.POINTER(C.c_int32))
    if sink_decay is not None:
        a.sd_alpha, a.sd_rho = _ptr(sink_decay[0]), _ptr(sink_decay[1])
    if rope is not None:
        a.rope = 1
        a.rope_cos, a.rope_sin = _ptr(rope[0]), _ptr(rope[1])


# attention-op timing probe: CUDA-event pairs around every forward attention launch, the same
# protocol as the reference's AttnOpProbe (qwen/nanogpt/bench_qwen_prefill_triton.py:186-225)
_ATTN_EVENTS = None


def attention_timing(enable):
    """Start (True) or stop (False) collecting event pairs; stopping returns the collected list."""
    global _ATTN_EVENTS
    got = _ATTN_EVENTS
    _ATTN_EVENTS = [] if enable else None
    return got


class _FusedMixedAttn(torch.autograd.Function):
    """Mirror of kernel/fused_attn.py:626-647."""

    @staticmethod
    def forward(ctx, q, k, v, patt, alpha, rho, z, frozen, hidx, pidx, kvidx, sm_scale, rope, sink_decay,
                token_major_out=False):
        gqa = kvidx is not None
        B, Hv, T, HD = v.shape
        H = frozen.numel()
        if gqa and token_major_out:
            # (B, H, T, hd) view of a (B, T, H, hd) buffer: out.transpose(1, 2).reshape(B, T, H * hd) is then free
            out = torch.empty((B, T, H, HD), device=v.device, dtype=v.dtype).transpose(1, 2)
        elif gqa:
            out = torch.empty((B, H, T, HD), device=v.device, dtype=v.dtype)  # qwen/kernel/fused_attn.py:586
        else:
            out = torch.empty_like(v)  # keeps v's strides (kernel/fused_attn.py:575)
        need_bwd = any(t is not None and t.requires_grad for t in (q, k, v))
        lse = torch.empty((B, H, T), device=v.device, dtype=torch.float32) if need_bwd else None
        a, keep = SafMixedAttnArgs(), []
        _fill_mixed(a, q, k, v, out, lse, patt, alpha, rho, z, frozen, hidx, pidx, kvidx, sm_scale, rope,
                    sink_decay, keep)
        if v.dtype == torch.bfloat16 and HD in (64, 96, 128) and q is not None and q.size(1) > 0:
            # tile queue of the persistent forward kernel: two zeroed ints owned by this call (torch's allocator
            # hands the block out again only in stream order, and a CUDA graph capture gives it a private pool)
            sched = torch.zeros(2, dtype=torch.int32, device=v.device)
            keep.append(sched)
            a.sched = sched.data_ptr()
        if _ATTN_EVENTS is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _call(v, lib.saf_mixed_attn_fwd, C.byref(a))
            e1.record()
            _ATTN_EVENTS.append((e0, e1))
        else:
            _call(v, lib.saf_mixed_attn_fwd, C.byref(a))
        ctx.save_for_backward(q, k, v, patt, alpha, rho, z, frozen, hidx, pidx, out, lse,
                              *(rope or ()), *(sink_decay or ()))
        ctx.sm_scale = sm_scale
        ctx.has_rope = rope is not None
        ctx.has_sd = sink_decay is not None
        ctx.gqa = gqa
        return out

    @staticmethod
    def backward(ctx, do):
        if ctx.gqa:
            raise NotImplementedError("fused_mixed_attn backward with kvidx (GQA) is not implemented")
        saved = ctx.saved_tensors
        q, k, v, patt, alpha, rho, z, frozen, hidx, pidx, out, lse = saved[:12]
        rest = list(saved[12:])
        rope = (rest.pop(0), rest.pop(0)) if ctx.has_rope else None
        sink_decay = (rest.pop(0), rest.pop(0)) if ctx.has_sd else None
        B, H, T, HD = v.shape
        do = do.contiguous()
        dq = torch.zeros_like(q)  # frozen heads keep exactly zero (kernel/fused_attn.py:597-598)
        dk = torch.zeros_like(k)
        dv = torch.empty_like(v)
        delta = torch.empty((B, H, T), device=v.device, dtype=torch.float32)
        g, keep = SafMixedAttnBwdArgs(), []
        g.struct_size = C.sizeof(SafMixedAttnBwdArgs)
        _fill_mixed(g.fwd, q, k, v, out, lse, patt, alpha, rho, z, frozen, hidx, pidx, None, ctx.sm_scale, rope,
                    sink_decay, keep)
        g.dout, g.dq, g.dk, g.dv, g.delta = _st(do), _st(dq), _st(dk), _st(dv), _st(delta)
        _call(v, lib.saf_mixed_attn_bwd, C.byref(g))
        return (dq, dk, dv) + (None,) * 12


class _RotatedCopy(torch.autograd.Function):
    """Rotated private copy of q or k, (B, N, T, hd) -> same shape (token-major strides), with the adjoint rotation
    of the gradient in backward.  Used when `fused_mixed_attn(rope=)` is asked for on tensors the tensor-core
    kernels take: they read q, k by TMA straight into the MMA operands, so the rotation happens once here instead
    of once per (query tile, key tile) pair."""

    @staticmethod
    def _rotate(y, B, N, T, hd, cos, sin, inverse):
        _call(y, lib.saf_rope_slabs, y.data_ptr(), N * hd, B * T, N, hd, T, None, cos.data_ptr(), sin.data_ptr(), _dt(y),
                                 inverse)

    @staticmethod
    def forward(ctx, x, cos, sin):
        B, N, T, hd = x.shape
        y = x.detach().transpose(1, 2).contiguous()
        if y.data_ptr() == x.data_ptr():
            y = y.clone()
        _RotatedCopy._rotate(y, B, N, T, hd, cos, sin, 0)
        ctx.save_for_backward(cos, sin)
        return y.transpose(1, 2)

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        B, N, T, hd = g.shape
        g2 = g.transpose(1, 2).contiguous()
        if g2.data_ptr() == g.data_ptr():
            g2 = g2.clone()
        _RotatedCopy._rotate(g2, B, N, T, hd, cos, sin, 1)
        return g2.transpose(1, 2), None, None


def fused_mixed_attn(q, k, v, patt, frozen, hidx=None, pidx=None,
                     sm_scale=None, alpha=None, rho=None, z=None,
                     rho_band=None, validate=True, kvidx=None, *, rope=None, sink_decay=None,
                     token_major_out=False):
    """Causal attention over all heads at once; frozen heads use a fixed pattern.

    Same positional/keyword contract as the reference (kernel/fused_attn.py:650-734;
    `kvidx` as in qwen/kernel/fused_attn.py:667-768):
      v (B,H,T,hd) [GQA: (B,HKV,T,hd)], q,k (B,U,T,hd) live heads only [GQA k: (B,HKV,T,hd)],
      patt (P,S,S) or None, frozen (H,) int32 states 0 live / 1 dense / 2 decomposed,
      hidx/pidx/kvidx (H,) int32 maps, alpha/rho/z (H,S); rho_band is accepted and ignored
      (these kernels index rho directly).
    Additions (keyword-only, default off):
      rope=(cos, sin): fp32 (T,hd) tables; q and k are rotated while they are loaded (CUDA-core kernels) or once
        into private copies ahead of the tensor-core kernels (bf16, head_dim 64 / 128).
      sink_decay=(a, r): fp32 (H,) tensors; heads with state 3 use the structured
        pattern a[j=0] + (1-a) r^(i-j)/Z_i through an O(T) scan.
      token_major_out=True (with kvidx): the (B, H, T, hd) result is a view of a (B, T, H, hd) buffer instead of the
        reference's contiguous tensor, so the caller's transpose(1, 2).reshape(B, T, H * hd) copies nothing.
    alpha / rho that require grad receive their exact gradients (z is then recomputed from them).
    """
    _require_cuda(v, "v")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(v.size(-1))
    train_patterns = (alpha is not None and torch.is_grad_enabled()
                      and (alpha.requires_grad or (rho is not None and rho.requires_grad)))
    if train_patterns:
        # learnable alpha / rho (supplement/trainable_patterns.py:62-88): the normalisers follow the current
        # parameter values, the fused call sees detached buffers, and PatternGradient adds their gradients
        if kvidx is not None:
            raise NotImplementedError("trainable patterns with kvidx (GQA) are not implemented")
        from . import trainable_patterns as _tp
        alpha_p, rho_p = alpha, rho
        z = _tp.current_normalisers(alpha, rho, v.shape[-2])
        alpha, rho = alpha.detach(), rho.detach()
    if alpha is not None and z is None:
        z = decomposed_logz(alpha, rho)
    if validate:
        assert q.ndim == k.ndim == v.ndim == 4, "q, k, v must be 4-D"
        B, Hv, T, HD = v.shape
        H = frozen.numel()
        if kvidx is None:
            assert q.shape == k.shape, "q and k must have the same compact shape"
            assert Hv == H, "v must hold one head per entry of frozen"
        else:
            assert k.shape == v.shape, "with kvidx, k and v share the (B, HKV, T, HD) shape"
            assert kvidx.shape == (H,) and kvidx.dtype == torch.int32, "kvidx must be (H,) int32"
        assert q.shape[0] == B and q.shape[2:] == (T, HD), \
            "q/k batch, sequence, and head dimensions must match v"
        for name, t in (("hidx", hidx), ("pidx", pidx)):
            if t is not None:
                assert t.shape == (H,), "frozen, hidx, and pidx must have one entry per output head"
                assert t.dtype == torch.int32, "frozen, hidx, and pidx must be int32"
                assert t.device == v.device, "head-state and index tensors must be on v.device"
        assert frozen.dtype == torch.int32, "frozen, hidx, and pidx must be int32"
        assert frozen.device == v.device, "head-state and index tensors must be on v.device"
        assert q.device == k.device == v.device, "q, k, v must share a device"
        states = host_ints(frozen)
        if patt is not None:
            assert patt.ndim == 3 and patt.shape[1] >= T and patt.shape[2] >= T, \
                "patt must have shape (P, S, S) with S >= T"
            assert patt.device == v.device, "patt must be on v.device"
            if pidx is None:
                assert patt.shape[0] >= H, "identity pattern mapping requires at least H pattern rows"
            elif states is not None and 1 in states:
                pl = host_ints(pidx)
                dense = [pl[h] for h in range(H) if states[h] == 1]
                assert min(dense) >= 0 and max(dense) < patt.shape[0], \
                    "pidx for dense-frozen heads must index patt"
        else:
            assert states is None or 1 not in states, "dense-frozen heads require patt"
        if alpha is not None:
            assert rho is not None and alpha.shape == rho.shape == z.shape, \
                "alpha, rho, and z must have matching (H, S) shapes"
            assert alpha.shape[0] == H and alpha.shape[1] >= T, \
                "decomposed buffers must have shape (H, S) with S >= T"
            assert alpha.device == rho.device == z.device == v.device, \
                "decomposed buffers must be on v.device"
        else:
            assert states is None or 2 not in states, "decomposed-frozen heads require alpha/rho/z"
        if sink_decay is None:
            assert states is None or 3 not in states, "sink-decay heads require sink_decay=(a, r)"
    if (rope is not None and q.dtype == torch.bfloat16 and v.size(-1) in (64, 96, 128) and q.size(1) > 0
            and rope[0].dtype == torch.float32 and rope[0].is_contiguous() and rope[1].is_contiguous()):
        # tensor-core kernels: rotate q, k once into private copies (see _RotatedCopy) and run without in-kernel RoPE
        q = _RotatedCopy.apply(q, rope[0], rope[1])
        k = _RotatedCopy.apply(k, rope[0], rope[1])
        rope = None
    out = _FusedMixedAttn.apply(q, k, v, patt, alpha, rho, z, frozen, hidx, pidx, kvidx, sm_scale, rope,
                                sink_decay, token_major_out)
    if train_patterns:
        out = _tp.PatternGradient.apply(out, v, alpha_p, rho_p, z, frozen)
    return out


# ---------------------------------------------------------------------------
# frozen heads only
# ---------------------------------------------------------------------------
def _fill_pv(p, patt, v, y, fz_idx, T, sink_decay):
    B, nf, _, hd = v.shape
    p.struct_size = C.sizeof(SafFrozenPvArgs)
    p.dtype = _dt(v)
    p.B, p.NF, p.T, p.HD = B, nf, T, hd
    if patt is not None:
        p.patt = _st(patt)
        p.patt_dtype = _dt(patt)
        p.S = patt.shape[1]
    p.v, p.y = _st(v), _st(y)
    p.status = _status_ptr(v.device)
    p.fz_idx = _ptr(fz_idx)
    if sink_decay is not None:
        p.sd_alpha, p.sd_rho = _ptr(sink_decay[0]), _ptr(sink_decay[1])


class _FrozenPV(torch.autograd.Function):
    """Mirror of kernel/frozen_attn.py:168-182."""

    @staticmethod
    def forward(ctx, patt, v, fz_idx, T, sink_decay):
        B, nf, Tv, hd = v.shape
        y = torch.empty((B, nf, T, hd), device=v.device, dtype=v.dtype)
        p = SafFrozenPvArgs()
        _fill_pv(p, patt, v, y, fz_idx, T, sink_decay)
        _call(v, lib.saf_frozen_pv_fwd, C.byref(p))
        ctx.save_for_backward(patt, fz_idx, *(sink_decay or ()))
        ctx.has_sd = sink_decay is not None
        ctx.v_shape, ctx.v_dtype, ctx.T = v.shape, v.dtype, T
        return y

    @staticmethod
    def backward(ctx, dy):
        saved = ctx.saved_tensors
        patt, fz_idx = saved[0], saved[1]
        sink_decay = (saved[2], saved[3]) if ctx.has_sd else None
        dy = dy.contiguous()
        dv = torch.empty(ctx.v_shape, device=dy.device, dtype=ctx.v_dtype)
        if ctx.v_shape[2] != ctx.T:
            dv.zero_()
        p = SafFrozenPvArgs()
        _fill_pv(p, patt, dy, dv, fz_idx, ctx.T, sink_decay)
        _call(dy, lib.saf_frozen_pv_bwd, C.byref(p))
        return None, dv, None, None, None


def frozen_pv(patt, v, fz_idx, T, *, sink_decay=None):
    """y[b,f] = patt[fz_idx[f], :T, :T] @ v[b,f] -> (B, nf, T, hd)  (kernel/frozen_attn.py:185-192).
    sink_decay=(a, r) fp32 (nf,) tensors switch to the structured scan; patt may then be None."""
    _require_cuda(v, "v")
    return _FrozenPV.apply(patt, v, fz_idx, T, sink_decay)


# ---------------------------------------------------------------------------
# indexed linear
# ---------------------------------------------------------------------------
_SLAB_CACHE = {}


def _slabs_of(rows, want=None):
    """Decompose a unique-row index tensor into equal runs of consecutive rows.

    Returns (slab, [row0...]); `want` forces the slab width (every run must be a
    multiple of it).  One device->host copy per distinct index tensor object and version."""
    if want is not None:
        slab, row0 = _slabs_of(rows)
        if slab % want and want % slab:
            raise ValueError("rows do not form runs of %d consecutive rows" % want)
        if slab == want:
            return slab, row0
        if slab > want:
            return want, [r + o for r in row0 for o in range(0, slab, want)]
        step = want // slab   # merge consecutive blocks of one run
        merged = row0[::step]
        for i, r in enumerate(merged):
            if row0[i * step:(i + 1) * step] != list(range(r, r + want, slab)):
                raise ValueError("rows do not form runs of %d consecutive rows" % want)
        return want, merged
    hit = _SLAB_CACHE.get(id(rows))
    if hit is not None and hit[0]() is rows and hit[1] == _ver(rows):
        return hit[2]
    if rows.is_cuda and torch.cuda.is_current_stream_capturing():
        raise RuntimeError("index tensor not seen before CUDA graph capture: run one warm-up call first")
    r = [int(x) for x in rows.detach().cpu().tolist()]
    runs, start = [], 0
    for i in range(1, len(r) + 1):
        if i == len(r) or r[i] != r[i - 1] + 1:
            runs.append((r[start], i - start))
            start = i
    slab = 0
    for _, n in runs:
        slab = math.gcd(slab, n)
    slab = max(slab, 1)
    if slab % 64 == 0:
        slab = 64   # the tensor-core GEMM addresses weights in 64-row blocks
    row0 = []
    for first, n in runs:
        row0.extend(range(first, first + n, slab))
    out = (slab, row0)
    if len(_SLAB_CACHE) > 1024:
        _SLAB_CACHE.clear()
    _SLAB_CACHE[id(rows)] = (weakref.ref(rows), _ver(rows), out)
    return out


def _autocast_args(x, *ts):
    """kernel/indexed_linear.py:18-25."""
    dev = "cuda" if x.is_cuda else "cpu"
    if torch.is_autocast_enabled(dev):
        dt = torch.get_autocast_dtype(dev)
        return (x.to(dt),) + tuple(None if t is None else t.to(dt) for t in ts)
    return (x,) + ts


def _lin_args(x2, weights, biases, slab, slab_weight, slab_row0, keep, transposed=False, rope=None, T=0,
              slab_rope=None):
    a = SafIndexedLinearArgs()
    a.struct_size = C.sizeof(SafIndexedLinearArgs)
    a.dtype = _dt(weights[0])
    a.M, a.C = x2.shape[0], (weights[0].shape[0] if transposed else weights[0].shape[1])
    a.n_weights = len(weights)
    a.n_slabs, a.slab = len(slab_row0), slab
    a.T = T
    a.x, a.ldx = x2.data_ptr(), x2.stride(0)
    a.status = _status_ptr(x2.device)
    for i, w in enumerate(weights):
        a.weights[i] = w.data_ptr()
        a.biases[i] = _ptr(biases[i]) if biases is not None else None
        if transposed:
            a.ldw[i], a.cdw[i], a.rows_w[i] = w.stride(1), w.stride(0), w.shape[1]
        else:
            a.ldw[i], a.cdw[i], a.rows_w[i] = w.stride(0), w.stride(1), w.shape[0]
    sw = (C.c_int32 * len(slab_weight))(*slab_weight)
    sr = (C.c_int32 * len(slab_row0))(*slab_row0)
    keep += [sw, sr]
    a.slab_weight = C.cast(sw, C.POINTER(C.c_int32))
    a.slab_row0 = C.cast(sr, C.POINTER(C.c_int32))
    if slab_rope is not None:
        sp = (C.c_int32 * len(slab_rope))(*slab_rope)
        keep.append(sp)
        a.slab_rope = C.cast(sp, C.POINTER(C.c_int32))
        a.rope_cos, a.rope_sin = _ptr(rope[0]), _ptr(rope[1])
    return a


def _as_2d(x):
    x2 = x.reshape(-1, x.size(-1))
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    return x2


def _check_lin(x, *ws):
    _require_cuda(x, "x")
    for w in ws:
        if w.dtype != x.dtype:
            raise TypeError("x and weights must share a dtype (got %s and %s)" % (x.dtype, w.dtype))
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("indexed linear takes float32 or bfloat16")


class _RowSlicedLinearN(torch.autograd.Function):
    """[F.linear(x, w_i[rows], b_i[rows]) for each weight] stacked on features, weights read in place.
    Mirror of kernel/indexed_linear.py:28-55 (one weight) and :86-122 (two weights)."""

    @staticmethod
    def forward(ctx, x, rows, nw, rope, *wb):
        # rope = None or (cos, sin, T, head_dim): every slab is one head and is rotated in the epilogue
        weights, biases = list(wb[:nw]), list(wb[nw:])
        _check_lin(x, *weights)
        slab, row0 = _slabs_of(rows, want=rope[3] if rope is not None else None)
        x2 = _as_2d(x)
        n_per = len(row0)
        sw = [i for i in range(nw) for _ in range(n_per)]
        sr = row0 * nw
        keep = []
        if rope is not None:
            a = _lin_args(x2, weights, biases, slab, sw, sr, keep, rope=rope[:2], T=rope[2], slab_rope=[1] * len(sr))
        else:
            a = _lin_args(x2, weights, biases, slab, sw, sr, keep)
        out = torch.empty((x2.shape[0], nw * n_per * slab), device=x.device, dtype=x.dtype)
        a.out, a.ldo = out.data_ptr(), out.stride(0)
        _call(x, lib.saf_indexed_linear_fwd, C.byref(a))
        ctx.save_for_backward(x, rows, *weights, *(rope[:2] if rope is not None else ()))
        ctx.nw = nw
        ctx.rope = None if rope is None else (rope[2], rope[3])
        ctx.has_bias = [b is not None for b in biases]
        return out.view(*x.shape[:-1], out.shape[-1])

    @staticmethod
    def backward(ctx, dout):
        x, rows = ctx.saved_tensors[:2]
        nw = ctx.nw
        weights = list(ctx.saved_tensors[2:2 + nw])
        slab, row0 = _slabs_of(rows, want=ctx.rope[1] if ctx.rope is not None else None)
        n_per = len(row0)
        sw = [i for i in range(nw) for _ in range(n_per)]
        sr = row0 * nw
        dout2 = _as_2d(dout)
        x2 = _as_2d(x)
        if ctx.rope is not None:
            # gradient w.r.t. the un-rotated projection: adjoint rotation of a private copy
            cos, sin = ctx.saved_tensors[2 + nw:4 + nw]
            dout2 = dout2.clone() if dout2.data_ptr() == dout.data_ptr() else dout2
            _call(x, lib.saf_rope_slabs, dout2.data_ptr(), dout2.stride(0), dout2.shape[0], len(sr), slab, ctx.rope[0],
                                     None, cos.data_ptr(), sin.data_ptr(), _dt(dout2), 1)
        dx = None
        grads_w = [None] * nw
        grads_b = [None] * nw
        if ctx.needs_input_grad[0]:
            keep = []
            a = _lin_args(x2, weights, None, slab, sw, sr, keep)
            dx2 = torch.empty_like(x2)
            _call(x, lib.saf_indexed_linear_bwd_dx, C.byref(a), dout2.data_ptr(), dout2.stride(0), dx2.data_ptr(),
                                                dx2.stride(0), None)
            dx = dx2.view(x.shape)
        # forward's arguments: x, rows, nw, rope, then the weights, then the biases
        need_w = any(ctx.needs_input_grad[4 + i] for i in range(nw))
        need_b = any(ctx.has_bias[i] and ctx.needs_input_grad[4 + nw + i] for i in range(nw))
        if need_w or need_b:
            # rows of no slab stay exactly zero (kernel/indexed_linear.py:112-115)
            dws = [torch.zeros_like(w) for w in weights]
            dbs = [torch.zeros(w.size(0), device=dout.device, dtype=dout.dtype) if ctx.has_bias[i] else None
                   for i, w in enumerate(weights)]
            keep = []
            a = _lin_args(x2, dws, dbs, slab, sw, sr, keep)
            _call(x, lib.saf_indexed_linear_bwd_dw, C.byref(a), dout2.data_ptr(), dout2.stride(0))
            grads_w, grads_b = dws, dbs
        return (dx, None, None, None, *grads_w, *grads_b)


class _ColPermutedLinear(torch.autograd.Function):
    """F.linear(y, weight[:, cols], bias), cols a full permutation (kernel/indexed_linear.py:58-83)."""

    @staticmethod
    def forward(ctx, y, weight, bias, cols):
        _check_lin(y, weight)
        slab, col0 = _slabs_of(cols)
        y2 = _as_2d(y)
        keep = []
        # selection rows = columns of W: address W through its transpose
        a = _lin_args(y2, [weight], None, slab, [0] * len(col0), col0, keep, transposed=True)
        out = torch.empty((y2.shape[0], weight.shape[0]), device=y.device, dtype=y.dtype)
        _call(y, lib.saf_indexed_linear_bwd_dx, C.byref(a), y2.data_ptr(), y2.stride(0), out.data_ptr(), out.stride(0),
                                            _ptr(bias))
        ctx.save_for_backward(y, weight, cols)
        ctx.has_bias = bias is not None
        return out.view(*y.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dout):
        y, weight, cols = ctx.saved_tensors
        slab, col0 = _slabs_of(cols)
        dout2 = _as_2d(dout)
        y2 = _as_2d(y)
        dy = dw = db = None
        if ctx.needs_input_grad[0]:
            keep = []
            a = _lin_args(dout2, [weight], None, slab, [0] * len(col0), col0, keep, transposed=True)
            dy2 = torch.empty_like(y2)
            a.out, a.ldo = dy2.data_ptr(), dy2.stride(0)
            # dy[m, j] = sum_o dout[m, o] W[o, cols[j]]: a forward product over the transposed weight
            _call(y, lib.saf_indexed_linear_fwd, C.byref(a))
            dy = dy2.view(y.shape)
        if ctx.needs_input_grad[1]:
            dw = torch.empty_like(weight)  # full permutation: every column written
            keep = []
            a = _lin_args(dout2, [dw], None, slab, [0] * len(col0), col0, keep, transposed=True)
            # dW[o, cols[j]] = sum_m dout[m, o] y[m, j]:  "dout" role = y, "x" role = dout
            _call(y, lib.saf_indexed_linear_bwd_dw, C.byref(a), y2.data_ptr(), y2.stride(0))
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dout2.sum(0)
        return dy, dw, db, None


def linear_rows(x, weight, bias, rows):
    """Linear over a unique-row slice of `weight` (kernel/indexed_linear.py:125-128)."""
    x, weight, bias = _autocast_args(x, weight, bias)
    return _RowSlicedLinearN.apply(x, rows, 1, None, weight, bias)


def linear_rows2(x, w1, w2, b1, b2, rows, *, rope=None, head_dim=None):
    """(..., 2R) = [x @ w1[rows]^T + b1[rows], x @ w2[rows]^T + b2[rows]] (kernel/indexed_linear.py:131-135).

    Addition (keyword-only, default off): rope=(cos, sin) fp32 (T, head_dim) tables with `rows` made of whole
    heads of `head_dim` rows: every head of the result is rotated (nanogpt/model.py:57-99) in the GEMM
    epilogue; the backward applies the adjoint rotation to the incoming gradient first."""
    x, w1, w2, b1, b2 = _autocast_args(x, w1, w2, b1, b2)
    rp = None
    if rope is not None:
        if head_dim is None:
            head_dim = rope[0].shape[-1]
        rp = (rope[0], rope[1], x.shape[-2], head_dim)
    return _RowSlicedLinearN.apply(x, rows, 2, rp, w1, w2, b1, b2)


def linear_permuted_cols(y, weight, bias, cols):
    """Linear over a column-permuted `weight` (kernel/indexed_linear.py:138-141)."""
    y, weight, bias = _autocast_args(y, weight, bias)
    return _ColPermutedLinear.apply(y, weight, bias, cols)


def qkv_projection(x, wq, wk, wv, live_heads, head_dim, rope=None, T=None, biases=None, grouped=False):
    """One GEMM for [Q(live heads) | K(live heads) | V(all heads)], weights read in place,
    RoPE applied to the Q and K slabs in the GEMM epilogue when `rope=(cos, sin)` is given.

    Inference-side fusion of what the reference does with a cached gathered weight,
    F.linear and separate RoPE kernels (nanogpt/model.py:981-990, 1007-1008).
    grouped=True is the grouped-query layout: wk and wv hold the HKV raw KV heads, every one of them is projected
    (several query heads share one, so none can be dropped, qwen/nanogpt/hybrid_prior_attention.py:551-557) and
    the result is [Q(live heads) | K(HKV heads) | V(HKV heads)].
    Returns (M, (2U + H) * head_dim) [grouped: (U + 2 HKV) * head_dim]; no autograd (use linear_rows2 when training)."""
    _check_lin(x, wq, wk, wv)
    x2 = _as_2d(x)
    H = wv.shape[0] // head_dim
    U = len(live_heads)
    if grouped:
        HK = wk.shape[0] // head_dim
        sw = [0] * U + [1] * HK + [2] * H
        sr = [h * head_dim for h in live_heads] + [h * head_dim for h in range(HK)] + [h * head_dim for h in range(H)]
        srope = ([1] * (U + HK) + [0] * H) if rope is not None else None
    else:
        sw = [0] * U + [1] * U + [2] * H
        sr = [h * head_dim for h in live_heads] * 2 + [h * head_dim for h in range(H)]
        srope = ([1] * (2 * U) + [0] * H) if rope is not None else None
    keep = []
    a = _lin_args(x2, [wq, wk, wv], biases, head_dim, sw, sr, keep, rope=rope,
                  T=(T if T is not None else x.shape[-2]), slab_rope=srope)
    out = torch.empty((x2.shape[0], len(sw) * head_dim), device=x.device, dtype=x.dtype)
    a.out, a.ldo = out.data_ptr(), out.stride(0)
    _call(x, lib.saf_indexed_linear_fwd, C.byref(a))
    return out


# ---------------------------------------------------------------------------
# rest of the transformer block around the attention path (inference, bf16)
# ---------------------------------------------------------------------------
def layer_norm(x, weight, bias=None, eps=1e-5):
    """F.layer_norm(x, (C,), weight, bias, eps) as the reference's LayerNorm does (nanogpt/model.py:45-54).
    No autograd (prefill path)."""
    _require_cuda(x, "x")
    x2 = _as_2d(x)
    w = weight if weight.dtype == x.dtype else weight.to(x.dtype)
    b = None if bias is None else (bias if bias.dtype == x.dtype else bias.to(x.dtype))
    out = torch.empty_like(x2)
    _call(x, lib.saf_layernorm_fwd, x2.data_ptr(), x2.stride(0), w.data_ptr(), _ptr(b), out.data_ptr(), out.stride(0),
                                x2.shape[0], x2.shape[1], float(eps), _dt(x2))
    return out.view(x.shape)


def rms_norm(x, weight, eps=1e-6):
    """x / sqrt(mean(x^2) + eps) * weight over the last dimension (the RMSNorm of Qwen-shaped blocks).
    No autograd (prefill path)."""
    _require_cuda(x, "x")
    x2 = _as_2d(x)
    w = weight if weight.dtype == x.dtype else weight.to(x.dtype)
    out = torch.empty_like(x2)
    _call(x, lib.saf_rmsnorm_fwd, x2.data_ptr(), x2.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0),
          x2.shape[0], x2.shape[1], float(eps), _dt(x2))
    return out.view(x.shape)


_ALL_ROWS64 = {}
_GATE_UP_ROWS = {}


def linear_swiglu(x, w_gate, w_up):
    """silu(x @ w_gate^T) * (x @ w_up^T) in ONE GEMM launch: 64-row blocks of the two weights alternate in the
    tile's B operand, and the epilogue multiplies each gate block with its up block before the store -- the
    gated MLP of the Qwen-shaped blocks without the (M, 2 * hidden) intermediate.  bf16, hidden a multiple of
    128, no bias, no autograd."""
    _check_lin(x, w_gate, w_up)
    if x.dtype != torch.bfloat16:
        raise TypeError("linear_swiglu runs on the bf16 tensor-core path only")
    N = w_gate.shape[0]
    if w_up.shape != w_gate.shape or N % 128:
        raise ValueError("gate and up weights must share a shape with a multiple of 128 rows")
    x2 = _as_2d(x)
    tab = _GATE_UP_ROWS.get(N)
    if tab is None:
        sw, sr = [], []
        for r0 in range(0, N, 64):
            sw += [0, 1]
            sr += [r0, r0]
        tab = _GATE_UP_ROWS[N] = (sw, sr)
    keep = []
    a = _lin_args(x2, [w_gate, w_up], None, 64, tab[0], tab[1], keep)
    out = torch.empty((x2.shape[0], N), device=x.device, dtype=x.dtype)
    a.out, a.ldo = out.data_ptr(), out.stride(0)
    a.act = _cabi.ACT_SWIGLU
    _call(x, lib.saf_indexed_linear_fwd, C.byref(a))
    return out.view(*x.shape[:-1], N)


def linear_act(x, weight, bias=None, act=None, residual=None):
    """[residual +] act(F.linear(x, weight, bias)) in one GEMM launch: the c_fc + GELU and c_proj + residual
    steps of the reference's MLP / Block (nanogpt/model.py:1202-1207, 1237-1240).  act: None or "gelu"
    (exact erf form, nn.GELU()).  bf16 tensors, output features a multiple of 64; no autograd."""
    _check_lin(x, weight)
    if x.dtype != torch.bfloat16:
        raise TypeError("linear_act runs on the bf16 tensor-core path only")
    N = weight.shape[0]
    if N % 64:
        raise ValueError("output features must be a multiple of 64")
    x2 = _as_2d(x)
    row0 = _ALL_ROWS64.get(N)
    if row0 is None:
        row0 = _ALL_ROWS64[N] = list(range(0, N, 64))
    keep = []
    a = _lin_args(x2, [weight], [bias] if bias is not None else None, 64, [0] * len(row0), row0, keep)
    out = torch.empty((x2.shape[0], N), device=x.device, dtype=x.dtype)
    a.out, a.ldo = out.data_ptr(), out.stride(0)
    if act is not None:
        if act != "gelu":
            raise ValueError("unknown activation %r" % (act,))
        a.act = _cabi.ACT_GELU
    if residual is not None:
        r2 = _as_2d(residual)
        if r2.shape != out.shape or r2.dtype != out.dtype:
            raise ValueError("residual must match the output")
        a.residual, a.ldr = r2.data_ptr(), r2.stride(0)
        keep.append(r2)
    _call(x, lib.saf_indexed_linear_fwd, C.byref(a))
    return out.view(*x.shape[:-1], N)
