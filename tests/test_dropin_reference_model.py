"""The reference's unmodified nanogpt/model.py binds to this repository's `kernel` package when that package
is imported first, and -- on a GPU -- drives the CUDA kernels through it.  Needs a checkout of the reference
(named by SAF_REFERENCE_ROOT); skipped elsewhere."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the reference checkout is named by the environment; without it these tests are skipped
REF = os.environ.get("SAF_REFERENCE_ROOT") or ""
needs_reference = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "nanogpt")), reason="reference tree not present")


@needs_reference
def test_reference_model_imports_this_kernel_package():
    code = f"""
import sys
sys.path.insert(0, {os.path.join(ROOT, 'selective-attention-freezing_b200')!r})
import kernel
sys.path.insert(1, {os.path.join(REF, 'nanogpt')!r})
import model
assert model.fused_mixed_attn.__module__ == 'saf_b200.ops', model.fused_mixed_attn.__module__
assert model.linear_rows2.__module__ == 'saf_b200.ops'
import torch
cfg = model.GPTConfig(block_size=64, vocab_size=64, n_layer=1, n_head=2, n_embd=64, bias=False, dropout=0.0,
                      position_encoding='rope', rand_attn_dynamic=True)
attn = model.CausalSelfAttention(cfg).eval()
attn.freeze_heads([1], torch.rand(1, 64, 64))
rope = model.RotaryEmbedding(32, 64)(64, torch.float32)
with torch.no_grad():
    y = attn(torch.randn(1, 64, 64), rope=rope)      # CPU tensors: *_usable() is False, the reference's torch path runs
assert y.shape == (1, 64, 64)
print('ok')
"""
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr[-2000:]


@pytest.mark.gpu
@needs_reference
def test_reference_model_drives_the_cuda_kernels():
    """The reference's own CausalSelfAttention (unmodified source) on CUDA tensors over this `kernel` package:
    benchmark configuration 0 in fp32 and bf16 against the vectors the reference produced on its own eager path,
    its fused-dispatch counter rising (nanogpt/model.py:33-38, 975-976), and a training step whose frozen heads
    get exactly-zero Q/K weight-gradient rows."""
    code = f"""
import sys, os
import numpy as np
sys.path.insert(0, {ROOT!r})
sys.path.insert(0, {os.path.join(ROOT, 'selective-attention-freezing_b200')!r})
import kernel
from saf_b200 import ops
sys.path.insert(2, {os.path.join(REF, 'nanogpt')!r})
import model
import torch
from tests.golden import cases
assert model.fused_mixed_attn.__module__ == 'saf_b200.ops'
G = np.load({os.path.join(ROOT, 'tests', 'golden', 'reference_vectors.npz')!r})
B, T, C, H, fz, seed, kind = cases.LAYER_CASES['config0']
x, ws = cases.layer_inputs(B, T, C, H, seed)
patt, _ = cases.layer_patterns(kind, len(fz), T, seed)
want = torch.from_numpy(G['layer_config0_eager_sample'])
for dtype, tol in ((torch.float32, 1e-3), (torch.bfloat16, 2e-2)):
    cfg = model.GPTConfig(block_size=T, vocab_size=64, n_layer=1, n_head=H, n_embd=C, dropout=0.0, bias=False,
                          position_encoding='rope', rand_attn_dynamic=True, freeze_pattern_dtype='float32')
    attn = model.CausalSelfAttention(cfg, layer_idx=0)
    with torch.no_grad():
        for lin, w in zip((attn.q_proj, attn.k_proj, attn.v_proj, attn.c_proj), ws):
            lin.weight.copy_(w)
    attn.freeze_heads(fz, patt)
    attn = attn.cuda().to(dtype).eval()
    rope = model.RotaryEmbedding(C // H, T, base=10000.0)(T, dtype)
    rope = tuple(t.cuda() for t in rope)
    n0, l0 = model.fused_dispatch_count(), ops.launch_count()
    with torch.inference_mode():
        y = attn(x.cuda().to(dtype), rope=rope)
    torch.cuda.synchronize()
    assert model.fused_dispatch_count() == n0 + 1, 'the reference module did not take its fused path'
    assert ops.launch_count() > l0, 'the CUDA library did not launch'
    s, _, _ = cases.sample(y.float().cpu(), 24, 24)
    err = (s - want).abs().max().item()
    assert err <= tol, (str(dtype), err)
    print('forward', dtype, 'max-abs vs reference eager vectors', err)
# training step through a fresh reference module (its freeze caches above were built under inference mode and
# cannot enter autograd): linear_rows2 + fused backward of this package
attn = model.CausalSelfAttention(cfg, layer_idx=0)
with torch.no_grad():
    for lin, w in zip((attn.q_proj, attn.k_proj, attn.v_proj, attn.c_proj), ws):
        lin.weight.copy_(w)
attn.freeze_heads(fz, patt)
attn = attn.cuda().train()
rope = tuple(t.cuda() for t in model.RotaryEmbedding(C // H, T, base=10000.0)(T, torch.float32))
hd = C // H
for T_s in (320, T):       # B*T <= 1024 takes the reference's full-projection branch, the other its linear_rows2 branch
    xs = x[:, :T_s].cuda().requires_grad_(True)
    rope_s = tuple(t[..., :T_s, :] for t in rope)
    attn.zero_grad(set_to_none=True)
    n0 = model.fused_dispatch_count()
    y = attn(xs, rope=rope_s)
    y.square().sum().backward()
    assert model.fused_dispatch_count() == n0 + 1
    for h in range(H):
        g = attn.q_proj.weight.grad[h * hd:(h + 1) * hd].abs().max().item()
        assert (g == 0.0) == (h in fz), (T_s, h, g)
    print('training step T =', T_s, 'frozen Q rows exactly zero')
assert ops.device_status() == 0
print('ok')
"""
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=900)
    assert out.returncode == 0 and "ok" in out.stdout, (out.stdout[-1500:], out.stderr[-3000:])
    print(out.stdout)
