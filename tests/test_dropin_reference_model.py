"""The reference's unmodified nanogpt/model.py binds to this repository's `kernel` package when that package
is imported first.  Needs the reference tree (present in the build container only); skipped elsewhere."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the reference checkout: named by the environment, else looked for beside this repository
REF = os.environ.get("SAF_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "nanogpt")), reason="reference tree not present")
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
