"""Shapes of the benchmark workloads (plain data: this file imports nothing, so a process that must not load
the CUDA library -- the CPU reference arm of the benchmark -- can read it by path)."""

WORKLOADS = {
    # name: layers, heads, head_dim, frozen heads per layer, sequence, batch per GPU
    # c0: the single fp32 layer the reference can run on a CPU (heads 2, 5, 8 frozen)
    "c0": dict(n_layer=1, n_head=12, head_dim=64, n_frozen=3, T=1024, B=2, rope_base=10000.0, dtype="float32",
               frozen_heads=[2, 5, 8]),
    "c1": dict(n_layer=12, n_head=12, head_dim=64, n_frozen=3, T=4096, B=16, rope_base=10000.0),
    "c2": dict(n_layer=12, n_head=12, head_dim=64, n_frozen=3, T=16384, B=4, rope_base=10000.0),
    "c3": dict(n_layer=24, n_head=16, head_dim=128, n_frozen=4, T=8192, B=2, rope_base=10000.0),
    # Qwen2.5-1.5B-shaped grouped-query prefill: 12 query heads on 2 KV heads, q/k/v bias, gated MLP 8960
    "c4": dict(n_layer=28, n_head=12, n_kv=2, head_dim=128, n_frozen=3, T=8192, B=8, rope_base=1000000.0,
               hidden=1536, mlp=8960, qkv_bias=True),
    "tiny_gqa": dict(n_layer=2, n_head=6, n_kv=2, head_dim=64, n_frozen=2, T=384, B=2, rope_base=1000000.0,
                     hidden=256, mlp=512, qkv_bias=True),
    # the reference's own ~1B recipe (nanogpt/config/train_gpt_1b_rope.py): 32 layers, 16 heads x 96
    "r1b": dict(n_layer=32, n_head=16, head_dim=96, n_frozen=4, T=8192, B=2, rope_base=10000.0),
    "tiny": dict(n_layer=2, n_head=4, head_dim=64, n_frozen=1, T=512, B=2, rope_base=10000.0),
}
