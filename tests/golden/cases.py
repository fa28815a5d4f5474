"""Seeded input builders shared by the fixture generator (which runs the reference) and the tests
(which run the oracle and the CUDA library).  Everything is drawn from torch CPU generators, so
both sides rebuild bit-identical inputs from the seed alone."""
import torch

LAYER_CASES = {
    # name: (B, T, C, H, frozen heads, seed, kind)
    "config0": (2, 1024, 768, 12, [2, 5, 8], 1337, "sink_decay"),          # benchmark configuration 0
    "small_sink": (2, 192, 128, 4, [1, 3], 11, "sink_decay"),
    "small_rand": (1, 97, 128, 4, [0], 12, "random"),
}
DECOMP_LAYER = ("small_decomp", 2, 128, 128, 4, [0], [2], 13)   # name, B, T, C, H, dense, decomposed, seed


def layer_inputs(B, T, C, H, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, T, C, generator=g)
    ws = [torch.randn(C, C, generator=g) * 0.02 for _ in range(4)]   # q, k, v, c_proj
    return x, ws


def sink_decay_params(n, seed):
    g = torch.Generator().manual_seed(seed)
    a = 0.05 + 0.25 * torch.rand(n, generator=g, dtype=torch.float64)
    r = 0.8 + 0.19 * torch.rand(n, generator=g, dtype=torch.float64)
    return a, r


def sink_decay_pattern(a, r, T):
    """fp64 (n, T, T): a[j=0] + (1-a) r^(i-j) / Z_i on the causal triangle."""
    i = torch.arange(T, dtype=torch.float64)
    dist = i[:, None] - i[None, :]
    out = []
    for aa, rr in zip(a.tolist(), r.tolist()):
        dec = torch.where(dist >= 0, torch.tensor(rr, dtype=torch.float64) ** dist.clamp(min=0),
                          torch.zeros((), dtype=torch.float64))
        p = (1.0 - aa) * dec / dec.sum(-1, keepdim=True)
        p[:, 0] += aa
        out.append(p)
    return torch.stack(out)


def random_pattern(n, T, seed):
    g = torch.Generator().manual_seed(seed)
    p = torch.rand(n, T, T, generator=g).tril()
    return p / p.sum(-1, keepdim=True)


def layer_patterns(kind, n, T, seed):
    if kind == "sink_decay":
        a, r = sink_decay_params(n, seed + 1)
        return sink_decay_pattern(a, r, T).float(), (a, r)
    return random_pattern(n, T, seed + 1), None


def decomp_vectors(H, S, seed, scale=0.8):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(H, S, generator=g) * scale, torch.randn(H, S, generator=g) * scale


def op_inputs(B, H, T, hd, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(B, H, T, hd, generator=g) for _ in range(3)]


def sample(t, rows=16, cols=16):
    """Deterministic sub-sample of the last two dims + whole-tensor checksums."""
    T, D = t.shape[-2], t.shape[-1]
    ri = torch.linspace(0, T - 1, min(rows, T)).long()
    ci = torch.linspace(0, D - 1, min(cols, D)).long()
    return t[..., ri, :][..., ci].contiguous(), t.double().sum().item(), t.double().abs().sum().item()
