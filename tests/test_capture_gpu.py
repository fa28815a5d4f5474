"""GPU parity of the fused controller statistics (saf_attention_moments) against the CPU oracle, which restates
the reference's reductions of the captured attention tensor (nanogpt/dynamic_freeze.py:96-193)."""
import pytest
import torch

from oracle import saf_oracle as O

pytestmark = pytest.mark.gpu

CASES = [
    # B, U, T, hd, batches
    (3, 2, 300, 64, 2),
    (2, 3, 517, 64, 3),        # ragged T, not a multiple of 4: scalar stores
    (1, 2, 1024, 128, 2),      # single-sample batches: zero within-batch M2, all variance from the merge
    (4, 1, 640, 128, 1),
    (5, 2, 256, 64, 2),        # more samples than ring stages
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"B{c[0]}U{c[1]}T{c[2]}d{c[3]}x{c[4]}")
def test_attention_moments_match_captured_reductions(case):
    from saf_b200.capture import AttentionMoments
    B, U, T, hd, nb = case
    gen = torch.Generator().manual_seed(T + hd + B)
    acc = AttentionMoments(U, T, "cuda")
    count, mean, m2 = 0, None, None
    negent = torch.zeros(U, dtype=torch.float64)
    for _ in range(nb):
        q = (torch.randn(B, U, T, hd, generator=gen) * 1.3).bfloat16()
        k = torch.randn(B, U, T, hd, generator=gen).bfloat16()
        att = O.attention_probs(q.double(), k.double())
        bn, bm, b2 = O.centered_batch_reduced_moments(att)
        count, mean, m2 = O.merge_reduced_moments(count, mean, m2, bn, bm, b2)
        negent += O.negative_entropy_sum(att)
        acc.update(q.cuda(), k.cuda())
    assert acc.count == count
    got_mean = acc.mean.cpu().double()
    # probabilities come from bf16 tensor-core scores with fp32 statistics: absolute error per cell well under 1e-3,
    # relative L2 of the whole mean matrix under 1e-3
    assert O.max_abs(got_mean, mean) <= 2e-3, O.max_abs(got_mean, mean)
    assert O.rel_l2(got_mean, mean) <= 2e-3
    assert not got_mean.triu(1).any()                       # exact zeros above the diagonal
    rel = ((acc.head_m2.cpu() - m2).abs() / m2.abs().clamp_min(1e-12)).max().item()
    assert rel <= 1e-2 or (m2.abs().max() < 1e-9 and acc.head_m2.abs().max() < 1e-6), rel
    rel_e = ((acc.neg_entropy.cpu() - negent).abs() / negent.abs()).max().item()
    assert rel_e <= 2e-3, rel_e
    var = acc.per_head_variance().cpu()
    ref_var = (m2 / max(count - 1, 1) / (T * T)).float()
    assert torch.allclose(var, ref_var, rtol=1e-2, atol=1e-12)
    kl = acc.mean_forward_kl().cpu()
    ref_kl = O.mean_forward_kl(negent, mean.float(), count)
    assert torch.allclose(kl, ref_kl, rtol=2e-2, atol=2e-4), (kl, ref_kl)


def test_attention_moments_golden_vectors():
    """On the reference's own vectors (q, k rounded to bf16 for the tensor cores)."""
    import os
    import numpy as np
    from saf_b200.capture import AttentionMoments
    G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))
    acc = AttentionMoments(2, 40, "cuda")
    # head_dim 16 has no tensor-core kernel: pad q, k with zero columns to 64 (scores unchanged) and keep the scale
    for bi in range(2):
        q = torch.from_numpy(G[f"st_q{bi}"])
        k = torch.from_numpy(G[f"st_k{bi}"])
        qp = torch.zeros(*q.shape[:-1], 64)
        kp = torch.zeros(*k.shape[:-1], 64)
        qp[..., :16], kp[..., :16] = q, k
        acc.update(qp.bfloat16().cuda(), kp.bfloat16().cuda(), sm_scale=16 ** -0.5)
        assert O.max_abs(acc.mean.cpu(), torch.from_numpy(G[f"st_mean{bi}"])) <= 2e-2
    m2 = torch.from_numpy(G["st_m2_1"])
    assert ((acc.head_m2.cpu() - m2).abs() / m2).max() <= 5e-2
    ne = torch.from_numpy(G["st_negent1"])
    assert ((acc.neg_entropy.cpu() - ne).abs() / ne.abs()).max() <= 2e-2


def test_attention_moments_refuses_unsupported():
    from saf_b200.capture import AttentionMoments
    from saf_b200._cabi import SafError
    acc = AttentionMoments(1, 64, "cuda")
    q = torch.randn(1, 1, 64, 32, device="cuda").bfloat16()
    with pytest.raises(SafError):
        acc.update(q, q)


def test_module_statistics_equal_reductions_of_the_eager_capture():
    """SafCausalSelfAttention.set_statistics on the fused bf16 path gives, for the live heads, what the reference's
    controller computes from the eager capture (`_last_attn`, nanogpt/dynamic_freeze.py:664-745)."""
    from types import SimpleNamespace
    from saf_b200.attention import SafCausalSelfAttention, rope_tables
    from saf_b200.capture import AttentionMoments, LogitMoments
    C_, H, T, B = 512, 8, 384, 3
    cfg = SimpleNamespace(n_embd=C_, n_head=H, block_size=T, bias=False, dropout=0.0, position_encoding="rope",
                          rand_attn_prior_repr="dense", freeze_pattern_dtype="bfloat16")
    torch.manual_seed(3)
    m = SafCausalSelfAttention(cfg).cuda().bfloat16().eval()
    a, r = O.sink_decay_params(2, seed=5)
    m.freeze_heads_sink_decay([1, 6], a.float().cuda(), r.float().cuda())
    live = [h for h in range(H) if h not in (1, 6)]
    cos, sin = rope_tables(C_ // H, T, device="cuda")
    rope = (cos.view(1, 1, T, -1), sin.view(1, 1, T, -1))
    acc = AttentionMoments(len(live), T, "cuda")
    lacc = LogitMoments(len(live), T, "cuda", with_var=True)
    count, mean, m2 = 0, None, None
    lcount, lmean, lm2 = 0, None, None
    negent = torch.zeros(len(live), dtype=torch.float64)
    for step in range(2):
        x = (torch.randn(B, T, C_, generator=torch.Generator().manual_seed(step)) * 2).bfloat16().cuda()
        with torch.no_grad():
            m.set_statistics(acc, lacc)
            y_fast = m(x, rope=rope)
            m.set_statistics(None)
            m.set_capture(True)
            y_eager = m(x, rope=rope)
            att = m._last_attn[:, live].float().cpu()
            lg = m._last_logits[:, live].float().cpu()
            m.set_capture(False)
        lbn, lbm, lb2 = O.centered_batch_moments(lg)
        lcount, lmean, lm2 = O.merge_moments(lcount, lmean, lm2, lbn, lbm, lb2)
        assert (y_fast.float() - y_eager.float()).abs().max() <= 5e-2
        bn, bm, b2 = O.centered_batch_reduced_moments(att)
        count, mean, m2 = O.merge_reduced_moments(count, mean, m2, bn, bm, b2)
        negent += O.negative_entropy_sum(att)
    assert acc.count == count == 2 * B
    # the eager capture holds bf16 probabilities, the fused path fp32 ones from bf16 q, k
    assert O.max_abs(acc.mean.cpu(), mean) <= 1e-2
    assert O.rel_l2(acc.mean.cpu(), mean) <= 2e-2
    assert ((acc.head_m2.cpu() - m2).abs() / m2).max() <= 5e-2
    assert ((acc.neg_entropy.cpu() - negent).abs() / negent.abs()).max() <= 2e-2
    # raw scores: the eager capture holds bf16 logits (relative error 2^-9 on scores of size up to ~10)
    assert lacc.count == lcount
    assert O.max_abs(lacc.mean.cpu(), lmean) <= 5e-2
    assert O.rel_l2(lacc.mean.cpu(), lmean) <= 1e-2
    assert O.rel_l2(lacc.m2.cpu().double(), lm2) <= 3e-2


@pytest.mark.parametrize("T", [1, 37, 129])
def test_attention_moments_small_and_ragged(T):
    from saf_b200.capture import AttentionMoments
    B, U, hd = 3, 2, 64
    gen = torch.Generator().manual_seed(T)
    q = torch.randn(B, U, T, hd, generator=gen).bfloat16()
    k = torch.randn(B, U, T, hd, generator=gen).bfloat16()
    att = O.attention_probs(q.double(), k.double())
    bn, bm, b2 = O.centered_batch_reduced_moments(att)
    acc = AttentionMoments(U, T, "cuda").update(q.cuda(), k.cuda())
    assert acc.count == B
    assert O.max_abs(acc.mean.cpu().double(), bm) <= 2e-3
    assert (acc.head_m2.cpu() - b2).abs().max() <= 1e-2 * max(b2.abs().max().item(), 1e-6) + 1e-9
    ne = O.negative_entropy_sum(att)
    assert (acc.neg_entropy.cpu() - ne).abs().max() <= 2e-3 * max(ne.abs().max().item(), 1.0)


LOGIT_CASES = [
    # B, U, T, hd, batches, with_var
    (3, 2, 300, 64, 2, True),
    (2, 3, 517, 64, 3, True),      # ragged T, not a multiple of 4: scalar stores
    (1, 2, 384, 128, 2, True),     # single-sample batches: all of M2 comes from the merge
    (4, 1, 640, 128, 1, False),
    (5, 2, 256, 64, 2, False),     # more samples than ring stages, mean only
    (2, 1, 37, 64, 2, True),
]


@pytest.mark.parametrize("case", LOGIT_CASES, ids=lambda c: f"B{c[0]}U{c[1]}T{c[2]}d{c[3]}x{c[4]}v{int(c[5])}")
def test_logit_moments_match_captured_reductions(case):
    """LogitMoments against the restated _centered_batch_moments / _merge_moments of the raw scores
    (nanogpt/dynamic_freeze.py:62-93, :721-737), upper triangle included."""
    from saf_b200.capture import LogitMoments
    B, U, T, hd, nb, with_var = case
    gen = torch.Generator().manual_seed(7 * T + hd + B)
    acc = LogitMoments(U, T, "cuda", with_var=with_var)
    count, mean, m2 = 0, None, None
    for _ in range(nb):
        q = (torch.randn(B, U, T, hd, generator=gen) * 1.3).bfloat16()
        k = torch.randn(B, U, T, hd, generator=gen).bfloat16()
        lg = O.raw_logits(q.double(), k.double())
        bn, bm, b2 = O.centered_batch_moments(lg)
        count, mean, m2 = O.merge_moments(count, mean, m2, bn, bm, b2)
        acc.update(q.cuda(), k.cuda())
    assert acc.count == count
    # fp32 accumulation of exact bf16 products on the tensor core, fp32 statistics: scores are O(1..10)
    assert O.max_abs(acc.mean.cpu().double(), mean) <= 1e-4, O.max_abs(acc.mean.cpu().double(), mean)
    assert acc.mean.triu(1).abs().max() > 0 or T == 1       # nothing masked
    if with_var:
        got = acc.m2.cpu().double()
        assert O.max_abs(got, m2) <= 1e-4 * max(m2.abs().max().item(), 1.0), O.max_abs(got, m2)
        assert O.rel_l2(got, m2) <= 1e-4
        std = acc.std().cpu().double()
        ref = (m2 / max(count - 1, 1)).clamp_min(0).sqrt()
        assert O.max_abs(std, ref) <= 1e-3
    else:
        assert acc.m2 is None


def test_logit_moments_golden_vectors():
    """On the reference's own vectors (q, k rounded to bf16 for the tensor cores, head_dim 16 padded with zeros)."""
    import os
    import numpy as np
    from saf_b200.capture import LogitMoments
    G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))
    acc = LogitMoments(2, 40, "cuda", with_var=True)
    for bi in range(2):
        q = torch.from_numpy(G[f"st_q{bi}"])
        k = torch.from_numpy(G[f"st_k{bi}"])
        qp = torch.zeros(*q.shape[:-1], 64)
        kp = torch.zeros(*k.shape[:-1], 64)
        qp[..., :16], kp[..., :16] = q, k
        acc.update(qp.bfloat16().cuda(), kp.bfloat16().cuda(), sm_scale=16 ** -0.5)
        # the bf16 rounding of q and k moves a score of size ~1 by up to ~2e-2
        assert O.max_abs(acc.mean.cpu(), torch.from_numpy(G[f"lg_mean{bi}"])) <= 3e-2
    m2 = torch.from_numpy(G["lg_m2_1"])
    assert O.rel_l2(acc.m2.cpu().double(), m2) <= 2e-2


def test_logit_moments_leave_probability_statistics_alone():
    """The two quantities share a kernel: a probability update after a logit update still matches the oracle."""
    from saf_b200.capture import AttentionMoments, LogitMoments
    B, U, T, hd = 2, 2, 200, 64
    gen = torch.Generator().manual_seed(11)
    q = torch.randn(B, U, T, hd, generator=gen).bfloat16()
    k = torch.randn(B, U, T, hd, generator=gen).bfloat16()
    LogitMoments(U, T, "cuda").update(q.cuda(), k.cuda())
    acc = AttentionMoments(U, T, "cuda").update(q.cuda(), k.cuda())
    att = O.attention_probs(q.double(), k.double())
    assert O.max_abs(acc.mean.cpu().double(), att.mean(0)) <= 2e-3
