"""Categorical sampling (``kuiops_multinomial_f32``).  PyTorch's multinomial cannot be matched
draw for draw (its stream is private to its kernels), so parity has two parts: the kernel against
the CPU restatement of its own documented stream and summation order, bit for bit; and the
distribution of the draws against the probabilities (chi-square), next to PyTorch's own draws."""
import numpy as np
import pytest
import torch

from oracle import kuiops_oracle as O


def test_philox_known_answers():
    """Known-answer vectors of Philox4x32-10 as published with the Random123 library."""
    assert O.philox4x32_10((0, 0, 0, 0), (0, 0)) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert O.philox4x32_10((0xffffffff,) * 4, (0xffffffff,) * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert O.philox4x32_10((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0)) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_oracle_never_draws_weightless_entries_and_follows_the_distribution():
    rng = np.random.default_rng(0)
    P = rng.random((4, 700)).astype(np.float32)
    P[0, :650] = 0
    P[1] = 0
    P[1, 333] = 2.5                                   # one-hot
    P[2, ::2] = 0
    draws = O.multinomial(P, 64, seed=7, offset=12)
    assert (draws[0] >= 650).all() and (draws[1] == 333).all() and (draws[2] % 2 == 1).all()
    assert not np.array_equal(draws, O.multinomial(P, 64, seed=7, offset=16))        # another stream position
    assert np.array_equal(draws, O.multinomial(P, 64, seed=7, offset=12))
    # chi-square of 6000 draws from a 12-way distribution (99.9 % quantile of chi2 with 11 dof: 31.3)
    w = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12], dtype=np.float32)
    d = O.multinomial(np.tile(w, (60, 1)), 100, seed=1, offset=0).reshape(-1)
    exp = w / w.sum() * d.size
    chi2 = ((np.bincount(d, minlength=12) - exp) ** 2 / exp).sum()
    assert chi2 < 31.3, chi2


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(3, 5, 4), (7, 127, 1), (5, 128, 8), (6, 4099, 5), (4, 128256, 3), (33, 1000, 2)])
def test_kernel_matches_its_documented_stream_bit_for_bit(cuda, m, n, k):
    from kuipy import _ffi
    g = torch.Generator().manual_seed(m * 1000 + n)
    P = torch.rand(m, n, generator=g)
    P[0, : n // 2] = 0
    if m > 2:
        P[2] = torch.softmax(torch.randn(n, generator=g) * 3, -1)               # what a sampler actually sees
    got = _ffi.multinomial(P.cuda(), k, seed=0x1234567890ABCDEF, offset=8)
    want = O.multinomial(P.numpy(), k, seed=0x1234567890ABCDEF, offset=8)
    assert np.array_equal(got.cpu().numpy(), want)
    assert _ffi.check_status(torch.device("cuda", 0)) == 0
    # rows that do not start on a 16-byte boundary (odd n): same draws from a misaligned view
    if n % 4 and m > 1:
        sub = P.cuda()[1:]
        assert np.array_equal(_ffi.multinomial(sub, k, seed=5, offset=0).cpu().numpy(), O.multinomial(P.numpy()[1:], k, seed=5, offset=0))


@pytest.mark.gpu
def test_draws_follow_the_probabilities_like_pytorch_own(cuda):
    from kuipy import _ffi
    torch.manual_seed(0)
    n, rows = 50, 40000
    w = torch.softmax(torch.randn(n) * 1.5, -1)
    P = w.repeat(rows, 1).cuda()
    ours = _ffi.multinomial(P, 1, seed=99, offset=0).reshape(-1)
    theirs = torch.multinomial(P, 1).reshape(-1)
    exp = (w * rows).double().numpy()
    crit = 85.4                                        # 99.9 % quantile of chi-square with 49 degrees of freedom
    for name, d in (("kuiops", ours), ("torch", theirs)):
        cnt = torch.bincount(d.cpu(), minlength=n).double().numpy()
        chi2 = ((cnt - exp) ** 2 / exp).sum()
        assert chi2 < crit, (name, chi2)
    # an invalid weight is reported through the status word and counts as zero
    bad = P[:2].clone()
    bad[0, 3] = -1.0
    bad[1, :] = 0
    out = _ffi.multinomial(bad, 1, seed=1, offset=0)
    assert _ffi.check_status(P.device) != 0 and int(out[0, 0]) != 3


@pytest.mark.gpu
def test_torch_multinomial_is_offloaded_and_follows_the_generator(cuda, gates):
    import kuipy
    from kuipy import _ffi
    gates("wide")
    P = torch.softmax(torch.randn(16, 5000, generator=torch.Generator().manual_seed(3)), -1).cuda()
    n0 = _ffi.launch_count()
    with kuipy.KuiperMode():
        torch.manual_seed(1234)
        a = torch.multinomial(P, 1)
        b = torch.multinomial(P, 1)                    # the generator's offset moved on: another draw
        torch.manual_seed(1234)
        a2 = torch.multinomial(P, 1)
        c = torch.multinomial(P, 6, replacement=True)
        d = torch.multinomial(P, 6, replacement=False)  # dependent draws: left to PyTorch
    assert _ffi.launch_count() - n0 >= 4
    assert a.shape == (16, 1) and a.dtype == torch.int64 and torch.equal(a, a2) and not torch.equal(a, b)
    assert c.shape == (16, 6) and d.shape == (16, 6)
    assert all(len(set(r.tolist())) == 6 for r in d.cpu())
    seed = torch.cuda.default_generators[0].initial_seed()
    assert seed == 1234
    assert np.array_equal(a.cpu().numpy(), O.multinomial(P.cpu().numpy(), 1, seed=1234, offset=0))


# ---- fused sampler: temperature, top-k, top-p, draw (kuiops_sample_topk_topp_f32) ---------------------------
def _filtered_distribution(row, temperature, top_k, top_p):
    """The distribution HuggingFace's temperature -> top-k -> top-p warpers leave (fp64), token id -> probability."""
    z = row.astype(np.float64) / temperature
    order = np.lexsort((np.arange(z.size), -z))[:top_k]
    p = np.exp(z[order] - z[order].max())
    p /= p.sum()
    before = np.concatenate(([0.0], np.cumsum(p)[:-1]))
    keep = before < top_p
    keep[0] = True
    q = np.where(keep, p, 0.0)
    return order, q / q.sum()


def test_sampler_oracle_keeps_the_nucleus_and_follows_the_distribution():
    rng = np.random.default_rng(3)
    logits = (rng.standard_normal((1, 900)) * 2).astype(np.float32)
    order, q = _filtered_distribution(logits[0], 0.7, 40, 0.8)
    allowed = set(order[q > 0].tolist())
    rows = np.tile(logits, (4000, 1))
    ids, prob, _ = O.sample_topk_topp(rows, 0.7, 40, 0.8, seed=11, offset=4)
    assert set(ids.tolist()) <= allowed
    counts = np.array([(ids == t).sum() for t in order[q > 0]])
    exp = q[q > 0] * ids.size
    big = exp >= 5
    chi2 = ((counts[big] - exp[big]) ** 2 / exp[big]).sum()
    assert chi2 < 2.5 * big.sum() + 20, (chi2, big.sum())
    # the reported probability is the filtered distribution's
    lookup = dict(zip(order.tolist(), q.tolist()))
    assert np.allclose(prob, [lookup[t] for t in ids.tolist()], rtol=1e-4)
    # top_k = 1 and a tiny nucleus are greedy
    g1, _, _ = O.sample_topk_topp(logits, 1.0, 1, 1.0, seed=1, offset=0)
    g2, _, _ = O.sample_topk_topp(logits, 1.0, 50, 1e-6, seed=1, offset=0)
    assert g1[0] == g2[0] == logits[0].argmax()


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,top_k,top_p,temp", [(5, 100, 50, 0.9, 0.7), (64, 128256, 50, 0.8, 0.7), (33, 4099, 1024, 0.95, 1.3),
                                                  (7, 300, 500, 1.0, 1.0), (4, 2000, 1, 0.5, 0.1), (9, 50000, 20, 1e-6, 2.0)])
def test_sampler_matches_the_oracle(cuda, m, n, top_k, top_p, temp):
    from kuipy import _ffi
    g = torch.Generator().manual_seed(m * 1000 + n)
    logits = torch.randn(m, n, generator=g) * 3
    ids, prob = _ffi.sample_topk_topp(logits.cuda(), temp, top_k, top_p, seed=0xABCDEF0123, offset=12, want_prob=True)
    want, wprob, margin = O.sample_topk_topp(logits.numpy(), temp, top_k, top_p, seed=0xABCDEF0123, offset=12)
    ids, prob = ids.cpu().numpy(), prob.cpu().numpy()
    sure = margin > 1e-5              # elsewhere one bit of an exp may move a threshold across a running sum
    assert (~sure).sum() <= max(1, m // 10)
    assert np.array_equal(ids[sure], want[sure])
    assert np.allclose(prob[sure], wprob[sure], rtol=1e-4, atol=1e-7)
    # every pick, sure or not, lies inside the set the filters keep
    for r in range(m):
        order, q = _filtered_distribution(logits.numpy()[r], temp, min(top_k, n), top_p)
        assert ids[r] in set(order[q > 1e-12].tolist()) or not sure[r]
    # another position of the stream gives other draws, the same position the same
    again = _ffi.sample_topk_topp(logits.cuda(), temp, top_k, top_p, seed=0xABCDEF0123, offset=12).cpu().numpy()
    assert np.array_equal(again, ids)


@pytest.mark.gpu
def test_sampler_distribution_and_edge_rows(cuda):
    from kuipy import _ffi
    rng = np.random.default_rng(5)
    row = (rng.standard_normal(5000) * 2.5).astype(np.float32)
    order, q = _filtered_distribution(row, 0.7, 50, 0.8)
    logits = torch.from_numpy(np.tile(row, (8192, 1))).cuda()
    ids = _ffi.sample_topk_topp(logits, 0.7, 50, 0.8, seed=21, offset=0).cpu().numpy()
    kept = order[q > 0]
    assert set(ids.tolist()) <= set(kept.tolist())
    counts = np.array([(ids == t).sum() for t in kept])
    exp = q[q > 0] * ids.size
    big = exp >= 5
    chi2 = ((counts[big] - exp[big]) ** 2 / exp[big]).sum()
    assert chi2 < 2.5 * big.sum() + 20, (chi2, big.sum())
    # rows with infinities and NaN: the largest entry (NaN above +inf) is the only candidate left
    bad = torch.randn(3, 1000)
    bad[0, 17] = float("inf")
    bad[1, 400] = float("nan")
    bad[2, :] = float("-inf")
    got = _ffi.sample_topk_topp(bad.cuda(), 1.0, 50, 0.9, seed=1, offset=0).cpu().numpy()
    assert got[0] == 17 and got[1] == 400 and got[2] == 0
    # contract
    with pytest.raises(_ffi.KuiopsError):
        _ffi.sample_topk_topp(bad.cuda(), 0.0, 50, 0.9)
    with pytest.raises(_ffi.KuiopsError):
        _ffi.sample_topk_topp(torch.randn(2, 3000).cuda(), 1.0, 2000, 0.9)      # more than 1024 candidates
