"""The sampling kernels alone against the plain sampling oracle."""
import numpy as np
import pytest
import torch

from plain import llama_plain as P

pytestmark = pytest.mark.gpu


def _dev(a, dtype):
    return torch.tensor(a, dtype=dtype, device="cuda")


def test_argmax_lowest_index_wins_ties():
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(0)
    V = 128256 + 3
    logits = rng.standard_normal((5, V)).astype(np.float32)
    logits[0, [77, 5000, 120000]] = 9.0
    logits[1, V - 1] = 11.0
    logits[2, :] = -3.5                       # all equal: index 0
    logits[3, 0] = 50.0
    logits[4, [V - 2, V - 1]] = 12.0
    ids = torch.empty(5, dtype=torch.int32, device="cuda")
    vals = torch.empty(5, dtype=torch.float32, device="cuda")
    K.argmax(_dev(logits, torch.float32), ids, vals)
    assert ids.tolist() == [P.argmax_lowest(r) for r in logits] == [77, V - 1, 0, 0, V - 2]
    assert vals.tolist() == [9.0, 11.0, -3.5, 50.0, 12.0]


CDF_NOISE = 4e-6      # float32 summation noise of a cumulative distribution that ends at 1


def _lands_in(cum, ids, got, u):
    """The picked id is the one whose stretch of the cumulative distribution holds u, up to summation noise."""
    where = np.nonzero(ids == got)[0]
    assert where.size == 1, f"{got} is not a candidate"
    i = int(where[0])
    below = cum[i - 1] if i > 0 else 0.0
    last = i == len(cum) - 1
    assert below - CDF_NOISE <= u and (last or u < cum[i] + CDF_NOISE), (u, got, below, cum[i])


def _pick(logits, temp, top_k, top_p, us, one_block_per_row=False):
    from stratum_b200 import kernels as K
    n = len(us)
    L = _dev(np.repeat(logits[None], n, 0), torch.float32)
    ids = torch.empty(n, dtype=torch.int32, device="cuda")
    vals = torch.empty(n, dtype=torch.float32, device="cuda")
    K.sample(L, _dev([temp] * n, torch.float32), _dev([top_k] * n, torch.int32), _dev([top_p] * n, torch.float32),
             _dev(us, torch.float32), ids, vals, one_block_per_row=one_block_per_row)
    got = ids.tolist()
    assert vals.tolist() == [float(logits[g]) for g in got]
    return got


@pytest.mark.parametrize("one_block", [False, True])
@pytest.mark.parametrize("vocab", [320, 5000, 8192, 50001, 128256])
def test_temperature_draws_follow_the_inverse_cdf(vocab, one_block):
    """(From 8,192 logits on a row is cut over 32 blocks; one_block: the kernel with one block a row.)"""
    rng = np.random.default_rng(vocab)
    logits = (rng.standard_normal(vocab) * 2.0).astype(np.float32)
    us = np.concatenate([rng.random(2000), [0.0, 0.999999]]).astype(np.float32)
    got = _pick(logits, 0.8, 0, 1.0, us, one_block)
    ids, probs = P.filtered_distribution(logits, np.float32(0.8), 0, 1.0)
    cum = np.cumsum(probs)
    for u, g in zip(us, got):
        _lands_in(cum, ids, g, u)
    # and the draws have the distribution's shape: the most likely token comes up about as often as it should
    top = int(np.argmax(probs))
    assert abs(sum(g == top for g in got) / len(got) - probs[top]) < 4 * np.sqrt(probs[top] / len(got)) + 1e-3


@pytest.mark.parametrize("top_k, top_p", [(5, 1.0), (0, 0.7), (40, 0.9), (600, 0.95), (1, 1.0)])
def test_top_k_top_p_candidates(top_k, top_p):
    rng = np.random.default_rng(7)
    vocab = 50000
    logits = (rng.standard_normal(vocab) * 3.0).astype(np.float32)
    logits[[10, 20, 30]] = logits.max() + 0.5             # a tie at the very top: lower ids come first
    us = rng.random(600).astype(np.float32)
    got = _pick(logits, 1.3, top_k, top_p, us)
    # the row cut over 32 blocks and the row in one block keep the same candidates in the same order: the same picks
    assert got == _pick(logits, 1.3, top_k, top_p, us, one_block_per_row=True)
    k = top_k if 0 < top_k <= 512 else 512                # a filtered draw keeps at most 512 candidates
    ids, probs = P.filtered_distribution(logits, np.float32(1.3), k, top_p)
    cum = np.cumsum(probs)
    assert set(got) <= set(ids.tolist())
    for u, g in zip(us, got):
        _lands_in(cum, ids, g, u)
    if top_k == 1:
        assert set(got) == {10}


def test_greedy_rows_and_sampled_rows_in_one_launch():
    from stratum_b200 import kernels as K
    rng = np.random.default_rng(3)
    logits = rng.standard_normal((3, 1000)).astype(np.float32)
    ids = torch.empty(3, dtype=torch.int32, device="cuda")
    K.sample(_dev(logits, torch.float32), _dev([0.0, 1.0, -1.0], torch.float32), _dev([0, 0, 0], torch.int32),
             _dev([1.0, 1.0, 1.0], torch.float32), _dev([0.5, 0.5, 0.5], torch.float32), ids)
    got = ids.tolist()
    assert got[0] == int(logits[0].argmax()) and got[2] == int(logits[2].argmax())
    i, p = P.filtered_distribution(logits[1], 1.0, 0, 1.0)
    assert got[1] == P.sample_inverse_cdf(i, p, 0.5)


@pytest.mark.parametrize("vocab", [8192, 20011, 128256])
def test_rows_cut_over_blocks_ties_and_odd_rows(vocab):
    """Ties that straddle the cut inside a stretch and across stretches, a row of equal logits, logits of -inf,
    more candidates asked for than a stretch holds: the 32-block kernel against the plain oracle and the one-block
    kernel."""
    rng = np.random.default_rng(vocab + 1)
    us = rng.random(300).astype(np.float32)
    chunk = (vocab + 31) // 32
    cases = []
    a = (rng.standard_normal(vocab) * 2.0).astype(np.float32)
    top = float(a.max()) + 1.0
    a[[3, chunk - 1, chunk, 5 * chunk + 7, vocab - 1]] = top       # five equal at the top, in three stretches
    cases.append(("tie across stretches", a, 3))                    # only the three lowest ids survive
    b = np.full(vocab, -1.25, dtype=np.float32)
    cases.append(("all equal", b, 7))                               # ids 0..6
    cases.append(("all equal, more wanted than a stretch keeps", b, 100))   # the one-block kernel does this row
    c = (rng.standard_normal(vocab) * 2.0).astype(np.float32)
    c[rng.random(vocab) < 0.5] = -np.inf
    cases.append(("half of them -inf", c, 40))
    d = (rng.standard_normal(vocab) * 0.01).astype(np.float32)
    d[: chunk // 2] += 10.0                                         # the first stretch alone holds the best 512
    cases.append(("one stretch holds all candidates", d, 512))
    for name, logits, k in cases:
        for top_p in (1.0, 0.835):        # (no multiple of 1/7 or 1/100: the rows of equal logits meet no exact boundary)
            got = _pick(logits, 0.9, k, top_p, us)
            assert got == _pick(logits, 0.9, k, top_p, us, one_block_per_row=True), name
            ids, probs = P.filtered_distribution(logits, np.float32(0.9), k, top_p)
            cum = np.cumsum(probs)
            assert set(got) <= set(ids.tolist()), name
            for u, g in zip(us, got):
                _lands_in(cum, ids, g, u)
    assert set(_pick(cases[0][1], 0.9, 3, 1.0, us)) <= {3, chunk - 1, chunk}
    assert set(_pick(cases[1][1], 0.9, 7, 1.0, us)) == set(range(7))
    # without filters, and greedy rows, on the same odd rows
    for name, logits, _ in (cases[0], cases[1], cases[3]):
        got = _pick(logits, 0.9, 0, 1.0, us)
        ids, probs = P.filtered_distribution(logits, np.float32(0.9), 0, 1.0)
        cum = np.cumsum(probs)
        for u, g in zip(us, got):
            _lands_in(cum, ids, g, u)
        assert _pick(logits, 0.0, 0, 1.0, us[:3]) == [P.argmax_lowest(logits)] * 3
