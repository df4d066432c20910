"""CPU tests of the oracle: it restates the reference's formulas, so it is checked against
float64, against an independent implementation (torch.log_softmax), against algebraic
properties of log-softmax, and against the committed fixtures."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from helpers import from_bits, load_golden, max_abs
from oracle import oracle


def _case(rows, vocab, dtype, seed, scale=3.0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((rows, vocab), generator=g) * scale).to(dtype)
    ids = torch.randint(0, vocab, (rows,), generator=g)
    return x, ids


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("temp", [1.0, 0.7])
def test_selective_matches_float64(dtype, temp):
    x, ids = _case(16, 151936, dtype, 1)
    lp, lse, raw = oracle.selective_logprob(x, ids, temp)
    ref = oracle.selective_logprob_f64(x, ids, temp)
    assert max_abs(lp, ref) < 5e-6
    assert torch.equal(raw, x.float().gather(1, ids[:, None]).squeeze(1))


def test_selective_matches_torch_log_softmax():
    x, ids = _case(8, 5000, torch.float32, 2)
    lp, _, _ = oracle.selective_logprob(x, ids, 0.7)
    ref = torch.log_softmax(x.double() / 0.7, dim=-1).gather(1, ids[:, None]).squeeze(1)
    assert max_abs(lp, ref) < 5e-6


def test_full_reference_formula_matches_torch():
    x, _ = _case(4, 3000, torch.float32, 3)
    assert max_abs(oracle.log_softmax_reference(x, 1.3), torch.log_softmax(x.double() / 1.3, -1)) < 5e-6


def test_metal_order_bf16_within_reference_test_tolerance():
    # mlx-impl/tests/test_logprob_comparison.py:84-102: bf16 [1, 151936] ~ N(0,1), tol 5e-3
    # against logits - logsumexp(logits) evaluated in bf16.
    g = torch.Generator().manual_seed(4)
    x = torch.randn((1, 151936), generator=g).to(torch.bfloat16)
    out = oracle.log_softmax_metal_order(x, 1.0)
    assert out.dtype == torch.bfloat16
    lse_bf16 = oracle.logsumexp_f32(x.float()).to(torch.bfloat16)
    expected = (x.float() - lse_bf16.float()[:, None]).to(torch.bfloat16)
    assert max_abs(out, expected) < 5e-3


def test_metal_order_fp32_close_to_reference_formula():
    x, _ = _case(3, 4097, torch.float32, 5)
    assert max_abs(oracle.log_softmax_metal_order(x, 0.7), oracle.log_softmax_reference(x, 0.7)) < 2e-5


@settings(max_examples=25, deadline=None)
@given(seed=st.integers(0, 10_000), shift=st.floats(-50, 50), vocab=st.integers(1, 600))
def test_shift_invariance(seed, shift, vocab):
    x, ids = _case(3, vocab, torch.float32, seed)
    a, _, _ = oracle.selective_logprob(x, ids, 1.0)
    b, _, _ = oracle.selective_logprob(x + shift, ids, 1.0)
    assert max_abs(a, b) < 1e-4


@settings(max_examples=20, deadline=None)
@given(seed=st.integers(0, 10_000), temp=st.floats(0.2, 4.0))
def test_temperature_is_a_scale_of_the_logits(seed, temp):
    x, ids = _case(3, 257, torch.float32, seed)
    a, _, _ = oracle.selective_logprob(x, ids, temp)
    b, _, _ = oracle.selective_logprob(x / np.float32(temp), ids, 1.0)
    assert max_abs(a, b) < 1e-5


def test_full_rows_normalise_and_permute():
    x, ids = _case(4, 999, torch.float32, 7)
    full = oracle.log_softmax_reference(x, 0.9)
    assert max_abs(torch.logsumexp(full.double(), -1), torch.zeros(4)) < 1e-5
    perm = torch.randperm(999, generator=torch.Generator().manual_seed(1))
    inv = torch.argsort(perm)
    a, _, _ = oracle.selective_logprob(x, ids, 0.9)
    b, _, _ = oracle.selective_logprob(x[:, perm], inv[ids], 0.9)
    assert max_abs(a, b) < 1e-5


def test_edge_rows():
    x = torch.zeros((3, 10))
    x[1, :] = float("-inf")
    x[1, 3] = 2.0
    x[2, :] = 7.5
    ids = torch.tensor([0, 3, 9])
    lp, _, _ = oracle.selective_logprob(x, ids, 1.0)
    assert max_abs(lp, torch.tensor([-np.log(10.0), 0.0, -np.log(10.0)])) < 1e-6
    # vocab of one column: log-prob is exactly 0
    lp1, _, _ = oracle.selective_logprob(torch.tensor([[3.25]]), torch.tensor([0]), 0.5)
    assert float(lp1) == 0.0
    # no rows
    lp0, _, _ = oracle.selective_logprob(torch.zeros((0, 5)), torch.zeros((0,), dtype=torch.int64), 1.0)
    assert lp0.shape == (0,)


def test_sharded_triples_combine_to_unsharded():
    g = torch.Generator().manual_seed(8)
    hidden = torch.randn((20, 64), generator=g).to(torch.bfloat16)
    weight = (torch.randn((1000, 64), generator=g) * 0.05).to(torch.bfloat16)
    ids = torch.randint(0, 1000, (20,), generator=g)
    lp, lse = oracle.lm_head_logprob(hidden, weight, ids, 0.8)
    for world in (1, 2, 4, 7):
        per = (1000 + world - 1) // world
        ms, ss, ts = [], [], []
        for r in range(world):
            b, e = min(1000, r * per), min(1000, (r + 1) * per)
            m, s, t = oracle.shard_triple(hidden, weight[b:e], b, ids, 0.8)
            ms.append(m), ss.append(s), ts.append(t)
        lp2, lse2 = oracle.combine_triples(torch.stack(ms), torch.stack(ss), torch.stack(ts))
        assert max_abs(lp, lp2) < 1e-5 and max_abs(lse, lse2) < 1e-5


def test_dual_matches_per_sequence_selective_and_masks():
    g = torch.Generator().manual_seed(9)
    pol = (torch.randn((3, 5, 300), generator=g) * 3).to(torch.bfloat16)
    ref = (pol.float() + 0.1 * torch.randn((3, 5, 300), generator=g)).to(torch.bfloat16)
    ids = torch.randint(0, 300, (3, 5), generator=g)
    lengths = torch.tensor([0, 3, 5])
    p, r, kl = oracle.dual_logprob_kl(pol, ref, ids, lengths, 0.7)
    assert float(p[0].abs().max()) == 0.0 and float(kl[1, 3:].abs().max()) == 0.0
    a, _, _ = oracle.selective_logprob(pol[2], ids[2], 0.7)
    assert max_abs(p[2], a) == 0.0
    assert float(kl.min()) >= 0.0
    d = (r - p)[2]
    assert max_abs(kl[2], torch.exp(d) - d - 1) < 1e-7


@pytest.mark.parametrize("name,dtype", [("selective_bf16.npz", torch.bfloat16),
                                        ("selective_fp32.npz", torch.float32)])
def test_golden_selective(name, dtype):
    gld = load_golden(name)
    x = from_bits(gld["logits"], dtype)
    lp, lse, raw = oracle.selective_logprob(x, torch.from_numpy(gld["ids"]), float(gld["temp"]))
    assert max_abs(lp, torch.from_numpy(gld["logprob"])) < 1e-6
    assert max_abs(lse, torch.from_numpy(gld["lse"])) < 1e-6
    assert torch.equal(raw, torch.from_numpy(gld["raw"]))
    full = oracle.log_softmax_metal_order(x, float(gld["temp"]))
    assert max_abs(full.float(), from_bits(gld["full"], dtype).float()) < (1e-6 if dtype == torch.float32 else 0.07)


def test_golden_lm_head_and_dual():
    gld = load_golden("lm_head.npz")
    lp, lse = oracle.lm_head_logprob(from_bits(gld["hidden"], torch.bfloat16),
                                     from_bits(gld["weight"], torch.bfloat16),
                                     torch.from_numpy(gld["ids"]), float(gld["temp"]))
    assert max_abs(lp, torch.from_numpy(gld["logprob"])) < 1e-5
    gld = load_golden("dual_bf16.npz")
    p, r, kl = oracle.dual_logprob_kl(from_bits(gld["policy"], torch.bfloat16),
                                      from_bits(gld["ref"], torch.bfloat16),
                                      torch.from_numpy(gld["ids"]), torch.from_numpy(gld["lengths"]),
                                      float(gld["temp"]))
    assert max_abs(p, torch.from_numpy(gld["lp_policy"])) < 1e-6
    assert max_abs(kl, torch.from_numpy(gld["kl"])) < 1e-6
