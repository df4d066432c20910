"""Seeded random shapes: row counts, vocabulary sizes (odd ones included), element offsets of the
first row and row pitches drawn at random, every mode against the oracle.  The fixed cases of
the other files pin the known edges; this one looks for the ones nobody thought of."""
import os
import random

import pytest
import torch

from helpers import TOL, max_abs
from oracle import oracle

pytestmark = pytest.mark.gpu

# TOME_TEST_SEED_OFFSET=n shifts every seed of this file: the same tests over other shapes
SEED_OFFSET = int(os.environ.get("TOME_TEST_SEED_OFFSET", "0")) * 100000


def _draw(rng, max_rows, max_vocab):
    rows = rng.choice([1, 2, 3, rng.randint(4, 64), rng.randint(65, max_rows)])
    vocab = rng.choice([rng.randint(1, 40), rng.randint(41, 5000), rng.randint(5001, max_vocab)])
    offset = rng.choice([0, 0, rng.randint(1, 9)])
    pitch = vocab + offset + rng.choice([0, 0, rng.randint(1, 17)])
    dtype = rng.choice([torch.float32, torch.bfloat16])
    temp = rng.choice([1.0, 0.7, 1.3])
    return rows, vocab, offset, pitch, dtype, temp


def _view(rows, vocab, offset, pitch, dtype, seed, dev):
    g = torch.Generator().manual_seed(seed)
    wide = (torch.randn((rows, pitch), generator=g) * 3.0).to(dtype)
    return wide[:, offset:offset + vocab], wide.to(dev)[:, offset:offset + vocab]


@pytest.mark.parametrize("seed", range(120))
def test_selective_random_shapes(cuda_device, seed):
    import tome_b200
    rng = random.Random(1000 + seed + SEED_OFFSET)
    rows, vocab, offset, pitch, dtype, temp = _draw(rng, 900, 70000)
    x, xd = _view(rows, vocab, offset, pitch, dtype, seed, cuda_device)
    ids = torch.randint(0, vocab, (rows,), generator=torch.Generator().manual_seed(seed), dtype=torch.int32)
    lp, lse, raw = tome_b200.selective_log_softmax(xd, ids.to(cuda_device), temp, return_lse=True,
                                                   return_target_logit=True, check=True)
    o_lp, o_lse, o_raw = oracle.selective_logprob(x, ids, temp)
    assert max_abs(lp, o_lp) <= TOL[dtype], (rows, vocab, offset, pitch, dtype)
    assert max_abs(lse, o_lse) <= TOL[dtype]
    assert torch.equal(raw.cpu(), o_raw)


@pytest.mark.parametrize("seed", range(80))
def test_full_matrix_random_shapes(cuda_device, seed):
    import tome_b200
    rng = random.Random(2000 + seed + SEED_OFFSET)
    rows, vocab, offset, pitch, dtype, temp = _draw(rng, 500, 60000)
    x, xd = _view(rows, vocab, offset, pitch, dtype, seed, cuda_device)
    out = tome_b200.fused_log_softmax(xd, temp)
    ref = oracle.log_softmax_metal_order(x.contiguous(), temp)
    tol = 1e-4 if dtype == torch.float32 else 0.0625 + 1e-6   # one bf16 ulp near -12
    assert out.shape == ref.shape and out.dtype == dtype
    assert max_abs(out.float(), ref.float()) <= tol, (rows, vocab, offset, pitch, dtype)
    # a contiguous input of the same values: output and input rows now sit alike on the 16-byte
    # grid, which sends rows of an odd length through the bulk-copy kernels
    out2 = tome_b200.fused_log_softmax(xd.contiguous(), temp)
    assert torch.equal(out2, out) or max_abs(out2.float(), ref.float()) <= tol


@pytest.mark.parametrize("seed", range(100))
def test_sampling_random_shapes(cuda_device, monkeypatch, seed):
    import tome_b200
    rng = random.Random(3000 + seed + SEED_OFFSET)
    rows, vocab, offset, pitch, dtype, temp = _draw(rng, 700, 60000)
    k = rng.choice([1, 5, 20, 33, 64])
    form = rng.choice(["default", "rows", "stream", "stream_warp", "stream_parts"])
    if form == "rows":
        monkeypatch.setenv("TOME_K4_STREAM", "0")
    elif form != "default":
        monkeypatch.setenv("TOME_K4_STREAM", "1")
        if form == "stream_warp":
            monkeypatch.setenv("TOME_K4_FINISH", "warp")
        if form == "stream_parts":
            monkeypatch.setenv("TOME_K4_PARTS", rng.choice(["2", "4"]))
    x, xd = _view(rows, vocab, offset, pitch, dtype, seed, cuda_device)
    tok, lp, tk_i, tk_v = tome_b200.sample_topk_logprob(xd, temp, k, seed=seed, offset=3,
                                                        return_topk=True, check=True)
    kk = min(k, vocab)
    for r in sorted({0, rows // 2, rows - 1}):
        idx, _ = oracle.topk_sampling_distribution(x[r], temp, k)
        assert tk_i[r, :kk].cpu().tolist() == idx.tolist(), (r, rows, vocab, offset, pitch, dtype, form)
        assert int(tok[r]) in idx.tolist()
    o_lp, _, _ = oracle.selective_logprob(x, tok.cpu(), temp)
    assert max_abs(lp, o_lp) <= TOL[dtype], (rows, vocab, offset, pitch, dtype, form)


@pytest.mark.parametrize("seed", range(40))
def test_dual_and_ragged_random_shapes(cuda_device, seed):
    """Policy / reference scoring with the k3 KL estimate over ragged windows, and the packed
    single-model form, on random sequence counts, lengths, windows and vocabulary sizes."""
    import tome_b200
    rng = random.Random(4000 + seed + SEED_OFFSET)
    n_seq = rng.choice([1, 2, rng.randint(3, 12)])
    seq_len = rng.choice([1, 2, rng.randint(3, 24)])
    vocab = rng.choice([rng.randint(1, 40), rng.randint(41, 5000), rng.randint(5001, 30000)])
    dtype = rng.choice([torch.float32, torch.bfloat16])
    temp = rng.choice([1.0, 0.7])
    g = torch.Generator().manual_seed(seed)
    pol = (torch.randn((n_seq, seq_len, vocab), generator=g) * 3.0).to(dtype)
    ref = (pol.float() + torch.randn((n_seq, seq_len, vocab), generator=g) * 0.3).to(dtype)
    ids = torch.randint(0, vocab, (n_seq, seq_len), generator=g, dtype=torch.int32)
    starts = torch.tensor([rng.randint(0, seq_len) for _ in range(n_seq)], dtype=torch.int32)
    lengths = torch.tensor([rng.randint(0, seq_len + 2) for _ in range(n_seq)], dtype=torch.int32)
    dev = cuda_device
    p, r, kl = tome_b200.grpo_dual_logprob_kl(pol.to(dev), ref.to(dev), ids.to(dev), lengths.to(dev),
                                              temp, starts=starts.to(dev), check=True)
    o_p, o_r, o_kl = oracle.dual_logprob_kl(pol, ref, ids, lengths, temp, starts)
    tol = TOL[dtype]
    assert max_abs(p, o_p) <= tol and max_abs(r, o_r) <= tol and max_abs(kl, o_kl) <= 2 * tol
    clamped = [max(0, min(int(l), seq_len - int(s))) for s, l in zip(starts, lengths)]
    targets = [torch.randint(0, vocab, (c,), generator=g, dtype=torch.int32) for c in clamped]
    packed, offsets = tome_b200.ragged_logprobs(pol.to(dev), torch.cat(targets).to(dev), lengths.to(dev),
                                                temp, starts=starts.to(dev), check=True)
    want = oracle.ragged_logprobs(pol, targets, lengths, temp, starts)
    off = offsets.cpu().tolist()
    assert off == [0] + torch.tensor(clamped).cumsum(0).tolist()
    for i in range(n_seq):
        if clamped[i]:
            assert max_abs(packed[off[i]:off[i + 1]], want[i]) <= tol


@pytest.mark.parametrize("seed", range(60))
def test_fused_lm_head_random_shapes(cuda_device, seed):
    """The fused LM head + log-prob on random row counts, hidden sizes (multiples of 8) and
    vocabulary sizes, alone and with the final RMSNorm and the bf16-rounded logits, sharded or
    not, against the oracle (2e-3, the fused head's tolerance)."""
    import tome_b200
    from tome_b200 import synthetic
    rng = random.Random(5000 + seed + SEED_OFFSET)
    rows = rng.choice([1, rng.randint(2, 127), 128, rng.randint(129, 700)])
    k = 8 * rng.choice([1, rng.randint(2, 16), rng.randint(17, 96)])
    vocab = rng.choice([rng.randint(1, 255), 256, rng.randint(257, 6000)])
    temp = rng.choice([1.0, 0.7, 1.5])
    hidden, weight, ids = synthetic.cfg3_lm_head(rows, k, vocab, "cpu", 6000 + seed, 0.05)
    dev = cuda_device
    form = rng.choice(["plain", "norm", "rounded", "sharded"])
    if form == "plain":
        lp, lse = tome_b200.lm_head_logprob(hidden.to(dev), weight.to(dev), ids.to(dev), temp, check=True)
        o_lp, o_lse = oracle.lm_head_logprob(hidden, weight, ids, temp)
    elif form == "norm":
        g = torch.Generator().manual_seed(seed)
        nw = (1.0 + 0.1 * torch.randn(k, generator=g)).to(torch.bfloat16)
        lp, lse = tome_b200.lm_head_logprob(hidden.to(dev), weight.to(dev), ids.to(dev), temp,
                                            norm_weight=nw.to(dev), eps=1e-6, check=True)
        o_lp, o_lse = oracle.lm_head_logprob(oracle.rms_norm(hidden, nw, 1e-6), weight, ids, temp)
    elif form == "rounded":
        lp, lse = tome_b200.lm_head_logprob(hidden.to(dev), weight.to(dev), ids.to(dev), temp,
                                            round_logits=True, check=True)
        o_lp, o_lse = oracle.lm_head_logprob(hidden, weight, ids, temp, round_to_bf16=True)
    else:  # vocabulary shards of one process, combined as the ranks of a vocab-parallel head do
        world = rng.choice([2, 3, 5])
        hd, wd, idd = hidden.to(dev), weight.to(dev), ids.to(dev)
        ms, ss, ts = [], [], []
        for r in range(world):
            b, e = synthetic.shard_bounds(vocab, r, world)
            if e <= b:
                continue
            m, s_, t = tome_b200.lm_head_partials(hd, wd[b:e].contiguous(), b, idd, temp)
            ms.append(m), ss.append(s_), ts.append(t)
        lp, lse = tome_b200.combine_triples(torch.stack(ms), torch.stack(ss), torch.stack(ts))
        o_lp, o_lse = oracle.lm_head_logprob(hidden, weight, ids, temp)
    # rounded logits: one that sits on a bf16 rounding boundary may round the other way on the
    # GPU (different fp32 summation order), one bf16 ulp of the target logit; the norm may differ
    # from the oracle's by an ulp of the hidden state
    tol = {"plain": 2e-3, "sharded": 2e-3, "norm": 5e-3, "rounded": 2e-3 + 2 ** -6}[form]
    assert max_abs(lse, o_lse) <= tol, (form, rows, k, vocab, max_abs(lse, o_lse))
    assert max_abs(lp, o_lp) <= tol, (form, rows, k, vocab, max_abs(lp, o_lp))


@pytest.mark.parametrize("seed", range(40))
def test_paged_kv_random_shapes(cuda_device, seed):
    """Paged KV gather and update (mlx-impl/paged_kv.py) on random pool sizes, head counts,
    block sizes, head dimensions, tables, offsets and lengths; byte-exact against the oracle's
    loops."""
    import tome_b200
    rng = random.Random(7000 + seed + SEED_OFFSET)
    dtype = rng.choice([torch.bfloat16, torch.float32])
    H = rng.randint(1, 4)
    bs = rng.choice([1, 4, 16, 32])
    D = rng.choice([8, 64, 128]) if dtype == torch.bfloat16 else rng.choice([4, 64, 128])
    B = rng.randint(1, 6)
    per_seq = rng.randint(1, 6)
    num_blocks = B * per_seq + rng.randint(0, 5)
    g = torch.Generator().manual_seed(seed)
    k_pool = torch.randn((num_blocks, H, bs, D), generator=g).to(dtype)
    v_pool = torch.randn((num_blocks, H, bs, D), generator=g).to(dtype)
    tables = torch.randperm(num_blocks, generator=g)[: B * per_seq].reshape(B, per_seq).to(torch.int32)
    cap = per_seq * bs
    dev = cuda_device
    # gather
    offsets = torch.tensor([rng.randint(0, cap) for _ in range(B)], dtype=torch.int32)
    max_len = rng.randint(1, cap + 3)
    k_out, v_out = tome_b200.gather_paged_kv(tables.to(dev), offsets.to(dev), k_pool.to(dev),
                                             v_pool.to(dev), max_len)
    o_k, o_v = oracle.gather_paged_kv(tables, offsets, k_pool, v_pool, max_len)
    assert torch.equal(k_out.cpu(), o_k) and torch.equal(v_out.cpu(), o_v), (H, bs, D, B, per_seq, max_len)
    # update (disjoint blocks per sequence, writes may run off the table's end)
    s_new = rng.randint(1, cap + 2)
    k_new = torch.randn((B, H, s_new, D), generator=g).to(dtype)
    v_new = torch.randn((B, H, s_new, D), generator=g).to(dtype)
    start = torch.tensor([rng.randint(0, cap) for _ in range(B)], dtype=torch.int32)
    lengths = torch.tensor([rng.randint(0, s_new) for _ in range(B)], dtype=torch.int32)
    kp, vp = k_pool.to(dev), v_pool.to(dev)
    tome_b200.update_paged_kv(k_new.to(dev), v_new.to(dev), tables.to(dev), start.to(dev), kp, vp,
                              lengths=lengths.to(dev))
    o_k, o_v = oracle.update_paged_kv(k_new, v_new, tables, start, k_pool, v_pool, bs, lengths)
    assert torch.equal(kp.cpu(), o_k) and torch.equal(vp.cpu(), o_v), (H, bs, D, B, per_seq, s_new)
