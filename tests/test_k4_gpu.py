"""GPU tests of the fused top-k sampling + log-prob kernel.  The random stream is the
library's own, so parity with the reference's sampler is checked in distribution; everything
deterministic (the top-k set and its order, the greedy path, the log-prob of whatever token
was drawn) is checked exactly against the oracle."""
import pytest
import torch

from helpers import TOL, max_abs
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["small_batches_split", "one_cta_per_row"])
def small_batch_path(request, monkeypatch):
    """Few long rows normally share each row among a cluster of CTAs; the second run of every
    test switches that off so the same cases also reach the one-CTA-per-row kernel."""
    if request.param == "one_cta_per_row":
        monkeypatch.setenv("TOME_K4_SPLIT", "0")
    else:
        monkeypatch.delenv("TOME_K4_SPLIT", raising=False)
    return request.param


def _case(rows, vocab, dtype, seed, scale=3.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn((rows, vocab), generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab", [1, 5, 20, 21, 600, 8192, 8193, 151936])
def test_topk_set_and_logprob(cuda_device, dtype, vocab):
    import tome_b200
    x = _case(6, vocab, dtype, 200 + vocab % 89)
    tok, lp, tk_i, tk_v = tome_b200.sample_topk_logprob(x.to(cuda_device), 0.7, 20, seed=3,
                                                        return_topk=True)
    k = min(20, vocab)
    for r in range(x.shape[0]):
        idx, probs = oracle.topk_sampling_distribution(x[r], 0.7, 20)
        assert tk_i[r, :k].cpu().tolist() == idx.tolist()          # exact set AND order
        assert torch.equal(tk_v[r, :k].cpu(), x[r].float()[idx])   # raw logits, bit-exact
        assert (tk_i[r, k:] == -1).all()
        assert int(tok[r]) in idx.tolist()
    o_lp, _, _ = oracle.selective_logprob(x, tok.cpu(), 0.7)
    assert max_abs(lp, o_lp) <= TOL[dtype]


def test_greedy_is_first_argmax_scored_at_temperature_one(cuda_device):
    import tome_b200
    x = _case(9, 5000, torch.bfloat16, 7)
    x[3, 100] = x[3].max()       # a tie for the maximum: the first index wins
    x[3, 4000] = x[3].max()
    tok, lp = tome_b200.sample_topk_logprob(x.to(cuda_device), 0.0)
    assert tok.cpu().tolist() == torch.argmax(x.float(), dim=-1).tolist()
    o_lp, _, _ = oracle.selective_logprob(x, tok.cpu(), 1.0)
    assert max_abs(lp, o_lp) <= 2e-3


def test_ties_masks_and_adversarial_orders(cuda_device):
    """bf16 ties across the k-th place, -inf masks, a constant row, ascending and descending
    rows (the ascending one makes every new logit a candidate)."""
    import tome_b200
    vocab = 30000
    x = _case(6, vocab, torch.bfloat16, 8, scale=0.25)   # coarse values: many exact ties
    x[1, : vocab - 7] = float("-inf")                     # fewer finite logits than k
    x[2, :] = 1.5                                         # constant row
    x[3] = torch.linspace(-8, 8, vocab).to(torch.bfloat16)            # ascending
    x[4] = torch.linspace(8, -8, vocab).to(torch.bfloat16)            # descending
    x[5, ::3] = float("-inf")
    tok, lp, tk_i, tk_v = tome_b200.sample_topk_logprob(x.to(cuda_device), 1.3, 20, seed=11,
                                                        return_topk=True)
    for r in range(6):
        idx, _ = oracle.topk_sampling_distribution(x[r], 1.3, 20)
        assert tk_i[r].cpu().tolist() == idx.tolist(), r
    assert int(tok[1]) >= vocab - 7                       # never a masked token
    o_lp, _, _ = oracle.selective_logprob(x, tok.cpu(), 1.3)
    assert max_abs(lp, o_lp) <= 2e-3


def test_draws_follow_the_topk_softmax(cuda_device):
    """20000 independent rows with the same logits: the empirical token frequencies must match
    softmax(top-k logits / T) (chi-square, 19 degrees of freedom, p = 1e-4 bound 50.0)."""
    import tome_b200
    g = torch.Generator().manual_seed(9)
    row = (torch.randn((1, 4000), generator=g) * 2.0)
    n = 20000
    x = row.expand(n, -1).contiguous().to(cuda_device)
    tok, _ = tome_b200.sample_topk_logprob(x, 0.8, 20, seed=1234, offset=5)
    idx, probs = oracle.topk_sampling_distribution(row[0], 0.8, 20)
    counts = torch.stack([(tok.cpu() == int(i)).sum() for i in idx]).double()
    assert int(counts.sum()) == n
    chi2 = float((((counts - n * probs) ** 2) / (n * probs)).sum())
    assert chi2 < 50.0, chi2
    # reproducible for the same (seed, offset); different for another offset
    tok2, _ = tome_b200.sample_topk_logprob(x, 0.8, 20, seed=1234, offset=5)
    tok3, _ = tome_b200.sample_topk_logprob(x, 0.8, 20, seed=1234, offset=6)
    assert torch.equal(tok, tok2) and not torch.equal(tok, tok3)


def test_rollout_step_shape_and_argument_errors(cuda_device):
    import tome_b200
    x = _case(64, 151936, torch.bfloat16, 10)             # B = 64 sequences, one decode step
    tok, lp = tome_b200.sample_topk_logprob(x.to(cuda_device).view(8, 8, -1), 0.7)
    assert tok.shape == (8, 8) and lp.shape == (8, 8) and tok.dtype == torch.int32
    o_lp, _, _ = oracle.selective_logprob(x, tok.cpu().reshape(-1), 0.7)
    assert max_abs(lp.reshape(-1), o_lp) <= 2e-3
    with pytest.raises(tome_b200.TomeArgumentError):
        tome_b200.sample_topk_logprob(x.to(cuda_device), 0.7, top_k=65)
    with pytest.raises(tome_b200.TomeArgumentError):
        tome_b200.sample_topk_logprob(x.to(cuda_device), -1.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unaligned_rows_and_extreme_k(cuda_device, dtype):
    """A vocabulary that is not a multiple of the vector width makes every other row start off
    a 16-byte boundary (scalar path); top_k = 1 and top_k = 64 are the ends of the range."""
    import tome_b200
    x = _case(7, 1003, dtype, 21)
    for k in (1, 64):
        tok, lp, tk_i, tk_v = tome_b200.sample_topk_logprob(x.to(cuda_device), 0.9, k, seed=5,
                                                            return_topk=True)
        for r in range(7):
            idx, _ = oracle.topk_sampling_distribution(x[r], 0.9, k)
            assert tk_i[r].cpu().tolist() == idx.tolist()
        o_lp, _, _ = oracle.selective_logprob(x, tok.cpu(), 0.9)
        assert max_abs(lp, o_lp) <= TOL[dtype]
    # a sliced view: odd base offset as well
    view = x.to(cuda_device)[:, 1:1000]
    tok, lp = tome_b200.sample_topk_logprob(view, 0.0)
    assert tok.cpu().tolist() == torch.argmax(x[:, 1:1000].float(), dim=-1).tolist()


@pytest.mark.parametrize("finish", ["kernel", "warp"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("vocab", [24, 600, 4096 + 8, 40000, 151936])
def test_large_batches_take_the_streaming_path(cuda_device, monkeypatch, dtype, vocab, finish):
    """Large bf16 batches go through the TMA-pipelined kernel (forced here for fp32 too); rows
    it cannot finish (sorted, constant or heavily tied ones overflow its small candidate ring)
    come back marked and are redone by the one-CTA-per-row kernel.  Both must give the
    oracle's top-k."""
    import tome_b200
    monkeypatch.setenv("TOME_K4_STREAM", "1")
    # the rows are finished by a kernel of their own or by the streaming kernel's producer warp
    monkeypatch.setenv("TOME_K4_FINISH", finish)
    rows = 1200 if vocab < 100000 else 700
    x = _case(rows, vocab, dtype, 300 + vocab % 71)
    x[5] = torch.linspace(-8, 8, vocab).to(dtype)          # ascending: overflows the ring
    x[6, :] = 0.5                                           # constant
    x[7, : vocab // 2] = float("-inf")
    tok, lp, tk_i, tk_v = tome_b200.sample_topk_logprob(x.to(cuda_device), 0.7, 20, seed=8, offset=2,
                                                        return_topk=True)
    assert int(tok.min()) >= 0                              # no row left marked
    k = min(20, vocab)
    for r in list(range(12)) + list(range(rows - 5, rows)) + [400, rows // 2 + 77]:
        idx, _ = oracle.topk_sampling_distribution(x[r], 0.7, 20)
        assert tk_i[r, :k].cpu().tolist() == idx.tolist(), r
        assert torch.equal(tk_v[r, :k].cpu(), x[r].float()[idx])
        assert int(tok[r]) in idx.tolist()
    o_lp, _, _ = oracle.selective_logprob(x, tok.cpu(), 0.7)
    assert max_abs(lp, o_lp) <= TOL[dtype]
    # greedy on the same batch
    tok0, lp0 = tome_b200.sample_topk_logprob(x.to(cuda_device), 0.0)
    assert tok0.cpu().tolist() == torch.argmax(x.float(), dim=-1).tolist()
    o_lp0, _, _ = oracle.selective_logprob(x, tok0.cpu(), 1.0)
    assert max_abs(lp0, o_lp0) <= TOL[dtype]


@pytest.mark.parametrize("parts", ["2", "4"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,vocab", [(100, 151936), (290, 40000 + 5), (700, 20000), (9, 4096 + 8)])
def test_rows_cut_into_parts_give_the_same_tokens(cuda_device, monkeypatch, dtype, rows, vocab, parts):
    """Batches smaller than the streaming kernel's grid have their rows cut into 2 or 4 work
    items, each with a threshold, a (max, sum-exp) pair and lists of its own, which the finish
    kernel puts together.  Same top-k lists and tokens as the one-CTA-per-row kernel, also when
    there are more items than CTAs (700 rows), when a row is too short to be cut (4104 logits
    in bf16: one copy per row) and when the rows end off the 16-byte grid."""
    import tome_b200
    wide = _case(rows, vocab + 3, dtype, 900 + rows)
    wide[1] = torch.linspace(-8, 8, vocab + 3).to(dtype)       # ascending: overflows the lists
    wide[2, :] = 0.5                                           # constant
    wide[3, : vocab // 2] = float("-inf")                      # a part without a finite logit
    wide[4, vocab // 3] = float("nan")
    wide[5] = float("-inf")
    wide[5, vocab - 1] = 2.0                                   # a single finite logit, in the last part
    wide[6, vocab - 2:] = 50.0                                 # the winners sit past the last 16-byte boundary
    pad = (-(vocab + 3)) % 8                                   # row pitch: a multiple of 16 bytes
    xd = torch.nn.functional.pad(wide, (0, pad)).to(cuda_device)[:, :vocab]
    x = wide[:, :vocab]
    monkeypatch.setenv("TOME_K4_STREAM", "0")
    t0, lp0, i0, v0 = tome_b200.sample_topk_logprob(xd, 0.7, 20, seed=3, offset=4, return_topk=True)
    monkeypatch.setenv("TOME_K4_STREAM", "1")
    monkeypatch.setenv("TOME_K4_PARTS", parts)
    for _ in range(2):  # twice: the scratch keeps the call before
        t1, lp1, i1, v1 = tome_b200.sample_topk_logprob(xd, 0.7, 20, seed=3, offset=4,
                                                        return_topk=True)
        assert torch.equal(t0, t1) and torch.equal(i0, i1)
        assert torch.equal(v0.nan_to_num(), v1.nan_to_num())
        ok = ~torch.isnan(lp0)
        assert torch.equal(ok, ~torch.isnan(lp1))
        assert max_abs(lp0[ok], lp1[ok]) <= (1e-5 if dtype == torch.float32 else 1e-4)
    for r in [0, 3, 6, 7, rows - 1]:
        idx, _ = oracle.topk_sampling_distribution(x[r], 0.7, 20)
        assert i1[r, : len(idx)].cpu().tolist() == idx.tolist(), r
    keep = [r for r in range(rows) if r != 4]
    o_lp, _, _ = oracle.selective_logprob(x[keep], t1.cpu()[keep], 0.7)
    assert max_abs(lp1.cpu()[keep], o_lp) <= TOL[dtype]
    # a wide top-k with rows in parts: more logits reach the finish (or the row kernel)
    t2, _, i2, _ = tome_b200.sample_topk_logprob(xd, 0.7, 64, seed=3, offset=4, return_topk=True)
    for r in [0, 7]:
        idx, _ = oracle.topk_sampling_distribution(x[r], 0.7, 64)
        assert i2[r, : len(idx)].cpu().tolist() == idx.tolist(), r


@pytest.mark.parametrize("form", ["kernel", "warp", "parts2"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,vocab", [(600, 50257), (150, 151937), (40, 4099)])
def test_streaming_path_with_rows_off_the_16_byte_grid(cuda_device, monkeypatch, dtype, rows, vocab, form):
    """Contiguous rows of an odd length: every row starts at another place of the 16-byte
    grid.  The streaming kernel copies a row from its first boundary to its last, notes vector
    numbers counted from there, and the elements outside count as one more short vector, which
    is where some rows here hold their winners.  Same tokens and top-k as the row kernel."""
    import tome_b200
    x = _case(rows, vocab, dtype, 500 + rows)
    x[1, 0] = 40.0                                  # before the first boundary (rows 1, 2, ...)
    x[2, vocab - 1] = 40.0                          # after the last one
    x[3, :7] = 45.0
    x[4] = torch.linspace(-8, 8, vocab).to(dtype)   # overflows the lists: row kernel
    x[5, vocab // 2] = float("nan")
    xd = x.to(cuda_device)
    monkeypatch.setenv("TOME_K4_STREAM", "0")
    t0, lp0, i0, v0 = tome_b200.sample_topk_logprob(xd, 0.7, 20, seed=6, offset=2, return_topk=True)
    monkeypatch.setenv("TOME_K4_STREAM", "1")
    if form == "parts2":
        monkeypatch.setenv("TOME_K4_PARTS", "2")
    else:
        monkeypatch.setenv("TOME_K4_PARTS", "1")
        monkeypatch.setenv("TOME_K4_FINISH", form)
    t1, lp1, i1, v1 = tome_b200.sample_topk_logprob(xd, 0.7, 20, seed=6, offset=2, return_topk=True)
    assert torch.equal(t0, t1) and torch.equal(i0, i1) and torch.equal(v0, v1)
    ok = ~torch.isnan(lp0)
    assert torch.equal(ok, ~torch.isnan(lp1)) and not bool(ok[5])
    assert max_abs(lp0[ok], lp1[ok]) <= (1e-5 if dtype == torch.float32 else 1e-4)
    for r in [0, 1, 2, 3, 6, rows - 1]:
        idx, _ = oracle.topk_sampling_distribution(x[r], 0.7, 20)
        assert i1[r, : len(idx)].cpu().tolist() == idx.tolist(), r
    keep = [r for r in range(rows) if r != 5]
    o_lp, _, _ = oracle.selective_logprob(x[keep], t1.cpu()[keep], 0.7)
    assert max_abs(lp1.cpu()[keep], o_lp) <= TOL[dtype]


def test_streaming_path_draws_follow_the_topk_softmax(cuda_device, monkeypatch):
    import tome_b200
    g = torch.Generator().manual_seed(10)
    row = (torch.randn((1, 4096), generator=g) * 2.0).to(torch.bfloat16)
    n = 20000
    x = row.expand(n, -1).contiguous().to(cuda_device)
    tok, _ = tome_b200.sample_topk_logprob(x, 0.8, 20, seed=99, offset=1)
    idx, probs = oracle.topk_sampling_distribution(row[0], 0.8, 20)
    counts = torch.stack([(tok.cpu() == int(i)).sum() for i in idx]).double()
    assert int(counts.sum()) == n
    chi2 = float((((counts - n * probs) ** 2) / (n * probs)).sum())
    assert chi2 < 50.0, chi2
    # the same draws as the one-CTA-per-row kernel makes for the same (seed, offset, row)
    tok_small, _ = tome_b200.sample_topk_logprob(x[:512], 0.8, 20, seed=99, offset=1)
    assert torch.equal(tok[:512], tok_small)
    monkeypatch.setenv("TOME_K4_STREAM", "0")
    tok_all, _ = tome_b200.sample_topk_logprob(x, 0.8, 20, seed=99, offset=1)
    assert torch.equal(tok, tok_all)


@pytest.mark.parametrize("split", ["2", "4", "8"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_split_rows_give_the_same_tokens_as_one_cta_per_row(cuda_device, monkeypatch, split, dtype):
    """The cluster path must return the identical top-k lists and tokens (the draw depends on
    the row's top-k only); the log-prob may differ by the summation order."""
    import tome_b200
    vocab = 151936 - 3                      # rows off the 16-byte grid from the second one on
    x = _case(5, vocab, dtype, 4242)
    x[1, : vocab - 11] = float("-inf")      # whole parts without a finite logit
    x[2] = torch.linspace(-8, 8, vocab).to(dtype)   # ascending: the top-k sits in the last part
    x[3, 16:] = x[3, 16:].clamp(max=0.5)    # heavy ties at the cap
    xd = x.to(cuda_device)
    monkeypatch.setenv("TOME_K4_SPLIT", "0")
    t0, lp0, i0, v0 = tome_b200.sample_topk_logprob(xd, 0.8, 20, seed=5, offset=9, return_topk=True)
    monkeypatch.setenv("TOME_K4_SPLIT", split)
    t1, lp1, i1, v1 = tome_b200.sample_topk_logprob(xd, 0.8, 20, seed=5, offset=9, return_topk=True,
                                                    check=True)
    assert torch.equal(i0, i1) and torch.equal(v0, v1) and torch.equal(t0, t1)
    assert max_abs(lp0, lp1) <= 1e-5
    for r in range(x.shape[0]):
        idx, _ = oracle.topk_sampling_distribution(x[r], 0.8, 20)
        assert i1[r, : len(idx)].cpu().tolist() == idx.tolist()
    o_lp, _, _ = oracle.selective_logprob(x, t1.cpu(), 0.8)
    assert max_abs(lp1, o_lp) <= TOL[dtype]


def test_workspace_entry_point_checks_its_scratch(cuda_device, monkeypatch):
    """The scratch-taking entry point: size query, too-small and misaligned scratch are refused
    before anything is launched, and without scratch the call still works (row kernel)."""
    import tome_b200
    from tome_b200 import _lib
    lib = _lib.lib
    rows, vocab = 400, 8192
    assert lib.tome_sample_workspace_bytes(rows, vocab) > rows * 256 * 8
    assert lib.tome_sample_workspace_bytes(8, vocab) == 0          # small batch: no scratch
    assert lib.tome_sample_workspace_bytes(rows, 1000) == 0        # short rows: row kernel
    x = _case(rows, vocab, torch.bfloat16, 77).to(cuda_device)
    tok = torch.empty(rows, dtype=torch.int32, device=cuda_device)
    lp = torch.empty(rows, dtype=torch.float32, device=cuda_device)
    ws = torch.empty(4096, dtype=torch.uint8, device=cuda_device)
    args = (x.data_ptr(), _lib.TOME_BF16, rows, vocab, vocab, 0.7, 20, 1, 2, tok.data_ptr(),
            lp.data_ptr(), None, None)
    assert lib.tome_sample_topk_logprob_ws(*args, ws.data_ptr(), 4096, None, None) == -6
    need = lib.tome_sample_workspace_bytes(rows, vocab)
    big = torch.empty(need + 16, dtype=torch.uint8, device=cuda_device)
    assert lib.tome_sample_topk_logprob_ws(*args, big.data_ptr() + 4, need, None, None) == -2
    assert lib.tome_sample_topk_logprob_ws(*args, None, 0, None, None) == 0
    t_row = tok.clone()
    assert lib.tome_sample_topk_logprob_ws(*args, big.data_ptr(), need, None, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(t_row, tok)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_three_kernel_path_when_every_row_overflows(cuda_device, monkeypatch, dtype):
    """Sorted, constant and fully masked rows overflow the per-row lists of the large-batch
    path; every such row must come back from the row kernel with the same answer."""
    import tome_b200
    rows, vocab = 400, 20000
    x = torch.empty((rows, vocab), dtype=dtype)
    x[0::4] = torch.linspace(-8, 8, vocab).to(dtype)       # ascending
    x[1::4] = 0.25                                          # constant
    x[2::4] = torch.linspace(8, -8, vocab).to(dtype)       # descending: top-k in the sample
    x[3::4] = float("-inf")
    x[3::4, 17] = 1.0                                       # a single finite logit
    xd = x.to(cuda_device)
    monkeypatch.setenv("TOME_K4_STREAM", "0")
    t0, lp0, i0, _ = tome_b200.sample_topk_logprob(xd, 0.9, 20, seed=4, offset=7, return_topk=True)
    monkeypatch.setenv("TOME_K4_STREAM", "1")
    t1, lp1, i1, _ = tome_b200.sample_topk_logprob(xd, 0.9, 20, seed=4, offset=7, return_topk=True,
                                                   check=True)
    assert int(t1.min()) >= 0
    assert torch.equal(t0, t1) and torch.equal(i0, i1)
    # rows that did not overflow were summed by the streaming pass (bf16: two of eight
    # exponentials by polynomial), the others by the row kernel
    assert max_abs(lp0, lp1) <= (1e-5 if dtype == torch.float32 else 1e-4)
    for r in range(4):
        idx, _ = oracle.topk_sampling_distribution(x[r], 0.9, 20)
        assert i1[r, : len(idx)].cpu().tolist() == idx.tolist()


@pytest.mark.parametrize("stream", ["0", "kernel", "warp"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rows_with_too_few_numbers(cuda_device, monkeypatch, stream, dtype):
    """A NaN is never a candidate.  A row with fewer than top_k logits that are not NaN draws
    from what it has and pads the top-k outputs; a row of NaNs gives token -1, log-prob NaN and
    a status bit, never an index left over from another row."""
    import tome_b200
    monkeypatch.setenv("TOME_K4_STREAM", "0" if stream == "0" else "1")
    if stream != "0":
        monkeypatch.setenv("TOME_K4_FINISH", stream)
    rows, vocab, k = 6, 32768, 20
    nan = float("nan")
    x = _case(rows, vocab, dtype, 77)
    x[1] = nan
    x[2] = nan
    x[2, 5], x[2, 20000], x[2, vocab - 1] = 1.0, 3.0, 2.0
    x[4, 100] = nan
    xd = x.to(cuda_device)
    for _ in range(2):  # twice: nothing may survive from the call before
        tok, lp, tk_i, tk_v = tome_b200.sample_topk_logprob(xd, 0.7, k, seed=1, return_topk=True)
        assert int(tok[1]) == -1 and bool(torch.isnan(lp[1])) and bool((tk_i[1] == -1).all())
        assert bool(torch.isinf(tk_v[1]).all())
        assert tk_i[2, :3].cpu().tolist() == [20000, vocab - 1, 5] and bool((tk_i[2, 3:] == -1).all())
        assert tk_v[2, :3].cpu().tolist() == [3.0, 2.0, 1.0] and bool(torch.isinf(tk_v[2, 3:]).all())
        assert int(tok[2]) in (5, 20000, vocab - 1) and bool(torch.isnan(lp[2]))
        x4 = x[4].clone()
        x4[100] = float("-inf")
        idx4, _ = oracle.topk_sampling_distribution(x4, 0.7, k)
        assert tk_i[4].cpu().tolist() == idx4.tolist() and int(tok[4]) in idx4.tolist()
        assert bool(torch.isnan(lp[4]))
        for r in (0, 3, 5):
            idx, _ = oracle.topk_sampling_distribution(x[r], 0.7, k)
            assert tk_i[r].cpu().tolist() == idx.tolist() and int(tok[r]) in idx.tolist()
        clean = torch.tensor([0, 3, 5])
        o_lp, _, _ = oracle.selective_logprob(x[clean], tok.cpu()[clean], 0.7)
        assert max_abs(lp.cpu()[clean], o_lp) <= TOL[dtype]
    with pytest.raises(tome_b200.TomeRuntimeError):
        tome_b200.check_device_status(cuda_device)
    tome_b200.check_device_status(cuda_device)  # the word was cleared


@pytest.mark.parametrize("rows", [64, 400])
def test_sampling_on_concurrent_streams(cuda_device, rows):
    """Four streams sample different batches at once, each with outputs and scratch of its own
    (the kernels of a call are chained by programmatic launches within their stream); every
    stream gets what it gets alone."""
    import tome_b200
    xs = [_case(rows, 32768 + 8 * i, torch.bfloat16, 900 + i).to(cuda_device) for i in range(4)]
    alone = [tome_b200.sample_topk_logprob(x, 0.7, 20, seed=5, offset=i) for i, x in enumerate(xs)]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(device=cuda_device) for _ in xs]
    outs = [(torch.empty(rows, dtype=torch.int32, device=cuda_device),
             torch.empty(rows, dtype=torch.float32, device=cuda_device)) for _ in xs]
    scratch = [torch.empty(max(16, tome_b200.sample_workspace_bytes(rows, x.shape[1])), dtype=torch.uint8,
                           device=cuda_device) for x in xs]
    for _ in range(5):
        for i, (x, st) in enumerate(zip(xs, streams)):
            with torch.cuda.stream(st):
                tome_b200.sample_topk_logprob(x, 0.7, 20, seed=5, offset=i, out=outs[i],
                                              workspace=scratch[i])
    torch.cuda.synchronize()
    for (tok, lp), (tok1, lp1) in zip(outs, alone):
        assert torch.equal(tok, tok1) and torch.equal(lp, lp1)
    tome_b200.check_device_status(cuda_device)
