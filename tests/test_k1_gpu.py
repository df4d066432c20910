"""GPU parity tests of the streaming log-softmax kernels (selective / full / dual) against
the CPU oracle, through the C ABI.  Tolerances: max-abs 1e-4 for fp32 logits, 2e-3 for bf16
logits; the gathered target logit must be bit-exact."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import (METAL_CASES, TOL, from_bits, load_golden, max_abs, metal_case_inputs,
                     metal_case_view)
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["small_batches_split", "one_cta_per_row", "two_pass_full"])
def small_batch_path(request, monkeypatch):
    """Few rows normally share each row among a cluster of CTAs; the second run of every test
    switches that off so the same cases also reach the streaming, cluster and plain-load
    kernels; the third also sends the full-matrix mode to the two-pass pipeline."""
    monkeypatch.delenv("TOME_K1_SPLIT", raising=False)
    monkeypatch.delenv("TOME_K1_FULL_CLUSTER", raising=False)
    if request.param != "small_batches_split":
        monkeypatch.setenv("TOME_K1_SPLIT", "0")
        monkeypatch.setenv("TOME_K1_FULL_CLUSTER", "0" if request.param == "two_pass_full" else "1")
    return request.param


def _case(rows, vocab, dtype, seed, scale=3.0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((rows, vocab), generator=g) * scale).to(dtype)
    ids = torch.randint(0, vocab, (rows,), generator=g, dtype=torch.int32)
    return x, ids


def _check_selective(x, ids, temp, dev, tol=None):
    import tome_b200
    lp, lse, raw = tome_b200.selective_log_softmax(x.to(dev), ids.to(dev), temp, return_lse=True,
                                                   return_target_logit=True, check=True)
    o_lp, o_lse, o_raw = oracle.selective_logprob(x, ids, temp)
    tol = TOL[x.dtype] if tol is None else tol
    assert lp.dtype == torch.float32 and lp.shape == ids.shape
    assert max_abs(lp, o_lp) <= tol, (max_abs(lp, o_lp), tol)
    assert max_abs(lse, o_lse) <= tol
    assert torch.equal(raw.cpu(), o_raw), "gathered target logit must be bit-exact"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab", [1, 7, 8, 9, 4095, 4096, 4097, 16392, 32768 + 16, 151936])
def test_selective_vocab_edges(cuda_device, dtype, vocab):
    x, ids = _case(5, vocab, dtype, 100 + vocab % 97)
    _check_selective(x, ids, 1.0, cuda_device)
    _check_selective(x, ids, 0.7, cuda_device)


@pytest.mark.parametrize("rows", [1, 2, 147, 148, 149, 300])
def test_selective_row_counts(cuda_device, rows):
    x, ids = _case(rows, 4096 + 8, torch.bfloat16, rows)
    _check_selective(x, ids, 0.7, cuda_device)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [75, 300, 591, 593, 1024, 2 * 592 - 1, 2 * 592 + 5])
def test_selective_row_counts_around_a_round_of_ctas(cuda_device, monkeypatch, dtype, rows):
    """The rows of a thin last round are shared by clusters of four CTAs (a quarter of the row
    each, merged over distributed shared memory).  Forced here for every row count, up to four
    shared rows per cluster; the same cases with the sharing switched off must agree."""
    import tome_b200
    vocab = 151936 if rows in (300, 1024) else 60000     # 24 / 12 chunks per row, or 10 / 5
    x, ids = _case(rows, vocab, dtype, seed=40 + rows)
    x[3, : vocab // 2] = float("-inf")       # a quarter without a finite logit
    x[5] = -1.0e30                           # the exact fallback, on a shared row when rows < CTAs
    x[rows - 1, vocab - 1] = 30.0            # the maximum in the last quarter of the last row
    monkeypatch.setenv("TOME_K1_TAIL", "2")  # share whatever the last round holds
    _check_selective(x, ids, 0.7, cuda_device)
    xd, idd = x.to(cuda_device), ids.to(cuda_device)
    shared = tome_b200.local_compute_logprobs(xd, idd, 0.7)
    monkeypatch.setenv("TOME_K1_TAIL", "0")
    plain = tome_b200.local_compute_logprobs(xd, idd, 0.7)
    assert max_abs(shared, plain) <= 2e-6 * 20     # summation order only
    tome_b200.check_device_status(cuda_device)


def test_selective_targets_at_the_ends(cuda_device):
    x, ids = _case(4, 151936, torch.bfloat16, 5)
    ids[:] = torch.tensor([0, 151935, 151936 - 384, 4096], dtype=torch.int32)
    _check_selective(x, ids, 1.0, cuda_device)


def test_selective_masked_columns_and_constant_rows(cuda_device):
    x, ids = _case(4, 10000, torch.float32, 6)
    x[0, :9000] = float("-inf")
    ids[0] = 9500
    x[1, :] = 3.0
    x[2, :] = -1e30
    x[2, 17] = 0.0
    ids[2] = 17
    _check_selective(x, ids, 1.0, cuda_device)
    lp = __import__("tome_b200").selective_log_softmax(x.to(cuda_device), ids.to(cuda_device), 1.0)
    assert abs(float(lp[2])) < 1e-6
    # a masked target scores -inf, as in the oracle
    ids[0] = 3
    lp = __import__("tome_b200").selective_log_softmax(x.to(cuda_device), ids.to(cuda_device), 1.0)
    assert float(lp[0]) == float("-inf")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selective_mask_values_and_extreme_magnitudes(cuda_device, dtype):
    """Finite mask fills (-1e30, finfo.min, -1e9) over long runs of a row, rows that lie
    entirely below the streaming floor, and huge positive logits: all must match the oracle."""
    x, ids = _case(8, 40000, dtype, 14)
    lowest = torch.finfo(dtype).min
    x[0, :30000] = -1e30
    x[1, 5000:] = lowest
    x[2, ::2] = -1e9
    x[3, :] = -2.0e6                      # whole row below the floor, constant
    x[4, :] = -3.0e6
    x[4, 777] = -2.9e6                    # below the floor with one clear winner
    x[5, :] = x[5, :] * 1e18              # huge magnitudes of both signs
    x[6, :] = 1e20
    x[7, :39000] = lowest
    x[7, 39000:] = -1e30
    ids[:] = torch.tensor([35000, 100, 1, 5, 777, 9, 11, 39500], dtype=torch.int32)
    _check_selective(x, ids, 1.0, cuda_device)
    _check_selective(x[:5], ids[:5], 0.7, cuda_device)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_nan_logit_gives_nan_wherever_it_sits(cuda_device, dtype):
    """mx.logsumexp (mlx-impl/node.py:401) and the Metal kernel's sum give NaN for a row that
    holds a NaN.  The bf16 fast path computes some exponentials of every 8-logit vector with a
    polynomial that clamps its argument, so the NaN's position within the vector matters: one
    row per position, plus clean rows that must stay finite."""
    import tome_b200
    vocab = 8192 + 24
    rows = 16
    x, ids = _case(rows, vocab, dtype, seed=5150)
    for r in range(8):
        x[r, 4096 + 8 * r + r] = float("nan")      # position r of its vector (rows are aligned)
    x[8, 3] = float("nan")
    x[9, vocab - 1] = float("nan")                 # in the tail past the last 16-byte boundary
    lp, lse = tome_b200.selective_log_softmax(x.to(cuda_device), ids.to(cuda_device), 0.7,
                                              return_lse=True)
    o_lp, o_lse, _ = oracle.selective_logprob(x, ids, 0.7)
    assert torch.isnan(o_lse[:10]).all() and torch.isfinite(o_lse[10:]).all()
    assert torch.isnan(lse[:10]).all() and torch.isnan(lp[:10]).all()
    assert max_abs(lp[10:], o_lp[10:]) <= TOL[dtype]
    full = tome_b200.fused_log_softmax(x.to(cuda_device), 0.7)
    assert torch.isnan(full[:10].float()).all()
    assert torch.isfinite(full[10:].float()).all()
    tome_b200.check_device_status(cuda_device)


@pytest.mark.parametrize("poly", ["1", "2"])
def test_selective_polynomial_exp_variants(cuda_device, poly):
    """The FMA-pipe exp2 variants (TOME_K1_POLY, read once per process) in a child process."""
    import os
    import subprocess
    import sys
    code = (
        "import sys, torch; sys.path.insert(0, %r); sys.path.insert(0, %r)\n"
        "import tome_b200; from oracle import oracle; from tome_b200 import synthetic\n"
        "x, ids = synthetic.cfg2_rollout_bf16(rows=300)\n"
        "lp = tome_b200.local_compute_logprobs(x.cuda(), ids.cuda(), 0.7)\n"
        "ref, _, _ = oracle.selective_logprob(x, ids, 0.7)\n"
        "err = float((lp.cpu() - ref).abs().max()); print(err); assert err <= 2e-3\n"
    ) % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
         os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, TOME_K1_POLY=poly)
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True,
                         timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr


@pytest.mark.parametrize("bulk", ["1", "0"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selective_rows_off_the_16_byte_grid(cuda_device, monkeypatch, dtype, bulk):
    """Odd base offsets and row pitches that are no multiple of 16 bytes: the bulk-copy pipeline
    copies every row from its first 16-byte boundary and reads the few elements before and
    after with ordinary loads (TOME_K1_BULK=0: the plain-load kernel).  Targets at both ends."""
    import tome_b200
    monkeypatch.setenv("TOME_K1_BULK", bulk)
    x, ids = _case(6, 1003, dtype, 8)
    xd = x.to(cuda_device)
    view = xd[:, 1:1000]
    ids = ids.clamp(max=998)
    ids[0], ids[1], ids[2], ids[3] = 0, 998, 5, 993
    lp = tome_b200.local_compute_logprobs(view, ids.to(cuda_device), 0.7)
    o_lp, _, _ = oracle.selective_logprob(x[:, 1:1000], ids, 0.7)
    assert max_abs(lp, o_lp) <= TOL[dtype]
    # long contiguous rows of an odd length (every row starts at another place of the grid),
    # more rows than CTAs, the largest logit of some rows outside the 16-byte boundaries
    for rows, vocab in ((700, 50257), (37, 151937), (300, 17), (300, 5)):
        x, ids = _case(rows, vocab, dtype, 80 + rows)
        x[1, 0] = 30.0
        x[2, vocab - 1] = 30.0
        x[3, : min(vocab - 1, 9)] = float("-inf")
        ids[1], ids[2] = 0, vocab - 1
        _check_selective(x, ids, 0.7, cuda_device)


def test_dual_and_ragged_rows_off_the_16_byte_grid(cuda_device):
    """The windowed modes on a vocabulary of odd size (policy and reference rows start at
    different places of the 16-byte grid when their bases differ)."""
    import tome_b200
    from tome_b200 import synthetic
    pol, ref, ids, lengths, temp = synthetic.cfg5_dual(5, 12, 8209, "cpu", 31, min_len=0)
    _check_dual(pol, ref, ids, lengths, temp, cuda_device)
    # the reference logits one element further along the grid than the policy's
    wide_p = torch.zeros((5, 12, 8210), dtype=pol.dtype)
    wide_r = torch.zeros((5, 12, 8210), dtype=ref.dtype)
    wide_p[..., :8209] = pol
    wide_r[..., 1:] = ref
    p, r, kl = tome_b200.grpo_dual_logprob_kl(wide_p.to(cuda_device)[..., :8209],
                                              wide_r.to(cuda_device)[..., 1:], ids.to(cuda_device),
                                              lengths.to(cuda_device), temp, check=True)
    o_p, o_r, o_kl = oracle.dual_logprob_kl(pol, ref, ids, lengths, temp, None)
    assert max_abs(p, o_p) <= 2e-3 and max_abs(r, o_r) <= 2e-3 and max_abs(kl, o_kl) <= 4e-3
    g = torch.Generator().manual_seed(61)
    n_seq, seq_len, vocab = 4, 10, 6001
    logits = (torch.randn((n_seq, seq_len, vocab), generator=g) * 3).to(torch.bfloat16)
    lengths = torch.tensor([10, 3, 0, 7], dtype=torch.int32)
    targets = [torch.randint(0, vocab, (int(l),), generator=g, dtype=torch.int32) for l in lengths]
    packed, offsets = tome_b200.ragged_logprobs(logits.to(cuda_device), torch.cat(targets).to(cuda_device),
                                                lengths.to(cuda_device), 0.7, check=True)
    want = oracle.ragged_logprobs(logits, targets, lengths, 0.7, None)
    off = offsets.cpu().tolist()
    for i in range(n_seq):
        assert max_abs(packed[off[i]:off[i + 1]], want[i]) <= 2e-3


def test_selective_strided_rows_and_leading_dims(cuda_device):
    import tome_b200
    x, ids = _case(12, 2048, torch.bfloat16, 9)
    xd = x.to(cuda_device)
    wide = torch.zeros((12, 4096), dtype=torch.bfloat16, device=cuda_device)
    wide[:, :2048] = xd
    lp = tome_b200.local_compute_logprobs(wide[:, :2048], ids.to(cuda_device), 1.0)
    o_lp, _, _ = oracle.selective_logprob(x, ids, 1.0)
    assert max_abs(lp, o_lp) <= 2e-3
    lp3 = tome_b200.local_compute_logprobs(xd.view(3, 4, 2048), ids.view(3, 4).to(cuda_device), 1.0)
    assert lp3.shape == (3, 4) and max_abs(lp3.reshape(-1), o_lp) <= 2e-3


def test_temperature_zero_means_one(cuda_device):
    import tome_b200
    x, ids = _case(3, 500, torch.float32, 10)
    a = tome_b200.local_compute_logprobs(x.to(cuda_device), ids.to(cuda_device), 0.0)
    b = tome_b200.local_compute_logprobs(x.to(cuda_device), ids.to(cuda_device), 1.0)
    assert torch.equal(a, b)


def test_empty_input(cuda_device):
    import tome_b200
    x = torch.zeros((0, 128), dtype=torch.bfloat16, device=cuda_device)
    ids = torch.zeros((0,), dtype=torch.int32, device=cuda_device)
    assert tome_b200.local_compute_logprobs(x, ids, 1.0).shape == (0,)
    assert tome_b200.fused_log_softmax(x, 1.0).shape == (0, 128)


def test_out_of_range_target_sets_status_and_nan(cuda_device):
    import tome_b200
    x, ids = _case(4, 100, torch.float32, 11)
    ids[2] = 100
    lp = tome_b200.local_compute_logprobs(x.to(cuda_device), ids.to(cuda_device), 1.0)
    assert torch.isnan(lp[2]) and not torch.isnan(lp[[0, 1, 3]]).any()
    with pytest.raises(tome_b200.TomeRuntimeError):
        tome_b200.check_device_status(cuda_device)
    tome_b200.check_device_status(cuda_device)  # cleared by the failed check


def test_bounded_wait_runs_out_and_reports(cuda_device):
    """A wait on a barrier nothing signals must give up after its limit, set TOME_DEV_TIMEOUT
    and leave the context usable (no trap, no hang)."""
    import time
    import tome_b200
    from tome_b200 import _lib
    tome_b200.check_device_status(cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    gave_up = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    t0 = time.perf_counter()
    st = _lib.lib.tome_selftest_bounded_wait(2_000_000, status.data_ptr(), gave_up.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert int(gave_up) == 1 and int(status) & _lib.DEV_TIMEOUT
    assert _lib.lib.tome_selftest_bounded_wait(0, None, None, None) == -4
    # the context still works
    x, ids = _case(3, 100, torch.float32, 1)
    _check_selective(x, ids, 1.0, cuda_device)


def test_outputs_stay_inside_their_buffers(cuda_device):
    from tome_b200 import _lib
    rows, vocab, pad = 37, 5000, 64
    x, ids = _case(rows, vocab, torch.bfloat16, 12)
    xd, idd = x.to(cuda_device), ids.to(cuda_device)
    bufs = [torch.full((rows + 2 * pad,), 1234.5, dtype=torch.float32, device=cuda_device) for _ in range(3)]
    ptrs = [b.data_ptr() + pad * 4 for b in bufs]
    st = _lib.lib.tome_selective_logprob(xd.data_ptr(), 1, rows, vocab, vocab, idd.data_ptr(), 1.0,
                                         ptrs[0], ptrs[1], ptrs[2], None,
                                         torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    for b in bufs:
        assert float((b[:pad] - 1234.5).abs().max()) == 0 and float((b[-pad:] - 1234.5).abs().max()) == 0
    o_lp, _, _ = oracle.selective_logprob(x, ids, 1.0)
    assert max_abs(bufs[0][pad:pad + rows], o_lp) <= 2e-3


def test_cfg1_shape_fp32(cuda_device):
    from tome_b200 import synthetic
    x, ids = synthetic.cfg1_selective_fp32(rows=256)
    _check_selective(x, ids, 1.0, cuda_device)
    _check_selective(x, ids, 0.7, cuda_device)


def test_cfg2_shape_bf16_planted(cuda_device):
    from tome_b200 import synthetic
    x, ids = synthetic.cfg2_rollout_bf16(rows=512)
    _check_selective(x, ids, 1.0, cuda_device)


def test_cfg2_full_size_properties(cuda_device):
    """20480 x 151936 bf16 (6.2 GB), generated on the device: every row's lse against an
    independent torch reduction on the GPU, a 256-row sample against the oracle, and
    invariance under a row permutation."""
    import tome_b200
    from tome_b200 import synthetic
    x, ids = synthetic.cfg2_rollout_bf16(device=cuda_device)
    lp, lse, raw = tome_b200.selective_log_softmax(x, ids, 1.0, return_lse=True,
                                                   return_target_logit=True, check=True)
    for b in range(0, x.shape[0], 2048):
        ref = torch.logsumexp(x[b:b + 2048].float(), dim=-1)
        assert max_abs(lse[b:b + 2048], ref) <= 2e-3
    assert torch.equal(raw, x.gather(1, ids.long()[:, None]).squeeze(1).float())
    sample = torch.arange(0, x.shape[0], 80, device=cuda_device)
    o_lp, _, _ = oracle.selective_logprob(x[sample].cpu(), ids[sample].cpu(), 1.0)
    assert max_abs(lp[sample], o_lp) <= 2e-3
    lp_rev = tome_b200.local_compute_logprobs(x[sample.flip(0)], ids[sample.flip(0)], 1.0)
    assert torch.equal(lp_rev.flip(0), tome_b200.local_compute_logprobs(x[sample], ids[sample], 1.0))


# ------------------------------------------------------------------ full matrix (compat)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 151936), (3, 4097), (5, 8), (2, 3), (149, 1024), (2, 4, 520)])
def test_full_log_softmax_matches_metal_order(cuda_device, dtype, shape):
    import tome_b200
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(shape, generator=g).to(dtype)
    for temp in (1.0, 0.7):
        out = tome_b200.fused_log_softmax(x.to(cuda_device), temp)
        assert out.dtype == dtype and out.shape == x.shape
        ref = oracle.log_softmax_metal_order(x, temp)
        if dtype == torch.float32:
            assert max_abs(out, ref) <= 1e-4
        else:
            # outputs are bf16 values near -12: one bf16 ulp there is 0.0625; lse rounding may
            # differ by one ulp between two fp32 summation orders
            assert max_abs(out.float(), ref.float()) <= 0.0625 + 1e-6
            assert float((out.cpu() == ref).float().mean()) >= 0.99


def test_full_log_softmax_into_a_given_buffer(cuda_device):
    import tome_b200
    x, _ = _case(5, 4097, torch.float32, 91, scale=1.0)
    xd = x.to(cuda_device)
    out = torch.full_like(xd, 7.0)
    got = tome_b200.fused_log_softmax(xd, 0.7, out=out)
    assert got.data_ptr() == out.data_ptr()
    assert max_abs(out, oracle.log_softmax_metal_order(x, 0.7)) <= 1e-4
    with pytest.raises(ValueError):
        tome_b200.fused_log_softmax(xd, 0.7, out=out[:, :100])


def test_full_log_softmax_reference_unit_test_shape(cuda_device):
    # mlx-impl/tests/test_logprob_comparison.py:84-102 with its 5e-3 tolerance
    import tome_b200
    g = torch.Generator().manual_seed(1)
    x = torch.randn((1, 151936), generator=g).to(torch.bfloat16)
    out = tome_b200.fused_log_softmax(x.to(cuda_device), temperature=1.0)
    lse = oracle.logsumexp_f32(x.float()).to(torch.bfloat16)
    expected = (x.float() - lse.float()[:, None]).to(torch.bfloat16)
    # the reference asserts 5e-3 on its own bf16 outputs; here: at most one bf16 ulp (0.0625 near
    # -12, from the rounding of the lse) and at least 99 % of the outputs bit-equal
    assert max_abs(out.float(), expected.float()) <= 0.0625 + 1e-6
    assert float((out.cpu() == expected).float().mean()) >= 0.99
    full32 = tome_b200.fused_log_softmax(x.float().to(cuda_device), 1.0)
    assert max_abs(torch.logsumexp(full32.double(), -1), torch.zeros(1)) < 1e-4


def test_fused_log_softmax_with_targets_is_selective(cuda_device):
    import tome_b200
    x, ids = _case(9, 3000, torch.float32, 13)
    full = tome_b200.fused_log_softmax(x.to(cuda_device), 0.7)
    sel = tome_b200.fused_log_softmax(x.to(cuda_device), 0.7, targets=ids.to(cuda_device))
    assert max_abs(full.gather(1, ids.long().to(cuda_device)[:, None]).squeeze(1), sel) <= 1e-4


# ------------------------------------------------------------------ dual scoring + KL
def _check_dual(pol, ref, ids, lengths, temp, dev, starts=None, tol=2e-3):
    import tome_b200
    p, r, kl = tome_b200.grpo_dual_logprob_kl(pol.to(dev), ref.to(dev), ids.to(dev), lengths.to(dev),
                                              temp, starts=None if starts is None else starts.to(dev),
                                              check=True)
    o_p, o_r, o_kl = oracle.dual_logprob_kl(pol, ref, ids, lengths, temp, starts)
    assert max_abs(p, o_p) <= tol and max_abs(r, o_r) <= tol
    assert max_abs(kl, o_kl) <= 2 * tol
    return p, r, kl


def test_dual_ragged(cuda_device):
    from tome_b200 import synthetic
    pol, ref, ids, lengths, temp = synthetic.cfg5_dual(6, 24, 8200, "cpu", 21, min_len=0)
    lengths[0], lengths[1] = 0, 24
    p, r, kl = _check_dual(pol, ref, ids, lengths, temp, cuda_device)
    assert float(p[0].abs().max()) == 0 and float(kl[0].abs().max()) == 0


def test_dual_windows_with_starts_and_poisoned_padding(cuda_device):
    from tome_b200 import synthetic
    pol, ref, ids, lengths, temp = synthetic.cfg5_dual(5, 16, 2048, "cpu", 22, min_len=0)
    starts = torch.tensor([0, 3, 15, 16, 7], dtype=torch.int32)
    lengths = torch.tensor([4, 13, 5, 2, 0], dtype=torch.int32)  # two get clamped
    pol_p, ref_p = pol.clone(), ref.clone()
    for i in range(5):
        st = int(starts[i]); ln = max(0, min(int(lengths[i]), 16 - st))
        mask = torch.ones(16, dtype=torch.bool); mask[st:st + ln] = False
        pol_p[i, mask] = float("nan"); ref_p[i, mask] = float("nan")
    p, r, kl = _check_dual(pol_p, ref_p, ids, lengths, temp, cuda_device, starts=starts)
    assert not torch.isnan(p).any() and not torch.isnan(kl).any()


def test_dual_and_ragged_beyond_the_sequence_limit_of_one_call(cuda_device):
    """More sequences than one library call takes (1024): the wrappers go in slices, the packed
    form writing each slice behind the one before."""
    import tome_b200
    g = torch.Generator().manual_seed(24)
    n_seq, seq_len, vocab = 2500, 3, 300
    pol = (torch.randn((n_seq, seq_len, vocab), generator=g) * 2).to(torch.bfloat16)
    ref = (pol.float() + torch.randn((n_seq, seq_len, vocab), generator=g) * 0.2).to(torch.bfloat16)
    ids = torch.randint(0, vocab, (n_seq, seq_len), generator=g, dtype=torch.int32)
    lengths = torch.randint(0, seq_len + 2, (n_seq,), generator=g, dtype=torch.int32)
    starts = torch.randint(0, seq_len + 1, (n_seq,), generator=g, dtype=torch.int32)
    dev = cuda_device
    p, r, kl = tome_b200.grpo_dual_logprob_kl(pol.to(dev), ref.to(dev), ids.to(dev), lengths.to(dev),
                                              0.7, starts=starts.to(dev), check=True)
    o_p, o_r, o_kl = oracle.dual_logprob_kl(pol, ref, ids, lengths, 0.7, starts)
    assert max_abs(p, o_p) <= 2e-3 and max_abs(r, o_r) <= 2e-3 and max_abs(kl, o_kl) <= 4e-3
    clamped = [max(0, min(int(l), seq_len - int(s))) for s, l in zip(starts, lengths)]
    targets = [torch.randint(0, vocab, (c,), generator=g, dtype=torch.int32) for c in clamped]
    packed, offsets, lse = tome_b200.ragged_logprobs(pol.to(dev), torch.cat(targets).to(dev),
                                                     lengths.to(dev), 0.7, starts=starts.to(dev),
                                                     return_lse=True, check=True)
    assert offsets.cpu().tolist() == [0] + torch.tensor(clamped).cumsum(0).tolist()
    want = oracle.ragged_logprobs(pol, targets, lengths, 0.7, starts)
    got = packed.cpu()
    off = offsets.cpu().tolist()
    for i in list(range(0, n_seq, 97)) + [1023, 1024, 1025, 2047, 2048, n_seq - 1]:
        if clamped[i]:
            assert max_abs(got[off[i]:off[i + 1]], want[i]) <= 2e-3, i
    assert not torch.isnan(lse).any()


def test_dual_at_the_sequence_limit(cuda_device):
    """1024 sequences per library call is the limit (the prefix sums live in shared memory)."""
    import tome_b200
    g = torch.Generator().manual_seed(23)
    n_seq, seq_len, vocab = 1024, 3, 520
    pol = (torch.randn((n_seq, seq_len, vocab), generator=g) * 2).to(torch.bfloat16)
    ref = (pol.float() + 0.1 * torch.randn((n_seq, seq_len, vocab), generator=g)).to(torch.bfloat16)
    ids = torch.randint(0, vocab, (n_seq, seq_len), generator=g, dtype=torch.int32)
    lengths = torch.randint(0, seq_len + 1, (n_seq,), generator=g, dtype=torch.int32)
    _check_dual(pol, ref, ids, lengths, 0.7, cuda_device)
    # one sequence more is refused by the library before any pointer is used (the Python
    # wrappers slice such batches, see the test above)
    from tome_b200 import _lib
    fake = 0x1000
    assert _lib.lib.tome_dual_logprob_kl(fake, fake, _lib.TOME_BF16, 1025, 1, 16, 16, fake, fake, None,
                                         1.0, fake, fake, fake, None, None) == -9


def test_dual_fp32_and_cfg5_shape(cuda_device):
    from tome_b200 import synthetic
    pol, ref, ids, lengths, temp = synthetic.cfg5_dual(2, 96, 151936, "cpu", 1005)
    _check_dual(pol, ref, ids, lengths, temp, cuda_device)
    _check_dual(pol[:, :8, :5000].float().contiguous(), ref[:, :8, :5000].float().contiguous(),
                ids[:, :8] % 5000, torch.tensor([8, 3], dtype=torch.int32), 1.0, cuda_device, tol=1e-4)


def test_cfg5_full_size_consistency(cuda_device):
    """cfg5 at full size (2 x 32 x 768 x 151936 bf16, ragged): the dual kernel must agree with
    two runs of the selective kernel on the active rows, the KL with its formula, masked
    positions must be zero, and a sample of rows must match the oracle."""
    import tome_b200
    from tome_b200 import synthetic
    pol, ref, tg, lengths, temp = synthetic.cfg5_dual(device=cuda_device)
    p, r, kl = tome_b200.grpo_dual_logprob_kl(pol, ref, tg, lengths, temp, check=True)
    pos = torch.arange(768, device=cuda_device)[None, :]
    active = pos < lengths[:, None]
    assert float(p[~active].abs().max()) == 0 and float(kl[~active].abs().max()) == 0
    sel_p = tome_b200.local_compute_logprobs(pol, tg, temp)
    sel_r = tome_b200.local_compute_logprobs(ref, tg, temp)
    assert max_abs(p[active], sel_p[active]) <= 1e-5 and max_abs(r[active], sel_r[active]) <= 1e-5
    d = (r - p)[active]
    assert max_abs(kl[active], torch.exp(d) - d - 1) <= 1e-6
    rows = torch.nonzero(active.reshape(-1)).squeeze(1)[::97][:128]
    flat_p = pol.view(-1, pol.shape[-1])
    o_lp, _, _ = oracle.selective_logprob(flat_p[rows].cpu(), tg.reshape(-1)[rows].cpu(), temp)
    assert max_abs(p.reshape(-1)[rows], o_lp) <= 2e-3


# ------------------------------------------------------------------ ragged, packed (wire layout)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_ragged_packed_matches_per_sequence_loop(cuda_device, dtype):
    import tome_b200
    g = torch.Generator().manual_seed(60)
    n_seq, seq_len, vocab = 7, 20, 6000
    logits = (torch.randn((n_seq, seq_len, vocab), generator=g) * 3).to(dtype)
    starts = torch.tensor([0, 4, 19, 20, 3, 0, 10], dtype=torch.int32)   # prompt_len - 1
    lengths = torch.tensor([20, 9, 5, 3, 0, 1, 10], dtype=torch.int32)   # two get clamped
    clamped = [max(0, min(int(l), seq_len - int(s))) for s, l in zip(starts, lengths)]
    targets = [torch.randint(0, vocab, (c,), generator=g, dtype=torch.int32) for c in clamped]
    # poison everything outside the windows: it must never be read
    poisoned = logits.clone()
    for i in range(n_seq):
        mask = torch.ones(seq_len, dtype=torch.bool)
        mask[int(starts[i]):int(starts[i]) + clamped[i]] = False
        poisoned[i, mask] = float("nan")
    packed, offsets, lse = tome_b200.ragged_logprobs(
        poisoned.to(cuda_device), torch.cat(targets).to(cuda_device), lengths.to(cuda_device), 0.7,
        starts=starts.to(cuda_device), return_lse=True, check=True)
    want = oracle.ragged_logprobs(logits, targets, lengths, 0.7, starts)
    assert offsets.cpu().tolist() == [0] + torch.tensor(clamped).cumsum(0).tolist()
    assert packed.shape == (sum(clamped),) and not torch.isnan(packed).any()
    off = offsets.cpu().tolist()
    for i in range(n_seq):
        assert max_abs(packed[off[i]:off[i + 1]], want[i]) <= TOL[dtype]


def test_ragged_wrong_target_count_is_reported(cuda_device):
    import tome_b200
    logits = torch.zeros((2, 4, 64), dtype=torch.float32, device=cuda_device)
    lengths = torch.tensor([4, 2], dtype=torch.int32, device=cuda_device)
    tg = torch.zeros(5, dtype=torch.int32, device=cuda_device)  # windows cover 6 positions
    with pytest.raises(ValueError):  # too many targets: caught on the host after the call
        tome_b200.ragged_logprobs(logits, torch.cat([tg, tg]), lengths, 1.0, check=True)
    with pytest.raises(tome_b200.TomeRuntimeError):  # too few: the kernel scores what fits
        tome_b200.ragged_logprobs(logits, tg, lengths, 1.0, check=True)
    packed, offsets = tome_b200.ragged_logprobs(logits, tg, lengths, 1.0)
    assert packed.shape == (5,) and offsets.cpu().tolist() == [0, 4, 6]
    with pytest.raises(tome_b200.TomeRuntimeError):
        tome_b200.check_device_status(cuda_device)


# ------------------------------------------------------------------ committed fixtures
@pytest.mark.parametrize("name,dtype", [("selective_bf16.npz", torch.bfloat16),
                                        ("selective_fp32.npz", torch.float32)])
def test_golden_selective_and_full(cuda_device, name, dtype):
    import tome_b200
    gld = load_golden(name)
    x = from_bits(gld["logits"], dtype).to(cuda_device)
    ids = torch.from_numpy(gld["ids"]).to(cuda_device)
    temp = float(gld["temp"])
    lp, lse, raw = tome_b200.selective_log_softmax(x, ids, temp, return_lse=True,
                                                   return_target_logit=True)
    assert max_abs(lp, torch.from_numpy(gld["logprob"])) <= TOL[dtype]
    assert max_abs(lse, torch.from_numpy(gld["lse"])) <= TOL[dtype]
    assert torch.equal(raw.cpu(), torch.from_numpy(gld["raw"]))
    full = tome_b200.fused_log_softmax(x, temp)
    want = from_bits(gld["full"], dtype)
    assert max_abs(full.float(), want.float()) <= (1e-4 if dtype == torch.float32 else 0.0625 + 1e-6)


def test_golden_dual(cuda_device):
    import tome_b200
    gld = load_golden("dual_bf16.npz")
    p, r, kl = tome_b200.grpo_dual_logprob_kl(
        from_bits(gld["policy"], torch.bfloat16).to(cuda_device),
        from_bits(gld["ref"], torch.bfloat16).to(cuda_device),
        torch.from_numpy(gld["ids"]).to(cuda_device), torch.from_numpy(gld["lengths"]).to(cuda_device),
        float(gld["temp"]))
    assert max_abs(p, torch.from_numpy(gld["lp_policy"])) <= 2e-3
    assert max_abs(r, torch.from_numpy(gld["lp_ref"])) <= 2e-3
    assert max_abs(kl, torch.from_numpy(gld["kl"])) <= 4e-3


@pytest.mark.parametrize("split", ["2", "4", "8"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selective_every_cluster_size(cuda_device, monkeypatch, split, dtype):
    """Each cluster size on rows whose vector count does not divide by it, aligned and not."""
    monkeypatch.setenv("TOME_K1_SPLIT", split)
    for rows, vocab in ((5, 151936), (3, 4099), (2, 9), (4, 1)):
        x, ids = _case(rows, vocab, dtype, seed=700 + vocab % 97)
        _check_selective(x, ids, 0.7, cuda_device)
    base, ids = _case(6, 1000 + 3, dtype, seed=77)
    view = base[:, 3:]  # rows start off the 16-byte grid
    ids = ids % view.shape[1]
    import tome_b200
    lp = tome_b200.selective_log_softmax(base.to(cuda_device)[:, 3:], ids.to(cuda_device), 1.3,
                                         check=True)
    o_lp, _, _ = oracle.selective_logprob(view.contiguous(), ids, 1.3)
    assert max_abs(lp, o_lp) <= TOL[dtype]


@pytest.mark.parametrize("split", ["2", "4", "8"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_full_every_cluster_size(cuda_device, monkeypatch, split, dtype):
    import tome_b200
    monkeypatch.setenv("TOME_K1_SPLIT", split)
    tol = 1e-4 if dtype == torch.float32 else 0.0625 + 1e-6
    for rows, vocab in ((5, 151936), (3, 4099), (2, 9), (4, 1)):
        x, _ = _case(rows, vocab, dtype, seed=900 + vocab % 89, scale=1.0)
        out = tome_b200.fused_log_softmax(x.to(cuda_device), 0.7)
        assert max_abs(out.float(), oracle.log_softmax_metal_order(x, 0.7).float()) <= tol
    # input rows off the 16-byte grid while the output rows are on it
    base, _ = _case(6, 1024 + 3, dtype, seed=78, scale=1.0)
    out = tome_b200.fused_log_softmax(base.to(cuda_device)[:, 3:], 1.0)
    ref = oracle.log_softmax_metal_order(base[:, 3:].contiguous(), 1.0)
    assert out.shape == ref.shape and max_abs(out.float(), ref.float()) <= tol


@pytest.mark.parametrize("small_batch_path", ["small_batches_split"], indirect=True)  # env set below
@pytest.mark.parametrize("form", ["1", "s1", "s2", "s4", "s8"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab", [8, 24, 25, 7000, 7001, 50257, 51200, 51200 + 8, 102400, 151936,
                                   151936 + 4, 151937, 300000])
def test_full_cluster_kernel_sizes(cuda_device, monkeypatch, small_batch_path, form, dtype, vocab):
    """The cluster kernel with every cluster size (1, 2, 4, 8 CTAs per row) on row lengths from
    less than one chunk per CTA (some CTAs of a cluster get nothing) to many chunks per CTA;
    more rows than clusters so that ring slots, pair slots and lse entries are reused.  Odd row
    lengths put every row at another place of the 16-byte grid (input and output rows alike):
    the copies then run from a row's first boundary to its last."""
    import tome_b200
    monkeypatch.setenv("TOME_K1_SPLIT", "0")
    monkeypatch.setenv("TOME_K1_FULL_CLUSTER", form)
    rows = 700 if vocab <= 7000 else (330 if vocab < 100000 else 160)
    x, _ = _case(rows, vocab, dtype, seed=31 + vocab % 83, scale=1.0)
    x[3, : vocab // 2] = float("-inf")          # a part of a row without a finite logit
    x[5] = -1.0e30                              # far below the streaming floor: exact fallback
    xd = x.to(cuda_device)
    out = tome_b200.fused_log_softmax(xd, 0.7)
    ref = oracle.log_softmax_metal_order(x, 0.7)
    tol = 1e-4 if dtype == torch.float32 else 0.0625 + 1e-6
    finite = torch.isfinite(ref.float())
    assert torch.equal(torch.isfinite(out.float()).cpu(), finite)
    assert max_abs(out.float().cpu()[finite], ref.float()[finite]) <= tol
    tome_b200.check_device_status(cuda_device)


@pytest.mark.parametrize("case_no", range(len(METAL_CASES)))
def test_against_outputs_of_the_reference_metal_kernel(cuda_device, case_no):
    """tests/golden/metal_kernel.npz: what the reference's own kernel body computes for these
    inputs (run on the CPU under an emulation of the Metal execution model)."""
    import tome_b200
    golden = load_golden("metal_kernel.npz")
    dtype_name, rows, vocab, temp = METAL_CASES[case_no]
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype_name]
    logits, targets = metal_case_inputs(dtype_name, rows, vocab, case_no)
    want = from_bits(golden[f"out_{case_no}"], dtype)
    got = metal_case_view(tome_b200.fused_log_softmax(logits.to(cuda_device), temp).cpu(), vocab)
    if dtype == torch.float32:
        assert max_abs(got, want) <= 1e-4
        # the policy call site gathers the kernel's output at the sampled token
        lp = tome_b200.fused_log_softmax(logits.to(cuda_device), temp,
                                         targets=targets.to(cuda_device), check=True)
        assert max_abs(lp, torch.from_numpy(golden[f"at_target_{case_no}"].copy())) <= 1e-4
    else:
        assert max_abs(got.float(), want.float()) <= 0.0625 + 1e-6      # one bf16 ulp near -12
        assert float((got == want).float().mean()) >= 0.99
