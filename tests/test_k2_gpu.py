"""GPU parity tests of the fused LM-head + log-prob kernel (tcgen05 / TMEM) against the CPU
oracle, through the C ABI.  Tolerance: max-abs 2e-3 on log-probs (bf16 operands, fp32
accumulation; the oracle multiplies the same bf16 values in fp32)."""
import pytest
import torch

from helpers import from_bits, load_golden, max_abs
from oracle import oracle

pytestmark = pytest.mark.gpu

TOL = 2e-3


def _run(rows, k, vocab, temp, dev, seed=0, w_scale=0.05):
    import tome_b200
    from tome_b200 import synthetic
    hidden, weight, ids = synthetic.cfg3_lm_head(rows, k, vocab, "cpu", 3000 + seed, w_scale)
    lp, lse = tome_b200.lm_head_logprob(hidden.to(dev), weight.to(dev), ids.to(dev), temp, check=True)
    o_lp, o_lse = oracle.lm_head_logprob(hidden, weight, ids, temp)
    assert lp.shape == (rows,) and lp.dtype == torch.float32
    assert max_abs(lse, o_lse) <= TOL, ("lse", max_abs(lse, o_lse))
    assert max_abs(lp, o_lp) <= TOL, ("logprob", max_abs(lp, o_lp))


def test_one_tile(cuda_device):
    _run(128, 64, 256, 1.0, cuda_device)


@pytest.mark.parametrize("rows", [1, 40, 127, 129, 300])
def test_row_tails(cuda_device, rows):
    _run(rows, 128, 512, 1.0, cuda_device, seed=rows)


@pytest.mark.parametrize("vocab", [8, 255, 257, 700, 4096 + 48, 18992])
def test_vocab_tails(cuda_device, vocab):
    _run(130, 192, vocab, 0.7, cuda_device, seed=vocab)


@pytest.mark.parametrize("k", [8, 72, 200, 1024, 4096])
def test_hidden_sizes(cuda_device, k):
    _run(140, k, 1000, 1.0, cuda_device, seed=k, w_scale=0.02)


def test_many_bands_and_row_tile_groups(cuda_device):
    # K = 4096 makes bands short (8 column tiles) and row-tile groups small
    _run(128 * 41, 4096, 256 * 20, 0.9, cuda_device, seed=5, w_scale=0.015)


def test_cfg3_shape_row_slice(cuda_device):
    # Qwen3-0.6B head shape with a 512-row slice of the 16384 rows
    _run(512, 1024, 151936, 1.0, cuda_device, seed=7, w_scale=0.02)


@pytest.mark.parametrize("rows,k,seed,scale", [(16384, 1024, 1003, 0.02), (32768, 4096, 1004, 0.015)])
def test_full_size_heads_against_an_independent_gpu_reduction(cuda_device, rows, k, seed, scale):
    """cfg3 / cfg4 at full size: every row's logsumexp and target log-prob against
    torch.matmul (fp32 accumulate, bf16 logits up-cast) + torch.logsumexp in row chunks, and a
    64-row sample against the CPU oracle."""
    import tome_b200
    from tome_b200 import synthetic
    hidden, weight, ids = synthetic.cfg3_lm_head(rows, k, 151936, cuda_device, seed, scale)
    lp, lse = tome_b200.lm_head_logprob(hidden, weight, ids, 1.0, check=True)
    worst = 0.0
    for b in range(0, rows, 2048):
        logits = torch.matmul(hidden[b:b + 2048], weight.t()).float()   # bf16-rounded logits
        ref_lse = torch.logsumexp(logits, dim=-1)
        ref_lp = logits.gather(1, ids[b:b + 2048].long()[:, None]).squeeze(1) - ref_lse
        # the reference path rounds logits to bf16 (ulp 2^-6 at |x| < 8): lse moves by far less
        # (errors average out), the gathered target logit by up to half an ulp
        assert max_abs(lse[b:b + 2048], ref_lse) <= 5e-3
        worst = max(worst, max_abs(lp[b:b + 2048], ref_lp))
        del logits
    assert worst <= 5e-3 + 2 ** -7, worst
    sample = torch.arange(0, rows, rows // 64, device=cuda_device)
    o_lp, o_lse = oracle.lm_head_logprob(hidden[sample].cpu(), weight.cpu(), ids[sample].cpu(), 1.0)
    assert max_abs(lp[sample], o_lp) <= TOL and max_abs(lse[sample], o_lse) <= TOL


def test_peaked_and_large_magnitude_logits(cuda_device):
    """Weights scaled so that logits reach |x| ~ 100 (300 after the temperature) with a sharply peaked softmax, low
    temperature on top: the exponent arithmetic (x*c - fl(max*c) with the residual folded
    back) must stay inside the tolerance relative to the size of the numbers involved."""
    import tome_b200
    from tome_b200 import synthetic
    hidden, weight, ids = synthetic.cfg3_lm_head(256, 512, 6000, "cpu", 52, 1.0)
    for temp in (1.0, 0.3):
        lp, lse = tome_b200.lm_head_logprob(hidden.to(cuda_device), weight.to(cuda_device),
                                            ids.to(cuda_device), temp, check=True)
        o_lp, o_lse = oracle.lm_head_logprob(hidden, weight, ids, temp)
        scale = float(o_lse.abs().max())
        assert scale > 60                       # the case is what it claims to be
        # fp32 carries ~7 digits: allow 2e-3 absolute or 2e-6 relative to the magnitude
        tol = max(TOL, 2e-6 * scale * 10)
        assert max_abs(lse, o_lse) <= tol and max_abs(lp, o_lp) <= 2 * tol, (max_abs(lp, o_lp), tol)


def test_leading_dims_and_golden(cuda_device):
    import tome_b200
    gld = load_golden("lm_head.npz")
    hidden = from_bits(gld["hidden"], torch.bfloat16).to(cuda_device)
    weight = from_bits(gld["weight"], torch.bfloat16).to(cuda_device)
    ids = torch.from_numpy(gld["ids"]).to(cuda_device)
    lp, lse = tome_b200.lm_head_logprob(hidden.view(4, 10, -1), weight, ids.view(4, 10), float(gld["temp"]))
    assert lp.shape == (4, 10)
    assert max_abs(lp.reshape(-1), torch.from_numpy(gld["logprob"])) <= TOL
    assert max_abs(lse.reshape(-1), torch.from_numpy(gld["lse"])) <= TOL


def test_shards_combine_to_the_unsharded_result(cuda_device):
    import tome_b200
    from tome_b200 import synthetic
    hidden, weight, ids = synthetic.cfg4_vocab_parallel(200, 256, 3000, "cpu", 1004)
    hd, wd, idd = hidden.to(cuda_device), weight.to(cuda_device), ids.to(cuda_device)
    full_lp, full_lse = tome_b200.lm_head_logprob(hd, wd, idd, 0.8)
    o_lp, o_lse = oracle.lm_head_logprob(hidden, weight, ids, 0.8)
    assert max_abs(full_lp, o_lp) <= TOL
    for world in (2, 4, 8):
        ms, ss, ts = [], [], []
        for r in range(world):
            b, e = synthetic.shard_bounds(3000, r, world)
            m, s, t = tome_b200.lm_head_partials(hd, wd[b:e].contiguous(), b, idd, 0.8)
            om, os_, ot = oracle.shard_triple(hidden, weight[b:e], b, ids, 0.8)
            assert max_abs(m, om) <= TOL and max_abs(t, ot) <= TOL
            assert max_abs(s.cpu() / os_, torch.ones_like(os_)) <= TOL
            ms.append(m), ss.append(s), ts.append(t)
        lp, lse = tome_b200.combine_triples(torch.stack(ms), torch.stack(ss), torch.stack(ts))
        assert max_abs(lp, o_lp) <= TOL and max_abs(lse, o_lse) <= TOL
        # the packed form of the all-reduce exchange: pre-summed target column
        lp2, _ = tome_b200.combine_triples(torch.stack(ms), torch.stack(ss),
                                           torch.stack(ts).sum(0, keepdim=True))
        assert max_abs(lp2, o_lp) <= TOL


def test_vocab_parallel_single_process_equals_unsharded(cuda_device):
    import tome_b200
    from tome_b200 import synthetic
    hidden, weight, ids = synthetic.cfg3_lm_head(100, 64, 900, "cpu", 31)
    hd, wd, idd = hidden.to(cuda_device), weight.to(cuda_device), ids.to(cuda_device)
    a, _ = tome_b200.lm_head_logprob_vocab_parallel(hd, wd, 0, idd, 1.0)
    b, _ = tome_b200.lm_head_logprob(hd, wd, idd, 1.0)
    assert max_abs(a, b) <= 1e-5


def test_out_of_range_target_is_reported(cuda_device):
    import tome_b200
    from tome_b200 import synthetic
    hidden, weight, ids = synthetic.cfg3_lm_head(64, 64, 500, "cpu", 32)
    ids[3] = 500
    tome_b200.lm_head_logprob(hidden.to(cuda_device), weight.to(cuda_device), ids.to(cuda_device), 1.0)
    with pytest.raises(tome_b200.TomeRuntimeError):
        tome_b200.check_device_status(cuda_device)


def test_caller_workspace_and_size_check(cuda_device):
    import tome_b200
    from tome_b200 import synthetic
    hidden, weight, ids = synthetic.cfg3_lm_head(64, 64, 500, "cpu", 33)
    need = tome_b200.lm_head_workspace_bytes(64, 64, 500)
    ws = torch.empty(need, dtype=torch.uint8, device=cuda_device)
    lp, _ = tome_b200.lm_head_logprob(hidden.to(cuda_device), weight.to(cuda_device),
                                      ids.to(cuda_device), 1.0, workspace=ws)
    o_lp, _ = oracle.lm_head_logprob(hidden, weight, ids, 1.0)
    assert max_abs(lp, o_lp) <= TOL
    with pytest.raises(ValueError):
        tome_b200.lm_head_logprob(hidden.to(cuda_device), weight.to(cuda_device), ids.to(cuda_device),
                                  1.0, workspace=ws[: need - 16])


def test_final_rmsnorm_and_model_tail(cuda_device):
    """RMSNorm kernel against the oracle (one bf16 ulp), then norm + head + log-prob in one
    call against the oracle's tail of Qwen3.__call__ (model.py:536-538)."""
    import tome_b200
    g = torch.Generator().manual_seed(50)
    x = (torch.randn((300, 1024), generator=g) * 3).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn((1024,), generator=g)).to(torch.bfloat16)
    y = tome_b200.rms_norm(x.to(cuda_device), w.to(cuda_device), 1e-6)
    ref = oracle.rms_norm(x, w, 1e-6)
    assert y.dtype == torch.bfloat16 and y.shape == x.shape
    rel = ((y.cpu().float() - ref.float()).abs() / ref.float().abs().clamp_min(1e-3)).max()
    assert float(rel) <= 2 ** -7, float(rel)   # at most one bf16 ulp
    assert float((y.cpu() == ref).float().mean()) > 0.99
    weight = (torch.randn((3000, 1024), generator=g) * 0.02).to(torch.bfloat16)
    ids = torch.randint(0, 3000, (300,), generator=g, dtype=torch.int32)
    lp, lse = tome_b200.lm_head_logprob(x.to(cuda_device), weight.to(cuda_device), ids.to(cuda_device),
                                        0.7, norm_weight=w.to(cuda_device), eps=1e-6)
    o_lp, o_lse = oracle.lm_head_logprob(ref, weight, ids, 0.7)
    assert max_abs(lp, o_lp) <= 5e-3 and max_abs(lse, o_lse) <= 5e-3  # norm may differ by an ulp


def test_bf16_rounded_logits_switch(cuda_device):
    """round_logits=True must reproduce the oracle evaluated on bf16-rounded logits (the
    reference's materialised path), which differs visibly from the un-rounded result."""
    import tome_b200
    from tome_b200 import synthetic
    hidden, weight, ids = synthetic.cfg3_lm_head(260, 512, 5000, "cpu", 51, 0.05)
    hd, wd, idd = hidden.to(cuda_device), weight.to(cuda_device), ids.to(cuda_device)
    lp_r, lse_r = tome_b200.lm_head_logprob(hd, wd, idd, 1.0, round_logits=True)
    o_lp_r, o_lse_r = oracle.lm_head_logprob(hidden, weight, ids, 1.0, round_to_bf16=True)
    # a logit that sits on a bf16 rounding boundary may round the other way on the GPU
    # (different fp32 summation order): allow one bf16 ulp of the target logit
    assert max_abs(lse_r, o_lse_r) <= TOL
    assert max_abs(lp_r, o_lp_r) <= TOL + 2 ** -6
    lp_u, _ = tome_b200.lm_head_logprob(hd, wd, idd, 1.0)
    o_lp_u, _ = oracle.lm_head_logprob(hidden, weight, ids, 1.0)
    assert max_abs(lp_u, o_lp_u) <= TOL
    assert max_abs(o_lp_r, o_lp_u) > TOL  # the switch matters


def test_single_cta_tiles_variant(cuda_device):
    """TOME_K2_PAIR=0 selects the cta_group::1 kernel (read once per process): child process."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import sys, torch; sys.path.insert(0, %r)\n"
        "import tome_b200; from oracle import oracle; from tome_b200 import synthetic\n"
        "for rows, k, vocab in ((300, 192, 4096 + 48), (129, 1024, 700)):\n"
        "    h, w, ids = synthetic.cfg3_lm_head(rows, k, vocab, 'cpu', 5, 0.05)\n"
        "    lp, lse = tome_b200.lm_head_logprob(h.cuda(), w.cuda(), ids.cuda(), 0.7, check=True)\n"
        "    o_lp, o_lse = oracle.lm_head_logprob(h, w, ids, 0.7)\n"
        "    err = float((lp.cpu() - o_lp).abs().max()); print(err); assert err <= 2e-3\n"
    ) % root
    env = dict(os.environ, TOME_K2_PAIR="0")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True,
                         timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr


def test_alternating_shapes_reuse_cached_plans(cuda_device):
    """Band plans are cached by shape (more shapes here than the cache holds, revisited in a
    different order): every call must still get the plan of its own shape."""
    shapes = [(128 * i + 7 * i, 64 + 8 * (i % 3), 256 * (i % 5 + 1) + 16 * i) for i in range(1, 20)]
    for rows, k, vocab in shapes + shapes[::-3] + shapes[:4]:
        _run(rows, k, vocab, 1.0, cuda_device, seed=rows % 17)
