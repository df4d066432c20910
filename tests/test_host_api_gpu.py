"""GPU tests of the host-side forms a decode loop uses: preallocated outputs (``out=``) and
calls bound once and launched many times (``tome_b200.bind_*``).  The reference makes the same
call at every decode step with the same shapes (mlx-impl/node.py:590-605); these forms must give
what the plain functions give."""
import pytest
import torch

from helpers import max_abs
from oracle import oracle

pytestmark = pytest.mark.gpu


def _logits(rows, vocab, dtype, seed, dev):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((rows, vocab), generator=g) * 3.0).to(dtype)
    ids = torch.randint(0, vocab, (rows,), generator=g, dtype=torch.int32)
    return x, ids, x.to(dev), ids.to(dev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_out_arguments_receive_the_results(cuda_device, dtype):
    import tome_b200
    x, ids, xd, idd = _logits(24, 40000, dtype, 5, cuda_device)
    out = torch.full((24,), 7.0, dtype=torch.float32, device=cuda_device)
    lse = torch.full((24,), 7.0, dtype=torch.float32, device=cuda_device)
    got = tome_b200.selective_log_softmax(xd, idd, 0.7, out=out, out_lse=lse)
    assert got[0].data_ptr() == out.data_ptr() and got[1].data_ptr() == lse.data_ptr()
    o_lp, o_lse, _ = oracle.selective_logprob(x, ids, 0.7)
    tol = 1e-4 if dtype == torch.float32 else 2e-3
    assert max_abs(out, o_lp) <= tol and max_abs(lse, o_lse) <= tol
    assert tome_b200.local_compute_logprobs(xd, idd, 0.7, out=out).data_ptr() == out.data_ptr()
    tok = torch.full((24,), -5, dtype=torch.int32, device=cuda_device)
    got_tok, got_lp = tome_b200.sample_topk_logprob(xd, 0.7, 20, seed=3, offset=4, out=(tok, out))
    ref_tok, ref_lp = tome_b200.sample_topk_logprob(xd, 0.7, 20, seed=3, offset=4)
    assert got_tok.data_ptr() == tok.data_ptr() and got_lp.data_ptr() == out.data_ptr()
    assert torch.equal(tok, ref_tok) and torch.equal(out, ref_lp)
    with pytest.raises(ValueError):
        tome_b200.selective_log_softmax(xd, idd, 0.7, out=out[:5])
    with pytest.raises(ValueError):
        tome_b200.selective_log_softmax(xd, idd, 0.7, out=out.double())
    with pytest.raises(ValueError):
        tome_b200.sample_topk_logprob(xd, 0.7, 20, out=(out, out))    # tokens must be int32


@pytest.mark.parametrize("rows", [8, 700])
def test_bound_calls_track_their_buffers(cuda_device, rows):
    """A bound call reads whatever its tensors hold when it is launched."""
    import tome_b200
    vocab = 20000
    x, ids, xd, idd = _logits(rows, vocab, torch.bfloat16, 11, cuda_device)
    sel = tome_b200.bind_selective(xd, idd, 0.7)
    full = tome_b200.bind_log_softmax(xd, 0.7)
    smp = tome_b200.bind_sample(xd, 0.7, 20, seed=9)
    for round_no in range(2):
        (lp,) = sel()
        (mat,) = full()
        tok, tlp = smp(round_no + 1)
        assert torch.equal(lp, tome_b200.local_compute_logprobs(xd, idd, 0.7))
        assert torch.equal(mat, tome_b200.fused_log_softmax(xd, 0.7))
        ref_tok, ref_lp = tome_b200.sample_topk_logprob(xd, 0.7, 20, seed=9, offset=round_no + 1)
        assert torch.equal(tok, ref_tok) and max_abs(tlp, ref_lp) <= 1e-6
        # new contents in the same storage for the second round
        x2, ids2, _, _ = _logits(rows, vocab, torch.bfloat16, 12, cuda_device)
        xd.copy_(x2)
        idd.copy_(ids2)
    tome_b200.check_device_status(cuda_device)
    with pytest.raises(ValueError):
        tome_b200.bind_selective(xd[:, ::2], idd)          # rows must be contiguous
    with pytest.raises(ValueError):
        tome_b200.bind_selective(xd, idd.long())           # ids must be int32 on the device
