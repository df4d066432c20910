"""GPU test of the allocation-free LM-head entry point (collected last on purpose).

`tome_lmhead_logprob_static` keeps its scratch in a fixed array inside the library instead
of taking a workspace, for hosts that cannot allocate device memory themselves.  It must
give the same numbers as `tome_lmhead_logprob` with a caller-provided workspace, on two
calls in a row (the array is shared and keeps the previous call's contents), and it must
refuse problems whose scratch does not fit.  The calls go through the C ABI with ctypes.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-3  # the tolerance of the fused LM-head tests


def _call_pair(lib, hidden, weight, ids, temp, stream):
    rows, k = hidden.shape
    vocab = weight.shape[0]
    dev = hidden.device
    need = lib.tome_lmhead_workspace_bytes(rows, k, vocab)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    ref_lp = torch.empty(rows, dtype=torch.float32, device=dev)
    ref_lse = torch.empty_like(ref_lp)
    st = lib.tome_lmhead_logprob(hidden.data_ptr(), weight.data_ptr(), rows, k, vocab,
                                 ids.data_ptr(), temp, 0, ref_lp.data_ptr(), ref_lse.data_ptr(),
                                 ws.data_ptr(), need, None, stream)
    assert st == 0, lib.tome_last_error_string()
    lp = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
    lse = torch.full((rows,), float("nan"), dtype=torch.float32, device=dev)
    st = lib.tome_lmhead_logprob_static(hidden.data_ptr(), weight.data_ptr(), rows, k, vocab,
                                        ids.data_ptr(), temp, lp.data_ptr(), lse.data_ptr(),
                                        None, stream)
    assert st == 0, lib.tome_last_error_string()
    torch.cuda.synchronize()
    return (lp - ref_lp).abs().max().item(), (lse - ref_lse).abs().max().item()


def test_static_scratch_matches_workspace_variant_twice(cuda_device):
    from tome_b200 import _lib, synthetic
    lib = _lib.lib
    assert lib.tome_lmhead_static_scratch_bytes() == 8 << 20
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    # two different problems back to back: the second must not see the first one's leftovers
    cases = [(300, 256, 5000, 0.8, 41), (1000, 128, 2100, 1.0, 42)]
    for rows, k, vocab, temp, seed in cases:
        hidden, weight, ids = synthetic.cfg3_lm_head(rows, k, vocab, "cpu", seed, 0.05)
        hd, wd, idd = hidden.to(cuda_device), weight.to(cuda_device), ids.to(cuda_device)
        err_lp, err_lse = _call_pair(lib, hd, wd, idd, temp, stream)
        assert err_lp <= TOL and err_lse <= TOL, (rows, k, vocab, err_lp, err_lse)
    # the same problem again, straight after: identical to its own first answer
    err_lp, err_lse = _call_pair(lib, hd, wd, idd, 1.0, stream)
    assert err_lp <= TOL and err_lse <= TOL


def test_static_scratch_large_problem_and_no_allocation(cuda_device):
    """A problem whose scratch takes several MiB of the 8 MiB array (many rows against a wide
    vocabulary, small K), so that the plane offsets inside the array are used, and a check of
    the claim itself: once the first call on the device is over, further calls change neither
    the driver's free-memory figure nor torch's own allocation count."""
    from tome_b200 import _lib, synthetic
    lib = _lib.lib
    rows, k, vocab = 8192, 64, 120000
    need = lib.tome_lmhead_workspace_bytes(rows, k, vocab)
    assert (2 << 20) < need <= lib.tome_lmhead_static_scratch_bytes(), need
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    hidden, weight, ids = synthetic.cfg3_lm_head(rows, k, vocab, cuda_device, 44, 0.05)
    err_lp, err_lse = _call_pair(lib, hidden, weight, ids, 0.9, stream)   # includes the first call
    assert err_lp <= TOL and err_lse <= TOL, (err_lp, err_lse)
    lp = torch.empty(rows, dtype=torch.float32, device=cuda_device)
    lse = torch.empty_like(lp)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(cuda_device)[0]
    allocated_before = torch.cuda.memory_allocated(cuda_device)
    allocs_before = torch.cuda.memory_stats(cuda_device).get("allocation.all.allocated", 0)
    for _ in range(3):
        st = lib.tome_lmhead_logprob_static(hidden.data_ptr(), weight.data_ptr(), rows, k, vocab,
                                            ids.data_ptr(), 0.9, lp.data_ptr(), lse.data_ptr(),
                                            None, stream)
        assert st == 0, lib.tome_last_error_string()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(cuda_device)[0] == free_before
    assert torch.cuda.memory_allocated(cuda_device) == allocated_before
    assert torch.cuda.memory_stats(cuda_device).get("allocation.all.allocated", 0) == allocs_before


def test_static_scratch_python_wrapper_and_oracle(cuda_device):
    import tome_b200
    from oracle import oracle
    from tome_b200 import synthetic
    hidden, weight, ids = synthetic.cfg3_lm_head(200, 64, 900, "cpu", 43, 0.05)
    hd, wd, idd = hidden.to(cuda_device), weight.to(cuda_device), ids.to(cuda_device)
    lp = torch.empty(200, dtype=torch.float32, device=cuda_device)
    lse = torch.empty_like(lp)
    for _ in range(2):
        tome_b200.lm_head_logprob_static(hd, wd, idd, 0.7, lp, lse)
    o_lp, o_lse = oracle.lm_head_logprob(hidden, weight, ids, 0.7)
    assert (lp.cpu() - o_lp).abs().max().item() <= TOL
    assert (lse.cpu() - o_lse).abs().max().item() <= TOL
    # shapes that would make the kernels run past a buffer are refused before the call
    with pytest.raises(ValueError):
        tome_b200.lm_head_logprob_static(hd, wd, idd[:-1], 0.7, lp, lse)
    with pytest.raises(ValueError):
        tome_b200.lm_head_logprob_static(hd, wd, idd, 0.7, lp[:-1], lse)
    with pytest.raises(ValueError):
        tome_b200.lm_head_logprob_static(hd, wd, idd, 0.7, lp, lse[:10])
    with pytest.raises(ValueError):
        tome_b200.lm_head_logprob_static(hd, wd[:, :32].contiguous(), idd, 0.7, lp, lse)
    with pytest.raises(tome_b200.TomeRuntimeError):
        tome_b200.lm_head_logprob_static(hd, wd, idd, 0.7, lp, lse.cpu())


def test_static_scratch_rejects_oversized_problems(cuda_device):
    from tome_b200 import _lib
    lib = _lib.lib
    rows, k, vocab = 65536, 1024, 151936
    assert lib.tome_lmhead_workspace_bytes(rows, k, vocab) > lib.tome_lmhead_static_scratch_bytes()
    fake = 0x1000  # rejected on the host before any pointer is used
    st = lib.tome_lmhead_logprob_static(fake, fake, rows, k, vocab, fake, 1.0, fake, None, None, None)
    assert st == -9
    assert b"scratch" in lib.tome_last_error_string()
    with pytest.raises(_lib.TomeArgumentError):
        _lib.check(st)
