"""The hot calls are asynchronous, allocate nothing themselves and take the caller's stream,
so they can be recorded into a CUDA graph and replayed (a decode loop at small batch is bound
by launch overhead otherwise).  Each call is warmed up once outside capture first."""
import pytest
import torch

from helpers import max_abs
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_selective_sampling_and_head_replay_from_a_cuda_graph(cuda_device):
    import tome_b200
    from tome_b200 import synthetic
    g = torch.Generator().manual_seed(70)
    x = (torch.randn((16, 4096), generator=g) * 3).to(torch.bfloat16).to(cuda_device)
    ids = torch.randint(0, 4096, (16,), generator=g, dtype=torch.int32).to(cuda_device)
    hidden, weight, hids = synthetic.cfg3_lm_head(130, 128, 1000, "cpu", 71, 0.05)
    hd, wd, hidd = hidden.to(cuda_device), weight.to(cuda_device), hids.to(cuda_device)
    ws = torch.empty(tome_b200.lm_head_workspace_bytes(130, 128, 1000), dtype=torch.uint8,
                     device=cuda_device)

    def step():
        lp = tome_b200.local_compute_logprobs(x, ids, 0.7)
        tok, tlp = tome_b200.sample_topk_logprob(x, 0.7, 20, seed=3, offset=9)
        hlp, _ = tome_b200.lm_head_logprob(hd, wd, hidd, 1.0, workspace=ws)
        return lp, tok, tlp, hlp

    side = torch.cuda.Stream(device=cuda_device)
    side.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(side):
        eager = step()                      # warm-up: function attributes, status word
    torch.cuda.current_stream(cuda_device).wait_stream(side)
    torch.cuda.synchronize()

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    x.copy_((x.float() * 0.5 + 0.25).to(torch.bfloat16))   # new inputs, same buffers
    graph.replay()
    torch.cuda.synchronize()
    o_lp, _, _ = oracle.selective_logprob(x.cpu(), ids.cpu(), 0.7)
    assert max_abs(captured[0], o_lp) <= 2e-3
    o_tlp, _, _ = oracle.selective_logprob(x.cpu(), captured[1].cpu(), 0.7)
    assert max_abs(captured[2], o_tlp) <= 2e-3
    o_hlp, _ = oracle.lm_head_logprob(hidden, weight, hids, 1.0)
    assert max_abs(captured[3], o_hlp) <= 2e-3
    assert not torch.equal(captured[0], eager[0])           # the replay really recomputed
    tome_b200.check_device_status(cuda_device)


def test_large_batch_sampling_and_full_matrix_replay_from_a_cuda_graph(cuda_device):
    """The streaming sampling path (scratch allocated by the wrapper inside the capture; its
    kernels are chained by programmatic launches) and
    the cluster full-matrix kernel, captured and replayed on new inputs."""
    import tome_b200
    g = torch.Generator().manual_seed(72)
    x = (torch.randn((400, 8192), generator=g) * 3).to(torch.bfloat16).to(cuda_device)
    wide = (torch.randn((300, 70000), generator=g) * 2).to(cuda_device)    # fp32, 280 KB rows
    out = torch.empty_like(wide)

    def step():
        tok, tlp = tome_b200.sample_topk_logprob(x, 0.7, 20, seed=3, offset=9)
        tome_b200.fused_log_softmax(wide, 0.7, out=out)
        return tok, tlp

    side = torch.cuda.Stream(device=cuda_device)
    side.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(side):
        eager = step()
    torch.cuda.current_stream(cuda_device).wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    x.copy_((x.float() * 0.5 + 0.25).to(torch.bfloat16))
    wide.mul_(0.5)
    graph.replay()
    torch.cuda.synchronize()
    o_tlp, _, _ = oracle.selective_logprob(x.cpu(), captured[0].cpu(), 0.7)
    assert max_abs(captured[1], o_tlp) <= 2e-3
    for r in (0, 199, 399):
        idx, _ = oracle.topk_sampling_distribution(x[r].cpu(), 0.7, 20)
        assert int(captured[0][r]) in idx.tolist()
    assert max_abs(out[:8], oracle.log_softmax_metal_order(wide[:8].cpu(), 0.7)) <= 1e-4
    assert eager[0].shape == captured[0].shape
    tome_b200.check_device_status(cuda_device)
