"""Two-rank NCCL test of the vocab-parallel head on real GPUs (skipped with fewer than two).
Each rank is a child process that owns one GPU; the per-shard triples come from the fused
kernel, the exchange is the single all-reduce, and every rank must reproduce the unsharded
result of the oracle."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist
    from datetime import timedelta
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=timedelta(seconds=60))
    try:
        import tome_b200
        from oracle import oracle
        from tome_b200 import synthetic
        hidden, weight, ids = synthetic.cfg4_vocab_parallel(300, 256, 5000, "cpu", 1004)
        b, e = synthetic.shard_bounds(5000, rank, world)
        lp, lse = tome_b200.lm_head_logprob_vocab_parallel(
            hidden.to(dev), weight[b:e].contiguous().to(dev), b, ids.to(dev), 0.8)
        tome_b200.check_device_status(dev)
        o_lp, o_lse = oracle.lm_head_logprob(hidden, weight, ids, 0.8)
        out[rank] = (float((lp.cpu() - o_lp).abs().max()), float((lse.cpu() - o_lse).abs().max()))
    except Exception as exc:
        out[rank] = repr(exc)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_gpu_vocab_parallel_matches_unsharded(built_lib):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        out = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert not p.is_alive(), "a rank hung"
        res = dict(out)
    for r in (0, 1):
        assert isinstance(res.get(r), tuple), res.get(r)
        assert res[r][0] <= 2e-3 and res[r][1] <= 2e-3, res[r]
