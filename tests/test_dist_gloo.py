"""World-size-2 CPU (gloo) test of the vocab-parallel exchange: pack -> one SUM all-reduce ->
merge.  The per-shard triples come from the oracle here (kernels need a GPU); the packing and
the collective are the product's host code."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, fail_rank, out):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    from datetime import timedelta
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=20))
    try:
        from oracle import oracle
        from tome_b200 import dist as tdist, synthetic
        hidden, weight, ids = synthetic.cfg3_lm_head(33, 64, 1000, "cpu", 77)
        b, e = synthetic.shard_bounds(1000, rank, world)
        m, s, t = oracle.shard_triple(hidden, weight[b:e], b, ids, 0.7)
        if rank == fail_rank:
            raise RuntimeError("injected host-side failure before the collective")
        packed = tdist.pack_triples(m, s, t, rank, world)
        assert packed.shape == (2 * world + 1, 33)
        m_all, s_all, t_sum = tdist.exchange_triples(packed)
        lp, lse = oracle.combine_triples(m_all, s_all, t_sum)
        ref_lp, ref_lse = oracle.lm_head_logprob(hidden, weight, ids, 0.7)
        out[rank] = (float((lp - ref_lp).abs().max()), float((lse - ref_lse).abs().max()))
    except Exception as exc:  # reported to the parent instead of a silent hang
        out[rank] = repr(exc)
    finally:
        dist.destroy_process_group()


def _late_worker(rank, world, port, timeout_s, delay_s, out):
    """Rank 1 reaches the collective `delay_s` seconds late; rank 0 waits at most `timeout_s`."""
    import time
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    from datetime import timedelta
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=120))
    try:
        from tome_b200 import dist as tdist
        packed = tdist.pack_triples(torch.ones(5), torch.ones(5), torch.zeros(5), rank, world)
        dist.barrier()
        if rank == 1:
            time.sleep(delay_s)
        t0 = time.monotonic()
        try:
            tdist.exchange_triples(packed, timeout_s=timeout_s)
            out[rank] = ("completed", time.monotonic() - t0)
        except Exception as exc:
            out[rank] = (type(exc).__name__, time.monotonic() - t0)
        if rank == 0 and out[rank][0] != "completed":
            time.sleep(delay_s)  # stay until the late peer has had its partner
    finally:
        dist.destroy_process_group()


def _run_late(timeout_s, delay_s):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        out = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_late_worker, args=(r, 2, port, timeout_s, delay_s, out))
                 for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert not p.is_alive(), "a rank hung"
        return dict(out)


def _run(world, fail_rank=-1):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        out = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, fail_rank, out)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert not p.is_alive(), "a rank hung"
        return dict(out)


@pytest.mark.timeout(300)
def test_two_ranks_agree_with_unsharded_oracle():
    out = _run(2)
    assert set(out) == {0, 1}
    for r in (0, 1):
        assert isinstance(out[r], tuple), out[r]
        assert out[r][0] < 1e-5 and out[r][1] < 1e-5


@pytest.mark.timeout(300)
def test_rank_failure_surfaces_as_an_error_not_a_hang():
    # rank 1 raises before the all-reduce; rank 0's collective must end with an error
    # (peer closed / timeout) rather than block for ever
    out = _run(2, fail_rank=1)
    assert "injected" in out[1]
    assert isinstance(out[0], str), "rank 0 should have seen the collective fail"


def test_pack_layout():
    sys.path.insert(0, ROOT)
    from tome_b200 import dist as tdist
    m = torch.tensor([1.0, 2.0])
    s = torch.tensor([3.0, 4.0])
    t = torch.tensor([5.0, 0.0])
    p = tdist.pack_triples(m, s, t, rank=1, world=3)
    assert p.shape == (7, 2)
    assert torch.equal(p[1], m) and torch.equal(p[4], s) and torch.equal(p[6], t)
    assert float(p[[0, 2, 3, 5]].abs().sum()) == 0.0


@pytest.mark.timeout(300)
def test_exchange_timeout_raises_instead_of_waiting_for_the_group_timeout():
    # rank 1 comes 8 s late, rank 0 allows 2 s: it must raise long before the group's 120 s
    out = _run_late(timeout_s=2.0, delay_s=8.0)
    assert out[0][0] == "TomeRuntimeError", out
    assert out[0][1] < 2.0 + 5.0, out
    # a peer that is merely slow, within the limit, is waited for
    out = _run_late(timeout_s=30.0, delay_s=1.0)
    assert out[0][0] == "completed" and out[1][0] == "completed", out
