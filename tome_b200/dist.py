"""Vocab-parallel LM head: each rank owns a row shard of the weight matrix.

One process per GPU.  Rank r holds weight rows ``[vocab_offset, vocab_offset + V_local)``;
hidden states and targets are replicated.  Every rank reduces its shard to a per-row triple
``(m, s, t)`` with the fused kernel, the triples are exchanged with ONE ``all_reduce`` over
a zero-padded packed buffer (NCCL over NVLink on GPUs), and a merge kernel forms the
log-probs on every rank.  The reference has no sharded head (it serves one model per
process, mlx-impl/node.py:966-970); parity is defined against the unsharded result.
"""
from __future__ import annotations

import time
from typing import Optional

import torch
import torch.distributed as dist

from . import ops
from ._lib import TomeRuntimeError


def pack_triples(m: torch.Tensor, s: torch.Tensor, t: torch.Tensor, rank: int, world: int,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Packed exchange buffer ``[2*world + 1, rows]`` of one rank.

    Row ``rank`` holds ``m``, row ``world + rank`` holds ``s``, the last row holds ``t``; all
    other rows are zero, so that a SUM all-reduce leaves every rank with every shard's
    ``(m, s)`` pair and with the target logit (only the owning shard contributes a non-zero).
    """
    rows = m.shape[0]
    if out is None:
        out = torch.zeros((2 * world + 1, rows), dtype=torch.float32, device=m.device)
    else:
        out.zero_()
    out[rank].copy_(m)
    out[world + rank].copy_(s)
    out[2 * world].copy_(t)
    return out


def exchange_triples(packed: torch.Tensor, group=None, timeout_s: Optional[float] = None):
    """The single collective of the path: SUM all-reduce of the packed buffer, in place.

    Returns views ``(m_all [world, rows], s_all [world, rows], t_sum [1, rows])``.

    With ``timeout_s`` the all-reduce is issued asynchronously and the host polls it: if it
    has not completed after that many seconds (a peer that died or never made the call), a
    ``TomeRuntimeError`` is raised instead of waiting for the process group's own timeout
    (ten minutes by default).  The wait then holds the calling thread until the collective is
    done, so use it where a stalled step must be noticed, not in a loop tuned for overlap.
    After the error the group is in an undefined state: tear it down.
    """
    world = (packed.shape[0] - 1) // 2
    if world > 1:
        if timeout_s is None:
            dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
        else:
            work = dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group, async_op=True)
            deadline = time.monotonic() + float(timeout_s)
            pause = 50e-6
            while not work.is_completed():
                if time.monotonic() > deadline:
                    raise TomeRuntimeError(
                        f"the all-reduce of the vocab-parallel head did not complete within "
                        f"{timeout_s} s: a peer is gone or never made the call")
                time.sleep(pause)
                pause = min(2 * pause, 5e-3)
            work.wait()  # completed: orders the current stream after the collective
    return packed[:world], packed[world:2 * world], packed[2 * world:]


def lm_head_logprob_vocab_parallel(hidden: torch.Tensor, weight_shard: torch.Tensor,
                                   vocab_offset: int, ids: torch.Tensor, temp: float = 1.0,
                                   group=None, *, workspace: Optional[torch.Tensor] = None,
                                   packed: Optional[torch.Tensor] = None,
                                   timeout_s: Optional[float] = None):
    """``(logprob, lse)`` of ``ids`` under the full-vocabulary softmax, head sharded by rows.

    ``weight_shard`` is this rank's ``[V_local, K]`` slice starting at global row
    ``vocab_offset``; ``ids`` are global indices.  All ranks of ``group`` must call this with
    the same ``hidden``/``ids``.  ``packed`` may be a reusable ``[2*world+1, rows]`` fp32 buffer.
    ``timeout_s`` bounds the wait for the peers (see :func:`exchange_triples`).
    """
    if dist.is_available() and dist.is_initialized():
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
    else:
        world, rank = 1, 0
    rows = hidden.numel() // hidden.shape[-1]
    if packed is None:
        packed = torch.zeros((2 * world + 1, rows), dtype=torch.float32, device=hidden.device)
    else:
        if packed.shape != (2 * world + 1, rows) or packed.dtype != torch.float32 or \
                not packed.is_contiguous():
            raise ValueError(f"packed must be a contiguous fp32 [{2 * world + 1}, {rows}] tensor")
        packed.zero_()
    # the kernel writes this rank's slots of the exchange buffer directly
    ops.lm_head_partials(hidden, weight_shard, vocab_offset, ids, temp, workspace=workspace,
                         out=(packed[rank], packed[world + rank], packed[2 * world]))
    m_all, s_all, t_sum = exchange_triples(packed, group, timeout_s)
    lp, lse = ops.combine_triples(m_all, s_all, t_sum)
    lead = hidden.shape[:-1]
    return lp.reshape(lead), lse.reshape(lead)
