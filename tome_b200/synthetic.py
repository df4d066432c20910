"""Seeded synthetic inputs with the shapes and value distributions of the five workloads.

No dataset or checkpoint is involved: the reference measures on ad-hoc prompts and the real
Qwen3 weights are not available offline, so random tensors of the named shapes stand in.
Vocabulary 151936 and hidden size 1024 are the reference's Qwen3-0.6B constants
(mlx-impl/node.py:950-964).  Each generator takes ``rows`` (or ``n_seq``) so that tests can
draw the same distribution at a size a CPU oracle finishes in seconds.  A generator seeded
on CPU and one seeded on a GPU give different streams; parity tests generate on CPU and
copy, so that the oracle and the kernels see identical bits.
"""
from __future__ import annotations

import torch

VOCAB = 151936
SEEDS = {"cfg1": 1001, "cfg2": 1002, "cfg3": 1003, "cfg4": 1004, "cfg5": 1005}


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _randn_chunked(shape, g, device, scale: float, dtype, chunk_rows: int = 2048) -> torch.Tensor:
    """Normal(0, scale^2) drawn in fp32 row chunks, stored as ``dtype`` (bounds peak memory)."""
    out = torch.empty(shape, dtype=dtype, device=device)
    flat = out.view(-1, shape[-1])
    for b in range(0, flat.shape[0], chunk_rows):
        e = min(flat.shape[0], b + chunk_rows)
        flat[b:e] = (torch.randn((e - b, shape[-1]), generator=g, device=device,
                                 dtype=torch.float32) * scale).to(dtype)
    return out


def cfg1_selective_fp32(rows: int = 1024, vocab: int = VOCAB, device="cpu", seed: int = 1001):
    """fp32 logits [rows, vocab] ~ N(0, 2^2); int32 targets uniform in [0, vocab)."""
    g = _gen(seed, device)
    logits = _randn_chunked((rows, vocab), g, device, 2.0, torch.float32)
    targets = torch.randint(0, vocab, (rows,), generator=g, device=device, dtype=torch.int32)
    return logits, targets


def cfg2_rollout_bf16(rows: int = 20480, vocab: int = VOCAB, device="cpu", seed: int = 1002,
                      chunk_rows: int = 2048):
    """bf16 logits [rows, vocab] ~ N(0, 3^2) with one planted column per row set to +12
    (the "argmax" token); targets are the planted column with p = 0.7, else uniform.
    20480 rows stand for 4 prompts x group 8 x 640 tokens."""
    g = _gen(seed, device)
    logits = torch.empty((rows, vocab), dtype=torch.bfloat16, device=device)
    planted = torch.randint(0, vocab, (rows,), generator=g, device=device)
    for b in range(0, rows, chunk_rows):
        e = min(rows, b + chunk_rows)
        x = torch.randn((e - b, vocab), generator=g, device=device, dtype=torch.float32) * 3.0
        x.scatter_(1, planted[b:e, None], 12.0)
        logits[b:e] = x.to(torch.bfloat16)
    keep = torch.rand((rows,), generator=g, device=device) < 0.7
    other = torch.randint(0, vocab, (rows,), generator=g, device=device)
    targets = torch.where(keep, planted, other).to(torch.int32)
    return logits, targets


def cfg3_lm_head(rows: int = 16384, hidden_dim: int = 1024, vocab: int = VOCAB, device="cpu",
                 seed: int = 1003, w_scale: float = 0.02):
    """hidden bf16 [rows, hidden_dim] ~ N(0,1); tied-embedding stand-in W bf16
    [vocab, hidden_dim] ~ N(0, 0.02^2); int32 targets uniform."""
    g = _gen(seed, device)
    hidden = _randn_chunked((rows, hidden_dim), g, device, 1.0, torch.bfloat16)
    weight = _randn_chunked((vocab, hidden_dim), g, device, w_scale, torch.bfloat16, 8192)
    targets = torch.randint(0, vocab, (rows,), generator=g, device=device, dtype=torch.int32)
    return hidden, weight, targets


def cfg4_vocab_parallel(rows: int = 32768, hidden_dim: int = 4096, vocab: int = VOCAB,
                        device="cpu", seed: int = 1004):
    """8B-class head: hidden bf16 [rows, 4096] ~ N(0,1); W bf16 [vocab, 4096] ~ N(0, 0.015^2).
    Every rank draws the same tensors from the same seed and keeps its own row slice of W."""
    return cfg3_lm_head(rows, hidden_dim, vocab, device, seed, w_scale=0.015)


def shard_bounds(vocab: int, rank: int, world: int):
    """Row range [begin, end) of the weight matrix owned by ``rank`` (contiguous, even split;
    151936 divides evenly by 1, 2, 4 and 8)."""
    per = (vocab + world - 1) // world
    begin = min(vocab, rank * per)
    return begin, min(vocab, begin + per)


def cfg5_dual(n_seq: int = 32, seq_len: int = 768, vocab: int = VOCAB, device="cpu",
              seed: int = 1005, min_len: int = 64, chunk_rows: int = 1024):
    """Policy logits bf16 [n_seq, seq_len, vocab] ~ N(0, 3^2); reference = policy + N(0, 0.1^2);
    completion lengths uniform in [min_len, seq_len]; targets uniform; temperature 0.7."""
    g = _gen(seed, device)
    rows = n_seq * seq_len
    policy = torch.empty((rows, vocab), dtype=torch.bfloat16, device=device)
    ref = torch.empty((rows, vocab), dtype=torch.bfloat16, device=device)
    for b in range(0, rows, chunk_rows):
        e = min(rows, b + chunk_rows)
        x = torch.randn((e - b, vocab), generator=g, device=device, dtype=torch.float32) * 3.0
        policy[b:e] = x.to(torch.bfloat16)
        x += torch.randn((e - b, vocab), generator=g, device=device, dtype=torch.float32) * 0.1
        ref[b:e] = x.to(torch.bfloat16)
    lo = min(min_len, seq_len)
    lengths = torch.randint(lo, seq_len + 1, (n_seq,), generator=g, device=device,
                            dtype=torch.int32)
    targets = torch.randint(0, vocab, (n_seq, seq_len), generator=g, device=device,
                            dtype=torch.int32)
    return (policy.view(n_seq, seq_len, vocab), ref.view(n_seq, seq_len, vocab), targets,
            lengths, 0.7)
