"""CPU oracle: a restatement of the reference's log-prob arithmetic.  TEST INFRASTRUCTURE ONLY.

Nothing in the product imports this file.  Only ``tests/``, ``__graft_entry__.smoke()`` and
the CPU-baseline / reference legs of ``bench.py`` use it, and only as the checker or as the
timed CPU baseline.

PARITY.  Pinned for the full-matrix kernel and the policy call site, unpinned for the rest:

* ``log_softmax_metal_order`` (mlx-impl/model.py:14-89) and, through it, the policy call site
  ``fused_log_softmax(...)[b, token]`` (mlx-impl/node.py:590, 605) are pinned to OUTPUTS OF THE
  REFERENCE'S OWN KERNEL: oracle/build_ref.py compiles the reference's Metal kernel body,
  unmodified and from where it lies in the reference checkout, around a CPU emulation of the
  Metal execution model (oracle/metal_emulation.cpp); tests/golden/metal_kernel.npz holds what
  it computes (tests/golden/make_metal_golden.py), and tests/test_metal_reference.py holds this
  file against it (fp32: within 4e-6, bf16: bit-exact on the fixture).  Not the reference's in
  that run: Apple's fast::exp / fast::log are libm's, simdgroup sums add in butterfly order.
  ``gather_paged_kv`` is pinned the same way (mlx-impl/paged_kv.py:57-116, byte-exact).
* PARITY UNPINNED for ``local_compute_logprobs`` (node.py:400-404) and everything built on it:
  the reference computes those with MLX array ops (``mlx>=0.30.6``, unpinned in the
  reference's pyproject.toml and not vendored), MLX is not installed here and cannot be
  installed offline, and the reference holds no golden vectors or known-answer tests for the
  path (its only numeric test, mlx-impl/tests/test_logprob_comparison.py:84-102, draws unseeded
  random logits and compares against ``logits - mx.logsumexp(logits)`` within 5e-3).  Those
  functions are pinned by FORMULA only, cross-checked against float64 and
  ``torch.log_softmax`` in tests/test_oracle.py and against the pinned function above (the two
  differ by one rounding: division by T against multiplication by 1/T); the other fixtures
  under tests/golden/ were produced by this file (tests/golden/make_golden.py).

Each function names the reference lines it follows.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch


def _f32(x) -> torch.Tensor:
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(x)
    return x.detach().to("cpu").to(torch.float32)


def _i64(x) -> torch.Tensor:
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(x)
    return x.detach().to("cpu").to(torch.int64)


def logsumexp_f32(x: torch.Tensor) -> torch.Tensor:
    """Max-shifted logsumexp over the last axis in fp32 (what ``mx.logsumexp`` computes,
    mlx-impl/node.py:402)."""
    m = x.max(dim=-1, keepdim=True).values
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    return (m + torch.log(torch.exp(x - m).sum(dim=-1, keepdim=True))).squeeze(-1)


def selective_logprob(logits, ids, temp: float, chunk_rows: int = 512):
    """mlx-impl/node.py:400-404 (``local_compute_logprobs``).

        logits = logits.astype(float32) / temp
        log_z = logsumexp(logits, axis=-1)
        token_logits = take_along_axis(logits, ids)
        return token_logits - log_z

    Returns ``(logprob, lse, raw_target_logit)`` as fp32 tensors of the leading shape.
    """
    V = logits.shape[-1]
    lead = tuple(logits.shape[:-1])
    flat = logits.reshape(-1, V)
    idx = _i64(ids).reshape(-1)
    temp32 = torch.tensor(float(temp), dtype=torch.float32)
    lp = torch.empty(flat.shape[0], dtype=torch.float32)
    lse = torch.empty_like(lp)
    raw = torch.empty_like(lp)
    for b in range(0, flat.shape[0], chunk_rows):
        e = min(flat.shape[0], b + chunk_rows)
        x32 = _f32(flat[b:e])
        x = x32 / temp32
        z = logsumexp_f32(x)
        tok = x.gather(1, idx[b:e, None]).squeeze(1)
        lp[b:e] = tok - z
        lse[b:e] = z
        raw[b:e] = x32.gather(1, idx[b:e, None]).squeeze(1)
    return lp.reshape(lead), lse.reshape(lead), raw.reshape(lead)


def selective_logprob_f64(logits, ids, temp: float, chunk_rows: int = 256):
    """The same formula in float64, used to bound the fp32 oracle's own error."""
    V = logits.shape[-1]
    lead = tuple(logits.shape[:-1])
    flat = logits.reshape(-1, V)
    idx = _i64(ids).reshape(-1)
    lp = torch.empty(flat.shape[0], dtype=torch.float64)
    for b in range(0, flat.shape[0], chunk_rows):
        e = min(flat.shape[0], b + chunk_rows)
        x = _f32(flat[b:e]).to(torch.float64) / float(temp)
        z = torch.logsumexp(x, dim=-1)
        lp[b:e] = x.gather(1, idx[b:e, None]).squeeze(1) - z
    return lp.reshape(lead)


def log_softmax_reference(logits, temp: float = 1.0) -> torch.Tensor:
    """The expectation of the reference's kernel test,
    mlx-impl/tests/test_logprob_comparison.py:90: ``x - logsumexp(x, keepdims=True)``,
    evaluated in fp32 on ``x = logits / temp``.  Returns fp32 ``[..., V]``."""
    x = _f32(logits) / torch.tensor(float(temp), dtype=torch.float32)
    return x - logsumexp_f32(x).unsqueeze(-1)


def log_softmax_metal_order(logits, temp: float = 1.0) -> torch.Tensor:
    """Order of operations of the Metal kernel, mlx-impl/model.py:27-65.

        inv_temp = 1 / temp                                  (:27)
        row_max  = max_j float(x_j) * inv_temp               (:28-42)
        sum_exp  = sum_j exp(float(x_j) * inv_temp - row_max)(:43-55)
        lse      = T(row_max + log(sum_exp))                 (:56-57)
        out_j    = T(float(x_j) * inv_temp) - lse            (:58-65), subtraction in T

    Returns a tensor of the input dtype T (fp32 or bf16).
    """
    if isinstance(logits, np.ndarray):
        logits = torch.from_numpy(logits)
    T = logits.dtype
    inv = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(float(temp), dtype=torch.float32)
    x = _f32(logits) * inv
    row_max = x.max(dim=-1, keepdim=True).values
    sum_exp = torch.exp(x - row_max).sum(dim=-1, keepdim=True)
    lse = (row_max + torch.log(sum_exp)).to(T)
    scaled = x.to(T)
    if T == torch.float32:
        return scaled - lse
    return (scaled.to(torch.float32) - lse.to(torch.float32)).to(T)


def rms_norm(x, weight, eps: float = 1e-6) -> torch.Tensor:
    """mlx-impl/model.py:336-343 (``mx.fast.rms_norm(x, weight, eps)``), applied to the last
    hidden states at model.py:536: ``x * rsqrt(mean(x^2) + eps) * weight`` in fp32, rounded once
    to the input dtype.  (Where MLX's kernel places its casts is not visible from the
    reference; results can differ from it by one bf16 ulp.)"""
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(x)
    x32 = _f32(x)
    inv = torch.rsqrt((x32 * x32).mean(dim=-1, keepdim=True) + torch.tensor(eps, dtype=torch.float32))
    return (x32 * inv * _f32(weight)).to(x.dtype)


def lm_head_logits(hidden, weight, round_to_bf16: bool = False) -> torch.Tensor:
    """mlx-impl/model.py:538: ``x @ embed_tokens.weight.T`` with bf16 operands and fp32
    accumulation.  ``round_to_bf16`` reproduces the materialised bf16 logits of the
    reference; the fused kernel never rounds, so the un-rounded form is the primary oracle."""
    x = _f32(hidden) @ _f32(weight).T
    if round_to_bf16:
        x = x.to(torch.bfloat16).to(torch.float32)
    return x


def lm_head_logprob(hidden, weight, ids, temp: float = 1.0, round_to_bf16: bool = False,
                    chunk_rows: int = 256):
    """LM head (model.py:538) followed by ``local_compute_logprobs`` (node.py:400-404).
    Returns ``(logprob, lse)``."""
    K = hidden.shape[-1]
    lead = tuple(hidden.shape[:-1])
    h = hidden.reshape(-1, K)
    idx = _i64(ids).reshape(-1)
    lp = torch.empty(h.shape[0], dtype=torch.float32)
    lse = torch.empty_like(lp)
    w32 = _f32(weight)
    for b in range(0, h.shape[0], chunk_rows):
        e = min(h.shape[0], b + chunk_rows)
        x = _f32(h[b:e]) @ w32.T
        if round_to_bf16:
            x = x.to(torch.bfloat16).to(torch.float32)
        a, z, _ = selective_logprob(x, idx[b:e], temp)
        lp[b:e] = a
        lse[b:e] = z
    return lp.reshape(lead), lse.reshape(lead)


def shard_triple(hidden, weight_shard, vocab_offset: int, ids, temp: float = 1.0):
    """Per-row triple of one vocabulary shard (no counterpart in the reference, which has no
    sharded head): ``m = max_j x_j / temp``, ``s = sum_j exp(x_j/temp - m)``,
    ``t = x_target/temp`` if ``vocab_offset <= id < vocab_offset + V_local`` else 0."""
    x = lm_head_logits(hidden.reshape(-1, hidden.shape[-1]), weight_shard)
    x = x / torch.tensor(float(temp), dtype=torch.float32)
    idx = _i64(ids).reshape(-1) - int(vocab_offset)
    m = x.max(dim=-1).values
    s = torch.exp(x - m[:, None]).sum(dim=-1)
    owned = (idx >= 0) & (idx < x.shape[1])
    safe = torch.where(owned, idx, torch.zeros_like(idx))
    t = torch.where(owned, x.gather(1, safe[:, None]).squeeze(1), torch.zeros_like(m))
    return m, s, t


def combine_triples(m, s, t):
    """Merge of shard triples ``[parts, rows]``: ``M = max m``, ``S = sum s * exp(m - M)``,
    ``lse = M + log S``, ``logprob = sum t - lse``.  Returns ``(logprob, lse)``."""
    m, s, t = _f32(m), _f32(s), _f32(t)
    M = m.max(dim=0).values
    S = (s * torch.exp(m - M[None, :])).sum(dim=0)
    lse = M + torch.log(S)
    return t.sum(dim=0) - lse, lse


def ragged_logprobs(logits, targets_per_seq, lengths, temp: float = 1.0, starts=None):
    """mlx-impl/node.py:446-458, the per-sequence loop of ``_process_ref_logprobs_batched``:

        c_logits = logits[i, p_len - 1 : p_len - 1 + len(c_toks)]
        lps = local_compute_logprobs(c_logits, c_targets, temperature or 1.0)
        ... ref_log_probs.extend(lps.tolist())

    ``targets_per_seq[i]`` are the completion tokens of sequence ``i``; returns the list of
    per-sequence fp32 tensors (what lands in ``Completion.ref_log_probs``)."""
    n_seq, seq_len, _ = logits.shape
    lengths = _i64(lengths).reshape(-1)
    starts_t = torch.zeros_like(lengths) if starts is None else _i64(starts).reshape(-1)
    out = []
    for i in range(n_seq):
        st = int(max(0, min(int(starts_t[i]), seq_len)))
        ln = int(max(0, min(int(lengths[i]), seq_len - st)))
        if ln == 0:
            out.append(torch.zeros(0, dtype=torch.float32))
            continue
        lp, _, _ = selective_logprob(logits[i, st:st + ln], _i64(targets_per_seq[i])[:ln], temp or 1.0)
        out.append(lp)
    return out


def topk_sampling_distribution(logits_row, temperature: float, top_k: int = 20):
    """The distribution ``_sample_token`` draws from (mlx-impl/node.py:894-907): the ``top_k``
    largest of ``logits / temperature`` (ties: lower index first, as a stable sort gives) and
    the categorical probabilities ``softmax(top_logits)`` over them.  Temperature 0 is argmax.
    Returns ``(indices int64 [k], probabilities float64 [k])`` ordered by descending logit."""
    x = _f32(logits_row).reshape(-1)
    k = min(top_k, x.numel())
    if not temperature or temperature <= 0:
        return torch.argmax(x).reshape(1), torch.ones(1, dtype=torch.float64)
    order = torch.sort(x, descending=True, stable=True).indices[:k]
    top = (x[order] / torch.tensor(float(temperature), dtype=torch.float32)).to(torch.float64)
    return order, torch.softmax(top, dim=0)


def dual_logprob_kl(policy_logits, ref_logits, ids, lengths, temp: float = 1.0,
                    starts=None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """GRPO dual scoring on the ragged completion window of each sequence.

    Window: mlx-impl/node.py:446-451 (``logits[i, p_len-1 : p_len-1+len(c)]`` scored with
    ``local_compute_logprobs``).  KL: ``exp(r - p) - (r - p) - 1`` with r the reference and p
    the policy log-prob; the reference leaves this formula to its external trainer.  Outputs
    are fp32 ``[n_seq, seq_len]`` and zero outside the windows.
    """
    n_seq, seq_len, V = policy_logits.shape
    idx = _i64(ids).reshape(n_seq, seq_len)
    lengths = _i64(lengths).reshape(-1)
    starts_t = torch.zeros_like(lengths) if starts is None else _i64(starts).reshape(-1)
    lp_p = torch.zeros((n_seq, seq_len), dtype=torch.float32)
    lp_r = torch.zeros_like(lp_p)
    kl = torch.zeros_like(lp_p)
    for i in range(n_seq):
        st = int(max(0, min(int(starts_t[i]), seq_len)))
        ln = int(max(0, min(int(lengths[i]), seq_len - st)))
        if ln == 0:
            continue
        p, _, _ = selective_logprob(policy_logits[i, st:st + ln], idx[i, st:st + ln], temp)
        r, _, _ = selective_logprob(ref_logits[i, st:st + ln], idx[i, st:st + ln], temp)
        d = r - p
        lp_p[i, st:st + ln] = p
        lp_r[i, st:st + ln] = r
        kl[i, st:st + ln] = torch.exp(d) - d - 1.0
    return lp_p, lp_r, kl


def gather_paged_kv(block_tables, offsets, k_pool, v_pool, max_seq_len: int):
    """mlx-impl/paged_kv.py:57-116, thread body restated as loops: for s < offsets[b] the token
    comes from ``pool[block_tables[b, s // bs], h, s % bs, :]``, otherwise it is zero."""
    bt = _i64(block_tables)
    off = _i64(offsets)
    _, H, bs, D = k_pool.shape
    B = bt.shape[0]
    k_out = torch.zeros((B, H, max_seq_len, D), dtype=k_pool.dtype)
    v_out = torch.zeros_like(k_out)
    for b in range(B):
        for s in range(min(int(off[b]), max_seq_len)):
            phys = int(bt[b, s // bs])
            k_out[b, :, s, :] = k_pool[phys, :, s % bs, :]
            v_out[b, :, s, :] = v_pool[phys, :, s % bs, :]
    return k_out, v_out


def update_paged_kv(k_new, v_new, block_tables, offsets, k_pool, v_pool, block_size: int,
                    lengths=None):
    """mlx-impl/paged_kv.py:6-54 line by line (each piece of ``block_size`` tokens is written at
    the START of its physical block, pieces past the table are dropped); returns new pools."""
    bt = _i64(block_tables)
    off = _i64(offsets)
    B, H, S_new, D = k_new.shape
    ln = _i64(lengths) if lengths is not None else torch.full((B,), S_new, dtype=torch.int64)
    k_out, v_out = k_pool.clone(), v_pool.clone()
    for b in range(B):
        n_write = int(ln[b])
        for i in range((n_write + block_size - 1) // block_size):
            logical = (int(off[b]) + i * block_size) // block_size
            if logical >= bt.shape[1]:
                break
            phys = int(bt[b, logical])
            start, end = i * block_size, min((i + 1) * block_size, n_write)
            if end - start <= 0:
                continue
            piece_k = k_new[b, :, start:end, :]
            k_out[phys, :, : piece_k.shape[1], :] = piece_k
            v_out[phys, :, : piece_k.shape[1], :] = v_new[b, :, start:end, :]
    return k_out, v_out
