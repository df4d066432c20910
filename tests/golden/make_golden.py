"""Regenerates the fixtures in this directory from the CPU oracle (oracle/oracle.py).

    python tests/golden/make_golden.py

The reference has no golden vectors for this path and its MLX arithmetic cannot run here
(MLX is not installed; the Metal kernel is Apple-only), so the vectors are produced by the
oracle, which restates the reference's formulas.  bf16 tensors are stored as their uint16
bit patterns.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle  # noqa: E402
from tome_b200 import synthetic  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def selective(name, dtype, rows, vocab, temp, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((rows, vocab), generator=g) * 3.0)
    x[0, 5] = 12.0
    if rows > 2:
        x[2, : vocab // 2] = float("-inf")  # masked columns
    x = x.to(dtype)
    ids = torch.randint(0, vocab, (rows,), generator=g, dtype=torch.int32)
    ids[0] = 5
    ids[-1] = vocab - 1
    if rows > 2:
        ids[2] = vocab - 2
    lp, lse, raw = oracle.selective_logprob(x, ids, temp)
    full = oracle.log_softmax_metal_order(x, temp)
    np.savez_compressed(os.path.join(HERE, name), logits=bits(x), ids=ids.numpy(),
                        temp=np.float32(temp), logprob=lp.numpy(), lse=lse.numpy(),
                        raw=raw.numpy(), full=bits(full),
                        dtype=str(dtype).replace("torch.", ""))


def lm_head(name, rows, k, vocab, temp, seed):
    hidden, weight, ids = synthetic.cfg3_lm_head(rows, k, vocab, "cpu", seed)
    lp, lse = oracle.lm_head_logprob(hidden, weight, ids, temp)
    np.savez_compressed(os.path.join(HERE, name), hidden=bits(hidden), weight=bits(weight),
                        ids=ids.numpy(), temp=np.float32(temp), logprob=lp.numpy(),
                        lse=lse.numpy())


def dual(name, n_seq, seq_len, vocab, seed):
    pol, ref, ids, lengths, temp = synthetic.cfg5_dual(n_seq, seq_len, vocab, "cpu", seed,
                                                       min_len=0)
    lengths[0] = 0
    lengths[-1] = seq_len
    lp_p, lp_r, kl = oracle.dual_logprob_kl(pol, ref, ids, lengths, temp)
    np.savez_compressed(os.path.join(HERE, name), policy=bits(pol), ref=bits(ref),
                        ids=ids.numpy(), lengths=lengths.numpy(), temp=np.float32(temp),
                        lp_policy=lp_p.numpy(), lp_ref=lp_r.numpy(), kl=kl.numpy())


if __name__ == "__main__":
    selective("selective_bf16.npz", torch.bfloat16, 6, 4099, 0.7, 11)
    selective("selective_fp32.npz", torch.float32, 5, 2500, 1.0, 12)
    lm_head("lm_head.npz", 40, 72, 700, 0.9, 13)
    dual("dual_bf16.npz", 4, 6, 1032, 14)
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))
