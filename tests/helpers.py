"""Shared helpers of the test-suite."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Tolerances of the path (max-abs on log-probs): fp32 logits 1e-4, bf16 logits 2e-3.
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-3}


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name)))


def from_bits(arr: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    if dtype == torch.bfloat16:
        return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(arr.copy())


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.detach().cpu().to(torch.float64)
    b = b.detach().cpu().to(torch.float64)
    both_inf = torch.isinf(a) & torch.isinf(b) & (torch.sign(a) == torch.sign(b))
    d = torch.where(both_inf, torch.zeros_like(a), (a - b).abs())
    return float(d.max()) if d.numel() else 0.0


# ---------------------------------------------------------------- reference-kernel fixtures
# Cases of tests/golden/metal_kernel.npz: (dtype name, rows, vocab, temperature).  The inputs
# are not stored: they come from integer arithmetic that is exact in fp32 (and then rounded
# to bf16 for the bf16 cases), so every machine regenerates the same bits.
METAL_CASES = [(d, r, v, t)
               for d in ("float32", "bfloat16")
               for (r, v) in ((3, 7), (3, 4097), (2, 8192), (2, 151936))
               for t in (1.0, 0.7)]
METAL_STRIDE = 64  # rows longer than 8192 store every 64th output


def metal_case_inputs(dtype_name: str, rows: int, vocab: int, case_no: int):
    """(logits, targets) of a fixture case.  Logits are multiples of 6/32768 in [-6, 6); row 1
    has every fifth column masked with -inf; targets are never masked columns."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    j = np.arange(vocab, dtype=np.int64)[None, :]
    h = (j * 2654435761 + r * 40503 + case_no * 977) % 65536
    x = ((h - 32768).astype(np.float32) * np.float32(6.0 / 32768.0)).astype(np.float32)
    if rows > 1:
        x[1, ::5] = -np.inf
    t = ((np.arange(rows, dtype=np.int64) * 7919 + case_no * 31) % vocab)
    t = np.where(t % 5 == 0, (t + 1) % vocab, t)
    if vocab >= 5:
        t = np.where(t % 5 == 0, (t + 1) % vocab, t)
    logits = torch.from_numpy(x)
    if dtype_name == "bfloat16":
        logits = logits.to(torch.bfloat16)
    return logits, torch.from_numpy(t.astype(np.int32))


def metal_case_view(out: torch.Tensor, vocab: int) -> torch.Tensor:
    """The part of a case's output that the fixture stores."""
    return out if vocab <= 8192 else out[:, ::METAL_STRIDE]
