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
