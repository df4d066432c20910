"""The oracle's restatement against outputs of the REFERENCE's own Metal kernel.

tests/golden/metal_kernel.npz holds what the reference's kernel body (mlx-impl/model.py:14-66)
computes for the fixture cases when it is compiled, unmodified, for the CPU around an
emulation of the Metal execution model (oracle/metal_emulation.cpp, oracle/build_ref.py,
tests/golden/make_metal_golden.py).  These tests pin oracle/oracle.py to those outputs; the
GPU tests hold the CUDA kernels against the same file."""
import ctypes
import os

import numpy as np
import pytest
import torch

from helpers import (METAL_CASES, from_bits, load_golden, max_abs, metal_case_inputs,
                     metal_case_view)
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libmetal_ref.so")
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def golden():
    return load_golden("metal_kernel.npz")


@pytest.mark.parametrize("case_no", range(len(METAL_CASES)))
def test_full_matrix_restatement_matches_the_reference_kernel(golden, case_no):
    dtype_name, rows, vocab, temp = METAL_CASES[case_no]
    dtype = DTYPES[dtype_name]
    logits, _ = metal_case_inputs(dtype_name, rows, vocab, case_no)
    want = from_bits(golden[f"out_{case_no}"], dtype)
    got = metal_case_view(oracle.log_softmax_metal_order(logits, temp), vocab)
    assert got.shape == want.shape
    if dtype == torch.float32:
        # different summation order only: a few ulp of values near -12
        assert max_abs(got, want) <= 4e-6
    else:
        assert max_abs(got.float(), want.float()) <= 0.0625 + 1e-6      # one bf16 ulp near -12
        assert float((got == want).float().mean()) >= 0.999


@pytest.mark.parametrize("case_no", [n for n, c in enumerate(METAL_CASES) if c[0] == "float32"])
def test_selective_restatement_matches_the_policy_call_site(golden, case_no):
    """mlx-impl/node.py:590,605: fused_log_softmax(logits.astype(f32), T)[b, token] is the
    kernel's output at the token.  The selective formula (node.py:400-404) divides by T where
    the kernel multiplies by 1/T: a rounding of difference."""
    _, rows, vocab, temp = METAL_CASES[case_no]
    logits, targets = metal_case_inputs("float32", rows, vocab, case_no)
    want = torch.from_numpy(golden[f"at_target_{case_no}"].copy())
    got, _, _ = oracle.selective_logprob(logits, targets, temp)
    assert max_abs(got, want) <= 1e-5


@pytest.mark.skipif(not os.path.exists(REF_LIB),
                    reason="oracle/_ref/libmetal_ref.so not built (needs a reference checkout)")
def test_the_built_reference_kernel_reproduces_the_fixture(golden):
    lib = ctypes.CDLL(REF_LIB)
    for case_no, (dtype_name, rows, vocab, temp) in enumerate(METAL_CASES):
        if vocab > 8192 and case_no % 2:
            continue  # keep the CPU suite short: the long rows at one temperature
        logits, _ = metal_case_inputs(dtype_name, rows, vocab, case_no)
        if dtype_name == "float32":
            x = logits.numpy().copy()
            fn = lib.metal_fused_log_softmax_f32
        else:
            x = logits.view(torch.int16).numpy().copy()
            fn = lib.metal_fused_log_softmax_bf16
        out = np.empty_like(x)
        assert fn(x.ctypes.data_as(ctypes.c_void_p), ctypes.c_float(temp),
                  out.ctypes.data_as(ctypes.c_void_p), rows, vocab) == 0
        t = torch.from_numpy(out)
        t = t if dtype_name == "float32" else t.view(torch.bfloat16)
        want = from_bits(golden[f"out_{case_no}"], DTYPES[dtype_name])
        kept = metal_case_view(t, vocab)
        same = (kept == want) | (torch.isnan(kept.float()) & torch.isnan(want.float()))
        assert bool(same.all())


def test_paged_gather_restatement_matches_the_reference_kernel(golden):
    """mlx-impl/paged_kv.py:57-116 compiled for the CPU (same recipe) against the oracle's loop."""
    as_bf16 = lambda a: from_bits(a, torch.bfloat16)  # noqa: E731
    k_out, v_out = oracle.gather_paged_kv(
        torch.from_numpy(golden["gather_tables"].copy()), torch.from_numpy(golden["gather_offsets"].copy()),
        as_bf16(golden["gather_k_pool"]), as_bf16(golden["gather_v_pool"]),
        int(golden["gather_max_seq_len"]))
    assert torch.equal(k_out.view(torch.int16), as_bf16(golden["gather_k_out"]).view(torch.int16))
    assert torch.equal(v_out.view(torch.int16), as_bf16(golden["gather_v_out"]).view(torch.int16))
