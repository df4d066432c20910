"""Regenerates tests/golden/metal_kernel.npz from the REFERENCE's own kernel.

    python oracle/build_ref.py            # needs a reference checkout (see that file)
    python tests/golden/make_metal_golden.py

The reference's full-matrix log-softmax is a Metal kernel (mlx-impl/model.py:14-89).  Its
body is compiled for the CPU, unmodified, by oracle/build_ref.py around an emulation of the
Metal execution model (oracle/metal_emulation.cpp), and this script runs that library on the
fixture cases of tests/helpers.py.  The stored outputs are therefore outputs of the
reference's code, not of this repository's restatement; the tests hold both the restatement
(oracle/oracle.py) and the CUDA kernels against them.  Two things are not the reference's:
Apple's fast::exp / fast::log are libm's expf / logf here, and the simdgroup reductions add
in butterfly order.  bf16 tensors are stored as their uint16 bit patterns.
"""
import ctypes
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

from helpers import METAL_CASES, metal_case_inputs, metal_case_view  # noqa: E402


def load_reference_kernel():
    path = os.path.join(ROOT, "oracle", "_ref", "libmetal_ref.so")
    if not os.path.exists(path):
        raise SystemExit("oracle/_ref/libmetal_ref.so is missing: run python oracle/build_ref.py")
    return ctypes.CDLL(path)


def run_reference_kernel(lib, logits: torch.Tensor, temp: float) -> torch.Tensor:
    rows, vocab = logits.shape
    if logits.dtype == torch.float32:
        x = logits.contiguous().numpy().copy()
        out = np.empty_like(x)
        fn = lib.metal_fused_log_softmax_f32
    else:
        x = logits.contiguous().view(torch.int16).numpy().copy()
        out = np.empty_like(x)
        fn = lib.metal_fused_log_softmax_bf16
    rc = fn(x.ctypes.data_as(ctypes.c_void_p), ctypes.c_float(temp),
            out.ctypes.data_as(ctypes.c_void_p), rows, vocab)
    if rc != 0:
        raise RuntimeError("the emulated kernel did not finish")
    t = torch.from_numpy(out)
    return t if logits.dtype == torch.float32 else t.view(torch.bfloat16)


def main():  # noqa: D103
    lib = load_reference_kernel()
    arrays = {}
    for n, (dtype_name, rows, vocab, temp) in enumerate(METAL_CASES):
        logits, targets = metal_case_inputs(dtype_name, rows, vocab, n)
        out = run_reference_kernel(lib, logits, temp)
        kept = metal_case_view(out, vocab).contiguous()
        at_target = out[torch.arange(rows), targets.long()].contiguous()
        if dtype_name == "bfloat16":
            kept = kept.view(torch.int16).numpy().view(np.uint16)
            at_target = at_target.view(torch.int16).numpy().view(np.uint16)
        else:
            kept, at_target = kept.numpy(), at_target.numpy()
        arrays[f"out_{n}"] = kept
        arrays[f"at_target_{n}"] = at_target
    arrays.update(paged_gather_case(lib))
    np.savez_compressed(os.path.join(HERE, "metal_kernel.npz"), **arrays)
    print(f"wrote {len(METAL_CASES)} log-softmax cases and the paged-KV gather case")


def paged_gather_case(lib):
    """mlx-impl/paged_kv.py:57-116 run on a small pool: sequences of length 0, mid-block, a
    whole number of blocks and the full table; inputs are stored with the outputs."""
    g = torch.Generator().manual_seed(20260)
    B, H, D, bs, max_blocks, max_seq_len, num_blocks = 4, 2, 8, 4, 5, 20, 11
    k_pool = torch.randint(0, 65536, (num_blocks, H, bs, D), generator=g, dtype=torch.int32)
    v_pool = torch.randint(0, 65536, (num_blocks, H, bs, D), generator=g, dtype=torch.int32)
    k_pool, v_pool = k_pool.numpy().astype(np.uint16), v_pool.numpy().astype(np.uint16)
    tables = torch.randint(0, num_blocks, (B, max_blocks), generator=g, dtype=torch.int32).numpy()
    offsets = np.array([0, 7, 12, 20], dtype=np.int32)
    k_out = np.full((B, H, max_seq_len, D), 0xFFFF, dtype=np.uint16)
    v_out = np.full_like(k_out, 0xFFFF)

    def ptr(a):
        return a.ctypes.data_as(ctypes.c_void_p)

    rc = lib.metal_gather_paged_kv(ptr(tables), ptr(offsets), ptr(k_pool), ptr(v_pool), ptr(k_out),
                                   ptr(v_out), 2, B, H, D, bs, max_blocks, max_seq_len)
    if rc != 0:
        raise RuntimeError("the emulated gather kernel failed")
    return {"gather_k_pool": k_pool, "gather_v_pool": v_pool, "gather_tables": tables,
            "gather_offsets": offsets, "gather_k_out": k_out, "gather_v_out": v_out,
            "gather_max_seq_len": np.int32(max_seq_len)}


if __name__ == "__main__":
    main()
