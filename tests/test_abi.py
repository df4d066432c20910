"""CPU tests of the C-ABI boundary: the library loads without a GPU, exports every symbol
the header declares, and rejects bad arguments on the host before touching CUDA."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tome_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tome_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared_symbols()
    for must in ["tome_selective_logprob", "tome_log_softmax_full", "tome_dual_logprob_kl",
                 "tome_lmhead_logprob", "tome_lmhead_partials", "tome_combine_triples",
                 "tome_lmhead_workspace_bytes", "tome_version"]:
        assert must in names


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    for name in _declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_table_matches_header(built_lib):
    from tome_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared_symbols()
    assert _lib.lib.tome_version() == 100
    assert _lib.lib.tome_status_string(-3) == b"TOME_ERR_BAD_DTYPE"


def test_argument_errors_are_caught_on_the_host(built_lib):
    from tome_b200 import _lib
    lib = _lib.lib
    fake = ctypes.c_void_p(0x1000)  # never dereferenced: every call below fails its checks
    # unknown dtype
    assert lib.tome_selective_logprob(fake, 7, 4, 16, 16, fake, 1.0, fake, None, None, None, None) == -3
    # row stride smaller than the vocabulary
    assert lib.tome_selective_logprob(fake, 0, 4, 16, 8, fake, 1.0, fake, None, None, None, None) == -5
    # temperature must be positive and finite
    assert lib.tome_selective_logprob(fake, 0, 4, 16, 16, fake, 0.0, fake, None, None, None, None) == -7
    assert lib.tome_selective_logprob(fake, 0, 4, 16, 16, fake, float("nan"), fake, None, None, None, None) == -7
    # null logits with rows > 0
    assert lib.tome_selective_logprob(None, 0, 4, 16, 16, fake, 1.0, fake, None, None, None, None) == -1
    # zero rows is a no-op that succeeds without a device
    assert lib.tome_selective_logprob(None, 1, 0, 16, 16, None, 1.0, None, None, None, None, None) == 0
    # negative shape
    assert lib.tome_log_softmax_full(fake, 0, -1, 16, 16, 1.0, fake, 16, None, None, None) == -4
    # dual: too many sequences for one call
    assert lib.tome_dual_logprob_kl(fake, fake, 1, 5000, 4, 16, 16, fake, fake, None, 1.0, fake,
                                    fake, fake, None, None) == -9
    assert lib.tome_ragged_logprob(fake, 1, 5000, 4, 16, 16, fake, 8, fake, None, 1.0, fake, None,
                                   None, None, None) == -9
    assert lib.tome_sample_topk_logprob(fake, 1, 4, 16, 16, 0.7, 0, 1, 0, fake, fake, None, None,
                                        None, None) == -4
    # fused head: hidden size must keep rows 16-byte aligned
    assert lib.tome_lmhead_logprob(fake, fake, 4, 12, 64, fake, 1.0, 0, fake, None, fake, 1 << 20,
                                   None, None) == -8
    # fused head: workspace too small
    need = lib.tome_lmhead_workspace_bytes(256, 64, 1000)
    assert need > 0
    assert lib.tome_lmhead_logprob(fake, fake, 256, 64, 1000, fake, 1.0, 0, fake, None, fake,
                                   need - 1, None, None) == -6
    assert b"workspace" in lib.tome_last_error_string()
    assert lib.tome_rmsnorm_bf16(fake, fake, 4, 12, 1e-6, fake, None) == -8
    with pytest.raises(_lib.TomeArgumentError):
        _lib.check(-6)
    assert lib.tome_combine_triples(fake, fake, 2, 3, fake, 2, 1, 8, fake, None, None) == -5


def test_cpu_tensors_are_rejected_not_emulated(built_lib):
    import torch
    import tome_b200
    x = torch.zeros((2, 8))
    ids = torch.zeros(2, dtype=torch.int64)
    with pytest.raises(tome_b200.TomeRuntimeError):
        tome_b200.local_compute_logprobs(x, ids, 1.0)
    with pytest.raises(tome_b200.TomeRuntimeError):
        tome_b200.fused_log_softmax(x, 1.0)


def test_sampling_workspace_query_needs_no_gpu(built_lib, monkeypatch):
    from tome_b200 import _lib
    monkeypatch.delenv("TOME_K4_STREAM", raising=False)
    q = _lib.lib.tome_sample_workspace_bytes
    assert q(8, 151936) == 0 and q(4096, 100) == 0 and q(0, 151936) == 0
    per_row = 4 * 112 * 8          # four lists of 112 eight-byte entries per row
    assert q(4096, 151936) >= 4096 * per_row
    assert q(4096, 151936) < 4096 * (per_row + 64)
    assert q(200, 151936) > 0      # fp32 batches of this size take the streaming path
    monkeypatch.setenv("TOME_K4_STREAM", "0")
    assert q(4096, 151936) == 0
