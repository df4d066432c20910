"""tome_b200: LM-head logits -> per-token log-probabilities on B200 (sm_100a).

The functions keep the call signatures of the reference's hot path
(``fused_log_softmax`` in mlx-impl/model.py:77-89 and ``local_compute_logprobs`` in
mlx-impl/node.py:400-404), with torch CUDA tensors in place of ``mx.array``.

The CUDA library is loaded on first use of any of these names, so that
``python -m tome_b200.build`` can (re)build it even when the existing ``.so`` is stale.
"""
import importlib

_OPS = ["BoundCall", "bind_log_softmax", "bind_sample", "bind_selective", "check_device_status",
        "combine_triples", "fused_log_softmax", "gather_paged_kv", "grpo_dual_logprob_kl",
        "lm_head_logprob", "lm_head_logprob_static", "lm_head_partials",
        "lm_head_workspace_bytes", "local_compute_logprobs", "local_compute_logprobs_host",
        "ragged_logprobs", "rms_norm", "sample_topk_logprob", "sample_workspace_bytes",
        "selective_log_softmax", "update_paged_kv"]
_DIST = ["lm_head_logprob_vocab_parallel", "pack_triples", "exchange_triples"]
_LIB = ["TomeArgumentError", "TomeRuntimeError"]

__all__ = _OPS + _DIST + _LIB


def __getattr__(name):
    if name in _OPS:
        return getattr(importlib.import_module(".ops", __name__), name)
    if name in _DIST:
        return getattr(importlib.import_module(".dist", __name__), name)
    if name in _LIB:
        return getattr(importlib.import_module("._lib", __name__), name)
    if name in ("ops", "dist", "_lib", "synthetic", "build"):
        return importlib.import_module("." + name, __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
