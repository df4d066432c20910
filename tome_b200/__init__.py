"""tome_b200: LM-head logits -> per-token log-probabilities on B200 (sm_100a).

The functions keep the call signatures of the reference's hot path
(``fused_log_softmax`` in mlx-impl/model.py:77-89 and ``local_compute_logprobs`` in
mlx-impl/node.py:400-404), with torch CUDA tensors in place of ``mx.array``.
"""
from .ops import (  # noqa: F401
    check_device_status,
    combine_triples,
    fused_log_softmax,
    grpo_dual_logprob_kl,
    lm_head_logprob,
    lm_head_partials,
    lm_head_workspace_bytes,
    local_compute_logprobs,
    local_compute_logprobs_host,
    selective_log_softmax,
)
from .dist import lm_head_logprob_vocab_parallel, pack_triples  # noqa: F401
from ._lib import TomeArgumentError, TomeRuntimeError  # noqa: F401

__all__ = [
    "fused_log_softmax", "local_compute_logprobs", "selective_log_softmax",
    "local_compute_logprobs_host", "lm_head_logprob", "lm_head_partials",
    "lm_head_workspace_bytes", "combine_triples", "grpo_dual_logprob_kl",
    "lm_head_logprob_vocab_parallel", "pack_triples", "check_device_status",
    "TomeArgumentError", "TomeRuntimeError",
]
