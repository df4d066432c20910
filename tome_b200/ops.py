"""Host-side mirror of the reference's log-prob interface, over the C ABI.

Every function takes torch CUDA tensors, passes raw device pointers to ``libtome_b200.so``
and launches on torch's current stream.  torch is used for memory and streams only; the
arithmetic happens in the library's kernels and nowhere else (CPU tensors are rejected).

Reference call sites mirrored here
  * ``fused_log_softmax(logits, temperature=1.0)``      mlx-impl/model.py:77-89
  * ``local_compute_logprobs(logits, ids, temp)``        mlx-impl/node.py:400-404
  * ``x @ embed_tokens.weight.T`` then the above         mlx-impl/model.py:538
  * ``temperature or 1.0`` (greedy decoding scores at temperature 1)
                                                         mlx-impl/node.py:331,356,451,558,590
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import TOME_BF16, TOME_F32, TomeRuntimeError, check, lib

_DTYPES = {torch.float32: TOME_F32, torch.bfloat16: TOME_BF16}
# sequences tome_dual_logprob_kl / tome_ragged_logprob take per call (the wrappers slice larger batches)
MAX_SEQ_PER_CALL = 1024
_status_words: dict = {}


def _status_word(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    word = _status_words.get(key)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = word
    return word


def check_device_status(device=None) -> None:
    """Read (and clear) the device status word; raise if a kernel reported a problem.

    Kernels never trap.  A target index outside the vocabulary or a bounded wait that ran
    out is recorded in a device word instead, which this call inspects.  It synchronises
    with the device, so the hot calls do not do it on their own unless ``check=True``.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _status_word(device)
    bits = int(word.item())
    if bits == 0:
        return
    word.zero_()
    problems = []
    if bits & _lib.DEV_TARGET_OUT_OF_RANGE:
        problems.append("a target index lies outside [0, vocab)")
    if bits & _lib.DEV_RAGGED_OVERFLOW:
        problems.append("the ragged windows cover more positions than the packed arrays hold")
    if bits & _lib.DEV_BLOCK_OUT_OF_RANGE:
        problems.append("a paged-KV block-table entry lies outside the pool")
    if bits & _lib.DEV_NO_CANDIDATE:
        problems.append("sampling met a row without a single logit that is not NaN")
    if bits & _lib.DEV_TIMEOUT:
        problems.append("a bounded device-side wait ran out (TOME_DEV_TIMEOUT)")
    raise TomeRuntimeError("; ".join(problems) or f"device status {bits}")


def _require_cuda(name: str, t: torch.Tensor) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise TomeRuntimeError(
            f"{name} lives on {t.device}: tome_b200 runs on CUDA devices only (no CPU fallback)")


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"logits must be float32 or bfloat16, got {t.dtype}") from None


def _rows_view(logits: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """[..., V] -> 2-D [rows, V] whose last dim is contiguous; returns (view, row stride)."""
    if logits.dim() == 0:
        raise ValueError("logits needs at least one dimension")
    V = logits.shape[-1]
    if logits.dim() == 2 and logits.stride(1) == 1 and logits.stride(0) >= V:
        return logits, logits.stride(0)
    flat = logits.reshape(-1, V)
    if flat.numel() and (flat.stride(1) != 1 or flat.stride(0) < V):
        flat = flat.contiguous()
    return flat, (flat.stride(0) if flat.shape[0] > 1 else max(V, 1))


def _ids32(ids: torch.Tensor, n: int, device: torch.device) -> torch.Tensor:
    if not isinstance(ids, torch.Tensor):
        ids = torch.as_tensor(ids)
    if ids.is_floating_point():
        raise TypeError("token ids must be an integer tensor")
    ids = ids.reshape(-1)
    if ids.numel() != n:
        raise ValueError(f"expected {n} token ids, got {ids.numel()}")
    if ids.device != device:
        ids = ids.to(device, non_blocking=True)
    if ids.dtype != torch.int32:
        ids = ids.to(torch.int32)
    return ids.contiguous()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(device: torch.device) -> int:
    """Handle of torch's current stream on ``device`` (the fast accessor when torch has it)."""
    if _raw_stream is not None:
        index = device.index if device.index is not None else torch.cuda.current_device()
        return _raw_stream(index)
    return torch.cuda.current_stream(device).cuda_stream


class _NoSwitch:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def _on(device: torch.device):
    """Context in which ``device`` is the current CUDA device; free when it already is (the
    library launches on the current device, and switching costs several microseconds)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _out_rows(name: str, t: Optional[torch.Tensor], rows: int, device: torch.device,
              dtype: torch.dtype = torch.float32) -> None:
    if t is None:
        return
    if not isinstance(t, torch.Tensor) or t.dtype != dtype or t.device != device or \
            t.numel() != rows or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous {dtype} tensor of {rows} elements on {device}")


def selective_log_softmax(logits: torch.Tensor, ids: torch.Tensor, temp: float = 1.0, *,
                          return_lse: bool = False, return_target_logit: bool = False,
                          check: bool = False, out: Optional[torch.Tensor] = None,
                          out_lse: Optional[torch.Tensor] = None):
    """Log-probability of ``ids[i]`` under ``softmax(logits[i] / temp)``, fp32, one pass.

    Same arithmetic as ``local_compute_logprobs`` (mlx-impl/node.py:400-404): logits are
    up-cast to fp32, divided by ``temp``, reduced with a max-shifted logsumexp, and the target
    column is gathered.  ``logits`` is ``[..., V]`` in bf16 or fp32, ``ids`` has the leading
    shape.  ``temp`` of 0 or None means 1.0, as at the reference call sites.  ``out`` (and
    ``out_lse``, which implies ``return_lse``) name contiguous fp32 tensors with one element
    per row to write into instead of fresh allocations; a decode loop that passes them and
    int32 ids on the device pays for nothing but the launch.
    """
    if not isinstance(logits, torch.Tensor) or not logits.is_cuda:
        _require_cuda("logits", logits)
    temp = float(temp or 1.0)
    device = logits.device
    if logits.dim() == 2 and logits.stride(1) == 1 and logits.stride(0) >= logits.shape[1]:
        flat, stride = logits, logits.stride(0)
    else:
        flat, stride = _rows_view(logits)
    rows, V = flat.shape
    if isinstance(ids, torch.Tensor) and ids.dtype == torch.int32 and ids.device == device \
            and ids.numel() == rows and ids.is_contiguous():
        ids32 = ids
    else:
        ids32 = _ids32(ids, rows, device)
    if out is None:
        out = torch.empty(rows, dtype=torch.float32, device=device)
    else:
        _out_rows("out", out, rows, device)
    if out_lse is not None:
        _out_rows("out_lse", out_lse, rows, device)
        lse, return_lse = out_lse, True
    else:
        lse = torch.empty(rows, dtype=torch.float32, device=device) if return_lse else None
    raw = torch.empty(rows, dtype=torch.float32, device=device) if return_target_logit else None
    with _on(device):
        status = lib.tome_selective_logprob(
            flat.data_ptr(), _DTYPES.get(flat.dtype, -1), rows, V, stride, ids32.data_ptr(), temp,
            out.data_ptr(), _ptr(lse), _ptr(raw), _status_word(device).data_ptr(), _stream(device))
    if status:
        if flat.dtype not in _DTYPES:
            _dtype_code(flat)
        _lib.check(status)
    if check:
        check_device_status(device)
    lead = logits.shape[:-1]
    if len(lead) != 1:
        out = out.reshape(lead)
        lse = None if lse is None else lse.reshape(lead)
        raw = None if raw is None else raw.reshape(lead)
    if not (return_lse or return_target_logit):
        return out
    result = [out]
    if return_lse:
        result.append(lse)
    if return_target_logit:
        result.append(raw)
    return tuple(result)


def local_compute_logprobs(logits: torch.Tensor, ids: torch.Tensor, temp: float, *,
                           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Drop-in for the closure of the same name in mlx-impl/node.py:400-404 (``out``: see
    :func:`selective_log_softmax`)."""
    return selective_log_softmax(logits, ids, temp, out=out)


def local_compute_logprobs_host(logits_host: torch.Tensor, ids_host: torch.Tensor, temp: float,
                                device=None, staging: Optional[dict] = None) -> torch.Tensor:
    """Host-buffer form of :func:`local_compute_logprobs`: host logits in, host fp32 out.

    Copies the (ideally pinned) host logits and ids to the device, runs the kernel and
    copies the log-probs back; this is the call an integration makes when the logits live
    in host memory.  ``staging`` may hold reusable device/pinned buffers between calls.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    staging = {} if staging is None else staging
    key = (tuple(logits_host.shape), logits_host.dtype)
    if staging.get("key") != key:
        staging["key"] = key
        staging["logits"] = torch.empty(logits_host.shape, dtype=logits_host.dtype, device=device)
        staging["ids"] = torch.empty(ids_host.shape, dtype=torch.int32, device=device)
        staging["out"] = torch.empty(ids_host.shape, dtype=torch.float32).pin_memory()
    staging["logits"].copy_(logits_host, non_blocking=True)
    staging["ids"].copy_(ids_host.to(torch.int32), non_blocking=True)
    lp = selective_log_softmax(staging["logits"], staging["ids"], temp)
    staging["out"].copy_(lp, non_blocking=True)
    torch.cuda.current_stream(device).synchronize()
    return staging["out"]


def fused_log_softmax(logits: torch.Tensor, temperature: float = 1.0, *,
                      targets: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                      check: bool = False) -> torch.Tensor:
    """Drop-in for ``fused_log_softmax`` of mlx-impl/model.py:77-89.

    Without ``targets`` it returns the full ``[..., V]`` log-softmax in the dtype of
    ``logits`` with the Metal kernel's order of operations (scale by ``1/temperature``, round
    to the dtype, subtract the rounded logsumexp).  With ``targets`` it returns only the fp32
    log-probs of those columns, which turns the call sites' ``lp[b, token]`` pattern
    (mlx-impl/node.py:590-605) into one call that never writes the matrix.  ``out`` (same shape
    and dtype as ``logits``, contiguous) receives the matrix instead of a fresh allocation.
    """
    if targets is not None:
        return selective_log_softmax(logits, targets, temperature, check=check)
    if not isinstance(logits, torch.Tensor) or not logits.is_cuda:
        _require_cuda("logits", logits)
    temperature = float(temperature or 1.0)
    device = logits.device
    if logits.dim() == 2 and logits.stride(1) == 1 and logits.stride(0) >= logits.shape[1]:
        flat, stride = logits, logits.stride(0)
    else:
        flat, stride = _rows_view(logits)
    rows, V = flat.shape
    if out is None:
        out = torch.empty((rows, V), dtype=flat.dtype, device=device)
    elif (out.shape != logits.shape or out.dtype != flat.dtype or out.device != device
          or not out.is_contiguous()):
        raise ValueError("out must be a contiguous tensor with the shape, dtype and device of logits")
    with _on(device):
        status = lib.tome_log_softmax_full(
            flat.data_ptr(), _DTYPES.get(flat.dtype, -1), rows, V, stride, temperature,
            out.data_ptr(), V, None, _status_word(device).data_ptr(), _stream(device))
    if status:
        if flat.dtype not in _DTYPES:
            _dtype_code(flat)
        _lib.check(status)
    if check:
        check_device_status(device)
    return out if out.shape == logits.shape else out.reshape(logits.shape)


def grpo_dual_logprob_kl(policy_logits: torch.Tensor, ref_logits: torch.Tensor,
                         ids: torch.Tensor, lengths: torch.Tensor, temp: float = 1.0, *,
                         starts: Optional[torch.Tensor] = None, check: bool = False):
    """Policy and reference log-probs of a ragged window per sequence, plus the k3 KL.

    ``policy_logits`` and ``ref_logits`` are ``[n_seq, seq_len, V]``; ``ids`` is
    ``[n_seq, seq_len]``; ``lengths`` (and optional ``starts``) give the scored window
    ``[start, start + length)`` of each sequence, the completion slice of
    mlx-impl/node.py:446-451.  Returns ``(lp_policy, lp_ref, kl)``, fp32 ``[n_seq, seq_len]``,
    zero outside the windows, with ``kl = exp(r - p) - (r - p) - 1``.  Rows outside the
    windows are never read.  Any number of sequences (the library takes 1024 per call; larger
    batches go in slices).
    """
    _require_cuda("policy_logits", policy_logits)
    _require_cuda("ref_logits", ref_logits)
    if policy_logits.shape != ref_logits.shape or policy_logits.dtype != ref_logits.dtype:
        raise ValueError("policy_logits and ref_logits must agree in shape and dtype")
    if policy_logits.dim() != 3:
        raise ValueError("expected logits of shape [n_seq, seq_len, V]")
    temp = float(temp or 1.0)
    n_seq, seq_len, V = policy_logits.shape
    device = policy_logits.device
    pol = policy_logits if policy_logits.is_contiguous() else policy_logits.contiguous()
    ref = ref_logits if ref_logits.is_contiguous() else ref_logits.contiguous()
    ids32 = _ids32(ids, n_seq * seq_len, device)
    len32 = _ids32(lengths, n_seq, device)
    st32 = None if starts is None else _ids32(starts, n_seq, device)
    outs = [torch.empty((n_seq, seq_len), dtype=torch.float32, device=device) for _ in range(3)]
    ids2 = ids32.view(n_seq, seq_len)
    with _on(device):
        # the library takes MAX_SEQ_PER_CALL sequences per call: larger batches go in slices
        for i0 in range(0, max(n_seq, 1), MAX_SEQ_PER_CALL):
            n = min(MAX_SEQ_PER_CALL, n_seq - i0)
            status = lib.tome_dual_logprob_kl(
                pol[i0:].data_ptr(), ref[i0:].data_ptr(), _dtype_code(pol), n, seq_len, V, V,
                ids2[i0:].data_ptr(), len32[i0:].data_ptr(),
                None if st32 is None else st32[i0:].data_ptr(), temp, outs[0][i0:].data_ptr(),
                outs[1][i0:].data_ptr(), outs[2][i0:].data_ptr(), _status_word(device).data_ptr(),
                _stream(device))
            _lib.check(status)
    if check:
        check_device_status(device)
    return tuple(outs)


def ragged_logprobs(logits: torch.Tensor, targets_packed: torch.Tensor, lengths: torch.Tensor,
                    temp: float = 1.0, *, starts: Optional[torch.Tensor] = None,
                    return_lse: bool = False, check: bool = False):
    """Log-probs of the completion tokens of every sequence of one model, packed back to back.

    The batched form of the loop in ``_process_ref_logprobs_batched`` (mlx-impl/node.py:446-458):
    for sequence ``i`` the rows ``[starts[i], starts[i] + lengths[i])`` of ``logits[i]`` are
    scored against ``lengths[i]`` consecutive entries of ``targets_packed`` (the completion
    tokens), and the fp32 results are written sequence after sequence, the layout of
    ``Completion.ref_log_probs`` on the wire (scheduler/proto/inference.proto:108-112).
    ``logits`` is ``[n_seq, seq_len, V]``.  Returns ``(packed, offsets)`` (plus the packed
    logsumexp with ``return_lse``); ``packed[offsets[i]:offsets[i+1]]`` belongs to sequence
    ``i``.  Rows outside the windows are never read.  Any number of sequences; beyond the 1024
    the library takes per call the batch goes in slices, which costs one synchronising read of
    the slices' starting offsets.
    """
    _require_cuda("logits", logits)
    if logits.dim() != 3:
        raise ValueError("expected logits of shape [n_seq, seq_len, V]")
    temp = float(temp or 1.0)
    n_seq, seq_len, V = logits.shape
    device = logits.device
    lg = logits if logits.is_contiguous() else logits.contiguous()
    tg = _ids32(targets_packed, int(targets_packed.numel()), device)
    len32 = _ids32(lengths, n_seq, device)
    st32 = None if starts is None else _ids32(starts, n_seq, device)
    total = int(tg.numel())
    out = torch.empty(total, dtype=torch.float32, device=device)
    lse = torch.empty(total, dtype=torch.float32, device=device) if return_lse else None
    offsets = torch.empty(n_seq + 1, dtype=torch.int32, device=device)
    if n_seq <= MAX_SEQ_PER_CALL:
        with _on(device):
            status = lib.tome_ragged_logprob(
                lg.data_ptr(), _dtype_code(lg), n_seq, seq_len, V, V, tg.data_ptr(), total,
                len32.data_ptr(), _ptr(st32), temp, out.data_ptr(), _ptr(lse), offsets.data_ptr(),
                _status_word(device).data_ptr(), _stream(device))
        _lib.check(status)
    else:
        # more sequences than one call takes: slices of MAX_SEQ_PER_CALL, each writing behind
        # the one before.  Where a slice begins in the packed arrays is needed on the host
        # (one synchronising read of a few integers); the windows are clamped as the kernel
        # clamps them.
        begin = torch.zeros_like(len32) if st32 is None else st32.clamp(0, seq_len)
        window = torch.minimum(len32.clamp(min=0), seq_len - begin)
        firsts = list(range(0, n_seq, MAX_SEQ_PER_CALL))
        ends = torch.cumsum(window, 0, dtype=torch.int64)
        bases = [0] + ends[[f - 1 for f in firsts[1:]]].tolist()
        with _on(device):
            for i0, base in zip(firsts, bases):
                n = min(MAX_SEQ_PER_CALL, n_seq - i0)
                base = min(int(base), total)
                status = lib.tome_ragged_logprob(
                    lg[i0:].data_ptr(), _dtype_code(lg), n, seq_len, V, V,
                    tg.data_ptr() + 4 * base, total - base, len32[i0:].data_ptr(),
                    None if st32 is None else st32[i0:].data_ptr(), temp,
                    out.data_ptr() + 4 * base, None if lse is None else lse.data_ptr() + 4 * base,
                    offsets[i0:].data_ptr(), _status_word(device).data_ptr(), _stream(device))
                _lib.check(status)
                offsets[i0:i0 + n + 1] += base
    if check:
        check_device_status(device)  # raises if the windows needed more than `total` entries
        if int(offsets[-1].item()) != total:
            raise ValueError(f"targets_packed holds {total} ids but the windows cover "
                             f"{int(offsets[-1].item())} positions")
    return (out, offsets, lse) if return_lse else (out, offsets)


_sample_ws_bytes: dict = {}


def sample_workspace_bytes(rows: int, vocab: int) -> int:
    """Scratch bytes :func:`sample_topk_logprob` uses for a batch of this shape (0 for the
    batches that need none)."""
    key = (rows, vocab, os.environ.get("TOME_K4_STREAM"), os.environ.get("TOME_K4_PARTS"))
    n = _sample_ws_bytes.get(key)
    if n is None:
        n = _sample_ws_bytes[key] = int(lib.tome_sample_workspace_bytes(rows, vocab))
    return n


def sample_topk_logprob(logits: torch.Tensor, temperature: float, top_k: int = 20, *,
                        seed: int = 0, offset: int = 0, return_topk: bool = False,
                        check: bool = False, out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                        workspace: Optional[torch.Tensor] = None):
    """Sample one token per row and score it, on the device, in one pass over the logits.

    The batched replacement of the rollout's per-sequence loop (mlx-impl/node.py:593-610):
    ``_sample_token`` (node.py:894-907, top-k temperature sampling) plus the gather of the
    sampled token's log-prob from ``fused_log_softmax`` (node.py:590, 605).  ``temperature``
    0 means greedy (argmax) scored at temperature 1, as in the reference.  Returns
    ``(tokens int32 [...], logprobs fp32 [...])`` and, with ``return_topk``, the top-k indices
    and raw logits.  Draws depend only on ``(seed, offset, row)``; advance ``offset`` per step.
    ``out`` may name the ``(tokens, logprobs)`` tensors to write into (contiguous, one element
    per row) and ``workspace`` a scratch tensor of :func:`sample_workspace_bytes` bytes, which a
    decode loop reuses from step to step.  A row without a single logit that is not NaN gets
    token -1 and log-prob NaN.  ``check=True`` synchronises and raises if the kernels reported
    a device status.
    """
    if not isinstance(logits, torch.Tensor) or not logits.is_cuda:
        _require_cuda("logits", logits)
    device = logits.device
    if logits.dim() == 2 and logits.stride(1) == 1 and logits.stride(0) >= logits.shape[1]:
        flat, stride = logits, logits.stride(0)
    else:
        flat, stride = _rows_view(logits)
    rows, V = flat.shape
    if out is None:
        tokens = torch.empty(rows, dtype=torch.int32, device=device)
        lp = torch.empty(rows, dtype=torch.float32, device=device)
    else:
        tokens, lp = out
        _out_rows("out[0] (tokens)", tokens, rows, device, torch.int32)
        _out_rows("out[1] (logprobs)", lp, rows, device)
    tk_i = torch.empty((rows, top_k), dtype=torch.int32, device=device) if return_topk else None
    tk_v = torch.empty((rows, top_k), dtype=torch.float32, device=device) if return_topk else None
    # large batches take a streaming path that needs scratch (0: not a batch of this shape)
    nbytes = sample_workspace_bytes(rows, V)
    ws = None
    if nbytes:
        ws = _workspace(nbytes, device, workspace)
        nbytes = ws.numel() * ws.element_size()
    with _on(device):
        status = lib.tome_sample_topk_logprob_ws(
            flat.data_ptr(), _DTYPES.get(flat.dtype, -1), rows, V, stride, float(temperature or 0.0),
            int(top_k), int(seed) & (2 ** 64 - 1), int(offset) & (2 ** 64 - 1), tokens.data_ptr(),
            lp.data_ptr(), _ptr(tk_i), _ptr(tk_v), _ptr(ws), nbytes,
            _status_word(device).data_ptr(), _stream(device))
    if status:
        if flat.dtype not in _DTYPES:
            _dtype_code(flat)
        _lib.check(status)
    if check:
        check_device_status(device)
    lead = logits.shape[:-1]
    if len(lead) != 1:
        tokens, lp = tokens.reshape(lead), lp.reshape(lead)
    if return_topk:
        return tokens, lp, tk_i.reshape(*lead, top_k), tk_v.reshape(*lead, top_k)
    return tokens, lp


class BoundCall:
    """One library call with everything but the stream resolved ahead of time.

    The rollout makes the same call at every decode step (mlx-impl/node.py:590-605: same
    shapes, same buffers); binding it once keeps the per-step host work down to fetching
    torch's current stream and one foreign call.  ``outputs`` holds the tensors the call writes.
    The bound tensors must keep their storage (write new logits INTO them); the object keeps
    them alive.  Calls go to the stream that is current when they are made.
    """
    __slots__ = ("_fn", "_head", "_tail", "_device", "_index", "outputs", "_keep")

    def __init__(self, fn, head, tail, device, outputs, keep):
        self._fn, self._head, self._tail = fn, tuple(head), tuple(tail)
        self._device = device
        self._index = device.index if device.index is not None else torch.cuda.current_device()
        self.outputs, self._keep = outputs, keep

    def __call__(self, *step_args):
        """Launch.  ``step_args`` are the per-step values of the call (sampling: the offset)."""
        if self._index != torch.cuda.current_device():
            with torch.cuda.device(self._index):
                status = self._fn(*self._head, *step_args, *self._tail, _stream(self._device))
        else:
            status = self._fn(*self._head, *step_args, *self._tail, _stream(self._device))
        if status:
            _lib.check(status)
        return self.outputs


def _bind_rows(logits: torch.Tensor):
    _require_cuda("logits", logits)
    if logits.dim() != 2 or logits.stride(1) != 1 or logits.stride(0) < logits.shape[1]:
        raise ValueError("a bound call needs 2-D logits [rows, V] with contiguous rows")
    return logits.shape[0], logits.shape[1], logits.stride(0), _dtype_code(logits)


def bind_selective(logits: torch.Tensor, ids: torch.Tensor, temp: float = 1.0, *,
                   out: Optional[torch.Tensor] = None,
                   out_lse: Optional[torch.Tensor] = None) -> BoundCall:
    """:func:`local_compute_logprobs` as a :class:`BoundCall`: ``call()`` scores the current
    contents of ``logits`` against the current contents of ``ids`` (int32, on the device) and
    returns ``outputs = (logprobs,)`` or ``(logprobs, lse)``."""
    rows, V, stride, code = _bind_rows(logits)
    device = logits.device
    _out_rows("ids", ids, rows, device, torch.int32)
    if out is None:
        out = torch.empty(rows, dtype=torch.float32, device=device)
    _out_rows("out", out, rows, device)
    _out_rows("out_lse", out_lse, rows, device)
    head = (logits.data_ptr(), code, rows, V, stride, ids.data_ptr(), float(temp or 1.0),
            out.data_ptr(), _ptr(out_lse), None, _status_word(device).data_ptr())
    outputs = (out,) if out_lse is None else (out, out_lse)
    return BoundCall(lib.tome_selective_logprob, head, (), device, outputs, (logits, ids))


def bind_log_softmax(logits: torch.Tensor, temperature: float = 1.0, *,
                     out: Optional[torch.Tensor] = None) -> BoundCall:
    """:func:`fused_log_softmax` (the full matrix) as a :class:`BoundCall`; ``outputs = (out,)``."""
    rows, V, stride, code = _bind_rows(logits)
    device = logits.device
    if out is None:
        out = torch.empty((rows, V), dtype=logits.dtype, device=device)
    elif out.shape != logits.shape or out.dtype != logits.dtype or out.device != device or \
            not out.is_contiguous():
        raise ValueError("out must be a contiguous tensor with the shape, dtype and device of logits")
    head = (logits.data_ptr(), code, rows, V, stride, float(temperature or 1.0), out.data_ptr(), V,
            None, _status_word(device).data_ptr())
    return BoundCall(lib.tome_log_softmax_full, head, (), device, (out,), (logits,))


def bind_sample(logits: torch.Tensor, temperature: float, top_k: int = 20, *, seed: int = 0,
                out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                workspace: Optional[torch.Tensor] = None) -> BoundCall:
    """:func:`sample_topk_logprob` as a :class:`BoundCall`: ``call(offset)`` draws one token per
    row from the current contents of ``logits``; ``outputs = (tokens, logprobs)``.  The scratch
    of large batches is allocated here once (or taken from ``workspace``) and reused by every
    call, so calls of one bound object must not overlap on the device."""
    rows, V, stride, code = _bind_rows(logits)
    device = logits.device
    if out is None:
        out = (torch.empty(rows, dtype=torch.int32, device=device),
               torch.empty(rows, dtype=torch.float32, device=device))
    tokens, lp = out
    _out_rows("out[0] (tokens)", tokens, rows, device, torch.int32)
    _out_rows("out[1] (logprobs)", lp, rows, device)
    nbytes = sample_workspace_bytes(rows, V)
    ws = _workspace(nbytes, device, workspace) if nbytes else None
    head = (logits.data_ptr(), code, rows, V, stride, float(temperature or 0.0), int(top_k),
            int(seed) & (2 ** 64 - 1))
    tail = (tokens.data_ptr(), lp.data_ptr(), None, None, _ptr(ws),
            0 if ws is None else ws.numel() * ws.element_size(), _status_word(device).data_ptr())
    return BoundCall(lib.tome_sample_topk_logprob_ws, head, tail, device, (tokens, lp), (logits, ws))


def lm_head_workspace_bytes(rows: int, hidden_dim: int, vocab_local: int) -> int:
    """Scratch bytes the fused LM-head kernels need for these sizes."""
    return int(lib.tome_lmhead_workspace_bytes(rows, hidden_dim, vocab_local))


def _lm_head_inputs(hidden: torch.Tensor, weight: torch.Tensor):
    _require_cuda("hidden", hidden)
    _require_cuda("weight", weight)
    if hidden.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("hidden and weight must be bfloat16")
    if weight.dim() != 2 or hidden.shape[-1] != weight.shape[1]:
        raise ValueError(f"hidden [..., K] and weight [V, K] disagree: {tuple(hidden.shape)} "
                         f"vs {tuple(weight.shape)}")
    h2 = hidden.reshape(-1, hidden.shape[-1])
    if not h2.is_contiguous():
        h2 = h2.contiguous()
    w2 = weight if weight.is_contiguous() else weight.contiguous()
    return h2, w2


def _workspace(nbytes: int, device: torch.device, workspace: Optional[torch.Tensor]) -> torch.Tensor:
    if workspace is not None:
        if workspace.device != device or workspace.numel() * workspace.element_size() < nbytes:
            raise ValueError(f"workspace must be a CUDA tensor of at least {nbytes} bytes on {device}")
        return workspace
    return torch.empty(max(nbytes, 16), dtype=torch.uint8, device=device)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """The model's final RMSNorm (mlx-impl/model.py:336-343, applied at :536), bf16 in/out,
    fp32 arithmetic: ``x * rsqrt(mean(x^2) + eps) * weight``."""
    _require_cuda("x", x)
    _require_cuda("weight", weight)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("x and weight must be bfloat16")
    dim = x.shape[-1]
    if weight.shape != (dim,):
        raise ValueError(f"weight must have shape ({dim},)")
    x2 = x.reshape(-1, dim)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    w = weight if weight.is_contiguous() else weight.contiguous()
    out = torch.empty_like(x2)
    with _on(x2.device):
        status = lib.tome_rmsnorm_bf16(x2.data_ptr(), w.data_ptr(), x2.shape[0], dim, float(eps),
                                       out.data_ptr(), _stream(x2.device))
    _lib.check(status)
    return out.reshape(x.shape)


def _head_flags(round_logits: bool) -> int:
    return _lib.LMHEAD_ROUND_LOGITS_BF16 if round_logits else 0


def lm_head_partials(hidden: torch.Tensor, weight_shard: torch.Tensor, vocab_offset: int,
                     ids: torch.Tensor, temp: float = 1.0, *,
                     workspace: Optional[torch.Tensor] = None, round_logits: bool = False,
                     out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None):
    """Per-row triple ``(m, s, t)`` of one vocabulary shard of the LM head (fp32 ``[rows]`` each).

    ``m = max_j(x_j)/temp``, ``s = sum_j exp(x_j/temp - m)``, ``t = x_target/temp`` if the
    shard owns the target else 0, for ``x = hidden @ weight_shard.T``; no logits are stored.
    ``ids`` are global vocabulary indices; ``vocab_offset`` is the global index of shard row 0.
    ``out`` may name three contiguous fp32 ``[rows]`` tensors to write into (for instance rows of
    the exchange buffer of the vocab-parallel path).
    """
    h2, w2 = _lm_head_inputs(hidden, weight_shard)
    temp = float(temp or 1.0)
    rows, K = h2.shape
    V_local = w2.shape[0]
    device = h2.device
    ids32 = _ids32(ids, rows, device)
    nbytes = lm_head_workspace_bytes(rows, K, V_local)
    ws = _workspace(nbytes, device, workspace)
    if out is None:
        m, s, t = (torch.empty(rows, dtype=torch.float32, device=device) for _ in range(3))
    else:
        m, s, t = out
        for x in (m, s, t):
            if x.dtype != torch.float32 or x.shape != (rows,) or not x.is_contiguous() or \
                    x.device != device:
                raise ValueError("out must hold three contiguous fp32 [rows] tensors on the device")
    with _on(device):
        status = lib.tome_lmhead_partials(
            h2.data_ptr(), w2.data_ptr(), rows, K, V_local, int(vocab_offset), ids32.data_ptr(),
            temp, _head_flags(round_logits), m.data_ptr(), s.data_ptr(), t.data_ptr(), ws.data_ptr(),
            ws.numel() * ws.element_size(), _status_word(device).data_ptr(), _stream(device))
    _lib.check(status)
    return m, s, t


def lm_head_logprob(hidden: torch.Tensor, weight: torch.Tensor, ids: torch.Tensor,
                    temp: float = 1.0, *, workspace: Optional[torch.Tensor] = None,
                    norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                    round_logits: bool = False, check: bool = False):
    """``(logprob, lse)`` of ``ids`` under ``softmax((hidden @ weight.T) / temp)``, fused.

    Replaces the LM head matmul (mlx-impl/model.py:538) followed by
    ``local_compute_logprobs`` (mlx-impl/node.py:400-404); the ``[rows, V]`` logits never
    exist in memory.  ``hidden`` is ``[..., K]`` bf16, ``weight`` ``[V, K]`` bf16 (the tied
    embedding), outputs are fp32 with the leading shape of ``hidden``.

    ``norm_weight`` applies the model's final RMSNorm (mlx-impl/model.py:536) to ``hidden``
    first, which makes the call a replacement for the whole tail of ``Qwen3.__call__``.
    ``round_logits=True`` rounds every logit to bf16 before it is reduced, as the reference's
    materialised bf16 logits are; the default reduces the un-rounded fp32 accumulators.
    """
    if norm_weight is not None:
        hidden = rms_norm(hidden, norm_weight, eps)
    h2, w2 = _lm_head_inputs(hidden, weight)
    temp = float(temp or 1.0)
    rows, K = h2.shape
    V = w2.shape[0]
    device = h2.device
    ids32 = _ids32(ids, rows, device)
    nbytes = lm_head_workspace_bytes(rows, K, V)
    ws = _workspace(nbytes, device, workspace)
    lp = torch.empty(rows, dtype=torch.float32, device=device)
    lse = torch.empty(rows, dtype=torch.float32, device=device)
    with _on(device):
        status = lib.tome_lmhead_logprob(
            h2.data_ptr(), w2.data_ptr(), rows, K, V, ids32.data_ptr(), temp,
            _head_flags(round_logits), lp.data_ptr(), lse.data_ptr(), ws.data_ptr(),
            ws.numel() * ws.element_size(),
            _status_word(device).data_ptr(), _stream(device))
    _lib.check(status)
    if check:
        check_device_status(device)
    lead = hidden.shape[:-1]
    return lp.reshape(lead), lse.reshape(lead)


def lm_head_logprob_static(hidden: torch.Tensor, weight: torch.Tensor, ids: torch.Tensor,
                           temp: float, out_logprob: torch.Tensor,
                           out_lse: Optional[torch.Tensor] = None, *,
                           dev_status: Optional[torch.Tensor] = None) -> None:
    """:func:`lm_head_logprob` for hosts that cannot allocate device memory around the call.

    The library allocates nothing: ``hidden`` ``[rows, K]`` and ``weight`` ``[V, K]`` must
    already be contiguous bf16, ``ids`` contiguous int32 ``[rows]``, and the fp32 outputs
    ``[rows]`` are written in place.  The kernel's scratch is a fixed 8 MiB array inside the
    library (see ``tome_lmhead_logprob_static`` in the header), so sizes that need more raise
    ``TomeArgumentError``; calls on one GPU must not overlap in time.  The first call on a
    device resolves the array's address: make it before stream capture.  The logits are reduced
    un-rounded (there is no ``round_logits`` switch on this entry point).  ``dev_status`` is the
    caller's int32 status word; without it this wrapper uses the module's own word, whose 4
    bytes torch allocates on the first call per device: pass one to allocate nothing at all.
    """
    for name, t, dt in (("hidden", hidden, torch.bfloat16), ("weight", weight, torch.bfloat16),
                        ("ids", ids, torch.int32), ("out_logprob", out_logprob, torch.float32),
                        ("out_lse", out_lse, torch.float32)):
        if t is None and name == "out_lse":
            continue
        _require_cuda(name, t)
        if t.dtype != dt or not t.is_contiguous():
            raise TypeError(f"{name} must be a contiguous {dt} tensor")
        if t.device != hidden.device:
            raise ValueError(f"{name} lives on {t.device}, hidden on {hidden.device}")
    if hidden.dim() != 2 or weight.dim() != 2 or hidden.shape[1] != weight.shape[1]:
        raise ValueError(f"hidden [rows, K] and weight [V, K] disagree: {tuple(hidden.shape)} "
                         f"vs {tuple(weight.shape)}")
    rows, K = hidden.shape
    for name, t in (("ids", ids), ("out_logprob", out_logprob), ("out_lse", out_lse)):
        if t is not None and t.numel() != rows:
            raise ValueError(f"{name} holds {t.numel()} elements, expected one per row ({rows})")
    device = hidden.device
    if dev_status is None:
        dev_status = _status_word(device)  # 4 bytes, allocated on the first call per device
    elif dev_status.dtype != torch.int32 or dev_status.device != device or dev_status.numel() < 1:
        raise ValueError("dev_status must be an int32 tensor on the device of hidden")
    with _on(device):
        status = lib.tome_lmhead_logprob_static(
            hidden.data_ptr(), weight.data_ptr(), rows, K, weight.shape[0], ids.data_ptr(),
            float(temp or 1.0), out_logprob.data_ptr(), _ptr(out_lse),
            dev_status.data_ptr(), _stream(device))
    _lib.check(status)


def combine_triples(m: torch.Tensor, s: torch.Tensor, t: torch.Tensor):
    """Merge per-part triples: ``m``, ``s`` are ``[parts, rows]``; ``t`` is ``[t_parts, rows]``
    (``t_parts`` = 1 when already summed).  Returns ``(logprob, lse)``, fp32 ``[rows]``."""
    for name, x in (("m", m), ("s", s), ("t", t)):
        _require_cuda(name, x)
        if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
            raise ValueError(f"{name} must be a contiguous fp32 [parts, rows] tensor")
    if m.shape != s.shape or t.shape[1] != m.shape[1]:
        raise ValueError("m, s and t disagree in shape")
    parts, rows = m.shape
    device = m.device
    lp = torch.empty(rows, dtype=torch.float32, device=device)
    lse = torch.empty(rows, dtype=torch.float32, device=device)
    with _on(device):
        status = lib.tome_combine_triples(m.data_ptr(), s.data_ptr(), rows, parts, t.data_ptr(),
                                          rows, t.shape[0], rows, lp.data_ptr(), lse.data_ptr(),
                                          _stream(device))
    _lib.check(status)
    return lp, lse


def _paged_args(block_tables, offsets, k_pool, v_pool):
    for name, t in (("block_tables", block_tables), ("offsets", offsets), ("k_pool", k_pool),
                    ("v_pool", v_pool)):
        _require_cuda(name, t)
    if k_pool.shape != v_pool.shape or k_pool.dtype != v_pool.dtype or k_pool.dim() != 4:
        raise ValueError("k_pool and v_pool must be [num_blocks, H, block_size, D] of one dtype")
    if not (k_pool.is_contiguous() and v_pool.is_contiguous()):
        raise ValueError("the pools must be contiguous")
    if k_pool.element_size() not in (2, 4):
        raise TypeError("pool elements must be 2 or 4 bytes wide")
    bt = block_tables.to(torch.int32).contiguous()
    off = offsets.to(torch.int32).contiguous()
    if bt.dim() != 2 or off.shape != (bt.shape[0],):
        raise ValueError("block_tables must be [B, max_blocks] and offsets [B]")
    return bt, off


def gather_paged_kv(block_tables: torch.Tensor, offsets: torch.Tensor, k_pool: torch.Tensor,
                    v_pool: torch.Tensor, max_seq_len: int):
    """Drop-in for ``gather_paged_kv`` (mlx-impl/paged_kv.py:57-116): dense
    ``[B, H, max_seq_len, D]`` keys and values from the paged pool, zero past ``offsets[b]``.
    The sizes the reference passes separately are read from the tensors."""
    bt, off = _paged_args(block_tables, offsets, k_pool, v_pool)
    num_blocks, H, block_size, D = k_pool.shape
    B, max_blocks = bt.shape
    device = k_pool.device
    k_out = torch.empty((B, H, max_seq_len, D), dtype=k_pool.dtype, device=device)
    v_out = torch.empty_like(k_out)
    with _on(device):
        status = lib.tome_gather_paged_kv(
            bt.data_ptr(), off.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
            k_pool.element_size(), B, H, D, block_size, max_blocks, num_blocks, int(max_seq_len),
            k_out.data_ptr(), v_out.data_ptr(), _status_word(device).data_ptr(), _stream(device))
    _lib.check(status)
    return k_out, v_out


def update_paged_kv(k_new: torch.Tensor, v_new: torch.Tensor, block_tables: torch.Tensor,
                    offsets: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                    lengths: Optional[torch.Tensor] = None):
    """``update_paged_kv`` of mlx-impl/paged_kv.py:6-54 with the pool updated IN PLACE (the
    reference returns new arrays): the first ``lengths[b]`` tokens of ``k_new[b]``/``v_new[b]``
    (``[B, H, S_new, D]``) are written into the blocks the table names.  Returns the pools."""
    bt, off = _paged_args(block_tables, offsets, k_pool, v_pool)
    _require_cuda("k_new", k_new)
    _require_cuda("v_new", v_new)
    num_blocks, H, block_size, D = k_pool.shape
    B, max_blocks = bt.shape
    if k_new.shape != v_new.shape or k_new.dim() != 4 or k_new.shape[0] != B or \
            k_new.shape[1] != H or k_new.shape[3] != D or k_new.dtype != k_pool.dtype:
        raise ValueError("k_new/v_new must be [B, H, S_new, D] in the pool's dtype")
    kn = k_new if k_new.is_contiguous() else k_new.contiguous()
    vn = v_new if v_new.is_contiguous() else v_new.contiguous()
    ln = None if lengths is None else lengths.to(device=k_pool.device, dtype=torch.int32).contiguous()
    device = k_pool.device
    with _on(device):
        status = lib.tome_update_paged_kv(
            kn.data_ptr(), vn.data_ptr(), bt.data_ptr(), off.data_ptr(), _ptr(ln),
            k_pool.data_ptr(), v_pool.data_ptr(), k_pool.element_size(), B, H, kn.shape[2], D,
            block_size, max_blocks, num_blocks, _status_word(device).data_ptr(), _stream(device))
    _lib.check(status)
    return k_pool, v_pool
