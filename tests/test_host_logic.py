"""CPU tests of the host-side helpers: view handling, id conversion, workload generators, the
band planner's workspace sizes (pure host arithmetic inside the library)."""
import pytest
import torch


def test_rows_view_keeps_strided_rows_and_flattens_leading_dims(built_lib):
    from tome_b200 import ops
    x = torch.zeros((6, 40))
    v, stride = ops._rows_view(x)
    assert v.data_ptr() == x.data_ptr() and stride == 40
    wide = torch.zeros((6, 64))[:, :40]            # row pitch 64, no copy needed
    v, stride = ops._rows_view(wide)
    assert v.data_ptr() == wide.data_ptr() and stride == 64 and v.shape == (6, 40)
    v, stride = ops._rows_view(torch.zeros((2, 3, 40)))
    assert v.shape == (6, 40) and stride == 40
    t = torch.zeros((40, 6)).t()                   # last dim not contiguous: copied
    v, stride = ops._rows_view(t)
    assert v.is_contiguous() and v.shape == (6, 40) and stride == 40
    with pytest.raises(ValueError):
        ops._rows_view(torch.tensor(1.0))


def test_ids_are_converted_and_counted(built_lib):
    from tome_b200 import ops
    ids = ops._ids32(torch.tensor([[1, 2], [3, 4]], dtype=torch.int64), 4, torch.device("cpu"))
    assert ids.dtype == torch.int32 and ids.shape == (4,) and ids.tolist() == [1, 2, 3, 4]
    assert ops._ids32([5, 6], 2, torch.device("cpu")).tolist() == [5, 6]
    with pytest.raises(ValueError):
        ops._ids32(torch.zeros(3, dtype=torch.int32), 4, torch.device("cpu"))
    with pytest.raises(TypeError):
        ops._ids32(torch.zeros(4), 4, torch.device("cpu"))


def test_generators_are_seeded_and_shaped():
    from tome_b200 import synthetic
    a, ta = synthetic.cfg2_rollout_bf16(rows=16, vocab=4096)
    b, tb = synthetic.cfg2_rollout_bf16(rows=16, vocab=4096)
    assert torch.equal(a, b) and torch.equal(ta, tb) and a.dtype == torch.bfloat16
    assert bool((a.float() == 12.0).any(dim=1).all())          # every row has its planted column
    hits = a.float().gather(1, ta.long()[:, None]).squeeze(1) == 12.0
    assert 0.3 < float(hits.float().mean()) <= 1.0              # targets hit it with p = 0.7
    pol, ref, tg, lengths, temp = synthetic.cfg5_dual(4, 32, 512)
    assert pol.shape == (4, 32, 512) and tg.shape == (4, 32) and temp == 0.7
    assert int(lengths.min()) >= 32 and int(lengths.max()) <= 32   # min_len clipped to seq_len
    assert 0.0 < float((pol.float() - ref.float()).abs().mean()) < 0.3
    h, w, t = synthetic.cfg4_vocab_parallel(8, 64, 100)
    assert h.shape == (8, 64) and w.shape == (100, 64) and float(w.float().std()) < 0.03
    bounds = [synthetic.shard_bounds(151936, r, 8) for r in range(8)]
    assert bounds[0] == (0, 18992) and bounds[-1] == (132944, 151936)
    assert all(bounds[i][1] == bounds[i + 1][0] for i in range(7))


def test_workspace_sizes_follow_the_band_plan(built_lib):
    from tome_b200 import _lib
    ws = _lib.lib.tome_lmhead_workspace_bytes
    assert ws(0, 1024, 1000) == 0 and ws(16, 1024, 0) == 0
    # Qwen3-0.6B head, 16384 rows: 38 bands of 16 column tiles -> fits the 8 MiB static scratch
    assert ws(16384, 1024, 151936) == 3 * 38 * 16384 * 4
    assert ws(16384, 1024, 151936) <= _lib.lib.tome_lmhead_static_scratch_bytes()
    # one column tile: one band; the size scales with rows
    assert ws(128, 64, 256) == 3 * 1 * 128 * 4
    assert ws(256, 64, 256) == 2 * ws(128, 64, 256)
    # the plan never depends on the caller's device: same answer twice
    assert ws(32768, 4096, 18992) == ws(32768, 4096, 18992) > 0
