"""GPU tests of the paged KV gather/update kernels: byte-exact against the oracle's loop
restatement of mlx-impl/paged_kv.py."""
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def _pool(num_blocks, H, bs, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn((num_blocks, H, bs, D), generator=g).to(dtype)
    v = torch.randn((num_blocks, H, bs, D), generator=g).to(dtype)
    return k, v


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gather_matches_reference_loops(cuda_device, dtype):
    import tome_b200
    num_blocks, H, bs, D, B = 40, 3, 16, 64, 5
    k_pool, v_pool = _pool(num_blocks, H, bs, D, dtype, 1)
    g = torch.Generator().manual_seed(2)
    tables = torch.stack([torch.randperm(num_blocks, generator=g)[:6] for _ in range(B)]).to(torch.int32)
    offsets = torch.tensor([0, 1, 16, 37, 96], dtype=torch.int32)   # empty, partial, full table
    max_len = 96
    k_out, v_out = tome_b200.gather_paged_kv(tables.to(cuda_device), offsets.to(cuda_device),
                                             k_pool.to(cuda_device), v_pool.to(cuda_device), max_len)
    o_k, o_v = oracle.gather_paged_kv(tables, offsets, k_pool, v_pool, max_len)
    assert k_out.dtype == dtype and k_out.shape == (B, H, max_len, D)
    assert torch.equal(k_out.cpu(), o_k) and torch.equal(v_out.cpu(), o_v)
    tome_b200.check_device_status(cuda_device)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_update_matches_reference_loops_and_round_trips(cuda_device, dtype):
    import tome_b200
    num_blocks, H, bs, D, B, S_new = 32, 2, 16, 128, 4, 50
    k_pool, v_pool = _pool(num_blocks, H, bs, D, dtype, 3)
    g = torch.Generator().manual_seed(4)
    perm = torch.randperm(num_blocks, generator=g)
    tables = perm[: B * 4].reshape(B, 4).to(torch.int32)             # disjoint blocks
    k_new = torch.randn((B, H, S_new, D), generator=g).to(dtype)
    v_new = torch.randn((B, H, S_new, D), generator=g).to(dtype)
    offsets = torch.tensor([0, 0, 16, 48], dtype=torch.int32)        # last two run off the table
    lengths = torch.tensor([50, 7, 40, 33], dtype=torch.int32)
    kp, vp = k_pool.to(cuda_device), v_pool.to(cuda_device)
    tome_b200.update_paged_kv(k_new.to(cuda_device), v_new.to(cuda_device), tables.to(cuda_device),
                              offsets.to(cuda_device), kp, vp, lengths=lengths.to(cuda_device))
    o_k, o_v = oracle.update_paged_kv(k_new, v_new, tables, offsets, k_pool, v_pool, bs, lengths)
    assert torch.equal(kp.cpu(), o_k) and torch.equal(vp.cpu(), o_v)
    # flush from position 0 then gather gives the tokens back (kvcache.py:186-257)
    kp2, vp2 = k_pool.to(cuda_device), v_pool.to(cuda_device)
    zero = torch.zeros(B, dtype=torch.int32, device=cuda_device)
    tome_b200.update_paged_kv(k_new.to(cuda_device), v_new.to(cuda_device), tables.to(cuda_device),
                              zero, kp2, vp2, lengths=lengths.to(cuda_device))
    kg, vg = tome_b200.gather_paged_kv(tables.to(cuda_device), lengths.to(cuda_device), kp2, vp2, S_new)
    for b in range(B):
        n = int(lengths[b])
        assert torch.equal(kg[b, :, :n].cpu(), k_new[b, :, :n]) and torch.equal(vg[b, :, :n].cpu(), v_new[b, :, :n])
        assert float(kg[b, :, n:].abs().max() if n < S_new else 0) == 0
    # no lengths: everything is written
    kp3, vp3 = k_pool.to(cuda_device), v_pool.to(cuda_device)
    tome_b200.update_paged_kv(k_new.to(cuda_device), v_new.to(cuda_device), tables.to(cuda_device),
                              zero, kp3, vp3)
    o_k3, _ = oracle.update_paged_kv(k_new, v_new, tables, torch.zeros(B), k_pool, v_pool, bs)
    assert torch.equal(kp3.cpu(), o_k3)


def test_bad_table_entries_are_reported_not_followed(cuda_device):
    import tome_b200
    k_pool, v_pool = _pool(4, 1, 16, 64, torch.bfloat16, 5)
    tables = torch.tensor([[0, 9]], dtype=torch.int32)                # 9 is outside the pool
    offsets = torch.tensor([32], dtype=torch.int32)
    k_out, _ = tome_b200.gather_paged_kv(tables.to(cuda_device), offsets.to(cuda_device),
                                         k_pool.to(cuda_device), v_pool.to(cuda_device), 32)
    assert torch.equal(k_out[0, :, :16].cpu(), k_pool[0]) and float(k_out[0, :, 16:].abs().max()) == 0
    with pytest.raises(tome_b200.TomeRuntimeError):
        tome_b200.check_device_status(cuda_device)
    with pytest.raises(tome_b200.TomeArgumentError):                  # head_dim * 2 bytes % 16 != 0
        bad = torch.zeros((4, 1, 16, 4), dtype=torch.bfloat16, device=cuda_device)
        tome_b200.gather_paged_kv(tables.to(cuda_device), offsets.to(cuda_device), bad, bad, 8)


def test_gather_against_output_of_the_reference_metal_kernel(cuda_device):
    """tests/golden/metal_kernel.npz holds what the reference's own gather kernel body
    (mlx-impl/paged_kv.py:57-116, compiled for the CPU by oracle/build_ref.py) produces."""
    import tome_b200
    from helpers import from_bits, load_golden
    gold = load_golden("metal_kernel.npz")
    as_bf16 = lambda name: from_bits(gold[name], torch.bfloat16)  # noqa: E731
    k_out, v_out = tome_b200.gather_paged_kv(
        torch.from_numpy(gold["gather_tables"].copy()).to(cuda_device),
        torch.from_numpy(gold["gather_offsets"].copy()).to(cuda_device),
        as_bf16("gather_k_pool").to(cuda_device), as_bf16("gather_v_pool").to(cuda_device),
        int(gold["gather_max_seq_len"]))
    tome_b200.check_device_status(cuda_device)
    assert torch.equal(k_out.cpu().view(torch.int16), as_bf16("gather_k_out").view(torch.int16))
    assert torch.equal(v_out.cpu().view(torch.int16), as_bf16("gather_v_out").view(torch.int16))
