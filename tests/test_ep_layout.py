"""Host-side layout of the P2P exchange areas (no GPU, no kernels): offsets, views and pointer tables."""
import torch

from flaggems_sglang_b200 import ep


def test_receive_area_layout_and_pointer_tables():
    world, max_tokens, k, H = 4, 10, 2, 64
    xcs = ep.PeerExchange.emulated(world, max_tokens, k, H, torch.bfloat16, device="cpu")
    assert len(xcs) == world
    for r, xc in enumerate(xcs):
        assert (xc.rank, xc.world) == (r, world)
        # worst case: every slot of every rank lands here, each local expert padded to the row block of the kernels
        worst = world * max_tokens * k + xc.e_local * (xc.block - 1)
        assert xc.z_slots == max_tokens * k and xc.capacity == -(-worst // xc.block) * xc.block
        assert xc.rows.shape == (xc.capacity, H) and xc.rows.dtype == torch.bfloat16 and xc.scales is None
        assert xc.weights.shape == (xc.capacity,) and xc.weights.dtype == torch.float32 and xc.src.shape == (xc.capacity, 2)
        assert xc.z.shape == (xc.z_slots, H)
        # every area starts on a 256-byte boundary inside the allocation and areas do not overlap
        spans = sorted(v for v in xc._off.values() if v[1])
        for (o, n), (o2, _) in zip(spans, spans[1:]):
            assert o % 256 == 0 and o + n <= o2
        assert spans[-1][0] + spans[-1][1] <= xc.nbytes
        # entry j of a pointer table is rank j's area; entry `rank` is the own view
        for name, view in (("rows", xc.rows), ("weights", xc.weights), ("src", xc.src), ("z", xc.z)):
            table = xc.ptrs[name]
            assert table.dtype == torch.int64 and table.numel() == world
            assert int(table[r]) == view.data_ptr()
            assert [int(p) for p in table] == [getattr(other, name).data_ptr() for other in xcs]
    xcs[0].close()  # emulated instances own nothing: a no-op


def test_capacity_override_and_row_alignment_rule():
    xcs = ep.PeerExchange.emulated(2, 8, 4, 128, torch.bfloat16, capacity=5, device="cpu")
    blk = xcs[0].block  # a capacity override is rounded up to whole row blocks
    assert xcs[0].capacity == blk and xcs[0].rows.shape == (blk, 128) and xcs[0].z.shape == (32, 128)
    # e4m3 exchange: one byte per channel plus one fp32 scale per 128 channels, quantised by the sender
    xq = ep.PeerExchange.emulated(2, 8, 4, 256, torch.bfloat16, device="cpu", num_local_experts=4, intermediate_size=256,
                                  fp8=True)[1]
    assert xq.rows.dtype == torch.float8_e4m3fn and xq.rows.shape == (xq.capacity, 256)
    assert xq.scales.shape == (xq.capacity, 2) and xq.scales.dtype == torch.float32 and xq.z.dtype == torch.bfloat16
    try:
        ep.PeerExchange.emulated(2, 8, 4, 12, torch.bfloat16, device="cpu")  # 24-byte rows
    except ValueError as e:
        assert "16 bytes" in str(e)
    else:
        raise AssertionError("rows that are not a multiple of 16 bytes must be refused")
