"""The peer-store kernel that reassembles y / C across ranks, driven on one GPU.

The "peers" here are further buffers of the same device: the kernel sees only pointers, so offsets,
ragged heads and tails and the several-peers-per-launch indexing are exercised exactly as with
peer-mapped memory.  The multi-rank protocol around it is covered by the 2-rank CPU tests.
"""
import ctypes

import pytest
import torch

from ops_sparse_b200 import _lib as L

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("offset,count", [(0, 0), (0, 1), (3, 2), (1, 4099), (4, 1 << 20), (7, (1 << 20) + 5),
                                          (12345, 3_000_001)])
@pytest.mark.parametrize("peers", [1, 3, 7])
def test_push_slice_copies_exactly_the_block(offset, count, peers):
    lib = L.lib()
    total = offset + count + 9
    gen = torch.Generator(device="cuda").manual_seed(offset * 31 + count)
    src = torch.rand(total, device="cuda", generator=gen)
    dst = [torch.full((total,), -1.0, device="cuda") for _ in range(peers)]
    ptrs = (ctypes.c_void_p * peers)(*[d.data_ptr() for d in dst])
    lib.aclsp_b200_push_slice_kernel_do(src.data_ptr(), ptrs, peers, offset, count, 0x1)
    torch.cuda.synchronize()
    for d in dst:
        assert torch.equal(d[offset:offset + count], src[offset:offset + count])
        assert bool((d[:offset] == -1.0).all()) and bool((d[offset + count:] == -1.0).all())
