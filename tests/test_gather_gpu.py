"""The peer-store kernel that reassembles y / C across ranks, driven on one GPU.

The "peers" here are further buffers of the same device: the kernel sees only pointers, so offsets,
ragged heads and tails and the several-peers-per-launch indexing are exercised exactly as with
peer-mapped memory.  The multi-rank protocol around it is covered by the 2-rank CPU tests.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as O
from ops_sparse_b200 import _lib as L
from ops_sparse_b200 import api
from tests.gpu_util import SpmmCase, SpmvCase, random_csr

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


@pytest.mark.parametrize("name", ["c1", "c4"])
def test_graph_replay_of_a_step_equals_the_eager_step(name):
    """One rank: the step captured as a CUDA graph gives the bits of the kernel-by-kernel step."""
    from ops_sparse_b200 import sharded, workloads
    cfg = workloads.make(name, rows=8192 if name == "c4" else None)
    op_cls = sharded.ShardedSpMV if cfg["kind"] == "spmv" else sharded.ShardedSpMM
    op = op_cls(cfg, 0, 1, torch.device("cuda:0"))
    local = op.y_local if cfg["kind"] == "spmv" else op.c_local
    start = local.clone()
    eager = op.step(1.25, 0.5).clone()
    assert op.capture(1.25, 0.5)
    for _ in range(2):
        local.copy_(start)
        replayed = op.step(1.25, 0.5)
        torch.cuda.synchronize()
        assert torch.equal(replayed, eager)
    local.copy_(start)
    assert torch.equal(op.step(1.0, 0.0), op.step(1.0, 0.0))  # other scalars: eager path, still valid


@pytest.mark.parametrize("name,beta,pad", [("c1", 0.0, 5), ("c1", 0.5, 5), ("c3", 0.5, 5), ("c4", 0.0, 5),
                                           ("c4", -0.25, 5), ("c2", 0.0, 5), ("c2", 0.5, 8), ("c2", 0.0, 8)])
@pytest.mark.parametrize("mirrors", [1, 7])
def test_mirrors_receive_exactly_what_the_output_receives(name, beta, pad, mirrors):
    """Every element the product writes lands in each mirror too, bit for bit; nothing else is touched.  pad: guard
    elements either side of each mirror; 5 also puts the mirrors off 16-byte alignment (word stores), 8 keeps them
    on it (the row-block kernel of c2 then sends 16-byte vectors; 29791 rows: the last block is partial)."""
    from ops_sparse_b200 import api, workloads
    cfg = workloads.make(name, rows={"c1": None, "c2": 29791, "c3": 40000, "c4": 6000}[name])
    dev = torch.device("cuda:0")
    spmv = cfg["kind"] == "spmv"
    rows, cols = cfg["rows"], cfg["cols"]
    handle = api.Handle()
    mat = api.CsrMatrix(rows, cols, torch.from_numpy(cfg["row_ptr"]).to(dev), torch.from_numpy(cfg["col_ind"]).to(dev),
                        torch.from_numpy(cfg["values"]).to(dev), 0, nnz=cfg["nnz"])
    out0 = torch.from_numpy(cfg["y"] if spmv else cfg["c"]).to(dev)
    def run(with_mirrors):
        out = out0.clone()
        bufs = [torch.full((out.numel() + 2 * pad,), 7.0, device=dev) for _ in range(mirrors if with_mirrors else 0)]
        if spmv:
            y = api.DnVec(out)
            op = api.SpMV(handle, mat, api.DnVec(torch.from_numpy(cfg["x"]).to(dev)), y)
            target = y
        else:
            n = cfg["n"]
            c = api.DnMat(rows, n, n, out)
            op = api.SpMM(handle, mat, api.DnMat(cols, n, n, torch.from_numpy(cfg["b"]).to(dev)), c)
            target = c
        if with_mirrors:
            target.set_mirrors([b.data_ptr() + 4 * pad for b in bufs])
        op.preprocess()
        op(1.5, beta)
        torch.cuda.synchronize()
        return out, bufs
    plain, _ = run(False)
    mirrored, bufs = run(True)
    assert torch.equal(plain, mirrored)
    for b in bufs:
        assert torch.equal(b[pad:-pad], mirrored.reshape(-1))
        assert bool((b[:pad] == 7.0).all()) and bool((b[-pad:] == 7.0).all())


def test_mirror_list_is_validated():
    from ops_sparse_b200 import api
    y = api.DnVec(torch.zeros(8, device="cuda"))
    with pytest.raises(api.AclsparseError):
        y.set_mirrors([1] * 8)  # more than 7
    with pytest.raises(api.AclsparseError):
        y.set_mirrors([0])      # null mirror
    y.set_mirrors([])           # clears


def test_node_barrier_announces_waits_and_gives_up_within_its_limit():
    """The node barrier on one GPU.  The "peers" are further state blocks of the same device whose flags the
    test sets by hand, so no kernel ever waits for another kernel: (1) peers that have arrived let the barrier
    through and receive this rank's epoch; (2) a peer that never arrives makes the barrier give up after its
    poll limit, the status call reports EXECUTION_FAILED and names the rank, nothing hangs; (3) the next
    barrier, with every peer present, succeeds again."""
    lib = L.lib()
    world, rank = 4, 1
    states = [torch.zeros(32, dtype=torch.int32, device="cuda") for _ in range(world)]  # epoch, status, -, -, flag[16]
    ptrs = (ctypes.c_void_p * world)(*[s.data_ptr() for s in states])
    local = states[rank]
    missing = ctypes.c_int(-1)

    def arrive(epoch, ranks):
        for r in ranks:
            local[4 + r] = epoch
        torch.cuda.synchronize()

    # (1) everyone is there
    arrive(1, [0, 2, 3])
    assert lib.aclsparseB200NodeBarrier(0x1, local.data_ptr(), ptrs, world, rank, 1000) == L.SUCCESS
    assert lib.aclsparseB200NodeBarrierStatus(0x1, local.data_ptr(), ctypes.byref(missing)) == L.SUCCESS
    for r in (0, 2, 3):
        assert int(states[r][4 + rank]) == 1          # announced to every peer
    assert int(local[0]) == 1
    # (2) rank 2 never announces epoch 2: the wait runs out after 2000 polls (well under a second)
    arrive(2, [0, 3])
    assert lib.aclsparseB200NodeBarrier(0x1, local.data_ptr(), ptrs, world, rank, 2000) == L.SUCCESS  # enqueue
    st = lib.aclsparseB200NodeBarrierStatus(0x1, local.data_ptr(), ctypes.byref(missing))
    assert st == L.EXECUTION_FAILED and missing.value == 2
    assert int(states[0][4 + rank]) == 2              # it did announce itself before giving up
    # (3) the record was cleared; with every peer present the next barrier is fine
    arrive(3, [0, 2, 3])
    assert lib.aclsparseB200NodeBarrier(0x1, local.data_ptr(), ptrs, world, rank, 2000) == L.SUCCESS
    assert lib.aclsparseB200NodeBarrierStatus(0x1, local.data_ptr(), ctypes.byref(missing)) == L.SUCCESS
    # argument checks never reach the device
    assert lib.aclsparseB200NodeBarrier(0x1, None, ptrs, world, rank, 0) == L.INVALID_VALUE
    assert lib.aclsparseB200NodeBarrier(0x1, local.data_ptr(), ptrs, 17, rank, 0) == L.INVALID_VALUE
    assert lib.aclsparseB200NodeBarrier(0x1, local.data_ptr(), ptrs, world, 4, 0) == L.INVALID_VALUE


@pytest.mark.parametrize("shape", ["row_blocks", "tiles", "spmm"])
def test_closing_barrier_of_a_product(shape):
    """The same barrier as the end of a product (aclsparseB200DnVecSetClosingBarrier / DnMat...), on one GPU in
    the same form: the peers' flags are set by hand before the launch, so nothing waits for another kernel.
    The product's last kernel (the row-block kernel, the SpMV carry fix-up or the SpMM carry fix-up) announces
    this rank's epoch to every peer, leaves the CTA ticket counter at zero and the result unchanged; a peer
    that never arrives makes it give up within its limit, and the product is still right."""
    lib = L.lib()
    rng = np.random.default_rng(17)
    world, rank = 3, 2
    states = [torch.zeros(32, dtype=torch.int32, device="cuda") for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[s.data_ptr() for s in states])
    local = states[rank]
    missing = ctypes.c_int(-1)
    rows, cols = 6000, 5000
    lengths = rng.integers(3, 12, rows) if shape == "row_blocks" else rng.poisson(9, rows)
    if shape != "row_blocks":
        lengths[100] = 4500  # a row that crosses tiles: the fix-up kernels have carries to join
    rp, ci = random_csr(rng, lengths, cols)
    va = rng.standard_normal(ci.size).astype(np.float32)
    if shape == "spmm":
        n = 8
        b = rng.standard_normal((cols, n)).astype(np.float32)
        case = SpmmCase(rp, ci, va, cols, n, b, n, np.zeros((rows, n), np.float32), n)
        truth = O.spmm_f64(rp, ci, va, b, n, np.zeros((rows, n), np.float32), n, n, cols)
        out = case.mc
    else:
        x = rng.standard_normal(cols).astype(np.float32)
        case = SpmvCase(rp, ci, va, x, np.zeros(rows, np.float32))
        truth = O.spmv_f64(rp, ci, va, x, np.zeros(rows, np.float32))
        out = case.vy
    case.op.preprocess()
    torch.cuda.synchronize()  # the host knows the longest row: one SpMV kernel (row blocks) or two (tiles)

    def arrive(epoch, ranks):
        for r in ranks:
            local[4 + r] = epoch
        torch.cuda.synchronize()

    def product_ok():
        got = case.run(preprocess=False).reshape(truth.shape)
        return O.check_tolerance(got, truth)[0] == 0

    before = api.kernel_launches()
    assert product_ok()
    plain_launches = api.kernel_launches() - before
    out.set_closing_barrier(local.data_ptr(), ptrs, world, rank, 2000)
    # (1) both peers are there
    arrive(1, [0, 1])
    before = api.kernel_launches()
    assert product_ok()
    assert api.kernel_launches() - before == plain_launches       # no kernel of its own
    assert lib.aclsparseB200NodeBarrierStatus(0x1, local.data_ptr(), ctypes.byref(missing)) == L.SUCCESS
    assert [int(states[r][4 + rank]) for r in (0, 1)] == [1, 1]  # announced to every peer
    assert int(local[0]) == 1 and int(local[2]) == 0              # epoch counted, tickets back at zero
    # (2) rank 0 never announces epoch 2: the last CTA gives up after 2000 polls; the product is complete
    arrive(2, [1])
    assert product_ok()
    st = lib.aclsparseB200NodeBarrierStatus(0x1, local.data_ptr(), ctypes.byref(missing))
    assert st == L.EXECUTION_FAILED and missing.value == 0
    assert int(states[1][4 + rank]) == 2 and int(local[2]) == 0
    # (3) the next product, with every peer present, is fine; then the barrier is taken off again
    arrive(3, [0, 1])
    assert product_ok()
    assert lib.aclsparseB200NodeBarrierStatus(0x1, local.data_ptr(), ctypes.byref(missing)) == L.SUCCESS
    out.set_closing_barrier(0, None, 0, 0)
    assert product_ok() and int(local[0]) == 3
