"""Multi-rank host logic on CPU: nnz-balanced row blocks, shard slicing and the all-gather (gloo, 2 ranks).

The per-rank product is a stand-in from the test oracle: what is under test is the partition,
the rebased shards and the reassembly, which are the same code the NCCL path runs.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from ops_sparse_b200 import sharded, workloads


def test_aligned_bounds_keep_the_partition_valid():
    """Inner boundaries move to multiples of 32 rows (so that every rank's block of y starts on a 128-byte
    boundary); the ends stay, the order stays, ranks may end up without rows."""
    for raw in ([0, 1000, 2047, 2049, 5000], [0, 3, 5, 9], [0, 10, 20, 40], [0, 16, 48, 49], [0, 0, 0, 7]):
        got = sharded.align_bounds(np.array(raw, np.int32), 32)
        assert got.dtype == np.int32 and got[0] == raw[0] and got[-1] == raw[-1]
        assert np.all(np.diff(got) >= 0)
        assert all(int(b) % 32 == 0 or int(b) == raw[-1] for b in got[1:-1])
        assert np.all(np.abs(got[1:-1].astype(np.int64) - np.array(raw[1:-1])) <= 32)


def test_bounds_match_the_oracle_twin():
    rng = np.random.default_rng(2)
    for lens in (rng.poisson(16, 5000), np.clip(rng.zipf(2.0, 4000), 1, 2000), np.zeros(100, int),
                 np.concatenate([rng.integers(1, 9, 500), np.zeros(40, int)])):
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        nnz = int(rp[-1])
        for base in (0, 1):
            for parts in (1, 2, 3, 4, 8):
                got = sharded.row_block_bounds_host(rp + base, nnz, parts, base)
                np.testing.assert_array_equal(got, O.row_block_bounds(rp + base, nnz, parts, base))


def test_shards_tile_the_matrix():
    cfg = workloads.make("c3", rows=1 << 13)
    bounds = sharded.row_block_bounds_host(cfg["row_ptr"], cfg["nnz"], 4)
    seen_rows, seen_nnz = 0, 0
    for g in range(4):
        ptr, col, val = sharded.shard_csr(cfg["row_ptr"], cfg["col_ind"], cfg["values"], bounds, g)
        assert ptr[0] == 0 and ptr[-1] == col.size == val.size
        np.testing.assert_array_equal(np.diff(ptr), np.diff(cfg["row_ptr"][bounds[g]:bounds[g + 1] + 1]))
        seen_rows += ptr.size - 1
        seen_nnz += col.size
    assert (seen_rows, seen_nnz) == (cfg["rows"], cfg["nnz"])
    per = np.diff(cfg["row_ptr"][bounds].astype(np.int64))
    assert per.max() - per.min() <= 2 * np.diff(cfg["row_ptr"]).max()


def _spmv_stand_in(local, x, y_local, alpha, beta):
    ptr, col, val = local
    out = O.spmv_f64(ptr, col, val, x.numpy(), y_local.numpy(), alpha, beta)
    y_local.copy_(torch.from_numpy(out.astype(np.float32)))


def _spmm_stand_in(local, b, c_local, alpha, beta):
    ptr, col, val = local
    n = b.shape[1]
    out = O.spmm_f64(ptr, col, val, b.numpy(), n, c_local.numpy(), n, n, b.shape[0], alpha, beta)
    c_local.copy_(torch.from_numpy(out.astype(np.float32)))


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = workloads.make("c3", rows=1 << 12)
        op = sharded.ShardedSpMV(cfg, rank, world, torch.device("cpu"), local_product=_spmv_stand_in)
        y = op.step(cfg["alpha"], cfg["beta"]).numpy()
        truth = O.spmv_f64(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["x"], cfg["y"], cfg["alpha"],
                           cfg["beta"])
        bad, _, _ = O.check_tolerance(y, truth)
        cfg4 = workloads.make("c4", rows=1 << 10)
        op4 = sharded.ShardedSpMM(cfg4, rank, world, torch.device("cpu"), local_product=_spmm_stand_in)
        c = op4.step(1.0, 0.0).numpy()
        truth4 = O.spmm_f64(cfg4["row_ptr"], cfg4["col_ind"], cfg4["values"], cfg4["b"], 128, cfg4["c"], 128, 128,
                            cfg4["cols"])
        bad4, _, _ = O.check_tolerance(c, truth4)
        results[rank] = (int(bad), int(bad4), y.shape[0], tuple(c.shape))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_gather_reassembles_the_product():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert dict(results) == {0: (0, 0, 1 << 12, (1 << 10, 128)), 1: (0, 0, 1 << 12, (1 << 10, 128))}


def test_reassembly_modes_off_gpu_and_single_rank():
    """Without CUDA every reassembly mode resolves to the all-gather; one rank returns its block untouched."""
    cfg = workloads.make("c1")
    for mode in ("multicast", "fused", "push", "nccl"):
        op = sharded.ShardedSpMV(cfg, 0, 1, torch.device("cpu"), local_product=_spmv_stand_in, gather=mode)
        assert op.gather_mode == "nccl"
        assert not op.capture(1.0, 0.0)         # nothing to record without the CUDA operators
        op.reassemble_in_kernel(True)           # and nothing to register
        y = op.step(cfg["alpha"], cfg["beta"])
        assert y.data_ptr() == op.y_local.data_ptr() and y.shape == (cfg["rows"],)
        truth = O.spmv_f64(cfg["row_ptr"], cfg["col_ind"], cfg["values"], cfg["x"], cfg["y"], cfg["alpha"], cfg["beta"])
        assert O.check_tolerance(y.numpy(), truth)[0] == 0
