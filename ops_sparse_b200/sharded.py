"""Row-block sharding of CSR SpMV / SpMM over the GPUs of one node.

One process per GPU (``torch.distributed``, NCCL over NVLink).  The matrix is cut
into ``world_size`` contiguous row blocks that balance the non-zeros:

    bounds[g] = min{ r : rowOffsets[r] - base >= ceil(g * nnz / G) },   bounds[G] = rows

Rank g holds rows [bounds[g], bounds[g+1]) of A (row offsets rebased to start at
0, its slice of the column indices and values), a full replica of x or B, and
computes its slice of y or C with the single-GPU operators.  The only exchange
is the reassembly of y / C on every rank, in one of four ways:

* ``multicast`` (default on GPUs): as ``fused`` below, but the single mirror is the
  NVLink multicast address of the symmetric buffer: the kernels write finished
  rows with ``multimem.st`` and NVSwitch delivers them to every GPU, so a rank
  sends its row block once, not once per peer.  ``fused`` is used instead at two
  ranks and where the buffer has no multicast mapping.
* ``fused``: the result lives in a symmetric-memory buffer that
  every rank maps, and the peers' buffers are registered as mirrors of the local
  output (``aclsparseB200DnVecSetMirrors`` / ``DnMatSetMirrors``): the product
  kernels store each finished row into all ranks' buffers themselves, over
  NVLink, while the rest of the matrix is still being multiplied.  The library's
  node barrier (``aclsparseB200NodeBarrier``: one small kernel whose waits are
  bounded and report through a status word) closes the step.  No padding, no
  concatenation, no separate transfer.
* ``push``: same buffers, but the product writes its row block locally and one
  further kernel (``aclsp_b200_push_slice_kernel_do``) stores the block into all
  peers' buffers before the barrier.
* ``nccl``: an all-gather; row blocks have unequal row counts, so slices travel
  padded to the largest block and are compacted by one concatenation afterwards.

The reference library is single-device; this layer has no counterpart there.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np
import torch
import torch.distributed as dist

from . import _lib as L


def row_block_bounds_host(row_ptr: np.ndarray, nnz: int, parts: int, index_base: int = 0) -> np.ndarray:
    """Host evaluation of the bounds formula above (the device version is aclsparseB200RowBlockBounds)."""
    offs = np.asarray(row_ptr, dtype=np.int64)[:-1] - index_base
    targets = (np.arange(parts + 1, dtype=np.int64) * nnz + parts - 1) // parts
    bounds = np.searchsorted(offs, targets, side="left").astype(np.int32)
    bounds[parts] = offs.size
    return bounds


def shard_csr(row_ptr: np.ndarray, col_ind: np.ndarray, values: np.ndarray, bounds: np.ndarray, rank: int,
              index_base: int = 0):
    """Rank's row block as a self-contained CSR: rebased row offsets and the matching index / value slices."""
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    p0, p1 = int(row_ptr[r0]) - index_base, int(row_ptr[r1]) - index_base
    local_ptr = (np.asarray(row_ptr[r0:r1 + 1], dtype=np.int64) - row_ptr[r0] + index_base).astype(np.int32)
    return local_ptr, col_ind[p0:p1], values[p0:p1]


def align_bounds(bounds: np.ndarray, multiple: int) -> np.ndarray:
    """The inner boundaries of a row partition moved to the nearest multiple of ``multiple`` rows (the ends stay):
    every rank's block of a result vector then starts on a 128-byte boundary for ``multiple`` = 32, which lets the
    product kernels send their rows to the other GPUs as whole 16-byte vectors.  The balance by non-zeros moves
    by at most ``multiple`` / 2 rows per boundary."""
    out = np.asarray(bounds, dtype=np.int64).copy()
    rows = int(out[-1])
    for g in range(1, out.size - 1):
        moved = int(round(int(out[g]) / multiple)) * multiple
        out[g] = min(max(moved, int(out[g - 1])), rows)
    return out.astype(np.int32)


class _Gather:
    """All-gather of unequal row blocks: padded slots, then one concatenation."""

    def __init__(self, bounds: np.ndarray, rank: int, width: int, device, group=None):
        self.rows = np.diff(bounds).astype(np.int64)
        self.rank, self.width, self.group = rank, width, group
        self.world = self.rows.size
        self.max_rows = int(self.rows.max()) if self.rows.size else 0
        shape = (self.world, max(self.max_rows, 1), width) if width > 1 else (self.world, max(self.max_rows, 1))
        self.slots = torch.zeros(shape, dtype=torch.float32, device=device)
        self.local = self.slots[rank][: int(self.rows[rank])]

    def run(self) -> torch.Tensor:
        if self.world == 1:
            return self.local
        dist.all_gather_into_tensor(self.slots.view(-1), self.slots[self.rank].reshape(-1), group=self.group)
        return torch.cat([self.slots[g][: int(self.rows[g])] for g in range(self.world)])


class _PushGather:
    """Reassembly by peer stores into a symmetric-memory result buffer (see the module docstring).

    The buffer of step k is overwritten by the peers' pushes of step k+1: a consumer that still reads
    it then must copy it first, exactly as with a reused all-gather output.
    """

    def __init__(self, bounds: np.ndarray, rank: int, width: int, device, group=None, fused=False, multicast=False):
        import torch.distributed._symmetric_memory as symm
        if not multicast:  # plain peer stores only: keep the buffer off NVLink multicast objects
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.rank, self.width = rank, width
        self.world = bounds.size - 1
        group = group if group is not None else dist.group.WORLD
        total = int(bounds[-1])
        shape = (max(total, 1), width) if width > 1 else (max(total, 1),)
        self.full = symm.empty(shape, dtype=torch.float32, device=device)
        self.full.zero_()
        self.handle = symm.rendezvous(self.full, group=group)
        r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
        self.local = self.full[r0:r1]
        self.offset, self.count = r0 * width, (r1 - r0) * width
        ptrs = [int(p) for g, p in enumerate(self.handle.buffer_ptrs) if g != rank]
        self.peers = (ctypes.c_void_p * max(len(ptrs), 1))(*ptrs)
        self.num_peers = len(ptrs)
        self.fused = fused
        # Peers' addresses of this rank's row block: the mirrors of the local output in fused mode.
        self.mirror_ptrs = [p + self.offset * 4 for p in ptrs]
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0) if multicast else 0
        self.multicast_ptr = mc + self.offset * 4 if mc else 0
        self._lib = L.lib()
        # State of the library's own node barrier (AclspNodeBarrierState: 128 bytes per rank, zero-filled,
        # addressable by every rank).  Its waits are bounded and report through a status word.
        self.barrier_state = symm.empty((32,), dtype=torch.int32, device=device)
        self.barrier_state.zero_()
        state_handle = symm.rendezvous(self.barrier_state, group=group)
        self.barrier_peers = (ctypes.c_void_p * self.world)(*[int(p) for p in state_handle.buffer_ptrs])
        # True while the product's last kernel ends with the barrier itself (the output descriptor's closing
        # barrier): run() then launches nothing.
        self.barrier_in_kernel = False
        torch.cuda.synchronize()
        dist.barrier(group=group)  # every state is zero before any rank announces an epoch

    def run(self) -> torch.Tensor:
        if not self.fused:
            stream = torch.cuda.current_stream().cuda_stream or 0x1
            self._lib.aclsp_b200_push_slice_kernel_do(self.full.data_ptr(), self.peers, self.num_peers, self.offset,
                                                      self.count, stream)
        if self.barrier_in_kernel:
            return self.full
        stream = torch.cuda.current_stream().cuda_stream or 0x1
        status = self._lib.aclsparseB200NodeBarrier(stream, self.barrier_state.data_ptr(), self.barrier_peers,
                                                    self.world, self.rank, 0)
        if status != L.SUCCESS:
            raise RuntimeError(f"aclsparseB200NodeBarrier returned {status}")
        return self.full

    def check_barriers(self) -> None:
        """Synchronises and raises if a barrier since the last call gave up waiting for a rank."""
        missing = ctypes.c_int(-1)
        stream = torch.cuda.current_stream().cuda_stream or 0x1
        status = self._lib.aclsparseB200NodeBarrierStatus(stream, self.barrier_state.data_ptr(), ctypes.byref(missing))
        if status != L.SUCCESS:
            raise RuntimeError(f"node barrier: rank {missing.value} did not arrive within the limit "
                               f"(status {L.STATUS_NAMES.get(status, status)})")


def _make_gather(mode: str, bounds, rank, width, device, group):
    """``fused`` / ``push`` where symmetric memory can be set up, else the all-gather; returns (gather, mode used)."""
    world = bounds.size - 1
    if mode == "multicast" and world == 2:
        mode = "fused"  # one peer: a multicast store saves nothing over the plain peer store
    if mode in ("multicast", "fused", "push") and world > 1 and torch.device(device).type == "cuda":
        try:
            g = _PushGather(bounds, rank, width, device, group, fused=mode != "push", multicast=mode == "multicast")
            return g, ("fused" if mode == "multicast" and not g.multicast_ptr else mode)
        except Exception as err:  # symmetric memory is optional plumbing; the all-gather gives the same result
            import warnings
            warnings.warn(f"symmetric-memory push unavailable ({err!r}); using the NCCL all-gather")
    return _Gather(bounds, rank, width, device, group), "nccl"


class _GraphedStep:
    """CUDA-graph replay of one whole step (product kernels, push kernel, barrier).

    At several GPUs a step is a few tens of microseconds of device work behind four launches, which the
    host cannot issue that fast one by one; replaying them as one graph keeps the step device-bound.
    Only the symmetric-memory modes are captured (their launches are all plain kernels on one stream).
    """

    _graph = None
    _step_launches = None
    _captured_launches = 0
    _product_graph = None
    _out = None
    _group = None

    def reassemble_in_kernel(self, on: bool) -> None:
        """Registers (or clears) the other ranks' buffers as mirrors of the local output (fused / multicast)."""
        if self._out is None or self.gather_mode not in ("fused", "multicast"):
            return
        if not on:
            self._out.set_mirrors([])
        elif self.gather_mode == "multicast":
            self._out.set_multicast_mirror(self.gather.multicast_ptr)
        else:
            self._out.set_mirrors(self.gather.mirror_ptrs)
        # ACLSPARSE_SHARDED_FUSED_BARRIER=1: the step's barrier rides on the product's last kernel (its
        # closing barrier) on every rank that launches a product; a rank without rows launches the barrier
        # kernel.  Off by default: measured on 4 GPUs the step is 3 to 6 us SLOWER that way (c2 60.7 against
        # 57.1 us, c3 218 against 212 us): every CTA ends with a system-scope fence that waits for its
        # multimem stores to be acknowledged, and the last CTA's ticket and the flag exchange come after that
        # wait instead of overlapping the kernel's drain.
        fuse = on and self.r1 > self.r0 and os.environ.get("ACLSPARSE_SHARDED_FUSED_BARRIER", "0") == "1"
        g = self.gather
        if fuse:
            self._out.set_closing_barrier(g.barrier_state.data_ptr(), g.barrier_peers, g.world, g.rank)
        else:
            self._out.set_closing_barrier(0, None, 0, 0)
        g.barrier_in_kernel = fuse

    def _capture(self, body):
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        self.handle.set_stream(side.cuda_stream)
        try:
            with torch.cuda.stream(side):
                # A plan belongs to the stream it was built on: preprocess again on this one, so that the
                # captured step holds the product kernels only, then run once eagerly so that nothing
                # lazy (and no unanswered question about the matrix) is left for the capture.
                if self.r1 > self.r0:
                    self.op.preprocess(1.0, 0.0)
                body()
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = int(L.lib().aclsp_b200_kernel_launches())
            with torch.cuda.graph(graph, stream=side):
                body()
            self._captured_launches = int(L.lib().aclsp_b200_kernel_launches()) - before
        finally:
            self.handle.set_stream(torch.cuda.current_stream().cuda_stream)
        return graph

    def capture(self, alpha: float, beta: float) -> bool:
        """Records ``step(alpha, beta)`` into a graph that later ``step`` calls with the same scalars replay."""
        if self._product is not None or (self.world > 1 and self.gather_mode == "nccl"):
            return False
        self._graph = (self._capture(lambda: self._eager_step(alpha, beta)), float(alpha), float(beta))
        self._step_launches = self._captured_launches
        return True

    def capture_product(self, alpha: float, beta: float):
        """The local product alone (no reassembly step) as a graph; returns a callable that replays it."""
        if self._product is not None or self.r1 <= self.r0:
            return None
        graph = self._capture(lambda: self.op(alpha, beta))
        self._product_graph = graph  # kept alive with the operator
        return graph.replay

    # ---- what the benchmark reports about the operator
    def launches_per_step(self, alpha: float, beta: float) -> int:
        """Kernels of this library launched per step on this rank, counted by the library itself: the launches
        recorded into the step's graph, or those of one eager step where the step is not captured."""
        if self._graph is not None and self._step_launches is not None:
            return self._step_launches
        before = int(L.lib().aclsp_b200_kernel_launches())
        self._eager_step(alpha, beta)
        return int(L.lib().aclsp_b200_kernel_launches()) - before

    # ---- inputs that arrive from the host: every rank uploads one share, the shares are all-gathered
    def pinned_input_share(self, cfg: dict) -> torch.Tensor:
        """This rank's share of x (or of the rows of B) in pinned host memory, padded to the common share size."""
        src = torch.from_numpy(cfg["x"] if self.kind == "spmv" else cfg["b"])
        lo = min(self.rank * self._share, src.shape[0])
        hi = min(lo + self._share, src.shape[0])
        out = torch.zeros((self._share,) + tuple(src.shape[1:]), dtype=torch.float32).pin_memory()
        out[: hi - lo].copy_(src[lo:hi])
        return out

    def load_input_share(self, host_share: torch.Tensor) -> None:
        """Host -> device copy of this rank's share, then the all-gather that completes every replica."""
        lo = self.rank * self._share
        mine = self._input_pad[lo:lo + self._share]
        mine.copy_(host_share, non_blocking=True)
        if self.world > 1:
            dist.all_gather_into_tensor(self._input_pad.view(-1), mine.reshape(-1), group=self._group)

    def _make_input(self, full: np.ndarray, device) -> torch.Tensor:
        """Replica of x / B inside a buffer padded to world_size equal shares; returns the unpadded view."""
        rows = full.shape[0]
        self._share = (rows + self.world - 1) // self.world
        self._input_pad = torch.zeros((self._share * self.world,) + tuple(full.shape[1:]), dtype=torch.float32,
                                      device=device)
        view = self._input_pad[:rows]
        view.copy_(torch.from_numpy(full))
        return view

    def close(self) -> None:
        """Drops graphs, descriptors and device arrays (the benchmark measures several operators in one process)."""
        self._graph = None
        self._product_graph = None
        for name in ("op", "mat", "handle", "gather", "d_ptr", "d_col", "d_val", "x", "b", "y_local", "c_local",
                     "_input_pad", "_out"):
            if hasattr(self, name):
                setattr(self, name, None)

    def step(self, alpha: float, beta: float) -> torch.Tensor:
        """One product: local row block, then the reassembly; returns the full result (identical on every rank)."""
        if self._graph is not None and self._graph[1:] == (float(alpha), float(beta)):
            self._graph[0].replay()
            return self.gather.full if self.world > 1 else self.gather.local
        return self._eager_step(alpha, beta)


class ShardedSpMV(_GraphedStep):
    """y = alpha * A * x + beta * y with A row-block sharded over the ranks of ``group``.

    ``local_product(local_csr, x, y_local, alpha, beta)`` computes one rank's slice; by default it is
    the single-GPU C API.  (The multi-process CPU tests inject a stand-in here to exercise the
    partition / gather logic without a GPU; there is no CPU implementation in this package.)
    """

    def __init__(self, cfg: dict, rank: int, world: int, device, group=None, local_product=None, gather="multicast"):
        self.rank, self.world, self.device, self._group = rank, world, device, group
        self.kind = "spmv"
        self.algorithm = "exact fp32 products (hi + lo), fp64 row sums"
        self.kernel_names = "SpmvRowBlockKernel + SpmvTileKernel + SpmvCarryFixupKernel"
        base = cfg.get("index_base", 0)
        self.bounds = align_bounds(row_block_bounds_host(cfg["row_ptr"], cfg["nnz"], world, base), 32)
        self.local_ptr, self.local_col, self.local_val = shard_csr(cfg["row_ptr"], cfg["col_ind"], cfg["values"],
                                                                   self.bounds, rank, base)
        self.r0, self.r1 = int(self.bounds[rank]), int(self.bounds[rank + 1])
        self.gather, self.gather_mode = _make_gather(gather, self.bounds, rank, 1, device, group)
        self.x = self._make_input(cfg["x"], device)
        self.y_local = self.gather.local
        self.y_local.copy_(torch.from_numpy(cfg["y"][self.r0:self.r1]).to(device))
        self._product = local_product
        if local_product is None:
            from . import api
            self.d_ptr = torch.from_numpy(self.local_ptr).to(device)
            self.d_col = torch.from_numpy(np.ascontiguousarray(self.local_col)).to(device)
            self.d_val = torch.from_numpy(np.ascontiguousarray(self.local_val)).to(device)
            self.handle = api.Handle()
            self.mat = api.CsrMatrix(self.r1 - self.r0, cfg["cols"], self.d_ptr, self.d_col, self.d_val, base,
                                     nnz=int(self.local_col.size))
            self.op = api.SpMV(self.handle, self.mat, api.DnVec(self.x), api.DnVec(self.y_local,
                                                                                   size=self.r1 - self.r0))
            self._out = self.op.y
            self.reassemble_in_kernel(True)
            if self.r1 > self.r0:
                self.op.preprocess()

    def _eager_step(self, alpha: float, beta: float) -> torch.Tensor:
        if self._product is not None:
            self._product((self.local_ptr, self.local_col, self.local_val), self.x, self.y_local, alpha, beta)
        elif self.r1 > self.r0:
            self.op(alpha, beta)
        return self.gather.run()


class ShardedSpMM(_GraphedStep):
    """C = alpha * A * B + beta * C (row-major B and C) with A row-block sharded over the ranks."""

    def __init__(self, cfg: dict, rank: int, world: int, device, group=None, local_product=None, gather="multicast",
                 alg: int = L.SPMM_ALG_DEFAULT):
        self.rank, self.world, self.device, self._group = rank, world, device, group
        self.kind = "spmm"
        self.algorithm = "fp64 products, fp64 row sums (every algorithm value)"
        self.kernel_names = "SpmmTileKernel + SpmmCarryFixupKernel"
        base = cfg.get("index_base", 0)
        n = cfg["n"]
        self.bounds = row_block_bounds_host(cfg["row_ptr"], cfg["nnz"], world, base)
        self.local_ptr, self.local_col, self.local_val = shard_csr(cfg["row_ptr"], cfg["col_ind"], cfg["values"],
                                                                   self.bounds, rank, base)
        self.r0, self.r1 = int(self.bounds[rank]), int(self.bounds[rank + 1])
        self.gather, self.gather_mode = _make_gather(gather, self.bounds, rank, n, device, group)
        self.b = self._make_input(cfg["b"], device)
        self.c_local = self.gather.local
        self.c_local.copy_(torch.from_numpy(cfg["c"][self.r0:self.r1]).to(device))
        self._product = local_product
        if local_product is None:
            from . import api
            self.d_ptr = torch.from_numpy(self.local_ptr).to(device)
            self.d_col = torch.from_numpy(np.ascontiguousarray(self.local_col)).to(device)
            self.d_val = torch.from_numpy(np.ascontiguousarray(self.local_val)).to(device)
            self.handle = api.Handle()
            rows = self.r1 - self.r0
            self.mat = api.CsrMatrix(rows, cfg["cols"], self.d_ptr, self.d_col, self.d_val, base,
                                     nnz=int(self.local_col.size))
            if rows > 0:
                self.op = api.SpMM(self.handle, self.mat, api.DnMat(cfg["cols"], n, n, self.b),
                                   api.DnMat(rows, n, n, self.c_local), alg=alg)
                self._out = self.op.c
                self.reassemble_in_kernel(True)
                self.op.preprocess()

    def _eager_step(self, alpha: float, beta: float) -> torch.Tensor:
        if self._product is not None:
            self._product((self.local_ptr, self.local_col, self.local_val), self.b, self.c_local, alpha, beta)
        elif self.r1 > self.r0:
            self.op(alpha, beta)
        return self.gather.run()


def init_process_group_from_env(backend: "str | None" = None):
    """RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* from the environment (torchrun); returns (rank, world, device)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    device = torch.device(f"cuda:{local}") if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group(backend or ("nccl" if cuda else "gloo"), rank=rank, world_size=world)
    return rank, world, device


__all__ = ["row_block_bounds_host", "shard_csr", "ShardedSpMV", "ShardedSpMM", "init_process_group_from_env", "L"]
