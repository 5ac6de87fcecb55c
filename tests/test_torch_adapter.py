"""The PyTorch adapter: argument checks on CPU (no launch is reached), results on the GPU.

Follows the reference's adapter tests (test/spmm/python/test_torch_extension.py, which drive the extension with
mocked device tensors to pin the argument checks, and its on-device cases that compare with a dense product).
"""
import numpy as np
import pytest
import torch

from ops_sparse_b200 import torch_adapter as TA


def _csr_cpu(rows=4, cols=5):
    dense = torch.arange(rows * cols, dtype=torch.float32).reshape(rows, cols) % 3
    return dense.to_sparse_csr()


def test_mv_argument_checks_come_before_any_launch():
    mat = _csr_cpu()
    vec = torch.ones(5)
    with pytest.raises(ValueError, match="sparse CSR layout"):
        TA.mv(mat.to_dense(), vec)
    with pytest.raises(ValueError, match="CUDA device"):
        TA.mv(mat, vec)  # a CPU tensor is refused: there is no host implementation behind the adapter
    with pytest.raises(TypeError, match="defined tensor"):
        TA.mv(None, vec)


def test_array_entry_argument_checks():
    rp = torch.tensor([0, 1, 2], dtype=torch.int32)
    ci = torch.tensor([0, 1], dtype=torch.int32)
    va = torch.ones(2)
    x, y = torch.ones(2), torch.zeros(2)
    with pytest.raises(ValueError, match="CUDA tensor"):
        TA.spmv_csr(rp, ci, va, x, y)
    with pytest.raises(ValueError, match="CUDA tensor"):
        TA.spmv_workspace(rp, ci, va, x, y)


@pytest.mark.gpu
def test_array_entry_checks_on_device_tensors():
    dev = "cuda:0"
    rp = torch.tensor([0, 1, 2], dtype=torch.int32, device=dev)
    ci = torch.tensor([0, 1], dtype=torch.int32, device=dev)
    va = torch.ones(2, device=dev)
    x, y = torch.ones(2, device=dev), torch.zeros(2, device=dev)
    with pytest.raises(TypeError, match="int32"):
        TA.spmv_csr(rp.long(), ci, va, x, y)
    with pytest.raises(ValueError, match="length mismatch"):
        TA.spmv_csr(rp, ci[:1], va, x, y)
    with pytest.raises(ValueError, match="base must be 0 or 1"):
        TA.spmv_csr(rp, ci, va, x, y, base=2)
    with pytest.raises(ValueError, match="trans must be N, T or H"):
        TA.spmv_csr(rp, ci, va, x, y, trans="X")
    with pytest.raises(ValueError, match="x is too small"):
        TA.spmv_csr(rp, ci, va, x[:1], y, cols=2)
    with pytest.raises(ValueError, match="y is too small"):
        TA.spmv_csr(rp, ci, va, x, y[:1])
    assert TA.spmv_workspace(rp, ci, va, x, y) > 0
    out = TA.spmv_csr(rp, ci, va, x, y, alpha=2.0, beta=0.0)
    torch.cuda.synchronize()
    assert out.data_ptr() == y.data_ptr() and y.tolist() == [2.0, 2.0]
    # transposed products go through the same entry (the adapter passes op(A) on to the library)
    rp3 = torch.tensor([0, 2, 3], dtype=torch.int32, device=dev)   # the reference's 2 x 3 fixture
    ci3 = torch.tensor([0, 2, 1], dtype=torch.int32, device=dev)
    va3 = torch.tensor([2.0, 3.0, 4.0], device=dev)
    xt, yt = torch.tensor([1.0, 2.0], device=dev), torch.ones(3, device=dev)
    for trans in ("T", "H"):
        yt.fill_(1.0)
        TA.spmv_csr(rp3, ci3, va3, xt, yt, alpha=2.0, beta=3.0, trans=trans)
        torch.cuda.synchronize()
        assert yt.tolist() == [7.0, 19.0, 9.0]


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols,density", [(1, 1, 1.0), (257, 193, 0.05), (4096, 4096, 0.004), (50, 3000, 0.3)])
def test_mv_and_addmm_match_the_oracle_and_torch(rows, cols, density):
    from oracle import oracle as O
    gen = torch.Generator().manual_seed(rows * 7 + cols)
    dense = torch.rand(rows, cols, generator=gen) * 2 - 1
    dense[torch.rand(rows, cols, generator=gen) > density] = 0
    mat = dense.to_sparse_csr().cuda()  # int64 indices, as PyTorch builds them
    rp = mat.crow_indices().cpu().numpy().astype(np.int32)
    ci = mat.col_indices().cpu().numpy().astype(np.int32)
    va = mat.values().cpu().numpy()
    vec = torch.rand(cols, generator=gen) * 2 - 1
    y = TA.mv(mat, vec.cuda())
    truth = O.spmv_f64(rp, ci, va, vec.numpy(), np.zeros(rows, np.float32), 1.0, 0.0)
    assert O.check_tolerance(y.cpu().numpy(), truth)[0] == 0
    n = 64
    b = torch.rand(cols, n, generator=gen) * 2 - 1
    c0 = torch.rand(rows, n, generator=gen)
    got = TA.addmm(c0.cuda(), mat, b.cuda(), beta=0.5, alpha=1.5)
    want = 0.5 * c0.double() + 1.5 * (dense.double() @ b.double())
    assert got.shape == (rows, n)
    scale = (dense.abs().double() @ b.abs().double()) * 1.5 + 0.5 * c0.abs().double()
    bound = (cols + 4) * 2.0 ** -24 * scale + 1e-6  # forward bound of plain fp32 accumulation (the default SpMM)
    assert bool(((got.cpu().double() - want).abs() <= bound).all())
    assert torch.allclose(TA.mm(mat, b.cuda()).cpu().double(), dense.double() @ b.double(), rtol=1e-4, atol=1e-4)


@pytest.mark.gpu
def test_empty_shapes():
    mat = torch.zeros(0, 5).to_sparse_csr().cuda()
    assert TA.mv(mat, torch.ones(5, device="cuda")).shape == (0,)
    mat = torch.zeros(3, 5).to_sparse_csr().cuda()
    assert TA.mv(mat, torch.ones(5, device="cuda")).tolist() == [0.0, 0.0, 0.0]
    out = TA.addmm(torch.ones(3, 2, device="cuda"), mat, torch.ones(5, 2, device="cuda"), beta=2.0)
    assert out.tolist() == [[2.0, 2.0]] * 3
