"""B200-native CSR SpMV / SpMM behind the aclsparse C API.

``libops_sparse.so`` (built from ``csrc/``) is the product; this package is the
thin Python layer over it:

  _lib       ctypes binding of the C ABI (fails loudly when the library is missing)
  api        handle / descriptor / three-phase operator wrappers for CUDA tensors
  sharded    row-block sharding over several GPUs (one process per GPU, NCCL)
  workloads  seeded synthetic inputs of the benchmark configurations
"""
from . import _lib  # noqa: F401

__all__ = ["_lib", "api", "sharded", "workloads"]
