"""triton_distributed_b200: a Blackwell-native compute/communication overlap library.

PyTorch is the framework layer; every hot op is a hand-written sm_100a CUDA kernel (tcgen05/TMEM GEMMs
fed by TMA, P2P and NVLS ``multimem`` traffic issued from inside the kernels) on top of a symmetric heap
built from cuMem handles and an NVLS multicast object.  The Python API keeps the names of the
Triton-distributed library it replaces (``initialize_distributed``, ``create_ag_gemm_context`` /
``ag_gemm``, ``create_gemm_rs_context`` / ``gemm_rs``, ``all_reduce`` ...).

The importable package name uses an underscore because a hyphen is not a legal Python identifier.
"""
from .runtime import (  # noqa: F401
    DistConfig,
    CommTimeoutError,
    initialize_distributed,
    finalize_distributed,
    get_runtime,
    symm_tensor,
    symm_tensors,
    symm_free,
    nvshmem_create_tensor,
    nvshmem_create_tensors,
    nvshmem_free_tensor_sync,
    nvshmem_barrier_all_on_stream,
    barrier_all_on_stream,
)
from . import ops, parallel, models, utils  # noqa: F401

__version__ = "0.1.0"
