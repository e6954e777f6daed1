"""oneccl_b200: a Blackwell-native collective communication library with the
capabilities of oneCCL.

Layers (bottom to top):

* ``csrc/``               native runtime: KVS bootstrap, CPU transport / scheduler /
                          algorithms, symmetric heap, sm_100a collective and fused GEMM kernels,
                          the ``ccl::`` C++ API (``csrc/include/oneapi/ccl.hpp``) and a flat C API;
* ``oneccl_b200.ops``     Python wrappers of the device kernels;
* ``oneccl_b200.comm``    communicators, KVS, CPU and GPU collectives on tensors;
* ``oneccl_b200.parallel`` data / tensor / expert / pipeline parallel building blocks;
* ``oneccl_b200.models``  the benchmark models (GPT-2, TP MLP block, MoE layer);
* ``oneccl_b200.torch_backend`` the ``torch.distributed`` backend named ``ccl``.
"""
from ._lib import CclError, load  # noqa: F401

__version__ = "0.1.0"
