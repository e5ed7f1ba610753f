"""ps_lite_b200: a Blackwell-native parameter server with the capabilities of dmlc/ps-lite.

Layers (bottom to top):

* ``libpsb200_device.so`` (``src/kernels``, ``src/device``): sm_100a CUDA data plane --
  symmetric heap, fused push/pull kernels, sparse tables, the tcgen05 GEMM fused with pull.
* ``libpsb200_core.so`` (``src/core``, ``src/van``): C++17 host runtime with the reference's
  public API (``include/ps``): Postoffice, Customer, vans, KVWorker/KVServer, SimpleApp.
* :mod:`ps_lite_b200.parallel`: torch-facing objects built on both.
* :mod:`ps_lite_b200.models`: the workloads used by the benchmarks.
"""
from . import _lib  # noqa: F401

__version__ = "0.1.0"
