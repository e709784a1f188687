"""glake_b200 — the vTensor decode hot path of GLakeServe for B200 (sm_100a).

Modules mirror the reference's interfaces for this path:
  vmmAllocator            the pybind module of GLakeServe/vmm_allocator
  vmm_allocator           the KV_cache wrapper (vmm_allocator/vmm_allocator.py)
  ops                     reshape_and_cache / paged_attention_v1 / fwd_kvcache
  backend                 attention-backend binding, cache engine, step driver
Everything runs in libvtensor.so (hand-written CUDA + a C++ VMM allocator); the
package raises at import when that library has not been built.
"""
from . import _lib  # noqa: F401  (raises ImportError when libvtensor.so is missing)
from ._lib import VTensorError  # noqa: F401

__all__ = ["VTensorError"]
