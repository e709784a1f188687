"""Same surface as GLakeServe/vmm_allocator/vmm_allocator.py:5-19."""
from .. import vmmAllocator


class KV_cache:
    """One layer's K (or V) pointer table: ``.kv_cache`` is the table object,
    ``.vmm_ptr`` its device address as an int, ``.layer_index`` the layer."""

    def __init__(self, max_seqs, layer_index: int) -> None:
        self.max_seqs = max_seqs
        self.layer_index = layer_index
        self.kv_cache = vmmAllocator.KVCache(self.max_seqs)
        self.vmm_ptr = self.kv_cache.getKVCachePtr()
