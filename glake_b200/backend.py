"""Host-side mirror of the reference's vTensor attention backend for decode:

* :class:`VTensorCacheEngine`  – what ``CacheEngine.__init__`` builds
  (GLakeServe/vllm/worker/cache_engine.py:53-129): one ``KVcacheSegment`` per
  sequence slot, one K and one V pointer table per layer, and the same base
  addresses as int64 device tensors for the append op.
* :class:`VTensorMetadata`     – the vTensor fields of ``XFormersMetadata``
  (GLakeServe/vllm/attention/backends/xformers.py:65-127).
* :func:`prepare_step`         – the allocator work ``LlamaModel.forward`` does
  before the layer loop (GLakeServe/vllm/model_executor/models/llama.py:307-341).
* :class:`VTensorAttentionImpl` – ``XFormersImpl.forward`` for the decode branch
  (xformers.py:269-433): append via ``reshape_and_cache``, then ``fwd_kvcache``.

PyTorch supplies device memory and the current stream; the work is done by the
CUDA kernels behind :mod:`glake_b200.ops`.
"""
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from . import ops, vmmAllocator
from .vmm_allocator.vmm_allocator import KV_cache

PHY_GRAN = vmmAllocator.granularitySize


def _round_up(x, m):
    return (x + m - 1) // m * m


class VTensorCacheEngine:
    def __init__(self, num_layers, num_kv_heads, head_size, max_num_seqs, max_num_batched_tokens,
                 cache_dtype="auto", cache_seqs=0, cache_tokens=0, device="cuda"):
        self.num_layers, self.num_kv_heads, self.head_size = num_layers, num_kv_heads, head_size
        self.cache_dtype = cache_dtype
        self.dtype_size = 1 if cache_dtype in ("fp8", "fp8_e4m3") else 2
        self.device = torch.device(device)
        self.token_size = num_kv_heads * head_size * self.dtype_size
        # cache_engine.py:55-57: room for max_num_batched_tokens rows, whole chunks
        self.max_context_size = _round_up(max_num_batched_tokens * self.token_size, PHY_GRAN)
        self.kv_batch_stride = self.max_context_size
        self.vmm_kvcache_segment = []
        cache_token_size = PHY_GRAN * cache_tokens
        for index in range(max_num_seqs):
            if cache_seqs > 0:
                seg = vmmAllocator.KVcacheSegment(num_layers, self.max_context_size, cache_token_size,
                                                  index < cache_seqs)
            else:
                seg = vmmAllocator.KVcacheSegment(num_layers, self.max_context_size, 0, False)
            self.vmm_kvcache_segment.append(seg)
        # per layer (K table, V table)  — cache_engine.py:111-129
        self.gpu_cache = [(KV_cache(max_num_seqs, i), KV_cache(max_num_seqs, i)) for i in range(num_layers)]
        vmmAllocator.copy_kv_cache([k.kv_cache for k, _ in self.gpu_cache], [v.kv_cache for _, v in self.gpu_cache],
                                   self.vmm_kvcache_segment)
        # the same addresses as int64 tensors for reshape_and_cache — cache_engine.py:98-109
        self.k_cache_ptr, self.v_cache_ptr = [], []
        for layer in range(num_layers):
            kp = [s.getKeyDevicePtr(layer) for s in self.vmm_kvcache_segment]
            vp = [s.getValueDevicePtr(layer) for s in self.vmm_kvcache_segment]
            self.k_cache_ptr.append(torch.tensor(kp, dtype=torch.int64, device=self.device))
            self.v_cache_ptr.append(torch.tensor(vp, dtype=torch.int64, device=self.device))

    def close(self):
        for k, v in self.gpu_cache:
            k.kv_cache.close()
            v.kv_cache.close()
        for s in self.vmm_kvcache_segment:
            s.close()
        self.gpu_cache, self.vmm_kvcache_segment = [], []


@dataclass
class VTensorMetadata:
    """Per-step inputs of the backend.  ``slot_mapping_list[i]`` is the slot of
    batch entry i, ``seq_lens`` the context lengths INCLUDING this step's tokens."""
    slot_mapping_list: List[int]
    seq_lens: List[int]
    kv_num_heads: int
    kv_head_size: int
    num_prefills: int = 0
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0
    max_query_len: int = 1
    set_used_size: Optional[List[int]] = None
    extend_seq_list: List[int] = field(default_factory=list)
    kv_elem_size: int = 2
    # filled by prepare_step
    slot_mapping: Optional[torch.Tensor] = None      # int64 [B] slot ids (device)
    seq_lens_tensor: Optional[torch.Tensor] = None   # int32 [B] (device)
    cache_seq_lens: Optional[torch.Tensor] = None    # int32 [B] prefill source-row offsets
    slot_m: Optional[torch.Tensor] = None            # int64 [B] destination byte offsets
    max_seq_len: int = 0
    k_cache_segment_ptr_list: Optional[list] = None
    v_cache_segment_ptr_list: Optional[list] = None
    kvcache_segment: Optional[list] = None


def prepare_step(meta: VTensorMetadata, engine: VTensorCacheEngine, device=None):
    """Allocator work of one model step, before the layer loop (llama.py:307-341):
    wait (bounded) for growths that this step needs, queue the next ones, obtain
    each entry's byte offset, upload the small per-step tensors."""
    device = device or engine.device
    slots = meta.slot_mapping_list
    segs = [engine.vmm_kvcache_segment[s] for s in slots]
    meta.kvcache_segment = segs
    meta.k_cache_segment_ptr_list = engine.k_cache_ptr
    meta.v_cache_segment_ptr_list = engine.v_cache_ptr
    kv_size = meta.kv_num_heads * meta.kv_head_size * meta.kv_elem_size
    decode = meta.num_prefills == 0
    if decode:
        if vmmAllocator.query_cycle(slots):
            vmmAllocator.wait_ready(slots)
        kv_size_list = [kv_size] * len(slots)
        for seg, slot_id in zip(segs, meta.extend_seq_list):
            if slot_id != -1:
                seg.eagerExtend(kv_size, slot_id)
        rows = [1] * len(slots)
    else:
        rows = meta.query_lens if getattr(meta, "query_lens", None) else meta.seq_lens
        kv_size_list = [n * kv_size for n in rows]
    set_used = meta.set_used_size if meta.set_used_size is not None else [0] * len(slots)
    slot_m = vmmAllocator.extend_kv_cache_batch(None, None, slots, kv_size_list, segs, set_used, kv_size, decode)
    # one small pinned staging buffer -> one H2D copy for all per-step integers
    n = len(slots)
    starts, acc = [], 0
    for r in rows:
        starts.append(acc)
        acc += r
    host = torch.tensor(slot_m + list(slots) + list(meta.seq_lens) + starts, dtype=torch.int64).pin_memory()
    dev = host.to(device, non_blocking=True)
    meta.slot_m = dev[:n]
    meta.slot_mapping = dev[n:2 * n]
    meta.seq_lens_tensor = dev[2 * n:3 * n].to(torch.int32)
    meta.cache_seq_lens = dev[3 * n:4 * n].to(torch.int32)
    meta.max_seq_len = max(meta.seq_lens) if meta.seq_lens else 0
    return meta


class VTensorAttentionImpl:
    """Decode branch of the reference's ``XFormersImpl`` on the vTensor layout."""

    def __init__(self, num_heads, head_size, scale, num_kv_heads=None, kv_cache_dtype="auto"):
        self.num_heads, self.head_size, self.scale = num_heads, head_size, float(scale)
        self.num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        self.kv_cache_dtype = kv_cache_dtype
        assert self.num_heads % self.num_kv_heads == 0
        if head_size != 128:
            raise ValueError("head size 128 only")

    def forward(self, query, key, value, key_cache: KV_cache, value_cache: KV_cache, attn_metadata: VTensorMetadata,
                kv_scale: float = 1.0, k_scale=None, v_scale=None):
        """query ``[tokens, H*D]``, key/value ``[tokens, KVH*D]`` -> ``[tokens, H*D]``."""
        query = query.view(-1, self.num_heads, self.head_size)
        key = key.view(-1, self.num_kv_heads, self.head_size)
        value = value.view(-1, self.num_kv_heads, self.head_size)
        m = attn_metadata
        if m.num_prefills > 0:
            raise NotImplementedError("prefill goes through glake_b200.prefill")
        layer = key_cache.layer_index
        ops.reshape_and_cache(key, value, m.k_cache_segment_ptr_list[layer], m.v_cache_segment_ptr_list[layer],
                              m.slot_m, m.slot_mapping, m.seq_lens_tensor, m.cache_seq_lens, 1,
                              self.num_kv_heads, self.head_size, self.kv_cache_dtype, k_scale, v_scale)
        output, _ = ops.fwd_kvcache(query.unsqueeze(1), key_cache.vmm_ptr, value_cache.vmm_ptr, m.max_seq_len,
                                    self.num_kv_heads, m.slot_mapping.size(0), m.slot_mapping, None, None,
                                    m.seq_lens_tensor, None, None, None, None, None, None, self.scale, True, -1, -1,
                                    None, 4, kv_cache_dtype=self.kv_cache_dtype, k_scale=k_scale, v_scale=v_scale)
        return output.view(-1, self.num_heads * self.head_size)
