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
import time
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from . import ops, vmmAllocator
from .vmm_allocator.vmm_allocator import KV_cache



class nvtx_range:
    """NVTX range on the host timeline, as the reference puts around the allocator wait, the
    growth requests and each layer's attention (GLakeServe/vllm/model_executor/models/llama.py:242-261,
    :323-337); a no-op where CUDA is not initialised."""

    def __init__(self, name):
        self.name = name
        self.on = torch.cuda.is_available() and torch.cuda.is_initialized()

    def __enter__(self):
        if self.on:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if self.on:
            torch.cuda.nvtx.range_pop()


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
        self.max_context_size = _round_up(max_num_batched_tokens * self.token_size, vmmAllocator.granularitySize)
        self.kv_batch_stride = self.max_context_size
        self.vmm_kvcache_segment = []
        cache_token_size = vmmAllocator.granularitySize * cache_tokens
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

    def prefill_maps(self, layer):
        """TMA tensor maps of this layer's ranges for ``ops.prefill_attention(..., maps=...)``
        (built on first use; None when the kv-head count or cache dtype rules the path out)."""
        if self.dtype_size != 2 or not ops.prefill_tma_supported(self.num_kv_heads):
            return None
        if not hasattr(self, "_prefill_maps"):
            self._prefill_maps = {}
        if layer not in self._prefill_maps:
            segs = self.vmm_kvcache_segment
            self._prefill_maps[layer] = ops.prefill_maps(
                [s.getKeyDevicePtr(layer) for s in segs], [s.getValueDevicePtr(layer) for s in segs],
                self.num_kv_heads, self.head_size, self.max_context_size // self.token_size, self.device)
        return self._prefill_maps[layer]

    def decode_maps(self, layer, num_heads):
        """TMA tensor maps of this layer's fp8 ranges for ``ops.decode_step(..., maps=...)`` (the
        tcgen05 decode kernel; built on first use; None when the shape or cache dtype rules it out)."""
        if self.dtype_size != 1 or not ops.decode_tma_supported(num_heads, self.num_kv_heads, "fp8_e4m3"):
            return None
        if not hasattr(self, "_decode_maps"):
            self._decode_maps = {}
        if layer not in self._decode_maps:
            segs = self.vmm_kvcache_segment
            self._decode_maps[layer] = ops.decode_maps(
                [s.getKeyDevicePtr(layer) for s in segs], [s.getValueDevicePtr(layer) for s in segs],
                self.num_kv_heads, self.head_size, self.max_context_size // self.token_size, self.device)
        return self._decode_maps[layer]

    def close(self):
        self._prefill_maps = {}
        self._decode_maps = {}
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
    query_lens: Optional[List[int]] = None           # prefill: NEW tokens per entry (default: seq_lens, i.e. no prefix)
    # filled by prepare_step
    slot_mapping: Optional[torch.Tensor] = None      # int64 [B] slot ids (device)
    seq_lens_tensor: Optional[torch.Tensor] = None   # int32 [B] (device)
    cache_seq_lens: Optional[torch.Tensor] = None    # int32 [B] prefill source-row offsets
    query_lens_tensor: Optional[torch.Tensor] = None # int32 [B] rows each entry appends (1 for decode)
    slot_m: Optional[torch.Tensor] = None            # int64 [B] destination byte offsets
    max_seq_len: int = 0
    k_cache_segment_ptr_list: Optional[list] = None
    v_cache_segment_ptr_list: Optional[list] = None
    kvcache_segment: Optional[list] = None


def prepare_step_host(meta: VTensorMetadata, engine: VTensorCacheEngine):
    """Host half of the allocator work of one model step (llama.py:307-341): wait
    (bounded) for growths this step needs, queue the next ones, obtain each entry's
    byte offset.  Returns (byte offsets, source-row starts) as Python lists."""
    slots = meta.slot_mapping_list
    segs = [engine.vmm_kvcache_segment[s] for s in slots]
    meta.kvcache_segment = segs
    meta.k_cache_segment_ptr_list = engine.k_cache_ptr
    meta.v_cache_segment_ptr_list = engine.v_cache_ptr
    kv_size = meta.kv_num_heads * meta.kv_head_size * meta.kv_elem_size
    decode = meta.num_prefills == 0
    if decode:
        if vmmAllocator.query_cycle(slots):
            with nvtx_range("sync phy memory"):
                vmmAllocator.wait_ready(slots)
        kv_size_list = [kv_size] * len(slots)
        with nvtx_range("eager_extend"):
            for seg, slot_id in zip(segs, meta.extend_seq_list):
                if slot_id != -1:
                    seg.eagerExtend(kv_size, slot_id)
        rows = [1] * len(slots)
    else:
        rows = meta.query_lens if meta.query_lens else meta.seq_lens
        kv_size_list = [n * kv_size for n in rows]
    set_used = meta.set_used_size if meta.set_used_size is not None else [0] * len(slots)
    slot_m = vmmAllocator.extend_kv_cache_batch(None, None, slots, kv_size_list, segs, set_used, kv_size, decode)
    starts, acc = [], 0
    for r in rows:
        starts.append(acc)
        acc += r
    meta.max_seq_len = max(meta.seq_lens) if meta.seq_lens else 0
    meta.max_query_len = max(rows) if rows else 0
    meta._rows = list(rows)
    return slot_m, starts


def prepare_step(meta: VTensorMetadata, engine: VTensorCacheEngine, device=None):
    """prepare_step_host plus the upload of the small per-step tensors (the
    reference's ``torch.tensor(slot_m, device="cuda")``, llama.py:341) in one copy."""
    device = device or engine.device
    slot_m, starts = prepare_step_host(meta, engine)
    slots = meta.slot_mapping_list
    n = len(slots)
    host = torch.tensor(slot_m + list(slots) + list(meta.seq_lens) + starts + meta._rows, dtype=torch.int64).pin_memory()
    dev = host.to(device, non_blocking=True)
    meta.slot_m = dev[:n]
    meta.slot_mapping = dev[n:2 * n]
    meta.seq_lens_tensor = dev[2 * n:3 * n].to(torch.int32)
    meta.cache_seq_lens = dev[3 * n:4 * n].to(torch.int32)
    meta.query_lens_tensor = dev[4 * n:5 * n].to(torch.int32)
    return meta


class VTensorAttentionImpl:
    """The reference's ``XFormersImpl`` on the vTensor layout: the decode branch
    (xformers.py:389-433) as one fused launch, and the prompt / prefix-extend branch
    (xformers.py:310-388) as multi-row append + causal attention over the range."""

    def __init__(self, num_heads, head_size, scale, num_kv_heads=None, kv_cache_dtype="auto"):
        self.num_heads, self.head_size, self.scale = num_heads, head_size, float(scale)
        self.num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        self.kv_cache_dtype = kv_cache_dtype
        assert self.num_heads % self.num_kv_heads == 0
        if head_size != 128:
            raise ValueError("head size 128 only")

    def forward(self, query, key, value, key_cache: KV_cache, value_cache: KV_cache, attn_metadata: VTensorMetadata,
                kv_scale: float = 1.0, k_scale=None, v_scale=None, prefill_maps=None, decode_maps=None):
        """query ``[tokens, H*D]``, key/value ``[tokens, KVH*D]`` -> ``[tokens, H*D]``.
        ``prefill_maps``: the layer's tensor-map table (``VTensorCacheEngine.prefill_maps``),
        used by the prompt branch when given; ``decode_maps``: the one of an fp8 cache for the
        decode branch (``VTensorCacheEngine.decode_maps``: the tcgen05 kernel).  ``k_scale`` / ``v_scale``: the layer's per-kv-head
        scales of an fp8 cache (``ops.kv_scales`` of the first prompt's rows, then frozen)."""
        with nvtx_range("vtensor attention: prompt" if attn_metadata.num_prefills > 0 else "vtensor attention: decode"):
            return self._forward(query, key, value, key_cache, value_cache, attn_metadata, k_scale, v_scale,
                                 prefill_maps, decode_maps)

    def _forward(self, query, key, value, key_cache, value_cache, attn_metadata, k_scale, v_scale, prefill_maps,
                 decode_maps=None):
        query = query.view(-1, self.num_heads, self.head_size)
        key = key.view(-1, self.num_kv_heads, self.head_size)
        value = value.view(-1, self.num_kv_heads, self.head_size)
        m = attn_metadata
        if m.num_prefills > 0:
            layer = key_cache.layer_index
            fp8 = self.kv_cache_dtype not in ("auto", "bf16", "bfloat16", None)
            if fp8:
                prefill_maps = None      # maps of the fp8 ranges do not apply: the kernels run on widened scratch
            # the new rows go into the ranges first (entry i: query_lens[i] rows from source row
            # cache_seq_lens[i]), then the new tokens attend over prefix + new tokens
            ops.reshape_and_cache(key, value, m.k_cache_segment_ptr_list[layer], m.v_cache_segment_ptr_list[layer],
                                  m.slot_m, m.slot_mapping, m.query_lens_tensor, m.cache_seq_lens,
                                  max(m.max_query_len, 2), self.num_kv_heads, self.head_size, self.kv_cache_dtype,
                                  k_scale, v_scale)
            output = torch.empty_like(query)
            ops.prefill_attention(output, query, key_cache.vmm_ptr, value_cache.vmm_ptr, self.num_kv_heads, self.scale,
                                  m.slot_mapping, m.seq_lens_tensor, m.query_lens_tensor, m.cache_seq_lens,
                                  m.max_query_len, maps=prefill_maps, kv_cache_dtype=self.kv_cache_dtype,
                                  k_scale=k_scale, v_scale=v_scale)
            return output.view(-1, self.num_heads * self.head_size)
        # append + attention of the layer as one fused step (one kernel launch for a
        # bf16 cache); equivalent to ops.reshape_and_cache followed by ops.fwd_kvcache
        output = torch.empty_like(query)
        ops.decode_step(output, query, key, value, key_cache.vmm_ptr, value_cache.vmm_ptr, m.slot_m, m.slot_mapping,
                        m.seq_lens_tensor, m.max_seq_len, self.num_kv_heads, self.scale, self.kv_cache_dtype,
                        k_scale, v_scale, maps=decode_maps)
        return output.view(-1, self.num_heads * self.head_size)


class DecodeRunner:
    """One decode step of the hot path over all layers, replayed as a CUDA graph.

    The reference captures its decode step in CUDA graphs as well
    (GLakeServe/vllm/worker/model_runner.py:782-930); what makes that possible on
    the vTensor layout is that a slot's K/V base addresses never change while it
    grows, so a captured kernel stays valid across steps.  Per step the host only
    does the allocator bookkeeping (and maps chunks when a sequence crosses a
    2 MiB boundary), writes ~24 bytes per sequence into a pinned staging buffer and
    replays.  ``host_io=True`` adds the copies of pinned host q/k/v to the device
    and of the outputs back to pinned host memory to the graph.
    """

    BUCKET = 2048  # graphs are keyed by max context rounded up to this many tokens

    def __init__(self, engine: VTensorCacheEngine, impl: VTensorAttentionImpl, batch, host_io=False,
                 k_scale=None, v_scale=None, overlap=True, post_layer=None, launches_per_post_layer=0):
        """``post_layer(layer)``, when given, is called on the runner's stream after every
        layer's attention, inside the captured graph: the place of what the model does
        between two attention layers, e.g. the tensor-parallel all-reduces after o_proj
        and down_proj (GLakeServe/vllm/model_executor/layers/linear.py:690-691)."""
        self.engine, self.impl, self.batch, self.host_io = engine, impl, batch, host_io
        self.post_layer, self.launches_per_post_layer = post_layer, launches_per_post_layer
        self.prepare_seconds = []     # host time of the allocator bookkeeping of each step
        # consecutive layers touch disjoint ranges: let layer l+1 start as layer l drains
        self.overlap = overlap and engine.num_layers > 1
        self.k_scale, self.v_scale = k_scale, v_scale
        dev, layers = engine.device, engine.num_layers
        hd, kd = impl.num_heads * impl.head_size, impl.num_kv_heads * impl.head_size
        self.q = torch.zeros(layers, batch, hd, dtype=torch.bfloat16, device=dev)
        self.k = torch.zeros(layers, batch, kd, dtype=torch.bfloat16, device=dev)
        self.v = torch.zeros(layers, batch, kd, dtype=torch.bfloat16, device=dev)
        self.out = torch.zeros(layers, batch, hd, dtype=torch.bfloat16, device=dev)
        # two pinned staging sets used alternately, so that the host can fill step n+1's
        # integers while step n still runs; each: byte offsets | slot ids, seq lens | row starts
        self.h64 = [torch.zeros(2 * batch, dtype=torch.int64).pin_memory() for _ in range(2)]
        self.h32 = [torch.zeros(2 * batch, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.staged = [None, None]   # event recorded after a staging set has been copied to the device
        self.n_steps = 0
        self.d64 = torch.zeros(2 * batch, dtype=torch.int64, device=dev)
        self.d32 = torch.zeros(2 * batch, dtype=torch.int32, device=dev)
        if host_io:
            self.hq, self.hk, self.hv = (torch.zeros_like(t, device="cpu").pin_memory() for t in (self.q, self.k, self.v))
            self.hout = torch.zeros_like(self.out, device="cpu").pin_memory()
        self.graphs = {}
        self.workspace = None   # private scratch: the overlapped launches need it zero-filled and to themselves
        self.kernel_launches_per_step = 0
        self.stream = torch.cuda.Stream(device=dev)
        if host_io:
            self.s_in, self.s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
            self.ev_in = [torch.cuda.Event() for _ in range(layers)]
            self.ev_out = [torch.cuda.Event() for _ in range(layers)]
            # Layers per copy.  Only the first host->device copy and the last device->host copy of a step
            # are exposed (the others hide behind the kernels), and every group boundary is a cross-stream
            # dependency that interrupts the layer-to-layer overlap of the kernels: the input groups
            # therefore double from one layer up to 16 (each copy is in flight while the group before it
            # computes, which takes 8.4 GB/s of PCIe for the 7B shape), the output groups mirror them.
            sizes, left, n = [], layers, 1
            while left > 0:
                sizes.append(min(n, left))
                left -= sizes[-1]
                n = min(2 * n, 16)
            self.io_group = max(sizes)
            starts = [sum(sizes[:i]) for i in range(len(sizes))]
            self.in_groups = [(a, a + n) for a, n in zip(starts, sizes)]
            rstarts = [sum(sizes[::-1][:i]) for i in range(len(sizes))]
            self.out_groups = [(a, a + n) for a, n in zip(rstarts, sizes[::-1])]
            self.in_starts = {a for a, _ in self.in_groups}
            self.out_ends = {b - 1: a for a, b in self.out_groups}

    def _body(self, meta):
        """Everything the device does in one step after the per-step integers have
        arrived in d64 / d32, on the current stream."""
        main = torch.cuda.current_stream()
        b = self.batch
        n_layers = self.engine.num_layers
        if self.host_io:
            # Host q/k/v travel layer by layer on a side stream, one layer ahead of the
            # kernels, and each layer's output leaves on another as soon as it exists, so
            # the PCIe time hides behind the attention kernels instead of bracketing them.
            self.s_in.wait_stream(main)
            self.s_out.wait_stream(main)
            with torch.cuda.stream(self.s_in):
                for l0, l1 in self.in_groups:     # several layers per copy, so that a transfer is worth a DMA launch
                    self.q[l0:l1].copy_(self.hq[l0:l1], non_blocking=True)
                    self.k[l0:l1].copy_(self.hk[l0:l1], non_blocking=True)
                    self.v[l0:l1].copy_(self.hv[l0:l1], non_blocking=True)
                    self.ev_in[l0].record(self.s_in)
        for layer in range(n_layers):
            kc, vc = self.engine.gpu_cache[layer]
            ks = self.k_scale[layer] if self.k_scale is not None else None
            vs = self.v_scale[layer] if self.v_scale is not None else None
            if self.host_io and layer in self.in_starts:
                main.wait_event(self.ev_in[layer])
            torch.cuda.nvtx.range_push(f"layer {layer}: append + attention")
            ops.decode_step(self.out[layer].view(b, self.impl.num_heads, self.impl.head_size),
                            self.q[layer].view(b, self.impl.num_heads, self.impl.head_size), self.k[layer],
                            self.v[layer], kc.vmm_ptr, vc.vmm_ptr, self.d64[:b], self.d64[b:], self.d32[:b],
                            meta.max_seq_len, self.impl.num_kv_heads, self.impl.scale, self.impl.kv_cache_dtype,
                            ks, vs, overlap=self._overlap_mode(layer), workspace=self.workspace,
                            maps=self.engine.decode_maps(layer, self.impl.num_heads), clean_scratch=True)
            torch.cuda.nvtx.range_pop()
            if self.post_layer is not None:
                self.post_layer(layer)
            if self.host_io and layer in self.out_ends:
                l0 = self.out_ends[layer]
                self.ev_out[layer].record(main)
                self.s_out.wait_event(self.ev_out[layer])
                with torch.cuda.stream(self.s_out):
                    self.hout[l0:layer + 1].copy_(self.out[l0:layer + 1], non_blocking=True)
        if self.host_io:
            main.wait_stream(self.s_in)
            main.wait_stream(self.s_out)

    def _overlap_mode(self, layer):
        """Layer 0 follows the copies of the step's integers: an ordinary launch.  Later layers
        overlap the previous layer's launch outright when nothing sits between them, and only
        stream their old cache rows early when other kernels do (their q / k / v would be
        those kernels' outputs in a model)."""
        if not self.overlap or layer == 0:
            return False
        return "early_kv" if self.post_layer is not None else True

    def step(self, meta: VTensorMetadata):
        """Runs one decode step for ``meta`` (slot ids and context lengths as lists).
        Inputs are whatever ``self.q/k/v`` (or ``self.hq/hk/hv``) hold; outputs land
        in ``self.out`` (or ``self.hout``).  Asynchronous: returns after the replay
        has been enqueued on ``self.stream``."""
        assert len(meta.slot_mapping_list) == self.batch
        t0 = time.perf_counter()
        slot_m, starts = prepare_step_host(meta, self.engine)
        self.prepare_seconds.append(time.perf_counter() - t0)
        b = self.batch
        cur = self.n_steps % 2
        self.n_steps += 1
        if self.staged[cur] is not None:
            self.staged[cur].synchronize()   # its copy of two steps ago has long been done
        self.h64[cur].copy_(torch.tensor(slot_m + list(meta.slot_mapping_list), dtype=torch.int64))
        self.h32[cur].copy_(torch.tensor(list(meta.seq_lens) + starts, dtype=torch.int32))
        with torch.cuda.stream(self.stream):
            # stream-ordered: runs after the previous replay has finished with d64 / d32
            self.d64.copy_(self.h64[cur], non_blocking=True)
            self.d32.copy_(self.h32[cur], non_blocking=True)
            if self.staged[cur] is None:
                # blocking: a host thread that spins inside the driver while it waits slows the
                # allocator's worker thread, whose cuMemMap / cuMemSetAccess calls need the same locks
                self.staged[cur] = torch.cuda.Event(blocking=True)
            self.staged[cur].record(self.stream)
        bucket = (meta.max_seq_len + self.BUCKET - 1) // self.BUCKET * self.BUCKET
        graph = self.graphs.get(bucket)
        if graph is None:
            need = ops.new_workspace(self.engine.device, b, self.impl.num_heads, self.impl.head_size, bucket)
            if self.workspace is None or self.workspace.numel() < need.numel():
                self.stream.synchronize()
                self.workspace = need
                self.graphs.clear()     # older graphs captured the previous buffer's address
            capture_meta = VTensorMetadata(meta.slot_mapping_list, meta.seq_lens, meta.kv_num_heads,
                                           meta.kv_head_size, kv_elem_size=meta.kv_elem_size)
            capture_meta.max_seq_len = bucket
            with torch.cuda.stream(self.stream):
                self._body(capture_meta)        # warm-up outside capture (sets kernel attributes)
                self.stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                # thread-local capture mode: with collectives in the step, the process group's
                # watchdog thread may query events while the capture is open
                with torch.cuda.graph(graph, stream=self.stream, capture_error_mode="thread_local"):
                    self._body(capture_meta)
            self.graphs[bucket] = graph
            _, parts, variant = ops.attn_plan(b, self.impl.num_heads, self.impl.num_kv_heads, bucket,
                                              self.impl.kv_cache_dtype)
            # fused step: one kernel per layer; otherwise append + attention (+ merge)
            fused = variant == 2 and ops.step_is_fused(self.impl.kv_cache_dtype)
            per_layer = 1 if fused else 2 + (1 if parts > 1 else 0)
            self.kernel_launches_per_step = self.engine.num_layers * (per_layer + self.launches_per_post_layer)
            return  # the warm-up pass above already executed this step
        with torch.cuda.stream(self.stream):
            graph.replay()

    def synchronize(self):
        self.stream.synchronize()

    def status(self):
        """0 unless one of this runner's kernels gave up on a bounded wait (its results
        are then invalid).  Synchronises the runner's stream."""
        if self.workspace is None:
            return 0
        with torch.cuda.stream(self.stream):
            return ops.workspace_status(self.workspace)
