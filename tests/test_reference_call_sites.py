"""The reference's OWN Python call sites, loaded from a reference checkout and run
unmodified against this package in place of its native modules:

* GLakeServe/vmm_allocator/vmm_allocator.py (the ``KV_cache`` wrapper, lines 5-19)
  with ``sys.modules["vmmAllocator"]`` = glake_b200.vmmAllocator;
* GLakeServe/vllm/attention/ops/paged_attn.py (``PagedAttention.write_to_paged_cache``
  lines 62-87 and ``forward_decode`` lines 90-135) with ``vllm._custom_ops`` =
  glake_b200.ops;
* the allocator block of ``LlamaModel.forward``
  (GLakeServe/vllm/model_executor/models/llama.py:307-341) and the decode call of
  ``XFormersImpl.forward`` (GLakeServe/vllm/attention/backends/xformers.py:407-430),
  cut out of their files as text and executed verbatim (their modules import all of
  vllm, so they cannot be imported whole).

Host tests run on the mock driver; the GPU test runs a real decode step through
the same call sites and compares with the CPU oracle.  Everything here is skipped
when no reference checkout is found ($GLAKE_REFERENCE, or a directory named
"reference" beside the repository).
"""
import importlib.util
import inspect
import sys
import textwrap
import types
from types import SimpleNamespace
from typing import List

import pytest
import torch

from oracle.build_ref import reference_root

REF = reference_root()
pytestmark = pytest.mark.skipif(REF is None, reason="no reference checkout")


def _load_file(name, *rel):
    import os
    path = os.path.join(REF, "GLakeServe", *rel)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class _SysModules:
    """Temporarily installs stand-ins in sys.modules and restores what was there."""

    def __init__(self, **mods):
        self.mods = {k.replace("__", "."): v for k, v in mods.items()}

    def __enter__(self):
        self.saved = {k: sys.modules.get(k) for k in self.mods}
        sys.modules.update(self.mods)

    def __exit__(self, *exc):
        for k, v in self.saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def load_reference_kv_cache():
    """The reference's vmm_allocator.py with this package's allocator behind ``import vmmAllocator``."""
    from glake_b200 import vmmAllocator
    path_before = list(sys.path)
    with _SysModules(vmmAllocator=vmmAllocator):
        mod = _load_file("ref_vmm_allocator_py", "vmm_allocator", "vmm_allocator.py")
    sys.path[:] = path_before          # the file appends a system directory to sys.path
    return mod.KV_cache


def load_reference_paged_attention(ops_module):
    """The reference's paged_attn.py with ``ops_module`` as ``vllm._custom_ops``."""
    vllm = types.ModuleType("vllm")
    vllm._custom_ops = ops_module
    attention = types.ModuleType("vllm.attention")
    attention_ops = types.ModuleType("vllm.attention.ops")
    prefix = types.ModuleType("vllm.attention.ops.prefix_prefill")
    prefix.context_attention_fwd = None     # Triton prefix kernel: not on the vTensor path
    with _SysModules(vllm=vllm, vllm___custom_ops=ops_module, vllm__attention=attention,
                     vllm__attention__ops=attention_ops, vllm__attention__ops__prefix_prefill=prefix):
        mod = _load_file("ref_paged_attn_py", "vllm", "attention", "ops", "paged_attn.py")
    return mod.PagedAttention


def cut(rel, first_marker, last_marker, last_is_call=False):
    """Source text from the line containing first_marker through the line containing
    last_marker (or, with last_is_call, through the closing parenthesis of the call
    that starts at first_marker), dedented."""
    import os
    lines = open(os.path.join(REF, "GLakeServe", *rel)).read().splitlines()
    i = next(n for n, l in enumerate(lines) if first_marker in l)
    if last_is_call:
        depth, j = 0, i
        while True:
            depth += lines[j].count("(") - lines[j].count(")")
            if depth == 0:
                break
            j += 1
    else:
        j = next(n for n in range(i, len(lines)) if last_marker in lines[n])
    return textwrap.dedent("\n".join(lines[i:j + 1]))


def llama_allocator_block():
    return cut(("vllm", "model_executor", "models", "llama.py"), "k_cache: List[KV_cache] = []",
               "attn_metadata.slot_m = torch.tensor(slot_m")


def xformers_decode_call():
    return cut(("vllm", "attention", "backends", "xformers.py"), "output, _ = flash_attn_cuda.fwd_kvcache(", None,
               last_is_call=True)


class _HostTorch:
    """``torch`` for the llama.py block on a machine without a GPU: tensors stay on the
    host, NVTX ranges are no-ops; everything else is the real module."""
    int, int64 = torch.int, torch.int64
    cuda = SimpleNamespace(nvtx=SimpleNamespace(range_push=lambda *_: None, range_pop=lambda: None))

    @staticmethod
    def tensor(data, dtype=None, device=None):
        return torch.tensor(data, dtype=dtype)


def build_engine(KV_cache, layers, kvh, max_seqs, max_tokens, device):
    """What CacheEngine.__init__ builds (cache_engine.py:53-129), with the reference's KV_cache class."""
    from glake_b200 import vmmAllocator as A
    ctx = (max_tokens * kvh * 128 * 2 + A.granularitySize - 1) // A.granularitySize * A.granularitySize
    segs = [A.KVcacheSegment(layers, ctx, 0, False) for _ in range(max_seqs)]
    gpu_cache = [(KV_cache(max_seqs, i), KV_cache(max_seqs, i)) for i in range(layers)]
    A.copy_kv_cache([k.kv_cache for k, _ in gpu_cache], [v.kv_cache for _, v in gpu_cache], segs)
    k_ptr = [torch.tensor([s.getKeyDevicePtr(l) for s in segs], dtype=torch.int64, device=device) for l in range(layers)]
    v_ptr = [torch.tensor([s.getValueDevicePtr(l) for s in segs], dtype=torch.int64, device=device)
             for l in range(layers)]
    return segs, gpu_cache, k_ptr, v_ptr


def run_llama_block(block, torch_mod, KV_cache, gpu_cache, meta, n_layers):
    from glake_b200 import vmmAllocator
    ns = {"vmmAllocator": vmmAllocator, "torch": torch_mod, "List": List, "KV_cache": KV_cache,
          "kv_caches": gpu_cache, "attn_metadata": meta, "self": SimpleNamespace(layers=[None] * n_layers)}
    exec(block, ns)          # noqa: S102  (the point of the test: the reference's own lines)
    return ns


@pytest.fixture()
def mock_pool():
    from glake_b200 import vmmAllocator as A
    from glake_b200._lib import lib
    assert A._pool is None, "another test left a pool behind"
    lib.vt_use_mock_driver(1)
    lib.vt_mock_map_delay_us(0)
    assert A.init_physical_handle(256, 0)
    yield A
    A.shutdown()
    lib.vt_use_mock_driver(0)


def test_reference_kv_cache_wrapper_wraps_our_table(mock_pool):
    KV_cache = load_reference_kv_cache()
    kc = KV_cache(4, 2)
    assert kc.max_seqs == 4 and kc.layer_index == 2
    assert isinstance(kc.kv_cache, mock_pool.KVCache) and kc.vmm_ptr == kc.kv_cache.getKVCachePtr() != 0
    kc.kv_cache.close()


def test_reference_llama_allocator_block_on_the_mock_driver(mock_pool):
    """Prompt step then decode steps across a chunk boundary, driven by the reference's own lines."""
    A = mock_pool
    KV_cache = load_reference_kv_cache()
    block = llama_allocator_block()
    assert "extend_kv_cache_batch" in block and "eagerExtend" in block and "query_cycle" in block
    layers, kvh = 2, 32                       # row = 8 KiB -> 256 rows per 2 MiB chunk
    segs, gpu_cache, _, _ = build_engine(KV_cache, layers, kvh, 3, 4096, "cpu")
    slots = [2, 0]
    lens = [250, 7]
    row = kvh * 128 * 2
    meta = SimpleNamespace(kv_num_heads=kvh, kv_head_size=128, num_prefills=2, seq_lens=lens,
                           slot_mapping_list=slots, extend_seq_list=[], kvcache_segment=[segs[s] for s in slots],
                           set_used_size=[0, 0])
    run_llama_block(block, _HostTorch, KV_cache, gpu_cache, meta, layers)
    assert meta.slot_m.tolist() == [0, 0] and meta.slot_m.dtype == torch.int64
    assert [s.get_used_slot() for s in meta.kvcache_segment] == [250 * row, 7 * row]
    assert segs[2].actual_size == A.granularitySize
    for step in range(10):                    # slot 2 crosses 256 rows at step 6
        lens = [n + 1 for n in lens]
        ask = [2 if lens[0] == 252 else -1, -1]          # the scheduler asks a few rows early
        meta = SimpleNamespace(kv_num_heads=kvh, kv_head_size=128, num_prefills=0, seq_lens=lens,
                               slot_mapping_list=slots, extend_seq_list=ask,
                               kvcache_segment=[segs[s] for s in slots], set_used_size=[0, 0])
        run_llama_block(block, _HostTorch, KV_cache, gpu_cache, meta, layers)
        assert meta.slot_m.tolist() == [(lens[0] - 1) * row, (lens[1] - 1) * row]
        assert meta.decode_seq_len.tolist() == [1, 1]
    segs[2].wait()
    assert segs[2].actual_size == 2 * A.granularitySize and segs[0].actual_size == A.granularitySize
    for s in segs:
        s.close()
    for k, v in gpu_cache:
        k.kv_cache.close(), v.kv_cache.close()


def test_reference_positional_calls_bind_to_our_op_signatures():
    """Every positional argument of the reference's calls lands on the parameter of the
    same meaning in glake_b200.ops (checked by binding, nothing is launched)."""
    from glake_b200 import ops
    seen = {}

    class Recorder(types.ModuleType):
        def __getattr__(self, name):
            target = getattr(ops, name)

            def call(*args, **kwargs):
                seen[name] = inspect.signature(target).bind(*args, **kwargs).arguments
                return (args[0], None) if name == "fwd_kvcache" else None
            return call

    rec = Recorder("recorder")
    PagedAttention = load_reference_paged_attention(rec)
    t = lambda *shape, dtype=torch.bfloat16: torch.zeros(*shape, dtype=dtype)      # noqa: E731
    key, value, query = t(3, 4, 128), t(3, 4, 128), t(3, 8, 128)
    kp, vp = t(8, dtype=torch.int64), t(8, dtype=torch.int64)
    slot_m, slot_mapping = torch.tensor([10, 20, 30]), torch.tensor([5, 0, 3])
    seq_lens, cache_seq_lens = torch.tensor([4, 5, 6], dtype=torch.int32), torch.tensor([0, 1, 2], dtype=torch.int32)
    PagedAttention.write_to_paged_cache(key, value, kp, vp, slot_m, slot_mapping, seq_lens, cache_seq_lens, 1, 4, 128)
    a = seen["reshape_and_cache"]
    assert a["key"] is key and a["value"] is value and a["key_cache"] is kp and a["value_cache"] is vp
    assert a["slot_m"] is slot_m and a["slot_mapping"] is slot_mapping and a["seq_lens"] is seq_lens
    assert a["cache_seq_lens"] is cache_seq_lens and (a["max_seq_len"], a["num_kv_heads"], a["head_size"]) == (1, 4, 128)
    out = PagedAttention.forward_decode(query, 1234, 5678, seq_lens, 6, "auto", 4, 0.5, None, 1.0, slot_mapping)
    a = seen["paged_attention_v1"]
    assert out.shape == query.shape and a["out"] is out and a["query"] is query
    assert (a["key_cache"], a["value_cache"], a["num_kv_heads"], a["scale"]) == (1234, 5678, 4, 0.5)
    assert a["seq_lens"] is seq_lens and a["block_size"] == 1 and a["max_seq_len"] == 6 and a["alibi_slopes"] is None
    assert a["kv_cache_dtype"] == "auto" and a["kv_scale"] == 1.0 and a["slot_mapping"] is slot_mapping
    # the live decode call of the backend, its 22 positional arguments
    ns = {"flash_attn_cuda": rec, "decode_query": query, "key_cache": SimpleNamespace(vmm_ptr=1234),
          "value_cache": SimpleNamespace(vmm_ptr=5678),
          "attn_metadata": SimpleNamespace(max_seq_len=6, slot_mapping=slot_mapping, seq_lens_tensor=seq_lens),
          "self": SimpleNamespace(num_kv_heads=4, scale=0.5)}
    exec(xformers_decode_call(), ns)      # noqa: S102
    a = seen["fwd_kvcache"]
    assert a["q"].shape == (3, 1, 8, 128) and (a["k_table_ptr"], a["v_table_ptr"]) == (1234, 5678)
    assert (a["max_seq_len"], a["num_kv_heads"], a["batch"]) == (6, 4, 3) and a["slot_mapping"] is slot_mapping
    assert a["seq_lens"] is seq_lens and a["softmax_scale"] == 0.5 and a["causal"] is True
    assert (a["window_left"], a["window_right"], a["num_splits"]) == (-1, -1, 4)
    assert all(a[n] is None for n in ("k_new", "v_new", "rotary_cos", "rotary_sin", "cache_batch_idx", "block_table",
                                      "alibi_slopes", "out", "rotary_interleaved"))


@pytest.mark.gpu
def test_reference_call_sites_run_a_decode_step_on_the_gpu(oracle):
    """Two layers, a prompt step and four decode steps, driven entirely by the
    reference's lines: llama.py's allocator block, PagedAttention.write_to_paged_cache,
    then both decode attention calls it has (forward_decode -> paged_attention_v1 and
    the 22-argument fwd_kvcache), compared with the oracle."""
    import numpy as np
    from glake_b200 import ops
    from tests import gpu_util, synth
    from tests.test_oracle import SCALE
    gpu_util.ensure_pool()
    KV_cache = load_reference_kv_cache()
    PagedAttention = load_reference_paged_attention(ops)
    block, decode_call = llama_allocator_block(), xformers_decode_call()
    layers, h, kvh = 2, 8, 4
    slots, lens = [2, 0, 1], [300, 5, 1023]
    segs, gpu_cache, k_ptr, v_ptr = build_engine(KV_cache, layers, kvh, 3, 2048, "cuda")
    rs = np.random.RandomState(31)
    hist_k = [[synth.normal_bf16(rs, n, kvh, 128) for n in lens] for _ in range(layers)]
    hist_v = [[synth.normal_bf16(rs, n, kvh, 128) for n in lens] for _ in range(layers)]
    try:
        def meta_for(prefill):
            return SimpleNamespace(
                kv_num_heads=kvh, kv_head_size=128, num_prefills=len(lens) if prefill else 0, seq_lens=lens,
                slot_mapping_list=slots, extend_seq_list=[-1] * len(lens), kvcache_segment=[segs[s] for s in slots],
                set_used_size=[0] * len(lens), slot_mapping=torch.tensor(slots, dtype=torch.int64, device="cuda"),
                seq_lens_tensor=torch.tensor(lens, dtype=torch.int32, device="cuda"), max_seq_len=max(lens))
        meta = meta_for(True)
        run_llama_block(block, torch, KV_cache, gpu_cache, meta, layers)
        starts = torch.tensor([0, lens[0], lens[0] + lens[1]], dtype=torch.int32, device="cuda")
        for l in range(layers):
            PagedAttention.write_to_paged_cache(torch.cat(hist_k[l]).cuda(), torch.cat(hist_v[l]).cuda(), k_ptr[l],
                                                v_ptr[l], meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor, starts,
                                                max(lens), kvh, 128)
        for step in range(4):
            lens = [n + 1 for n in lens]
            meta = meta_for(False)
            run_llama_block(block, torch, KV_cache, gpu_cache, meta, layers)
            for l in range(layers):
                q = synth.normal_bf16(rs, len(lens), h, 128)
                nk, nv = synth.normal_bf16(rs, len(lens), kvh, 128), synth.normal_bf16(rs, len(lens), kvh, 128)
                key_cache, value_cache = gpu_cache[l]
                PagedAttention.write_to_paged_cache(nk.cuda(), nv.cuda(), k_ptr[key_cache.layer_index],
                                                    v_ptr[value_cache.layer_index], meta.slot_m, meta.slot_mapping,
                                                    meta.seq_lens_tensor, None, 1, kvh, 128)
                out1 = PagedAttention.forward_decode(q.cuda(), key_cache.vmm_ptr, value_cache.vmm_ptr,
                                                     meta.seq_lens_tensor, meta.max_seq_len, "auto", kvh, SCALE, None,
                                                     1.0, meta.slot_mapping)
                ns = {"flash_attn_cuda": ops, "decode_query": q.cuda(), "key_cache": key_cache,
                      "value_cache": value_cache, "attn_metadata": meta,
                      "self": SimpleNamespace(num_kv_heads=kvh, scale=SCALE)}
                exec(decode_call, ns)     # noqa: S102
                out2 = ns["output"].view(-1, h, 128)
                hist_k[l] = [torch.cat([a, b[None]]) for a, b in zip(hist_k[l], nk)]
                hist_v[l] = [torch.cat([a, b[None]]) for a, b in zip(hist_v[l], nv)]
                r = oracle.fill_ranges(hist_k[l], hist_v[l])
                port = oracle.port_decode_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32),
                                               kvh, SCALE)
                tol = torch.maximum(torch.full_like(port.float(), 2e-3), port.float().abs() * 2.0 ** -7)
                for got in (out1, out2):
                    assert bool(((got.cpu().float() - port.float()).abs() <= tol).all()), (step, l)
    finally:
        for s in segs:
            s.close()
        for k, v in gpu_cache:
            k.kv_cache.close(), v.kv_cache.close()
