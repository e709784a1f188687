"""Custom-op layer with the reference's call signatures
(GLakeServe/vllm/_custom_ops.py:34-52, :238-252 and the flash_attn_2_cuda.fwd_kvcache
call at GLakeServe/vllm/attention/backends/xformers.py:407-430), forwarding to
libvtensor's C ABI.  Tensors are only unwrapped to pointers and strides here; all
work happens in the CUDA kernels.  Non-CUDA tensors are rejected: there is no
CPU path.
"""
import ctypes
from ctypes import byref, c_size_t, c_void_p

import torch

from ._lib import VT_KV_BF16, VT_KV_FP8_E4M3, check, lib

_workspaces = {}


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("glake_b200 ops need CUDA tensors: there is no CPU fallback")


def _kv_dtype(kv_cache_dtype):
    if kv_cache_dtype in ("auto", "bf16", "bfloat16", None):
        return VT_KV_BF16
    if kv_cache_dtype in ("fp8", "fp8_e4m3"):
        return VT_KV_FP8_E4M3
    raise RuntimeError(f"unsupported kv_cache_dtype {kv_cache_dtype!r} (bf16 and fp8_e4m3 only)")


def new_workspace(device, batch, num_heads, head_size, max_seq_len):
    """A private, zero-filled scratch buffer for ``decode_step(..., workspace=...)``."""
    need = c_size_t()
    check(lib.vt_decode_attn_workspace_bytes(batch, num_heads, head_size, max_seq_len, byref(need)),
          "vt_decode_attn_workspace_bytes")
    return torch.zeros(need.value, dtype=torch.uint8, device=device)


def attn_workspace(device, batch, num_heads, head_size, max_seq_len):
    """Scratch for the split-K partials, cached per device and grown on demand.
    One buffer serves every layer because layers run back to back on one stream."""
    need = c_size_t()
    check(lib.vt_decode_attn_workspace_bytes(batch, num_heads, head_size, max_seq_len, byref(need)),
          "vt_decode_attn_workspace_bytes")
    key = (device.index if device.index is not None else torch.cuda.current_device())
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < need.value:
        buf = torch.zeros(max(need.value, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def reshape_and_cache(key, value, key_cache, value_cache, slot_m, slot_mapping, seq_lens, cache_seq_lens,
                      max_seq_len, num_kv_heads, head_size, kv_cache_dtype="auto", k_scale=None, v_scale=None):
    """Append K/V rows into the slots' contiguous ranges.

    Positional arguments as in the reference (csrc/cache.h:18-29): ``key_cache`` /
    ``value_cache`` are int64 device tensors of base addresses indexed by slot id,
    ``slot_m`` the per-entry destination byte offsets, ``slot_mapping`` the slot
    ids, ``max_seq_len`` 1 for decode.  The keyword arguments add the fp8 e4m3
    cache with per-kv-head scales (float32 device tensors of num_kv_heads)."""
    _require_cuda(key, value, key_cache, value_cache, slot_m, slot_mapping)
    if key.dtype != torch.bfloat16 or value.dtype != torch.bfloat16:
        raise RuntimeError("reshape_and_cache: key/value must be bfloat16")
    key = key.view(-1, num_kv_heads, head_size) if key.dim() == 2 else key
    value = value.view(-1, num_kv_heads, head_size) if value.dim() == 2 else value
    if key.stride(2) != 1 or key.stride(1) != head_size or value.stride(2) != 1 or value.stride(1) != head_size:
        raise RuntimeError("reshape_and_cache: key/value rows must be contiguous [kv_heads, head_size]")
    batch = slot_mapping.numel()
    with torch.cuda.device(key.device):
        check(lib.vt_append(_ptr(key), _ptr(value), key.stride(0), value.stride(0), _ptr(key_cache),
                            _ptr(value_cache), _ptr(slot_m), _ptr(slot_mapping), _ptr(seq_lens),
                            _ptr(cache_seq_lens), int(max_seq_len), batch, num_kv_heads, head_size,
                            _kv_dtype(kv_cache_dtype), _ptr(k_scale), _ptr(v_scale), _stream()), "vt_append")


VT_ROPE_WRITE_KEY = 1


def rotary_embedding_and_cache(positions, query, key, value, head_size, cos_sin_cache, is_neox, key_cache,
                               value_cache, slot_m, slot_mapping, seq_lens, cache_seq_lens, max_seq_len,
                               num_kv_heads, kv_cache_dtype="auto", k_scale=None, v_scale=None, write_key=False):
    """``rotary_embedding`` (GLakeServe/vllm/_custom_ops.py:81-90) and
    ``reshape_and_cache`` in one launch: ``query`` is rotated in place, the rotated
    key and the value rows go straight into the slots' ranges.  The first seven
    arguments are rotary_embedding's (plus ``value``), the rest reshape_and_cache's.
    ``key`` itself is only rewritten with ``write_key=True``."""
    _require_cuda(positions, query, key, value, cos_sin_cache, key_cache, value_cache, slot_m, slot_mapping)
    if not (query.dtype == key.dtype == value.dtype == cos_sin_cache.dtype == torch.bfloat16):
        raise RuntimeError("rotary_embedding_and_cache: bfloat16 tensors only")
    q2 = query.view(-1, query.shape[-1])
    k2 = key.view(-1, key.shape[-1])
    v2 = value.view(-1, value.shape[-1])
    if q2.stride(1) != 1 or k2.stride(1) != 1 or v2.stride(1) != 1 or not cos_sin_cache.is_contiguous():
        raise RuntimeError("rotary_embedding_and_cache: rows must be contiguous")
    if q2.shape[-1] % head_size or k2.shape[-1] != num_kv_heads * head_size or v2.shape[-1] != k2.shape[-1]:
        raise RuntimeError("rotary_embedding_and_cache: inconsistent head counts")
    with torch.cuda.device(query.device):
        check(lib.vt_rope_append(_ptr(positions), _ptr(q2), q2.stride(0), q2.shape[-1] // head_size, _ptr(k2), _ptr(v2),
                                 k2.stride(0), v2.stride(0), _ptr(cos_sin_cache), cos_sin_cache.shape[1],
                                 1 if is_neox else 0, _ptr(key_cache), _ptr(value_cache), _ptr(slot_m),
                                 _ptr(slot_mapping), _ptr(seq_lens), _ptr(cache_seq_lens), int(max_seq_len),
                                 slot_mapping.numel(), num_kv_heads, head_size, _kv_dtype(kv_cache_dtype),
                                 _ptr(k_scale), _ptr(v_scale), VT_ROPE_WRITE_KEY if write_key else 0, _stream()),
              "vt_rope_append")


def rms_norm(out, input, weight, epsilon):
    """out = rms_norm(input) * weight (GLakeServe/vllm/_custom_ops.py:104-106)."""
    _require_cuda(out, input, weight)
    if not (out.dtype == input.dtype == weight.dtype == torch.bfloat16):
        raise RuntimeError("rms_norm: bfloat16 tensors only")
    hidden = input.shape[-1]
    x, o = input.view(-1, hidden), out.view(-1, hidden)
    if x.stride(1) != 1 or o.stride(1) != 1:
        raise RuntimeError("rms_norm: rows must be contiguous")
    with torch.cuda.device(input.device):
        check(lib.vt_rms_norm(_ptr(o), _ptr(x), _ptr(weight), float(epsilon), x.shape[0], hidden, x.stride(0),
                              o.stride(0), _stream()), "vt_rms_norm")


def fused_add_rms_norm(input, residual, weight, epsilon):
    """residual += input; input = rms_norm(residual) * weight, both in place
    (GLakeServe/vllm/_custom_ops.py:109-111)."""
    _require_cuda(input, residual, weight)
    if not (input.dtype == residual.dtype == weight.dtype == torch.bfloat16):
        raise RuntimeError("fused_add_rms_norm: bfloat16 tensors only")
    if not (input.is_contiguous() and residual.is_contiguous()):
        raise RuntimeError("fused_add_rms_norm: contiguous tensors only")
    hidden = input.shape[-1]
    with torch.cuda.device(input.device):
        check(lib.vt_fused_add_rms_norm(_ptr(input), _ptr(residual), _ptr(weight), float(epsilon),
                                        input.numel() // hidden, hidden, _stream()), "vt_fused_add_rms_norm")


def kv_scales(x, num_kv_heads, head_size):
    """Per-kv-head scale = amax / 448 of x ([tokens, kv_heads, head_size] bf16)."""
    _require_cuda(x)
    x = x.view(-1, num_kv_heads, head_size)
    out = torch.empty(num_kv_heads, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.vt_kv_scales(_ptr(x), x.stride(0), x.shape[0], num_kv_heads, head_size, _ptr(out), _stream()),
              "vt_kv_scales")
    return out


def _decode(out, query, k_table, v_table, num_kv_heads, scale, seq_lens, max_seq_len, slot_ids, kv_dtype,
            k_scale, v_scale, lse, num_splits, maps=None):
    batch, num_heads, head_size = query.shape
    ws = attn_workspace(query.device, batch, num_heads, head_size, max_seq_len)
    if maps is not None and num_splits == 0:
        # plain attention through the tensor-map entry point (no rows to append)
        with torch.cuda.device(query.device):
            check(lib.vt_decode_step_tma(_ptr(out), out.stride(0), _ptr(query), query.stride(0), None, None, 0, 0, None,
                                         c_void_p(int(k_table)), c_void_p(int(v_table)), _ptr(slot_ids), _ptr(seq_lens),
                                         batch, num_heads, num_kv_heads, head_size, int(max_seq_len), float(scale),
                                         kv_dtype, _ptr(k_scale), _ptr(v_scale), _ptr(lse), _ptr(ws), ws.numel(), 0,
                                         _ptr(maps), _stream()), "vt_decode_step_tma")
        return
    with torch.cuda.device(query.device):
        check(lib.vt_decode_attn(_ptr(out), out.stride(0), _ptr(query), query.stride(0), c_void_p(int(k_table)),
                                 c_void_p(int(v_table)), _ptr(slot_ids), _ptr(seq_lens), batch, num_heads,
                                 num_kv_heads, head_size, int(max_seq_len), float(scale), kv_dtype, _ptr(k_scale),
                                 _ptr(v_scale), _ptr(lse), _ptr(ws), ws.numel(), int(num_splits), _stream()),
              "vt_decode_attn")


def paged_attention_v1(out, query, key_cache, value_cache, num_kv_heads, scale, seq_lens, block_size, max_seq_len,
                       alibi_slopes, kv_cache_dtype, kv_scale, slot_mapping, k_scale=None, v_scale=None,
                       num_splits=0, maps=None):
    """Decode attention with the reference's vTensor signature (csrc/ops.h:6-19):
    ``key_cache`` / ``value_cache`` are the device addresses (ints) of the per-layer
    pointer tables, ``slot_mapping`` the slot ids.  ``block_size`` must be 1 (the
    token-major contiguous layout, vllm/attention/ops/paged_attn.py:105).  ``maps`` (from
    :func:`decode_maps`, fp8 cache) selects the tcgen05 kernel where the head counts allow."""
    _require_cuda(out, query, seq_lens, slot_mapping, maps)
    if alibi_slopes is not None:
        raise RuntimeError("paged_attention_v1: ALiBi is not supported on the vTensor path")
    if block_size != 1:
        raise RuntimeError("paged_attention_v1: the vTensor layout is block_size 1")
    if query.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise RuntimeError("paged_attention_v1: bf16 only")
    kvd = _kv_dtype(kv_cache_dtype)
    if kvd == VT_KV_FP8_E4M3 and k_scale is None:
        k_scale = torch.full((num_kv_heads,), float(kv_scale), dtype=torch.float32, device=query.device)
        v_scale = k_scale
    _decode(out, query, key_cache, value_cache, num_kv_heads, scale, seq_lens, max_seq_len, slot_mapping, kvd,
            k_scale, v_scale, None, num_splits, maps)


def fwd_kvcache(q, k_table_ptr, v_table_ptr, max_seq_len, num_kv_heads, batch, slot_mapping, k_new, v_new,
                seq_lens, rotary_cos, rotary_sin, cache_batch_idx, block_table, alibi_slopes, out, softmax_scale,
                causal, window_left, window_right, rotary_interleaved, num_splits, kv_cache_dtype="auto",
                k_scale=None, v_scale=None):
    """The 22-positional-argument call the reference's backend makes into its
    flash-attention fork (xformers.py:407-430): q ``[B, 1, H, D]``, pointer-table
    addresses, ``slot_mapping`` slot ids, ``seq_lens`` int32.  Returns ``(out, lse)``
    with out ``[B, 1, H, D]`` and lse ``[B, H, 1]`` float32.  The arguments the
    reference always passes as None / -1 must be None / -1 here."""
    _require_cuda(q, slot_mapping, seq_lens)
    for name, v in (("k_new", k_new), ("v_new", v_new), ("rotary_cos", rotary_cos), ("rotary_sin", rotary_sin),
                    ("cache_batch_idx", cache_batch_idx), ("block_table", block_table),
                    ("alibi_slopes", alibi_slopes)):
        if v is not None:
            raise RuntimeError(f"fwd_kvcache: {name} is not supported on the vTensor path")
    if window_left != -1 or window_right != -1:
        raise RuntimeError("fwd_kvcache: sliding window is not supported")
    if q.dim() != 4:
        raise RuntimeError("fwd_kvcache: q must be [B, S, H, D]")
    if q.shape[1] != 1:
        # prefix-extend form (xformers.py:362-385): S new tokens per sequence, causal over the range
        if not causal:
            raise RuntimeError("fwd_kvcache: seqlen_q > 1 needs causal=True")
        b, s, h, d = q.shape
        qc = q.contiguous().view(b * s, h, d)
        o = out if out is not None else torch.empty(b, s, h, d, dtype=q.dtype, device=q.device)
        q_lens = torch.full((b,), s, dtype=torch.int32, device=q.device)
        q_start = torch.arange(b, dtype=torch.int32, device=q.device) * s
        prefill_attention(o.view(b * s, h, d), qc, k_table_ptr, v_table_ptr, num_kv_heads, softmax_scale,
                          slot_mapping, seq_lens, q_lens, q_start, s, kv_cache_dtype=kv_cache_dtype, k_scale=k_scale,
                          v_scale=v_scale)
        return o, None
    b, _, h, d = q.shape
    q3 = q.view(b, h, d) if q.is_contiguous() else q[:, 0]
    o = out if out is not None else torch.empty(b, 1, h, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(b, h, dtype=torch.float32, device=q.device)
    _decode(o.view(b, h, d), q3, k_table_ptr, v_table_ptr, num_kv_heads, softmax_scale, seq_lens, max_seq_len,
            slot_mapping, _kv_dtype(kv_cache_dtype), k_scale, v_scale, lse, 0)
    return o, lse.unsqueeze(-1)


def decode_step(out, query, key, value, key_cache, value_cache, slot_m, slot_mapping, seq_lens, max_seq_len,
                num_kv_heads, scale, kv_cache_dtype="auto", k_scale=None, v_scale=None, lse=None, overlap=False,
                workspace=None, maps=None, clean_scratch=False):
    """``reshape_and_cache`` (decode form) + ``paged_attention_v1`` in one call; one
    kernel launch for a bf16 cache.  ``key_cache`` / ``value_cache`` are the device
    addresses of the layer's pointer tables (ints), ``slot_m`` the destination byte
    offsets, ``slot_mapping`` the slot ids, ``seq_lens`` the contexts INCLUDING the
    appended token.  query/out ``[B, H, D]``, key/value ``[B, KVH, D]`` bf16.
    ``overlap=True`` lets the launch overlap the previous ``decode_step`` on the
    stream (VT_STEP_OVERLAP): only for a different layer's ranges, see vtensor.h;
    ``overlap="early_kv"`` (VT_STEP_EARLY_KV) is the form for inputs that the preceding
    kernel produces: cache rows stream early, q / key / value are read after it finished.
    Pass a private zero-filled ``workspace`` (uint8 tensor) in both cases.
    ``maps`` (from :func:`decode_maps`, fp8 cache only) selects the tcgen05 kernel where
    the head counts allow; other shapes run as without it.  ``clean_scratch=True``
    (VT_STEP_CLEAN_SCRATCH): ``workspace`` is private, was zero-filled once and is used by
    nothing but these calls, so the call need not clear its counters first."""
    _require_cuda(out, query, key, value, slot_m, slot_mapping, seq_lens, maps)
    batch, num_heads, head_size = query.shape
    key = key.view(batch, num_kv_heads, head_size)
    value = value.view(batch, num_kv_heads, head_size)
    if overlap and workspace is None:
        raise RuntimeError("decode_step(overlap=True) needs a private zero-filled workspace")
    ws = workspace if workspace is not None else attn_workspace(query.device, batch, num_heads, head_size,
                                                                max_seq_len)
    flags = (2 if overlap == "early_kv" else (1 if overlap else 0)) | (4 if clean_scratch else 0)
    if clean_scratch and workspace is None:
        raise RuntimeError("decode_step(clean_scratch=True) needs a private zero-filled workspace")
    if maps is not None:
        with torch.cuda.device(query.device):
            check(lib.vt_decode_step_tma(_ptr(out), out.stride(0), _ptr(query), query.stride(0), _ptr(key), _ptr(value),
                                         key.stride(0), value.stride(0), _ptr(slot_m), c_void_p(int(key_cache)),
                                         c_void_p(int(value_cache)), _ptr(slot_mapping), _ptr(seq_lens), batch,
                                         num_heads, num_kv_heads, head_size, int(max_seq_len), float(scale),
                                         _kv_dtype(kv_cache_dtype), _ptr(k_scale), _ptr(v_scale), _ptr(lse), _ptr(ws),
                                         ws.numel(), flags, _ptr(maps), _stream()), "vt_decode_step_tma")
        return
    with torch.cuda.device(query.device):
        check(lib.vt_decode_step(_ptr(out), out.stride(0), _ptr(query), query.stride(0), _ptr(key), _ptr(value),
                                 key.stride(0), value.stride(0), _ptr(slot_m), c_void_p(int(key_cache)),
                                 c_void_p(int(value_cache)), _ptr(slot_mapping), _ptr(seq_lens), batch, num_heads,
                                 num_kv_heads, head_size, int(max_seq_len), float(scale), _kv_dtype(kv_cache_dtype),
                                 _ptr(k_scale), _ptr(v_scale), _ptr(lse), _ptr(ws), ws.numel(), flags, _stream()),
              "vt_decode_step")


def step_is_fused(kv_cache_dtype):
    """Whether decode_step on the persistent schedule is ONE launch for this cache type: the
    attention kernel appends the new rows itself (bf16: copied, fp8: quantised on the way)."""
    return _kv_dtype(kv_cache_dtype) in (VT_KV_BF16, VT_KV_FP8_E4M3)


def prefill_tma_supported(num_kv_heads):
    """Whether ``prefill_maps`` / the TMA prefill path take this kv-head count (a
    32-token box must never straddle a 2 MiB chunk)."""
    return num_kv_heads & (num_kv_heads - 1) == 0 and num_kv_heads * 32 <= 8192


def prefill_maps(k_bases, v_bases, num_kv_heads, head_size, max_tokens, device):
    """Device table of TMA tensor maps for ``prefill_attention(..., maps=...)``:
    ``k_bases[i]`` / ``v_bases[i]`` are slot i's range bases of one layer
    (``getKeyDevicePtr`` / ``getValueDevicePtr``).  Valid while the slots live."""
    n = len(k_bases)
    kb = (ctypes.c_uint64 * n)(*[int(x) for x in k_bases])
    vb = (ctypes.c_uint64 * n)(*[int(x) for x in v_bases])
    host = torch.empty(n * 256 + 64, dtype=torch.uint8)
    off = (-host.data_ptr()) % 64
    with torch.cuda.device(device):
        check(lib.vt_prefill_maps_encode(kb, vb, n, num_kv_heads, head_size, int(max_tokens),
                                         c_void_p(host.data_ptr() + off)), "vt_prefill_maps_encode")
    return host[off: off + n * 256].to(device)


def decode_tma_supported(num_heads, num_kv_heads, kv_cache_dtype):
    """Whether ``decode_step(..., maps=...)`` runs the tcgen05 kernel for this shape (fp8 cache,
    kv heads a power of two >= 8, at most 4 q heads per kv head); other shapes ignore the maps."""
    g = num_heads // num_kv_heads
    return (_kv_dtype(kv_cache_dtype) == VT_KV_FP8_E4M3 and num_kv_heads % 8 == 0
            and num_kv_heads & (num_kv_heads - 1) == 0 and num_kv_heads <= 256 and g in (1, 2, 4))


def decode_maps(k_bases, v_bases, num_kv_heads, head_size, max_tokens, device, kv_cache_dtype="fp8"):
    """Device table of TMA tensor maps for ``decode_step(..., maps=...)`` over fp8 ranges:
    ``k_bases[i]`` / ``v_bases[i]`` are slot i's range bases of one layer.  Valid while the slots live."""
    n = len(k_bases)
    kb = (ctypes.c_uint64 * n)(*[int(x) for x in k_bases])
    vb = (ctypes.c_uint64 * n)(*[int(x) for x in v_bases])
    host = torch.empty(n * 256 + 64, dtype=torch.uint8)
    off = (-host.data_ptr()) % 64
    with torch.cuda.device(device):
        check(lib.vt_decode_maps_encode(kb, vb, n, num_kv_heads, head_size, _kv_dtype(kv_cache_dtype), int(max_tokens),
                                        c_void_p(host.data_ptr() + off)), "vt_decode_maps_encode")
    return host[off: off + n * 256].to(device)


def widen_fp8_ranges(key_cache, value_cache, num_kv_heads, head_size, slot_mapping, seq_lens, k_scale, v_scale,
                     pad_rows=64):
    """Dense bf16 copies of the slots' fp8 rows for the prompt kernels: returns
    (k_bases, v_bases, holder) where ``k_bases`` / ``v_bases`` are int64 device tensors
    of one scratch range address per batch entry (usable as pointer tables with slot ids
    0..B-1) and ``holder`` keeps the scratch alive.  Every entry's range is padded to a
    multiple of ``pad_rows`` rows so that whole-tile fetches at its ragged end stay
    inside the buffer.  Synchronises once to learn the context lengths."""
    lens = [int(x) for x in seq_lens.tolist()]
    row = num_kv_heads * head_size
    padded = [(n + pad_rows - 1) // pad_rows * pad_rows + pad_rows for n in lens]
    total = sum(padded)
    dev = seq_lens.device
    buf = torch.zeros(2, max(total, 1), row, dtype=torch.bfloat16, device=dev)
    starts, acc = [], 0
    for n in padded:
        starts.append(acc)
        acc += n
    kb = torch.tensor([buf[0].data_ptr() + s * row * 2 for s in starts], dtype=torch.int64, device=dev)
    vb = torch.tensor([buf[1].data_ptr() + s * row * 2 for s in starts], dtype=torch.int64, device=dev)
    with torch.cuda.device(dev):
        check(lib.vt_kv_widen(c_void_p(int(key_cache)), c_void_p(int(value_cache)), _ptr(slot_mapping), _ptr(seq_lens),
                              len(lens), num_kv_heads, head_size, max(lens) if lens else 0, _ptr(k_scale), _ptr(v_scale),
                              _ptr(kb), _ptr(vb), _stream()), "vt_kv_widen")
    return kb, vb, (buf, padded)


def prefill_attention(out, query, key_cache, value_cache, num_kv_heads, scale, slot_mapping, seq_lens, q_lens,
                      q_start, max_q_len, maps=None, kv_cache_dtype="auto", k_scale=None, v_scale=None):
    """Causal attention of the new tokens over the slots' whole ranges (the new rows
    already appended with ``reshape_and_cache``).  query/out ``[tokens, H, D]`` bf16,
    ``key_cache`` / ``value_cache`` the pointer-table addresses (ints), ``seq_lens``
    the contexts including the new tokens, ``q_lens`` / ``q_start`` int32 per entry.
    With ``maps`` (from :func:`prefill_maps`) K/V tiles are fetched by TMA tensor copies.
    An fp8 e4m3 cache (``kv_cache_dtype``, per-kv-head ``k_scale`` / ``v_scale``) is first
    widened into bf16 scratch ranges (:func:`widen_fp8_ranges`), over which the same
    kernels run, with tensor maps of the scratch where the head count allows."""
    _require_cuda(out, query, slot_mapping, seq_lens, q_lens, q_start, maps)
    if query.dtype != torch.bfloat16:
        raise RuntimeError("prefill_attention: bf16 only")
    n, num_heads, head_size = query.shape
    holder = None
    if _kv_dtype(kv_cache_dtype) == VT_KV_FP8_E4M3:
        if k_scale is None or v_scale is None:
            raise RuntimeError("prefill_attention: an fp8 cache needs k_scale and v_scale")
        kb, vb, holder = widen_fp8_ranges(key_cache, value_cache, num_kv_heads, head_size, slot_mapping, seq_lens,
                                          k_scale, v_scale)
        batch = slot_mapping.numel()
        key_cache, value_cache = kb.data_ptr(), vb.data_ptr()
        slot_mapping = torch.arange(batch, dtype=torch.int64, device=query.device)
        maps = None
        if prefill_tma_supported(num_kv_heads):
            maps = prefill_maps(kb.tolist(), vb.tolist(), num_kv_heads, head_size, max(holder[1]), query.device)
        holder = (holder, kb, vb, slot_mapping, maps)
    args = (_ptr(out), out.stride(0), _ptr(query), query.stride(0), c_void_p(int(key_cache)),
            c_void_p(int(value_cache)), _ptr(slot_mapping), _ptr(seq_lens), _ptr(q_lens),
            _ptr(q_start), slot_mapping.numel(), num_heads, num_kv_heads, head_size,
            int(max_q_len), float(scale), VT_KV_BF16, None)
    with torch.cuda.device(query.device):
        if maps is None:
            check(lib.vt_prefill_attn(*args, _stream()), "vt_prefill_attn")
        else:
            check(lib.vt_prefill_attn_tma(*args, _ptr(maps), _stream()), "vt_prefill_attn_tma")
    if holder is not None:
        # the scratch must outlive the kernels queued above: torch's allocator reuses a freed
        # block only in stream order on the stream that allocated it, which is this one
        del holder


def attn_plan(batch, num_heads, num_kv_heads, max_seq_len, kv_cache_dtype="auto", num_splits=0):
    """(tokens per partition, partitions per sequence, kernel variant) the library
    picks for this problem size."""
    a, b, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    check(lib.vt_decode_attn_plan(batch, num_heads, num_kv_heads, max_seq_len, _kv_dtype(kv_cache_dtype),
                                  num_splits, byref(a), byref(b), byref(c)), "vt_decode_attn_plan")
    return a.value, b.value, c.value


_VARIANTS = {None: -1, "auto": -1, "simt": 0, "mma": 1, "flat": 2}


def set_attn_tuning(variant="auto", part_tokens=0):
    """Process-wide planner override for benchmarks and tests: ``variant`` one of
    auto / simt / mma / flat, ``part_tokens`` tokens per split-K partition (0 = auto)."""
    check(lib.vt_attn_set_tuning(_VARIANTS[variant], int(part_tokens)), "vt_attn_set_tuning")


def workspace_status(workspace):
    """VT_OK (0) unless an attention kernel using this scratch buffer gave up on a
    bounded wait.  Synchronises the current stream."""
    code = ctypes.c_int()
    with torch.cuda.device(workspace.device):
        check(lib.vt_decode_attn_status(_ptr(workspace), _stream(), byref(code)), "vt_decode_attn_status")
    return code.value


def attn_status(device=None):
    """VT_OK (0) unless an attention kernel's bounded wait ran out since the
    workspace was created.  Synchronises the current stream."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    ws = _workspaces.get(dev.index if dev.index is not None else torch.cuda.current_device())
    if ws is None:
        return 0
    code = ctypes.c_int()
    check(lib.vt_decode_attn_status(_ptr(ws), _stream(), byref(code)), "vt_decode_attn_status")
    return code.value
