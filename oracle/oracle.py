"""TEST INFRASTRUCTURE — Python face of the CPU checker.

Two checkers live here and neither is ever imported by the product package:

* ``port``  – oracle/vt_oracle.c, a plain-C restatement of the path on the
  vTensor (token-major, contiguous-per-sequence) layout.
* ``ref``   – the reference's own CPU kernels
  (GLakeServe/csrc/cpu/attention.cpp, cache.cpp) compiled by
  oracle/build_ref.py into oracle/_ref/.  They only understand the upstream
  paged layout with block 16, so :func:`ref_decode_attn` first pushes every K/V
  row through the reference's ``reshape_and_cache`` with an identity block
  table and then calls ``paged_attention_v1`` (or ``_v2`` above 8192 tokens,
  the switch the reference makes at GLakeServe/vllm/attention/ops/paged_attn.py:116-117).
"""
import ctypes
import importlib.machinery
import importlib.util
import os
import subprocess

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
_PORT = None
_REF = {}

c_i64, c_i32, c_f32, c_vp = ctypes.c_int64, ctypes.c_int32, ctypes.c_float, ctypes.c_void_p


def load_port():
    """ctypes handle of the C restatement (built on demand with gcc)."""
    global _PORT
    if _PORT is None:
        so = os.path.join(HERE, "libvt_oracle.so")
        src = os.path.join(HERE, "vt_oracle.c")
        if not os.path.isfile(so) or os.path.getmtime(so) < os.path.getmtime(src):
            subprocess.check_call(["make", "-C", HERE, "-B", "libvt_oracle.so"],
                                  stdout=subprocess.DEVNULL)
        lib = ctypes.CDLL(so)
        lib.vto_f32_to_e4m3.restype = ctypes.c_uint8
        lib.vto_f32_to_e4m3.argtypes = [c_f32]
        lib.vto_e4m3_to_f32.restype = c_f32
        lib.vto_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        _PORT = lib
    return _PORT


def _cpu_has(flag):
    try:
        with open("/proc/cpuinfo") as f:
            return flag in f.read()
    except OSError:
        return False


def load_ref(variant=None):
    """The compiled reference CPU kernels, or None when they cannot run here.

    variant: "bf16" (AVX512-BF16 build, rounds outputs to nearest even) or
    "nobf16" (plain AVX-512 build, truncates outputs to bf16).  Default: the
    best one this CPU supports.
    """
    if variant is None:
        if not _cpu_has("avx512f"):
            return None
        variant = "bf16" if _cpu_has("avx512_bf16") else "nobf16"
    if variant in _REF:
        return _REF[variant]
    name = "vt_ref_" + variant
    path = os.path.join(HERE, "_ref", name + ".so")
    mod = None
    if os.path.isfile(path):
        try:
            loader = importlib.machinery.ExtensionFileLoader(name, path)
            spec = importlib.util.spec_from_loader(name, loader)
            mod = importlib.util.module_from_spec(spec)
            loader.exec_module(mod)
        except (ImportError, OSError):
            mod = None
    _REF[variant] = mod
    return mod


# --------------------------------------------------------------------------
# host-memory stand-in for the per-slot virtual ranges
# --------------------------------------------------------------------------

class HostRanges:
    """One K and one V byte range per slot in host memory plus the two pointer
    tables, shaped like the device-side tables (index = slot id)."""

    def __init__(self, n_slots, range_bytes):
        self.k = [torch.zeros(range_bytes, dtype=torch.uint8) for _ in range(n_slots)]
        self.v = [torch.zeros(range_bytes, dtype=torch.uint8) for _ in range(n_slots)]
        self.k_table = torch.tensor([t.data_ptr() for t in self.k], dtype=torch.int64)
        self.v_table = torch.tensor([t.data_ptr() for t in self.v], dtype=torch.int64)

    def k_rows(self, slot, n_tokens, kvh, d, fp8=False):
        return _rows(self.k[slot], n_tokens, kvh, d, fp8)

    def v_rows(self, slot, n_tokens, kvh, d, fp8=False):
        return _rows(self.v[slot], n_tokens, kvh, d, fp8)


def _rows(buf, n, kvh, d, fp8):
    if fp8:
        return buf[: n * kvh * d].view(n, kvh, d)
    return buf[: n * kvh * d * 2].view(torch.bfloat16).view(n, kvh, d)


def _p(t):
    return c_vp(t.data_ptr()) if t is not None else c_vp(0)


def port_append(ranges, key, value, byte_off, slot_ids, seq_lens=None, cache_seq_lens=None,
                max_seq_len=1, k_scale=None, v_scale=None):
    """reshape_and_cache on host ranges. key/value: [tokens, KVH, D] bf16 (dim-0 stride free)."""
    lib = load_port()
    b = slot_ids.numel()
    kvh, d = key.shape[1], key.shape[2]
    seq_lens = seq_lens if seq_lens is not None else torch.ones(b, dtype=torch.int32)
    cache_seq_lens = cache_seq_lens if cache_seq_lens is not None else torch.zeros(b, dtype=torch.int32)
    args = [_p(key), _p(value), c_i64(key.stride(0)), c_i64(value.stride(0)),
            _p(ranges.k_table), _p(ranges.v_table), _p(byte_off), _p(slot_ids),
            _p(seq_lens), _p(cache_seq_lens), ctypes.c_int(max_seq_len), ctypes.c_int(b),
            ctypes.c_int(kvh), ctypes.c_int(d)]
    if k_scale is None:
        lib.vto_append_bf16(*args)
    else:
        lib.vto_append_fp8(*args, _p(k_scale), _p(v_scale))


def port_kv_scales(x):
    """x: [tokens, KVH, D] bf16 -> float32 [KVH] = amax / 448."""
    lib = load_port()
    out = torch.empty(x.shape[1], dtype=torch.float32)
    lib.vto_kv_scales(_p(x), c_i64(x.stride(0)), ctypes.c_int(x.shape[0]),
                      ctypes.c_int(x.shape[1]), ctypes.c_int(x.shape[2]), _p(out))
    return out


def port_decode_attn(q, ranges, slot_ids, seq_lens, kvh, scale, k_scale=None, v_scale=None,
                     return_lse=False):
    """q: [B, H, D] bf16 -> out [B, H, D] bf16 (and lse [B, H] fp32)."""
    lib = load_port()
    b, h, d = q.shape
    out = torch.empty(b, h, d, dtype=torch.bfloat16)
    lse = torch.empty(b, h, dtype=torch.float32) if return_lse else None
    lib.vto_decode_attn(_p(out), c_i64(h * d), _p(q), c_i64(q.stride(0)), _p(ranges.k_table),
                        _p(ranges.v_table), _p(slot_ids), _p(seq_lens), ctypes.c_int(b),
                        ctypes.c_int(h), ctypes.c_int(kvh), ctypes.c_int(d), c_f32(scale),
                        ctypes.c_int(0 if k_scale is None else 1), _p(k_scale), _p(v_scale),
                        _p(lse))
    return (out, lse) if return_lse else out


def port_prefill_attn(q, ranges, slot_ids, seq_lens, q_lens, q_start, kvh, scale,
                      k_scale=None, v_scale=None):
    """q: [tokens, H, D] bf16; causal attention of the new tokens over the range."""
    lib = load_port()
    n, h, d = q.shape
    out = torch.zeros(n, h, d, dtype=torch.bfloat16)
    lib.vto_prefill_attn(_p(out), c_i64(h * d), _p(q), c_i64(q.stride(0)), _p(ranges.k_table),
                         _p(ranges.v_table), _p(slot_ids), _p(seq_lens), _p(q_lens), _p(q_start),
                         ctypes.c_int(slot_ids.numel()), ctypes.c_int(h), ctypes.c_int(kvh),
                         ctypes.c_int(d), c_f32(scale), ctypes.c_int(0 if k_scale is None else 1),
                         _p(k_scale), _p(v_scale))
    return out


def port_rotary_embedding(positions, query, key, head_size, cos_sin_cache, is_neox=True):
    """Rotates query [T, H*D] and key [T, KVH*D] (bf16, dim-0 stride free) in place."""
    lib = load_port()
    lib.vto_rotary_embedding(_p(positions), _p(query), _p(key), _p(cos_sin_cache),
                             ctypes.c_int(cos_sin_cache.shape[1]), c_i64(query.stride(0)),
                             c_i64(key.stride(0)), ctypes.c_int(query.shape[-1] // head_size),
                             ctypes.c_int(key.shape[-1] // head_size), ctypes.c_int(head_size),
                             ctypes.c_int(query.shape[0]), ctypes.c_int(1 if is_neox else 0))


def port_rms_norm(out, input, weight, epsilon, residual=None):
    """out = rms_norm(input [+ residual, stored back]) * weight; contiguous bf16 [T, hidden]."""
    lib = load_port()
    lib.vto_rms_norm(_p(out), _p(input), _p(residual), _p(weight), c_f32(epsilon),
                     ctypes.c_int(input.shape[0]), ctypes.c_int(input.shape[1]))


def make_cos_sin_cache(max_position, rot_dim, base=10000.0):
    """The table RotaryEmbedding builds
    (GLakeServe/vllm/model_executor/layers/rotary_embedding.py:71-93), in bf16.
    Evaluated in float64 so that the bf16 table does not depend on which
    vectorised cos/sin the host's math library picks."""
    import numpy as np
    inv_freq = 1.0 / (base ** (np.arange(0, rot_dim, 2, dtype=np.float64) / rot_dim))
    freqs = np.outer(np.arange(max_position, dtype=np.float64), inv_freq)
    table = np.concatenate((np.cos(freqs), np.sin(freqs)), axis=-1).astype(np.float32)
    return torch.from_numpy(table).to(torch.bfloat16)


def port_all_reduce(tensors):
    """Sum of the ranks' bf16 tensors the way the reference's custom all-reduce forms
    it (GLakeServe/csrc/custom_all_reduce.cuh:173-181): fp32 accumulation in rank
    order, one rounding to bf16."""
    acc = tensors[0].float()
    for t in tensors[1:]:
        acc = acc + t.float()
    return acc.to(torch.bfloat16)


def fill_ranges(k_list, v_list, range_bytes=None, k_scale=None, v_scale=None):
    """Build HostRanges holding the given per-sequence K/V ([L_i, KVH, D] bf16)
    by appending every row through the port's append (slot i = sequence i)."""
    n = len(k_list)
    kvh, d = k_list[0].shape[1], k_list[0].shape[2]
    e = 1 if k_scale is not None else 2
    need = max(k.shape[0] for k in k_list) * kvh * d * e
    r = HostRanges(n, range_bytes or need)
    lens = torch.tensor([k.shape[0] for k in k_list], dtype=torch.int32)
    starts = torch.zeros(n, dtype=torch.int32)
    starts[1:] = torch.cumsum(lens, 0)[:-1].to(torch.int32)
    port_append(r, torch.cat(k_list), torch.cat(v_list), torch.zeros(n, dtype=torch.int64),
                torch.arange(n, dtype=torch.int64), lens, starts, max_seq_len=int(lens.max()),
                k_scale=k_scale, v_scale=v_scale)
    return r


# --------------------------------------------------------------------------
# the reference's CPU kernels behind a layout adapter
# --------------------------------------------------------------------------

REF_BLOCK = 16          # static_assert(BLOCK_SIZE == 16), csrc/cpu/attention.cpp:236
REF_PARTITION = 512     # csrc/cpu/attention.cpp:656


class RefPagedCache:
    """Upstream paged bf16 cache filled through the reference's reshape_and_cache."""

    def __init__(self, ref, k_list, v_list):
        self.ref = ref
        kvh, d = k_list[0].shape[1], k_list[0].shape[2]
        self.kvh, self.d = kvh, d
        lens = [k.shape[0] for k in k_list]
        blocks = [(n + REF_BLOCK - 1) // REF_BLOCK for n in lens]
        self.max_blocks = max(max(blocks), 1)
        nb = sum(blocks) + 1
        x = 8  # 16 bytes / sizeof(bf16)
        self.key_cache = torch.zeros(nb, kvh, d // x, REF_BLOCK, x, dtype=torch.bfloat16)
        self.value_cache = torch.zeros(nb, kvh, d, REF_BLOCK, dtype=torch.bfloat16)
        self.block_tables = torch.zeros(len(k_list), self.max_blocks, dtype=torch.int32)
        base = 0
        slots = []
        for i, n in enumerate(lens):
            self.block_tables[i, : blocks[i]] = torch.arange(base, base + blocks[i], dtype=torch.int32)
            slots.append(torch.arange(n, dtype=torch.int64) + base * REF_BLOCK)
            base += blocks[i]
        self.seq_lens = torch.tensor(lens, dtype=torch.int32)
        self.append(torch.cat(k_list), torch.cat(v_list), torch.cat(slots))

    def append(self, key, value, slot_mapping):
        self.ref.reshape_and_cache(key.contiguous(), value.contiguous(), self.key_cache,
                                   self.value_cache, slot_mapping, "auto", 1.0)

    def gather(self, i):
        """Cache contents of sequence i back in [L, KVH, D] order (K, V)."""
        n = int(self.seq_lens[i])
        nb = (n + REF_BLOCK - 1) // REF_BLOCK
        blk = self.block_tables[i, :nb].long()
        k = self.key_cache[blk].permute(0, 3, 1, 2, 4).reshape(nb * REF_BLOCK, self.kvh, self.d)[:n]
        v = self.value_cache[blk].permute(0, 3, 1, 2).reshape(nb * REF_BLOCK, self.kvh, self.d)[:n]
        return k.contiguous(), v.contiguous()

    def attend(self, q, scale, force=None):
        b, h, d = q.shape
        out = torch.empty(b, h, d, dtype=torch.bfloat16)
        max_len = int(self.seq_lens.max())
        use_v2 = max_len > 8192 if force is None else force == "v2"
        if not use_v2:
            self.ref.paged_attention_v1(out, q, self.key_cache, self.value_cache, self.kvh,
                                        float(scale), self.block_tables, self.seq_lens, REF_BLOCK,
                                        max_len, None, "auto", 1.0)
        else:
            parts = (max_len + REF_PARTITION - 1) // REF_PARTITION
            tmp = torch.empty(b, h, parts, d, dtype=torch.bfloat16)
            es = torch.empty(b, h, parts, dtype=torch.float32)
            ml = torch.empty(b, h, parts, dtype=torch.float32)
            self.ref.paged_attention_v2(out, es, ml, tmp, q, self.key_cache, self.value_cache,
                                        self.kvh, float(scale), self.block_tables, self.seq_lens,
                                        REF_BLOCK, max_len, None, "auto", 1.0)
        return out


def ref_decode_attn(q, k_list, v_list, scale, variant=None, force=None):
    ref = load_ref(variant)
    if ref is None:
        raise RuntimeError("reference CPU kernels are not available on this machine")
    return RefPagedCache(ref, k_list, v_list).attend(q.contiguous(), scale, force)


# --------------------------------------------------------------------------
# plain fp32 PyTorch statement of the same math (third, independent witness)
# --------------------------------------------------------------------------

def torch_decode_attn(q, k_list, v_list, scale):
    """softmax(scale * q.K^T).V per sequence in fp32, as the reference's test
    states it (GLakeServe/tests/kernels/test_attention.py:43-111)."""
    b, h, d = q.shape
    out = torch.empty(b, h, d, dtype=torch.float32)
    for i in range(b):
        k, v = k_list[i].float(), v_list[i].float()
        g = h // k.shape[1]
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        w = torch.softmax(scale * torch.einsum("hd,thd->ht", q[i].float(), k), dim=-1)
        out[i] = torch.einsum("ht,thd->hd", w, v)
    return out
