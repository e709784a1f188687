"""Deterministic synthetic inputs for the parity tests and the golden fixtures.

numpy's legacy RandomState stream is frozen across numpy versions, so a seed
identifies the inputs for good; fixtures therefore store outputs plus a digest
of the inputs instead of the inputs themselves.
"""
import hashlib

import numpy as np
import torch


def normal_bf16(rs, *shape):
    return torch.from_numpy(rs.standard_normal(shape).astype(np.float32)).bfloat16()


def make_case(seed, lens, h, kvh, d=128):
    """Q [B,H,D]; per-sequence K, V [L_i, KVH, D]; all ~N(0,1) rounded to bf16.
    lens are context lengths INCLUDING the token appended in the decode step."""
    rs = np.random.RandomState(seed)
    q = normal_bf16(rs, len(lens), h, d)
    k = [normal_bf16(rs, n, kvh, d) for n in lens]
    v = [normal_bf16(rs, n, kvh, d) for n in lens]
    return q, k, v


def uniform_lens(seed, batch, lo, hi):
    rs = np.random.RandomState(seed + 7919)
    return [int(x) for x in rs.randint(lo, hi + 1, size=batch)]


def digest(*tensors):
    m = hashlib.sha256()
    for t in tensors:
        for x in (t if isinstance(t, (list, tuple)) else [t]):
            m.update(x.contiguous().view(torch.uint8).numpy().tobytes())
    return m.hexdigest()


# name -> (seed, lens or ("uniform", batch, lo, hi), H, KVH)
GOLDEN_CASES = {
    "gqa4_small": (1, [37, 512, 100, 16], 8, 2),
    "mha_edges": (2, [1, 2, 255, 256, 257], 4, 4),
    "mha_chunk_cross": (3, [1023, 1024, 1025], 8, 8),
    "gqa8": (4, [300, 2049, 64], 16, 2),
    "long_partitioned": (5, [9000, 8193], 8, 1),
    "config1_op": (0, ("uniform", 8, 512, 2048), 32, 32),
}


# Real-data cases at the context lengths of the long-context / fp8 / tensor-parallel
# configurations (name -> (seed, lens, H, KVH)); goldens come from the reference's CPU
# paged_attention_v2 (v1 up to 8192 tokens).  "fp8_ctx" is run with a bf16 cache by the
# reference (it has no fp8 kernel) and with both cache types by the GPU tests.
LONG_CASES = {
    "long_gqa4_32k": (6, [16384, 32768, 20011, 29999], 32, 8),
    "fp8_ctx_gqa4_8k": (7, [2048, 8192, 5000, 3333, 7777, 4097], 32, 8),
    "share_tp8_16k": (8, [4096, 16384, 9001, 12345], 8, 1),
    "share_tp4_16k": (9, [4099, 16384, 8192, 15000], 16, 2),
}


def golden_lens(name):
    seed, lens, h, kvh = GOLDEN_CASES[name] if name in GOLDEN_CASES else LONG_CASES[name]
    if isinstance(lens, tuple):
        lens = uniform_lens(seed, *lens[1:])
    return seed, lens, h, kvh


# name -> (seed, tokens, H, KVH, rot_dim, is_neox, max_position)
ROPE_CASES = {
    "rope_neox": (11, 12, 4, 2, 128, True, 4096),
    "rope_gptj_partial": (12, 9, 4, 1, 64, False, 2048),
}
# name -> (seed, tokens, hidden, epsilon)
NORM_CASES = {
    "norm_1024": (21, 6, 1024, 1e-5),
    "norm_4096": (22, 3, 4096, 1e-6),
}


def make_rope_case(seed, tokens, h, kvh, max_position, d=128):
    """positions int64 [T]; q [T, H*D]; k, v [T, KVH*D] ~N(0,1) bf16."""
    rs = np.random.RandomState(seed)
    pos = torch.from_numpy(rs.randint(0, max_position, size=tokens).astype(np.int64))
    return pos, normal_bf16(rs, tokens, h * d), normal_bf16(rs, tokens, kvh * d), normal_bf16(rs, tokens, kvh * d)


def make_norm_case(seed, tokens, hidden):
    """x, residual [T, hidden] ~N(0,1); weight [hidden] ~ 1 + 0.1 N(0,1); bf16."""
    rs = np.random.RandomState(seed)
    x, r = normal_bf16(rs, tokens, hidden), normal_bf16(rs, tokens, hidden)
    w = torch.from_numpy((1.0 + 0.1 * rs.standard_normal(hidden)).astype(np.float32)).bfloat16()
    return x, r, w


# name -> (seed, contexts, new tokens per sequence, H, KVH): causal attention of the new tokens over prefix + new
PREFILL_CASES = {
    "prefill_gqa4": (41, [37, 130, 64], [37, 50, 1], 8, 2),
    "prefill_mha_tile_edges": (42, [128, 129, 200], [128, 65, 127], 4, 4),
}


def make_prefill_queries(seed, q_lens, h, d=128):
    rs = np.random.RandomState(seed + 4242)
    return normal_bf16(rs, int(sum(q_lens)), h, d)
