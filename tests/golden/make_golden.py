"""Generates tests/golden/*.npz from the reference's own CPU kernels.

Runs only where the reference checkout and oracle/_ref exist (build them with
`python oracle/build_ref.py`).  For every case in tests/synth.py:GOLDEN_CASES
the flow is the decode step the reference performs: all but the last token of
every sequence are written with the reference's CPU reshape_and_cache
(GLakeServe/csrc/cpu/cache.cpp:103-128), the last token is appended by a second
call, then paged_attention_v1 / _v2 (GLakeServe/csrc/cpu/attention.cpp:415-430,
:730-746) produce the outputs that are stored.  Stored per case: output bits
(uint16 view of bf16), context lengths, a sha256 of the inputs, and a sha256 of
the cache contents gathered back to [token, kv_head, d] order.

tests/synth.py:ROPE_CASES and NORM_CASES go through the reference's CPU
rotary_embedding (GLakeServe/csrc/cpu/pos_encoding.cpp:169-198) and rms_norm /
fused_add_rms_norm (GLakeServe/csrc/cpu/layernorm.cpp:90-117); the rotated q / k
and the normalised rows are stored as bf16 bit patterns.

tests/synth.py:PREFILL_CASES: the reference's CPU backend has no prefix-prefill kernel
(its prompt path is xformers), so every new token is run through the reference's
CPU paged_attention_v1 as a decode query of its own over the tokens it may see
(context = its position + 1), which is what causal attention over prefix + new
tokens means; the outputs are stored in query order.

tests/synth.py:LONG_CASES are the same decode flow at the context lengths of the
long-context, fp8 and tensor-parallel configurations (up to 32 768 tokens, which
takes the reference's paged_attention_v2 and its 512-token partitions).

Usage: python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from tests import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def run_case(name):
    seed, lens, h, kvh = synth.golden_lens(name)
    q, k, v = synth.make_case(seed, lens, h, kvh)
    ref = O.load_ref("bf16")
    assert ref is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    # prefill all but the last token, then append the last one (decode step)
    # Blocks are sized for L tokens with the last row zeroed; token L-1 then goes
    # through the reference kernel in a second call.
    cache = O.RefPagedCache(ref, [torch.cat([x[:-1], torch.zeros_like(x[-1:])]) for x in k],
                            [torch.cat([x[:-1], torch.zeros_like(x[-1:])]) for x in v])
    last_slots = torch.tensor(
        [int(cache.block_tables[i, (n - 1) // O.REF_BLOCK]) * O.REF_BLOCK + (n - 1) % O.REF_BLOCK
         for i, n in enumerate(lens)], dtype=torch.int64)
    cache.append(torch.stack([x[-1] for x in k]), torch.stack([x[-1] for x in v]), last_slots)
    gathered = [cache.gather(i) for i in range(len(lens))]
    for i in range(len(lens)):
        assert torch.equal(gathered[i][0], k[i]) and torch.equal(gathered[i][1], v[i])
    scale = 128 ** -0.5
    out = cache.attend(q, scale)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        out_bits=out.view(torch.uint16).numpy(),
        lens=np.asarray(lens, dtype=np.int32),
        shape=np.asarray([len(lens), h, kvh, 128], dtype=np.int32),
        seed=np.asarray(seed),
        input_sha256=np.asarray(synth.digest(q, k, v)),
        cache_sha256=np.asarray(synth.digest([g[0] for g in gathered], [g[1] for g in gathered])),
        kernel=np.asarray("v2" if max(lens) > 8192 else "v1"),
    )
    print(name, "lens", lens[:8], "out", tuple(out.shape), "max|out|", float(out.float().abs().max()))


def bits(t):
    return t.contiguous().view(torch.uint16).numpy()


def run_rope_case(name):
    seed, tokens, h, kvh, rot, neox, max_pos = synth.ROPE_CASES[name]
    ref = O.load_ref("bf16")
    pos, q, k, v = synth.make_rope_case(seed, tokens, h, kvh, max_pos)
    cs = O.make_cos_sin_cache(max_pos, rot)
    sha = synth.digest(pos, q, k, v, cs)
    ref.rotary_embedding(pos, q, k, 128, cs, neox)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), q_bits=bits(q), k_bits=bits(k),
                        input_sha256=np.asarray(sha))
    print(name, "q", tuple(q.shape), "k", tuple(k.shape))


def run_norm_case(name):
    seed, tokens, hidden, eps = synth.NORM_CASES[name]
    ref = O.load_ref("bf16")
    x, r, w = synth.make_norm_case(seed, tokens, hidden)
    sha = synth.digest(x, r, w)
    plain = torch.empty_like(x)
    ref.rms_norm(plain, x, w, eps)
    fx, fr = x.clone(), r.clone()
    ref.fused_add_rms_norm(fx, fr, w, eps)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), plain_bits=bits(plain), fused_bits=bits(fx),
                        residual_bits=bits(fr), input_sha256=np.asarray(sha))
    print(name, tuple(x.shape))


def run_prefill_case(name):
    seed, lens, q_lens, h, kvh = synth.PREFILL_CASES[name]
    _, k, v = synth.make_case(seed, lens, h, kvh)
    q = synth.make_prefill_queries(seed, q_lens, h)
    ref = O.load_ref("bf16")
    cache = O.RefPagedCache(ref, k, v)
    rows, tables, ctx = [], [], []
    start = 0
    for i, (n, m) in enumerate(zip(lens, q_lens)):
        for j in range(m):
            rows.append(q[start + j])
            tables.append(cache.block_tables[i])
            ctx.append(n - m + j + 1)
        start += m
    qq = torch.stack(rows).contiguous()
    out = torch.empty_like(qq)
    ref.paged_attention_v1(out, qq, cache.key_cache, cache.value_cache, kvh, float(128 ** -0.5), torch.stack(tables).contiguous(),
                           torch.tensor(ctx, dtype=torch.int32), O.REF_BLOCK, max(ctx), None, "auto", 1.0)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), out_bits=bits(out),
                        input_sha256=np.asarray(synth.digest(q, k, v)))
    print(name, "queries", tuple(qq.shape), "max|out|", float(out.float().abs().max()))


if __name__ == "__main__":
    for name in list(synth.GOLDEN_CASES) + list(synth.LONG_CASES):
        run_case(name)
    for name in synth.ROPE_CASES:
        run_rope_case(name)
    for name in synth.NORM_CASES:
        run_norm_case(name)
    for name in synth.PREFILL_CASES:
        run_prefill_case(name)
