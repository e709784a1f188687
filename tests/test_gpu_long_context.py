"""GPU parity at the context lengths the long-context, fp8 and tensor-parallel
configurations really run at, on real N(0,1) data (not structured inputs), so that
the running-max rescale and the cross-piece / cross-partition merges are exercised
numerically over tens of thousands of tokens.

Checkers: the committed golden vectors made by the reference's own CPU kernels
(GLakeServe/csrc/cpu/attention.cpp:433-746, paged_attention_v2 with its 512-token
partitions above 8192 tokens, v1 below), the C restatement, and — when the compiled
reference kernels load on this host — those kernels run live.

Tolerances: bf16 cache <= 2e-3 max-abs; fp8 cache <= 3e-2 against the bf16-cache
result and <= 1e-2 against the fp8 restatement (the reference's own fp8 tolerance,
GLakeServe/tests/kernels/test_attention.py:271-274); cache bytes bit-exact.
"""
import numpy as np
import pytest
import torch

from tests import synth
from tests.test_oracle import SCALE, load_golden

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    from tests import gpu_util
    gpu_util.ensure_pool()
    return gpu_util


@pytest.fixture
def tuning():
    from glake_b200 import ops
    yield ops.set_attn_tuning
    ops.set_attn_tuning("auto")


def max_err(a, b):
    return float((a.float() - b.float()).abs().max())


# (planner override, forced split count)
BF16_MODES = [("auto", 0), ("flat", 0), ("mma", 0), ("mma", 4), ("mma", 61), ("simt", 0), ("simt", 7)]


@pytest.mark.parametrize("name", list(synth.LONG_CASES))
def test_long_context_real_data_against_the_reference(G, oracle, tuning, name):
    z, gold = load_golden(name)
    seed, lens, h, kvh = synth.golden_lens(name)
    q, k, v = synth.make_case(seed, lens, h, kvh)
    assert synth.digest(q, k, v) == str(z["input_sha256"])
    kv = G.GpuKV(k, v, kvh)
    try:
        rows_k = [kv.read_rows(i, "k") for i in range(len(lens))]
        rows_v = [kv.read_rows(i, "v") for i in range(len(lens))]
        assert synth.digest(rows_k, rows_v) == str(z["cache_sha256"]), "cache contents are not bit-exact"
        del rows_k, rows_v
        r = oracle.fill_ranges(k, v)
        port = oracle.port_decode_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32), kvh, SCALE)
        live = None
        if oracle.load_ref() is not None:
            live = oracle.ref_decode_attn(q, k, v, SCALE)
        for mode, splits in BF16_MODES:
            tuning(mode)
            out = kv.attend(q, SCALE, num_splits=splits)
            assert max_err(out, gold) <= 2e-3, (mode, splits, "golden", max_err(out, gold))
            assert max_err(out, port) <= 2e-3, (mode, splits, "restatement", max_err(out, port))
            if live is not None:
                assert max_err(out, live) <= 2e-3, (mode, splits, "live reference", max_err(out, live))
        tuning("auto")
        out, lse = kv.attend(q, SCALE, return_lse=True)
        _, plse = oracle.port_decode_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32), kvh,
                                          SCALE, return_lse=True)
        assert torch.allclose(lse, plse, atol=2e-3)
    finally:
        kv.close()


@pytest.mark.parametrize("name", ["fp8_ctx_gqa4_8k", "share_tp8_16k"])
def test_fp8_cache_at_full_context_with_scales_from_the_prefill_append(G, oracle, tuning, name):
    """Scales are amax / 448 per kv head over the PREFILL rows (vt_kv_scales at the first
    append), frozen; the decode step's row is quantised with them and saturates if larger."""
    from glake_b200 import ops
    _, gold16 = load_golden(name)
    seed, lens, h, kvh = synth.golden_lens(name)
    q, k, v = synth.make_case(seed, lens, h, kvh)
    pre_k = torch.cat([x[:-1] for x in k])
    pre_v = torch.cat([x[:-1] for x in v])
    ks = ops.kv_scales(pre_k.cuda(), kvh, 128)
    vs = ops.kv_scales(pre_v.cuda(), kvh, 128)
    assert torch.equal(ks.cpu(), oracle.port_kv_scales(pre_k)) and torch.equal(vs.cpu(), oracle.port_kv_scales(pre_v))
    kv8 = G.GpuKV(k, v, kvh, fp8=True, k_scale=ks, v_scale=vs)
    try:
        r8 = oracle.fill_ranges(k, v, k_scale=ks.cpu(), v_scale=vs.cpu())
        for i, n in enumerate(lens):
            assert torch.equal(kv8.read_rows(i, "k"), r8.k_rows(i, n, kvh, 128, fp8=True))
            assert torch.equal(kv8.read_rows(i, "v"), r8.v_rows(i, n, kvh, 128, fp8=True))
        port8 = oracle.port_decode_attn(q, r8, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32), kvh,
                                        SCALE, ks.cpu(), vs.cpu())
        for mode, splits in [("auto", 0), ("flat", 0), ("simt", 0), ("simt", 5)]:
            tuning(mode)
            o8 = kv8.attend(q, SCALE, num_splits=splits)
            assert max_err(o8, gold16) <= 3e-2, (mode, splits, "vs bf16-cache reference", max_err(o8, gold16))
            assert max_err(o8, port8) <= 1e-2, (mode, splits, "vs fp8 restatement", max_err(o8, port8))
    finally:
        kv8.close()


@pytest.mark.parametrize("h,kvh,fp8", [(8, 1, False), (2, 2, False), (4, 2, False), (8, 1, True), (4, 2, True),
                                        (8, 4, True)])
def test_many_short_streams_per_cta(G, oracle, tuning, h, kvh, fp8):
    """Around a thousand contexts of 1..150 tokens: every CTA of the persistent
    schedule walks through several whole streams, each published to and merged
    from the same scratch slot, with warps that own no merge item running ahead."""
    from glake_b200 import ops
    rs = np.random.RandomState(5150 + h + kvh)
    lens = [int(x) for x in rs.randint(1, 151, size=1000)]
    q, k, v = synth.make_case(900 + h + kvh, lens, h, kvh)
    ks = vs = None
    if fp8:
        ks = ops.kv_scales(torch.cat(k).cuda(), kvh, 128)
        vs = ops.kv_scales(torch.cat(v).cuda(), kvh, 128)
    kv = G.GpuKV(k, v, kvh, fp8=fp8, k_scale=ks, v_scale=vs)
    try:
        tuning("flat")
        outs = [kv.attend(q, SCALE) for _ in range(3)]
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), "results differ between identical calls"
        sl = torch.tensor(lens, dtype=torch.int32)
        if fp8:
            r = oracle.fill_ranges(k, v, k_scale=ks.cpu(), v_scale=vs.cpu())
            port = oracle.port_decode_attn(q, r, torch.arange(len(lens)), sl, kvh, SCALE, ks.cpu(), vs.cpu())
            err = (outs[0].float() - port.float()).abs()
            tol = torch.maximum(torch.full_like(err, 3e-2), port.float().abs() * 2.0 ** -6)
        else:
            r = oracle.fill_ranges(k, v)
            port = oracle.port_decode_attn(q, r, torch.arange(len(lens)), sl, kvh, SCALE)
            err = (outs[0].float() - port.float()).abs()
            tol = torch.maximum(torch.full_like(err, 2e-3), port.float().abs() * 2.0 ** -7)
        assert bool((err <= tol).all()), float((err - tol).max())
    finally:
        kv.close()


def test_fp8_decode_runner_two_layers_with_overlap_requested(G, oracle):
    """An fp8 cache takes append + attention as two launches per layer; asking the
    runner for layer-to-layer overlap must not let the attention read its newest row
    before the append wrote it."""
    from glake_b200 import ops
    from glake_b200.backend import DecodeRunner, VTensorAttentionImpl, VTensorCacheEngine, VTensorMetadata, prepare_step
    h, kvh, layers = 8, 8, 2
    lens0 = [300, 2, 1500, 65, 700, 129]
    rs = np.random.RandomState(4242)
    eng = VTensorCacheEngine(layers, kvh, 128, len(lens0), 2048, cache_dtype="fp8_e4m3")
    impl = VTensorAttentionImpl(h, 128, SCALE, kvh, kv_cache_dtype="fp8_e4m3")
    try:
        pre = [n - 1 for n in lens0]
        hist_k = [[synth.normal_bf16(rs, n, kvh, 128) for n in pre] for _ in range(layers)]
        hist_v = [[synth.normal_bf16(rs, n, kvh, 128) for n in pre] for _ in range(layers)]
        ks = torch.stack([ops.kv_scales(torch.cat(hist_k[l]).cuda(), kvh, 128) for l in range(layers)])
        vs = torch.stack([ops.kv_scales(torch.cat(hist_v[l]).cuda(), kvh, 128) for l in range(layers)])
        slots = list(range(len(lens0)))
        meta = VTensorMetadata(slots, pre, kvh, 128, num_prefills=len(pre), kv_elem_size=1)
        prepare_step(meta, eng)
        for l in range(layers):
            ops.reshape_and_cache(torch.cat(hist_k[l]).cuda(), torch.cat(hist_v[l]).cuda(), eng.k_cache_ptr[l],
                                  eng.v_cache_ptr[l], meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor,
                                  meta.cache_seq_lens, max(pre), kvh, 128, "fp8_e4m3", ks[l], vs[l])
        runner = DecodeRunner(eng, impl, len(lens0), host_io=False, k_scale=ks, v_scale=vs, overlap=True)
        lens = list(pre)
        for step in range(4):
            lens = [n + 1 for n in lens]
            q = synth.normal_bf16(rs, layers, len(lens), h * 128)
            nk = synth.normal_bf16(rs, layers, len(lens), kvh * 128)
            nv = synth.normal_bf16(rs, layers, len(lens), kvh * 128)
            runner.q.copy_(q), runner.k.copy_(nk), runner.v.copy_(nv)
            runner.step(VTensorMetadata(slots, lens, kvh, 128, num_decode_tokens=len(lens), kv_elem_size=1))
            runner.synchronize()
            for l in range(layers):
                hist_k[l] = [torch.cat([a, b.view(1, kvh, 128)]) for a, b in zip(hist_k[l], nk[l])]
                hist_v[l] = [torch.cat([a, b.view(1, kvh, 128)]) for a, b in zip(hist_v[l], nv[l])]
                r = oracle.fill_ranges(hist_k[l], hist_v[l], k_scale=ks[l].cpu(), v_scale=vs[l].cpu())
                port = oracle.port_decode_attn(q[l].view(len(lens), h, 128), r, torch.arange(len(lens)),
                                               torch.tensor(lens, dtype=torch.int32), kvh, SCALE, ks[l].cpu(), vs[l].cpu())
                got = runner.out[l].view(len(lens), h, 128).cpu()
                err = (got.float() - port.float()).abs()
                tol = torch.maximum(torch.full_like(err, 1e-2), port.float().abs() * 2.0 ** -6)
                assert bool((err <= tol).all()), (step, l, float((err - tol).max()))
        assert runner.status() == 0
    finally:
        eng.close()


@pytest.mark.parametrize("h,kvh", [(8, 2), (8, 8), (6, 3)])
def test_backend_prompt_extend_decode_over_an_fp8_cache(G, oracle, h, kvh):
    """The backend binding with an fp8 cache end to end: a prompt (scales = amax / 448 of
    its rows, computed at that first append and frozen), a prefix-extend step, then decode
    steps, two layers.  The prompt kernels run over widened scratch ranges; every phase is
    compared with the fp8 restatement (which dequantises to bf16 exactly as the widening
    does) and the cache bytes with its bytes."""
    from glake_b200 import ops
    from glake_b200.backend import VTensorAttentionImpl, VTensorCacheEngine, VTensorMetadata, prepare_step
    layers = 2
    eng = VTensorCacheEngine(layers, kvh, 128, 4, 2048, cache_dtype="fp8_e4m3")
    impl = VTensorAttentionImpl(h, 128, SCALE, kvh, kv_cache_dtype="fp8_e4m3")
    rs = np.random.RandomState(79 + kvh)
    slots, ctx = [1, 2], [0, 0]
    hist_k = [[torch.empty(0, kvh, 128, dtype=torch.bfloat16) for _ in slots] for _ in range(layers)]
    hist_v = [[torch.empty(0, kvh, 128, dtype=torch.bfloat16) for _ in slots] for _ in range(layers)]
    scales = [None] * layers
    try:
        for phase, new in enumerate([[300, 77], [50, 200], [1, 1], [1, 1]]):
            decode = phase >= 2
            ctx = [a + b for a, b in zip(ctx, new)]
            if decode:
                meta = VTensorMetadata(slots, ctx, kvh, 128, num_decode_tokens=2, kv_elem_size=1)
            else:
                meta = VTensorMetadata(slots, ctx, kvh, 128, num_prefills=2, query_lens=new, kv_elem_size=1)
            prepare_step(meta, eng)
            n, starts = sum(new), [0, new[0]]
            for layer in range(layers):
                q = synth.normal_bf16(rs, n, h * 128)
                kk = synth.normal_bf16(rs, n, kvh * 128)
                vv = synth.normal_bf16(rs, n, kvh * 128)
                if scales[layer] is None:
                    scales[layer] = (ops.kv_scales(kk.cuda(), kvh, 128), ops.kv_scales(vv.cuda(), kvh, 128))
                ks, vs = scales[layer]
                kc, vc = eng.gpu_cache[layer]
                out = impl.forward(q.cuda(), kk.cuda(), vv.cuda(), kc, vc, meta, k_scale=ks, v_scale=vs).cpu()
                for i in range(2):
                    rows = slice(starts[i], starts[i] + new[i])
                    hist_k[layer][i] = torch.cat([hist_k[layer][i], kk[rows].view(-1, kvh, 128)])
                    hist_v[layer][i] = torch.cat([hist_v[layer][i], vv[rows].view(-1, kvh, 128)])
                r = oracle.fill_ranges(hist_k[layer], hist_v[layer], k_scale=ks.cpu(), v_scale=vs.cpu())
                port = oracle.port_prefill_attn(q.view(n, h, 128), r, torch.arange(2), torch.tensor(ctx, dtype=torch.int32),
                                                torch.tensor(new, dtype=torch.int32), torch.tensor(starts, dtype=torch.int32),
                                                kvh, SCALE, ks.cpu(), vs.cpu())
                err = (out.view(n, h, 128).float() - port.float()).abs()
                # prompt phases: same dequantised values as the restatement -> the bf16 tolerance (one ulp
                # where short contexts make outputs O(1)); decode phases: the fp8 tolerance of the decode kernel
                base = 1e-2 if decode else 2e-3
                tol = torch.maximum(torch.full_like(err, base), port.float().abs() * (2.0 ** -6 if decode else 2.0 ** -7))
                assert bool((err <= tol).all()), (phase, layer, float((err - tol).max()))
    finally:
        eng.close()


@pytest.mark.parametrize("h,kvh,fp8", [(8, 1, False), (8, 8, False), (8, 8, True)])
def test_early_kv_launch_reads_inputs_the_preceding_kernel_produces(G, oracle, h, kvh, fp8):
    """With other kernels between the layers' attention launches the runner uses the
    early-KV form of the step: launched as a programmatic dependent, it may stream old
    cache rows while the kernel in front of it still runs, but must not read q / k / v
    before that kernel finished.  Here that kernel is a one-rank vt_all_reduce (a copy
    that releases its dependents at once) which WRITES the next layer's q, k and v over
    NaN-filled buffers."""
    import ctypes
    from glake_b200 import ops
    from glake_b200.backend import DecodeRunner, VTensorAttentionImpl, VTensorCacheEngine, VTensorMetadata, prepare_step
    from tests.test_gpu_allreduce import Emulated
    layers, lens0 = 3, [300, 2, 1500, 65, 700, 129]
    b = len(lens0)
    dt = "fp8_e4m3" if fp8 else "auto"
    rs = np.random.RandomState(777 + kvh)
    eng = VTensorCacheEngine(layers, kvh, 128, b, 2048, cache_dtype=dt)
    impl = VTensorAttentionImpl(h, 128, SCALE, kvh, kv_cache_dtype=dt)
    E = Emulated(1, max_bytes=1 << 20)
    try:
        pre = [n - 1 for n in lens0]
        hist_k = [[synth.normal_bf16(rs, n, kvh, 128) for n in pre] for _ in range(layers)]
        hist_v = [[synth.normal_bf16(rs, n, kvh, 128) for n in pre] for _ in range(layers)]
        ks = vs = None
        if fp8:
            ks = torch.stack([ops.kv_scales(torch.cat(hist_k[l]).cuda(), kvh, 128) for l in range(layers)])
            vs = torch.stack([ops.kv_scales(torch.cat(hist_v[l]).cuda(), kvh, 128) for l in range(layers)])
        slots = list(range(b))
        meta = VTensorMetadata(slots, pre, kvh, 128, num_prefills=b, kv_elem_size=1 if fp8 else 2)
        prepare_step(meta, eng)
        for l in range(layers):
            ops.reshape_and_cache(torch.cat(hist_k[l]).cuda(), torch.cat(hist_v[l]).cuda(), eng.k_cache_ptr[l],
                                  eng.v_cache_ptr[l], meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor,
                                  meta.cache_seq_lens, max(pre), kvh, 128, dt, ks[l] if fp8 else None,
                                  vs[l] if fp8 else None)
        src = {}

        def produce_next_inputs(layer):
            nxt = layer + 1
            if nxt >= layers:
                return
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            for name in ("q", "k", "v"):
                dst = getattr(runner, name)[nxt]
                E.check(E.lib.vt_all_reduce(E.ars[0], ctypes.c_void_p(src[name][nxt].data_ptr()),
                                            ctypes.c_void_p(dst.data_ptr()), dst.numel(), stream), "vt_all_reduce")

        runner = DecodeRunner(eng, impl, b, host_io=False, k_scale=ks, v_scale=vs, overlap=True,
                              post_layer=produce_next_inputs, launches_per_post_layer=3)
        assert runner._overlap_mode(1) == "early_kv"
        for name in ("q", "k", "v"):
            src[name] = torch.zeros_like(getattr(runner, name))
        lens = list(pre)
        for step in range(3):
            lens = [n + 1 for n in lens]
            q = synth.normal_bf16(rs, layers, b, h * 128)
            nk = synth.normal_bf16(rs, layers, b, kvh * 128)
            nv = synth.normal_bf16(rs, layers, b, kvh * 128)
            src["q"].copy_(q), src["k"].copy_(nk), src["v"].copy_(nv)
            for name, t in (("q", q), ("k", nk), ("v", nv)):       # layer 0 gets its inputs directly, the others NaN
                getattr(runner, name).fill_(float("nan"))
                getattr(runner, name)[0].copy_(t[0])
            torch.cuda.synchronize()
            runner.step(VTensorMetadata(slots, lens, kvh, 128, num_decode_tokens=b, kv_elem_size=1 if fp8 else 2))
            runner.synchronize()
            for l in range(layers):
                hist_k[l] = [torch.cat([a, x.view(1, kvh, 128)]) for a, x in zip(hist_k[l], nk[l])]
                hist_v[l] = [torch.cat([a, x.view(1, kvh, 128)]) for a, x in zip(hist_v[l], nv[l])]
                sk, sv = (ks[l].cpu(), vs[l].cpu()) if fp8 else (None, None)
                r = oracle.fill_ranges(hist_k[l], hist_v[l], k_scale=sk, v_scale=sv)
                port = oracle.port_decode_attn(q[l].view(b, h, 128), r, torch.arange(b), torch.tensor(lens, dtype=torch.int32),
                                               kvh, SCALE, sk, sv)
                got = runner.out[l].view(b, h, 128).cpu()
                err = (got.float() - port.float()).abs()
                tol = torch.maximum(torch.full_like(err, 1e-2 if fp8 else 2e-3), port.float().abs() * 2.0 ** (-6 if fp8 else -7))
                assert bool((err <= tol).all()), (step, l, float(err.nan_to_num(nan=9e9).max()))
        assert runner.status() == 0 and E.status(0) == 0
    finally:
        E.close()
        eng.close()
