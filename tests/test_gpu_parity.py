"""GPU parity tests: every call goes through the C ABI (via the ctypes layer)
and is compared with the CPU oracle on the same seeded inputs.

Tolerances: cache contents bit-exact (bf16); attention max-abs <= 2e-3 against
the oracle on the benchmark-shaped cases (contexts >= 512, outputs well below
1), and 2e-3 or one bf16 ulp of the value, whichever is larger, on the
short-context edge cases whose outputs are O(1) (one ulp at 1.0 is 7.8e-3);
fp8 KV <= 3e-2 against the bf16-KV result."""
import os

import numpy as np
import pytest
import torch

from tests import synth
from tests.test_oracle import SCALE, load_golden

pytestmark = pytest.mark.gpu
UMMA = not os.environ.get("VT_PREFILL_ENGINE", "").startswith("m")   # with tensor maps: tcgen05 kernel unless mma.sync is forced


def close_2e3(a, b, ulp_slack=False):
    af, bf = a.float(), b.float()
    tol = torch.full_like(af, 2e-3)
    if ulp_slack:
        tol = torch.maximum(tol, torch.maximum(af.abs(), bf.abs()) * 2.0 ** -7)
    bad = (af - bf).abs() > tol
    return not bool(bad.any()), float((af - bf).abs().max())


@pytest.fixture
def force_variant():
    """force_variant(mode) overrides the planner's kernel choice for one test."""
    from glake_b200 import ops

    def force(mode):
        ops.set_attn_tuning(mode)
    yield force
    ops.set_attn_tuning("auto")


@pytest.fixture(scope="module")
def G():
    from tests import gpu_util
    gpu_util.ensure_pool()
    return gpu_util


@pytest.mark.parametrize("name", list(synth.GOLDEN_CASES))
def test_golden_cases_cache_bits_and_attention(G, oracle, name):
    z, gold = load_golden(name)
    seed, lens, h, kvh = synth.golden_lens(name)
    q, k, v = synth.make_case(seed, lens, h, kvh)
    kv = G.GpuKV(k, v, kvh)
    try:
        rows_k = [kv.read_rows(i, "k") for i in range(len(lens))]
        rows_v = [kv.read_rows(i, "v") for i in range(len(lens))]
        assert synth.digest(rows_k, rows_v) == str(z["cache_sha256"]), "cache contents are not bit-exact"
        out = kv.attend(q, SCALE)
        short = min(lens) < 512
        ok, err = close_2e3(out, gold, ulp_slack=short)
        assert ok, f"max abs err vs reference golden {err}"
        r = oracle.fill_ranges(k, v)
        port = oracle.port_decode_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32), kvh, SCALE)
        ok, err = close_2e3(out, port, ulp_slack=short)
        assert ok, f"max abs err vs oracle port {err}"
    finally:
        kv.close()


@pytest.mark.parametrize("h,kvh", [(4, 4), (8, 4), (8, 2), (8, 1), (16, 1), (32, 8), (12, 12), (3, 3)])
@pytest.mark.parametrize("mode", ["auto", "simt", "mma", "flat"])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_group_sizes_variants_and_forced_splits(G, oracle, force_variant, h, kvh, mode, splits):
    """Every kernel variant (SIMT split-K, tensor-core split-K, tensor-core flat
    schedule) on every head-group shape, with and without forced partitions."""
    force_variant(mode)
    if mode == "flat" and splits:
        pytest.skip("the flat schedule has no split count")
    lens = [1, 31, 32, 33, 700, 1300, 65, 64]
    q, k, v = synth.make_case(100 + h + kvh, lens, h, kvh)
    kv = G.GpuKV(k, v, kvh)
    try:
        out, lse = kv.attend(q, SCALE, return_lse=True) if splits == 0 else (kv.attend(q, SCALE, num_splits=splits), None)
        r = oracle.fill_ranges(k, v)
        port, plse = oracle.port_decode_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32),
                                             kvh, SCALE, return_lse=True)
        ok, err = close_2e3(out, port, ulp_slack=True)
        assert ok, err
        if lse is not None:
            assert torch.allclose(lse, plse, atol=2e-3)
    finally:
        kv.close()


def test_slot_indirection_and_strided_q(G, oracle):
    """Batch order differs from slot order; q is a view into a fused qkv buffer."""
    lens = [640, 90, 1500]
    h, kvh = 8, 4
    q, k, v = synth.make_case(7, lens, h, kvh)
    kv = G.GpuKV(k, v, kvh, slots=[5, 0, 3], max_slots=8)
    try:
        fused = torch.zeros(3, (h + 2 * kvh) * 128, dtype=torch.bfloat16, device="cuda")
        fused[:, : h * 128] = q.view(3, -1).cuda()
        qv = fused[:, : h * 128].view(3, h, 128)
        assert qv.stride(0) == (h + 2 * kvh) * 128
        from glake_b200 import ops
        out = torch.empty(3, h, 128, dtype=torch.bfloat16, device="cuda")
        ops.paged_attention_v1(out, qv, kv.k_table, kv.v_table, kvh, SCALE, kv.meta.seq_lens_tensor, 1,
                               kv.meta.max_seq_len, None, "auto", 1.0, kv.meta.slot_mapping)
        r = oracle.fill_ranges(k, v)
        port = oracle.port_decode_attn(q, r, torch.arange(3), torch.tensor(lens, dtype=torch.int32), kvh, SCALE)
        ok, err = close_2e3(out.cpu(), port, ulp_slack=True)
        assert ok, err
    finally:
        kv.close()


def test_append_strided_source_padding_and_growth_keeps_data(G, oracle):
    """Decode append from a fused-qkv view, a padded entry (offset -1), and a
    chunk-boundary crossing: rows written before the growth keep their bits and
    the range keeps its base address."""
    from glake_b200 import ops
    from glake_b200.backend import VTensorCacheEngine, VTensorMetadata, prepare_step
    kvh = 8                                      # row = 2 KiB -> 1024 tokens per 2 MiB chunk
    eng = VTensorCacheEngine(1, kvh, 128, 3, 4096)
    try:
        rs = np.random.RandomState(9)
        pre = [1020, 5, 1023]
        kcat = synth.normal_bf16(rs, sum(pre), kvh, 128).cuda()
        vcat = synth.normal_bf16(rs, sum(pre), kvh, 128).cuda()
        meta = VTensorMetadata([0, 1, 2], pre, kvh, 128, num_prefills=3)
        prepare_step(meta, eng)
        ops.reshape_and_cache(kcat, vcat, eng.k_cache_ptr[0], eng.v_cache_ptr[0], meta.slot_m, meta.slot_mapping,
                              meta.seq_lens_tensor, meta.cache_seq_lens, max(pre), kvh, 128)
        bases = [s.getKeyDevicePtr(0) for s in eng.vmm_kvcache_segment]
        mapped0 = [s.actual_size for s in eng.vmm_kvcache_segment]
        assert mapped0 == [2 << 20] * 3
        new_rows = []
        lens = list(pre)
        for step in range(6):                     # slots 0 and 2 cross into a second chunk
            fused = synth.normal_bf16(rs, 3, 3 * kvh * 128).cuda()
            kd = fused[:, : kvh * 128].view(3, kvh, 128)
            vd = fused[:, kvh * 128: 2 * kvh * 128].view(3, kvh, 128)
            lens = [n + 1 for n in lens]
            meta = VTensorMetadata([0, 1, 2], lens, kvh, 128, num_decode_tokens=3,
                                   extend_seq_list=[0, -1, 2] if step == 0 else [-1, -1, -1])
            prepare_step(meta, eng)
            if step == 3:                         # padded entry: offset -1 must leave slot 1 untouched
                meta.slot_m = meta.slot_m.clone()
                meta.slot_m[1] = -1
            ops.reshape_and_cache(kd, vd, eng.k_cache_ptr[0], eng.v_cache_ptr[0], meta.slot_m, meta.slot_mapping,
                                  meta.seq_lens_tensor, meta.cache_seq_lens, 1, kvh, 128)
            new_rows.append((kd.cpu(), vd.cpu(), step == 3))
        torch.cuda.synchronize()
        assert [s.getKeyDevicePtr(0) for s in eng.vmm_kvcache_segment] == bases
        assert eng.vmm_kvcache_segment[0].actual_size == 4 << 20 and eng.vmm_kvcache_segment[1].actual_size == 2 << 20
        # read back and compare bit for bit
        holder = G.GpuKV.__new__(G.GpuKV)
        holder.engine, holder.kvh, holder.fp8, holder.layer, holder.slots, holder.lens = eng, kvh, False, 0, [0, 1, 2], lens
        start = 0
        for i in range(3):
            got_k, got_v = holder.read_rows(i, "k"), holder.read_rows(i, "v")
            assert torch.equal(got_k[: pre[i]], kcat[start: start + pre[i]].cpu())
            assert torch.equal(got_v[: pre[i]], vcat[start: start + pre[i]].cpu())
            for step, (kd, vd, padded) in enumerate(new_rows):
                if i == 1 and padded:
                    assert not torch.equal(got_k[pre[i] + step], kd[i])
                else:
                    assert torch.equal(got_k[pre[i] + step], kd[i]) and torch.equal(got_v[pre[i] + step], vd[i])
            start += pre[i]
    finally:
        eng.close()


@pytest.mark.parametrize("h,kvh", [(8, 8), (32, 8), (8, 1), (16, 2), (16, 4), (16, 1), (3, 3)])
@pytest.mark.parametrize("mode", ["auto", "simt"])
def test_fp8_kv_cache(G, oracle, force_variant, h, kvh, mode):
    """fp8 e4m3 cache on the tensor-core flat schedule (f16 MMAs) and on the SIMT
    split-K kernel, every head-group shape incl. the ones that pack several token
    rows into one bulk copy."""
    force_variant(mode)
    lens = [520, 2100, 64, 1, 129]
    q, k, v = synth.make_case(40 + kvh, lens, h, kvh)
    from glake_b200 import ops
    ks = ops.kv_scales(torch.cat(k).cuda(), kvh, 128)
    vs = ops.kv_scales(torch.cat(v).cuda(), kvh, 128)
    assert torch.equal(ks.cpu(), oracle.port_kv_scales(torch.cat(k)))
    kv8 = G.GpuKV(k, v, kvh, fp8=True, k_scale=ks, v_scale=vs)
    kv16 = G.GpuKV(k, v, kvh)
    try:
        r8 = oracle.fill_ranges(k, v, k_scale=ks.cpu(), v_scale=vs.cpu())
        for i, n in enumerate(lens):       # stored bytes equal the oracle's sat(x / scale)
            assert torch.equal(kv8.read_rows(i, "k"), r8.k_rows(i, n, kvh, 128, fp8=True))
            assert torch.equal(kv8.read_rows(i, "v"), r8.v_rows(i, n, kvh, 128, fp8=True))
        o8 = kv8.attend(q, SCALE)
        o16 = kv16.attend(q, SCALE)
        long_ctx = [i for i, n in enumerate(lens) if n >= 512]
        assert (o8.float() - o16.float())[long_ctx].abs().max() <= 3e-2
        port8 = oracle.port_decode_attn(q, r8, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32), kvh,
                                        SCALE, ks.cpu(), vs.cpu())
        # the reference's own fp8 tolerance (1e-2), or two bf16 ulps where short contexts make outputs O(1)
        err = (o8.float() - port8.float()).abs()
        assert bool((err <= torch.maximum(torch.full_like(err, 1e-2), port8.float().abs() * 2.0 ** -6)).all())
    finally:
        kv8.close()
        kv16.close()


@pytest.mark.parametrize("h,kvh,fp8", [(8, 1, False), (8, 2, False), (8, 4, False), (32, 32, False), (16, 1, False),
                                        (3, 3, False), (8, 8, True), (8, 1, True), (4, 2, True), (16, 4, True),
                                        (16, 1, True), (3, 3, True)])
def test_fused_decode_step_appends_and_attends(G, oracle, h, kvh, fp8):
    """vt_decode_step = append + attention in one call (one launch for bf16): the
    cache must hold the new rows bit for bit afterwards and the output must match
    the oracle on the extended context, over several steps incl. tile and chunk
    boundaries (63/64/65 tokens, 2 MiB crossing for 8 KiB rows)."""
    from glake_b200 import ops
    from glake_b200.backend import VTensorMetadata, prepare_step
    lens = [1, 62, 63, 64, 255, 700]
    rs = np.random.RandomState(321 + h)
    q0, k, v = synth.make_case(50 + h + kvh, lens, h, kvh)
    ks = vs = None
    if fp8:
        ks = ops.kv_scales(torch.cat(k).cuda(), kvh, 128)
        vs = ops.kv_scales(torch.cat(v).cuda(), kvh, 128)
    kv = G.GpuKV(k, v, kvh, fp8=fp8, k_scale=ks, v_scale=vs)
    try:
        dt = "fp8_e4m3" if fp8 else "auto"
        for step in range(3):
            nk = synth.normal_bf16(rs, len(lens), kvh, 128)
            nv = synth.normal_bf16(rs, len(lens), kvh, 128)
            q = synth.normal_bf16(rs, len(lens), h, 128)
            lens = [n + 1 for n in lens]
            k = [torch.cat([a, b[None]]) for a, b in zip(k, nk)]
            v = [torch.cat([a, b[None]]) for a, b in zip(v, nv)]
            meta = VTensorMetadata(kv.slots, lens, kvh, 128, num_decode_tokens=len(lens), kv_elem_size=1 if fp8 else 2)
            prepare_step(meta, kv.engine)
            out = torch.empty(len(lens), h, 128, dtype=torch.bfloat16, device="cuda")
            ops.decode_step(out, q.cuda(), nk.cuda(), nv.cuda(), kv.k_table, kv.v_table, meta.slot_m, meta.slot_mapping,
                            meta.seq_lens_tensor, meta.max_seq_len, kvh, SCALE, dt, ks, vs)
            torch.cuda.synchronize()
            kv.lens = lens
            if fp8:
                r = oracle.fill_ranges(k, v, k_scale=ks.cpu(), v_scale=vs.cpu())
                for i, n in enumerate(lens):
                    assert torch.equal(kv.read_rows(i, "k"), r.k_rows(i, n, kvh, 128, fp8=True))
                    assert torch.equal(kv.read_rows(i, "v"), r.v_rows(i, n, kvh, 128, fp8=True))
                port = oracle.port_decode_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32),
                                               kvh, SCALE, ks.cpu(), vs.cpu())
                # the reference's own fp8 tolerance, or two bf16 ulps where the short
                # contexts make outputs O(1) (the oracle rounds dequantised values to bf16)
                err = (out.cpu().float() - port.float()).abs()
                assert bool((err <= torch.maximum(torch.full_like(err, 1e-2), port.float().abs() * 2.0 ** -6)).all())
            else:
                for i in range(len(lens)):
                    assert torch.equal(kv.read_rows(i, "k"), k[i]) and torch.equal(kv.read_rows(i, "v"), v[i])
                r = oracle.fill_ranges(k, v)
                port = oracle.port_decode_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32),
                                               kvh, SCALE)
                ok, err = close_2e3(out.cpu(), port, ulp_slack=True)
                assert ok, (step, err)
    finally:
        kv.close()


def test_backend_forward_decode_steps(G, oracle):
    """The attention-backend binding over several decode steps and two layers:
    prepare_step -> reshape_and_cache -> fwd_kvcache, against the oracle."""
    from glake_b200.backend import VTensorAttentionImpl, VTensorCacheEngine, VTensorMetadata, prepare_step
    h, kvh, layers = 8, 4, 2
    eng = VTensorCacheEngine(layers, kvh, 128, 4, 2048)
    impl = VTensorAttentionImpl(h, 128, SCALE, kvh)
    rs = np.random.RandomState(77)
    lens = [0, 0, 0]
    slots = [2, 0, 3]
    hist_k = [[[] for _ in slots] for _ in range(layers)]
    hist_v = [[[] for _ in slots] for _ in range(layers)]
    try:
        for step in range(5):
            lens = [n + 1 for n in lens]
            meta = VTensorMetadata(slots, lens, kvh, 128, num_decode_tokens=3)
            prepare_step(meta, eng)
            for layer in range(layers):
                q = synth.normal_bf16(rs, 3, h * 128)
                kk = synth.normal_bf16(rs, 3, kvh * 128)
                vv = synth.normal_bf16(rs, 3, kvh * 128)
                kc, vc = eng.gpu_cache[layer]
                out = impl.forward(q.cuda(), kk.cuda(), vv.cuda(), kc, vc, meta).cpu()
                for i in range(3):
                    hist_k[layer][i].append(kk[i].view(kvh, 128))
                    hist_v[layer][i].append(vv[i].view(kvh, 128))
                kl = [torch.stack(x) for x in hist_k[layer]]
                vl = [torch.stack(x) for x in hist_v[layer]]
                r = oracle.fill_ranges(kl, vl)
                port = oracle.port_decode_attn(q.view(3, h, 128), r, torch.arange(3),
                                               torch.tensor(lens, dtype=torch.int32), kvh, SCALE)
                ok, err = close_2e3(out.view(3, h, 128), port, ulp_slack=True)
                assert ok, (step, layer, err)
    finally:
        eng.close()


@pytest.mark.parametrize("use_maps", [False, True])
def test_backend_forward_prompt_extend_decode(G, oracle, use_maps):
    """The backend binding through a request's life: prompts, a prefix-extend chunk
    (new tokens appended behind the cached prefix and attending over prefix + new),
    then decode steps; two layers; every output against the oracle."""
    from glake_b200.backend import VTensorAttentionImpl, VTensorCacheEngine, VTensorMetadata, prepare_step
    h, kvh, layers = 8, 2, 2
    eng = VTensorCacheEngine(layers, kvh, 128, 3, 1024)
    impl = VTensorAttentionImpl(h, 128, SCALE, kvh)
    rs = np.random.RandomState(78)
    slots = [1, 2]
    ctx = [0, 0]
    hist_k = [[torch.empty(0, kvh, 128, dtype=torch.bfloat16) for _ in slots] for _ in range(layers)]
    hist_v = [[torch.empty(0, kvh, 128, dtype=torch.bfloat16) for _ in slots] for _ in range(layers)]
    try:
        for phase, new in enumerate([[300, 77], [50, 200], [1, 1], [1, 1]]):
            decode = phase >= 2
            ctx = [a + b for a, b in zip(ctx, new)]
            if decode:
                meta = VTensorMetadata(slots, ctx, kvh, 128, num_decode_tokens=2)
            else:
                meta = VTensorMetadata(slots, ctx, kvh, 128, num_prefills=2, query_lens=new)
            prepare_step(meta, eng)
            n = sum(new)
            starts = [0, new[0]]
            for layer in range(layers):
                q = synth.normal_bf16(rs, n, h * 128)
                kk = synth.normal_bf16(rs, n, kvh * 128)
                vv = synth.normal_bf16(rs, n, kvh * 128)
                kc, vc = eng.gpu_cache[layer]
                maps = eng.prefill_maps(layer) if use_maps else None
                out = impl.forward(q.cuda(), kk.cuda(), vv.cuda(), kc, vc, meta, prefill_maps=maps).cpu()
                for i in range(2):
                    rows = slice(starts[i], starts[i] + new[i])
                    hist_k[layer][i] = torch.cat([hist_k[layer][i], kk[rows].view(-1, kvh, 128)])
                    hist_v[layer][i] = torch.cat([hist_v[layer][i], vv[rows].view(-1, kvh, 128)])
                r = oracle.fill_ranges(hist_k[layer], hist_v[layer])
                port = oracle.port_prefill_attn(q.view(n, h, 128), r, torch.arange(2), torch.tensor(ctx, dtype=torch.int32),
                                                torch.tensor(new, dtype=torch.int32), torch.tensor(starts, dtype=torch.int32),
                                                kvh, SCALE)
                ok, err = close_2e3(out.view(n, h, 128), port, ulp_slack=True)
                assert ok, (phase, layer, err)
    finally:
        eng.close()


@pytest.mark.parametrize("h,kvh", [(8, 1), (8, 8)])
def test_decode_runner_graph_replay_with_layer_overlap(G, oracle, h, kvh):
    """DecodeRunner: all layers of a step in one CUDA graph, consecutive layers
    overlapped with programmatic dependent launch.  Several replays (the graph is
    captured on the first step), every layer's output and cache rows against the
    oracle."""
    from glake_b200.backend import DecodeRunner, VTensorAttentionImpl, VTensorCacheEngine, VTensorMetadata, prepare_step
    from glake_b200 import ops
    layers, lens0 = 4, [300, 1, 1500, 65]
    rs = np.random.RandomState(17 + kvh)
    eng = VTensorCacheEngine(layers, kvh, 128, len(lens0), 2048)
    impl = VTensorAttentionImpl(h, 128, SCALE, kvh)
    holder = G.GpuKV.__new__(G.GpuKV)
    holder.engine, holder.kvh, holder.fp8, holder.slots = eng, kvh, False, list(range(len(lens0)))
    try:
        # context: prefill through the append kernel, layer by layer
        hist_k = [[synth.normal_bf16(rs, n - 1, kvh, 128) for n in lens0] for _ in range(layers)]
        hist_v = [[synth.normal_bf16(rs, n - 1, kvh, 128) for n in lens0] for _ in range(layers)]
        pre = [n - 1 for n in lens0]
        meta = VTensorMetadata(holder.slots, pre, kvh, 128, num_prefills=len(pre))
        prepare_step(meta, eng)
        for l in range(layers):
            ops.reshape_and_cache(torch.cat(hist_k[l]).cuda(), torch.cat(hist_v[l]).cuda(), eng.k_cache_ptr[l],
                                  eng.v_cache_ptr[l], meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor,
                                  meta.cache_seq_lens, max(pre), kvh, 128)
        runner = DecodeRunner(eng, impl, len(lens0), host_io=True)
        assert runner.overlap
        lens = list(pre)
        for step in range(4):
            lens = [n + 1 for n in lens]
            q = synth.normal_bf16(rs, layers, len(lens), h * 128)
            nk = synth.normal_bf16(rs, layers, len(lens), kvh * 128)
            nv = synth.normal_bf16(rs, layers, len(lens), kvh * 128)
            runner.hq.copy_(q), runner.hk.copy_(nk), runner.hv.copy_(nv)
            runner.step(VTensorMetadata(holder.slots, lens, kvh, 128, num_decode_tokens=len(lens)))
            runner.synchronize()
            for l in range(layers):
                hist_k[l] = [torch.cat([a, b.view(1, kvh, 128)]) for a, b in zip(hist_k[l], nk[l])]
                hist_v[l] = [torch.cat([a, b.view(1, kvh, 128)]) for a, b in zip(hist_v[l], nv[l])]
                holder.layer, holder.lens = l, lens
                for i in range(len(lens)):
                    assert torch.equal(holder.read_rows(i, "k"), hist_k[l][i])
                    assert torch.equal(holder.read_rows(i, "v"), hist_v[l][i])
                r = oracle.fill_ranges(hist_k[l], hist_v[l])
                port = oracle.port_decode_attn(q[l].view(len(lens), h, 128), r, torch.arange(len(lens)),
                                               torch.tensor(lens, dtype=torch.int32), kvh, SCALE)
                ok, err = close_2e3(runner.hout[l].view(len(lens), h, 128), port, ulp_slack=True)
                assert ok, (step, l, err)
        assert ops.attn_status() == 0
    finally:
        eng.close()


@pytest.mark.parametrize("h,kvh", [(4, 4), (8, 2), (8, 1)])
def test_prefill_attention_over_the_range(G, oracle, h, kvh):
    """Prefix-extend: the new tokens' causal attention over prefix + new tokens,
    through vt_prefill_attn, against the oracle; ragged q_lens incl. tile edges
    (63/64/65), empty prefix and long prefix; then the padded fwd_kvcache form."""
    from glake_b200 import ops
    lens = [1, 64, 65, 200, 331, 700]          # total context per sequence
    q_lens = [1, 64, 63, 200, 31, 130]         # of which new
    _, k, v = synth.make_case(600 + h + kvh, lens, h, kvh)
    rs = np.random.RandomState(8)
    kv = G.GpuKV(k, v, kvh)
    try:
        starts = np.concatenate([[0], np.cumsum(q_lens)[:-1]]).astype(np.int32)
        q = synth.normal_bf16(rs, int(sum(q_lens)), h, 128)
        out = torch.empty_like(q, device="cuda")
        ql = torch.tensor(q_lens, dtype=torch.int32)
        qs = torch.from_numpy(starts)
        ops.prefill_attention(out, q.cuda(), kv.k_table, kv.v_table, kvh, SCALE, kv.meta.slot_mapping,
                              kv.meta.seq_lens_tensor, ql.cuda(), qs.cuda(), max(q_lens))
        torch.cuda.synchronize()
        r = oracle.fill_ranges(k, v)
        port = oracle.port_prefill_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32), ql, qs,
                                        kvh, SCALE)
        ok, err = close_2e3(out.cpu(), port, ulp_slack=True)
        assert ok, err
        # the same through TMA tensor copies: identical arithmetic, so identical bits
        maps = kv.engine.prefill_maps(0)
        assert maps is not None
        out_t = torch.zeros_like(out)
        ops.prefill_attention(out_t, q.cuda(), kv.k_table, kv.v_table, kvh, SCALE, kv.meta.slot_mapping,
                              kv.meta.seq_lens_tensor, ql.cuda(), qs.cuda(), max(q_lens), maps=maps)
        torch.cuda.synchronize()
        ok, err = close_2e3(out_t.cpu(), port, ulp_slack=True)
        assert ok, err
        if not UMMA:                     # the mma.sync kernel does identical arithmetic on both copy paths
            assert torch.equal(out_t, out)
        # padded form: every sequence extends by the same 16 tokens
        s_new = 16
        lens2 = [n for n in lens if n >= s_new]
        idx = [i for i, n in enumerate(lens) if n >= s_new]
        qp = synth.normal_bf16(rs, len(idx), s_new, h, 128)
        slots = kv.meta.slot_mapping[idx].contiguous()
        sl = kv.meta.seq_lens_tensor[idx].contiguous()
        o2, _ = ops.fwd_kvcache(qp.cuda(), kv.k_table, kv.v_table, max(lens2), kvh, len(idx), slots, None, None, sl,
                                None, None, None, None, None, None, SCALE, True, -1, -1, None, 4)
        torch.cuda.synchronize()
        r2 = oracle.fill_ranges([k[i] for i in idx], [v[i] for i in idx])
        port2 = oracle.port_prefill_attn(qp.view(-1, h, 128), r2, torch.arange(len(idx)),
                                         torch.tensor(lens2, dtype=torch.int32),
                                         torch.full((len(idx),), s_new, dtype=torch.int32),
                                         torch.arange(len(idx), dtype=torch.int32) * s_new, kvh, SCALE)
        ok, err = close_2e3(o2.cpu().view(-1, h, 128), port2, ulp_slack=True)
        assert ok, err
    finally:
        kv.close()


@pytest.mark.parametrize("name", list(synth.PREFILL_CASES))
def test_prefill_against_reference_golden(G, name):
    """Both prefill kernels against golden vectors made by the reference's CPU decode kernel
    (one decode query per new token over the tokens it may see)."""
    from glake_b200 import ops
    from tests.test_oracle import GOLDEN, _from_bits, prefill_case_inputs
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    lens, q_lens, h, kvh, q, k, v, starts = prefill_case_inputs(name)
    assert synth.digest(q, k, v) == str(z["input_sha256"]), "input generator drifted"
    gold = _from_bits(z["out_bits"])
    kv = G.GpuKV(k, v, kvh)
    try:
        ql = torch.tensor(q_lens, dtype=torch.int32).cuda()
        for maps in (None, kv.engine.prefill_maps(0)):
            out = torch.zeros_like(q, device="cuda")
            ops.prefill_attention(out, q.cuda(), kv.k_table, kv.v_table, kvh, SCALE, kv.meta.slot_mapping,
                                  kv.meta.seq_lens_tensor, ql, starts.cuda(), max(q_lens), maps=maps)
            torch.cuda.synchronize()
            ok, err = close_2e3(out.cpu(), gold, ulp_slack=True)
            assert ok, (maps is not None, err)
    finally:
        kv.close()


@pytest.mark.parametrize("h,kvh", [(8, 2), (4, 4)])
def test_prefill_long_prompts_both_copy_paths(G, oracle, h, kvh):
    """Prompts beyond 1536 tokens take the 112-row tile shape; contexts end inside a
    2 MiB chunk, at a tile edge and one row past a chunk boundary."""
    from glake_b200 import ops
    rows_per_chunk = (2 << 20) // (kvh * 256)
    lens = [1700, rows_per_chunk + 1, 2048]
    q_lens = [1700, 1601, 333]
    _, k, v = synth.make_case(900 + kvh, lens, h, kvh)
    rs = np.random.RandomState(9)
    kv = G.GpuKV(k, v, kvh)
    try:
        starts = np.concatenate([[0], np.cumsum(q_lens)[:-1]]).astype(np.int32)
        q = synth.normal_bf16(rs, int(sum(q_lens)), h, 128)
        ql, qs = torch.tensor(q_lens, dtype=torch.int32), torch.from_numpy(starts)
        r = oracle.fill_ranges(k, v)
        port = oracle.port_prefill_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32), ql, qs,
                                        kvh, SCALE)
        outs = []
        for maps in (None, kv.engine.prefill_maps(0)):
            out = torch.zeros_like(q, device="cuda")
            ops.prefill_attention(out, q.cuda(), kv.k_table, kv.v_table, kvh, SCALE, kv.meta.slot_mapping,
                                  kv.meta.seq_lens_tensor, ql.cuda(), qs.cuda(), max(q_lens), maps=maps)
            torch.cuda.synchronize()
            ok, err = close_2e3(out.cpu(), port, ulp_slack=True)
            assert ok, err
            outs.append(out)
        if not UMMA:
            assert torch.equal(outs[0], outs[1])
    finally:
        kv.close()


@pytest.mark.parametrize("h,kvh,scale", [(4, 4, 1.0), (8, 1, 0.6), (16, 2, SCALE)])
def test_prefill_tensor_core_path_rescales_and_edges(G, oracle, h, kvh, scale):
    """The tcgen05 prefill kernel where its own machinery matters: logits large enough
    that row maxima jump by more than 2^8 between tiles (the O rows in tensor memory are
    rescaled), a single tile, a one-token extension of a long prefix, query counts that
    are no multiple of 128, an entry with nothing to do."""
    from glake_b200 import ops
    lens = [40, 129, 777, 1500, 300]
    q_lens = [40, 129, 1, 700, 0]
    _, k, v = synth.make_case(1200 + h, lens, h, kvh)
    rs = np.random.RandomState(10)
    kv = G.GpuKV(k, v, kvh)
    try:
        starts = np.concatenate([[0], np.cumsum(q_lens)[:-1]]).astype(np.int32)
        q = synth.normal_bf16(rs, int(sum(q_lens)), h, 128)
        ql, qs = torch.tensor(q_lens, dtype=torch.int32), torch.from_numpy(starts)
        r = oracle.fill_ranges(k, v)
        port = oracle.port_prefill_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32), ql, qs,
                                        kvh, scale)
        out = torch.zeros_like(q, device="cuda")
        ops.prefill_attention(out, q.cuda(), kv.k_table, kv.v_table, kvh, scale, kv.meta.slot_mapping,
                              kv.meta.seq_lens_tensor, ql.cuda(), qs.cuda(), max(q_lens), maps=kv.engine.prefill_maps(0))
        torch.cuda.synchronize()
        ok, err = close_2e3(out.cpu(), port, ulp_slack=True)
        assert ok, err
    finally:
        kv.close()


def test_prefill_full_size_engines_agree_and_normalise(G):
    """4096-token prompts, 32 q heads over 8 kv heads (two CTAs per SM, 64 K/V tiles per CTA):
    the tcgen05 kernel (tensor maps) and the mma.sync kernel (row copies) are independent
    implementations of the same fp32 softmax and must agree to 2e-3 (or one bf16 ulp where the
    output is O(1)); with V = 1 every output
    must be exactly 1 (each visible token counted once, sums and rescales consistent)."""
    from glake_b200 import ops
    from glake_b200.backend import VTensorCacheEngine, VTensorMetadata, prepare_step
    b, h, kvh, n = 2, 32, 8, 4096
    gen = torch.Generator(device="cuda").manual_seed(5)
    eng = VTensorCacheEngine(1, kvh, 128, b, n + 8)
    try:
        meta = VTensorMetadata(list(range(b)), [n] * b, kvh, 128, num_prefills=b)
        prepare_step(meta, eng)
        k = torch.randn(b * n, kvh, 128, device="cuda", generator=gen).bfloat16()
        q = torch.randn(b * n, h, 128, device="cuda", generator=gen).bfloat16()
        ql = torch.full((b,), n, dtype=torch.int32, device="cuda")
        qs = torch.arange(b, dtype=torch.int32, device="cuda") * n
        kt, vt = eng.gpu_cache[0][0].vmm_ptr, eng.gpu_cache[0][1].vmm_ptr
        for ones in (False, True):
            v = torch.ones_like(k) if ones else torch.randn(b * n, kvh, 128, device="cuda", generator=gen).bfloat16()
            ops.reshape_and_cache(k, v, eng.k_cache_ptr[0], eng.v_cache_ptr[0], meta.slot_m, meta.slot_mapping,
                                  meta.seq_lens_tensor, meta.cache_seq_lens, n, kvh, 128)
            outs = []
            for maps in (None, eng.prefill_maps(0)):
                out = torch.zeros_like(q)
                ops.prefill_attention(out, q, kt, vt, kvh, SCALE, meta.slot_mapping, meta.seq_lens_tensor, ql, qs, n, maps=maps)
                torch.cuda.synchronize()
                outs.append(out)
            if ones:
                assert bool((outs[0] == 1).all()) and bool((outs[1] == 1).all())
            else:
                ok, err = close_2e3(outs[0], outs[1], ulp_slack=True)   # first rows attend few tokens: outputs of O(1)
                assert ok, err
                assert float(outs[1].float().abs().max()) > 0.05       # not trivially zero
    finally:
        eng.close()


@pytest.mark.parametrize("seed", range(12))
def test_flat_schedule_random_batches(G, oracle, seed):
    """Randomised batches for the persistent flat schedule: piece boundaries, stream
    merges, empty sequences, fewer tiles than CTAs, more sequences than the
    shared-memory base cache holds (> 256), every (kv heads per CTA, rows per copy)
    shape, bf16 and fp8; fused step and plain attention must agree with the oracle."""
    from glake_b200 import ops
    from glake_b200.backend import VTensorMetadata, prepare_step
    rs = np.random.RandomState(1000 + seed)
    kvh = int(rs.choice([1, 2, 4, 8, 12]))
    g = int(rs.choice([1, 2, 4, 8])) if kvh != 12 else 1
    h = kvh * g
    fp8 = bool(seed % 3 == 2) and kvh != 12
    if seed == 5:
        batch, hi = 300, 40                   # many short sequences
    elif seed == 7:
        batch, hi = 3, 20000                  # few long ones: streams cut into many pieces
    else:
        batch, hi = int(rs.randint(1, 40)), int(rs.choice([3, 70, 700, 3000]))
    lens = [int(x) for x in rs.randint(1, hi + 1, size=batch)]
    q, k, v = synth.make_case(2000 + seed, lens, h, kvh)
    ks = vs = None
    if fp8:
        ks = ops.kv_scales(torch.cat(k).cuda(), kvh, 128)
        vs = ops.kv_scales(torch.cat(v).cuda(), kvh, 128)
    kv = G.GpuKV(k, v, kvh, fp8=fp8, k_scale=ks, v_scale=vs)
    try:
        out, lse = kv.attend(q, SCALE, return_lse=True)
        if fp8:
            r = oracle.fill_ranges(k, v, k_scale=ks.cpu(), v_scale=vs.cpu())
            port, plse = oracle.port_decode_attn(q, r, torch.arange(batch), torch.tensor(lens, dtype=torch.int32), kvh,
                                                 SCALE, ks.cpu(), vs.cpu(), return_lse=True)
            err = (out.float() - port.float()).abs()
            # The oracle rounds every dequantised K/V element to bf16 as the reference does, the
            # kernel keeps fp8 * scale exact; on contexts of a few dozen tokens that alone moves
            # outputs by ~1e-2, so these random cases use the fp8 contract tolerance (3e-2).
            tol = torch.maximum(torch.full_like(err, 3e-2), port.float().abs() * 2.0 ** -6)
            worst = int((err - tol).argmax())
            assert bool((err <= tol).all()), (float(err.flatten()[worst]), float(port.float().flatten()[worst]), lens)
            assert torch.allclose(lse, plse, atol=2e-2)
        else:
            r = oracle.fill_ranges(k, v)
            port, plse = oracle.port_decode_attn(q, r, torch.arange(batch), torch.tensor(lens, dtype=torch.int32), kvh,
                                                 SCALE, return_lse=True)
            ok, err = close_2e3(out, port, ulp_slack=True)
            assert ok, err
            assert torch.allclose(lse, plse, atol=2e-3)
            # same batch with some sequences emptied: zeros there, others unchanged
            if batch >= 3:
                sl = kv.meta.seq_lens_tensor.clone()
                kv.meta.seq_lens_tensor[::3] = 0
                out2 = kv.attend(q, SCALE)
                kv.meta.seq_lens_tensor.copy_(sl)
                assert torch.equal(out2[::3], torch.zeros_like(out2[::3]))
                keep = [i for i in range(batch) if i % 3]
                # the tile list is cut differently now, so sums associate differently: equal up to rounding
                ok, err = close_2e3(out2[keep], out[keep], ulp_slack=True)
                assert ok, err
    finally:
        kv.close()


def test_full_size_properties_config3_shape(G):
    """The long-context GQA shape at full length, one sequence pair (32 q / 8 kv heads, 16k-32k
    tokens), too long for the scalar oracle in seconds, checked through
    size-independent properties: (1) V == 1 everywhere -> every output is 1;
    (2) V[t] = e_(t mod 128) and K == 0 -> uniform softmax, output[d] = count_d / L;
    (3) forced split counts agree with each other."""
    h, kvh = 32, 8
    lens = [16384 + 777, 32768]
    rs = np.random.RandomState(12)
    q = synth.normal_bf16(rs, 2, h, 128)
    k = [synth.normal_bf16(rs, n, kvh, 128) for n in lens]
    ones = [torch.ones(n, kvh, 128, dtype=torch.bfloat16) for n in lens]
    kv = G.GpuKV(k, ones, kvh)
    try:
        out = kv.attend(q, SCALE)
        assert (out.float() - 1).abs().max() <= 2e-3
        a = kv.attend(q, SCALE, num_splits=7)
        b = kv.attend(q, SCALE, num_splits=64)
        assert (a.float() - b.float()).abs().max() <= 2e-3
    finally:
        kv.close()
    zeros = [torch.zeros(n, kvh, 128, dtype=torch.bfloat16) for n in lens]
    onehot = []
    for n in lens:
        v = torch.zeros(n, kvh, 128, dtype=torch.bfloat16)
        v[torch.arange(n), :, torch.arange(n) % 128] = 1
        onehot.append(v)
    kv = G.GpuKV(zeros, onehot, kvh)
    try:
        out = kv.attend(q, SCALE).float()
        for i, n in enumerate(lens):
            want = torch.bincount(torch.arange(n) % 128, minlength=128).float() / n
            assert (out[i] - want[None, :]).abs().max() <= 2e-3
    finally:
        kv.close()


@pytest.mark.parametrize("name,batch,h,kvh,lo,hi,fp8", [
    ("7b-layer", 64, 32, 32, 1024, 4096, False),
    ("70b-share-tp2", 64, 32, 4, 4096, 16384, False),
    ("70b-share-tp8", 64, 8, 1, 4096, 16384, False),
    ("gqa-fp8", 128, 32, 8, 2048, 8192, True),
])
def test_full_size_properties_of_the_bench_shapes(G, name, batch, h, kvh, lo, hi, fp8):
    """One layer of every benchmark shape at FULL size (up to 2.6 GB of KV), where
    the scalar oracle would take minutes: K == 0 makes the softmax uniform, and V
    one-hot in (t mod 128) turns the output into a histogram of the tokens read,
    output[d] = |{t < L : t mod 128 == d}| / L, exact only if every token of every
    sequence is read exactly once across tiles, pieces and merges; V == 1 with random
    K checks the normalisation (every output is 1)."""
    from glake_b200 import ops
    g = torch.Generator().manual_seed(77)
    lens = torch.randint(lo, hi + 1, (batch,), generator=g).tolist()
    dev = "cuda"
    ks = vs = None
    if fp8:
        ks = torch.ones(kvh, device=dev)
        vs = torch.ones(kvh, device=dev)
    q = torch.randn(batch, h, 128, generator=g).bfloat16()
    ar = torch.arange(hi, device=dev)
    onehot_full = torch.zeros(hi, 128, dtype=torch.bfloat16, device=dev)
    onehot_full[ar, ar % 128] = 1
    zeros = [torch.zeros(n, kvh, 128, dtype=torch.bfloat16, device=dev) for n in lens]
    onehot = [onehot_full[:n, None, :].expand(n, kvh, 128).contiguous() for n in lens]
    kv = G.GpuKV(zeros, onehot, kvh, fp8=fp8, k_scale=ks, v_scale=vs)
    try:
        out = kv.attend(q, SCALE).float()
        for i, n in enumerate(lens):
            want = torch.bincount(torch.arange(n) % 128, minlength=128).float() / n
            assert (out[i] - want[None, :]).abs().max() <= 2e-3, (name, i, n)
    finally:
        kv.close()
    del zeros, onehot
    rk = [torch.randn(n, kvh, 128, device=dev, dtype=torch.bfloat16) for n in lens]
    ones = [torch.ones(n, kvh, 128, dtype=torch.bfloat16, device=dev) for n in lens]
    if fp8:
        ks = torch.full((kvh,), 6.0 / 448.0, device=dev)
    kv = G.GpuKV(rk, ones, kvh, fp8=fp8, k_scale=ks, v_scale=vs)
    try:
        out = kv.attend(q, SCALE).float()
        assert (out - 1).abs().max() <= 2e-3, name
    finally:
        kv.close()


def test_slot_lifecycle_on_the_real_driver(G):
    """release_seq keeps the pre-cached prefix of a slot mapped (and its bytes
    intact), preempt_seq unmaps everything, chunks return to the pool, base
    addresses survive, and a reused slot serves a new sequence correctly."""
    from glake_b200 import ops, vmmAllocator as A
    from glake_b200.backend import VTensorMetadata, prepare_step, VTensorCacheEngine
    kvh, row = 8, 8 * 128 * 2                      # 2 KiB rows, 1024 rows per chunk
    free0 = A.showFreeBlocks()
    eng = VTensorCacheEngine(2, kvh, 128, 2, 8192, cache_seqs=1, cache_tokens=1)   # slot 0 pre-cached with 1 chunk
    try:
        seg0, seg1 = eng.vmm_kvcache_segment
        assert seg0.actual_size == 2 << 20 and seg1.actual_size == 0
        assert A.showFreeBlocks() == free0 - 4                                       # 2 layers x (K + V)
        bases = [seg0.getKeyDevicePtr(1), seg1.getValueDevicePtr(0)]
        rs = np.random.RandomState(2)
        lens = [3000, 1500]
        k = [synth.normal_bf16(rs, n, kvh, 128) for n in lens]
        v = [synth.normal_bf16(rs, n, kvh, 128) for n in lens]
        meta = VTensorMetadata([0, 1], lens, kvh, 128, num_prefills=2)
        prepare_step(meta, eng)
        for layer in range(2):
            ops.reshape_and_cache(torch.cat(k).cuda(), torch.cat(v).cuda(), eng.k_cache_ptr[layer], eng.v_cache_ptr[layer],
                                  meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor, meta.cache_seq_lens, max(lens),
                                  kvh, 128)
        torch.cuda.synchronize()
        assert seg0.actual_size == 6 << 20 and seg1.actual_size == 4 << 20          # 3 and 2 chunks per range
        assert A.showFreeBlocks() == free0 - 4 * (3 + 2)
        seg0.release_seq(0)                          # finished: keeps its 1-chunk prefix
        seg1.preempt_seq(1)                          # preempted: everything goes back
        assert (seg0.actual_size, seg0.used_size, seg1.actual_size) == (2 << 20, 0, 0)
        assert A.showFreeBlocks() == free0 - 4
        assert [seg0.getKeyDevicePtr(1), seg1.getValueDevicePtr(0)] == bases
        holder = G.GpuKV.__new__(G.GpuKV)
        holder.engine, holder.kvh, holder.fp8, holder.layer, holder.slots, holder.lens = eng, kvh, False, 1, [0, 1], [1024, 0]
        assert torch.equal(holder.read_rows(0, "k"), k[0][:1024])      # the kept chunk still holds the old rows
        # both slots serve new sequences
        lens2 = [700, 2100]
        q, k2, v2 = synth.make_case(91, lens2, 16, kvh)
        meta = VTensorMetadata([0, 1], lens2, kvh, 128, num_prefills=2)
        prepare_step(meta, eng)
        ops.reshape_and_cache(torch.cat(k2).cuda(), torch.cat(v2).cuda(), eng.k_cache_ptr[0], eng.v_cache_ptr[0],
                              meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor, meta.cache_seq_lens, max(lens2), kvh, 128)
        out = torch.empty(2, 16, 128, dtype=torch.bfloat16, device="cuda")
        ops.paged_attention_v1(out, q.cuda(), eng.gpu_cache[0][0].vmm_ptr, eng.gpu_cache[0][1].vmm_ptr, kvh, SCALE,
                               meta.seq_lens_tensor, 1, max(lens2), None, "auto", 1.0, meta.slot_mapping)
        from oracle import oracle as O
        r = O.fill_ranges(k2, v2)
        port = O.port_decode_attn(q, r, torch.arange(2), torch.tensor(lens2, dtype=torch.int32), kvh, SCALE)
        ok, err = close_2e3(out.cpu(), port, ulp_slack=True)
        assert ok, err
    finally:
        eng.close()
    assert A.showFreeBlocks() == free0


def test_empty_batch_and_zero_length(G):
    from glake_b200 import ops
    q = torch.zeros(0, 8, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(q)
    sl = torch.zeros(0, dtype=torch.int32, device="cuda")
    sm = torch.zeros(0, dtype=torch.int64, device="cuda")
    ops.paged_attention_v1(out, q, 0, 0, 8, SCALE, sl, 1, 0, None, "auto", 1.0, sm)   # no-op, no launch
    lens = [3, 1]
    qq, k, v = synth.make_case(5, lens, 4, 4)
    kv = G.GpuKV(k, v, 4)
    try:
        kv.meta.seq_lens_tensor[1] = 0          # a sequence with no context yields zeros
        out = kv.attend(qq, SCALE)
        assert torch.equal(out[1], torch.zeros_like(out[1]))
    finally:
        kv.close()


def test_rejects_cpu_tensors_and_unsupported_shapes():
    from glake_b200 import ops
    with pytest.raises(RuntimeError):
        ops.paged_attention_v1(torch.zeros(1, 4, 128, dtype=torch.bfloat16), torch.zeros(1, 4, 128, dtype=torch.bfloat16),
                               0, 0, 4, 1.0, torch.ones(1, dtype=torch.int32), 1, 1, None, "auto", 1.0,
                               torch.zeros(1, dtype=torch.int64))
    q = torch.zeros(1, 6, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):          # 6 q heads over 2 kv heads: group 3 is not supported
        ops.paged_attention_v1(torch.empty_like(q), q, 1 << 20, 1 << 20, 2, 1.0,
                               torch.ones(1, dtype=torch.int32, device="cuda"), 1, 1, None, "auto", 1.0,
                               torch.zeros(1, dtype=torch.int64, device="cuda"))
