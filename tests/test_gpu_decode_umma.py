"""The tcgen05 decode kernel for fp8 ranges (vt_decode_step_tma) against the oracle and
against the mma.sync kernel it replaces: fused steps over tile, chunk and stream-piece
boundaries, plain attention, the overlap launch forms and CUDA-graph replay."""
import numpy as np
import pytest
import torch

from tests import synth

pytestmark = pytest.mark.gpu
SCALE = 128 ** -0.5


@pytest.fixture(scope="module")
def G():
    from tests import gpu_util
    gpu_util.ensure_pool()
    return gpu_util


def _tol_ok(out, port):
    # the reference's own fp8 tolerance (1e-2), or two bf16 ulps where short contexts make outputs O(1)
    err = (out.float() - port.float()).abs()
    return bool((err <= torch.maximum(torch.full_like(err, 1e-2), port.float().abs() * 2.0 ** -6)).all()), float(err.max())


@pytest.mark.parametrize("h,kvh", [(32, 8), (8, 8), (16, 8), (32, 16)])
def test_fused_steps_match_oracle_and_cache_bytes(G, oracle, h, kvh):
    from glake_b200 import ops
    from glake_b200.backend import VTensorMetadata, prepare_step
    lens = [1, 31, 32, 33, 63, 64, 255, 700, 2047]
    rs = np.random.RandomState(11 + h + kvh)
    q0, k, v = synth.make_case(90 + h + kvh, lens, h, kvh)
    ks = ops.kv_scales(torch.cat(k).cuda(), kvh, 128)
    vs = ops.kv_scales(torch.cat(v).cuda(), kvh, 128)
    kv = G.GpuKV(k, v, kvh, fp8=True, k_scale=ks, v_scale=vs)
    try:
        assert ops.decode_tma_supported(h, kvh, "fp8_e4m3")
        maps = kv.engine.decode_maps(0, h)
        assert maps is not None
        for step in range(3):
            nk = synth.normal_bf16(rs, len(lens), kvh, 128)
            nv = synth.normal_bf16(rs, len(lens), kvh, 128)
            q = synth.normal_bf16(rs, len(lens), h, 128)
            lens = [n + 1 for n in lens]
            k = [torch.cat([a, b[None]]) for a, b in zip(k, nk)]
            v = [torch.cat([a, b[None]]) for a, b in zip(v, nv)]
            meta = VTensorMetadata(kv.slots, lens, kvh, 128, num_decode_tokens=len(lens), kv_elem_size=1)
            prepare_step(meta, kv.engine)
            out = torch.empty(len(lens), h, 128, dtype=torch.bfloat16, device="cuda")
            lse = torch.empty(len(lens), h, dtype=torch.float32, device="cuda")
            ws = ops.attn_workspace(out.device, len(lens), h, 128, meta.max_seq_len)
            ops.decode_step(out, q.cuda(), nk.cuda(), nv.cuda(), kv.k_table, kv.v_table, meta.slot_m, meta.slot_mapping,
                            meta.seq_lens_tensor, meta.max_seq_len, kvh, SCALE, "fp8_e4m3", ks, vs, lse=lse, workspace=ws,
                            maps=maps)
            torch.cuda.synchronize()
            assert ops.workspace_status(ws) == 0
            kv.lens = lens
            r = oracle.fill_ranges(k, v, k_scale=ks.cpu(), v_scale=vs.cpu())
            for i, n in enumerate(lens):
                assert torch.equal(kv.read_rows(i, "k"), r.k_rows(i, n, kvh, 128, fp8=True)), (step, i)
                assert torch.equal(kv.read_rows(i, "v"), r.v_rows(i, n, kvh, 128, fp8=True)), (step, i)
            port = oracle.port_decode_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32),
                                           kvh, SCALE, ks.cpu(), vs.cpu())
            ok, err = _tol_ok(out.cpu(), port)
            assert ok, (step, err)
            # the mma.sync kernel on the same (already extended) ranges: plain attention, no maps
            ref = torch.empty_like(out)
            lse_ref = torch.empty_like(lse)
            ops._decode(ref, q.cuda(), kv.k_table, kv.v_table, kvh, SCALE, meta.seq_lens_tensor, meta.max_seq_len,
                        meta.slot_mapping, ops._kv_dtype("fp8_e4m3"), ks, vs, lse_ref, 0)
            torch.cuda.synchronize()
            assert float((out.float() - ref.float()).abs().max()) <= 2e-2
            assert float((lse - lse_ref).abs().max()) <= 2e-2
    finally:
        kv.close()


def _attend(kv, q, maps, h):
    from glake_b200 import ops
    qd = q.cuda()
    out = torch.empty_like(qd)
    ops.paged_attention_v1(out, qd, kv.k_table, kv.v_table, kv.kvh, SCALE, kv.meta.seq_lens_tensor, 1,
                           kv.meta.max_seq_len, None, "fp8_e4m3", 1.0, kv.meta.slot_mapping, k_scale=kv.k_scale,
                           v_scale=kv.v_scale, maps=maps)
    torch.cuda.synchronize()
    assert ops.attn_status() == 0
    return out.cpu()


def test_full_context_golden_with_scales_from_the_prefill_append(G, oracle):
    """Config-4 shape (32 q / 8 kv heads, contexts up to 8k) on real data: against the committed
    output of the reference's CPU kernel over a bf16 cache (<= 3e-2) and against the fp8
    restatement (<= 1e-2); scales amax / 448 over the prefill rows, frozen."""
    from glake_b200 import ops
    from tests.test_oracle import load_golden
    name = "fp8_ctx_gqa4_8k"
    _, gold16 = load_golden(name)
    seed, lens, h, kvh = synth.golden_lens(name)
    assert ops.decode_tma_supported(h, kvh, "fp8_e4m3")
    q, k, v = synth.make_case(seed, lens, h, kvh)
    ks = ops.kv_scales(torch.cat([x[:-1] for x in k]).cuda(), kvh, 128)
    vs = ops.kv_scales(torch.cat([x[:-1] for x in v]).cuda(), kvh, 128)
    kv = G.GpuKV(k, v, kvh, fp8=True, k_scale=ks, v_scale=vs)
    try:
        r8 = oracle.fill_ranges(k, v, k_scale=ks.cpu(), v_scale=vs.cpu())
        port8 = oracle.port_decode_attn(q, r8, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32), kvh,
                                        SCALE, ks.cpu(), vs.cpu())
        o8 = _attend(kv, q, kv.engine.decode_maps(0, h), h)
        assert float((o8.float() - gold16.float()).abs().max()) <= 3e-2
        assert float((o8.float() - port8.float()).abs().max()) <= 1e-2
    finally:
        kv.close()


@pytest.mark.parametrize("h,kvh", [(16, 8), (16, 16)])
def test_many_short_streams_per_cta(G, oracle, h, kvh):
    """Around a thousand contexts of 1..150 tokens: every CTA walks through several whole streams
    (each published to and merged from the same scratch slot, both consumer sets, streams of a
    single tile leave one set empty), identical results on identical calls."""
    from glake_b200 import ops
    rs = np.random.RandomState(6160 + h + kvh)
    lens = [int(x) for x in rs.randint(1, 151, size=1000)]
    q, k, v = synth.make_case(950 + h + kvh, lens, h, kvh)
    ks = ops.kv_scales(torch.cat(k).cuda(), kvh, 128)
    vs = ops.kv_scales(torch.cat(v).cuda(), kvh, 128)
    kv = G.GpuKV(k, v, kvh, fp8=True, k_scale=ks, v_scale=vs)
    try:
        maps = kv.engine.decode_maps(0, h)
        outs = [_attend(kv, q, maps, h) for _ in range(3)]
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), "results differ between identical calls"
        r = oracle.fill_ranges(k, v, k_scale=ks.cpu(), v_scale=vs.cpu())
        port = oracle.port_decode_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32), kvh, SCALE,
                                       ks.cpu(), vs.cpu())
        ok, err = _tol_ok(outs[0], port)
        assert ok, err
    finally:
        kv.close()


def test_shapes_the_kernel_does_not_take_run_as_without_maps(G, oracle):
    """8 q heads per kv head is outside the tcgen05 kernel's shapes: the engine hands out no maps and
    the entry point, given maps of another shape's table, falls back to the mma.sync kernel."""
    from glake_b200 import ops
    assert not ops.decode_tma_supported(64, 8, "fp8_e4m3") and not ops.decode_tma_supported(32, 8, "auto")
    assert not ops.decode_tma_supported(8, 4, "fp8_e4m3")
    lens = [40, 700]
    q, k, v = synth.make_case(77, lens, 64, 8)
    ks = ops.kv_scales(torch.cat(k).cuda(), 8, 128)
    vs = ops.kv_scales(torch.cat(v).cuda(), 8, 128)
    kv = G.GpuKV(k, v, 8, fp8=True, k_scale=ks, v_scale=vs)
    try:
        assert kv.engine.decode_maps(0, 64) is None
        maps = kv.engine.decode_maps(0, 32)          # a valid table for these ranges; the 64-head call must ignore it
        got = _attend(kv, q, maps, 64)
        ref = _attend(kv, q, None, 64)
        assert torch.equal(got, ref)
    finally:
        kv.close()


@pytest.mark.parametrize("seed", range(6))
def test_random_batches_with_emptied_sequences(G, oracle, seed):
    """Randomised batches: piece boundaries, stream merges, fewer tiles than CTAs, more than 256
    sequences, a few long streams cut into many pieces; then the same batch with every third
    sequence emptied (zeros there, the others unchanged up to the order of the sums)."""
    from glake_b200 import ops
    rs = np.random.RandomState(3000 + seed)
    kvh = int(rs.choice([8, 16]))
    g = int(rs.choice([1, 2, 4]))
    h = kvh * g
    if seed == 1:
        batch, hi = 300, 40
    elif seed == 2:
        batch, hi = 3, 20000
    else:
        batch, hi = int(rs.randint(1, 40)), int(rs.choice([3, 70, 700, 3000]))
    lens = [int(x) for x in rs.randint(1, hi + 1, size=batch)]
    q, k, v = synth.make_case(4000 + seed, lens, h, kvh)
    ks = ops.kv_scales(torch.cat(k).cuda(), kvh, 128)
    vs = ops.kv_scales(torch.cat(v).cuda(), kvh, 128)
    kv = G.GpuKV(k, v, kvh, fp8=True, k_scale=ks, v_scale=vs)
    try:
        maps = kv.engine.decode_maps(0, h)
        assert maps is not None
        out = _attend(kv, q, maps, h)
        r = oracle.fill_ranges(k, v, k_scale=ks.cpu(), v_scale=vs.cpu())
        port = oracle.port_decode_attn(q, r, torch.arange(batch), torch.tensor(lens, dtype=torch.int32), kvh, SCALE,
                                       ks.cpu(), vs.cpu())
        # the oracle rounds every dequantised element to bf16, the kernel keeps fp8 * scale exact: on
        # contexts of a few dozen tokens that alone moves outputs by ~1e-2 (the fp8 contract tolerance, 3e-2)
        err = (out.float() - port.float()).abs()
        tol = torch.maximum(torch.full_like(err, 3e-2), port.float().abs() * 2.0 ** -6)
        assert bool((err <= tol).all()), (float((err - tol).max()), lens)
        ref = _attend(kv, q, None, h)                         # the mma.sync kernel on the same ranges
        assert float((out.float() - ref.float()).abs().max()) <= 2e-2
        if batch >= 3:
            sl = kv.meta.seq_lens_tensor.clone()
            kv.meta.seq_lens_tensor[::3] = 0
            out2 = _attend(kv, q, maps, h)
            kv.meta.seq_lens_tensor.copy_(sl)
            assert torch.equal(out2[::3], torch.zeros_like(out2[::3]))
            keep = [i for i in range(batch) if i % 3]
            assert float((out2[keep].float() - out[keep].float()).abs().max()) <= 4e-3
    finally:
        kv.close()
