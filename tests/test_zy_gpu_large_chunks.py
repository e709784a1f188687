"""The path on a pool of 8 MiB chunks (vmmAllocator.set_chunk_bytes): the driver charges per
chunk, so larger chunks are a supported tuning.  Append, decode attention (bf16, and fp8 on
the tcgen05 kernel over tensor maps) and the TMA prefill must not care where a chunk ends:
contexts here end just before, at and after an 8 MiB boundary of their ranges."""
import numpy as np
import pytest
import torch

from tests import synth

pytestmark = pytest.mark.gpu
SCALE = 128 ** -0.5
MiB = 1 << 20


@pytest.fixture
def G8():
    from glake_b200 import vmmAllocator as A
    from tests import gpu_util
    gpu_util.ensure_pool()
    try:
        A.shutdown()                       # needs every earlier engine closed
    except Exception as exc:               # a leaked segment of an earlier test: not this test's subject
        pytest.skip(f"the shared pool could not be released: {exc}")
    A.set_chunk_bytes(8 * MiB)
    try:
        assert A.init_physical_handle(1024, torch.cuda.current_device())
        yield gpu_util
    finally:
        A.shutdown()
        A.set_chunk_bytes(2 * MiB)


@pytest.mark.parametrize("fp8", [False, True])
def test_decode_and_prefill_across_8mib_chunk_ends(G8, oracle, fp8):
    from glake_b200 import ops, vmmAllocator as A
    assert A.granularitySize == 8 * MiB
    h, kvh = 16, 8
    rows_per_chunk = 8 * MiB // (kvh * 128 * (1 if fp8 else 2))          # 8192 (fp8) / 4096 (bf16) tokens
    lens = [rows_per_chunk - 1, rows_per_chunk, rows_per_chunk + 1, 2 * rows_per_chunk + 17, 40]
    q, k, v = synth.make_case(2024 + fp8, lens, h, kvh)
    ks = vs = None
    if fp8:
        ks = ops.kv_scales(torch.cat(k).cuda(), kvh, 128)
        vs = ops.kv_scales(torch.cat(v).cuda(), kvh, 128)
    kv = G8.GpuKV(k, v, kvh, fp8=fp8, k_scale=ks, v_scale=vs)
    try:
        seg = kv.engine.vmm_kvcache_segment[3]
        assert seg.actual_size % (8 * MiB) == 0 and seg.actual_size >= 3 * 8 * MiB
        sl = torch.tensor(lens, dtype=torch.int32)
        if fp8:
            r = oracle.fill_ranges(k, v, k_scale=ks.cpu(), v_scale=vs.cpu())
            for i, n in enumerate(lens):
                assert torch.equal(kv.read_rows(i, "k"), r.k_rows(i, n, kvh, 128, fp8=True))
            port = oracle.port_decode_attn(q, r, torch.arange(len(lens)), sl, kvh, SCALE, ks.cpu(), vs.cpu())
            maps = kv.engine.decode_maps(0, h)
            assert maps is not None
            out = torch.empty(len(lens), h, 128, dtype=torch.bfloat16, device="cuda")
            ops.paged_attention_v1(out, q.cuda(), kv.k_table, kv.v_table, kvh, SCALE, kv.meta.seq_lens_tensor, 1,
                                   kv.meta.max_seq_len, None, "fp8_e4m3", 1.0, kv.meta.slot_mapping, k_scale=ks,
                                   v_scale=vs, maps=maps)
            torch.cuda.synchronize()
            assert ops.attn_status() == 0
            err = (out.cpu().float() - port.float()).abs()
            assert bool((err <= torch.maximum(torch.full_like(err, 1e-2), port.float().abs() * 2.0 ** -6)).all()), float(err.max())
            assert float((kv.attend(q, SCALE).float() - port.float()).abs().max()) <= 1e-2     # the mma.sync engine
        else:
            for i in range(len(lens)):
                assert torch.equal(kv.read_rows(i, "k"), k[i]) and torch.equal(kv.read_rows(i, "v"), v[i])
            r = oracle.fill_ranges(k, v)
            port = oracle.port_decode_attn(q, r, torch.arange(len(lens)), sl, kvh, SCALE)
            got = kv.attend(q, SCALE)
            err = (got.float() - port.float()).abs()
            assert bool((err <= torch.maximum(torch.full_like(err, 2e-3), port.float().abs() * 2.0 ** -7)).all()), float(err.max())
            # prefix-extend over the same ranges with tensor copies: the last 70 tokens of every sequence as new tokens
            q_lens = [min(70, n) for n in lens]
            rs = np.random.RandomState(5)
            qp = synth.normal_bf16(rs, sum(q_lens), h, 128)
            ql = torch.tensor(q_lens, dtype=torch.int32)
            qs = torch.tensor([sum(q_lens[:i]) for i in range(len(lens))], dtype=torch.int32)
            outp = torch.empty(sum(q_lens), h, 128, dtype=torch.bfloat16, device="cuda")
            ops.prefill_attention(outp, qp.cuda(), kv.k_table, kv.v_table, kvh, SCALE, kv.meta.slot_mapping,
                                  kv.meta.seq_lens_tensor, ql.cuda(), qs.cuda(), max(q_lens), maps=kv.engine.prefill_maps(0))
            torch.cuda.synchronize()
            want = oracle.port_prefill_attn(qp, r, torch.arange(len(lens)), sl, ql, qs, kvh, SCALE)
            err = (outp.cpu().float() - want.float()).abs()
            assert bool((err <= torch.maximum(torch.full_like(err, 2e-3), want.float().abs() * 2.0 ** -7)).all()), float(err.max())
    finally:
        kv.close()
