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
