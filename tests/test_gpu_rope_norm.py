"""GPU parity of the element-wise steps either side of the attention: rotary
embedding fused with the KV append, rms_norm and fused_add_rms_norm — through the
C ABI, against the reference CPU kernels' golden vectors and the CPU oracle.

Tolerances: the rotation evaluates the same fp32 expression as the oracle, so q,
the rotated key written back and the bf16 cache rows are bit-exact, and fp8 cache
bytes equal the oracle's quantisation of the rotated key.  rms_norm sums the
squares in another order than the oracle: at most one bf16 rounding flip per
element (|a-b| <= 2^-7 * max(|a|,|b|))."""
import ctypes
import os

import numpy as np
import pytest
import torch

from tests import synth
from tests.test_oracle import GOLDEN, SCALE, _from_bits, one_ulp_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    from tests import gpu_util
    gpu_util.ensure_pool()
    return gpu_util


class Ranges:
    """Engine + metadata of one batch; rows are read back through vt_pool_read."""

    def __init__(self, G, kvh, n_slots, max_tokens, fp8=False):
        from glake_b200.backend import VTensorCacheEngine
        self.G, self.kvh, self.fp8 = G, kvh, fp8
        self.engine = VTensorCacheEngine(1, kvh, 128, n_slots, max_tokens, cache_dtype="fp8_e4m3" if fp8 else "auto")

    def step(self, slots, lens, prefill):
        from glake_b200.backend import VTensorMetadata, prepare_step
        kw = dict(num_prefills=len(slots)) if prefill else dict(num_decode_tokens=len(slots))
        meta = VTensorMetadata(slots, lens, self.kvh, 128, kv_elem_size=1 if self.fp8 else 2, **kw)
        prepare_step(meta, self.engine)
        return meta

    def rows(self, slot, n, which):
        from glake_b200 import vmmAllocator as A
        from glake_b200._lib import check, lib
        seg = self.engine.vmm_kvcache_segment[slot]
        base = seg.getKeyDevicePtr(0) if which == "k" else seg.getValueDevicePtr(0)
        out = torch.empty(n * self.kvh * 128 * (1 if self.fp8 else 2), dtype=torch.uint8)
        torch.cuda.synchronize()
        check(lib.vt_pool_read(A._pool, ctypes.c_void_p(out.data_ptr()), base, out.numel()), "vt_pool_read")
        return out.view(n, self.kvh, 128) if self.fp8 else out.view(torch.bfloat16).view(n, self.kvh, 128)

    def close(self):
        self.engine.close()


def rope_call(R, meta, pos, q, k, v, cs, neox, max_seq_len, **kw):
    from glake_b200 import ops
    e = R.engine
    ops.rotary_embedding_and_cache(pos, q, k, v, 128, cs, neox, e.k_cache_ptr[0], e.v_cache_ptr[0], meta.slot_m,
                                   meta.slot_mapping, meta.seq_lens_tensor, meta.cache_seq_lens, max_seq_len, R.kvh, **kw)
    torch.cuda.synchronize()


@pytest.mark.parametrize("name", list(synth.ROPE_CASES))
@pytest.mark.parametrize("write_key", [False, True])
def test_rope_append_golden_decode(G, oracle, name, write_key):
    """Every token of the golden case is one decode entry of its own slot."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    seed, tokens, h, kvh, rot, neox, max_pos = synth.ROPE_CASES[name]
    pos, q, k, v = synth.make_rope_case(seed, tokens, h, kvh, max_pos)
    cs = oracle.make_cos_sin_cache(max_pos, rot)
    gq, gk = _from_bits(z["q_bits"]), _from_bits(z["k_bits"])
    R = Ranges(G, kvh, tokens, 64)
    try:
        lens = [1] * tokens
        meta = R.step(list(range(tokens)), lens, prefill=False)
        qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
        rope_call(R, meta, pos.cuda(), qd, kd, vd, cs.cuda(), neox, 1, write_key=write_key)
        assert torch.equal(qd.cpu(), gq), "rotated query differs from the reference CPU kernel"
        assert torch.equal(kd.cpu(), gk if write_key else k)
        assert torch.equal(vd.cpu(), v)
        for i in range(tokens):
            assert torch.equal(R.rows(i, 1, "k").reshape(-1), gk[i]), f"cache K row of entry {i}"
            assert torch.equal(R.rows(i, 1, "v").reshape(-1), v[i])
    finally:
        R.close()


@pytest.mark.parametrize("neox,rot", [(True, 128), (False, 128), (True, 64), (False, 32)])
@pytest.mark.parametrize("fp8", [False, True])
def test_rope_append_prefill_strided_and_padded(G, oracle, neox, rot, fp8):
    """Ragged prefill entries out of a fused qkv buffer (strided views), one padded
    entry, fp8 quantisation of the rotated key, growth across chunk boundaries."""
    from glake_b200 import ops
    h, kvh = 8, 2
    lens = [700, 1, 1300, 37]                                  # kvh 2: 4096 bf16 rows per chunk ... fp8 8192
    slots = [2, 0, 3, 1]
    n = sum(lens)
    rs = np.random.RandomState(40 + rot)
    qkv = synth.normal_bf16(rs, n, (h + 2 * kvh) * 128)
    pos = torch.from_numpy(rs.randint(0, 4096, size=n).astype(np.int64))
    cs = oracle.make_cos_sin_cache(4096, rot)
    q, k, v = qkv.split([h * 128, kvh * 128, kvh * 128], dim=-1)
    # oracle: rotate copies, then append
    q_ref, k_ref = q.clone(), k.clone()
    oracle.port_rotary_embedding(pos, q_ref, k_ref, 128, cs, neox)
    k_scale = v_scale = None
    if fp8:
        k_scale = oracle.port_kv_scales(k_ref.view(n, kvh, 128))
        v_scale = oracle.port_kv_scales(v.reshape(n, kvh, 128))
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
    r = oracle.fill_ranges([k_ref[s:s + m].view(m, kvh, 128) for s, m in zip(starts, lens)],
                           [v[s:s + m].reshape(m, kvh, 128) for s, m in zip(starts, lens)],
                           k_scale=k_scale, v_scale=v_scale)
    R = Ranges(G, kvh, 4, 1400, fp8=fp8)
    try:
        meta = R.step(slots, lens, prefill=True)
        meta.slot_m[1] = -1                                     # entry 1 is padding: no cache write, still rotated
        d = qkv.cuda()
        qd, kd, vd = d.split([h * 128, kvh * 128, kvh * 128], dim=-1)
        kw = dict(kv_cache_dtype="fp8_e4m3", k_scale=k_scale.cuda(), v_scale=v_scale.cuda()) if fp8 else {}
        rope_call(R, meta, pos.cuda(), qd, kd, vd, cs.cuda(), neox, max(lens), **kw)
        back = d.cpu()
        assert torch.equal(back[:, : h * 128], q_ref)
        assert torch.equal(back[:, h * 128:], qkv[:, h * 128:])          # key and value untouched
        for i, (slot, m) in enumerate(zip(slots, lens)):
            if i == 1:
                continue
            assert torch.equal(R.rows(slot, m, "k"), r.k_rows(i, m, kvh, 128, fp8)), f"K rows of entry {i}"
            assert torch.equal(R.rows(slot, m, "v"), r.v_rows(i, m, kvh, 128, fp8)), f"V rows of entry {i}"
    finally:
        R.close()


def test_rope_append_then_attention_matches_oracle(G, oracle):
    """A decode step of a layer: rotate + append in one launch, then attend."""
    from glake_b200 import ops
    h, kvh = 16, 2
    lens = [513, 2048, 90, 1025]
    q, k, v = synth.make_case(77, lens, h, kvh)
    cs = oracle.make_cos_sin_cache(4096, 128)
    # the cache holds rotated keys of positions 0..L-1; rotate them on the host
    k_rot = []
    for x in k:
        xr = x.clone().view(x.shape[0], -1)
        dummy_q = torch.zeros(x.shape[0], 128, dtype=torch.bfloat16)
        oracle.port_rotary_embedding(torch.arange(x.shape[0]), dummy_q, xr, 128, cs, True)
        k_rot.append(xr.view_as(x))
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int64)
    q_ref = q.clone().view(len(lens), -1)
    oracle.port_rotary_embedding(pos, q_ref, torch.zeros(len(lens), 128, dtype=torch.bfloat16), 128, cs, True)
    r = oracle.fill_ranges(k_rot, v)
    port = oracle.port_decode_attn(q_ref.view_as(q), r, torch.arange(4), torch.tensor(lens, dtype=torch.int32), kvh, SCALE)
    R = Ranges(G, kvh, 4, 2100)
    try:
        pre = [n - 1 for n in lens]
        meta = R.step([0, 1, 2, 3], pre, prefill=True)
        e = R.engine
        ops.reshape_and_cache(torch.cat([x[:-1] for x in k_rot]).cuda(), torch.cat([x[:-1] for x in v]).cuda(),
                              e.k_cache_ptr[0], e.v_cache_ptr[0], meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor,
                              meta.cache_seq_lens, max(pre), kvh, 128)
        meta = R.step([0, 1, 2, 3], lens, prefill=False)
        qd = q.cuda().view(4, -1)
        kd = torch.stack([x[-1] for x in k]).cuda().view(4, -1)      # un-rotated newest keys
        vd = torch.stack([x[-1] for x in v]).cuda().view(4, -1)
        rope_call(R, meta, pos.cuda(), qd, kd, vd, cs.cuda(), True, 1)
        out = torch.empty(4, h, 128, dtype=torch.bfloat16, device="cuda")
        ops.paged_attention_v1(out, qd.view(4, h, 128), e.gpu_cache[0][0].vmm_ptr, e.gpu_cache[0][1].vmm_ptr, kvh, SCALE,
                               meta.seq_lens_tensor, 1, max(lens), None, "auto", 1.0, meta.slot_mapping)
        torch.cuda.synchronize()
        assert torch.equal(R.rows(1, lens[1], "k"), k_rot[1])
        err = float((out.cpu().float() - port.float()).abs().max())
        assert err <= 2e-3 or one_ulp_close(out.cpu(), port, 2e-3), err
    finally:
        R.close()


@pytest.mark.parametrize("name", list(synth.NORM_CASES))
def test_rms_norm_golden(G, name):
    from glake_b200 import ops
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    seed, tokens, hidden, eps = synth.NORM_CASES[name]
    x, r, w = synth.make_norm_case(seed, tokens, hidden)
    xd, rd, wd = x.cuda(), r.cuda(), w.cuda()
    out = torch.empty_like(xd)
    ops.rms_norm(out, xd, wd, eps)
    ops.fused_add_rms_norm(xd, rd, wd, eps)
    torch.cuda.synchronize()
    assert torch.equal(rd.cpu(), _from_bits(z["residual_bits"]))
    assert one_ulp_close(out.cpu(), _from_bits(z["plain_bits"]), 0.0)
    assert one_ulp_close(xd.cpu(), _from_bits(z["fused_bits"]), 0.0)
    assert (out.cpu() == _from_bits(z["plain_bits"])).float().mean() > 0.99


@pytest.mark.parametrize("tokens,hidden", [(64, 4096), (64, 8192), (7, 5120), (1, 16384), (3, 136)])
def test_rms_norm_shapes_against_the_oracle(G, oracle, tokens, hidden):
    from glake_b200 import ops
    x, r, w = synth.make_norm_case(100 + hidden, tokens, hidden)
    # plain, out of a strided view (a slice of a wider buffer)
    wide = torch.zeros(tokens, hidden + 64, dtype=torch.bfloat16)
    wide[:, :hidden] = x
    wd = wide.cuda()
    out = torch.empty(tokens, hidden, dtype=torch.bfloat16, device="cuda")
    ops.rms_norm(out, wd[:, :hidden], w.cuda(), 1e-5)
    ref = torch.empty_like(x)
    oracle.port_rms_norm(ref, x, w, 1e-5)
    assert one_ulp_close(out.cpu(), ref, 0.0)
    # fused, in place
    xd, rd = x.cuda(), r.cuda()
    ops.fused_add_rms_norm(xd, rd, w.cuda(), 1e-5)
    fx, fr = x.clone(), r.clone()
    oracle.port_rms_norm(fx, fx, w, 1e-5, residual=fr)
    assert torch.equal(rd.cpu(), fr)
    assert one_ulp_close(xd.cpu(), fx, 0.0)
    assert (xd.cpu() == fx).float().mean() > 0.99


def test_rope_and_norm_reject_what_they_cannot_do(G):
    from glake_b200 import VTensorError, ops
    R = Ranges(G, 1, 1, 64)
    try:
        meta = R.step([0], [1], prefill=False)
        q = torch.zeros(1, 128, dtype=torch.bfloat16, device="cuda")
        pos = torch.zeros(1, dtype=torch.int64, device="cuda")
        with pytest.raises(VTensorError):                      # rot_dim must be a multiple of 16
            rope_call(R, meta, pos, q, q.clone(), q.clone(), torch.zeros(8, 24, dtype=torch.bfloat16, device="cuda"), True, 1)
        with pytest.raises(RuntimeError):                      # no CPU path
            ops.rms_norm(torch.zeros(1, 8, dtype=torch.bfloat16), torch.zeros(1, 8, dtype=torch.bfloat16),
                         torch.zeros(8, dtype=torch.bfloat16), 1e-5)
        big = torch.zeros(1, 16384 + 8, dtype=torch.bfloat16, device="cuda")
        with pytest.raises(VTensorError):                      # rows beyond 16384 elements
            ops.rms_norm(torch.empty_like(big), big, big[0], 1e-5)
    finally:
        R.close()
