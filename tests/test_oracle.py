"""Pins the CPU checker: the C restatement against the golden vectors produced
by the reference's own CPU kernels, against those kernels run live (when the
prebuilt oracle/_ref loads on this CPU), and against plain fp32 PyTorch."""
import os

import numpy as np
import pytest
import torch

from tests import synth

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
SCALE = 128 ** -0.5


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = torch.from_numpy(z["out_bits"].copy()).view(torch.bfloat16)
    return z, out


def one_ulp_close(a, b, atol):
    """|a-b| <= atol, or a and b are neighbouring bf16 values (one rounding flip)."""
    af, bf = a.float(), b.float()
    ulp = torch.maximum(af.abs(), bf.abs()) * 2.0 ** -7
    return bool(((af - bf).abs() <= torch.maximum(torch.full_like(af, atol), ulp)).all())


@pytest.mark.parametrize("name", list(synth.GOLDEN_CASES) + list(synth.LONG_CASES))
def test_port_matches_golden(oracle, name):
    z, gold = load_golden(name)
    seed, lens, h, kvh = synth.golden_lens(name)
    assert lens == [int(x) for x in z["lens"]]
    q, k, v = synth.make_case(seed, lens, h, kvh)
    assert synth.digest(q, k, v) == str(z["input_sha256"]), "input generator drifted"
    r = oracle.fill_ranges(k, v)
    rows_k = [r.k_rows(i, n, kvh, 128) for i, n in enumerate(lens)]
    rows_v = [r.v_rows(i, n, kvh, 128) for i, n in enumerate(lens)]
    assert synth.digest(rows_k, rows_v) == str(z["cache_sha256"]), "cache contents differ"
    out = oracle.port_decode_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32),
                                  kvh, SCALE)
    if str(z["kernel"]) == "v1":
        # Same fp32 algorithm, different summation order: at most one bf16 rounding flip.
        assert one_ulp_close(out, gold, 1e-5)
        assert (out == gold).float().mean() > 0.99
    else:
        # Above 8192 tokens the reference merges 512-token partitions whose partial
        # outputs it keeps in bf16 (tmp_out, csrc/cpu/attention.cpp:436-441), so the
        # reference itself sits ~2e-4 from fp32 math there.
        assert one_ulp_close(out, gold, 5e-4)


@pytest.mark.parametrize("name", ["gqa4_small", "mha_edges", "gqa8"])
@pytest.mark.parametrize("force", ["v1", "v2"])
def test_port_matches_live_reference(oracle, name, force):
    if oracle.load_ref("bf16") is None or not oracle._cpu_has("avx512_bf16"):
        pytest.skip("prebuilt reference CPU kernels do not load on this CPU")
    seed, lens, h, kvh = synth.golden_lens(name)
    q, k, v = synth.make_case(seed, lens, h, kvh)
    ref = oracle.ref_decode_attn(q, k, v, SCALE, variant="bf16", force=force)
    r = oracle.fill_ranges(k, v)
    out = oracle.port_decode_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32),
                                  kvh, SCALE)
    assert one_ulp_close(out, ref, 1e-5 if force == "v1" else 5e-4)
    _, gold = load_golden(name)
    if force == "v1":
        assert torch.equal(ref, gold)


def test_port_matches_fp32_torch(oracle):
    seed, lens, h, kvh = 11, [5, 130, 700], 8, 4
    q, k, v = synth.make_case(seed, lens, h, kvh)
    r = oracle.fill_ranges(k, v)
    out, lse = oracle.port_decode_attn(q, r, torch.arange(3), torch.tensor(lens, dtype=torch.int32),
                                       kvh, SCALE, return_lse=True)
    ref = oracle.torch_decode_attn(q, k, v, SCALE)
    assert one_ulp_close(out, ref.bfloat16(), 1e-5)
    for i, n in enumerate(lens):
        kk = k[i].float().repeat_interleave(h // kvh, dim=1)
        want = torch.logsumexp(SCALE * torch.einsum("hd,thd->ht", q[i].float(), kk), dim=-1)
        assert torch.allclose(lse[i], want, atol=1e-4)


def test_append_decode_and_prefill_addressing(oracle):
    """Byte-offset addressing of reshape_and_cache: decode rows land at
    table[slot] + off, prefill rows at off + t*row, padded entries are skipped."""
    kvh, d, row = 4, 128, 4 * 128 * 2
    rng = oracle.HostRanges(6, 64 * row)
    rs = np.random.RandomState(3)
    # prefill: 3 sequences into slots 5, 0, 2
    lens = torch.tensor([7, 1, 20], dtype=torch.int32)
    starts = torch.tensor([0, 7, 8], dtype=torch.int32)
    key = synth.normal_bf16(rs, 28, kvh, d)
    val = synth.normal_bf16(rs, 28, kvh, d)
    slots = torch.tensor([5, 0, 2])
    off = torch.tensor([0, 3 * row, 0])
    oracle.port_append(rng, key, val, off, slots, lens, starts, max_seq_len=20)
    assert torch.equal(rng.k_rows(5, 7, kvh, d), key[:7])
    assert torch.equal(rng.v_rows(0, 4, kvh, d)[3], val[7])
    assert torch.equal(rng.k_rows(2, 20, kvh, d), key[8:])
    # decode: one row each, middle entry padded (-1), strided source (fused qkv)
    fused = synth.normal_bf16(rs, 3, 3 * kvh * d)
    kd = fused[:, : kvh * d].view(3, kvh, d)
    vd = fused[:, kvh * d: 2 * kvh * d].view(3, kvh, d)
    assert kd.stride(0) == 3 * kvh * d
    off = torch.tensor([7 * row, -1, 20 * row])
    before = rng.k[0].clone()
    oracle.port_append(rng, kd, vd, off, slots)
    assert torch.equal(rng.k_rows(5, 8, kvh, d)[7], kd[0])
    assert torch.equal(rng.v_rows(2, 21, kvh, d)[20], vd[2])
    assert torch.equal(rng.k[0], before)


def test_fp8_e4m3_conversion_pins(oracle):
    """Quantise/dequantise against torch's float8_e4m3fn and the reference's
    round-trip tolerance (GLakeServe/tests/kernels/test_cache.py:355-380)."""
    lib = oracle.load_port()
    xs = torch.cat([torch.linspace(-600, 600, 4001), torch.randn(4000) * 0.02,
                    torch.tensor([0.0, 448.0, 464.0, 465.0, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9,
                                  float("inf"), -float("inf")])])
    mine = torch.tensor([lib.vto_f32_to_e4m3(float(x)) for x in xs], dtype=torch.uint8)
    want = xs.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(mine, want)
    allb = torch.arange(256, dtype=torch.uint8)
    deq = torch.tensor([lib.vto_e4m3_to_f32(int(b)) for b in allb])
    want = allb.view(torch.float8_e4m3fn).float()
    assert torch.equal(deq.nan_to_num(7.0), want.nan_to_num(7.0))
    u = (torch.rand(2000) * 2 - 1) * 224
    rt = torch.tensor([lib.vto_e4m3_to_f32(lib.vto_f32_to_e4m3(float(x))) for x in u])
    assert torch.allclose(rt, u, atol=0.001, rtol=0.1)


def test_fp8_attention_close_to_bf16(oracle):
    seed, lens, h, kvh = 21, [64, 900], 8, 2
    q, k, v = synth.make_case(seed, lens, h, kvh)
    ks = oracle.port_kv_scales(torch.cat(k))
    vs = oracle.port_kv_scales(torch.cat(v))
    assert torch.allclose(ks, torch.cat(k).float().abs().amax(dim=(0, 2)) / 448)
    r8 = oracle.fill_ranges(k, v, k_scale=ks, v_scale=vs)
    r16 = oracle.fill_ranges(k, v)
    sl = torch.tensor(lens, dtype=torch.int32)
    o8 = oracle.port_decode_attn(q, r8, torch.arange(2), sl, kvh, SCALE, ks, vs)
    o16 = oracle.port_decode_attn(q, r16, torch.arange(2), sl, kvh, SCALE)
    assert (o8.float() - o16.float()).abs().max() < 3e-2
    # stored bytes follow sat(x / scale)
    want = (k[1].float() / ks[None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(r8.k_rows(1, lens[1], kvh, 128, fp8=True), want)


def test_prefill_attention_is_causal(oracle):
    seed, lens, h, kvh = 31, [40, 9], 4, 2
    q, k, v = synth.make_case(seed, lens, h, kvh)
    r = oracle.fill_ranges(k, v)
    q_lens = torch.tensor([8, 9], dtype=torch.int32)
    q_start = torch.tensor([0, 8], dtype=torch.int32)
    rs = np.random.RandomState(5)
    qq = synth.normal_bf16(rs, 17, h, 128)
    out = oracle.port_prefill_attn(qq, r, torch.arange(2), torch.tensor(lens, dtype=torch.int32),
                                   q_lens, q_start, kvh, SCALE)
    for i in range(2):
        for j in range(int(q_lens[i])):
            n = lens[i] - int(q_lens[i]) + j + 1
            want = oracle.torch_decode_attn(qq[int(q_start[i]) + j][None], [k[i][:n]], [v[i][:n]], SCALE)[0]
            assert one_ulp_close(out[int(q_start[i]) + j], want.bfloat16(), 1e-5)


def _from_bits(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def prefill_case_inputs(name):
    seed, lens, q_lens, h, kvh = synth.PREFILL_CASES[name]
    _, k, v = synth.make_case(seed, lens, h, kvh)
    q = synth.make_prefill_queries(seed, q_lens, h)
    starts = np.concatenate([[0], np.cumsum(q_lens)[:-1]]).astype(np.int32)
    return lens, q_lens, h, kvh, q, k, v, torch.from_numpy(starts)


@pytest.mark.parametrize("name", list(synth.PREFILL_CASES))
def test_port_prefill_matches_reference_golden(oracle, name):
    """Causal prefix attention of the restatement against the reference's CPU decode kernel run
    once per new token (stored golden): same fp32 algorithm, at most one bf16 rounding flip."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    lens, q_lens, h, kvh, q, k, v, starts = prefill_case_inputs(name)
    assert synth.digest(q, k, v) == str(z["input_sha256"]), "input generator drifted"
    gold = _from_bits(z["out_bits"])
    r = oracle.fill_ranges(k, v)
    out = oracle.port_prefill_attn(q, r, torch.arange(len(lens)), torch.tensor(lens, dtype=torch.int32),
                                   torch.tensor(q_lens, dtype=torch.int32), starts, kvh, SCALE)
    assert one_ulp_close(out, gold, 1e-5)
    assert (out == gold).float().mean() > 0.99


@pytest.mark.parametrize("name", list(synth.ROPE_CASES))
def test_port_rotary_matches_golden(oracle, name):
    """The restated rotary embedding reproduces the reference CPU kernel's q and k bit for bit."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    seed, tokens, h, kvh, rot, neox, max_pos = synth.ROPE_CASES[name]
    pos, q, k, v = synth.make_rope_case(seed, tokens, h, kvh, max_pos)
    cs = oracle.make_cos_sin_cache(max_pos, rot)
    assert synth.digest(pos, q, k, v, cs) == str(z["input_sha256"]), "input generator drifted"
    q0 = q.clone()
    oracle.port_rotary_embedding(pos, q, k, 128, cs, neox)
    assert torch.equal(q, _from_bits(z["q_bits"])) and torch.equal(k, _from_bits(z["k_bits"]))
    if rot < 128:   # elements beyond rot_dim pass through
        assert torch.equal(q.view(tokens, h, 128)[..., rot:], q0.view(tokens, h, 128)[..., rot:])


@pytest.mark.parametrize("name", list(synth.NORM_CASES))
def test_port_rms_norm_matches_golden(oracle, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    seed, tokens, hidden, eps = synth.NORM_CASES[name]
    x, r, w = synth.make_norm_case(seed, tokens, hidden)
    assert synth.digest(x, r, w) == str(z["input_sha256"]), "input generator drifted"
    plain = torch.empty_like(x)
    oracle.port_rms_norm(plain, x, w, eps)
    fx, fr = x.clone(), r.clone()
    oracle.port_rms_norm(fx, fx, w, eps, residual=fr)
    assert torch.equal(fr, _from_bits(z["residual_bits"]))          # one fp32 add, one rounding: exact
    # the sum of squares may be taken in another order: at most one bf16 rounding flip
    assert one_ulp_close(plain, _from_bits(z["plain_bits"]), 0.0)
    assert one_ulp_close(fx, _from_bits(z["fused_bits"]), 0.0)
    assert (plain == _from_bits(z["plain_bits"])).float().mean() > 0.99


def test_port_rotary_and_norm_match_live_reference(oracle):
    ref = oracle.load_ref()
    if ref is None:
        pytest.skip("prebuilt reference CPU kernels do not load on this CPU")
    exact = oracle._cpu_has("avx512_bf16")      # the plain AVX-512 build truncates instead of rounding
    pos, q, k, v = synth.make_rope_case(5, 33, 8, 8, 8192)
    for rot, neox in ((128, True), (128, False), (32, True)):
        cs = oracle.make_cos_sin_cache(8192, rot)
        q1, k1, q2, k2 = q.clone(), k.clone(), q.clone(), k.clone()
        ref.rotary_embedding(pos, q1, k1, 128, cs, neox)
        oracle.port_rotary_embedding(pos, q2, k2, 128, cs, neox)
        if exact:
            assert torch.equal(q1, q2) and torch.equal(k1, k2)
        else:
            assert one_ulp_close(q1, q2, 0.0) and one_ulp_close(k1, k2, 0.0)
    x, r, w = synth.make_norm_case(6, 5, 8192)
    a, b = x.clone(), x.clone()
    ra, rb = r.clone(), r.clone()
    ref.fused_add_rms_norm(a, ra, w, 1e-5)
    oracle.port_rms_norm(b, b, w, 1e-5, residual=rb)
    assert one_ulp_close(a, b, 0.0) and one_ulp_close(ra, rb, 0.0)
