"""A small decoder stack driven end to end through the library's ops, the way
LlamaDecoderLayer.forward chains them (GLakeServe/vllm/model_executor/models/llama.py:233-262,
:164-181): rms_norm / fused_add_rms_norm -> qkv projection -> rotary embedding fused
with the KV append -> prefill or decode attention over the slots' ranges -> output
projection.  Only the projections are plain torch matmuls.  The same sequence runs on
the CPU with the oracle's restatements (and fp32 matmuls rounded to bf16) and the
hidden states are compared after the prompt and after every decode step.

Tolerance: the projections accumulate in different orders on the two sides, so
activations drift by bf16 rounding flips that the next layers amplify; the test asks
for a relative error of the final hidden state below 3e-2 in the max norm, while a
wrong position, a misplaced cache row or a swapped residual gives errors of order 1."""
import numpy as np
import pytest
import torch

from tests import synth

pytestmark = pytest.mark.gpu

HID, H, KVH, D, LAYERS, EPS = 512, 4, 2, 128, 2, 1e-5
SCALE = D ** -0.5


def _weights():
    rs = np.random.RandomState(3)
    def w(*shape, s):
        return torch.from_numpy((rs.standard_normal(shape) * s).astype(np.float32)).bfloat16()
    return [dict(ln1=w(HID, s=0.1) + 1, ln2=w(HID, s=0.1) + 1, qkv=w(HID, (H + 2 * KVH) * D, s=HID ** -0.5),
                 o=w(H * D, HID, s=(H * D) ** -0.5)) for _ in range(LAYERS)]


def _mm(x, w):
    return (x.float() @ w.float()).to(torch.bfloat16)


class CpuStack:
    """The oracle side: per layer and sequence the rotated keys and the values seen so far."""

    def __init__(self, oracle, weights, cs):
        self.O, self.W, self.cs = oracle, weights, cs
        self.k = [[None, None] for _ in range(LAYERS)]      # [layer][seq] -> [t, KVH, D]
        self.v = [[None, None] for _ in range(LAYERS)]

    def forward(self, hidden, positions, seq_of_row):
        O = self.O
        residual = None
        for li, w in enumerate(self.W):
            if residual is None:
                residual = hidden.clone()
                x = torch.empty_like(hidden)
                O.port_rms_norm(x, hidden, w["ln1"], EPS)
            else:
                x = hidden.clone()
                O.port_rms_norm(x, x, w["ln1"], EPS, residual=residual)
            qkv = _mm(x, w["qkv"])
            q, k, v = [t.contiguous() for t in qkv.split([H * D, KVH * D, KVH * D], dim=-1)]
            O.port_rotary_embedding(positions, q, k, D, self.cs, True)
            out = torch.empty(len(seq_of_row), H, D, dtype=torch.bfloat16)
            for s in sorted(set(seq_of_row)):
                rows = [i for i, x_ in enumerate(seq_of_row) if x_ == s]
                kn, vn = k[rows].view(-1, KVH, D), v[rows].view(-1, KVH, D)
                self.k[li][s] = kn if self.k[li][s] is None else torch.cat([self.k[li][s], kn])
                self.v[li][s] = vn if self.v[li][s] is None else torch.cat([self.v[li][s], vn])
                n = self.k[li][s].shape[0]
                r = O.fill_ranges([self.k[li][s]], [self.v[li][s]])
                o = O.port_prefill_attn(q[rows].view(-1, H, D), r, torch.zeros(1, dtype=torch.int64),
                                        torch.tensor([n], dtype=torch.int32), torch.tensor([len(rows)], dtype=torch.int32),
                                        torch.zeros(1, dtype=torch.int32), KVH, SCALE)
                out[rows] = o
            hidden = _mm(out.view(-1, H * D), w["o"])
            x = hidden.clone()
            O.port_rms_norm(x, x, w["ln2"], EPS, residual=residual)     # stands in for the MLP block's norm
            hidden = x
        return hidden


def test_decoder_stack_prompt_then_decode_steps(oracle):
    from glake_b200 import ops
    from glake_b200.backend import VTensorCacheEngine, VTensorMetadata, prepare_step
    from tests import gpu_util
    gpu_util.ensure_pool()
    W = _weights()
    Wd = [{k: t.cuda() for k, t in w.items()} for w in W]
    cs = oracle.make_cos_sin_cache(512, D)
    csd = cs.cuda()
    prompts = [37, 150]
    rs = np.random.RandomState(4)
    eng = VTensorCacheEngine(LAYERS, KVH, D, 2, 256)
    cpu = CpuStack(oracle, W, cs)
    try:
        lens = list(prompts)
        for step in range(6):                                   # step 0 = prompts, then 5 decode steps
            prefill = step == 0
            if prefill:
                seq_of_row = [0] * prompts[0] + [1] * prompts[1]
                positions = torch.cat([torch.arange(n) for n in prompts])
            else:
                lens = [n + 1 for n in lens]
                seq_of_row = [0, 1]
                positions = torch.tensor([n - 1 for n in lens])
            hidden = synth.normal_bf16(rs, len(seq_of_row), HID)
            want = cpu.forward(hidden, positions, seq_of_row)

            meta = VTensorMetadata([0, 1], lens, KVH, D, **(dict(num_prefills=2) if prefill else dict(num_decode_tokens=2)))
            prepare_step(meta, eng)
            h, pos = hidden.cuda(), positions.cuda()
            residual = None
            for li, w in enumerate(Wd):
                if residual is None:
                    residual = h.clone()
                    x = torch.empty_like(h)
                    ops.rms_norm(x, h, w["ln1"], EPS)
                else:
                    x = h
                    ops.fused_add_rms_norm(x, residual, w["ln1"], EPS)
                qkv = x @ w["qkv"]
                q, k, v = qkv.split([H * D, KVH * D, KVH * D], dim=-1)      # strided views of the fused projection
                ops.rotary_embedding_and_cache(pos, q, k, v, D, csd, True, eng.k_cache_ptr[li], eng.v_cache_ptr[li],
                                               meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor, meta.cache_seq_lens,
                                               max(prompts) if prefill else 1, KVH)
                out = torch.empty(len(seq_of_row), H, D, dtype=torch.bfloat16, device="cuda")
                kt, vt = eng.gpu_cache[li][0].vmm_ptr, eng.gpu_cache[li][1].vmm_ptr
                q3 = q.reshape(-1, H, D)
                if prefill:
                    ql = torch.tensor(prompts, dtype=torch.int32, device="cuda")
                    ops.prefill_attention(out, q3, kt, vt, KVH, SCALE, meta.slot_mapping, meta.seq_lens_tensor, ql,
                                          meta.cache_seq_lens, max(prompts), maps=eng.prefill_maps(li))
                else:
                    ops.paged_attention_v1(out, q3, kt, vt, KVH, SCALE, meta.seq_lens_tensor, 1, max(lens), None, "auto",
                                           1.0, meta.slot_mapping)
                h = out.view(-1, H * D) @ w["o"]
                ops.fused_add_rms_norm(h, residual, w["ln2"], EPS)
            torch.cuda.synchronize()
            got = h.cpu().float()
            err = float((got - want.float()).abs().max() / want.float().abs().max())
            assert err < 3e-2, f"step {step}: relative error {err}"
    finally:
        eng.close()
