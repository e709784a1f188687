"""Helpers for the -m gpu parity tests: builds real vTensor ranges on the GPU
through the VMM allocator and the append kernel, all via the C ABI."""
import torch

from glake_b200 import ops, vmmAllocator as A
from glake_b200._lib import check, lib
from glake_b200.backend import VTensorCacheEngine, VTensorMetadata, prepare_step

POOL_CHUNKS = 4096  # 8 GiB of 2 MiB chunks, shared by the whole test session


def ensure_pool():
    if A._pool is None:
        assert torch.cuda.is_available()
        torch.cuda.init()
        torch.zeros(1, device="cuda")
        assert A.init_physical_handle(POOL_CHUNKS, torch.cuda.current_device())


class GpuKV:
    """One-layer (or n-layer) cache filled from per-sequence K/V lists:
    rows [0, L-1) by one prefill append, row L-1 by a decode append."""

    def __init__(self, k_list, v_list, kvh, fp8=False, n_layers=1, slots=None, max_slots=None,
                 k_scale=None, v_scale=None, layer=0):
        ensure_pool()
        self.kvh, self.fp8, self.layer = kvh, fp8, layer
        n = len(k_list)
        self.lens = [k.shape[0] for k in k_list]
        self.slots = list(range(n)) if slots is None else list(slots)
        max_slots = max_slots or (max(self.slots) + 1)
        max_tokens = max(self.lens) + 8
        self.engine = VTensorCacheEngine(n_layers, kvh, 128, max_slots, max_tokens,
                                         cache_dtype="fp8_e4m3" if fp8 else "auto")
        self.k_scale, self.v_scale = k_scale, v_scale
        dev = self.engine.device
        dt = "fp8_e4m3" if fp8 else "auto"
        e = 1 if fp8 else 2
        # prefill rows [0, L-1)
        pre = [x - 1 for x in self.lens]
        if max(pre) > 0:
            meta = VTensorMetadata(self.slots, pre, kvh, 128, num_prefills=n, kv_elem_size=e)
            prepare_step(meta, self.engine)
            kcat = torch.cat([k[:-1] for k in k_list]).to(dev)
            vcat = torch.cat([v[:-1] for v in v_list]).to(dev)
            ops.reshape_and_cache(kcat, vcat, self.engine.k_cache_ptr[layer], self.engine.v_cache_ptr[layer],
                                  meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor, meta.cache_seq_lens,
                                  max(pre), kvh, 128, dt, k_scale, v_scale)
        # decode append of the last row
        self.meta = VTensorMetadata(self.slots, self.lens, kvh, 128, num_decode_tokens=n, kv_elem_size=e)
        prepare_step(self.meta, self.engine)
        klast = torch.stack([k[-1] for k in k_list]).to(dev)
        vlast = torch.stack([v[-1] for v in v_list]).to(dev)
        ops.reshape_and_cache(klast, vlast, self.engine.k_cache_ptr[layer], self.engine.v_cache_ptr[layer],
                              self.meta.slot_m, self.meta.slot_mapping, self.meta.seq_lens_tensor,
                              self.meta.cache_seq_lens, 1, kvh, 128, dt, k_scale, v_scale)
        torch.cuda.synchronize()

    @property
    def k_table(self):
        return self.engine.gpu_cache[self.layer][0].vmm_ptr

    @property
    def v_table(self):
        return self.engine.gpu_cache[self.layer][1].vmm_ptr

    def read_rows(self, i, which="k"):
        """Cache bytes of sequence i copied back to the host as [L, kvh, 128]."""
        import ctypes
        seg = self.engine.vmm_kvcache_segment[self.slots[i]]
        base = seg.getKeyDevicePtr(self.layer) if which == "k" else seg.getValueDevicePtr(self.layer)
        nbytes = self.lens[i] * self.kvh * 128 * (1 if self.fp8 else 2)
        out = torch.empty(nbytes, dtype=torch.uint8)
        torch.cuda.synchronize()
        check(lib.vt_pool_read(A._pool, ctypes.c_void_p(out.data_ptr()), base, nbytes), "vt_pool_read")
        if self.fp8:
            return out.view(self.lens[i], self.kvh, 128)
        return out.view(torch.bfloat16).view(self.lens[i], self.kvh, 128)

    def attend(self, q, scale, num_splits=0, return_lse=False):
        dev = self.engine.device
        qd = q.to(dev)
        out = torch.empty_like(qd)
        if return_lse:
            o, lse = ops.fwd_kvcache(qd.unsqueeze(1), self.k_table, self.v_table, self.meta.max_seq_len, self.kvh,
                                     len(self.lens), self.meta.slot_mapping, None, None, self.meta.seq_lens_tensor,
                                     None, None, None, None, None, None, scale, True, -1, -1, None, 4,
                                     kv_cache_dtype="fp8_e4m3" if self.fp8 else "auto", k_scale=self.k_scale,
                                     v_scale=self.v_scale)
            torch.cuda.synchronize()
            return o[:, 0].cpu(), lse[..., 0].cpu()
        ops.paged_attention_v1(out, qd, self.k_table, self.v_table, self.kvh, scale, self.meta.seq_lens_tensor, 1,
                               self.meta.max_seq_len, None, "fp8_e4m3" if self.fp8 else "auto", 1.0,
                               self.meta.slot_mapping, k_scale=self.k_scale, v_scale=self.v_scale,
                               num_splits=num_splits)
        torch.cuda.synchronize()
        assert ops.attn_status() == 0
        return out.cpu()

    def close(self):
        self.engine.close()
