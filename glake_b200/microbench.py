"""Op-level microbenchmark of decode attention over vTensor ranges.

    python -m glake_b200.microbench B H KVH LO HI [fp8(0|1)] [num_splits] [iters]

Builds one layer of KV for B sequences with contexts uniform in [LO, HI] through
the allocator and the append kernel, then times ``paged_attention_v1`` with CUDA
events (median of ``iters``), reading a 256 MB buffer between iterations so that
L2 holds clean, unrelated lines.  Prints the plan the library picked and GB/s of
algorithmic bytes.  Environment knobs ``VT_ATTN_VARIANT`` / ``VT_ATTN_PART_TOKENS``
select a kernel variant / partition size.

    python -m glake_b200.microbench rope TOKENS H KVH [fp8(0|1)] [iters]
    python -m glake_b200.microbench norm TOKENS HIDDEN [iters]

time the element-wise steps either side of the attention: rotary embedding fused
with the KV append (a prefill of TOKENS rows into one slot, or with TOKENS <= 1024
a decode step of TOKENS entries), and rms_norm / fused_add_rms_norm.
"""
import sys
import torch
from . import ops, vmmAllocator as A
from .backend import VTensorCacheEngine, VTensorMetadata, prepare_step


def _time(run, iters):
    for _ in range(3): run()
    torch.cuda.synchronize()
    flush = torch.zeros(64<<20, dtype=torch.float32, device='cuda')
    ts=[]
    for _ in range(iters):
        flush.sum()  # read-only L2 flush: leaves clean lines behind
        a,z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); run(); z.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(z))
    ts.sort()
    return ts[len(ts)//2]


def rope_main():
    T,H,KVH = map(int, sys.argv[2:5])
    fp8 = len(sys.argv)>5 and sys.argv[5]=='1'
    iters = int(sys.argv[6]) if len(sys.argv)>6 else 20
    e = 1 if fp8 else 2
    decode = T <= 1024
    row = KVH*128*e
    torch.cuda.set_device(0); torch.zeros(1,device='cuda')
    n_slots = T if decode else 1
    assert A.init_physical_handle((2*n_slots if decode else 2*((T*row >> 21) + 2)) + 8, 0)
    dt = 'fp8_e4m3' if fp8 else 'auto'
    eng = VTensorCacheEngine(1, KVH, 128, n_slots, 8 if decode else T+8, cache_dtype=dt)
    if decode:
        meta = VTensorMetadata(list(range(T)), [1]*T, KVH, 128, num_decode_tokens=T, kv_elem_size=e)
    else:
        meta = VTensorMetadata([0], [T], KVH, 128, num_prefills=1, kv_elem_size=e)
    prepare_step(meta, eng)
    qkv = torch.randn(T, (H+2*KVH)*128, device='cuda', dtype=torch.bfloat16)
    q,k,v = qkv.split([H*128, KVH*128, KVH*128], dim=-1)
    pos = torch.randint(0, 4096, (T,), device='cuda')
    cs = torch.randn(4096, 128, device='cuda', dtype=torch.bfloat16)
    ks = torch.full((KVH,), 5/448, device='cuda'); vs = ks.clone()
    def run():
        ops.rotary_embedding_and_cache(pos, q, k, v, 128, cs, True, eng.k_cache_ptr[0], eng.v_cache_ptr[0], meta.slot_m,
                                       meta.slot_mapping, meta.seq_lens_tensor, meta.cache_seq_lens, 1 if decode else T,
                                       KVH, dt, ks if fp8 else None, vs if fp8 else None)
    ms = _time(run, iters)
    byt = T*(2*H*256 + 2*KVH*256 + 2*KVH*128*e + 2*256)
    print(f"rope+append T{T} H{H} KVH{KVH} fp8={fp8} {'decode' if decode else 'prefill'}: {ms*1e3:.1f} us  {byt/ms/1e6:.0f} GB/s  ({byt/2**20:.1f} MiB)", flush=True)


def norm_main():
    T,hidden = map(int, sys.argv[2:4])
    iters = int(sys.argv[4]) if len(sys.argv)>4 else 20
    torch.cuda.set_device(0)
    x = torch.randn(T, hidden, device='cuda', dtype=torch.bfloat16); r = torch.randn_like(x); o = torch.empty_like(x)
    w = torch.ones(hidden, device='cuda', dtype=torch.bfloat16)
    ms = _time(lambda: ops.rms_norm(o, x, w, 1e-5), iters)
    byt = T*hidden*4
    print(f"rms_norm T{T} hidden{hidden}: {ms*1e3:.1f} us  {byt/ms/1e6:.0f} GB/s  ({byt/2**20:.1f} MiB)", flush=True)
    ms = _time(lambda: ops.fused_add_rms_norm(x, r, w, 1e-5), iters)
    print(f"fused_add_rms_norm T{T} hidden{hidden}: {ms*1e3:.1f} us  {2*byt/ms/1e6:.0f} GB/s  ({2*byt/2**20:.1f} MiB)", flush=True)


def main():
    if sys.argv[1] == 'rope':
        return rope_main()
    if sys.argv[1] == 'norm':
        return norm_main()
    B,H,KVH,LO,HI = map(int, sys.argv[1:6])
    fp8 = len(sys.argv)>6 and sys.argv[6]=='1'
    splits = int(sys.argv[7]) if len(sys.argv)>7 else 0
    iters = int(sys.argv[8]) if len(sys.argv)>8 else 20
    e = 1 if fp8 else 2
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(LO, HI+1, (B,), generator=g).tolist()
    row = KVH*128*e
    need = sum((n*row + (2<<20)-1)//(2<<20) for n in lens)*2 + 16
    torch.cuda.set_device(0); torch.zeros(1,device='cuda')
    assert A.init_physical_handle(need, 0)
    dt = 'fp8_e4m3' if fp8 else 'auto'
    eng = VTensorCacheEngine(1, KVH, 128, B, HI+8, cache_dtype=dt)
    meta = VTensorMetadata(list(range(B)), lens, KVH, 128, num_prefills=B, kv_elem_size=e)
    prepare_step(meta, eng)
    tot = sum(lens)
    ks = torch.full((KVH,), 5/448, device='cuda'); vs = ks.clone()
    kcat = torch.randn(tot, KVH, 128, device='cuda', dtype=torch.bfloat16); vcat = torch.randn(tot, KVH, 128, device='cuda', dtype=torch.bfloat16)
    ops.reshape_and_cache(kcat, vcat, eng.k_cache_ptr[0], eng.v_cache_ptr[0], meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor, meta.cache_seq_lens, max(lens), KVH, 128, dt, ks if fp8 else None, vs if fp8 else None)
    del kcat, vcat
    q = torch.randn(B,H,128, device='cuda', dtype=torch.bfloat16); out = torch.empty_like(q)
    kc, vc = eng.gpu_cache[0]
    def run():
        ops.paged_attention_v1(out, q, kc.vmm_ptr, vc.vmm_ptr, KVH, 128**-0.5, meta.seq_lens_tensor, 1, max(lens), None, dt, 1.0, meta.slot_mapping, k_scale=ks if fp8 else None, v_scale=vs if fp8 else None, num_splits=splits)
    for _ in range(3): run()
    torch.cuda.synchronize()
    flush = torch.zeros(64<<20, dtype=torch.float32, device='cuda')
    ts=[]
    for _ in range(iters):
        flush.sum()  # read-only L2 flush: leaves clean lines behind
        a,z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); run(); z.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(z))
    ts.sort(); ms = ts[len(ts)//2]
    byt = tot*2*KVH*128*e + 2*B*H*128*2
    print(f"B{B} H{H} KVH{KVH} L[{LO},{HI}] fp8={fp8} splits={splits} plan={ops.attn_plan(B,H,KVH,max(lens),dt,splits)}: {ms*1e3:.1f} us  {byt/ms/1e6:.0f} GB/s  ({byt/2**20:.0f} MiB) min {byt/ts[0]/1e6:.0f}", flush=True)


if __name__ == "__main__":
    main()
