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

    python -m glake_b200.microbench prefill B H KVH L [tma(0|1)] [iters]

times causal prefill attention of B prompts of L tokens over their ranges (TFLOP/s
of the causal half, 2 * B * H * L^2 * 128 flops), with K/V tiles fetched by TMA
tensor copies (default) or by per-row bulk copies.

    torchrun --nproc-per-node N -m glake_b200.microbench allreduce [BYTES ...]

times the peer-memory all-reduce against torch.distributed (NCCL) for bf16 messages
of the given sizes (default 8 KiB .. 8 MiB): 100 calls captured in one CUDA graph,
device time per call, max over ranks.

The rope / norm modes time the element-wise steps either side of the attention: rotary embedding fused
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


def prefill_main():
    B,H,KVH,L = map(int, sys.argv[2:6])
    tma = not (len(sys.argv)>6 and sys.argv[6]=='0')
    iters = int(sys.argv[7]) if len(sys.argv)>7 else 10
    torch.cuda.set_device(0); torch.zeros(1,device='cuda')
    row = KVH*256
    assert A.init_physical_handle(B*2*((L*row+(2<<20)-1)//(2<<20))+16, 0)
    eng = VTensorCacheEngine(1, KVH, 128, B, L+8)
    meta = VTensorMetadata(list(range(B)), [L]*B, KVH, 128, num_prefills=B); prepare_step(meta, eng)
    k = torch.randn(B*L, KVH, 128, device='cuda', dtype=torch.bfloat16); v = torch.randn_like(k)
    ops.reshape_and_cache(k, v, eng.k_cache_ptr[0], eng.v_cache_ptr[0], meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor, meta.cache_seq_lens, L, KVH, 128)
    q = torch.randn(B*L, H, 128, device='cuda', dtype=torch.bfloat16); out = torch.empty_like(q)
    ql = torch.full((B,), L, dtype=torch.int32, device='cuda'); qs = torch.arange(B, dtype=torch.int32, device='cuda')*L
    kc, vc = eng.gpu_cache[0]
    maps = eng.prefill_maps(0) if tma else None
    def run(): ops.prefill_attention(out, q, kc.vmm_ptr, vc.vmm_ptr, KVH, 128**-0.5, meta.slot_mapping, meta.seq_lens_tensor, ql, qs, L, maps=maps)
    for _ in range(3): run()
    torch.cuda.synchronize()
    a,z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(); [run() for _ in range(iters)]; z.record(); torch.cuda.synchronize()
    ms = a.elapsed_time(z)/iters
    fl = 2*B*H*L*L*128
    print(f"prefill B{B} H{H} KVH{KVH} L{L} {'tensor copies' if maps is not None else 'row copies'}: {ms:.3f} ms  {fl/ms/1e9:.1f} TFLOP/s (causal flops)", flush=True)


def allreduce_main():
    import os
    import torch.distributed as dist
    from . import tp
    rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    world = dist.get_world_size()
    sizes = [int(a) for a in sys.argv[2:]] or [8 << 10, 64 << 10, 128 << 10, 256 << 10, 1 << 20, 2 << 20, 8 << 20]
    comm = tp.PeerAllReduce(max_size=max(max(sizes), 1 << 20))
    if os.environ.get("VT_AR_ONE_SHOT_BYTES"):
        comm.configure(one_shot_bytes=int(os.environ["VT_AR_ONE_SHOT_BYTES"]))
    if os.environ.get("VT_AR_PUSH_BYTES"):
        comm.configure(push_bytes=int(os.environ["VT_AR_PUSH_BYTES"]))
    calls = 100
    for nbytes in sizes:
        x = torch.randn(nbytes // 2, device='cuda').bfloat16(); y = torch.empty_like(x)
        res = {}
        impls = [("peer", lambda: comm.all_reduce(x, y))]
        if not os.environ.get("VT_AR_SKIP_NCCL"):
            impls.append(("nccl", lambda: dist.all_reduce(x)))
        if os.environ.get("VT_AR_SKIP_PEER"):
            impls = impls[1:]
        for name, fn in impls:
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for _ in range(3): fn()
                side.synchronize()
                g = torch.cuda.CUDAGraph()
                # thread-local capture mode: the process group's watchdog thread may touch events meanwhile
                with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
                    for _ in range(calls): fn()
            ts = []
            for _ in range(5):
                dist.barrier(); torch.cuda.synchronize()
                a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); g.replay(); z.record(); torch.cuda.synchronize()
                ts.append(a.elapsed_time(z) * 1e3 / calls)
            ts.sort()
            res[name] = tp.max_over_ranks(ts[len(ts)//2], device='cuda')
            del g                       # a live graph holding collective nodes stalls the teardown of the process group
            torch.cuda.synchronize()
        if rank == 0:
            nccl, peer = res.get("nccl", float("nan")), res.get("peer", float("nan"))
            print(f"all-reduce {world} ranks {nbytes >> 10:6d} KiB bf16: peer {peer:7.1f} us   nccl {nccl:7.1f} us   "
                  f"x{nccl / peer:.2f}", flush=True)
    st = comm.status()
    comm.close()
    if rank == 0:
        print("status", st, flush=True)
    dist.destroy_process_group()


def main():
    if sys.argv[1] == 'allreduce':
        return allreduce_main()
    if sys.argv[1] == 'prefill':
        return prefill_main()
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
