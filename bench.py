#!/usr/bin/env python
"""Benchmark of the vTensor decode hot path (KV append + decode attention over
VMM-contiguous ranges) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" = one decode step of the workload through the hot path: for every
layer, append the step's K/V rows and run single-query attention for the whole
batch.  The metric is decode-attention HBM throughput: algorithmic bytes (every K
and V byte of the context read once, Q read, O written, the appended rows read
and written) divided by device time, summed over all GPUs; decode tokens/s
through the same path is printed beside it.

Workloads (shapes from the task's config list; data is seeded synthetic N(0,1)):
  7b   32 layers, batch 64, 32 q / 32 kv heads, contexts U[1024,4096]   (N = 1 default)
  70b  80 layers, batch 64, 64 q /  8 kv heads, contexts U[4096,16384], heads
       sharded over the N ranks tensor-parallel style                  (N > 1 default)
  op1 / gqa-long / gqa-fp8   single-layer op-level cases for tuning

N > 1 is launched by torchrun, one rank per GPU; ranks share nothing on the data
path (attention has no collective), NCCL only carries the barrier and the
max-over-ranks time.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

D = 128
LOOKAHEAD_ROWS = 64   # decode steps between asking for a chunk and needing it
WORKLOADS = {
    #  name       layers  B    H   KVH   lo     hi     fp8
    "7b":       (32,    64,  32, 32,  1024,  4096,  False),
    "70b":      (80,    64,  64, 8,   4096,  16384, False),
    # one rank's share of the 70b workload at TP = 2 / 4 / 8, runnable on a single GPU (tuning)
    "70b-tp2":  (80,    64,  32, 4,   4096,  16384, False),
    "70b-tp4":  (80,    64,  16, 2,   4096,  16384, False),
    "70b-tp8":  (80,    64,  8,  1,   4096,  16384, False),
    "op1":      (1,     8,   32, 32,  512,   2048,  False),
    "gqa-long": (1,     32,  32, 8,   16384, 32768, False),
    "gqa-fp8":  (1,     128, 32, 8,   2048,  8192,  True),
}
WORKLOAD_TEXT = {
    "7b": "llama2-7b-shape decode step: 32 layers x (KV append + decode attention), batch 64, 32/32 heads, ctx U[1k,4k]",
    "70b": "llama3-70b-shape decode step, heads sharded over ranks: 80 layers x (KV append + decode attention), batch 64, 64/8 heads, ctx U[4k,16k]",
    "70b-tp2": "one rank's share (32/4 heads) of the llama3-70b-shape decode step at TP=2, on one GPU",
    "70b-tp4": "one rank's share (16/2 heads) of the llama3-70b-shape decode step at TP=4, on one GPU",
    "70b-tp8": "one rank's share (8/1 heads) of the llama3-70b-shape decode step at TP=8, on one GPU",
    "op1": "decode attention op, batch 8, 32/32 heads, ctx U[512,2048]",
    "gqa-long": "llama3-8b-shape GQA decode attention op, batch 32, 32/8 heads, ctx U[16k,32k]",
    "gqa-fp8": "llama3-8b-shape GQA decode attention op, fp8 e4m3 KV, batch 128, 32/8 heads, ctx U[2k,8k]",
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--num-splits", type=int, default=0)
    return ap.parse_args()


def context_lens(seed, batch, lo, hi):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (batch,), generator=g).tolist()


def algorithmic_bytes(lens, layers, h, kvh, e):
    """Per step, for the given per-rank head counts."""
    b = len(lens)
    attn = sum(lens) * 2 * kvh * D * e + 2 * b * h * D * 2
    append = b * 2 * kvh * D * (2 + e)
    return layers * attn, layers * append


# ----------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi sampled every 50 ms in a child process; only samples whose
    timestamp falls inside [mark_begin, mark_end] (the timed region) are kept."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        self.t0 = self.t1 = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime
        sm, sm_all, mx, reasons = [], [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                clk = float(parts[1])
                mx = float(parts[2])
            except ValueError:
                continue
            sm_all.append(clk)
            if self.t0 is not None and self.t1 is not None and not (self.t0 - 0.05 <= ts <= self.t1 + 0.05):
                continue
            sm.append(clk)
            for name, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        use = sm if sm else sm_all
        return {"sm_mhz": statistics.median(use) if use else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "samples_total": len(sm_all)}


# ----------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------
class Job:
    """Builds the per-rank KV state through the allocator + append kernel and
    runs decode steps through the backend binding."""

    def __init__(self, args, name, rank, world):
        import torch
        from glake_b200 import vmmAllocator as A
        from glake_b200.backend import VTensorAttentionImpl, VTensorCacheEngine, VTensorMetadata, prepare_step
        self.torch, self.A = torch, A
        self.VTensorMetadata, self.prepare_step = VTensorMetadata, prepare_step
        layers, b, h, kvh, lo, hi, fp8 = WORKLOADS[name]
        assert h % world == 0 and kvh % world == 0, "heads must divide over the ranks"
        self.layers, self.b, self.h, self.kvh = layers, b, h // world, kvh // world
        self.fp8, self.e = fp8, (1 if fp8 else 2)
        self.dtype = "fp8_e4m3" if fp8 else "auto"
        self.dev = torch.device("cuda", torch.cuda.current_device())
        self.lens = context_lens(args.seed, b, lo, hi)       # same on every rank
        total_steps = args.steps * 2 + args.warmup * 2 + 8    # device-resident pass + e2e pass
        row = self.kvh * D * self.e
        chunk = A.granularitySize
        need = sum(((n + total_steps) * row + chunk - 1) // chunk for n in self.lens) * 2 * layers
        t0 = time.time()
        if not A.init_physical_handle(need + 2 * layers * (b + 4), self.dev.index):   # + one look-ahead chunk per slot
            raise RuntimeError("chunk pool creation failed")
        self.engine = VTensorCacheEngine(layers, self.kvh, D, b, hi + total_steps + 8, cache_dtype=self.dtype)
        self.impl = VTensorAttentionImpl(self.h, D, D ** -0.5, self.kvh, kv_cache_dtype=self.dtype)
        self.slots = list(range(b))
        self.scale_k = self.scale_v = None
        gen = torch.Generator(device=self.dev).manual_seed(args.seed * 1000 + rank)
        self.gen = gen
        # prefill: contexts minus nothing; the timed steps append one more row each
        from glake_b200 import ops
        meta = VTensorMetadata(self.slots, self.lens, self.kvh, D, num_prefills=b, kv_elem_size=self.e)
        prepare_step(meta, self.engine)
        tot = sum(self.lens)
        if fp8:
            self.scale_k = torch.full((layers, self.kvh), 5.0 / 448.0, device=self.dev)   # amax of N(0,1) ~ 5
            self.scale_v = torch.full((layers, self.kvh), 5.0 / 448.0, device=self.dev)
        for layer in range(layers):
            kcat = torch.randn(tot, self.kvh, D, device=self.dev, dtype=torch.bfloat16, generator=gen)
            vcat = torch.randn(tot, self.kvh, D, device=self.dev, dtype=torch.bfloat16, generator=gen)
            ops.reshape_and_cache(kcat, vcat, self.engine.k_cache_ptr[layer], self.engine.v_cache_ptr[layer],
                                  meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor, meta.cache_seq_lens,
                                  max(self.lens), self.kvh, D, self.dtype,
                                  self.scale_k[layer] if fp8 else None, self.scale_v[layer] if fp8 else None)
            del kcat, vcat
        # prefill-time headroom (the reference maps 100 tokens past the prompt,
        # vmm_allocator.cpp:322-337): every slot starts with LOOKAHEAD_ROWS rows of room
        for seg, n in zip(self.engine.vmm_kvcache_segment, self.lens):
            while seg.actual_size < (n + LOOKAHEAD_ROWS) * row:
                if not seg.expandMultiSegment(1):
                    raise RuntimeError("chunk pool exhausted while mapping prefill headroom")
        torch.cuda.synchronize()
        self.setup_s = time.time() - t0
        # per-step inputs: one set per layer, reused every step (values do not matter for timing)
        from glake_b200.backend import DecodeRunner
        sk = self.scale_k if fp8 else None
        sv = self.scale_v if fp8 else None
        self.resident = DecodeRunner(self.engine, self.impl, b, host_io=False, k_scale=sk, v_scale=sv)
        self.hostio = DecodeRunner(self.engine, self.impl, b, host_io=True, k_scale=sk, v_scale=sv)
        for t in (self.resident.q, self.resident.k, self.resident.v):
            t.copy_(torch.randn(t.shape, device=self.dev, dtype=torch.bfloat16, generator=gen))
        self.hostio.hq.copy_(self.resident.q)
        self.hostio.hk.copy_(self.resident.k)
        self.hostio.hv.copy_(self.resident.v)
        torch.cuda.synchronize()
        self.launches = 0
        self.num_splits = args.num_splits

    def _meta(self):
        """Advance every sequence by one token; the scheduler's part of the step."""
        row = self.kvh * D * self.e
        self.lens = [n + 1 for n in self.lens]
        extend = []
        for slot, seg in zip(self.slots, self.engine.vmm_kvcache_segment):
            # the scheduler's rule: ask for the next chunk LOOKAHEAD rows before it is needed, so
            # that the background mapping (2 x layers driver calls) is long done by then
            extend.append(slot if seg.used_size + LOOKAHEAD_ROWS * row > seg.actual_size and seg.ready() else -1)
        return self.VTensorMetadata(self.slots, self.lens, self.kvh, D, num_decode_tokens=self.b,
                                    extend_seq_list=extend, kv_elem_size=self.e)

    def step_resident(self):
        self.resident.step(self._meta())
        self.launches += self.resident.kernel_launches_per_step

    def step_e2e(self):
        """Host buffers in, host buffer out: pinned q/k/v for every layer are copied
        to the device inside the step and the attention outputs are copied back."""
        self.hostio.step(self._meta())
        self.launches += self.hostio.kernel_launches_per_step

    def streams(self):
        return [self.resident.stream, self.hostio.stream]

    def time_attention_only(self, iters=3):
        """CUDA-event time of the decode-attention call alone (one layer's launch),
        averaged over layers x iters, for the roofline.  A spin kernel is queued
        first so that every timed launch is already waiting in the stream when the
        GPU reaches it (otherwise host launch latency would be counted)."""
        torch = self.torch
        from glake_b200 import ops
        sl = torch.tensor(self.lens, dtype=torch.int32, device=self.dev)
        sm = torch.tensor(self.slots, dtype=torch.int64, device=self.dev)
        mx = max(self.lens)
        out = torch.empty(self.b, self.h, D, dtype=torch.bfloat16, device=self.dev)
        q = self.resident.q
        evs = []
        torch.cuda.synchronize()
        for it in range(iters + 1):
            torch.cuda._sleep(int(4e6 + 1e5 * self.layers))
            for layer in range(self.layers):
                kc, vc = self.engine.gpu_cache[layer]
                a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                ops.paged_attention_v1(out, q[layer].view(self.b, self.h, D), kc.vmm_ptr, vc.vmm_ptr, self.kvh,
                                       D ** -0.5, sl, 1, mx, None, self.dtype, 1.0, sm,
                                       k_scale=self.scale_k[layer] if self.fp8 else None,
                                       v_scale=self.scale_v[layer] if self.fp8 else None, num_splits=self.num_splits)
                z.record()
                if it > 0:
                    evs.append((a, z))
            torch.cuda.synchronize()
        ms = [a.elapsed_time(z) for a, z in evs]
        return sum(ms) / len(ms)


def timed(job, fn, stream, steps, warmup, world, sampler=None):
    """W warm-up steps, barrier + synchronize, K timed steps bracketed by CUDA events
    on the stream the graphs replay on, synchronize, max over ranks."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    lens0 = list(job.lens)
    job.launches = 0
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    if sampler:
        sampler.mark_begin()
    a.record(stream)
    for i in range(steps):
        fn()
        marks[i].record(stream)
    z.record(stream)
    torch.cuda.synchronize()
    if sampler:
        sampler.mark_end()
    per_step = [a.elapsed_time(marks[0])] + [marks[i - 1].elapsed_time(marks[i]) for i in range(1, steps)]
    job.step_ms = sorted(per_step)
    ms = a.elapsed_time(z)
    if world > 1:
        from glake_b200 import tp
        ms = tp.max_over_ranks(ms, device="cuda")
        dist.barrier()
    # bytes of the timed steps: contexts grow by one per step
    attn = app = 0
    for s in range(steps):
        l = [n + 1 + s for n in lens0]
        x, y = algorithmic_bytes(l, job.layers, job.h, job.kvh, job.e)
        attn += x
        app += y
    return ms, attn, app, job.launches


def run_ours(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torchrun (one rank per GPU)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    name = args.workload if args.workload != "auto" else ("7b" if world == 1 else "70b")
    layers, b, h, kvh, lo, hi, fp8 = WORKLOADS[name]
    job = Job(args, name, rank, world)

    sampler = ClockSampler(local) if rank == 0 else None
    ms, attn_b, app_b, launches = timed(job, job.step_resident, job.resident.stream, args.steps, args.warmup, world,
                                        sampler)
    clocks = sampler.stop() if sampler else None
    step_ms = list(job.step_ms)
    st = job.A.stats()
    alloc_stats = {"chunks_total": st["chunks_total"], "chunks_free": st["chunks_free"], "map_calls": st["map_calls"],
                   "set_access_calls": st["set_access_calls"], "map_seconds": round(st["map_ns"] * 1e-9, 3), "of_which_set_access_seconds": round(st["access_ns"] * 1e-9, 3),
                   "async_growths": st["async_completed"]}
    attn_ms = job.time_attention_only()
    lens_now = list(job.lens)
    e2e = None
    if not args.no_e2e:
        ms2, attn2, app2, _ = timed(job, job.step_e2e, job.hostio.stream, args.steps, args.warmup, world)
        per_layer_in = b * (job.h + 2 * job.kvh) * D * 2
        e2e = {"value": round((attn2 + app2) * world / (ms2 * 1e-3) / 1e9, 2), "unit": "GB/s",
               "ms_per_step": round(ms2 / args.steps, 4),
               "tokens_per_s": round(b * args.steps / (ms2 * 1e-3), 1),
               "h2d_bytes_per_step": world * (job.layers * per_layer_in + b * 24),
               "d2h_bytes_per_step": world * job.layers * b * job.h * D * 2}
    status = __import__("glake_b200.ops", fromlist=["attn_status"]).attn_status()
    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    # roofline of the dominant kernel (decode attention, one layer's launch)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    # Dominant kernel: the (fused append +) decode-attention kernel, one launch per layer.  Its
    # average duration over the TIMED REGION is the step time divided by the launches per step
    # when the step consists of nothing else (fused step: one kernel per layer); the same call
    # timed alone with CUDA events (cold start and drain included) is reported beside it.
    per_launch_attn, _ = algorithmic_bytes(lens_now, 1, job.h, job.kvh, job.e)
    fused = launches == args.steps * job.layers
    region_ms = ms / (args.steps * job.layers) if fused else attn_ms
    mean_bytes = attn_b / (args.steps * job.layers)          # contexts grow during the region
    achieved = (mean_bytes if fused else per_launch_attn) / (region_ms * 1e-3) / 1e9
    standalone = per_launch_attn / (attn_ms * 1e-3) / 1e9
    traffic = load_traffic(name, per_launch_attn)
    from glake_b200 import ops
    part, parts, variant = ops.attn_plan(b, job.h, job.kvh, max(lens_now), job.dtype, args.num_splits)
    line = {
        "metric": "decode_attention_hbm_throughput",
        "value": round((attn_b + app_b) * world / (ms * 1e-3) / 1e9, 2),
        "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 4),
        "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None,
        "dtype": "bf16 in/out, fp32 accumulate" + (", fp8 e4m3 KV" if fp8 else ""),
        "data": "synthetic",
        "config": {"workload": WORKLOAD_TEXT[name], "name": name, "layers": job.layers, "batch": b,
                   "q_heads_per_gpu": job.h, "kv_heads_per_gpu": job.kvh, "head_dim": D,
                   "context_mean_at_end": round(sum(lens_now) / b, 1), "seed": args.seed,
                   "l2": "inputs larger than L2: each layer streams its own KV ranges (>= 1 GiB per layer-op), no flush needed",
                   "split_k": {"part_tokens": part, "max_parts": parts, "variant": ["simt split-k", "tensor-core split-k", "tensor-core flat persistent"][variant]},
                   "kv_setup_seconds": round(job.setup_s, 1), "cuda_graph": True, "parallelism": f"tp{world} (heads sharded, no collective in the path)"},
        "tokens_per_s": round(b * args.steps / (ms * 1e-3), 1),
        "step_ms": {"min": round(step_ms[0], 3), "median": round(step_ms[len(step_ms) // 2], 3),
                    "max": round(step_ms[-1], 3)},
        "allocator": alloc_stats,
        "pct_of_nominal_8TBs": round(100 * achieved / 8000.0, 1),
        "gpu_launches": launches,
        "kernel_status": status,
        "e2e": e2e,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": traffic,
                     "kernel": "attn_flat_kernel: fused KV append + decode attention of one layer" if fused
                     else "decode attention call of one layer (attention kernel + split-K merge kernel)",
                     "ms_per_launch": round(region_ms, 4), "algorithmic_bytes_per_launch": int(mean_bytes if fused else per_launch_attn),
                     "how": "timed region / launches (the step is these launches only)" if fused else "CUDA events around the call",
                     "standalone": {"ms_per_launch": round(attn_ms, 4), "achieved": round(standalone, 1),
                                    "frac": round(standalone / peak, 4),
                                    "note": "same call timed alone behind a spin kernel: includes cold start and drain"},
                     "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback"},
        "clocks": clocks,
    }
    if world == 1:
        line["prefill"] = prefill_probe(job, peaks)
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline(name, args.seed, world)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def load_traffic(name, algorithmic_bytes_per_launch):
    """DRAM bytes per attention launch: the traffic / algorithmic ratio of the
    committed ncu capture for this kernel (profiles/traffic.json, taken on a small
    case; traffic grows in proportion to the tokens read) times this launch's
    algorithmic bytes.  null when no capture covers the workload."""
    try:
        table = json.load(open(os.path.join(ROOT, "profiles", "traffic.json")))
        t = table.get(name)
        if t is None and name == "70b" and int(os.environ.get("WORLD_SIZE", "1")) == 8:
            t = table.get("70b-tp8")      # the 8-rank share of the 70B workload is that capture's kernel
        return int(t["ratio"] * algorithmic_bytes_per_launch) if t else None
    except (OSError, ValueError, KeyError, TypeError):
        return None


# ----------------------------------------------------------------------------
# CPU baseline / reference arm: the reference's own CPU-backend kernels
# ----------------------------------------------------------------------------
def prefill_probe(job, peaks, prompts=2, tokens=4096, iters=10):
    """Extra, outside the timed region and the metric: the prefill kernel of the same head
    shape on a few prompts taken from the pool's free chunks (causal TFLOP/s, CUDA events)."""
    try:
        torch = job.torch
        from glake_b200 import ops
        from glake_b200.backend import VTensorCacheEngine, VTensorMetadata, prepare_step
        if job.e != 2:
            return {"skipped": "bf16 KV only"}
        row = job.kvh * D * 2
        need = prompts * 2 * ((tokens * row + (2 << 20) - 1) // (2 << 20)) + 8
        if job.A.stats()["chunks_free"] < need:
            return {"skipped": "not enough free chunks"}
        eng = VTensorCacheEngine(1, job.kvh, D, prompts, tokens + 8)
        try:
            meta = VTensorMetadata(list(range(prompts)), [tokens] * prompts, job.kvh, D, num_prefills=prompts)
            prepare_step(meta, eng)
            g = torch.Generator(device="cuda").manual_seed(1)
            k = torch.randn(prompts * tokens, job.kvh, D, device="cuda", generator=g).bfloat16()
            v = torch.randn(prompts * tokens, job.kvh, D, device="cuda", generator=g).bfloat16()
            q = torch.randn(prompts * tokens, job.h, D, device="cuda", generator=g).bfloat16()
            ops.reshape_and_cache(k, v, eng.k_cache_ptr[0], eng.v_cache_ptr[0], meta.slot_m, meta.slot_mapping,
                                  meta.seq_lens_tensor, meta.cache_seq_lens, tokens, job.kvh, D)
            out = torch.empty_like(q)
            ql = torch.full((prompts,), tokens, dtype=torch.int32, device="cuda")
            qs = torch.arange(prompts, dtype=torch.int32, device="cuda") * tokens
            kt, vt = eng.gpu_cache[0][0].vmm_ptr, eng.gpu_cache[0][1].vmm_ptr
            maps = eng.prefill_maps(0)

            def run():
                ops.prefill_attention(out, q, kt, vt, job.kvh, D ** -0.5, meta.slot_mapping, meta.seq_lens_tensor, ql, qs,
                                      tokens, maps=maps)
            for _ in range(3):
                run()
            torch.cuda.synchronize()
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                run()
            z.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(z) / iters
            tf = 2.0 * prompts * job.h * tokens * tokens * D / (ms * 1e-3) / 1e12
            peak = float(peaks.get("bf16_tflops", 1590.0))
            legacy = os.environ.get("VT_PREFILL_ENGINE", "").startswith("m")
            return {"tflops_causal": round(tf, 1), "ms": round(ms, 4), "prompts": prompts, "tokens": tokens,
                    "q_heads": job.h, "kv_heads": job.kvh,
                    "kernel": "mma.sync" if (maps is None or legacy) else "tcgen05.mma, S/P/O in tensor memory, TMA tensor copies",
                    "peak_tflops": peak, "frac_of_peak": round(tf / peak, 4),
                    "note": "causal half of the flops only; P is applied as hi + lo bf16 halves, so the tensor cores "
                            "execute about 1.5 x this; not part of the metric or the timed region"}
        finally:
            eng.close()
    except Exception as exc:      # never let the extra take the bench line down
        return {"error": f"{type(exc).__name__}: {exc}"[:200]}


def cpu_sample(name, seed, world, budget_s=12.0, max_seqs=None):
    """Times the reference CPU attention (oracle/_ref; the C port if that cannot
    load) on ONE layer of the workload, all host threads.  Returns
    (GB/s of algorithmic attention bytes, seconds per layer-op, description)."""
    import torch
    from oracle import oracle as O
    layers, b, h, kvh, lo, hi, fp8 = WORKLOADS[name]
    h, kvh = h // world, kvh // world
    lens = context_lens(seed, b, lo, hi)
    if max_seqs:
        lens = lens[:max_seqs]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(len(lens), h, D, generator=g).bfloat16()
    k = [torch.randn(n, kvh, D, generator=g).bfloat16() for n in lens]
    v = [torch.randn(n, kvh, D, generator=g).bfloat16() for n in lens]
    ref = O.load_ref()
    scale = D ** -0.5
    if ref is not None:
        cache = O.RefPagedCache(ref, k, v)      # untimed layout conversion through the reference's reshape_and_cache
        fn = lambda: cache.attend(q, scale)
        kind = "reference"
    else:
        r = O.fill_ranges(k, v)
        sl = torch.tensor(lens, dtype=torch.int32)
        ids = torch.arange(len(lens))
        fn = lambda: O.port_decode_attn(q, r, ids, sl, kvh, scale)
        kind = "port"
    fn()
    times = []
    t_all = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_all < budget_s and len(times) < 50):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    attn, _ = algorithmic_bytes(lens, 1, h, kvh, 2)
    return attn / sec / 1e9, sec, kind, cores, len(lens), len(times)


def cpu_baseline(name, seed, world):
    gbs, sec, kind, cores, nseq, runs = cpu_sample(name, seed, world)
    layers = WORKLOADS[name][0]
    return {"value": round(gbs, 2), "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"one layer of {layers} ({nseq} sequences, bf16 KV), decode attention only, median of {runs} runs "
                      f"of {sec * 1e3:.1f} ms; the reference CPU backend has no fp8 KV",
            "ms_per_step_extrapolated": round(sec * layers * 1e3, 1)}


def run_reference(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload if args.workload != "auto" else ("7b" if world == 1 else "70b")
    layers, b, h, kvh, lo, hi, fp8 = WORKLOADS[name]
    # each "step" is a bounded sample: one layer-op of the step's `layers`
    budget = max(3.0, min(60.0, 2.0 * (args.steps + args.warmup)))
    gbs, sec, kind, cores, nseq, runs = cpu_sample(name, args.seed, world, budget_s=budget)
    line = {
        "impl": "reference", "metric": "decode_attention_hbm_throughput", "value": round(gbs * 1.0, 2), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * layers * 1e3, 2),
        "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "bf16 in/out, fp32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD_TEXT[name], "name": name, "layers": layers, "batch": b,
                   "note": "reference CPU-backend paged_attention (csrc/cpu/attention.cpp) on the host cores; "
                           "each step is a bounded sample of one layer, ms_per_step = sample x layers"},
        "tokens_per_s": round(b / (sec * layers), 2),
        "cpu_baseline": {"value": round(gbs, 2), "unit": "GB/s", "cores": cores, "kind": kind,
                         "sample": f"one layer of {layers}, {nseq} sequences, median of {runs} runs"},
        "e2e": {"value": round(gbs, 2), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
