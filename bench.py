#!/usr/bin/env python
"""Benchmark of the vTensor decode hot path (KV append + decode attention over
VMM-contiguous ranges) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    python bench.py --op decode|prefill|rope|norm|allreduce ARGS...      (op-level timings, see op_main)

One "step" = one decode step of the workload through the hot path: for every
layer, append the step's K/V rows and run single-query attention for the whole
batch (one fused launch per layer for a bf16 cache); on N > 1 GPUs each layer is
followed by the two tensor-parallel all-reduces of the model around it (after
o_proj and after down_proj).  There are no weight GEMMs in the step.  The metric
is decode-attention HBM throughput: algorithmic bytes (every K and V byte of the
context read once, Q read, O written, the appended rows read and written) divided
by device time, summed over all GPUs.

Workloads (shapes from the task's config list; data is seeded synthetic N(0,1)):
  7b   32 layers, batch 64, 32 q / 32 kv heads, contexts U[1024,4096]   (N = 1 default)
  70b  80 layers, batch 64, 64 q /  8 kv heads, contexts U[4096,16384], heads
       sharded over the N ranks tensor-parallel style                  (N > 1 default)
  op1 / gqa-long / gqa-fp8   op-level cases of the other configurations; the N = 1
       line carries them as extra records

N > 1 is launched by torchrun, one rank per GPU.  Attention itself has no
collective; NCCL carries the model-level all-reduces of the step, the barrier and
the max-over-ranks time.
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
WORKLOADS = {
    #  name       layers  B    H   KVH   lo     hi     fp8    hidden
    "7b":       (32,    64,  32, 32,  1024,  4096,  False, 4096),
    "70b":      (80,    64,  64, 8,   4096,  16384, False, 8192),
    # one rank's share of the 70b workload at TP = 2 / 4 / 8, runnable on a single GPU
    "70b-tp2":  (80,    64,  32, 4,   4096,  16384, False, 8192),
    "70b-tp4":  (80,    64,  16, 2,   4096,  16384, False, 8192),
    "70b-tp8":  (80,    64,  8,  1,   4096,  16384, False, 8192),
    # op-level configurations.  op1 holds 4 independent copies of its ranges ("layers"), cycled
    # call by call, so that a call never finds its 160 MiB of KV in the 126 MB L2
    "op1":      (4,     8,   32, 32,  512,   2048,  False, 4096),
    "gqa-long": (1,     32,  32, 8,   16384, 32768, False, 4096),
    "gqa-fp8":  (1,     128, 32, 8,   2048,  8192,  True,  4096),
}
WORKLOAD_TEXT = {
    "7b": "llama2-7b-shape decode step: 32 layers x (KV append + decode attention), batch 64, 32/32 heads, ctx U[1k,4k]",
    "70b": "llama3-70b-shape decode step, heads sharded over the ranks: 80 layers x (KV append + decode attention, "
           "all-reduce [64,8192] bf16 after o_proj, all-reduce after down_proj), batch 64, 64/8 heads, ctx U[4k,16k]",
    "70b-tp2": "one rank's share (32/4 heads) of the llama3-70b-shape decode step at TP=2, on one GPU, no collectives",
    "70b-tp4": "one rank's share (16/2 heads) of the llama3-70b-shape decode step at TP=4, on one GPU, no collectives",
    "70b-tp8": "one rank's share (8/1 heads) of the llama3-70b-shape decode step at TP=8, on one GPU, no collectives",
    "op1": "decode attention op (append one token, then attend), batch 8, 32/32 heads, ctx U[512,2048]",
    "gqa-long": "llama3-8b-shape GQA decode attention op, batch 32, 32/8 heads, ctx U[16k,32k]",
    "gqa-fp8": "llama3-8b-shape GQA decode attention op, fp8 e4m3 KV with per-head scales = amax/448 computed at "
               "the prefill append, batch 128, 32/8 heads, ctx U[2k,8k]",
}
METRIC = "decode_attention_hbm_throughput"


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
    ap.add_argument("--no-extras", action="store_true", help="skip the extra records (other configs, shares, growth run)")
    ap.add_argument("--num-splits", type=int, default=0)
    ap.add_argument("--op", nargs="+", help="op-level timing instead of the workload step, see op_main")
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


def shared_config(name, world, seed):
    """The `config` object both arms print: what is computed, not how."""
    layers, b, h, kvh, lo, hi, fp8, hidden = WORKLOADS[name]
    return {"workload": WORKLOAD_TEXT[name], "name": name, "layers": layers, "batch": b, "q_heads": h, "kv_heads": kvh,
            "head_dim": D, "context": [lo, hi], "kv_dtype": "fp8_e4m3" if fp8 else "bf16", "seed": seed,
            "parallelism": f"tp{world}: heads sharded" + (", 2 all-reduces of [batch, hidden] bf16 per layer" if world > 1 else ""),
            "weights": "none: the step is the hot path only (no GEMMs)",
            "l2": "inputs larger than L2: every launch streams its own KV ranges (>= 300 MB per launch), no flush needed"}


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
class Collectives:
    """The two model-level all-reduces that follow a layer's attention under tensor
    parallelism (GLakeServe/vllm/model_executor/layers/linear.py:690-691): the o_proj
    output and the down_proj output, each [batch, hidden] bf16.  kind "nccl" uses
    torch.distributed in place; "peer" the library's peer-memory all-reduce.  Both are
    checked once against the expected sum and then run on zero-filled buffers
    (in-place sums of anything else would overflow bf16 within a few steps; the time
    of an all-reduce does not depend on the values)."""

    def __init__(self, kind, batch, hidden, device):
        import torch
        import torch.distributed as dist
        self.kind, self.dist = kind, dist
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.x = [torch.zeros(batch, hidden, dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.y = [torch.zeros_like(t) for t in self.x]
        self.comm = None
        self.buffers = "plain device tensors"
        self._pool = self._backend = None
        if kind == "nccl":
            self._try_registered_buffers(batch, hidden, device)
        if kind == "peer":
            from glake_b200 import tp
            self.comm = tp.PeerAllReduce(max_size=max(1 << 20, batch * hidden * 2))
        want = float(self.world * (self.world + 1) // 2)
        for i in range(2):
            self.x[i].fill_(self.rank + 1)
        self(0)
        torch.cuda.synchronize()
        got = self.y if kind == "peer" else self.x
        assert all(bool((t == want).all()) for t in got), f"{kind} all-reduce: wrong sum"
        for t in self.x + self.y:
            t.zero_()
        torch.cuda.synchronize()

    def _graph_time(self, tensors, calls=20, replays=3):
        """Device time (ms, max over ranks) of `calls` NCCL all-reduces replayed from a CUDA graph."""
        import torch
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for _ in range(2):
                self.dist.all_reduce(tensors[0])
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
                for i in range(calls):
                    self.dist.all_reduce(tensors[i % 2])
            best = float("inf")
            for _ in range(replays):
                self.dist.barrier()
                torch.cuda.synchronize()
                a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(side)
                g.replay()
                z.record(side)
                side.synchronize()
                best = min(best, a.elapsed_time(z))
            del g
        torch.cuda.synchronize()
        t = torch.tensor([best], dtype=torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def _try_registered_buffers(self, batch, hidden, device):
        """NCCL can run its all-reduce on buffers that come from its own allocator and are
        registered with the communicator as a symmetric window (torch: a MemPool over the
        backend's allocator + register_mem_pool(pool, symm=True)).  On 8 B200s that takes the
        1 MiB call from 41 to 29 us; on 2 it is slower.  Both kinds of buffer are timed here
        (20 graph-replayed calls, max over ranks) and the faster one is used; any failure of
        the registration path leaves the plain tensors in place.  Collective: every rank
        takes the same decisions because they rest on all-reduced numbers."""
        import torch
        ok = torch.ones(1, device=device)
        try:
            pg = self.dist.distributed_c10d._get_default_group()
            backend = pg._get_backend(torch.device("cuda", torch.cuda.current_device()))
            pool = torch.cuda.MemPool(backend.mem_allocator)
            with torch.cuda.use_mem_pool(pool):
                reg = [torch.zeros(batch, hidden, dtype=torch.bfloat16, device=device) for _ in range(2)]
            backend.register_mem_pool(pool, True)
        except Exception:
            ok.zero_()
            reg = pool = backend = None
        self.dist.all_reduce(ok, op=self.dist.ReduceOp.MIN)
        if float(ok.item()) == 0.0:
            if pool is not None:
                try:
                    backend.deregister_mem_pool(pool)
                except Exception:
                    pass
            return
        t_plain, t_reg = self._graph_time(self.x), self._graph_time(reg)
        if t_reg < t_plain:
            self.x, self._pool, self._backend = reg, pool, backend
            self.buffers = (f"NCCL-allocated, registered as a symmetric window "
                            f"({t_reg / 20 * 1e3:.1f} us per call vs {t_plain / 20 * 1e3:.1f} us on plain tensors)")
        else:
            self.buffers = (f"plain device tensors ({t_plain / 20 * 1e3:.1f} us per call vs "
                            f"{t_reg / 20 * 1e3:.1f} us on NCCL-registered symmetric buffers)")
            del reg
            try:
                backend.deregister_mem_pool(pool)
            except Exception:
                pass

    def __call__(self, layer):
        if self.kind == "peer":
            self.comm.all_reduce(self.x[0], self.y[0])
            self.comm.all_reduce(self.x[1], self.y[1])
        else:
            self.dist.all_reduce(self.x[0])
            self.dist.all_reduce(self.x[1])

    def status(self):
        return self.comm.status() if self.comm is not None else 0

    def close(self):
        if self.comm is not None:
            self.comm.close()
            self.comm = None
        if self._pool is not None:
            import torch
            torch.cuda.synchronize()
            self.x = []
            try:
                self._backend.deregister_mem_pool(self._pool)
            except Exception:
                pass
            self._pool = self._backend = None


class Job:
    """Builds the per-rank KV state through the chunk accounting, the allocator and the
    append kernel, and runs decode steps through the backend binding."""

    def __init__(self, name, seed, rank, world, step_budget, num_splits=0):
        import torch
        from glake_b200 import chunk_manager as cm
        from glake_b200 import ops, vmmAllocator as A
        from glake_b200.backend import VTensorAttentionImpl, VTensorCacheEngine, VTensorMetadata, prepare_step
        self.torch, self.A, self.cm = torch, A, cm
        self.VTensorMetadata = VTensorMetadata
        layers, b, h, kvh, lo, hi, fp8, hidden = WORKLOADS[name]
        assert h % world == 0 and kvh % world == 0, "heads must divide over the ranks"
        self.name, self.layers, self.b, self.h, self.kvh, self.hidden = name, layers, b, h // world, kvh // world, hidden
        self.fp8, self.e = fp8, (1 if fp8 else 2)
        self.dtype = "fp8_e4m3" if fp8 else "auto"
        self.dev = torch.device("cuda", torch.cuda.current_device())
        self.lens = context_lens(seed, b, lo, hi)       # same on every rank
        self.num_splits = num_splits
        row = self.row = self.kvh * D * self.e
        chunk = A.granularitySize
        t0 = time.time()
        # the scheduler's side: logical chunk accounting per sequence, prompt + headroom at admission
        self.seqs = [cm.SequenceChunks(row) for _ in range(b)]
        for s, n in zip(self.seqs, self.lens):
            s.append_tokens(n)
        per_layer = sum(2 * (((n + step_budget + cm.PREFILL_HEADROOM_TOKENS + 8) * row + chunk - 1) // chunk)
                        for n in self.lens)
        self.manager = cm.ChunkSpaceManager(b, per_layer, watermark=0.0)
        if not A.init_physical_handle(per_layer * layers + 256, self.dev.index):     # + room for the prefill probe
            raise RuntimeError("chunk pool creation failed")
        self.engine = VTensorCacheEngine(layers, self.kvh, D, b, hi + step_budget + cm.PREFILL_HEADROOM_TOKENS + 16,
                                         cache_dtype=self.dtype)
        self.impl = VTensorAttentionImpl(self.h, D, D ** -0.5, self.kvh, kv_cache_dtype=self.dtype)
        for s in self.seqs:
            assert self.manager.allocate(s)
        self.slots = [s.slot for s in self.seqs]
        gen = self.gen = torch.Generator(device=self.dev).manual_seed(seed * 1000 + rank)
        meta = VTensorMetadata(self.slots, self.lens, self.kvh, D, num_prefills=b, kv_elem_size=self.e)
        prepare_step(meta, self.engine)
        tot = sum(self.lens)
        self.scale_k = self.scale_v = None
        if fp8:
            self.scale_k = torch.empty(layers, self.kvh, device=self.dev)
            self.scale_v = torch.empty(layers, self.kvh, device=self.dev)
        for layer in range(layers):
            kcat = torch.randn(tot, self.kvh, D, device=self.dev, dtype=torch.bfloat16, generator=gen)
            vcat = torch.randn(tot, self.kvh, D, device=self.dev, dtype=torch.bfloat16, generator=gen)
            if fp8:     # per-(layer, kv head) scale = amax / 448 over the prompt rows, frozen from here on
                self.scale_k[layer] = ops.kv_scales(kcat, self.kvh, D)
                self.scale_v[layer] = ops.kv_scales(vcat, self.kvh, D)
            ops.reshape_and_cache(kcat, vcat, self.engine.k_cache_ptr[layer], self.engine.v_cache_ptr[layer],
                                  meta.slot_m, meta.slot_mapping, meta.seq_lens_tensor, meta.cache_seq_lens,
                                  max(self.lens), self.kvh, D, self.dtype,
                                  self.scale_k[layer] if fp8 else None, self.scale_v[layer] if fp8 else None)
            del kcat, vcat
        for s in self.seqs:      # prompt + headroom mapped at admission; decode growth is asked for that far ahead
            cm.apply_allocate(s, self.engine.vmm_kvcache_segment[s.slot])
        torch.cuda.synchronize()
        self.setup_s = time.time() - t0
        self.runners = {}
        self.launches = 0
        self.steps_done = 0
        self.step_budget = step_budget

    def runner(self, key, host_io=False, post_layer=None, post_launches=0, overlap=True):
        """A DecodeRunner (CUDA-graph replay of the step) with this job's inputs loaded."""
        from glake_b200.backend import DecodeRunner
        torch = self.torch
        if key not in self.runners:
            r = DecodeRunner(self.engine, self.impl, self.b, host_io=host_io, k_scale=self.scale_k, v_scale=self.scale_v,
                             overlap=overlap, post_layer=post_layer, launches_per_post_layer=post_launches)
            g = torch.Generator(device=self.dev).manual_seed(4321)
            for t in (r.q, r.k, r.v):
                t.copy_(torch.randn(t.shape, device=self.dev, dtype=torch.bfloat16, generator=g))
            if host_io:
                r.hq.copy_(r.q), r.hk.copy_(r.k), r.hv.copy_(r.v)
            torch.cuda.synchronize()
            self.runners[key] = r
        return self.runners[key]

    def _meta(self):
        """Advance every sequence by one token: the scheduler's part of the step.  The chunk
        manager lists the slots whose logical reservation just outgrew what they hold; the
        model step hands them to the allocator's background worker."""
        assert self.steps_done < self.step_budget, "step budget of the pool exhausted"
        self.steps_done += 1
        self.lens = [n + 1 for n in self.lens]
        grow = []
        for s in self.seqs:
            s.append_tokens(1)
            assert self.manager.append_slots(s, grow)
        extend = [slot if slot in grow else -1 for slot in self.slots]
        return self.VTensorMetadata(self.slots, self.lens, self.kvh, D, num_decode_tokens=self.b,
                                    extend_seq_list=extend, kv_elem_size=self.e)

    def step(self, runner):
        runner.step(self._meta())
        self.launches += runner.kernel_launches_per_step

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
        q = next(iter(self.runners.values())).q
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
        assert ops.attn_status() == 0, "an attention kernel gave up on a bounded wait"
        ms = [a.elapsed_time(z) for a, z in evs]
        return sum(ms) / len(ms)

    def kernel_status(self):
        """Non-zero when any kernel of the timed runners gave up on a bounded wait (results invalid)."""
        return max([r.status() for r in self.runners.values()] + [0])

    def close(self):
        torch = self.torch
        torch.cuda.synchronize()
        for r in self.runners.values():
            r.graphs.clear()
        self.runners.clear()
        self.engine.close()
        self.A.shutdown()


def timed(job, runner, steps, warmup, world, sampler=None, barrier=True):
    """W warm-up steps, barrier + synchronize, K timed steps bracketed by CUDA events
    on the stream the graphs replay on, synchronize, max over ranks.  Returns
    (ms of the K steps, attention bytes, append bytes, launches, sorted per-step ms)."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        job.step(runner)
    torch.cuda.synchronize()
    if world > 1 and barrier:
        dist.barrier()
    torch.cuda.synchronize()
    lens0 = list(job.lens)
    job.launches = 0
    stream = runner.stream
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    if sampler:
        sampler.mark_begin()
    a.record(stream)
    for i in range(steps):
        job.step(runner)
        marks[i].record(stream)
    z.record(stream)
    torch.cuda.synchronize()
    if sampler:
        sampler.mark_end()
    per_step = [a.elapsed_time(marks[0])] + [marks[i - 1].elapsed_time(marks[i]) for i in range(1, steps)]
    ms = a.elapsed_time(z)
    if world > 1 and barrier:
        from glake_b200 import tp
        ms = tp.max_over_ranks(ms, device="cuda")
        dist.barrier()
    attn = app = 0
    for s in range(steps):          # contexts grow by one per step
        x, y = algorithmic_bytes([n + 1 + s for n in lens0], job.layers, job.h, job.kvh, job.e)
        attn += x
        app += y
    return ms, attn, app, job.launches, per_step


def rate(attn_b, app_b, ms, world=1):
    return round((attn_b + app_b) * world / (ms * 1e-3) / 1e9, 2)


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        return {}


def op_record(name, seed, calls, peak, with_cpu=False):
    """Extra record for one of the op-level configurations: the fused call (append one token,
    then attend) replayed >= `calls` times from CUDA graphs of 20 back-to-back calls, CUDA
    events around the replays, no overlap between consecutive calls.  Every call appends the
    same row at the same position (idempotent), so the contexts stay as generated."""
    try:
        import torch
        from glake_b200 import ops
        from glake_b200.backend import prepare_step
        job = Job(name, seed, 0, 1, 8)
        try:
            meta = prepare_step(job._meta(), job.engine)
            b, h, kvh = job.b, job.h, job.kvh
            g = torch.Generator(device=job.dev).manual_seed(4321)
            q = torch.randn(job.layers, b, h, D, device=job.dev, dtype=torch.bfloat16, generator=g)
            k = torch.randn(job.layers, b, kvh, D, device=job.dev, dtype=torch.bfloat16, generator=g)
            v = torch.randn(job.layers, b, kvh, D, device=job.dev, dtype=torch.bfloat16, generator=g)
            out = torch.empty_like(q)
            ws = ops.new_workspace(job.dev, b, h, D, meta.max_seq_len)

            def one_pass():
                for layer in range(job.layers):
                    kc, vc = job.engine.gpu_cache[layer]
                    ops.decode_step(out[layer], q[layer], k[layer], v[layer], kc.vmm_ptr, vc.vmm_ptr, meta.slot_m,
                                    meta.slot_mapping, meta.seq_lens_tensor, meta.max_seq_len, kvh, D ** -0.5, job.dtype,
                                    job.scale_k[layer] if job.fp8 else None, job.scale_v[layer] if job.fp8 else None,
                                    workspace=ws, maps=job.engine.decode_maps(layer, h), clean_scratch=True)
            per_graph = max(1, 20 // job.layers) * job.layers
            side = torch.cuda.Stream(device=job.dev)
            with torch.cuda.stream(side):
                one_pass()
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(per_graph // job.layers):
                        one_pass()
                for _ in range(3):
                    graph.replay()
                side.synchronize()
                replays = -(-calls // per_graph)
                sampler = ClockSampler(job.dev.index)
                sampler.mark_begin()
                a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(side)
                for _ in range(replays):
                    graph.replay()
                z.record(side)
                side.synchronize()
                sampler.mark_end()
                clocks = sampler.stop()
            n_calls = replays * per_graph
            ms = a.elapsed_time(z) / n_calls
            status = ops.workspace_status(ws)
            del graph
            attn_b, _ = algorithmic_bytes(job.lens, 1, h, kvh, job.e)
            _, parts, variant = ops.attn_plan(b, h, kvh, max(job.lens), job.dtype)
            gbs = attn_b / (ms * 1e-3) / 1e9
            rec = {"workload": WORKLOAD_TEXT[name], "calls": n_calls, "ms_per_call": round(ms, 5),
                   "algorithmic_bytes_per_call": int(attn_b), "GB/s": round(gbs, 1),
                   "frac": round(gbs / peak, 4), "pct_of_nominal_8TBs": round(gbs / 80.0, 1),
                   "kernel": ("tcgen05.mma kind::f8f6f4 flat persistent (TMA tensor copies, S/O in tensor memory)"
                              if variant == 2 and job.engine.decode_maps(0, h) is not None else
                              ["simt split-k", "tensor-core split-k", "mma.sync flat persistent"][variant])
                             + (", fused append" if variant == 2 and ops.step_is_fused(job.dtype) else ", separate append kernel"),
                   "gpu_launches": n_calls, "kernel_status": status,
                   "how": f"CUDA graphs of {per_graph} calls back to back, CUDA events around {replays} replays",
                   "clocks": {"sm_mhz": clocks.get("sm_mhz"), "reasons": clocks.get("reasons")}}
            if job.layers > 1:
                rec["l2"] = f"{job.layers} independent copies of the ranges cycled, so no call finds its KV in L2"
            if job.fp8:
                rec["kv_scales"] = "vt_kv_scales (amax/448 per kv head) at the prefill append, frozen"
        finally:
            job.close()
        if with_cpu:
            gb, sec, kind, cores, nseq, runs = cpu_sample(name, seed, budget_s=3.0)
            rec["reference_cpu"] = {"ms_per_call": round(sec * 1e3, 3), "GB/s": round(gb, 1), "cores": cores, "kind": kind}
        return rec
    except Exception as exc:      # an extra must not take the bench line down
        return {"error": f"{type(exc).__name__}: {exc}"[:300]}


def share_record(name, seed, steps, warmup, peak):
    """Extra record: one rank's share of the tensor-parallel workload on this GPU alone
    (no collectives): the same-workload anchor of the multi-GPU curve."""
    try:
        job = Job(name, seed, 0, 1, steps + warmup + 8)
        try:
            r = job.runner("share")
            sampler = ClockSampler(job.dev.index)
            ms, attn_b, app_b, launches, _ = timed(job, r, steps, warmup, 1, sampler)
            clocks = sampler.stop()
            alone_ms = job.time_attention_only()
            per_launch, _ = algorithmic_bytes(job.lens, 1, job.h, job.kvh, job.e)
            alone = per_launch / (alone_ms * 1e-3) / 1e9
            return {"workload": WORKLOAD_TEXT[name], "ms_per_step": round(ms / steps, 4), "GB/s": rate(attn_b, app_b, ms),
                    "frac": round(rate(attn_b, app_b, ms) / peak, 4),
                    "standalone": {"ms_per_launch": round(alone_ms, 4), "GB/s": round(alone, 1), "frac": round(alone / peak, 4)},
                    "gpu_launches": launches, "kernel_status": job.kernel_status(), "kv_setup_seconds": round(job.setup_s, 1),
                    "clocks": {"sm_mhz": clocks.get("sm_mhz"), "reasons": clocks.get("reasons")}}
        finally:
            job.close()
    except Exception as exc:
        return {"error": f"{type(exc).__name__}: {exc}"[:300]}


def growth_record(job, runner, steps):
    """Extra record: `steps` more decode steps with the allocator growing ranges under load
    (every sequence crosses chunk boundaries; growth is asked for a headroom ahead by the
    chunk manager and mapped by the background worker)."""
    st0 = job.A.stats()
    n0 = len(runner.prepare_seconds)
    ms, attn_b, app_b, _, per_step = timed(job, runner, steps, 0, 1)
    st1 = job.A.stats()
    host = runner.prepare_seconds[n0:]
    srt = sorted(per_step)
    return {"steps": steps, "GB/s": rate(attn_b, app_b, ms), "ms_per_step": round(ms / steps, 4),
            "step_ms": {"p50": round(srt[len(srt) // 2], 3), "p99": round(srt[min(len(srt) - 1, int(len(srt) * 0.99))], 3),
                        "max": round(srt[-1], 3)},
            "growths_completed": st1["async_completed"] - st0["async_completed"],
            "chunks_mapped": st1["map_calls"] - st0["map_calls"],
            "driver_seconds_in_growth": round((st1["map_ns"] - st0["map_ns"]) * 1e-9, 3),
            "steps_whose_host_bookkeeping_waited_over_1ms": sum(1 for t in host if t > 1e-3),
            "host_bookkeeping_ms": {"p50": round(sorted(host)[len(host) // 2] * 1e3, 3), "max": round(max(host) * 1e3, 3)},
            "lookahead": f"chunk manager headroom of {job.cm.PREFILL_HEADROOM_TOKENS} rows"}


def growth_record_large_chunks(name, seed, steps, chunk_mib):
    """Extra record: the growth run again on a pool of larger physical chunks.  The driver's cost
    of a growth is per chunk whatever its size (cuMemSetAccess 0.15 ms per handle), so 8 MiB
    chunks make a sequence grow a quarter as often for the same price per growth; the price is
    up to 8 MiB of slack per range.  Fresh pool and KV state; same workload, seeds and step count."""
    try:
        from glake_b200 import vmmAllocator as A
        A.set_chunk_bytes(chunk_mib << 20)
        try:
            job = Job(name, seed, 0, 1, steps + 24)
            try:
                r = job.runner("growth")
                timed(job, r, 3, 3, 1)
                rec = growth_record(job, r, steps)
                rec["chunk_mib"] = chunk_mib
                rec["kv_setup_seconds"] = round(job.setup_s, 1)
                rec["kernel_status"] = job.kernel_status()
                return rec
            finally:
                job.close()
        finally:
            A.shutdown()              # no-op after job.close(); releases the pool if the job never came up
            A.set_chunk_bytes(2 << 20)
    except Exception as exc:      # an extra must not take the bench line down
        return {"error": f"{type(exc).__name__}: {exc}"[:300]}


def run_ours(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torchrun (one rank per GPU)")
    torch.cuda.set_device(local)
    host_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        host_group = dist.new_group(backend="gloo")     # host-side barrier for the single-rank pass
    name = args.workload if args.workload != "auto" else ("7b" if world == 1 else "70b")
    layers, b, h, kvh, lo, hi, fp8, hidden = WORKLOADS[name]
    extras = not args.no_extras
    K, W = args.steps, args.warmup
    growth_steps = 256 if (world == 1 and extras and name == "7b") else 0
    passes = 2 + (3 if world > 1 else 0)
    job = Job(name, args.seed, rank, world, passes * (K + W) + growth_steps + 16, args.num_splits)
    peaks = load_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))

    nccl = peer = None
    if world > 1:
        nccl = Collectives("nccl", b, hidden, job.dev)
        head = job.runner("nccl", post_layer=nccl, post_launches=2)
    else:
        head = job.runner("resident")
    sampler = ClockSampler(local) if rank == 0 else None
    ms, attn_b, app_b, launches, per_step = timed(job, head, K, W, world, sampler)
    clocks = sampler.stop() if sampler else None
    step_ms = sorted(per_step)
    st = job.A.stats()
    alloc_stats = {"chunks_total": st["chunks_total"], "chunks_free": st["chunks_free"], "map_calls": st["map_calls"],
                   "set_access_calls": st["set_access_calls"], "map_seconds": round(st["map_ns"] * 1e-9, 3),
                   "of_which_set_access_seconds": round(st["access_ns"] * 1e-9, 3), "async_growths": st["async_completed"]}
    e2e = None
    if not args.no_e2e:
        hostio = job.runner("hostio", host_io=True, post_layer=nccl, post_launches=2 if nccl else 0)
        ms2, attn2, app2, _, _ = timed(job, hostio, K, W, world)
        per_layer_in = b * (job.h + 2 * job.kvh) * D * 2
        e2e = {"value": rate(attn2, app2, ms2, world), "unit": "GB/s", "ms_per_step": round(ms2 / K, 4),
               "path_tokens_per_s": round(b * K / (ms2 * 1e-3), 1),
               "h2d_bytes_per_step": world * (job.layers * per_layer_in + b * 24),
               "d2h_bytes_per_step": world * job.layers * b * job.h * D * 2}
    multi = None
    if world > 1:
        # the same step without the collectives, and with the peer-memory all-reduce in their place
        plain = job.runner("attention_only")
        ms_a, attn_a, app_a, _, _ = timed(job, plain, K, W, world)
        multi = {"attention_only": {"value": rate(attn_a, app_a, ms_a, world), "unit": "GB/s",
                                    "ms_per_step": round(ms_a / K, 4), "note": "same step without the all-reduces"}}
        try:
            peer = Collectives("peer", b, hidden, job.dev)
            pr = job.runner("peer", post_layer=peer, post_launches=2)
            ms_p, attn_p, app_p, _, _ = timed(job, pr, K, W, world)
            multi["peer_all_reduce"] = {"value": rate(attn_p, app_p, ms_p, world), "unit": "GB/s",
                                        "ms_per_step": round(ms_p / K, 4), "status": peer.status(),
                                        "note": "same step with vt_all_reduce (one launch over peer memory, plain peer "
                                                "loads and stores) in place of NCCL"}
        except Exception as exc:
            multi["peer_all_reduce"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        multi["all_reduce_ms_per_step"] = {"nccl": round((ms - ms_a) / K, 4),
                                           "peer": round((ms_p - ms_a) / K, 4) if "value" in multi["peer_all_reduce"] else None,
                                           "calls_per_step": 2 * job.layers, "bytes_per_call": b * hidden * 2}
        # rank 0's share with the other ranks idle
        dist.barrier(group=host_group)
        if rank == 0:
            ms_s, attn_s, app_s, _, _ = timed(job, plain, K, W, world, barrier=False)
            multi["single_gpu_share"] = {"value": rate(attn_s, app_s, ms_s), "unit": "GB/s", "ms_per_step": round(ms_s / K, 4),
                                         "note": "rank 0's share of the step (no all-reduces) with the other GPUs idle"}
        dist.barrier(group=host_group)
    attn_ms = job.time_attention_only()
    lens_now = list(job.lens)
    growth = None
    if growth_steps:
        try:
            growth = growth_record(job, head, growth_steps)
        except Exception as exc:
            growth = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    status = job.kernel_status()
    if nccl is not None:
        torch.cuda.synchronize()
    if rank != 0:
        if peer is not None:
            peer.close()
        job.close()
        if nccl is not None:
            nccl.close()
        dist.barrier()
        dist.destroy_process_group()
        return
    # roofline of the dominant kernel: the (fused append +) decode-attention kernel, one launch per layer
    from glake_b200 import ops
    per_launch_attn, _ = algorithmic_bytes(lens_now, 1, job.h, job.kvh, job.e)
    only_attention = world == 1 and launches == K * job.layers     # the step is these launches and nothing else
    standalone = per_launch_attn / (attn_ms * 1e-3) / 1e9
    if only_attention:
        region_ms = ms / (K * job.layers)
        bytes_per_launch = attn_b / (K * job.layers)               # contexts grow during the region
        how = "timed region / launches (the step is these launches only, consecutive layers overlap)"
    else:
        region_ms, bytes_per_launch = attn_ms, per_launch_attn
        how = "CUDA events around each launch, queued behind a spin kernel (the step has other kernels between the launches)"
    achieved = bytes_per_launch / (region_ms * 1e-3) / 1e9
    part, parts, variant = ops.attn_plan(b, job.h, job.kvh, max(lens_now), job.dtype, args.num_splits)
    fused = ops.step_is_fused(job.dtype) and variant == 2
    line = {
        "metric": METRIC,
        "value": rate(attn_b, app_b, ms, world),
        "unit": "GB/s",
        "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": round(ms / K, 4),
        "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None,
        "dtype": "bf16 in/out, fp32 accumulate" + (", fp8 e4m3 KV" if fp8 else ""),
        "data": "synthetic",
        "config": shared_config(name, world, args.seed),
        "details": {"q_heads_per_gpu": job.h, "kv_heads_per_gpu": job.kvh, "context_mean_at_end": round(sum(lens_now) / b, 1),
                    "split_k": {"part_tokens": part, "max_parts": parts,
                                "variant": ["simt split-k", "tensor-core split-k", "tensor-core flat persistent"][variant]},
                    "kv_setup_seconds": round(job.setup_s, 1), "cuda_graph": True,
                    "collectives_in_step": "2 x NCCL all-reduce of [batch, hidden] bf16 per layer, inside the CUDA graph"
                    if world > 1 else "none (one GPU)",
                    "nccl_buffers": nccl.buffers if nccl is not None else None},
        "path_tokens_per_s": round(b * K / (ms * 1e-3), 1),
        "path_tokens_per_s_note": "decode steps of the hot path only: no weight GEMMs are executed",
        "step_ms": {"min": round(step_ms[0], 3), "median": round(step_ms[len(step_ms) // 2], 3), "max": round(step_ms[-1], 3)},
        "allocator": alloc_stats,
        "pct_of_nominal_8TBs": round(100 * achieved / 8000.0, 1),
        "gpu_launches": launches,
        "kernel_status": status,
        "e2e": e2e,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": load_traffic(name, bytes_per_launch),
                     "kernel": "attn_flat_kernel: " + ("fused KV append + " if fused else "") + "decode attention of one layer",
                     "ms_per_launch": round(region_ms, 4), "algorithmic_bytes_per_launch": int(bytes_per_launch), "how": how,
                     "standalone": {"ms_per_launch": round(attn_ms, 4), "achieved": round(standalone, 1),
                                    "frac": round(standalone / peak, 4),
                                    "note": "the attention call timed alone behind a spin kernel: includes ramp-up and drain"},
                     "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback"},
        "clocks": clocks,
    }
    if multi:
        line["multi_gpu"] = multi
    if growth:
        line["allocator_growth_under_load"] = growth
    if world == 1:
        line["prefill"] = prefill_probe(job, peaks)
    if peer is not None:
        peer.close()
    job.close()
    if nccl is not None:
        nccl.close()
    if world == 1 and extras and name == "7b":
        line["configs"] = {"op1": op_record("op1", args.seed, 100, peak, with_cpu=not args.no_cpu_baseline),
                           "gqa-long": op_record("gqa-long", args.seed, 100, peak),
                           "gqa-fp8": op_record("gqa-fp8", args.seed, 100, peak)}
        line["70b_tp8_share"] = share_record("70b-tp8", args.seed, K, W, peak)
        line["allocator_growth_under_load_8mib_chunks"] = growth_record_large_chunks(name, args.seed, 256, 8)
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline(name, args.seed)
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
                    "note": "causal half of the flops only; not part of the metric or the timed region"}
        finally:
            eng.close()
    except Exception as exc:      # never let the extra take the bench line down
        return {"error": f"{type(exc).__name__}: {exc}"[:200]}


# ----------------------------------------------------------------------------
# CPU baseline / reference arm: the reference's own CPU-backend kernels
# ----------------------------------------------------------------------------
class CpuLayer:
    """One layer of the workload (ALL heads: the CPU does the whole problem whatever the
    GPU count) in the reference CPU backend's paged layout, ready to be timed."""

    def __init__(self, name, seed, max_seqs=None):
        import torch
        from oracle import oracle as O
        layers, b, h, kvh, lo, hi, fp8, hidden = WORKLOADS[name]
        lens = context_lens(seed, b, lo, hi)
        if max_seqs:
            lens = lens[:max_seqs]
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(len(lens), h, D, generator=g).bfloat16()
        k = [torch.randn(n, kvh, D, generator=g).bfloat16() for n in lens]
        v = [torch.randn(n, kvh, D, generator=g).bfloat16() for n in lens]
        ref = O.load_ref()
        scale = D ** -0.5
        if ref is not None:
            cache = O.RefPagedCache(ref, k, v)      # untimed layout conversion through the reference's reshape_and_cache
            self.fn = lambda: cache.attend(q, scale)
            self.kind = "reference"
        else:
            r = O.fill_ranges(k, v)
            sl = torch.tensor(lens, dtype=torch.int32)
            ids = torch.arange(len(lens))
            self.fn = lambda: O.port_decode_attn(q, r, ids, sl, kvh, scale)
            self.kind = "port"
        self.nseq = len(lens)
        self.bytes, _ = algorithmic_bytes(lens, 1, h, kvh, 2)

    def sample(self):
        t0 = time.perf_counter()
        self.fn()
        return time.perf_counter() - t0


def cpu_sample(name, seed, budget_s=12.0):
    """Median time of the reference CPU attention on ONE layer of the workload, all host
    threads, within a time budget.  Returns (GB/s, seconds, kind, cores, sequences, runs)."""
    layer = CpuLayer(name, seed)
    layer.sample()
    times = []
    t_all = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_all < budget_s and len(times) < 50):
        times.append(layer.sample())
    sec = statistics.median(times)
    return layer.bytes / sec / 1e9, sec, layer.kind, layer.cores, layer.nseq, len(times)


def cpu_baseline(name, seed):
    gbs, sec, kind, cores, nseq, runs = cpu_sample(name, seed)
    layers = WORKLOADS[name][0]
    return {"value": round(gbs, 2), "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"one layer of {layers} ({nseq} sequences, all heads, bf16 KV), decode attention only, median of "
                      f"{runs} runs of {sec * 1e3:.1f} ms; the reference CPU backend has no fp8 KV",
            "ms_per_step_extrapolated": round(sec * layers * 1e3, 1)}


def run_reference(args):
    """The reference's own CPU implementation of the path (its CPU-backend paged_attention
    kernels, csrc/cpu/attention.cpp) on the box's host cores.  A "step" of this arm is a
    bounded sample of the workload's step: ONE layer of it, at the full head count (the
    whole problem, whatever --gpus says).  W warm-up samples, then exactly K timed ones."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload if args.workload != "auto" else ("7b" if world == 1 else "70b")
    layers = WORKLOADS[name][0]
    layer = CpuLayer(name, args.seed)
    for _ in range(max(args.warmup, 1)):
        layer.sample()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        layer.sample()
    sec = (time.perf_counter() - t0) / args.steps
    gbs = round(layer.bytes / sec / 1e9, 2)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3),
        "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "bf16 in/out, fp32 accumulate", "data": "synthetic",
        "config": shared_config(name, world, args.seed),
        "details": {"step_is": f"a bounded sample: one layer of the {layers}-layer step, all heads, decode attention only",
                    "ms_per_full_step_extrapolated": round(sec * layers * 1e3, 2),
                    "path_tokens_per_s_extrapolated": round(WORKLOADS[name][1] / (sec * layers), 2)},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": layer.cores, "kind": layer.kind,
                         "sample": f"one layer of {layers}, {layer.nseq} sequences, all heads, mean of {args.steps} runs"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
# op-level timings (python bench.py --op ...): the commands behind profiles/*.md
# ----------------------------------------------------------------------------
def _time_calls(run, iters, flush=True):
    """Median CUDA-event time (ms) of run(); a 256 MB read between calls leaves clean,
    unrelated lines in L2."""
    import torch
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    junk = torch.zeros(64 << 20, dtype=torch.float32, device="cuda") if flush else None
    ts = []
    for _ in range(iters):
        if flush:
            junk.sum()
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run()
        z.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(z))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def op_main(argv):
    """--op decode B H KVH LO HI [fp8 0|1] [num_splits] [iters] [tcgen05 0|1]    one layer's decode attention call
       --op prefill B H KVH L [tma 0|1] [iters]                    causal prefill over the ranges, TFLOP/s
       --op rope TOKENS H KVH [fp8 0|1] [iters]                    RoPE fused with the KV append
       --op norm TOKENS HIDDEN [iters]                             rms_norm / fused_add_rms_norm
       --op allreduce [BYTES ...]   (under torchrun)               peer-memory all-reduce vs NCCL, 100 calls per graph
    Environment: VT_ATTN_VARIANT=simt|mma|flat and VT_ATTN_PART_TOKENS select a kernel variant / partition size."""
    import torch
    from glake_b200 import ops, vmmAllocator as A
    from glake_b200.backend import VTensorCacheEngine, VTensorMetadata, prepare_step
    mode, rest = argv[0], argv[1:]
    ints = [int(x) for x in rest]
    chunk = A.granularitySize
    if mode == "allreduce":
        return op_allreduce(ints)
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    if mode == "decode":
        B, H, KVH, LO, HI = ints[:5]
        fp8 = len(ints) > 5 and ints[5] == 1
        splits = ints[6] if len(ints) > 6 else 0
        iters = ints[7] if len(ints) > 7 else 20
        tma = len(ints) > 8 and ints[8] == 1      # fp8 only: the tcgen05 kernel over tensor maps
        e = 1 if fp8 else 2
        lens = context_lens(0, B, LO, HI)
        row = KVH * D * e
        assert A.init_physical_handle(sum((n * row + chunk - 1) // chunk for n in lens) * 2 + 16, 0)
        dt = "fp8_e4m3" if fp8 else "auto"
        eng = VTensorCacheEngine(1, KVH, D, B, HI + 8, cache_dtype=dt)
        meta = VTensorMetadata(list(range(B)), lens, KVH, D, num_prefills=B, kv_elem_size=e)
        prepare_step(meta, eng)
        tot = sum(lens)
        kcat = torch.randn(tot, KVH, D, device="cuda", dtype=torch.bfloat16)
        vcat = torch.randn(tot, KVH, D, device="cuda", dtype=torch.bfloat16)
        ks = ops.kv_scales(kcat, KVH, D) if fp8 else None
        vs = ops.kv_scales(vcat, KVH, D) if fp8 else None
        ops.reshape_and_cache(kcat, vcat, eng.k_cache_ptr[0], eng.v_cache_ptr[0], meta.slot_m, meta.slot_mapping,
                              meta.seq_lens_tensor, meta.cache_seq_lens, max(lens), KVH, D, dt, ks, vs)
        del kcat, vcat
        q = torch.randn(B, H, D, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        kc, vc = eng.gpu_cache[0]
        maps = eng.decode_maps(0, H) if tma else None

        def run():
            ops.paged_attention_v1(out, q, kc.vmm_ptr, vc.vmm_ptr, KVH, D ** -0.5, meta.seq_lens_tensor, 1, max(lens), None,
                                   dt, 1.0, meta.slot_mapping, k_scale=ks, v_scale=vs, num_splits=splits, maps=maps)
        ms, best = _time_calls(run, iters)
        byt = tot * 2 * KVH * D * e + 2 * B * H * D * 2
        print(f"decode B{B} H{H} KVH{KVH} L[{LO},{HI}] fp8={fp8} splits={splits} tcgen05={maps is not None} plan={ops.attn_plan(B, H, KVH, max(lens), dt, splits)}: "
              f"{ms * 1e3:.1f} us  {byt / ms / 1e6:.0f} GB/s  ({byt / 2 ** 20:.0f} MiB)  best {byt / best / 1e6:.0f} GB/s  "
              f"status {ops.attn_status()}", flush=True)
    elif mode == "prefill":
        B, H, KVH, L = ints[:4]
        tma = not (len(ints) > 4 and ints[4] == 0)
        iters = ints[5] if len(ints) > 5 else 10
        row = KVH * D * 2
        assert A.init_physical_handle(B * 2 * ((L * row + chunk - 1) // chunk) + 16, 0)
        eng = VTensorCacheEngine(1, KVH, D, B, L + 8)
        meta = VTensorMetadata(list(range(B)), [L] * B, KVH, D, num_prefills=B)
        prepare_step(meta, eng)
        k = torch.randn(B * L, KVH, D, device="cuda", dtype=torch.bfloat16)
        v = torch.randn_like(k)
        ops.reshape_and_cache(k, v, eng.k_cache_ptr[0], eng.v_cache_ptr[0], meta.slot_m, meta.slot_mapping,
                              meta.seq_lens_tensor, meta.cache_seq_lens, L, KVH, D)
        q = torch.randn(B * L, H, D, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        ql = torch.full((B,), L, dtype=torch.int32, device="cuda")
        qs = torch.arange(B, dtype=torch.int32, device="cuda") * L
        kc, vc = eng.gpu_cache[0]
        maps = eng.prefill_maps(0) if tma else None

        def run():
            ops.prefill_attention(out, q, kc.vmm_ptr, vc.vmm_ptr, KVH, D ** -0.5, meta.slot_mapping, meta.seq_lens_tensor,
                                  ql, qs, L, maps=maps)
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
        print(f"prefill B{B} H{H} KVH{KVH} L{L} {'tensor copies' if maps is not None else 'row copies'}: {ms:.3f} ms  "
              f"{2 * B * H * L * L * D / ms / 1e9:.1f} TFLOP/s (causal flops)", flush=True)
    elif mode == "rope":
        T, H, KVH = ints[:3]
        fp8 = len(ints) > 3 and ints[3] == 1
        iters = ints[4] if len(ints) > 4 else 20
        e = 1 if fp8 else 2
        decode = T <= 1024
        row = KVH * D * e
        n_slots = T if decode else 1
        assert A.init_physical_handle((2 * n_slots if decode else 2 * ((T * row >> 21) + 2)) + 8, 0)
        dt = "fp8_e4m3" if fp8 else "auto"
        eng = VTensorCacheEngine(1, KVH, D, n_slots, 8 if decode else T + 8, cache_dtype=dt)
        if decode:
            meta = VTensorMetadata(list(range(T)), [1] * T, KVH, D, num_decode_tokens=T, kv_elem_size=e)
        else:
            meta = VTensorMetadata([0], [T], KVH, D, num_prefills=1, kv_elem_size=e)
        prepare_step(meta, eng)
        qkv = torch.randn(T, (H + 2 * KVH) * D, device="cuda", dtype=torch.bfloat16)
        q, k, v = qkv.split([H * D, KVH * D, KVH * D], dim=-1)
        pos = torch.randint(0, 4096, (T,), device="cuda")
        cs = torch.randn(4096, D, device="cuda", dtype=torch.bfloat16)
        ks = torch.full((KVH,), 5 / 448, device="cuda")
        vs = ks.clone()

        def run():
            ops.rotary_embedding_and_cache(pos, q, k, v, D, cs, True, eng.k_cache_ptr[0], eng.v_cache_ptr[0], meta.slot_m,
                                           meta.slot_mapping, meta.seq_lens_tensor, meta.cache_seq_lens,
                                           1 if decode else T, KVH, dt, ks if fp8 else None, vs if fp8 else None)
        ms, _ = _time_calls(run, iters)
        byt = T * (2 * H * 256 + 2 * KVH * 256 + 2 * KVH * D * e + 2 * 256)
        print(f"rope+append T{T} H{H} KVH{KVH} fp8={fp8} {'decode' if decode else 'prefill'}: {ms * 1e3:.1f} us  "
              f"{byt / ms / 1e6:.0f} GB/s  ({byt / 2 ** 20:.1f} MiB)", flush=True)
    elif mode == "norm":
        T, hidden = ints[:2]
        iters = ints[2] if len(ints) > 2 else 20
        x = torch.randn(T, hidden, device="cuda", dtype=torch.bfloat16)
        r, o = torch.randn_like(x), torch.empty_like(x)
        w = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
        ms, _ = _time_calls(lambda: ops.rms_norm(o, x, w, 1e-5), iters)
        byt = T * hidden * 4
        print(f"rms_norm T{T} hidden{hidden}: {ms * 1e3:.1f} us  {byt / ms / 1e6:.0f} GB/s  ({byt / 2 ** 20:.1f} MiB)", flush=True)
        ms, _ = _time_calls(lambda: ops.fused_add_rms_norm(x, r, w, 1e-5), iters)
        print(f"fused_add_rms_norm T{T} hidden{hidden}: {ms * 1e3:.1f} us  {2 * byt / ms / 1e6:.0f} GB/s  "
              f"({2 * byt / 2 ** 20:.1f} MiB)", flush=True)
    else:
        raise SystemExit(op_main.__doc__)


def op_allreduce(sizes):
    import torch
    import torch.distributed as dist
    from glake_b200 import tp
    rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    world = dist.get_world_size()
    sizes = sizes or [8 << 10, 64 << 10, 128 << 10, 256 << 10, 1 << 20, 2 << 20, 8 << 20]
    comm = tp.PeerAllReduce(max_size=max(max(sizes), 1 << 20))
    if os.environ.get("VT_AR_ONE_SHOT_BYTES"):
        comm.configure(one_shot_bytes=int(os.environ["VT_AR_ONE_SHOT_BYTES"]))
    if os.environ.get("VT_AR_PUSH_BYTES"):
        comm.configure(push_bytes=int(os.environ["VT_AR_PUSH_BYTES"]))
    calls = 100
    for nbytes in sizes:
        x = torch.randn(nbytes // 2, device="cuda").bfloat16()
        y = torch.empty_like(x)
        res = {}
        impls = [("peer", lambda: comm.all_reduce(x, y))]
        if not os.environ.get("VT_AR_SKIP_NCCL"):
            impls.append(("nccl", lambda: dist.all_reduce(x)))
        if os.environ.get("VT_AR_SKIP_PEER"):
            impls = impls[1:]
        for name, fn in impls:
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for _ in range(3):
                    fn()
                side.synchronize()
                g = torch.cuda.CUDAGraph()
                # thread-local capture mode: the process group's watchdog thread may touch events meanwhile
                with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
                    for _ in range(calls):
                        fn()
            ts = []
            for _ in range(5):
                dist.barrier()
                torch.cuda.synchronize()
                a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                g.replay()
                z.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(z) * 1e3 / calls)
            ts.sort()
            res[name] = tp.max_over_ranks(ts[len(ts) // 2], device="cuda")
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


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        # torchrun exports OMP_NUM_THREADS=1 for its children; the reference's CPU kernels are OpenMP code
        # and this arm is meant to use every host core.  Must happen before any OpenMP runtime loads.
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    if a.op:
        op_main(a.op)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
