"""World-size-2 (and 4) CPU ranks over gloo: the head partition of the
tensor-parallel path.  Each rank attends only over its own kv heads (the CPU
oracle stands in for the kernel here; no GPU is involved), the per-rank outputs
are gathered, and the result must equal the unsharded computation bit for bit —
attention has no cross-head term, so sharding may not change a single value.
Also checks the model-level sum and the max-over-ranks step time."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests import synth


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, h, kvh, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from glake_b200 import tp
        from oracle import oracle as O
        lens = [70, 300, 33]
        q, k, v = synth.make_case(5, lens, h, kvh)           # same seed on every rank, like broadcast metadata
        sh = tp.shard_heads(h, kvh, world, rank)
        ql = q[:, sh.q_begin:sh.q_end].contiguous()
        kl = [x[:, sh.kv_begin:sh.kv_end].contiguous() for x in k]
        vl = [x[:, sh.kv_begin:sh.kv_end].contiguous() for x in v]
        r = O.fill_ranges(kl, vl)
        sl = torch.tensor(lens, dtype=torch.int32)
        out = O.port_decode_attn(ql, r, torch.arange(3), sl, sh.num_kv_heads, 128 ** -0.5)
        parts = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(parts, out)
        full = torch.cat(parts, dim=1)
        # model-level reduction after a row-parallel projection: sum of per-rank partial products
        w = torch.ones(sh.num_heads * 128, 4)
        partial = out.view(3, -1).float() @ w
        tp.all_reduce_sum(partial)
        same = tp.tensor_model_parallel_all_reduce(torch.full((4,), float(rank + 1)))   # no peer path on CPU: gloo
        assert same.tolist() == [world * (world + 1) / 2] * 4
        slowest = tp.max_over_ranks(10.0 + rank)
        if rank == 0:
            rf = O.fill_ranges(k, v)
            want = O.port_decode_attn(q, rf, torch.arange(3), sl, kvh, 128 ** -0.5)
            ret["equal"] = bool(torch.equal(full, want))
            ret["sum_ok"] = bool(torch.allclose(partial, want.view(3, -1).float() @ torch.ones(h * 128, 4), atol=1e-3))
            ret["slowest"] = slowest
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,h,kvh", [(2, 8, 2), (2, 8, 8), (4, 8, 2)])
def test_head_sharding_over_gloo_ranks(world, h, kvh):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, h, kvh, ret)) for r in range(world)]
        [p.start() for p in procs]
        [p.join(120) for p in procs]
        assert all(p.exitcode == 0 for p in procs)
        assert ret["equal"] and ret["sum_ok"] and ret["slowest"] == 10.0 + world - 1


def test_shard_arithmetic():
    from glake_b200 import tp
    s = tp.shard_heads(64, 8, 8, 3)
    assert (s.q_begin, s.q_end, s.kv_begin, s.kv_end) == (24, 32, 3, 4)
    s = tp.shard_heads(64, 8, 2, 1)
    assert (s.num_heads, s.num_kv_heads, s.kv_begin) == (32, 4, 4)
    s = tp.shard_heads(32, 2, 8, 5)          # fewer kv heads than ranks: replicated
    assert (s.num_heads, s.num_kv_heads, s.kv_begin) == (4, 1, 1)
    with pytest.raises(ValueError):
        tp.shard_heads(30, 8, 4, 0)
