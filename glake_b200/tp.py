"""Tensor-parallel head partition for the vTensor path.

Heads are sharded the way the reference's ``LlamaAttention.__init__`` does
(GLakeServe/vllm/model_executor/models/llama.py:106-122): rank ``r`` of ``tp``
owns q heads ``[r*H/tp, (r+1)*H/tp)`` and kv heads ``[r*KVH/tp, (r+1)*KVH/tp)``;
when there are fewer kv heads than ranks each kv head is replicated over
``tp/KVH`` ranks.  Every rank keeps its own chunk pool and its own per-slot ranges
with ``row = kv_heads_local * 128 * e`` bytes; append and attention touch local
memory only.  The only collectives around the path are the model-level sum after
``o_proj`` / ``down_proj`` (GLakeServe/vllm/model_executor/layers/linear.py:690-691),
done with ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests).
"""
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class HeadShard:
    rank: int
    tp: int
    q_begin: int
    q_end: int
    kv_begin: int
    kv_end: int

    @property
    def num_heads(self):
        return self.q_end - self.q_begin

    @property
    def num_kv_heads(self):
        return self.kv_end - self.kv_begin


def shard_heads(num_heads, num_kv_heads, tp, rank):
    if num_heads % tp != 0:
        raise ValueError(f"{num_heads} q heads do not divide over {tp} ranks")
    if not 0 <= rank < tp:
        raise ValueError("rank out of range")
    hq = num_heads // tp
    if num_kv_heads >= tp:
        if num_kv_heads % tp != 0:
            raise ValueError(f"{num_kv_heads} kv heads do not divide over {tp} ranks")
        hk = num_kv_heads // tp
        return HeadShard(rank, tp, rank * hq, (rank + 1) * hq, rank * hk, (rank + 1) * hk)
    if tp % num_kv_heads != 0:
        raise ValueError(f"{tp} ranks do not divide over {num_kv_heads} kv heads")
    kv = rank // (tp // num_kv_heads)        # replicated kv head (llama.py:119: max(1, KVH // tp))
    return HeadShard(rank, tp, rank * hq, (rank + 1) * hq, kv, kv + 1)


def slice_q(x, shard, head_size=128):
    """[tokens, H*D] or [tokens, H, D] -> this rank's q heads."""
    x3 = x.view(x.shape[0], -1, head_size)
    return x3[:, shard.q_begin:shard.q_end]


def slice_kv(x, shard, head_size=128):
    x3 = x.view(x.shape[0], -1, head_size)
    return x3[:, shard.kv_begin:shard.kv_end]


def all_reduce_sum(x, group=None):
    """Model-level tensor-parallel reduction (in place); identity without a process group."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
    return x


def max_over_ranks(value, device="cpu", group=None):
    """Max of a per-rank scalar (step time) over the ranks; used by the benchmark."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
