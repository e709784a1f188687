"""Tensor-parallel head partition for the vTensor path.

Heads are sharded the way the reference's ``LlamaAttention.__init__`` does
(GLakeServe/vllm/model_executor/models/llama.py:106-122): rank ``r`` of ``tp``
owns q heads ``[r*H/tp, (r+1)*H/tp)`` and kv heads ``[r*KVH/tp, (r+1)*KVH/tp)``;
when there are fewer kv heads than ranks each kv head is replicated over
``tp/KVH`` ranks.  Every rank keeps its own chunk pool and its own per-slot ranges
with ``row = kv_heads_local * 128 * e`` bytes; append and attention touch local
memory only.  The only collectives around the path are the model-level sum after
``o_proj`` / ``down_proj`` (GLakeServe/vllm/model_executor/layers/linear.py:690-691),
done with ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests) or, for
small bf16 messages on NVLink-connected GPUs, with :class:`PeerAllReduce`, the
counterpart of the reference's ``CustomAllreduce``
(GLakeServe/vllm/distributed/device_communicators/custom_all_reduce.py:76-275).
"""
import ctypes

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


class PeerAllReduce:
    """One-launch sum all-reduce of bf16 tensors up to ``max_size`` bytes over peer
    memory (libvtensor's ``vt_all_reduce``).  One instance per process and GPU; all
    ranks of ``group`` must sit on one node with peer access between their GPUs,
    construct it together and make the same sequence of calls.

    The 64-byte CUDA IPC handles of the per-rank buffers travel through
    ``group`` (``all_gather_object``), as the reference's do
    (custom_all_reduce.py:167-204)."""

    def __init__(self, group=None, device=None, max_size=8192 * 1024, n_ctas=0):
        from ._lib import check, lib
        self._lib, self._check = lib, check
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if not 2 <= self.world <= 8:
            raise ValueError("PeerAllReduce serves 2 to 8 ranks")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.max_size = max_size
        self._ar = ctypes.c_void_p()
        self._opened = []
        self._buf = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            need = ctypes.c_size_t()
            check(lib.vt_ar_buffer_bytes(max_size, ctypes.byref(need)), "vt_ar_buffer_bytes")
            check(lib.vt_ar_alloc(need.value, ctypes.byref(self._buf)), "vt_ar_alloc")
            handle = (ctypes.c_ubyte * 64)()
            check(lib.vt_ar_ipc_export(self._buf, handle), "vt_ar_ipc_export")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            peers = (ctypes.c_void_p * self.world)()
            for r, h in enumerate(handles):
                if r == self.rank:
                    peers[r] = self._buf.value
                else:
                    p = ctypes.c_void_p()
                    check(lib.vt_ar_ipc_open((ctypes.c_ubyte * 64).from_buffer_copy(h), ctypes.byref(p)),
                          "vt_ar_ipc_open")
                    self._opened.append(p)
                    peers[r] = p.value
            check(lib.vt_ar_create(self.rank, self.world, peers, max_size, n_ctas, ctypes.byref(self._ar)),
                  "vt_ar_create")
        dist.barrier(group=group)       # every buffer is zero-filled and mapped before anybody's first call

    def should_use(self, x):
        """The reference's ``should_custom_ar`` (csrc/custom_all_reduce.cu:58-68) for this
        implementation: bf16, contiguous, 16-byte multiples, within max_size."""
        return (x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() % 8 == 0
                and x.data_ptr() % 16 == 0 and 0 < x.numel() * 2 <= self.max_size)

    def all_reduce(self, x, out=None):
        """out (default: a new tensor) = sum of x over the ranks, on the current stream."""
        if not self.should_use(x):
            raise ValueError("tensor not eligible for the peer all-reduce (see should_use)")
        out = torch.empty_like(x) if out is None else out
        with torch.cuda.device(self.device):
            self._check(self._lib.vt_all_reduce(self._ar, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                                x.numel(), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)),
                        "vt_all_reduce")
        return out

    def status(self):
        """0, or non-zero once a wait for a peer ran out (synchronises)."""
        st = ctypes.c_uint32()
        with torch.cuda.device(self.device):
            self._check(self._lib.vt_ar_status(self._ar, ctypes.byref(st)), "vt_ar_status")
        return st.value

    def configure(self, wait_ns=0, one_shot_bytes=-1, push_bytes=-1, push2_bytes=-1):
        """Wait limit and the size thresholds of the four paths (see vt_ar_configure); -1 keeps a value."""
        with torch.cuda.device(self.device):
            self._check(self._lib.vt_ar_configure(self._ar, wait_ns, one_shot_bytes, push_bytes, push2_bytes),
                        "vt_ar_configure")

    def close(self):
        if self._ar:
            with torch.cuda.device(self.device):
                torch.cuda.synchronize()
                dist.barrier(group=self.group)      # nobody still reads a buffer that is about to go
                self._lib.vt_ar_destroy(self._ar)
                for p in self._opened:
                    self._lib.vt_ar_ipc_close(p)
                self._lib.vt_ar_free(self._buf)
            self._ar, self._opened = ctypes.c_void_p(), []


_peer_ar = None


def set_peer_all_reduce(comm):
    """Install (or with None remove) the communicator tensor_model_parallel_all_reduce tries first."""
    global _peer_ar
    _peer_ar = comm


def tensor_model_parallel_all_reduce(input_, group=None):
    """The reference's entry point (GLakeServe/vllm/distributed/communication_op.py:57-84):
    identity for one rank; the peer-memory path when a communicator is installed and
    the tensor qualifies (result in a new tensor); otherwise ``torch.distributed``
    in place.  Always use the return value."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return input_
    if _peer_ar is not None and _peer_ar.should_use(input_):
        return _peer_ar.all_reduce(input_)
    dist.all_reduce(input_, op=dist.ReduceOp.SUM, group=group)
    return input_


def max_over_ranks(value, device="cpu", group=None):
    """Max of a per-rank scalar (step time) over the ranks; used by the benchmark."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
