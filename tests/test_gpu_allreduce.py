"""GPU tests of the peer-memory all-reduce (vt_all_reduce).

On one GPU the ranks are emulated as ONE cooperative launch over all ranks' buffers
(vt_all_reduce_emulated), which exercises the whole protocol — staging, per-CTA
flags, one-shot and two-shot paths, double buffering over consecutive calls.  With
two or more GPUs a second test runs real ranks as child processes over CUDA IPC.
Results are bit-exact against the oracle (fp32 sum in rank order, one rounding) and
identical on every rank."""
import ctypes
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, world, n):
    rs = np.random.RandomState(seed)
    return [torch.from_numpy(rs.standard_normal(n).astype(np.float32)).bfloat16() for _ in range(world)]


class Emulated:
    """`world` communicators on the current GPU sharing `world` buffers."""

    def __init__(self, world, max_bytes=2 << 20, n_ctas=16):
        from glake_b200._lib import check, lib
        self.lib, self.check, self.world = lib, check, world
        need = ctypes.c_size_t()
        check(lib.vt_ar_buffer_bytes(max_bytes, ctypes.byref(need)), "vt_ar_buffer_bytes")
        self.bufs = []
        for _ in range(world):
            p = ctypes.c_void_p()
            check(lib.vt_ar_alloc(need.value, ctypes.byref(p)), "vt_ar_alloc")
            self.bufs.append(p)
        peers = (ctypes.c_void_p * world)(*[b.value for b in self.bufs])
        self.ars = []
        for r in range(world):
            a = ctypes.c_void_p()
            check(lib.vt_ar_create(r, world, peers, max_bytes, n_ctas, ctypes.byref(a)), "vt_ar_create")
            self.ars.append(a)

    def run(self, ins, outs):
        V = ctypes.c_void_p * self.world
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return self.lib.vt_all_reduce_emulated(V(*[a.value for a in self.ars]), V(*[t.data_ptr() for t in ins]),
                                               V(*[t.data_ptr() for t in outs]), self.world, ins[0].numel(), stream)

    def status(self, r):
        st = ctypes.c_uint32()
        self.check(self.lib.vt_ar_status(self.ars[r], ctypes.byref(st)), "vt_ar_status")
        return st.value

    def close(self):
        torch.cuda.synchronize()
        for a in self.ars:
            self.lib.vt_ar_destroy(a)
        for b in self.bufs:
            self.lib.vt_ar_free(b)


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_emulated_ranks_match_the_oracle(oracle, world):
    torch.zeros(1, device="cuda")
    E = Emulated(world)
    try:
        for a in E.ars:                                    # two-shot above 128 KiB, whatever the world size; no two-phase push
            E.check(E.lib.vt_ar_configure(a, 0, 128 << 10, -1, 0), "vt_ar_configure")
        # one-shot sizes, two-shot sizes, ragged vector counts, consecutive calls on both parities
        for call, n in enumerate([8, 8 * 37, 4096, 65536, 65536 + 8 * 5, 1 << 19, (1 << 19) + 8 * 123, 1 << 20, 8 * 3,
                                  1 << 20, 1 << 20]):
            ins = _inputs(100 * world + call, world, n)
            want = oracle.port_all_reduce(ins)
            d_in = [t.cuda() for t in ins]
            d_out = [torch.empty_like(t) for t in d_in] if call % 2 == 0 else d_in      # odd calls: in place
            assert E.run(d_in, d_out) == 0
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(d_out[r].cpu(), want), f"call {call} n {n} rank {r}"
        assert all(E.status(r) == 0 for r in range(world))
    finally:
        E.close()


@pytest.mark.parametrize("world", [2, 5, 8])
def test_emulated_push_path_buffer_rotation(oracle, world):
    """Messages up to 256 KiB take the flag-free path: data pushed into per-source slots,
    the sentinel restored one call later, three buffers in rotation.  Sizes shrink and grow
    from call to call (the restored range is the previous call's, not this one's), calls of
    the flag path sit in between, and an input word of two negative zeros — the sentinel's
    bit pattern — must come out as a zero sum."""
    E = Emulated(world)
    try:
        sizes = [8, 32768, 8, 8 * 511, 1 << 17, 32768, 1 << 18, 8 * 3, 1 << 17, 8, 8, 8, 1 << 19, 4096, 32768]
        for call, n in enumerate(sizes):
            ins = _inputs(5000 + 10 * world + call, world, n)
            if n >= 16:
                for t in ins:
                    t[8:10] = -0.0                                    # every rank sends the sentinel pattern there
                    t[12] = -0.0                                      # half a word of it: an ordinary value
            want = oracle.port_all_reduce(ins)
            d_in = [t.cuda() for t in ins]
            d_out = [torch.empty_like(t) for t in d_in] if call % 3 else d_in
            assert E.run(d_in, d_out) == 0
            torch.cuda.synchronize()
            for r in range(world):
                got = d_out[r].cpu()
                assert torch.equal(got.float(), want.float()), f"call {call} n {n} rank {r}"   # == treats -0 and +0 alike
        assert all(E.status(r) == 0 for r in range(world))
        # the same messages with the push path switched off give the same values
        for a in E.ars:
            E.check(E.lib.vt_ar_configure(a, 0, -1, 0, 0), "vt_ar_configure")
        ins = _inputs(77, world, 4096)
        d_in = [t.cuda() for t in ins]
        outs = [torch.empty_like(t) for t in d_in]
        assert E.run(d_in, outs) == 0
        torch.cuda.synchronize()
        assert all(torch.equal(o.cpu(), oracle.port_all_reduce(ins)) for o in outs)
    finally:
        E.close()


@pytest.mark.parametrize("world,n_ctas", [(2, 16), (3, 16), (8, 16), (8, 32)])
def test_emulated_two_phase_push_path(oracle, world, n_ctas):
    """Messages between 256 KiB and 2 MiB: scatter-reduce then broadcast through
    sentinel-filled buffers.  Sizes change from call to call (the restored ranges are the
    previous call's), vector counts that do not divide by CTAs x ranks, calls of the other
    paths in between, in-place calls, and inputs / sums that hit the sentinel's bit pattern."""
    E = Emulated(world, n_ctas=n_ctas)
    try:
        sizes = [1 << 19, 1 << 20, (1 << 18) + 8 * 7, 8, 1 << 19, (1 << 19) + 8 * 1001, 1 << 20, 32768, 1 << 20,
                 (1 << 17) + 8, 1 << 19, 1 << 19, 1 << 19]
        for call, n in enumerate(sizes):
            ins = _inputs(9000 + 10 * world + call, world, n)
            if n >= 24:
                for t in ins:
                    t[8:10] = -0.0                                    # every rank sends the sentinel pattern there
                    t[12] = -0.0
                ins[0][16:18] = 1.5                                   # ... and here values cancel to zero next to negative zeros
                ins[1][16:18] = -1.5
                for t in ins[2:]:
                    t[16:18] = -0.0
            want = oracle.port_all_reduce(ins)
            d_in = [t.cuda() for t in ins]
            d_out = [torch.empty_like(t) for t in d_in] if call % 3 else d_in
            assert E.run(d_in, d_out) == 0
            torch.cuda.synchronize()
            for r in range(world):
                got = d_out[r].cpu()
                assert torch.equal(got.float(), want.float()), f"call {call} n {n} rank {r}"   # == treats -0 and +0 alike
        assert all(E.status(r) == 0 for r in range(world))
    finally:
        E.close()


def test_emulated_forced_modes_agree(oracle):
    """The same message through the one-shot and the two-shot path gives the same bits."""
    E = Emulated(4)
    try:
        ins = _inputs(7, 4, 40000)
        want = oracle.port_all_reduce(ins)
        d_in = [t.cuda() for t in ins]
        for one_shot_bytes in (1 << 30, 0):
            for a in E.ars:
                E.check(E.lib.vt_ar_configure(a, 0, one_shot_bytes, -1, 0), "vt_ar_configure")
            outs = [torch.empty_like(t) for t in d_in]
            assert E.run(d_in, outs) == 0
            torch.cuda.synchronize()
            assert all(torch.equal(o.cpu(), want) for o in outs)
    finally:
        E.close()


def test_a_missing_peer_ends_in_a_status_not_a_hang():
    """Rank 0 of a two-rank communicator calls alone: the flag nobody sets makes its
    bounded wait run out, the call returns, the status word says so and the context
    stays usable."""
    from glake_b200._lib import VT_ERR_TOO_LARGE, VT_ERR_UNSUPPORTED
    E = Emulated(2, max_bytes=1 << 16)
    try:
        E.check(E.lib.vt_ar_configure(E.ars[0], 2_000_000, -1, -1, -1), "vt_ar_configure")       # 2 ms
        x = torch.ones(1024, dtype=torch.bfloat16, device="cuda")
        y = torch.empty_like(x)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert E.lib.vt_all_reduce(E.ars[0], ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr()), 1024, stream) == 0
        torch.cuda.synchronize()
        assert E.status(0) != 0 and E.status(1) == 0
        assert float((x + 1).sum()) == 2048.0                                         # the context still works
        big = torch.ones(1 << 16, dtype=torch.bfloat16, device="cuda")
        assert E.lib.vt_all_reduce(E.ars[0], ctypes.c_void_p(big.data_ptr()), ctypes.c_void_p(big.data_ptr()),
                                   big.numel(), stream) == VT_ERR_TOO_LARGE
        assert E.lib.vt_all_reduce(E.ars[0], ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr()), 12,
                                   stream) == VT_ERR_UNSUPPORTED
    finally:
        E.close()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from glake_b200 import tp
        from oracle import oracle as O
        comm = tp.PeerAllReduce(max_size=2 << 20)
        comm.configure(one_shot_bytes=128 << 10)           # so that the larger messages take the two-shot path
        tp.set_peer_all_reduce(comm)
        ok = True
        for call, n in enumerate([8, 4096, 65536 + 40, 1 << 19, 1 << 20, 1 << 20, 8 * 11]):
            ins = _inputs(900 + call, world, n)
            want = O.port_all_reduce(ins)
            out = tp.tensor_model_parallel_all_reduce(ins[rank].cuda())
            ok = ok and torch.equal(out.cpu(), want)
        comm.configure(push2_bytes=0)                      # the same large messages through the flag paths
        for call, n in enumerate([1 << 19, 1 << 20, 1 << 19]):
            ins = _inputs(950 + call, world, n)
            out = tp.tensor_model_parallel_all_reduce(ins[rank].cuda())
            ok = ok and torch.equal(out.cpu(), O.port_all_reduce(ins))
        comm.configure(push2_bytes=2 << 20)
        # a captured sequence of calls replays correctly with new inputs
        x = torch.zeros(1 << 16, dtype=torch.bfloat16, device="cuda")
        y = torch.empty_like(x)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            comm.all_reduce(x, y)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                comm.all_reduce(x, y)
                comm.all_reduce(y, y)
        for it in range(3):
            ins = _inputs(950 + it, world, 1 << 16)
            x.copy_(ins[rank])
            g.replay()
            torch.cuda.synchronize()
            once = O.port_all_reduce(ins)
            ok = ok and torch.equal(y.cpu(), O.port_all_reduce([once] * world))
        ok = ok and comm.status() == 0
        # a tensor the peer path does not take goes through torch.distributed
        f = torch.ones(10, device="cuda")
        ok = ok and float(tp.tensor_model_parallel_all_reduce(f)[0]) == world
        comm.close()
        ret[rank] = ok
    finally:
        tp.set_peer_all_reduce(None)
        dist.destroy_process_group()


def test_real_ranks_over_cuda_ipc(oracle):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret)) for r in range(world)]
        [p.start() for p in procs]
        [p.join(300) for p in procs]
        assert all(p.exitcode == 0 for p in procs)
        assert all(ret.get(r) for r in range(world)), dict(ret)
